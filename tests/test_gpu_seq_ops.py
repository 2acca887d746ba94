"""Each mechanism of the sequence-state decoders alone (umbrella_b200/ops_seq.py) against its plain statement in
oracle/seqstate.py, with inputs made so that a fault shows: one dominant key at a window's edge, a single far
key carried through the recurrent state, state handed from step to step, dirty slots."""
import pytest
import torch

import seq_helpers as H
from oracle import seqstate as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def g(seed):
    return torch.Generator().manual_seed(seed)


@pytest.fixture(scope="module")
def ops():
    from umbrella_b200 import ops_seq
    return ops_seq


# ---------------------------------------------------------------------------------------------- matrix products
@pytest.mark.parametrize("M,N,K", [(1, 40, 24), (70, 130, 96), (200, 64, 160), (3, 7, 5)])
def test_gemm_float32_and_bf16(ops, M, N, K):
    a, w = torch.randn(M, K, generator=g(1)), torch.randn(N, K, generator=g(2))
    ref = a.double() @ w.double().T
    assert H.rel_err(ops.gemm(a.to(DEV), w.to(DEV), out_f32=True), ref) < 1e-6
    ab, wb = a.bfloat16(), w.bfloat16()
    refb = ab.double() @ wb.double().T
    assert H.rel_err(ops.gemm(ab.to(DEV), wb.to(DEV), out_f32=True), refb) < 1e-5      # exact products, fp32 sums
    assert H.rel_err(ops.gemm(ab.to(DEV), wb.to(DEV)), refb) < 6e-3                    # rounded to bf16 on the way out


def test_gemm_row_results_do_not_depend_on_the_batch(ops):
    a, w = torch.randn(150, 96, generator=g(3)).bfloat16().to(DEV), torch.randn(80, 96, generator=g(4)).bfloat16().to(DEV)
    full = ops.gemm(a, w, out_f32=True)
    assert torch.equal(ops.gemm(a[64:].contiguous(), w, out_f32=True), full[64:])       # same kernel: bit-identical rows
    for rows in (slice(0, 1), slice(7, 9), slice(30, 46)):                               # the few-row kernel: rounding only
        assert H.rel_err(ops.gemm(a[rows].contiguous(), w, out_f32=True), full[rows]) < 1e-6
    few = ops.gemm(a[:16].contiguous(), w, out_f32=True)
    assert torch.equal(ops.gemm(a[3:4].contiguous(), w, out_f32=True), few[3:4])


def test_gemm_batched_over_heads(ops):
    Hh, D, R, M = 3, 32, 48, 21
    for dt, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-5)):
        q = torch.randn(M, Hh * D, generator=g(5)).to(dt)
        w = torch.randn(Hh, R, D, generator=g(6)).to(dt)
        ref = torch.einsum("mhd,hrd->mhr", q.double().view(M, Hh, D), w.double()).reshape(M, Hh * R)
        got = ops.gemm(q.to(DEV), w.to(DEV), out_f32=True, groups=Hh, a_goff=D, c_goff=R)
        assert H.rel_err(got, ref) < tol


@pytest.mark.parametrize("n", [37, 90])                 # one-block routing of a small step / routing spread over blocks
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_gemm_expert_sorted_rows_with_gated_activation(ops, dt, n):
    W, E, top, ff, limit = 64, 4, 2, 32, 0.7
    h = torch.randn(n, W, generator=g(7)).to(dt)
    router = torch.randn(E, W, generator=g(8))
    gu = (torch.randn(E, 2 * ff, W, generator=g(9)) * 0.3).to(dt)
    sel_w, grp_off, pair_tok, pair_pos, sel_e = ops.moe_route(h.to(DEV), router.to(DEV), top)
    y = ops.gemm(h.to(DEV), gu.to(DEV), groups=E, n=ff, dual=True, limit=limit, grp_off=grp_off, row_src=pair_tok,
                 rows=n * top, max_rows=n)
    idx, wts = O.route_top(h.double(), router.double(), top)
    assert torch.equal(sel_e.cpu().long(), idx) and H.rel_err(sel_w, wts) < 1e-5
    off = grp_off.cpu().tolist()
    assert off[0] == 0 and off[-1] == n * top
    for t in range(n):
        for j in range(top):
            e, p = int(idx[t, j]), int(pair_pos[t * top + j])
            assert off[e] <= p < off[e + 1] and int(pair_tok[p]) == t
            gate, up = gu[e, :ff].double(), gu[e, ff:].double()
            gg = torch.clamp(h[t].double() @ gate.T, max=limit)
            uu = torch.clamp(h[t].double() @ up.T, -limit, limit)
            ref = gg * torch.sigmoid(1.702 * gg) * (uu + 1)
            assert H.rel_err(y[p], ref) < (1e-5 if dt == torch.float32 else 1e-2)


def test_routing_of_a_token_does_not_depend_on_the_step_size(ops):
    # the same tokens routed alone (one block for the whole step) and inside a large step (a block per token): the same
    # experts in the same order and bit-equal weights
    W, E, top = 96, 12, 3
    h = torch.randn(300, W, generator=g(21)).to(DEV)
    router = torch.randn(E, W, generator=g(22)).to(DEV)
    big_w, _, _, _, big_e = ops.moe_route(h, router, top)
    for lo, hi in ((0, 1), (5, 13), (280, 300)):
        w, off, tok, pos, e = ops.moe_route(h[lo:hi].contiguous(), router, top)
        assert torch.equal(e, big_e[lo:hi]) and torch.equal(w, big_w[lo:hi])
        # pairs of an expert are listed in token order
        off = off.cpu().tolist()
        for x in range(E):
            assert tok[off[x]:off[x + 1]].cpu().tolist() == sorted(tok[off[x]:off[x + 1]].cpu().tolist())


# ---------------------------------------------------------------------------------------------- norm + token shift
def test_group_norm_and_shift_across_steps(ops):
    W, G, eps, slots = 48, 3, 1e-3, 3
    x = torch.randn(11, W, generator=g(10)) * 3
    w, mu = torch.randn(W, generator=g(11)), torch.rand(W, generator=g(12))
    h_ref = O.group_rms_norm(x.double(), w.double(), G, eps)
    hs_ref = O.token_shift(h_ref, mu.double())
    state = torch.full((2, slots, W), 7.0, device=DEV)                  # dirty: a fresh sequence must not read it
    xd, wd, mud = x.to(DEV), w.to(DEV), mu.to(DEV)
    b1 = ops.RaggedBatch([(2, 6, 0, 0)], DEV)
    h1, hs1 = ops.group_norm_shift(xd[:6].contiguous(), wd, mud, state, b1, G, eps)
    b2 = ops.RaggedBatch([(2, 1, 6, 1)], DEV)                           # one token: reads the half the first step wrote
    h2, hs2 = ops.group_norm_shift(xd[6:7].contiguous(), wd, mud, state, b2, G, eps)
    b3 = ops.RaggedBatch([(2, 4, 7, 0)], DEV)
    h3, hs3 = ops.group_norm_shift(xd[7:].contiguous(), wd, mud, state, b3, G, eps)
    assert H.rel_err(torch.cat([h1, h2, h3]), h_ref) < 1e-6
    assert H.row_err(torch.cat([hs1, hs2, hs3]), hs_ref) < 1e-5


# ---------------------------------------------------------------------------------------------- retention
def _ret_inputs(n, Hh, D, V, seed):
    qkvg = torch.randn(n, 2 * Hh * D + 2 * Hh * V, generator=g(seed))
    q, k, v, gt = qkvg.double().split([Hh * D, Hh * D, Hh * V, Hh * V], dim=1)
    return qkvg, q.reshape(n, Hh, D), k.reshape(n, Hh, D), v.reshape(n, Hh, V), gt


def _ret_ref(q, k, v, gt, D, rot, base, decay, eps):
    n = q.shape[0]
    o = O.retention_recurrence(O.rotate_half(q, rot, base), O.rotate_half(k, rot, base) * D ** -0.5, v, decay)
    return O.rms_norm(o, eps).reshape(n, -1) * (gt * torch.sigmoid(gt))


@pytest.mark.parametrize("Hh,D,V,rot", [(2, 16, 40, 8), (1, 24, 150, 24), (3, 8, 16, 0)])
def test_retention_whole_portions_and_batch(ops, Hh, D, V, rot):
    from umbrella_b200.models.seq_model import rotary_inv_freq
    n, base, eps = 45, 50.0, 1e-4
    decay = [0.5, 0.93, 0.9995][:Hh]
    qkvg, q, k, v, gt = _ret_inputs(n, Hh, D, V, 13)
    ref = _ret_ref(q, k, v, gt, D, rot, base, decay, eps)
    inv = (rotary_inv_freq(rot, base) if rot else torch.zeros(1)).to(DEV)
    dec = torch.tensor(decay, device=DEV)
    state = torch.full((3, Hh, D, V), 5.0, device=DEV)
    x = qkvg.to(DEV)
    whole = ops.retention(x, ops.RaggedBatch([(1, n, 0, 0)], DEV), Hh, D, V, rot, inv, dec, eps, state)
    assert H.row_err(whole, ref) < 2e-5
    # portions 9 + 1 + 2 + rest, in slot 0, while slot 2 runs another sequence in the same steps
    other, q2, k2, v2, g2 = _ret_inputs(n, Hh, D, V, 14)
    ref2 = _ret_ref(q2, k2, v2, g2, D, rot, base, decay, eps)
    y = other.to(DEV)
    outs, outs2, at = [], [], 0
    for m in (9, 1, 2, n - 12):
        both = torch.cat([x[at:at + m], y[at:at + m]])
        o = ops.retention(both, ops.RaggedBatch([(0, m, at, 0), (2, m, at, 0)], DEV), Hh, D, V, rot, inv, dec, eps, state)
        outs.append(o[:m]), outs2.append(o[m:])
        at += m
    assert H.row_err(torch.cat(outs), ref) < 2e-5 and H.row_err(torch.cat(outs2), ref2) < 2e-5


def test_retention_long_sequences_cut_into_segments(ops):
    """Few long sequences run as segments side by side (two passes with chained states): the same numbers as the single
    walk and as the oracle -- for a fresh sequence, for one that goes on from a carried state, next to a short one that is
    not cut, and with a last segment of a few tokens."""
    from umbrella_b200.models.seq_model import rotary_inv_freq
    Hh, D, V, rot, base, eps = 2, 16, 40, 8, 50.0, 1e-4
    decay = [0.93, 0.9995]
    inv, dec = rotary_inv_freq(rot, base).to(DEV), torch.tensor(decay, device=DEV)
    n = 700
    qkvg, q, k, v, gt = _ret_inputs(n, Hh, D, V, 23)
    ref = _ret_ref(q, k, v, gt, D, rot, base, decay, eps)
    other, q2, k2, v2, g2 = _ret_inputs(40, Hh, D, V, 24)
    ref2 = _ret_ref(q2, k2, v2, g2, D, rot, base, decay, eps)
    x, y = qkvg.to(DEV), other.to(DEV)
    for segments in (True, False):
        state = torch.full((3, Hh, D, V), 7.0, device=DEV)
        # step 1: 130 tokens of the long one; step 2: its other 570 (a carried state, cut) next to a fresh short one
        o1 = ops.retention(x[:130].contiguous(), ops.RaggedBatch([(2, 130, 0, 0)], DEV), Hh, D, V, rot, inv, dec, eps, state,
                           segments=segments)
        o2 = ops.retention(torch.cat([x[130:], y]), ops.RaggedBatch([(2, 570, 130, 0), (0, 40, 0, 0)], DEV), Hh, D, V, rot, inv,
                           dec, eps, state, segments=segments)
        assert H.row_err(torch.cat([o1, o2[:570]]), ref) < 2e-5, segments
        assert H.row_err(o2[570:], ref2) < 2e-5, segments
        if segments:
            cut_state = state.clone()
        else:
            assert H.rel_err(cut_state[2], state[2]) < 1e-5 and H.rel_err(cut_state[0], state[0]) < 1e-6
    # a length that leaves a last segment of one token
    state = torch.zeros((1, Hh, D, V), device=DEV)
    o = ops.retention(x[:385].contiguous(), ops.RaggedBatch([(0, 385, 0, 0)], DEV), Hh, D, V, rot, inv, dec, eps, state)
    assert H.row_err(o, ref[:385]) < 2e-5


def test_retention_carries_one_far_key(ops):
    """Only token 0 has a key and a value; the query sits 400 tokens later, reached through four separate steps."""
    Hh, D, V, n, decay = 1, 8, 32, 401, 0.99609375
    qkvg = torch.zeros(n, 2 * D + 2 * V)
    qkvg[0, D:2 * D] = 1.0                                       # k_0
    qkvg[0, 2 * D:2 * D + V] = torch.arange(1, V + 1).float()    # v_0
    qkvg[-1, :D] = 1.0                                           # q_400
    qkvg[:, 2 * D + V:] = 1.0                                    # gate
    x = qkvg.to(DEV)
    state = torch.zeros(1, Hh, D, V, device=DEV)
    dec, inv = torch.tensor([decay], device=DEV), torch.zeros(1, device=DEV)
    at, out = 0, None
    for m in (100, 1, 250, 50):
        out = ops.retention(x[at:at + m].contiguous(), ops.RaggedBatch([(0, m, at, 0)], DEV), Hh, D, V, 0, inv, dec, 0.0, state)
        at += m
    want = decay ** 400 * D * D ** -0.5 * torch.arange(1, V + 1).double()       # before the unit norm
    want = want / want.pow(2).mean().sqrt() * (1 / (1 + torch.exp(torch.tensor(-1.0, dtype=torch.float64))))
    assert H.rel_err(out[-1], want) < 1e-5
    assert H.rel_err(state[0, 0].sum(0), decay ** 400 * D ** -0.5 * D * torch.arange(1, V + 1).double()) < 1e-5


# ---------------------------------------------------------------------------------------------- latent attention
def _lat_ref(q_abs, c, scale, window):
    n, Hh, R = q_abs.shape
    kv = c.double()[:, None, :].expand(n, Hh, R)
    return O.windowed_softmax_attention(q_abs.double(), kv, kv, scale, window).reshape(n, Hh * R)


@pytest.mark.parametrize("dt,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
def test_latent_attention_portions_decode_and_batch(ops, dt, tol):
    n, Hh, R, window, scale = 60, 3, 40, 7, 0.4
    q_abs = torch.randn(n, Hh, R, generator=g(15))
    c = torch.randn(n, R, generator=g(16)).to(dt)
    ref = _lat_ref(q_abs, c.float(), scale, window)
    ring = torch.full((2, window, R), 9.0, dtype=dt, device=DEV)
    qd, cd = q_abs.reshape(n, Hh * R).to(DEV), c.to(DEV)
    whole = ops.latent_attention(qd, cd, ring, ops.RaggedBatch([(0, n, 0, 0)], DEV), Hh, window, scale)
    assert H.row_err(whole, ref) < tol
    outs, at = [], 0
    for m in [5, 2, 1, 1, 20, 3] + [1] * 28:                       # slot 1; portions, then decoding across ring wraps
        outs.append(ops.latent_attention(qd[at:at + m].contiguous(), cd[at:at + m].contiguous(), ring,
                                         ops.RaggedBatch([(1, m, at, 0)], DEV), Hh, window, scale))
        at += m
    assert at == n and H.row_err(torch.cat(outs), ref) < tol


@pytest.mark.parametrize("decode", [False, True])
def test_latent_attention_window_edge(ops, decode):
    """One key stands out.  The query that still sees it returns (almost) that key's latent; one token later it is gone."""
    R, window, n, key = 32, 12, 40, 17
    c = torch.randn(n, R, generator=g(17)) * 0.05
    c[key] = 0.0
    c[key, 3] = 6.0
    q_abs = torch.zeros(n, 1, R)
    q_abs[:, 0, 3] = 8.0                                           # score 48 for the marked key, about 0 for the others
    ring = torch.zeros((1, window, R), device=DEV)
    qd, cd = q_abs.reshape(n, R).to(DEV), c.to(DEV)
    pieces = [n] if not decode else [key + 2] + [1] * (n - key - 2)
    outs, at = [], 0
    for m in pieces:
        outs.append(ops.latent_attention(qd[at:at + m].contiguous(), cd[at:at + m].contiguous(), ring,
                                         ops.RaggedBatch([(0, m, at, 0)], DEV), 1, window, 1.0))
        at += m
    out = torch.cat(outs).cpu()
    inside, outside = key + window - 1, key + window
    assert out[inside, 3] > 5.9 and out[key, 3] > 5.9
    assert abs(out[outside, 3]) < 0.5 and abs(out[key - 1, 3]) < 0.5
    assert H.row_err(out, _lat_ref(q_abs, c, 1.0, window)) < 2e-5


# ---------------------------------------------------------------------------------------------- attention among a step's own tokens
@pytest.mark.parametrize("dt,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("Hh,D,V,window", [(3, 24, 40, 7), (2, 16, 96, 70), (1, 72, 8, 1), (2, 32, 64, 200)])
def test_window_attention_whole_and_batch(ops, dt, tol, Hh, D, V, window):
    lens = [150, 1, 64, 65, 3]                                      # over two row tiles, a single token, exactly one tile, one more
    n = sum(lens)
    q = torch.randn(n, Hh, D, generator=g(31)).to(dt)
    kv = torch.randn(n, Hh * (D + V), generator=g(32)).to(dt)       # keys | values side by side, as the step lays them out
    k, v = kv[:, :Hh * D].reshape(n, Hh, D), kv[:, Hh * D:].reshape(n, Hh, V)
    refs, at = [], 0
    for m in lens:
        refs.append(O.windowed_softmax_attention(q[at:at + m].double(), k[at:at + m].double(), v[at:at + m].double(), 0.3, window))
        at += m
    ref = torch.cat(refs).reshape(n, Hh * V)
    starts = [sum(lens[:i]) for i in range(len(lens))]
    kvd = kv.to(DEV)
    got = ops.window_attention(q.reshape(n, Hh * D).to(DEV), kvd[:, :Hh * D], kvd[:, Hh * D:],
                               ops.RaggedBatch([(i, m, 0, 0) for i, m in enumerate(lens)], DEV), Hh, window, 0.3)
    assert H.row_err(got, ref) < tol
    for i in (0, 3):                                                # each request alone: the same rows
        m, a = lens[i], starts[i]
        alone = ops.window_attention(q[a:a + m].reshape(m, Hh * D).to(DEV).contiguous(), kvd[a:a + m, :Hh * D], kvd[a:a + m, Hh * D:],
                                     ops.RaggedBatch([(0, m, 0, 0)], DEV), Hh, window, 0.3)
        assert torch.equal(alone, got[a:a + m])


def test_window_attention_edge_and_tile_border(ops):
    """One key stands out.  The last row that sees it returns its value, the next row does not; the key sits so that the
    edge falls on the border between two key tiles, and once just behind it."""
    D, V, n = 16, 8, 200
    for key, window in ((1, 63), (1, 64), (60, 70), (127, 2)):
        k = torch.randn(n, 1, D, generator=g(33)) * 0.05
        v = torch.randn(n, 1, V, generator=g(34)) * 0.05
        k[key] = 0.0
        k[key, 0, 5] = 6.0
        v[key, 0, 2] = 9.0
        q = torch.zeros(n, 1, D)
        q[:, 0, 5] = 8.0
        got = ops.window_attention(q.reshape(n, D).to(DEV), k.reshape(n, D).to(DEV), v.reshape(n, V).to(DEV),
                                   ops.RaggedBatch([(0, n, 0, 0)], DEV), 1, window, 1.0).cpu()
        inside, outside = key + window - 1, key + window
        assert got[inside, 2] > 8.9 and got[key, 2] > 8.9, (key, window)
        assert abs(got[outside, 2]) < 0.5 and abs(got[key - 1, 2]) < 0.5, (key, window)
        assert H.row_err(got, O.windowed_softmax_attention(q.double(), k.double(), v.double(), 1.0, window).reshape(n, V)) < 2e-5


# ---------------------------------------------------------------------------------------------- residual + depth mix
def test_depth_mix(ops):
    n, W, L = 9, 40, 3
    stack = torch.randn(L + 1, n, W, generator=g(18)).to(DEV)
    x, mix = torch.randn(n, W, generator=g(19)).to(DEV), torch.randn(n, W, generator=g(20)).to(DEV)
    shared = torch.randn(n, W, generator=g(21)).to(DEV)
    dw = torch.randn(L + 1, generator=g(22)).to(DEV)
    layer = L - 1
    got = ops.depth_mix(x, mix, stack, layer, dw, shared=shared)
    new = x.double() + (mix.double() + shared.double())
    ref = O.depth_average([stack[j].double() for j in range(L)] + [new], dw.double())
    assert H.rel_err(got, ref) < 1e-6 and H.rel_err(stack[L], new) < 1e-6
    assert H.rel_err(ops.depth_mix(x, mix, stack, layer, None), x.double() + mix.double()) < 1e-6
