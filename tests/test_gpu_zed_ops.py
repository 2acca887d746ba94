"""Each mechanism of the pre-norm layer form alone, on the GPU, against the plain statement in oracle/zedotar.py:
residual + norm, gated gelu products, the soft cap, convolution + rotary preparation across steps, cached attention
(window, pooled blocks, sink, sigmoid weights, gates; keys in the step, in the cache, in the block table) and mLSTM.
Inputs are shaped so that a fault shows: one key made dominant at a chosen distance, scores far below the sink, portions
that cut a pooled block or the convolution's reach, slots whose earlier owner left its state behind."""
import pytest
import torch

from oracle import zedotar as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, seed=0, scale=1.0):
    return scale * torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64)


def err(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def f32(t):
    return t.to(DEV, torch.float32).contiguous()


def steps_of(lengths_per_step):
    """[[(slot, n), ...], ...] -> per step the RaggedBatch descriptions [(slot, n, pos0, parity)], tracking positions."""
    pos, par, out = {}, {}, []
    for step in lengths_per_step:
        desc = []
        for slot, n in step:
            desc.append((slot, n, pos.get(slot, 0), par.get(slot, 0)))
            pos[slot] = pos.get(slot, 0) + n
            par[slot] = par.get(slot, 0) ^ 1
        out.append(desc)
    return out


# ---------------------------------------------------------------------------------------------- small pieces
def test_add_rms_norm_and_softcap():
    from umbrella_b200 import ops_seq as K
    for width in (40, 200, 1100):
        x, d, w = rnd(7, width, seed=1), rnd(7, width, seed=2), rnd(width, seed=3, scale=0.3)
        xs = f32(x)
        y, copy = K.add_rms_norm(xs, f32(d), f32(w), 1.0, 1e-5, want_copy=True)
        assert err(y, O.rms_norm_zero_centred(x + d, w, 1e-5)) < 2e-6
        assert err(xs, x + d) < 1e-6 and err(copy, x + d) < 1e-6            # the sum stays in the residual stream
        rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
        xs2 = f32(x)
        y2 = K.add_rms_norm(xs2, f32(d), f32(w), 1.0, 1e-5, rows=rows)
        assert err(y2, O.rms_norm_zero_centred((x + d)[[5, 0, 5]], w, 1e-5)) < 2e-6
        assert torch.equal(xs2.cpu(), x.float())                            # chosen rows: nothing is written back
        yb = K.add_rms_norm(f32(x), None, f32(w), 0.0, 1e-5, dtype=torch.bfloat16)
        assert err(yb, O.rms_norm_zero_centred(x, w - 1.0, 1e-5)) < 1e-2
    z = rnd(5, 33, seed=4, scale=20.0)
    assert err(K.softcap(f32(z), 7.5), O.softcap(z, 7.5)) < 2e-6


def test_gated_gelu_products():
    from umbrella_b200 import _lib_seq as S
    from umbrella_b200 import ops_seq as K
    for M, W, ff, dt, tol in ((5, 48, 40, torch.float32, 3e-6), (130, 64, 96, torch.float32, 3e-6),
                              (130, 64, 96, torch.bfloat16, 2e-2), (6, 64, 96, torch.bfloat16, 2e-2)):
        h = rnd(M, W, seed=5).to(torch.bfloat16).double()
        gate, up, down = (rnd(ff, W, seed=6, scale=W ** -0.5 * 3).to(torch.bfloat16).double(),
                          rnd(ff, W, seed=7, scale=W ** -0.5).to(torch.bfloat16).double(),
                          rnd(W, ff, seed=8, scale=ff ** -0.5).to(torch.bfloat16).double())
        y = K.gemm(h.to(DEV, dt), torch.cat([gate, up]).to(DEV, dt), dual=S.UMBS_ACT_GELU_TANH)
        ref = O.gelu_tanh(h @ gate.T) * (h @ up.T)
        assert err(y, ref) < tol
        out = K.gemm(y, down.to(DEV, dt), out_f32=True)
        assert err(out, O.gated_gelu_mlp(h, gate, up, down)) < max(tol, 2e-2 if dt == torch.bfloat16 else 0)


# ---------------------------------------------------------------------------------------------- convolution + rotary
@pytest.mark.parametrize("taps,rot_dims,values_are_keys", [(3, 8, True), (4, 16, True), (1, 6, False), (2, 0, False)])
def test_attention_prep_across_steps(taps, rot_dims, values_are_keys):
    """Two sequences fed in portions (some shorter than the convolution's reach) into slots that hold an earlier
    owner's rows; against the convolution and rotation of each whole sequence."""
    from umbrella_b200 import ops_seq as K
    H, G, D = 4, 2, 16
    V = D if values_are_keys else 24
    C, Cv = (H + G) * D, 0 if values_are_keys else G * V
    lens = {0: 23, 2: 9}
    proj = {s: rnd(n, C + Cv + 3, seed=10 + s) for s, n in lens.items()}
    bias, conv_w = rnd(C + Cv, seed=20, scale=0.5), rnd(C, taps, seed=21)
    rot = dict(dims=rot_dims, base=50.0, scaling=dict(kind="yarn", factor=3.0, original=16, fast=4.0, slow=1.0) if rot_dims else None)
    inv_freq, mag = (O.rotary_frequencies(rot) if rot_dims else (torch.zeros(1, dtype=torch.float64), 1.0))
    conv_state = torch.full((2, 3, max(taps - 1, 1), C), 7.0, dtype=torch.float32, device=DEV)      # dirty
    plan = steps_of([[(0, 1), (2, 4)], [(0, 1), (2, 1)], [(0, 2), (2, 4)], [(0, 19)]])
    got_q, got_kv, at = {0: [], 2: []}, {0: [], 2: []}, {0: 0, 2: 0}
    for desc in plan:
        rows = torch.cat([proj[s][at[s]:at[s] + n] for s, n, _, _ in desc])
        b = K.RaggedBatch(desc, DEV)
        q, kv = K.attention_prep(f32(rows), f32(bias), b, H, G, D, V, rot_dims, f32(inv_freq), mag, values_are_keys, taps,
                                 f32(conv_w) if taps > 1 else None, conv_state if taps > 1 else None)
        o = 0
        for s, n, _, _ in desc:
            got_q[s].append(q[o:o + n]), got_kv[s].append(kv[o:o + n])
            at[s] += n
            o += n
    for s, n in lens.items():
        u = proj[s][:, :C] + bias[:C]
        y = O.causal_conv(u, conv_w) if taps > 1 else u
        q_ref = O.rotate(y[:, :H * D].reshape(n, H, D), rot).reshape(n, H * D)
        k_ref = O.rotate(y[:, H * D:].reshape(n, G, D), rot).reshape(n, G * D)
        v_ref = y[:, H * D:] if values_are_keys else proj[s][:, C:C + Cv] + bias[C:]
        assert err(torch.cat(got_q[s]), q_ref) < 3e-6, s
        assert err(torch.cat(got_kv[s]), torch.cat([k_ref, v_ref], dim=1)) < 3e-6, s


# ---------------------------------------------------------------------------------------------- cached attention
def run_attention(q, k, v, plan_lengths, *, H, G, mode, window, pool, scale, head_bias=None, gate=None, gate_per_head=False,
                  kv_len=None, dtype=torch.float32, slot=1, split=True):
    """One sequence (q [n, H, D], k [n, G, D], v [n, G, V]) fed in the given portions through slot `slot` of dirty caches."""
    from umbrella_b200 import _lib_seq as S
    from umbrella_b200 import ops_seq as K
    n, D, V = q.shape[0], q.shape[2], v.shape[2]
    row = G * (D + V)
    kv_len = kv_len or (max(window, pool, 1) if window > 0 else n)
    cache = torch.full((3, kv_len, row), 3.0, dtype=dtype, device=DEV)
    pooled = torch.full((3, max(1, -(-n // pool)), row), -5.0, dtype=dtype, device=DEV) if pool else None
    kvrows = torch.cat([k.reshape(n, G * D), v.reshape(n, G * V)], dim=1)
    out, at = [], 0
    for desc in steps_of([[(slot, m)] for m in plan_lengths]):
        m = desc[0][1]
        b = K.RaggedBatch(desc, DEV)
        out.append(K.cached_attention(q[at:at + m].reshape(m, H * D).to(DEV, dtype), kvrows[at:at + m].to(DEV, dtype), cache, b,
                                      H, G, D, V, scale, mode={"softmax": S.UMBS_ATTN_SOFTMAX, "sink": S.UMBS_ATTN_SOFTMAX_SINK,
                                                               "sigmoid": S.UMBS_ATTN_SIGMOID}[mode],
                                      window=window, pool=pool, pool_cache=pooled, head_bias=f32(head_bias) if head_bias is not None else None,
                                      gate=f32(gate[at:at + m]) if gate is not None else None, gate_per_head=gate_per_head, split=split))
        at += m
    assert at == n
    return torch.cat(out).reshape(n, H, V)


PLANS = lambda n: ([n], [n - 40] + [1] * 40, [1] * n, [7, 2, 3, 64, 5] + [n - 81], [n - 3, 2, 1])


@pytest.mark.parametrize("window,pool", [(9, 4), (16, 16), (5, 7), (1, 1), (70, 0), (64, 8)])
def test_pooled_window_attention_every_cut(window, pool):
    H, G, D, V, n = 4, 2, 16, 24, 150
    q, k, v = rnd(n, H, D, seed=1), rnd(n, G, D, seed=2), rnd(n, G, V, seed=3)
    gate = rnd(n, H, seed=4)
    ref = O.pooled_window_attention(q, k, v, window, pool, 0.4) * torch.sigmoid(gate)[:, :, None]
    for plan in PLANS(n):
        got = run_attention(q, k, v, plan, H=H, G=G, mode="sink", window=window, pool=pool, scale=0.4, gate=gate, gate_per_head=True)
        assert err(got, ref) < 5e-6, plan[:4]


@pytest.mark.parametrize("distance", [15, 16, 17, 31, 32, 33, 47, 48])
def test_dominant_key_at_the_window_and_block_edges(distance):
    """Window 16, blocks of 8.  One key is made to tower over all others; the query sits `distance` tokens later.  Inside the
    window the row's output is that key's value; just outside it the key is seen only as an eighth of a block's mean, or --
    while its block is not yet wholly outside the window -- not at all.  In a prompt and while decoding."""
    H, G, D, V, n, window, pool, j = 2, 1, 16, 8, 80, 16, 8, 19
    i = j + distance
    q, k, v = rnd(n, H, D, seed=5, scale=0.1), rnd(n, G, D, seed=6, scale=0.1), rnd(n, G, V, seed=7)
    k[j, 0] = 0.0
    k[j, 0, 3] = 6.0
    q[i, :, 3] = 6.0
    ref = O.pooled_window_attention(q, k, v, window, pool, 1.0)
    seen_alone = distance < window
    assert (float((ref[i, 0] - v[j, 0]).abs().max()) < 1e-3) == seen_alone
    for plan in ([n], [i] + [1] * (n - i), [j + 1, i - j - 1, 1, n - i - 1], [1] * n):
        got = run_attention(q, k, v, plan, H=H, G=G, mode="sink", window=window, pool=pool, scale=1.0)
        assert err(got[i], ref[i]) < 5e-6 and err(got, ref) < 5e-6, (distance, plan[:3])


def test_sink_takes_the_weight_when_all_scores_are_low():
    H, G, D, V, n = 2, 2, 16, 16, 40
    q, k, v = rnd(n, H, D, seed=8), rnd(n, G, D, seed=9), rnd(n, G, V, seed=10) + 3.0
    q[:, :, 0], k[:, :, 0] = 30.0, -1.0                # every score about -30: the sink holds nearly all the weight
    with_sink = run_attention(q, k, v, [n - 5] + [1] * 5, H=H, G=G, mode="sink", window=12, pool=4, scale=1.0)
    without = run_attention(q, k, v, [n - 5] + [1] * 5, H=H, G=G, mode="softmax", window=12, pool=4, scale=1.0)
    ref = O.pooled_window_attention(q, k, v, 12, 4, 1.0)
    assert float(ref.abs().max()) < 1e-3 and float(with_sink.abs().max()) < 1e-3
    assert float(without.abs().min()) > 0.1            # a plain softmax would hand the weight to the keys
    assert err(with_sink, ref) < 1e-4


def test_sigmoid_attention_far_key_among_hundreds():
    """No softmax: with a bias of -9 every key weighs about 1e-4, except one far key whose score is raised to +9."""
    H, G, D, n, far = 4, 2, 16, 700, 11
    q, k, v = rnd(n, H, D, seed=11, scale=0.2), rnd(n, G, D, seed=12, scale=0.2), rnd(n, G, D, seed=13)
    k[far, :, 5] = 6.0
    q[n - 2:, :, 5] = 6.0                              # the last two rows, one of them decoded, look 690 tokens back
    pb, gate = torch.tensor([-9.0, -9.0, -8.0, -9.5], dtype=torch.float64), rnd(n, H * D, seed=14)
    ref = O.sigmoid_attention(q, k, v, 0.5, pb) * torch.sigmoid(gate).reshape(n, H, D)
    far_part = torch.sigmoid(torch.tensor(0.5 * 36.0) + pb)[:, None] * v[far].repeat_interleave(H // G, 0)
    assert float((ref[n - 1] / torch.sigmoid(gate[n - 1]).reshape(H, D) - far_part).abs().max()) < 0.5      # it dominates the row
    for plan in ([n], [n - 1, 1], [300, 2, 390, 1, 1, 1, 1, 1, 1, 1, 1]):
        got = run_attention(q, k, v, plan, H=H, G=G, mode="sigmoid", window=0, pool=0, scale=0.5, head_bias=pb, gate=gate)
        assert err(got, ref) < 5e-6, plan[:3]
    unsplit = run_attention(q, k, v, [n - 1, 1], H=H, G=G, mode="sigmoid", window=0, pool=0, scale=0.5, head_bias=pb, gate=gate, split=False)
    assert err(unsplit, ref) < 5e-6


def test_ragged_batch_and_bf16_storage():
    """Three sequences of unequal length in one step (one of them a single token), then decoded together; bf16 rows."""
    from umbrella_b200 import _lib_seq as S
    from umbrella_b200 import ops_seq as K
    H, G, D, V, window, pool = 4, 4, 32, 32, 20, 6
    lens, extra = (1, 75, 130), 9
    for dt, tol in ((torch.float32, 5e-6), (torch.bfloat16, 2e-2)):
        data = [tuple(rnd(n + extra, h, d, seed=20 + 3 * i + c).to(dt).double() for c, (h, d) in enumerate(((H, D), (G, D), (G, V))))
                for i, n in enumerate(lens)]
        refs = [O.pooled_window_attention(q, k, v, window, pool, 0.2) for q, k, v in data]
        cache = torch.zeros((4, window, G * (D + V)), dtype=dt, device=DEV)
        pooled = torch.zeros((4, 40, G * (D + V)), dtype=dt, device=DEV)
        slots = (3, 0, 2)
        plan = steps_of([[(s, n) for s, n in zip(slots, lens)]] + [[(s, 1) for s in slots]] * extra)
        at = [0, 0, 0]
        for desc in plan:
            qs = torch.cat([data[i][0][at[i]:at[i] + d[1]].reshape(d[1], H * D) for i, d in enumerate(desc)])
            kvs = torch.cat([torch.cat([data[i][1][at[i]:at[i] + d[1]].reshape(d[1], G * D),
                                        data[i][2][at[i]:at[i] + d[1]].reshape(d[1], G * V)], dim=1) for i, d in enumerate(desc)])
            got = K.cached_attention(qs.to(DEV, dt), kvs.to(DEV, dt), cache, K.RaggedBatch(desc, DEV), H, G, D, V, 0.2,
                                     mode=S.UMBS_ATTN_SOFTMAX_SINK, window=window, pool=pool, pool_cache=pooled)
            o = 0
            for i, d in enumerate(desc):
                assert err(got[o:o + d[1]].reshape(d[1], H, V), refs[i][at[i]:at[i] + d[1]]) < tol, (dt, i, at[i])
                o += d[1]
                at[i] += d[1]


# ---------------------------------------------------------------------------------------------- mLSTM
def mlstm_reference(proj, bias, H, D, V, cap, eps, norm_w):
    n = proj.shape[0]
    q, k = proj[:, :H * D].reshape(n, H, D) * D ** -0.5, proj[:, H * D:2 * H * D].reshape(n, H, D)
    v = proj[:, 2 * H * D:2 * H * D + H * V].reshape(n, H, V)
    g = proj[:, 2 * H * D + H * V:2 * H * D + 2 * H * V]
    i_pre, f_pre = proj[:, -2 * H:-H] + bias[:H], proj[:, -H:] + bias[H:]
    i_log = cap * torch.tanh(i_pre / cap)
    f_log = torch.nn.functional.logsigmoid(cap * torch.tanh(f_pre / cap))
    o = O.unit_rms(O.mlstm_recurrence(q, k, v, i_log, f_log), eps).reshape(n, H * V)
    return o * norm_w * torch.sigmoid(g)


@pytest.mark.parametrize("H,D,V,cap", [(3, 16, 20, 10.0), (2, 48, 32, 4.0), (1, 40, 31, 15.0), (2, 160, 64, 8.0)])
def test_mlstm_whole_portions_and_batches(H, D, V, cap):
    """Gate pre-activations large enough that the input gate's exponent reaches the cap and the running maximum moves;
    portions of 1 to 40 tokens; two sequences in one step; slots that hold an earlier owner's memory."""
    from umbrella_b200 import ops_seq as K
    rows = 2 * H * D + 2 * H * V + 2 * H
    lens = {1: 70, 0: 33}
    proj = {s: rnd(n, rows, seed=30 + s) for s, n in lens.items()}
    for s in proj:
        proj[s][:, -2 * H:] *= 6.0                     # gates well into the soft cap, both signs
    bias, norm_w = rnd(2 * H, seed=33), 1.0 + rnd(H * V, seed=34, scale=0.2)
    refs = {s: mlstm_reference(proj[s], bias, H, D, V, cap, 1e-5, norm_w) for s in lens}
    for lengths in ([[(1, 70), (0, 33)]], [[(1, 1), (0, 2)], [(1, 29), (0, 1)], [(1, 40), (0, 30)]],
                    [[(1, 35)]] + [[(1, 1)]] * 35 + [[(0, 33)]]):
        state = torch.full((2, H, D * (V + 1) + 1), 2.5, dtype=torch.float32, device=DEV)         # dirty
        at, got = {0: 0, 1: 0}, {0: [], 1: []}
        for desc in steps_of(lengths):
            x = torch.cat([proj[s][at[s]:at[s] + n] for s, n, _, _ in desc])
            out = K.mlstm(f32(x), f32(bias), K.RaggedBatch(desc, DEV), H, D, V, cap, 1e-5, f32(norm_w), state)
            o = 0
            for s, n, _, _ in desc:
                got[s].append(out[o:o + n])
                at[s] += n
                o += n
        for s in lens:
            if got[s]:
                assert err(torch.cat(got[s]), refs[s][:at[s]]) < 2e-5, (s, len(lengths))


def test_mlstm_long_sequences_cut_into_segments():
    """A step of few long sequences runs as segments side by side (two passes, chained states): a long prompt that starts
    from a carried state, with a short neighbour and one whose last segment is a single token, against the single walk
    of the oracle."""
    from umbrella_b200 import ops_seq as K
    H, D, V, cap = 2, 32, 40, 8.0
    rows = 2 * H * D + 2 * H * V + 2 * H
    lens = {0: 10 + 417, 1: 5, 2: 3 + 321}
    proj = {s: rnd(n, rows, seed=40 + s) for s, n in lens.items()}
    for s in proj:
        proj[s][:, -2 * H:] *= 4.0
    bias, norm_w = rnd(2 * H, seed=43), 1.0 + rnd(H * V, seed=44, scale=0.2)
    refs = {s: mlstm_reference(proj[s], bias, H, D, V, cap, 1e-5, norm_w) for s in lens}
    state = torch.full((3, H, D * (V + 1) + 1), -1.5, dtype=torch.float32, device=DEV)
    plan = steps_of([[(0, 10), (2, 3)], [(0, 417), (1, 5), (2, 321)]])
    at, got = {0: 0, 1: 0, 2: 0}, {0: [], 1: [], 2: []}
    for desc in plan:
        x = torch.cat([proj[s][at[s]:at[s] + n] for s, n, _, _ in desc])
        out = K.mlstm(f32(x), f32(bias), K.RaggedBatch(desc, DEV), H, D, V, cap, 1e-5, f32(norm_w), state, segments=True)
        o = 0
        for s, n, _, _ in desc:
            got[s].append(out[o:o + n])
            at[s] += n
            o += n
    for s in lens:
        assert err(torch.cat(got[s]), refs[s]) < 3e-5, s
    # the state the segmented step left is the single walk's: one more token from it
    extra = rnd(1, rows, seed=49)
    full = torch.cat([proj[0], extra])
    ref = mlstm_reference(full, bias, H, D, V, cap, 1e-5, norm_w)[-1:]
    out = K.mlstm(f32(extra), f32(bias), K.RaggedBatch([(0, 1, lens[0], 0)], DEV), H, D, V, cap, 1e-5, f32(norm_w), state)
    assert err(out, ref) < 3e-5


@pytest.mark.parametrize("D,V,mode", [(160, 200, "sink"), (256, 256, "sigmoid"), (72, 136, "softmax")])
def test_attention_with_large_and_uneven_heads(D, V, mode):
    """Heads above 128 (several passes over the key tile's dimensions, wider value tiles, more elements per lane in
    decode steps) and sizes that are no multiple of 32."""
    H, G, n = 2, 1, 90
    if mode == "sigmoid":
        V = D
    q, k, v = rnd(n, H, D, seed=51, scale=0.5), rnd(n, G, D, seed=52, scale=0.5), rnd(n, G, V, seed=53)
    if mode == "sigmoid":
        v = k.clone()
        pb = torch.tensor([-3.0, -2.0], dtype=torch.float64)
        ref = O.sigmoid_attention(q, k, v, 0.1, pb)
        kw = dict(window=0, pool=0, head_bias=pb)
    else:
        ref = O.pooled_window_attention(q, k, v, 24, 8, 0.1) if mode == "sink" else None
        kw = dict(window=24, pool=8)
    for plan in ([n], [n - 20] + [1] * 20, [33, 2, 55]):
        got = run_attention(q, k, v, plan, H=H, G=G, mode=mode, scale=0.1, **kw)
        if ref is None:                                 # plain softmax: no oracle form; every cut must give the same numbers
            ref = got.double().cpu()
        assert err(got, ref) < 5e-6, plan[:3]
