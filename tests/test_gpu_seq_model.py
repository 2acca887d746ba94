"""The sequence-state decoder on the GPU against the plain oracle (oracle/seqstate.py): whole prompts, decoding
token by token, prompts cut into portions, ragged batches, reused slots, long decoding, other sizes, both dtypes."""
import pytest
import torch

import seq_helpers as H
from oracle import seqstate as O

pytestmark = pytest.mark.gpu
TOL32 = 3e-5          # fp32 product vs float64 oracle, per-row relative rms of the logits


def toks(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


@pytest.fixture(scope="module")
def mixed():
    t = H.random_tensors(H.MIXED, seed=1)
    return H.MIXED, H.oracle_model(H.MIXED, t), H.product_model(H.MIXED, t, torch.float32)


def run(model, pieces, want_all=True):
    """Feed one sequence as the given portions through a fresh slot; -> logits of every position."""
    slot = model.cache.alloc_slot()
    out = [model.forward([(slot, p, range(len(p)))]) for p in pieces]
    model.cache.free_slot(slot)
    return torch.cat(out)


def cut(seq, sizes):
    out, i = [], 0
    for s in sizes:
        out.append(seq[i:i + s])
        i += s
    if i < len(seq):
        out.append(seq[i:])
    return [p for p in out if p]


def test_whole_prompt_and_layers(mixed):
    cfg, om, pm = mixed
    seq = toks(70, cfg["vocab"], 2)
    layers = []
    ref = O.forward(om, seq, layers)
    slot = pm.cache.alloc_slot()
    got, ly = pm.forward([(slot, seq, range(len(seq)))], layer_out=True)
    pm.cache.free_slot(slot)
    for i, l in enumerate(layers):
        assert H.row_err(ly[i], l) < TOL32, f"layer {i}"
    assert H.row_err(got, ref) < TOL32


def test_whole_prompt_over_latents_and_over_per_head_keys():
    """A whole prompt's latent attention runs over keys and values up-projected once per token; with that switched off it
    runs over the latents, as later portions and decode steps do.  Both are the oracle's numbers, also in one batch."""
    cfg = dict(H.MIXED, layers=[dict(H.LAT, window=40, heads=3, dim=24, vdim=40, mlp=H.MLP), dict(H.RET, mlp=None),
                                dict(H.LAT, window=100, mlp=None)])
    t = H.random_tensors(cfg, seed=12)
    om = H.oracle_model(cfg, t)
    seqs = [toks(n, cfg["vocab"], 40 + n) for n in (130, 1, 66)]
    refs = [O.forward(om, s) for s in seqs]
    for fresh in (True, False):
        pm = H.product_model(cfg, t, torch.float32, fresh_attention=fresh)
        slots = [pm.cache.alloc_slot() for _ in seqs]
        got = pm.forward([(slots[i], s, range(len(s))) for i, s in enumerate(seqs)])
        assert H.row_err(got, torch.cat(refs)) < TOL32, fresh
        nxt = pm.forward([(slots[0], [5], [0]), (slots[2], [7], [0])])           # decoding goes on from the ring either way
        assert H.row_err(nxt[0:1], O.forward(om, seqs[0] + [5])[-1:]) < TOL32
        assert H.row_err(nxt[1:2], O.forward(om, seqs[2] + [7])[-1:]) < TOL32


def test_first_tokens(mixed):
    cfg, om, pm = mixed
    for n in (1, 2, 3):
        seq = toks(n, cfg["vocab"], 10 + n)
        assert H.row_err(run(pm, [seq]), O.forward(om, seq)) < TOL32


def test_prefill_then_token_by_token(mixed):
    cfg, om, pm = mixed
    seq = toks(60, cfg["vocab"], 3)
    ref = O.forward(om, seq)
    assert H.row_err(run(pm, [[t] for t in seq]), ref) < TOL32                  # decoded from the first token on
    assert H.row_err(run(pm, [seq[:21]] + [[t] for t in seq[21:]]), ref) < TOL32


@pytest.mark.parametrize("sizes", [[2] * 40, [3, 2, 7, 1, 9, 2, 30], [8, 9, 33, 1, 1, 34], [50, 2, 2]])
def test_portions(mixed, sizes):
    cfg, om, pm = mixed
    seq = toks(86, cfg["vocab"], 4)
    assert H.row_err(run(pm, cut(seq, sizes)), O.forward(om, seq)) < TOL32


def test_unequal_batch_matches_each_alone(mixed):
    cfg, om, pm = mixed
    seqs = [toks(n, cfg["vocab"], 20 + n) for n in (1, 47, 13, 30)]
    refs = [O.forward(om, s) for s in seqs]
    slots = [pm.cache.alloc_slot() for _ in seqs]
    pre = [1, 40, 5, 30]                                  # prompt portions of different lengths, one of a single token
    got = [[] for _ in seqs]
    lg = pm.forward([(slots[i], s[:pre[i]], range(pre[i])) for i, s in enumerate(seqs)])
    o = 0
    for i in range(len(seqs)):
        got[i].append(lg[o:o + pre[i]])
        o += pre[i]
    at = list(pre)
    while any(at[i] < len(s) for i, s in enumerate(seqs)):          # decode together; shorter requests leave earlier
        live = [i for i, s in enumerate(seqs) if at[i] < len(s)]
        lg = pm.forward([(slots[i], [seqs[i][at[i]]], [0]) for i in live])
        for j, i in enumerate(live):
            got[i].append(lg[j:j + 1])
            at[i] += 1
    for i in range(len(seqs)):
        pm.cache.free_slot(slots[i])
        assert H.row_err(torch.cat(got[i]), refs[i]) < TOL32, f"request {i}"


def test_freed_slots_are_reused_without_leaking(mixed):
    cfg, om, pm = mixed
    a, b = toks(45, cfg["vocab"], 5), toks(38, cfg["vocab"], 6)
    s1 = pm.cache.alloc_slot()
    pm.forward([(s1, a, [])])
    pm.cache.free_slot(s1)
    free_before = list(pm.cache._free)
    s2 = pm.cache.alloc_slot()
    assert s2 == free_before[0]
    # take slots until the dirty one comes round again
    held = [s2]
    while s1 not in held:
        held.append(pm.cache.alloc_slot())
    got = torch.cat([pm.forward([(s1, b[:20], range(20))]), pm.forward([(s1, b[20:], range(18))])])
    for s in held:
        pm.cache.free_slot(s)
    assert H.row_err(got, O.forward(om, b)) < TOL32


def test_long_decoding_wraps_the_rings(mixed):
    cfg, om, pm = mixed
    seq = toks(150, cfg["vocab"], 7)                    # rings of 9, 33 and 1 rows wrap many times
    got = run(pm, [seq[:4]] + [[t] for t in seq[4:]])
    assert H.row_err(got, O.forward(om, seq)) < TOL32


def test_cache_growth_keeps_state(mixed):
    cfg, om, pm = mixed
    seq = toks(40, cfg["vocab"], 8)
    slot = pm.cache.alloc_slot()
    first = pm.forward([(slot, seq[:25], range(25))])
    pm.cache.grow(pm.cache.slots + 3)
    rest = pm.forward([(slot, seq[25:], range(15))])
    pm.cache.free_slot(slot)
    assert H.row_err(torch.cat([first, rest]), O.forward(om, seq)) < TOL32


@pytest.mark.parametrize("cfg", [H.ALIGNED, H.MIXED], ids=["aligned", "mixed"])
def test_bfloat16_mode(cfg):
    t = H.random_tensors(cfg, seed=3)
    om, pm = H.oracle_model(cfg, t), H.product_model(cfg, t, torch.bfloat16)
    seq = toks(64, cfg["vocab"], 9)
    ref = O.forward(om, seq)
    # bf16 rounding of a router logit can swap two nearly tied experts at a position: bound the bulk tightly and the
    # worst row loosely
    whole = run(pm, [seq])
    parts = run(pm, [seq[:30], seq[30:32]] + [[t] for t in seq[32:]])
    for got, want in ((whole, ref), (parts, ref), (parts, whole)):
        assert H.rel_err(got, want) < 4e-2 and H.row_err(got, want) < 0.3


def test_aligned_sizes_float32():
    t = H.random_tensors(H.ALIGNED, seed=4)
    om, pm = H.oracle_model(H.ALIGNED, t), H.product_model(H.ALIGNED, t, torch.float32)
    seq = toks(75, H.ALIGNED["vocab"], 11)
    assert H.row_err(run(pm, cut(seq, [40, 2, 1, 1, 31])), O.forward(om, seq)) < TOL32


def test_engine_greedy_generation_and_queue(tmp_path):
    from umbrella_b200.speculation.auto_engine import AutoEngine
    cfg = H.ALIGNED
    t = H.random_tensors(cfg, seed=5)
    om = H.oracle_model(cfg, t)
    path = H.write_checkpoint(str(tmp_path / "ckpt"), cfg, t)
    eng = AutoEngine.from_config("cuda:0", engine="batch", model=path, dtype="float32", max_batch=2, temperature=0.0)
    eng.initialize()
    prompts = [toks(n, cfg["vocab"], 30 + n) for n in (9, 1, 17)]
    outs = eng.generate_batch(prompts, max_new_tokens=6)            # three requests, batches of two: the queue runs twice
    for p, o in zip(prompts, outs):
        assert o == O.greedy(om, p, 6)
    assert eng.model.cache.live_slots == 0
    one = eng.generate(input_ids=prompts[0], max_new_tokens=6)
    assert one["generated_tokens"] == outs[0]
    assert eng._prefill(torch.tensor([prompts[2]]))
    tokens, _, _ = eng.speculative_decoding(max_new_tokens=6)
    assert tokens[:6] == outs[2]
    eng.reset()
    eng.update_generation_args(temperature=0.8, topk=8, topp=0.9)
    sampled = eng.generate_batch(prompts[:2], max_new_tokens=5)
    assert all(len(s) == 5 and all(0 <= x < cfg["vocab"] for x in s) for s in sampled)
