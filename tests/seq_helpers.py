"""Test-only helpers for the sequence-state decoders: small random models, built twice from the same tensors --
as the oracle's plain dict (float64, oracle/seqstate.py) and as the product model (SeqStateModel / a checkpoint
directory for the Radanex loader)."""
import json
import os

import torch

RET = dict(type="retention", heads=3, dim=16, vdim=32, rot_dims=8, rot_base=100.0, decay=[0.9, 0.97, 0.9990234375])
LAT = dict(type="latent", heads=2, dim=16, vdim=24, q_rank=40, kv_rank=48, window=9, scale=0.3)
MLP = dict(n_experts=5, top=2, ff=40, limit=1.5, shared_ff=24, shared_limit=2.5)

# a mixed stack that exercises every branch: both mixers, a layer without feed-forward, one without a shared expert,
# one with top = 1, rotary on part of the head, a window of 1
MIXED = dict(width=64, vocab=96, groups=2, eps=1e-5, layers=[
    dict(LAT, mlp=MLP),
    dict(RET, mlp=dict(MLP, shared_ff=0)),
    dict(LAT, window=33, heads=1, mlp=None),
    dict(RET, rot_dims=16, heads=1, decay=[0.75], mlp=dict(MLP, top=1, n_experts=3)),
    dict(LAT, window=1, mlp=dict(MLP, n_experts=0)),
])
# dimensions the bf16 tensor-core product takes (every K a multiple of 32)
ALIGNED = dict(width=128, vocab=160, groups=1, eps=1e-6, layers=[
    dict(RET, heads=4, dim=32, vdim=32, rot_dims=16, decay=[0.875, 0.9375, 0.984375, 0.998046875], mlp=dict(MLP, ff=64, shared_ff=32, n_experts=4)),
    dict(LAT, heads=4, dim=32, vdim=32, q_rank=64, kv_rank=64, window=20, mlp=dict(MLP, ff=64, shared_ff=32, n_experts=4)),
])


def _bf(t):
    return t.to(torch.bfloat16).to(torch.float32)          # values a bf16 checkpoint can hold


def random_tensors(cfg, seed=0):
    """name -> fp32 tensor (bf16-representable), with the checkpoint names of the Radanex family."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    r = lambda o, k, gain=1.0: _bf(gain * k ** -0.5 * torch.randn(o, k, generator=g))
    vec = lambda n: _bf(1 + 0.2 * torch.randn(n, generator=g))
    t = {"embed": _bf(torch.randn(cfg["vocab"], W, generator=g)), "head": r(cfg["vocab"], W), "final.norm": vec(W)}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        hv = L["heads"] * L["vdim"]
        t[p + "norm1"], t[p + "shift"] = vec(W), _bf(torch.rand(W, generator=g))
        t[p + "dwa"] = _bf(torch.softmax(torch.randn(i + 2, generator=g), 0) * 1.3)
        if L["type"] == "retention":
            for n, rows in (("q", L["heads"] * L["dim"]), ("k", L["heads"] * L["dim"]), ("v", hv), ("g", hv)):
                t[p + "mix." + n] = r(rows, W, 1.5)
        else:
            t[p + "mix.dq"], t[p + "mix.dq.norm"] = r(L["q_rank"], W), vec(L["q_rank"])
            t[p + "mix.uq"] = r(L["heads"] * L["dim"], L["q_rank"], 2.0)
            t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = r(L["kv_rank"], W), vec(L["kv_rank"])
            t[p + "mix.uk"] = r(L["heads"] * L["dim"], L["kv_rank"], 2.0)
            t[p + "mix.uv"] = r(hv, L["kv_rank"])
        t[p + "mix.o"] = r(W, hv)
        M = L["mlp"]
        if M is not None:
            if M["n_experts"]:
                t[p + "mlp.router"] = r(M["n_experts"], W, 3.0)
                for e in range(M["n_experts"]):
                    t[f"{p}mlp.e{e}.gate"], t[f"{p}mlp.e{e}.up"], t[f"{p}mlp.e{e}.down"] = r(M["ff"], W, 2.0), r(M["ff"], W, 2.0), r(W, M["ff"])
            if M["shared_ff"]:
                t[p + "mlp.shared.gate"], t[p + "mlp.shared.up"] = r(M["shared_ff"], W, 2.0), r(M["shared_ff"], W, 2.0)
                t[p + "mlp.shared.down"] = r(W, M["shared_ff"])
    return t


def oracle_model(cfg, t):
    d = lambda n: t[n].double()
    layers = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        o = {k: v for k, v in L.items() if k != "mlp"}
        o.update(norm=d(p + "norm1"), shift=d(p + "shift"), depth=d(p + "dwa"), o=d(p + "mix.o"))
        names = ("q", "k", "v", "g") if L["type"] == "retention" else ("dq", "uq", "dkv", "uk", "uv")
        o.update({n: d(p + "mix." + n) for n in names})
        if L["type"] == "latent":
            o["dq_norm"], o["dkv_norm"] = d(p + "mix.dq.norm"), d(p + "mix.dkv.norm")
        M = L["mlp"]
        o["mlp"] = None
        if M is not None:
            o["mlp"] = dict(router=d(p + "mlp.router") if M["n_experts"] else None, top=M["top"], limit=M["limit"],
                            experts=[tuple(d(f"{p}mlp.e{e}.{n}") for n in ("gate", "up", "down")) for e in range(M["n_experts"])],
                            shared=tuple(d(f"{p}mlp.shared.{n}") for n in ("gate", "up", "down")) if M["shared_ff"] else None,
                            shared_limit=M["shared_limit"])
        layers.append(o)
    return dict(width=cfg["width"], vocab=cfg["vocab"], groups=cfg["groups"], eps=cfg["eps"], embed=d("embed"),
                head=d("head"), final_norm=d("final.norm"), layers=layers)


def config_json(cfg):
    """The family's config.json for ``cfg``."""
    layers = []
    for L in cfg["layers"]:
        if L["type"] == "retention":
            mixer = dict(heads=L["heads"], dim=L["dim"], vdim=L["vdim"], decay=L["decay"],
                         rot=dict(dims=L["rot_dims"], base=L["rot_base"]))
        else:
            mixer = dict(heads=L["heads"], dim=L["dim"], vdim=L["vdim"], q_rank=L["q_rank"], kv_rank=L["kv_rank"],
                         scale=L["scale"], mask=dict(size=L["window"]))
        M, mlp = L["mlp"], None
        if M is not None:
            mlp = dict(kind="moe", router=dict(experts=M["n_experts"], top=M["top"]) if M["n_experts"] else None,
                       expert=dict(ff=M["ff"], limit=M["limit"]),
                       shared=dict(ff=M["shared_ff"], limit=M["shared_limit"]) if M["shared_ff"] else None)
        layers.append(dict(type="retention" if L["type"] == "retention" else "latent_attention", mixer=mixer, mlp=mlp))
    return dict(architecture="Radanex", width=cfg["width"], vocab=cfg["vocab"],
                norm=dict(eps=cfg["eps"], groups=cfg["groups"]), layers=layers)


def write_checkpoint(path, cfg, t):
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    json.dump(config_json(cfg), open(os.path.join(path, "config.json"), "w"))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}, os.path.join(path, "model.safetensors"))
    return path


def product_model(cfg, t, dtype=torch.float32, device="cuda:0", slots=4, tmp=None, **kw):
    """The product model over the same tensors, through the family's config reader and checkpoint loader."""
    import tempfile
    from umbrella_b200.models.auto_model import AutoModelLM
    d = write_checkpoint(tmp or tempfile.mkdtemp(prefix="seqckpt"), cfg, t)
    m = AutoModelLM.from_pretrained(d, device=device, dtype=dtype, slots=slots, **kw)
    m.alloc()
    return m


def rel_err(a, b):
    """rms(a - b) / rms(b) over everything."""
    a, b = a.double().cpu(), b.double().cpu()
    return float(((a - b).pow(2).mean() / b.pow(2).mean().clamp_min(1e-30)).sqrt())


def row_err(a, b):
    """Largest per-row rms difference relative to the rows' rms."""
    a, b = a.double().cpu(), b.double().cpu()
    return float(((a - b).pow(2).mean(-1).sqrt() / b.pow(2).mean(-1).sqrt().clamp_min(1e-30)).max())
