"""Test-only helpers for the Zedotar family: small random models, built twice from the same tensors -- as the
oracle's plain dict (float64, oracle/zedotar.py) and as the product model (a checkpoint directory read by the
family's config reader and loader)."""
import json
import os

import torch

ATT = dict(type="attention", heads=4, kv_heads=2, dim=16, vdim=24, window=9, pool=4, scale=0.3,
           rot=dict(dims=8, base=100.0, scaling=dict(factor=4.0, low=1.0, high=3.0, original=40)))
AT2 = dict(type="attention_2", heads=4, kv_heads=2, dim=16, vdim=16, conv=3, scale=0.25,
           rot=dict(dims=12, base=1000.0, scaling=dict(factor=2.5, original=24, fast=6.0, slow=1.0)))
MLS = dict(type="mlstm", heads=3, dim=16, vdim=20, gate_cap=10.0)

# every branch: the three mixers, layers without a feed-forward, a window of 1 with blocks of 1, as many key heads as query
# heads, one head, no rotary / unscaled rotary / rotary on the whole head, no convolution (1 tap) and 4 taps, a window that
# is no multiple of the block size and a block larger than the window
MIXED = dict(width=64, vocab=96, eps=1e-5, softcap=12.0, layers=[
    dict(MLS, ff=48),
    dict(ATT, ff=48),
    dict(AT2, ff=None),
    dict(ATT, window=1, pool=1, kv_heads=4, rot=None, ff=40),
    dict(MLS, heads=1, dim=24, vdim=32, gate_cap=3.0, ff=None),
    dict(AT2, conv=1, heads=1, kv_heads=1, dim=32, vdim=32, rot=dict(dims=32, base=50.0, scaling=None), ff=48),
    dict(ATT, window=5, pool=7, heads=2, kv_heads=1, dim=32, vdim=8, rot=dict(dims=32, base=10.0, scaling=None), ff=None),
    dict(AT2, conv=4, ff=48),
])
# dimensions the bf16 tensor-core product takes (every K a multiple of 32), no soft cap, a window without pooled blocks
ALIGNED = dict(width=128, vocab=160, eps=1e-6, softcap=None, layers=[
    dict(ATT, heads=4, kv_heads=1, dim=32, vdim=32, window=20, pool=0, ff=64),
    dict(MLS, heads=4, dim=32, vdim=32, ff=64),
    dict(AT2, heads=4, kv_heads=4, dim=32, vdim=32, conv=2, ff=64),
    dict(ATT, heads=2, kv_heads=2, dim=64, vdim=64, window=33, pool=16, ff=None),
])


def _bf(t):
    return t.to(torch.bfloat16).to(torch.float32)          # values a bf16 checkpoint can hold


def random_tensors(cfg, seed=0):
    """name -> fp32 tensor (bf16-representable), with the family's checkpoint names."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    r = lambda o, k, gain=1.0: _bf(gain * k ** -0.5 * torch.randn(o, k, generator=g))
    vec = lambda n, s=0.2: _bf(s * torch.randn(n, generator=g))
    t = {"embed": _bf(torch.randn(cfg["vocab"], W, generator=g)), "head": r(cfg["vocab"], W), "final.norm": vec(W)}
    for i, L in enumerate(cfg["layers"]):
        p, H, D, V = f"l{i}.", L["heads"], L["dim"], L["vdim"]
        t[p + "norm1"] = vec(W)
        if L["type"] == "mlstm":
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"], t[p + "mix.g"] = r(H * D, W, 1.5), r(H * D, W, 1.5), r(H * V, W), r(H * V, W)
            t[p + "mix.i"], t[p + "mix.f"] = r(H, W, 3.0), r(H, W, 3.0)
            t[p + "mix.i.b"], t[p + "mix.f.b"] = vec(H, 1.0), _bf(2.0 + torch.randn(H, generator=g))
            t[p + "mix.norm"] = _bf(1 + 0.2 * torch.randn(H * V, generator=g))
        else:
            G = L["kv_heads"]
            t[p + "mix.q"], t[p + "mix.q.b"] = r(H * D, W, 2.0), vec(H * D, 0.5)
            t[p + "mix.k"], t[p + "mix.k.b"] = r(G * D, W, 2.0), vec(G * D, 0.5)
            if L["type"] == "attention":
                t[p + "mix.v"], t[p + "mix.v.b"] = r(G * V, W), vec(G * V, 0.5)
                t[p + "mix.g"] = r(H, W, 2.0)
            else:
                if L["conv"] > 1:
                    t[p + "mix.q.conv"], t[p + "mix.k.conv"] = r(H * D, L["conv"], 1.5), r(G * D, L["conv"], 1.5)
                t[p + "mix.pb"] = _bf(-2.0 + torch.randn(H, generator=g))
                t[p + "mix.g"] = r(H * V, W, 2.0)
        t[p + "mix.o"] = r(W, H * V)
        if L["ff"]:
            t[p + "norm2"] = vec(W)
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = r(L["ff"], W, 2.0), r(L["ff"], W), r(W, L["ff"])
    return t


def _rot(L):
    rot = L.get("rot")
    if not rot:
        return dict(dims=0, base=1.0, scaling=None)
    sc = rot.get("scaling")
    if sc:
        sc = dict(sc, kind="llama3" if L["type"] == "attention" else "yarn")
    return dict(dims=rot["dims"], base=rot["base"], scaling=sc)


def oracle_model(cfg, t):
    d = lambda n: t[n].double()
    layers = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        o = dict(type=L["type"], heads=L["heads"], dim=L["dim"], vdim=L["vdim"], norm1=d(p + "norm1"))
        names = ["q", "k", "g", "o"]
        if L["type"] == "mlstm":
            names += ["v", "i", "f", "norm"]
            o.update(gate_cap=L["gate_cap"], i_b=d(p + "mix.i.b"), f_b=d(p + "mix.f.b"))
        else:
            o.update(kv_heads=L["kv_heads"], scale=L["scale"], rot=_rot(L), q_b=d(p + "mix.q.b"), k_b=d(p + "mix.k.b"))
            if L["type"] == "attention":
                names += ["v"]
                o.update(window=L["window"], pool=L["pool"], v_b=d(p + "mix.v.b"))
            else:
                one = lambda n: torch.ones(n, 1, dtype=torch.float64)
                o.update(pb=d(p + "mix.pb"),
                         q_conv=d(p + "mix.q.conv") if L["conv"] > 1 else one(L["heads"] * L["dim"]),
                         k_conv=d(p + "mix.k.conv") if L["conv"] > 1 else one(L["kv_heads"] * L["dim"]))
        o.update({n: d(p + "mix." + n) for n in names})
        o["mlp"], o["norm2"] = None, None
        if L["ff"]:
            o["norm2"], o["mlp"] = d(p + "norm2"), tuple(d(p + "mlp." + n) for n in ("gate", "up", "down"))
        layers.append(o)
    return dict(width=cfg["width"], vocab=cfg["vocab"], eps=cfg["eps"], softcap=cfg["softcap"], embed=d("embed"),
                head=d("head"), final_norm=d("final.norm"), layers=layers)


def config_json(cfg):
    """The family's config.json for ``cfg``."""
    layers = []
    for L in cfg["layers"]:
        mixer = dict(heads=L["heads"], dim=L["dim"], vdim=L["vdim"])
        if L["type"] == "mlstm":
            mixer["gate_cap"] = L["gate_cap"]
        else:
            mixer.update(kv_heads=L["kv_heads"], scale=L["scale"])
            if L.get("rot"):
                rot = dict(dims=L["rot"]["dims"], base=L["rot"]["base"])
                if L["rot"].get("scaling"):
                    rot["scaling"] = L["rot"]["scaling"]
                mixer["rot"] = rot
            if L["type"] == "attention":
                mixer["mask"] = dict(size=L["window"], pool=L["pool"]) if L["pool"] else dict(size=L["window"])
            else:
                mixer["conv"] = L["conv"]
        layers.append(dict(type=L["type"], mixer=mixer, mlp=dict(kind="dense", ff=L["ff"]) if L["ff"] else None))
    out = dict(architecture="Zedotar", width=cfg["width"], vocab=cfg["vocab"], norm=dict(eps=cfg["eps"]), layers=layers)
    if cfg["softcap"]:
        out["logit_softcap"] = cfg["softcap"]
    return out


def write_checkpoint(path, cfg, t):
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    json.dump(config_json(cfg), open(os.path.join(path, "config.json"), "w"))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}, os.path.join(path, "model.safetensors"))
    return path


def product_model(cfg, t, dtype=torch.float32, device="cuda:0", slots=4, tmp=None, **kw):
    """The product model over the same tensors, through the registry, the family's config reader and its loader."""
    import tempfile
    from umbrella_b200.models.auto_model import AutoModelLM
    d = write_checkpoint(tmp or tempfile.mkdtemp(prefix="zedckpt"), cfg, t)
    m = AutoModelLM.from_pretrained(d, device=device, dtype=dtype, slots=slots, **kw)
    m.alloc()
    return m


def row_err(a, b):
    """Largest per-row rms difference relative to the rms of the whole reference."""
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).pow(2).mean(-1).sqrt().max() / b.pow(2).mean().sqrt().clamp_min(1e-30))


def row_errs(a, b):
    """Per-row rms difference relative to the rms of the whole reference."""
    a, b = a.double().cpu(), b.double().cpu()
    return (a - b).pow(2).mean(-1).sqrt() / b.pow(2).mean().sqrt().clamp_min(1e-30)
