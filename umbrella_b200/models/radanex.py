"""Radanex: a hybrid sequence-state decoder family -- retention (decayed linear attention with rotary positions) and
sliding-window latent attention mixers in any order, each layer with a token-shifted mixer input, a routed
mixture of experts plus a shared expert run in parallel with the mixer off one grouped RMS norm, and a learned
depth-weighted average over all earlier residual streams.

This module is the family's front: config.json -> ``SeqModelSpec``, checkpoint tensor names -> ``load_layer`` dicts,
seeded synthetic weights for benchmarks and tests.  The computation is models/seq_model.py + csrc/seq.

config.json keys read here:
    architecture = "Radanex"; width; vocab; norm.eps, norm.groups;
    layers[i].type = "retention" | "latent_attention";
    layers[i].mixer: heads, dim, vdim and
        retention:        decay [heads], rot.dims, rot.base
        latent_attention: q_rank, kv_rank, scale, mask.size (window)
    layers[i].mlp = null | {kind: "moe", router: {experts, top}, expert: {ff, limit}, shared: {ff, limit} | null}
Tensors (safetensors, [out, in]): embed, head, final.norm, and per layer ``l<i>.``: norm1, shift, dwa, mix.{q,k,v,g,o}
or mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,o}, mlp.router, mlp.e<j>.{gate,up,down}, mlp.shared.{gate,up,down}.
"""
from __future__ import annotations

import json
import os

import torch

from .seq_model import SeqLayerSpec, SeqMlpSpec, SeqModelSpec, SeqStateModel

ARCHITECTURE = "Radanex"


def spec_from_config(cfg: dict) -> SeqModelSpec:
    if cfg.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config: architecture = {cfg.get('architecture')!r}")
    layers = []
    for entry in cfg["layers"]:
        kind, mx = entry["type"], entry["mixer"]
        l = SeqLayerSpec(mixer=kind, heads=int(mx["heads"]), dim=int(mx["dim"]), vdim=int(mx["vdim"]))
        if kind == "retention":
            rot = mx.get("rot") or {}
            l.rot_dims, l.rot_base = int(rot.get("dims", 0)), float(rot.get("base", 10000.0))
            l.decay = [float(x) for x in mx["decay"]]
            if len(l.decay) != l.heads:
                raise ValueError("retention: one decay per head")
        elif kind == "latent_attention":
            l.q_rank, l.kv_rank, l.scale = int(mx["q_rank"]), int(mx["kv_rank"]), float(mx["scale"])
            l.window = int(mx["mask"]["size"])
        else:
            raise ValueError(f"unknown layer type '{kind}'")
        mlp = entry.get("mlp")
        if mlp is not None:
            if mlp.get("kind", "moe") != "moe":
                raise ValueError(f"unknown feed-forward kind '{mlp.get('kind')}'")
            m = SeqMlpSpec()
            if mlp.get("router"):
                m.experts, m.top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
                m.ff, m.limit = int(mlp["expert"]["ff"]), float(mlp["expert"]["limit"])
            if mlp.get("shared"):
                m.shared_ff, m.shared_limit = int(mlp["shared"]["ff"]), float(mlp["shared"]["limit"])
            l.mlp = m
        layers.append(l)
    eos = cfg.get("eos_token_id", [])
    return SeqModelSpec(width=int(cfg["width"]), vocab=int(cfg["vocab"]), layers=layers,
                        norm_groups=int(cfg["norm"]["groups"]), norm_eps=float(cfg["norm"]["eps"]),
                        eos_token_id=list(eos) if isinstance(eos, (list, tuple)) else [int(eos)])


def is_radanex_dir(path) -> bool:
    f = os.path.join(str(path), "config.json")
    if not os.path.isfile(f):
        return False
    try:
        return json.load(open(f)).get("architecture") == ARCHITECTURE
    except (OSError, ValueError):
        return False


def layer_tensor_names(spec: SeqModelSpec, i: int) -> dict:
    """load_layer key -> checkpoint tensor name(s) of layer i."""
    l, p = spec.layers[i], f"l{i}."
    names = {"norm": p + "norm1", "shift": p + "shift", "depth": p + "dwa", "o": p + "mix.o"}
    if l.mixer == "retention":
        names.update({k: p + "mix." + k for k in ("q", "k", "v", "g")})
    else:
        names.update({"dq": p + "mix.dq", "dq_norm": p + "mix.dq.norm", "uq": p + "mix.uq", "dkv": p + "mix.dkv",
                      "dkv_norm": p + "mix.dkv.norm", "uk": p + "mix.uk", "uv": p + "mix.uv"})
    if l.mlp is not None:
        if l.mlp.experts:
            names["router"] = p + "mlp.router"
            names["experts"] = [tuple(f"{p}mlp.e{e}.{n}" for n in ("gate", "up", "down")) for e in range(l.mlp.experts)]
        if l.mlp.shared_ff:
            names["shared"] = tuple(f"{p}mlp.shared.{n}" for n in ("gate", "up", "down"))
    return names


class Radanex(SeqStateModel):
    """``Radanex(path_or_spec, ...)``; ``alloc()`` then ``load_checkpoint(path)`` or ``load_synthetic(seed)``."""

    def __init__(self, spec: SeqModelSpec, **kw):
        super().__init__(spec, **kw)
        for i, l in enumerate(spec.layers):
            l.shift, l.depth_average = True, True          # every layer of this family shifts and averages

    def load_checkpoint(self, path: str):
        from .checkpoint import SafetensorsIndex
        idx = SafetensorsIndex(path)
        get = idx.get
        self.load_head(get("embed"), get("head"), get("final.norm"))
        for i in range(self.num_layers):
            w = {}
            for key, name in layer_tensor_names(self.spec, i).items():
                if key == "experts":
                    w[key] = [tuple(get(n) for n in trio) for trio in name]
                elif key == "shared":
                    w[key] = tuple(get(n) for n in name)
                else:
                    w[key] = get(name)
            self.load_layer(i, w)
        idx.close()
        self.weights_source = path
        return self

    def load_synthetic(self, seed: int = 1234, gen_device: str | None = None):
        """Seeded random weights of the architecture (benchmarks, tests)."""
        dev = gen_device or str(self.device)
        head = synth_head(self.spec, seed, dev)
        self.load_head(head["embed"], head["head"], head["final_norm"])
        for i in range(self.num_layers):
            self.load_layer(i, synth_layer(self.spec, i, seed, dev))
        self.weights_source = f"synthetic(seed={seed})"
        return self


def _rand(gen, shape, scale, dev):
    return (scale * torch.randn(shape, generator=gen, device=dev)).to(torch.bfloat16)


def synth_head(spec: SeqModelSpec, seed: int, dev="cpu") -> dict:
    gen = torch.Generator(device=dev).manual_seed(seed - 1)
    return {"embed": _rand(gen, (spec.vocab, spec.width), 1.0, dev),
            "head": _rand(gen, (spec.vocab, spec.width), spec.width ** -0.5, dev),
            "final_norm": (1 + 0.1 * torch.randn(spec.width, generator=gen, device=dev)).to(torch.bfloat16)}


def synth_layer(spec: SeqModelSpec, i: int, seed: int, dev="cpu") -> dict:
    """bf16-representable tensors (as a checkpoint would hold them), so that every dtype mode sees the same weights."""
    gen = torch.Generator(device=dev).manual_seed(seed + i)
    l, W = spec.layers[i], spec.width
    r = lambda o, k, gain=1.0: _rand(gen, (o, k), gain * k ** -0.5, dev)
    vec = lambda n: (1 + 0.1 * torch.randn(n, generator=gen, device=dev)).to(torch.bfloat16)
    w = {"norm": vec(W), "shift": torch.rand(W, generator=gen, device=dev).to(torch.bfloat16),
         "depth": (torch.softmax(torch.randn(i + 2, generator=gen, device=dev), 0)).to(torch.bfloat16)}
    hv = l.heads * l.vdim
    if l.mixer == "retention":
        w.update(q=r(l.heads * l.dim, W), k=r(l.heads * l.dim, W), v=r(hv, W), g=r(hv, W))
    else:
        w.update(dq=r(l.q_rank, W), dq_norm=vec(l.q_rank), uq=r(l.heads * l.dim, l.q_rank, 2.0), dkv=r(l.kv_rank, W),
                 dkv_norm=vec(l.kv_rank), uk=r(l.heads * l.dim, l.kv_rank, 2.0), uv=r(hv, l.kv_rank))
    w["o"] = r(W, hv)
    if l.mlp is not None:
        m = l.mlp
        if m.experts:
            w["router"] = r(m.experts, W, 2.0)
            w["experts"] = [(r(m.ff, W), r(m.ff, W), r(W, m.ff)) for _ in range(m.experts)]
        if m.shared_ff:
            w["shared"] = (r(m.shared_ff, W), r(m.shared_ff, W), r(W, m.shared_ff))
    return w


def from_pretrained(path: str, device="cuda:0", dtype=torch.bfloat16, **kw) -> Radanex:
    """Model of a checkpoint directory (config.json + model.safetensors); ``alloc()`` loads the weights."""
    spec = spec_from_config(json.load(open(os.path.join(path, "config.json"))))
    model = Radanex(spec, device=device, dtype=dtype, model_name=path, **kw)
    base_alloc = model.alloc

    def alloc(**kwargs):
        base_alloc(**kwargs)
        if kwargs.get("synthetic") or "synthetic_seed" in kwargs:
            model.load_synthetic(kwargs.get("synthetic_seed", 1234))
        else:
            model.load_checkpoint(path)
        torch.cuda.synchronize(model.device)
        return model
    model.alloc = alloc
    return model
