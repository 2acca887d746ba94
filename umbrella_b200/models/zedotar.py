"""Zedotar: a pre-norm hybrid decoder family -- in any order given by its config.json, layers whose mixer is
  * ``attention``:   grouped-query attention with biases, rotary positions on part of each head (frequencies scaled by
                     wavelength), a sliding window plus one mean key/value per block of older tokens, a softmax with a
                     sink, and a sigmoid output gate per head;
  * ``attention_2``: grouped-query attention without a value projection (the values are the keys before the rotation),
                     a short causal convolution on q and k, YaRN-scaled rotary positions, causal sigmoid weights with a
                     bias per head instead of a softmax, and an element-wise sigmoid output gate;
  * ``mlstm``:       the matrix memory of xLSTM with soft-capped exponential gates and a running maximum,
each followed by a dense gelu(tanh)-gated feed-forward (or none).  Norms are RMS norms with weights stored around
zero; the logits pass a tanh soft cap.

This module is the family's front: config.json -> ``SeqModelSpec``, checkpoint tensor names -> ``load_layer`` dicts,
seeded synthetic weights for benchmarks and tests.  The computation is models/seq_model.py + csrc/seq: both
attention kinds are options of the framework's cached-attention mixer, mLSTM is a mixer of its own.

config.json keys read here:
    architecture = "Zedotar"; width; vocab; norm.eps; logit_softcap (optional);
    layers[i].type = "attention" | "attention_2" | "mlstm";
    layers[i].mixer: heads, dim, vdim and
        attention:   kv_heads, scale, mask.size, mask.pool, rot.{dims, base, scaling: {factor, low, high, original}}
        attention_2: kv_heads, scale, conv, rot.{dims, base, scaling: {factor, original, fast, slow}}
        mlstm:       gate_cap
    layers[i].mlp = null | {kind: "dense", ff}
Tensors (safetensors, [out, in]): embed, head, final.norm, and per layer ``l<i>.``: norm1, norm2, mix.{q,k,v,g,o} with
mix.{q,k,v}.b (attention), mix.{q,k}.conv and mix.pb (attention_2), mix.{i,f} with .b and mix.norm (mlstm),
mlp.{gate,up,down}.
"""
from __future__ import annotations

import json
import os

import torch

from .seq_model import (SeqLayerSpec, SeqMlpSpec, SeqModelSpec, SeqStateModel, rotary_inv_freq64,
                        scale_freq_by_wavelength, scale_freq_yarn)

ARCHITECTURE = "Zedotar"


def _rotary(l: SeqLayerSpec, rot: dict | None, kind: str):
    """Fills rot_dims / rot_base / inv_freq / rot_mag of ``l`` from a config ``rot`` entry; ``kind`` names the scaling rule."""
    if not rot or not int(rot.get("dims", 0)):
        return
    l.rot_dims, l.rot_base = int(rot["dims"]), float(rot["base"])
    if l.rot_dims % 2 or l.rot_dims > l.dim:
        raise ValueError("rot.dims must be even and at most the head size")
    f, sc = rotary_inv_freq64(l.rot_dims, l.rot_base), rot.get("scaling")
    if sc:
        if kind == "wavelength":
            f = scale_freq_by_wavelength(f, float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"]))
        else:
            f, l.rot_mag = scale_freq_yarn(f, l.rot_dims, l.rot_base, float(sc["factor"]), float(sc["original"]),
                                           float(sc["fast"]), float(sc["slow"]))
    l.inv_freq = [float(x) for x in f]


def spec_from_config(cfg: dict) -> SeqModelSpec:
    if cfg.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config: architecture = {cfg.get('architecture')!r}")
    layers = []
    for entry in cfg["layers"]:
        kind, mx = entry["type"], entry["mixer"]
        l = SeqLayerSpec(heads=int(mx["heads"]), dim=int(mx["dim"]), vdim=int(mx.get("vdim", mx["dim"])), form="prenorm", norm_offset=1.0,
                         shift=False, depth_average=False)
        if kind == "attention":
            l.mixer, l.kv_heads, l.scale = "cached_attention", int(mx.get("kv_heads", l.heads)), float(mx["scale"])
            l.attn_mode, l.gate_kind, l.bias = "softmax_sink", 1, True
            mask = mx.get("mask") or {}
            l.window, l.pool = int(mask.get("size", 0)), int(mask.get("pool", 0))
            if l.pool and not l.window:
                raise ValueError("attention: pooled blocks need a window")
            _rotary(l, mx.get("rot"), "wavelength")
        elif kind == "attention_2":
            l.mixer, l.kv_heads, l.scale = "cached_attention", int(mx.get("kv_heads", l.heads)), float(mx["scale"])
            l.attn_mode, l.gate_kind, l.bias, l.head_bias = "sigmoid", 2, True, True
            l.values_are_keys, l.taps, l.window = True, int(mx.get("conv", 1)), 0
            if l.vdim != l.dim:
                raise ValueError("attention_2: the values are the keys, so vdim must equal dim")
            _rotary(l, mx.get("rot"), "yarn")
        elif kind == "mlstm":
            l.mixer, l.gate_cap = "mlstm", float(mx["gate_cap"])
        else:
            raise ValueError(f"unknown layer type '{kind}'")
        if l.mixer == "cached_attention" and (l.kv_heads < 1 or l.heads % l.kv_heads):
            raise ValueError("heads must be a multiple of kv_heads")
        mlp = entry.get("mlp")
        if mlp is not None:
            if mlp.get("kind", "dense") != "dense":
                raise ValueError(f"unknown feed-forward kind '{mlp.get('kind')}'")
            l.mlp = SeqMlpSpec(shared_ff=int(mlp["ff"]), act="gelu_tanh")
        layers.append(l)
    eos = cfg.get("eos_token_id", [])
    return SeqModelSpec(width=int(cfg["width"]), vocab=int(cfg["vocab"]), layers=layers, norm_groups=1,
                        norm_eps=float(cfg["norm"]["eps"]), norm_offset=1.0,
                        logit_softcap=float(cfg.get("logit_softcap") or 0.0),
                        eos_token_id=list(eos) if isinstance(eos, (list, tuple)) else [int(eos)])


def layer_tensor_names(spec: SeqModelSpec, i: int) -> dict:
    """load_layer key -> checkpoint tensor name of layer i."""
    l, p = spec.layers[i], f"l{i}."
    names = {"norm": p + "norm1", "o": p + "mix.o", "q": p + "mix.q", "k": p + "mix.k", "g": p + "mix.g"}
    if l.mixer == "mlstm":
        names.update({"v": p + "mix.v", "i": p + "mix.i", "i_b": p + "mix.i.b", "f": p + "mix.f", "f_b": p + "mix.f.b",
                      "out_norm": p + "mix.norm"})
    else:
        names.update({"q_b": p + "mix.q.b", "k_b": p + "mix.k.b"})
        if not l.values_are_keys:
            names.update({"v": p + "mix.v", "v_b": p + "mix.v.b"})
        if l.taps > 1:
            names.update({"q_conv": p + "mix.q.conv", "k_conv": p + "mix.k.conv"})
        if l.head_bias:
            names["pb"] = p + "mix.pb"
    if l.mlp is not None:
        names["norm2"] = p + "norm2"
        names["dense"] = tuple(f"{p}mlp.{n}" for n in ("gate", "up", "down"))
    return names


class Zedotar(SeqStateModel):
    """``Zedotar(spec, ...)``; ``alloc()`` then ``load_checkpoint(path)`` or ``load_synthetic(seed)``."""

    def load_checkpoint(self, path: str):
        from .checkpoint import SafetensorsIndex
        idx = SafetensorsIndex(path)
        get = idx.get
        self.load_head(get("embed"), get("head"), get("final.norm"))
        for i in range(self.num_layers):
            w = {}
            for key, name in layer_tensor_names(self.spec, i).items():
                w[key] = tuple(get(n) for n in name) if isinstance(name, tuple) else get(name)
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
            "final_norm": _rand(gen, (spec.width,), 0.1, dev)}


def synth_layer(spec: SeqModelSpec, i: int, seed: int, dev="cpu") -> dict:
    """bf16 tensors (as a checkpoint would hold them), so that every dtype mode sees the same weights."""
    gen = torch.Generator(device=dev).manual_seed(seed + i)
    l, W = spec.layers[i], spec.width
    r = lambda o, k, gain=1.0: _rand(gen, (o, k), gain * k ** -0.5, dev)
    vec = lambda n, s=0.1: _rand(gen, (n,), s, dev)
    hv = l.heads * l.vdim
    w = {"norm": vec(W), "q": r(l.heads * l.dim, W), "o": r(W, hv, 0.5)}
    if l.mixer == "mlstm":
        w.update(k=r(l.heads * l.dim, W), v=r(hv, W), g=r(hv, W), i=r(l.heads, W), f=r(l.heads, W), i_b=vec(l.heads, 1.0),
                 f_b=(3.0 + torch.randn(l.heads, generator=gen, device=dev)).to(torch.bfloat16),
                 out_norm=(1 + 0.1 * torch.randn(hv, generator=gen, device=dev)).to(torch.bfloat16))
    else:
        w.update(k=r(l.kv_heads * l.dim, W), q_b=vec(l.heads * l.dim), k_b=vec(l.kv_heads * l.dim),
                 g=r(l.heads if l.gate_kind == 1 else hv, W))
        if not l.values_are_keys:
            w.update(v=r(l.kv_heads * l.vdim, W), v_b=vec(l.kv_heads * l.vdim))
        if l.taps > 1:
            w.update(q_conv=r(l.heads * l.dim, l.taps, 1.5), k_conv=r(l.kv_heads * l.dim, l.taps, 1.5))
        if l.head_bias:
            w["pb"] = (-4.0 + torch.randn(l.heads, generator=gen, device=dev)).to(torch.bfloat16)
    if l.mlp is not None:
        w["norm2"] = vec(W)
        w["dense"] = (r(l.mlp.shared_ff, W), r(l.mlp.shared_ff, W), r(W, l.mlp.shared_ff, 0.5))
    return w


def from_pretrained(path: str, device="cuda:0", dtype=torch.bfloat16, **kw) -> Zedotar:
    """Model of a checkpoint directory (config.json + model.safetensors); ``alloc()`` loads the weights."""
    spec = spec_from_config(json.load(open(os.path.join(path, "config.json"))))
    kw.pop("fresh_attention", None)
    model = Zedotar(spec, device=device, dtype=dtype, model_name=path, **kw)
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
