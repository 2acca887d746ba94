"""Plain, slow statement of the Zedotar mechanisms, one function per mechanism, in float64 on the CPU, written from
the equations -- the oracle the CUDA path is tested against.  It shares no code with umbrella_b200.  A model is a dict

    {"width", "vocab", "eps", "softcap", "embed", "head", "final_norm", "layers": [layer dict, ...]}
    layer: {"type": "attention" | "attention_2" | "mlstm", "norm1", "norm2" | None, "mlp": (gate, up, down) | None, ...}
      attention:   heads, kv_heads, dim, vdim, scale, window, pool, rot (dict), q, q_b, k, k_b, v, v_b, g, o
      attention_2: heads, kv_heads, dim, vdim, scale, rot (dict), q, q_b, k, k_b, q_conv, k_conv, pb, g, o
      mlstm:       heads, dim, vdim, gate_cap, q, k, v, i, i_b, f, f_b, g, norm, o
    rot: {"dims", "base", "scaling": None | {"kind": "llama3", factor, low, high, original}
                                          | {"kind": "yarn", factor, original, fast, slow}}

Every function takes a whole sequence [n, .]: no cache, no state, no batching.  Position i of a result depends on
tokens 0..i of that one sequence, which is what the product must reproduce however it is fed.
"""
import math

import torch

F64 = torch.float64


# ---------------------------------------------------------------------------------------------- norms, activations
def rms_norm_zero_centred(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * (1 + w): the weight is stored around zero."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * (1.0 + w)


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gated_gelu_mlp(h, gate, up, down):
    return (gelu_tanh(h @ gate.T) * (h @ up.T)) @ down.T


def softcap(z, cap):
    return cap * torch.tanh(z / cap)


# ---------------------------------------------------------------------------------------------- rotary positions
def rotary_frequencies(rot):
    """-> (f [dims / 2], magnitude): the frequencies after the scaling rule, and the factor on cos and sin."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    mag = 1.0
    if sc is None:
        pass
    elif sc["kind"] == "llama3":
        out = []
        for fi in f:
            wave = 2.0 * math.pi / fi
            if wave < sc["original"] / sc["high"]:
                out.append(fi)
            elif wave > sc["original"] / sc["low"]:
                out.append(fi / sc["factor"])
            else:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1.0 - s) * fi / sc["factor"] + s * fi)
        f = out
    elif sc["kind"] == "yarn":
        turn = lambda t: dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo = max(math.floor(turn(sc["fast"])), 0)
        hi = min(math.ceil(turn(sc["slow"])), dims - 1)
        out = []
        for i, fi in enumerate(f):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(fi / sc["factor"] * ramp + fi * (1.0 - ramp))
        f = out
        mag = 0.1 * math.log(sc["factor"]) + 1.0
    else:
        raise ValueError(sc["kind"])
    return torch.tensor(f, dtype=F64), mag


def rotate(x, rot):
    """x [n, heads, dim], position = row index; pairs (i, i + dims/2) of the first `dims` dimensions turn by p f_i."""
    dims = rot["dims"]
    if dims == 0:
        return x
    f, mag = rotary_frequencies(rot)
    half = dims // 2
    a = torch.arange(x.shape[0], dtype=F64)[:, None] * f[None, :]
    c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    out = x.clone()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ---------------------------------------------------------------------------------------------- short convolution
def causal_conv(u, w):
    """u [n, channels], w [channels, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    n, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(n):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                y[t] += w[:, j] * u[src]
    return y


# ---------------------------------------------------------------------------------------------- attention kinds
def pooled_window_attention(q, k, v, window, pool, scale):
    """q [n, H, D], k [n, G, D], v [n, G, V].  Row i sees tokens j with 0 <= i - j < window and, for every block b of
    `pool` tokens with b pool + pool - 1 <= i - window, the block's mean key and mean value.  One softmax over both,
    with a sink of score 0 and no value: p = exp(s) / (1 + sum exp(s)).  pool = 0: no blocks."""
    n, H, D = q.shape
    G, V = k.shape[1], v.shape[2]
    out = torch.zeros(n, H, V, dtype=F64)
    for h in range(H):
        g = h // (H // G)
        for i in range(n):
            keys, vals = [], []
            b = 0
            while pool and b * pool + pool - 1 <= i - window:
                keys.append(k[b * pool:(b + 1) * pool, g].mean(0))
                vals.append(v[b * pool:(b + 1) * pool, g].mean(0))
                b += 1
            for j in range(max(0, i - window + 1), i + 1):
                keys.append(k[j, g])
                vals.append(v[j, g])
            K, Vv = torch.stack(keys), torch.stack(vals)
            s = (K @ q[i, h]) * scale
            m = max(float(s.max()), 0.0)
            e = torch.exp(s - m)
            out[i, h] = (e[:, None] * Vv).sum(0) / (math.exp(-m) + e.sum())
    return out


def sigmoid_attention(q, k, v, scale, bias):
    """Causal, no softmax: out_i = sum_(j <= i) sigmoid(q_i . k_j scale + bias_h) v_j."""
    n, H, D = q.shape
    G = k.shape[1]
    out = torch.zeros(n, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        for i in range(n):
            w = torch.sigmoid((k[:i + 1, g] @ q[i, h]) * scale + bias[h])
            out[i, h] = (w[:, None] * v[:i + 1, g]).sum(0)
    return out


def mlstm_recurrence(q, k, v, i_log, f_log):
    """q, k [n, H, D], v [n, H, V], gates [n, H] (logarithms).  Stabilised matrix memory:
    m_t = max(f_t + m_(t-1), i_t) with m_0 = 0; S_t = e^(f_t + m_(t-1) - m_t) S_(t-1) + e^(i_t - m_t) k_t v_t^T, n_t the
    same with k_t alone; o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6)."""
    n, H, D = q.shape
    V = v.shape[2]
    out = torch.zeros(n, H, V, dtype=F64)
    for h in range(H):
        S, nv, m = torch.zeros(D, V, dtype=F64), torch.zeros(D, dtype=F64), 0.0
        for t in range(n):
            m_new = max(float(f_log[t, h]) + m, float(i_log[t, h]))
            a, b = math.exp(float(f_log[t, h]) + m - m_new), math.exp(float(i_log[t, h]) - m_new)
            S = a * S + b * torch.outer(k[t, h], v[t, h])
            nv = a * nv + b * k[t, h]
            m = m_new
            out[t, h] = (S.T @ q[t, h]) / (max(abs(float(nv @ q[t, h])), math.exp(-m)) + 1e-6)
    return out


# ---------------------------------------------------------------------------------------------- mixers
def attention_mixer(h, L):
    n, H, G, D, V = h.shape[0], L["heads"], L["kv_heads"], L["dim"], L["vdim"]
    q = (h @ L["q"].T + L["q_b"]).reshape(n, H, D)
    k = (h @ L["k"].T + L["k_b"]).reshape(n, G, D)
    v = (h @ L["v"].T + L["v_b"]).reshape(n, G, V)
    q, k = rotate(q, L["rot"]), rotate(k, L["rot"])
    o = pooled_window_attention(q, k, v, L["window"], L["pool"], L["scale"])
    o = o * torch.sigmoid(h @ L["g"].T)[:, :, None]                      # one gate per head
    return o.reshape(n, H * V) @ L["o"].T


def attention_2_mixer(h, L):
    n, H, G, D = h.shape[0], L["heads"], L["kv_heads"], L["dim"]
    q = causal_conv(h @ L["q"].T + L["q_b"], L["q_conv"]).reshape(n, H, D)
    k = causal_conv(h @ L["k"].T + L["k_b"], L["k_conv"]).reshape(n, G, D)
    v = k                                                                # the values are the keys before rotation
    q, kr = rotate(q, L["rot"]), rotate(k, L["rot"])
    o = sigmoid_attention(q, kr, v, L["scale"], L["pb"]).reshape(n, H * D)
    return (o * torch.sigmoid(h @ L["g"].T)) @ L["o"].T


def mlstm_mixer(h, L, eps):
    n, H, D, V, cap = h.shape[0], L["heads"], L["dim"], L["vdim"], L["gate_cap"]
    q = (h @ L["q"].T).reshape(n, H, D) * D ** -0.5
    k = (h @ L["k"].T).reshape(n, H, D)
    v = (h @ L["v"].T).reshape(n, H, V)
    i_log = cap * torch.tanh((h @ L["i"].T + L["i_b"]) / cap)
    f_log = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ L["f"].T + L["f_b"]) / cap))
    o = unit_rms(mlstm_recurrence(q, k, v, i_log, f_log), eps).reshape(n, H * V)
    return (o * L["norm"] * torch.sigmoid(h @ L["g"].T)) @ L["o"].T


# ---------------------------------------------------------------------------------------------- the model
def forward(model, tokens, layer_out=False):
    """-> logits [n, vocab] (and the residual stream after every layer, [layers, n, width])."""
    x = model["embed"][torch.as_tensor(tokens, dtype=torch.long)].to(F64)
    eps, streams = model["eps"], []
    for L in model["layers"]:
        h = rms_norm_zero_centred(x, L["norm1"], eps)
        if L["type"] == "attention":
            x = x + attention_mixer(h, L)
        elif L["type"] == "attention_2":
            x = x + attention_2_mixer(h, L)
        elif L["type"] == "mlstm":
            x = x + mlstm_mixer(h, L, eps)
        else:
            raise ValueError(L["type"])
        if L["mlp"] is not None:
            x = x + gated_gelu_mlp(rms_norm_zero_centred(x, L["norm2"], eps), *L["mlp"])
        streams.append(x)
    logits = rms_norm_zero_centred(x, model["final_norm"], eps) @ model["head"].T
    if model.get("softcap"):
        logits = softcap(logits, model["softcap"])
    return (logits, torch.stack(streams)) if layer_out else logits
