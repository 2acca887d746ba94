"""Plain, slow statement of the sequence-state decoder mechanisms, one function per mechanism, in float64 on the
CPU, written from the equations -- the oracle the CUDA path is tested against.  It shares no code with
umbrella_b200: a model is a plain dict

    {"width", "vocab", "groups", "eps", "embed", "head", "final_norm", "layers": [layer dict, ...]}
    layer: {"type": "retention" | "latent", "norm", "shift" | None, "depth" | None, "o", "mlp" | None,
            retention: "heads","dim","vdim","rot_dims","rot_base","decay", "q","k","v","g"
            latent:    "heads","dim","vdim","scale","window", "dq","dq_norm","uq","dkv","dkv_norm","uk","uv"}
    mlp: {"router" | None, "top", "experts": [(gate, up, down)], "limit", "shared": (gate, up, down) | None, "shared_limit"}

Every function takes a whole sequence [n, .]; there is no cache, no state and no batching here: position i of the
result depends on tokens 0..i of that one sequence, which is what the product must reproduce however it is fed.
"""
import math

import torch

F64 = torch.float64


def group_rms_norm(x, w, groups, eps):
    """x [n, d] split into `groups` equal consecutive parts, each divided by sqrt(mean(part^2) + eps); times w."""
    n, d = x.shape
    parts = x.reshape(n, groups, d // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    return parts.reshape(n, d) * w


def rms_norm(x, eps, w=None):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def token_shift(h, mu):
    """h_t + (h_(t-1) - h_t) * mu with h_(-1) = 0."""
    prev = torch.zeros_like(h)
    prev[1:] = h[:-1]
    return h + (prev - h) * mu


def rotate_half(x, rot_dims, base, positions=None):
    """x [n, heads, dim]: dimension i < rot_dims/2 pairs with i + rot_dims/2; angle = position * base^(-2i/rot_dims)."""
    if rot_dims == 0:
        return x
    n, half = x.shape[0], rot_dims // 2
    pos = torch.arange(n, dtype=F64) if positions is None else positions.to(F64)
    out = x.clone()
    for i in range(half):
        a = pos * base ** (-2.0 * i / rot_dims)
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[:, :, i], x[:, :, i + half]
        out[:, :, i] = u * c - v * s
        out[:, :, i + half] = v * c + u * s
    return out


def retention_recurrence(q, k, v, decay):
    """q, k [n, heads, dim], v [n, heads, vdim]: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t (no softmax)."""
    n, H, D = q.shape
    o = torch.zeros(n, H, v.shape[2], dtype=F64)
    for h in range(H):
        S = torch.zeros(D, v.shape[2], dtype=F64)
        for t in range(n):
            S = decay[h] * S + torch.outer(k[t, h], v[t, h])
            o[t, h] = S.T @ q[t, h]
    return o


def retention_mixer(hs, L, eps):
    n, H, D, V = hs.shape[0], L["heads"], L["dim"], L["vdim"]
    q = (hs @ L["q"].T).reshape(n, H, D)
    k = (hs @ L["k"].T).reshape(n, H, D)
    v = (hs @ L["v"].T).reshape(n, H, V)
    q = rotate_half(q, L["rot_dims"], L["rot_base"])
    k = rotate_half(k, L["rot_dims"], L["rot_base"]) * D ** -0.5
    o = rms_norm(retention_recurrence(q, k, v, L["decay"]), eps).reshape(n, H * V)
    g = hs @ L["g"].T
    return (o * (g * torch.sigmoid(g))) @ L["o"].T


def windowed_softmax_attention(q, k, v, scale, window):
    """q, k [n, heads, dim], v [n, heads, vdim]; position i sees j with 0 <= i - j < window."""
    n, H, _ = q.shape
    out = torch.zeros(n, H, v.shape[2], dtype=F64)
    for i in range(n):
        lo = max(0, i - window + 1)
        for h in range(H):
            s = (k[lo:i + 1, h] @ q[i, h]) * scale
            p = torch.softmax(s, 0)
            out[i, h] = p @ v[lo:i + 1, h]
    return out


def latent_attention_mixer(hs, L, eps):
    n, H, D, V = hs.shape[0], L["heads"], L["dim"], L["vdim"]
    cq = rms_norm(hs @ L["dq"].T, eps, L["dq_norm"])
    q = (cq @ L["uq"].T).reshape(n, H, D)
    c = rms_norm(hs @ L["dkv"].T, eps, L["dkv_norm"])
    k = (c @ L["uk"].T).reshape(n, H, D)
    v = (c @ L["uv"].T).reshape(n, H, V)
    return windowed_softmax_attention(q, k, v, L["scale"], L["window"]).reshape(n, H * V) @ L["o"].T


def gated_expert(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ down.T


def route_top(h, router, top):
    """-> (chosen experts [n, top], their weights: softmax over the chosen logits only)."""
    z = h @ router.T
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, -1)


def feed_forward(h, M):
    out = torch.zeros(h.shape[0], M["experts"][0][2].shape[0] if M["experts"] else M["shared"][2].shape[0], dtype=F64)
    if M.get("router") is not None:
        idx, w = route_top(h, M["router"], M["top"])
        for t in range(h.shape[0]):
            for j in range(M["top"]):
                g, u, d = M["experts"][int(idx[t, j])]
                out[t] += w[t, j] * gated_expert(h[t:t + 1], g, u, d, M["limit"])[0]
    if M.get("shared") is not None:
        out = out + gated_expert(h, *M["shared"], M["shared_limit"])
    return out


def depth_average(stack, w):
    return sum(w[j] * stack[j] for j in range(len(stack)))


def forward(model, tokens, layers_out=None):
    """Logits [n, vocab] of one sequence fed whole."""
    x = model["embed"][torch.as_tensor(tokens)]
    stack = [x]
    for L in model["layers"]:
        h = group_rms_norm(x, L["norm"], model["groups"], model["eps"])
        hs = token_shift(h, L["shift"]) if L.get("shift") is not None else h
        mix = retention_mixer(hs, L, model["eps"]) if L["type"] == "retention" else latent_attention_mixer(hs, L, model["eps"])
        new = x + (mix + feed_forward(h, L["mlp"])) if L.get("mlp") is not None else x + mix
        stack.append(new)
        x = depth_average(stack, L["depth"]) if L.get("depth") is not None else new
        if layers_out is not None:
            layers_out.append(x)
    return group_rms_norm(x, model["final_norm"], model["groups"], model["eps"]) @ model["head"].T


def greedy(model, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(model, toks)[-1].argmax()))
    return toks[len(prompt):]
