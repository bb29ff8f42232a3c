"""Kasovik, written out plainly: one function per mechanism, token by token where the design is a recurrence, all in
64-bit floats on the CPU. It shares nothing with the engine: tensors are taken by their stored names from a dict, and
every size comes from the configuration dict or a tensor's shape. The tests compare the engine with this.

Notation: x a token's row of the residual stream, h its normed copy, S a recurrent state [key channel, value channel].
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def embedding(w, cfg, tokens):
    """Scaled table rows plus a row of the bigram table chosen by (previous token, token); the first token of a
    sequence takes the table's last row."""
    e, b = cfg["embedding"], cfg["embedding"].get("bigram")
    x = w["embed"].to(F)[tokens] * e["scale"]
    if b is not None:
        rows = [b["buckets"] if i == 0 else (tokens[i - 1] * b["mul_prev"] + t * b["mul_cur"]) % b["buckets"]
                for i, t in enumerate(tokens)]
        x = x + w["bigram"].to(F)[rows]
    return x


def rotate(x, positions, base, dims):
    """x [T, heads, dim]: channel i < dims/2 pairs with channel i + dims/2; the rest pass."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    a = torch.tensor(positions, dtype=F)[:, None, None] * f
    u, v, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    return torch.cat((u * a.cos() - v * a.sin(), v * a.cos() + u * a.sin(), rest), -1)


def retention(w, p, m, h, eps):
    """Linear attention with one fixed decay per head: S ← decay·S + k vᵀ, o = Sᵀ q; no softmax, no denominator."""
    t, heads, dim, vdim = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].to(F).T).view(t, heads, dim)
    k = (h @ w[p + "k"].to(F).T).view(t, heads, dim)
    v = (h @ w[p + "v"].to(F).T).view(t, heads, vdim)
    pos = list(range(t))
    q = rotate(q, pos, m["rot"]["base"], m["rot"]["dims"])
    k = rotate(k, pos, m["rot"]["base"], m["rot"]["dims"]) * dim ** -0.5
    out = torch.zeros(t, heads, vdim, dtype=F)
    for a in range(heads):
        s = torch.zeros(dim, vdim, dtype=F)
        for i in range(t):
            s = m["decay"][a] * s + torch.outer(k[i, a], v[i, a])
            out[i, a] = s.T @ q[i, a]
    out = rms(out, eps).reshape(t, heads * vdim)
    g = h @ w[p + "g"].to(F).T
    return (out * g * torch.sigmoid(g)) @ w[p + "o"].to(F).T


def window_attention(w, p, m, h, eps):
    """Softmax attention over the last `mask.size` tokens whose values are the unnormed keys, with a sink in the
    denominator."""
    t, heads, groups, dim = h.shape[0], m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].to(F).T).view(t, heads, dim)
    k = (h @ w[p + "k"].to(F).T).view(t, groups, dim)
    v = k
    q, kn = rms(q, eps), rms(k, eps)
    sink = w[p + "sink"].to(F)
    size = m["mask"]["size"] if m.get("mask") else None
    out = torch.zeros(t, heads, dim, dtype=F)
    for a in range(heads):
        g = a // (heads // groups)
        for i in range(t):
            lo = 0 if size is None else max(0, i - size + 1)
            s = (kn[lo:i + 1, g] @ q[i, a]) * m["scale"]
            top = max(s.max().item(), sink[a].item())
            e = torch.exp(s - top)
            out[i, a] = (e[:, None] * v[lo:i + 1, g]).sum(0) / (e.sum() + math.exp(sink[a].item() - top))
    return out.reshape(t, heads * dim) @ w[p + "o"].to(F).T


def short_conv(x, taps):
    """x [T, C], taps [C, n]: the last column weighs the current token; zeros stand before the start."""
    t, n = x.shape[0], taps.shape[1]
    padded = torch.cat((torch.zeros(n - 1, x.shape[1], dtype=F), x), 0)
    return sum(padded[j:j + t] * taps[:, j] for j in range(n))


def silu(x):
    return x * torch.sigmoid(x)


def gated_delta(w, p, m, h, eps):
    """S ← g·S (per key channel); u = β (v − Sᵀk); S ← S + k uᵀ; o = Sᵀ q."""
    t, heads, groups, dim, vdim = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]

    def branch(name):
        return silu(short_conv(h @ w[p + name].to(F).T, w[p + name + ".conv"].to(F)))

    def unit(x):
        return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)

    q = unit(branch("q").view(t, groups, dim)) * dim ** -0.5
    k = unit(branch("k").view(t, groups, dim))
    v = branch("v").view(t, heads, vdim)
    beta = torch.sigmoid(h @ w[p + "b"].to(F).T)
    a = (h @ w[p + "a1"].to(F).T) @ w[p + "a2"].to(F).T + w[p + "dt_bias"].to(F)
    rate = torch.exp(w[p + "A_log"].to(F))
    decay = torch.exp(-rate[None, :, None] * torch.nn.functional.softplus(a).view(t, heads, dim))
    out = torch.zeros(t, heads, vdim, dtype=F)
    for a_ in range(heads):
        g = a_ // (heads // groups)
        s = torch.zeros(dim, vdim, dtype=F)
        for i in range(t):
            s = decay[i, a_][:, None] * s
            u = beta[i, a_] * (v[i, a_] - s.T @ k[i, g])
            s = s + torch.outer(k[i, g], u)
            out[i, a_] = s.T @ q[i, g]
    gate = torch.sigmoid((h @ w[p + "g1"].to(F).T) @ w[p + "g2"].to(F).T).view(t, heads, vdim)
    out = rms(out, eps) * w[p + "norm"].to(F) * gate
    return out.reshape(t, heads * vdim) @ w[p + "o"].to(F).T


def feed_forward(w, p, m, h):
    limit = m["limit"]
    g = torch.clamp(h @ w[p + "gate"].to(F).T + w[p + "gate.b"].to(F), max=limit)
    u = torch.clamp(h @ w[p + "up"].to(F).T + w[p + "up.b"].to(F), -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[p + "down"].to(F).T + w[p + "down.b"].to(F)


def mixer(w, layer, owner, h, eps):
    p, m = f"l{owner}.mix.", layer["mixer"]
    if layer["type"] == "retention":
        return retention(w, p, m, h, eps)
    if layer["type"] == "parallel":
        return (m["left_scale"] * window_attention(w, p + "left.", m["left"], h, eps)
                + m["right_scale"] * gated_delta(w, p + "right.", m["right"], h, eps))
    raise ValueError(layer["type"])


def forward(w, cfg, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence run whole. `layers_out`: a list that receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = embedding(w, cfg, tokens)
    for i, layer in enumerate(cfg["layers"]):
        owner = layer.get("weights_of", i)
        h = rms(x, eps) * w[f"l{owner}.norm1"].to(F)
        y = mixer(w, layer, owner, h, eps)
        if layer.get("mlp") is not None:
            y = y + feed_forward(w, f"l{owner}.mlp.", layer["mlp"], h)
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms(x, eps) * w["final.norm"].to(F)
    return x @ w["embed"].to(F).T
