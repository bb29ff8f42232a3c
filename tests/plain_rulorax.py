"""A plain, slow Rulorax decoder: whole sequences, no cache, one function per mechanism, CPU torch only.

The yardstick for the engine's Rulorax tests. It shares no code with `holon_b200`: it reads `config.json` and
`model.safetensors` itself and spells every formula out in the direct form (keys and values of every head are made
from the latent, nothing is folded into the queries), in the dtype of the tensors it is given (float64 in the tests).

The design: an embedding; layers that keep `streams` copies of the residual (hyper-connections) around a latent
attention mixer and a feed-forward (SwiGLU, or routed experts with an optional shared one); an RMS norm and a head.
"""
from __future__ import annotations

import json
import pathlib

import torch
from safetensors import safe_open


def read_folder(folder, dtype=torch.float64):
    """(config dict, {stored name: tensor}) with floating tensors as `dtype`."""
    folder = pathlib.Path(folder)
    config = json.loads((folder / "config.json").read_text())
    tensors = {}
    for shard in sorted(folder.glob("*.safetensors")):
        with safe_open(str(shard), framework="pt") as f:
            for name in f.keys():
                t = f.get_tensor(name)
                tensors[name] = t.to(dtype) if t.is_floating_point() else t
    return config, tensors


# ---------------------------------------------------------------- small pieces

def rms_norm(x, weight, eps):
    """x / sqrt(mean(x²) + eps) · weight over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def rotate(x, positions, base: float, dims: int):
    """Rotates the first `dims` entries of the last dimension of x [tokens, ..., n]: entry i pairs with i + dims/2,
    the angle of pair i at position p is p · base^(−2i/dims); the rest passes unchanged."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    angle = torch.as_tensor(positions, dtype=x.dtype)[:, None] * freq[None, :]
    shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (half,)
    cos, sin = angle.cos().reshape(shape), angle.sin().reshape(shape)
    u, v, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    return torch.cat((u * cos - v * sin, v * cos + u * sin, rest), dim=-1)


# ---------------------------------------------------------------- the mixer

def latent_kv(h, w, layer: int, m: dict, positions, eps):
    """What a layer with a down-projection of its own leaves for the keys and values: the normed latent [tokens,
    kv_rank] and the rotated key part [tokens, rot_dim] that all heads share."""
    p = f"l{layer}.mix."
    d = h @ w[p + "dkv"].T
    rank = m["kv_rank"]
    c = rms_norm(d[:, :rank], w[p + "dkv.norm"], eps)
    return c, rotate(d[:, rank:], positions, m["rot"]["base"], m["rot"]["dims"])


def latent_attention(h, w, layer: int, m: dict, positions, latent):
    """The mixer of layer `layer` on its input h [tokens, width]; `latent` = (c, rotated key part) of the layer
    whose down-projection it uses (its own, or the layer that `kv_from` names). Token i sees every j ≤ i."""
    p = f"l{layer}.mix."
    heads, dim, rot, vdim = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    t = h.shape[0]
    c, k_rot = latent
    q = (h @ w[p + "q"].T).reshape(t, heads, dim + rot)
    q_plain, q_rot = q[..., :dim], rotate(q[..., dim:], positions, m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ w[p + "uk"].T).reshape(t, heads, dim)
    v = (c @ w[p + "uv"].T).reshape(t, heads, vdim)
    scores = torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)
    scores = scores * m["scale"]
    seen = torch.tril(torch.ones(t, t, dtype=torch.bool))
    scores = scores.masked_fill(~seen, float("-inf"))
    out = torch.einsum("hij,jhd->ihd", torch.softmax(scores, dim=-1), v).reshape(t, heads * vdim)
    out = out * torch.sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


# ---------------------------------------------------------------- the feed-forwards

def dense_ff(h, w, prefix: str):
    gate, up = h @ w[prefix + "gate"].T, h @ w[prefix + "up"].T
    return (gate * torch.sigmoid(gate) * up) @ w[prefix + "down"].T


def expert(h, w, prefix: str):
    """down · relu(up · h)²."""
    return torch.relu(h @ w[prefix + "up"].T) ** 2 @ w[prefix + "down"].T


def route(h, w, prefix: str, r: dict):
    """(chosen experts [tokens, top], their weights): the largest softmax scores over all experts, times the
    router's scale, not renormalised."""
    s = torch.softmax(h @ w[prefix + "router"].T, dim=-1)
    score, chosen = torch.topk(s, r["top"], dim=-1)
    return chosen, score * r["scale"]


def moe_ff(h, w, prefix: str, mlp: dict):
    chosen, weight = route(h, w, prefix, mlp["router"])
    out = torch.zeros(h.shape[0], w[prefix + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weight[t]):
            out[t] += g * expert(h[t:t + 1], w, f"{prefix}e{e}.")[0]
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ w[prefix + "shared.sg"].T) * expert(h, w, prefix + "shared.")
    return out


def feed_forward(h, w, layer: int, mlp: dict):
    prefix = f"l{layer}.mlp."
    return dense_ff(h, w, prefix) if mlp["kind"] == "dense" else moe_ff(h, w, prefix, mlp)


# ---------------------------------------------------------------- hyper-connections

def hyper_read(xs, w, prefix: str):
    """The sublayer's input: the streams xs [streams, tokens, width] weighted by `in`."""
    return torch.einsum("s,stw->tw", w[prefix + "in"], xs)


def hyper_write(xs, y, w, prefix: str):
    """All streams at once from the old ones: x_t = Σ_s mix[s, t] x_s + out[t] · y."""
    return torch.einsum("st,sij->tij", w[prefix + "mix"], xs) + w[prefix + "out"][:, None, None] * y[None]


# ---------------------------------------------------------------- the model

def forward(config, w, ids, layers_out: list | None = None):
    """Logits [tokens, vocab] of one sequence; `layers_out` collects the sum of the streams after every layer."""
    eps = config["norm"]["eps"]
    positions = list(range(len(ids)))
    x = w["embed"][torch.as_tensor(ids, dtype=torch.long)]
    streams = config.get("streams")
    xs = torch.stack([x] * streams) if streams else None
    latents = {}
    for i, layer in enumerate(config["layers"]):
        m = layer["mixer"]
        for q in (1, 2):
            if q == 2 and layer.get("mlp") is None:
                continue
            u = hyper_read(xs, w, f"l{i}.hc{q}.") if streams else x
            h = rms_norm(u, w[f"l{i}.norm{q}"], eps)
            if q == 1:
                if "kv_from" not in m:
                    latents[i] = latent_kv(h, w, i, m, positions, eps)
                y = latent_attention(h, w, i, m, positions, latents[m.get("kv_from", i)])
            else:
                y = feed_forward(h, w, i, layer["mlp"])
            if streams:
                xs = hyper_write(xs, y, w, f"l{i}.hc{q}.")
            else:
                x = x + y
        if layers_out is not None:
            layers_out.append(xs.sum(0) if streams else x)
    x = xs.sum(0) if streams else x
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
