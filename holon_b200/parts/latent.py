"""Latent attention over a paged cache of one row per token.

Per token the layer keeps only c (the RMS-normed first `rank` outputs of the down-projection) and k_r (its last
`rot_dim` outputs, rotated by the token's position), which all heads share. Head h has queries q_h = [q_h^u (dim
unrotated) | q_h^r (rot_dim, rotated)], keys k_{h,j} = [W_uk,h c_j | k_r,j] and values v_{h,j} = W_uv,h c_j, and

    score_h(i, j) = (q_h^u(i) · W_uk,h c_j + q_h^r(i) · k_r,j) · scale,   j ≤ i,   softmax over j,
    out_h(i) = W_uv,h Σ_j p_h(i, j) c_j,   then · sigmoid(W_g x) element by element, then W_o.

Because W_uk,h and W_uv,h act on the cached row only, they are applied on the query's side: a_h(i) = W_uk,hᵀ q_h^u(i)
(`rank` numbers) makes q_h^u · W_uk,h c_j = a_h · c_j, so every head attends over the same rows [c_j | k_r,j] with
the query [a_h | q_h^r], the attention's value is c_j itself, and W_uv,h is applied once to the weighted sum. Keys and
values per head are never made; that holds for prompts and for decoding alike.

A layer without a down-projection of its own (`own_latent=False`) reads the cache entry another layer fills (the
run order says which) with its own W_uk, W_uv, queries, gate and output product.

The first products (q, gate, down-projection) are one merged product; the rotation table is the position part's.
"""
from __future__ import annotations

import torch

from ..config.spec import PartRef
from .base import BuildContext, PagedLatent, Part
from .linear import Linear


class LatentAttention(Part):
    def __init__(self, ctx: BuildContext, *, heads: int, dim: int, rot_dim: int, vdim: int, rank: int, scale: float,
                 hidden: int, norm: PartRef, position: PartRef | None, own_latent: bool = True, window: int = 0,
                 layer: int = 0) -> None:
        super().__init__()
        self.ctx, self.heads, self.dim, self.rot_dim, self.vdim, self.rank = ctx, heads, dim, rot_dim, vdim, rank
        self.scale, self.own_latent, self.window = float(scale), bool(own_latent), int(window)
        pieces = {"q": heads * (dim + rot_dim), "g": heads * vdim}
        if own_latent:
            pieces["dkv"] = rank + rot_dim
        self.first = self.add_child("first", Linear(ctx, "weight", hidden, pieces))
        self.uk = self.add_param("uk", (heads * dim, rank), "matrix")
        self.uv = self.add_param("uv", (heads * vdim, rank), "matrix")
        self.out = self.add_child("out", Linear(ctx, "weight", heads * vdim, {"o": hidden}))
        self.latent_norm = self.add_child("latent_norm", ctx.part(norm, dim=rank)) if own_latent else None
        self.position = self.add_child("position", ctx.part(position, head_dim=rot_dim)) if position and rot_dim else None
        self.uk_t = None                    # [heads, rank, dim]: W_uk per head, transposed (made in finalize)

    def loadables(self, prefix: str = ""):
        """Stored names: q, g, dkv, dkv.norm, uk, uv, o."""
        rename = {prefix + "latent_norm.weight": prefix + "dkv.norm"}
        for name, p, rows in super().loadables(prefix):
            for child in ("first.", "out."):
                if name.startswith(prefix + child):
                    name = prefix + name[len(prefix + child):]
            yield rename.get(name, name), p, rows

    def finalize(self) -> None:
        super().finalize()
        if self.uk.tensor is not None:
            self.uk_t = self.uk.tensor.view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()

    def cache(self) -> PagedLatent:
        return PagedLatent(self.rank, self.rot_dim, self.window)

    def slot_states(self):
        return ()

    @property
    def plan_group(self):
        return "latent", self.heads, self.rank, self.rot_dim, self.window

    def capture_plan(self, step, max_model_len: int):
        plan = getattr(self.ctx.kernels, "attention_capture_plan", None)
        return plan(step.rows, max_model_len) if plan is not None else None

    def forward(self, x: torch.Tensor, step, cache) -> torch.Tensor:
        t, k, ctx = x.shape[0], self.ctx.kernels, self.ctx
        heads, dim, rot, rank, vdim = self.heads, self.dim, self.rot_dim, self.rank, self.vdim
        fills = cache.fills and self.own_latent
        first = self.first.forward(x)                                   # [t, q | g | dkv]
        n_q, n_g = heads * (dim + rot), heads * vdim
        pos = self.position
        qa = ctx.empty(t, heads, rank + rot)                             # the folded queries [a_h | q_h^r]
        k.latent_prepare(qa, first, heads, dim, rot, rank, n_q + n_g if fills else -1, step.positions,
                         pos.table if pos else None, pos.rotary_dim if pos else 0,
                         self.latent_norm.weight.tensor if fills else None, self.latent_norm.eps if fills else 0.0,
                         cache.kv if fills else None, cache.group.write_index if fills else None)
        q_u = first[:, :n_q].view(t, heads, dim + rot)[:, :, :dim]
        k.linear_heads(qa[:, :, :rank], q_u, self.uk_t)                   # a_h = W_uk,hᵀ q_h^u
        mix = ctx.empty(t, heads, rank)
        k.latent_attention(mix, qa, cache.kv, cache.group.block_table, step.rows, self.scale, rank, self.window)
        o = ctx.empty(t, heads, vdim)
        k.linear_heads(o, mix, self.uv.tensor.view(heads, vdim, rank))    # W_uv,h on the weighted sum of latents
        o = o.view(t, n_g)
        k.sigmoid_gate(o, first[:, n_q:n_q + n_g])
        return self.out.forward(o)
