"""Parts that run side by side on the same input.

`ParallelBlock`: one norm, and mixer and feed-forward both read its output: with h = norm(x), x ← x + mixer(h) +
ffn(h). The residual sum is one kernel over all terms, in 32-bit, straight into the stream; where the block that runs
next is a parallel block too, the same kernel leaves that block's normed rows behind (`Residual.normed`), so a layer
has one launch for its sum and the next layer's norm.

`SideBySide`: a mixer made of two mixers that read the same input, result = left_scale · left + right_scale · right.
At most one of the two may ask for a paged cache; their fixed-size states are kept under `left.` and `right.` names.
Inside a `ParallelBlock` its two outputs go into the block's one sum as terms of their own.
"""
from __future__ import annotations

import dataclasses

import torch

from ..config.spec import PartRef
from .base import BuildContext, Part, Residual
from .model import LayerCache


class SideBySide(Part):
    def __init__(self, ctx: BuildContext, *, left: PartRef, right: PartRef, left_scale: float, right_scale: float,
                 hidden: int, layer: int = 0) -> None:
        super().__init__()
        self.ctx = ctx
        self.left = self.add_child("left", ctx.part(left, layer=layer, hidden=hidden))
        self.right = self.add_child("right", ctx.part(right, layer=layer, hidden=hidden))
        self.scales = (float(left_scale), float(right_scale))
        if self.left.cache() is not None and self.right.cache() is not None:
            raise ValueError("side by side: only one of the two mixers may keep a paged cache")

    def _sides(self):
        return (("left", self.left), ("right", self.right))

    def cache(self):
        return self.left.cache() if self.left.cache() is not None else self.right.cache()

    def slot_states(self):
        return tuple(dataclasses.replace(s, name=f"{side}.{s.name}") for side, part in self._sides()
                     for s in part.slot_states())

    @property
    def plan_group(self):
        return ("side",) + tuple(getattr(part, "plan_group", None) for _, part in self._sides())

    def capture_plan(self, step, max_model_len: int):
        return tuple(part.capture_plan(step, max_model_len) if hasattr(part, "capture_plan") else None
                     for _, part in self._sides())

    def terms(self, x: torch.Tensor, step, cache) -> list:
        """[(output, scale)] of the two mixers."""
        out = []
        for (side, part), scale in zip(self._sides(), self.scales):
            slots = {name[len(side) + 1:]: t for name, t in cache.slots.items() if name.startswith(side + ".")}
            paged = part.cache() is not None
            own = LayerCache(cache.kv if paged else None, cache.group if paged else None, cache.fills, slots)
            out.append((part.forward(x, step, own), scale))
        return out

    def forward(self, x: torch.Tensor, step, cache) -> torch.Tensor:
        (a, sa), (b, sb) = self.terms(x, step, cache)
        return (sa * a.float() + sb * b.float()).to(a.dtype)


class ParallelBlock(Part):
    def __init__(self, ctx: BuildContext, *, layer: int, hidden: int, mixer: PartRef, ffn: PartRef | None,
                 norm: PartRef) -> None:
        super().__init__()
        self.ctx = ctx
        self.norm = self.add_child("norm", ctx.part(norm, dim=hidden))
        self.mixer = self.add_child("mixer", ctx.part(mixer, layer=layer, hidden=hidden))
        self.ffn = self.add_child("ffn", ctx.part(ffn, layer=layer, hidden=hidden)) if ffn is not None else None

    def forward(self, stream: Residual, step, cache, after=None) -> Residual:
        x = self.norm.add(stream)                  # (folds in what a block of another kind may have left pending)
        step.link = None
        if hasattr(self.mixer, "terms"):
            terms = self.mixer.terms(x, step, cache)
        else:
            terms = [(self.mixer.forward(x, step, cache), 1.0)]
        bias = None
        if self.ffn is not None:
            if hasattr(self.ffn, "forward_biased"):            # the last product's bias rides in the sum
                y, bias = self.ffn.forward_biased(x, step)
            else:
                y = self.ffn.forward(x, step)
            terms.append((y, 1.0))
        k, nxt = self.ctx.kernels, getattr(after, "norm", None) if isinstance(after, ParallelBlock) else None
        if nxt is not None and hasattr(k, "sum_norm"):
            rows = self.ctx.empty(*stream.h.shape)
            k.sum_norm(stream.h, terms, bias, rows, nxt.weight.tensor, nxt.eps, nxt.offset)
            stream.normed, stream.normed_by = rows, nxt
        else:
            k.sum_into(stream.h, terms, bias)
        return stream
