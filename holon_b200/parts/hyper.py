"""A pre-norm block over `streams` copies of the residual (hyper-connections).

The model keeps x_1 .. x_S [tokens, hidden] in 32-bit, all equal to the embedding at the start. A sublayer f (the
mixer, then the feed-forward) with coefficients `in` [S], `out` [S] and `mix` [S, S] (indexed [from, to]) runs as

    u = Σ_s in[s] · x_s,   y = f(norm(u)),   x_t ← Σ_s mix[s, t] · x_s + out[t] · y   for all t at once;

what leaves the model is Σ_s x_s under the last norm. As in the pre-norm block the sums are folded into the next
norm's kernel: a sublayer's y stays pending on the streams with its `mix` and `out`, and one kernel writes the new
streams, reads them with the next sublayer's `in` and normalises.
"""
from __future__ import annotations

import torch

from ..config.spec import PartRef
from .base import BuildContext, Part, Residual


class Streams(Residual):
    """`xs` [tokens, S, hidden] in 32-bit; `delta` is the pending sublayer output y (engine dtype) with the
    coefficients (`mix`, `out`) that fold it in. `h` is the embedding's [tokens, hidden] until the first read has
    spread it over the streams."""

    __slots__ = ("xs", "streams", "mix", "out", "kernels")

    def __init__(self, source: Residual, streams: int, kernels) -> None:
        super().__init__(source.h, source.delta)
        if source.delta is not None or source.normed is not None:
            raise ValueError("hyper-connections start from a residual stream with nothing pending")
        self.xs, self.streams, self.mix, self.out, self.kernels = None, streams, None, None, kernels

    def read(self, coef_in, norm, index=None) -> torch.Tensor:
        """Folds the pending output in (all rows, unless `index` picks rows: then nothing is written), and returns
        norm(Σ_s coef_in[s] x_s) (coef_in None: all ones) of those rows."""
        first = self.xs is None
        t, hidden = self.h.shape
        if first:
            self.xs = torch.empty((t, self.streams, hidden), dtype=torch.float32, device=self.h.device)
        rows = t if index is None else index.shape[0]
        out = norm.ctx.empty(rows, hidden)
        self.kernels.hyper_mix_norm(out, self.xs, self.h if first else None, self.delta, self.mix, self.out, coef_in,
                                    norm.weight.tensor, norm.eps, norm.offset, index)
        if index is None:
            self.delta = self.mix = self.out = None
        elif first:
            self.xs = None                               # (a gather wrote nothing)
        return out

    def final_rows(self, norm, index: torch.Tensor) -> torch.Tensor:
        return self.read(None, norm, index)


class Hyper(Part):
    def __init__(self, ctx: BuildContext, *, streams: int, layer: int, hidden: int, mixer: PartRef,
                 ffn: PartRef | None, norm: PartRef) -> None:
        super().__init__()
        if not 1 <= streams <= 16:
            raise ValueError(f"hyper: {streams} streams; the kernel takes 1 to 16")
        self.ctx, self.streams = ctx, streams
        self.input_norm = self.add_child("input_norm", ctx.part(norm, dim=hidden))
        self.mixer = self.add_child("mixer", ctx.part(mixer, layer=layer, hidden=hidden))
        self.coef = {}
        subs = ("hc1",)
        self.post_norm = self.ffn = None
        if ffn is not None:
            self.post_norm = self.add_child("post_norm", ctx.part(norm, dim=hidden))
            self.ffn = self.add_child("ffn", ctx.part(ffn, layer=layer, hidden=hidden))
            subs = ("hc1", "hc2")
        for q in subs:
            self.coef[q] = (self.add_param(f"{q}.in", (streams,), "coef"), self.add_param(f"{q}.out", (streams,), "coef"),
                            self.add_param(f"{q}.mix", (streams, streams), "coef"))

    def forward(self, stream: Residual, step, cache, after=None) -> Residual:
        if not isinstance(stream, Streams):
            stream = Streams(stream, self.streams, self.ctx.kernels)
        elif stream.streams != self.streams:
            raise ValueError(f"hyper: the block has {self.streams} streams, the model carries {stream.streams}")
        step.link = None
        subs = [("hc1", self.input_norm, lambda x: self.mixer.forward(x, step, cache))]
        if self.ffn is not None:
            subs.append(("hc2", self.post_norm, lambda x: self.ffn.forward(x, step)))
        for q, norm, run in subs:
            c_in, c_out, c_mix = self.coef[q]
            x = stream.read(c_in.tensor, norm)
            stream.delta, stream.mix, stream.out = run(x), c_mix.tensor, c_out.tensor
        return stream
