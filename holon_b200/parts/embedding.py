"""Token embedding (a row gather, no scaling) and the output head (logits in 32-bit; a tied head reads the
embedding's table) (std/holon_std/ops/units.py:280-348)."""
from __future__ import annotations

import torch

from .base import BuildContext, Part, Residual, SlotState


class Embedding(Part):
    def __init__(self, ctx: BuildContext, *, vocab: int, hidden: int) -> None:
        super().__init__()
        self.ctx, self.vocab, self.hidden = ctx, vocab, hidden
        self.weight = self.add_param("weight", (vocab, hidden), "table")

    def forward(self, ids: torch.Tensor) -> Residual:
        h = self.ctx.empty(ids.shape[0], self.hidden, dtype=torch.float32)
        self.ctx.kernels.embed(h, self.weight.tensor, ids)
        return Residual(h)


class PairEmbedding(Embedding):
    """Table rows times `scale`, plus a row of a second table chosen by the token and the one before it: row
    (previous · mul_prev + token · mul_cur) mod buckets, and the table's last row (number `buckets`) for a sequence's
    first token. The previous token of a request's next step is part of its state: one int32 per slot, which the
    kernel reads for a row's first token and sets to the row's last. `buckets` None: no second table."""

    wants_step = True

    def __init__(self, ctx: BuildContext, *, vocab: int, hidden: int, scale: float = 1.0, buckets: int | None = None,
                 mul_prev: int = 0, mul_cur: int = 0) -> None:
        super().__init__(ctx, vocab=vocab, hidden=hidden)
        self.scale, self.buckets, self.mul_prev, self.mul_cur = float(scale), buckets, int(mul_prev), int(mul_cur)
        self.pair = self.add_param("pair", (buckets + 1, hidden), "table") if buckets else None

    def slot_states(self):
        return (SlotState("previous", (), "int32"),) if self.buckets else ()

    def forward(self, ids: torch.Tensor, step=None) -> Residual:
        from .model import EMBED_ENTRY
        h = self.ctx.empty(ids.shape[0], self.hidden, dtype=torch.float32)
        prev = step.entry_slots(EMBED_ENTRY)["previous"] if self.buckets else None
        self.ctx.kernels.embed_pair(h, self.weight.tensor, self.scale, self.pair.tensor if self.buckets else None, ids,
                                    step.positions, step.rows, prev, self.mul_prev, self.mul_cur, self.buckets or 0)
        return Residual(h)


class Head(Part):
    def __init__(self, ctx: BuildContext, *, vocab: int, hidden: int, tied: bool, embed: Embedding | None) -> None:
        super().__init__()
        self.ctx, self.vocab = ctx, vocab
        if tied and embed is None:
            raise ValueError("a tied head needs the embedding")
        self._embed = embed if tied else None
        self.weight = None if tied else self.add_param("weight", (vocab, hidden), "matrix")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = self._embed.weight.tensor if self._embed is not None else self.weight.tensor
        logits = self.ctx.empty(x.shape[0], self.vocab, dtype=torch.float32)
        self.ctx.kernels.linear(logits, x, w)
        return logits
