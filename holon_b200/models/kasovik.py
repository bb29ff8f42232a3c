"""Kasovik: its typed configuration and its recipe.

A decoder whose config.json lists its layers one by one (`layers[i]`: `type`, the mixer's sizes under `mixer`, the
feed-forward under `mlp` or null). A layer is a parallel block: one norm, and mixer and feed-forward both read it.
Mixer types: `retention` (a matrix state per head with a fixed decay, rotated q and k) and `parallel` (two mixers side
by side: `left`, attention over a sliding window whose values are the unnormed keys, with a sink in the softmax, and
`right`, a gated delta rule behind short convolutions). Feed-forwards are gated units with clamped inputs and biases.
A layer with `weights_of: j` has no tensors: it runs layer j's parts on a cache entry and state of its own, which here
is a second run of layer j in the run order. The embedding is scaled and adds a row of a token-pair table; the head is
the embedding table itself.

Keys read: `architecture`, `width`, `vocab`, `norm.eps`, `embedding.{scale, bigram.{buckets, mul_prev, mul_cur}}`,
`layers[i].{type, weights_of, mixer, mlp.{kind, ff, limit}}`; retention: `mixer.{heads, dim, vdim, decay, rot.{base,
dims}}`; parallel: `mixer.{left_scale, right_scale, left.{heads, kv_heads, dim, vdim, scale, mask.size}, right.{heads,
kv_heads, dim, vdim, conv}}`. Two sizes stand in no key of a stored model's config.json, the ranks of the delta rule's
low-rank decay and gate projections: `complete` reads them from the shapes of `l<i>.mix.right.a1` and `.g1` and enters
them as `right.decay_rank` and `right.gate_rank` (a config dict made by hand, for random weights, gives them itself).
Stored tensors: `embed`, `bigram`, `final.norm`, `l<i>.norm1`, `l<i>.mix.{q, k, v, g, o}` (retention),
`l<i>.mix.left.{q, k, sink, o}`, `l<i>.mix.right.{q, k, v, q.conv, k.conv, v.conv, b, a1, a2, dt_bias, A_log, g1, g2,
norm, o}`, `l<i>.mlp.{gate, up, down}` with `.b` each.
"""
from __future__ import annotations

import copy
import dataclasses
from collections.abc import Mapping
from typing import Any

from ..config.registry import ConfigError, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartRef, Run, WeightRule
from .rulorax import _get


@dataclasses.dataclass(frozen=True)
class RetentionSizes:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]
    rot_base: float
    rot_dims: int


@dataclasses.dataclass(frozen=True)
class WindowSizes:
    heads: int
    kv_heads: int
    dim: int
    scale: float
    window: int                   # 0: every earlier token is seen


@dataclasses.dataclass(frozen=True)
class DeltaSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int
    decay_rank: int
    gate_rank: int


@dataclasses.dataclass(frozen=True)
class SideBySideSizes:
    left: WindowSizes
    right: DeltaSizes
    left_scale: float
    right_scale: float


@dataclasses.dataclass(frozen=True)
class GatedUnit:
    ff: int
    limit: float


@dataclasses.dataclass(frozen=True)
class KasovikLayer:
    kind: str                     # "retention" | "parallel"
    mixer: RetentionSizes | SideBySideSizes
    mlp: GatedUnit | None
    weights_of: int | None = None


@dataclasses.dataclass(frozen=True)
class PairTable:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclasses.dataclass(frozen=True)
class KasovikConfig:
    width: int
    vocab: int
    eps: float
    embed_scale: float
    pairs: PairTable | None
    layers: tuple[KasovikLayer, ...]
    eos_token_ids: tuple[int, ...] = ()

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i runs with."""
        while self.layers[i].weights_of is not None:
            i = self.layers[i].weights_of
        return i

    @staticmethod
    def from_dict(c: Mapping[str, Any]) -> "KasovikConfig":
        listed = c.get("layers")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("config.json: 'layers' must list the layers")
        layers = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = _get(entry, "type", str, where)
            m = _get(entry, "mixer", Mapping, where)
            if kind == "retention":
                rot = _get(m, "rot", Mapping, where + ".mixer")
                decay = _get(m, "decay", (list, tuple), where + ".mixer")
                mixer = RetentionSizes(heads=_get(m, "heads", int, where), dim=_get(m, "dim", int, where),
                                       vdim=_get(m, "vdim", int, where), decay=tuple(float(d) for d in decay),
                                       rot_base=_get(rot, "base", float, where + ".mixer.rot"),
                                       rot_dims=_get(rot, "dims", int, where + ".mixer.rot"))
                if len(mixer.decay) != mixer.heads:
                    raise ConfigError(f"config.json: {where}.mixer.decay must list one decay per head")
                if mixer.rot_dims % 2 or not 0 <= mixer.rot_dims <= mixer.dim:
                    raise ConfigError(f"config.json: {where}.mixer.rot.dims must be even and at most dim")
                sizes = (mixer.heads, mixer.dim, mixer.vdim)
            elif kind == "parallel":
                lw, rw = where + ".mixer.left", where + ".mixer.right"
                left, right = _get(m, "left", Mapping, where + ".mixer"), _get(m, "right", Mapping, where + ".mixer")
                mask = left.get("mask")
                wl = WindowSizes(heads=_get(left, "heads", int, lw), kv_heads=_get(left, "kv_heads", int, lw),
                                 dim=_get(left, "dim", int, lw), scale=_get(left, "scale", float, lw),
                                 window=_get(mask, "size", int, lw + ".mask") if mask is not None else 0)
                if left.get("vdim", wl.dim) != wl.dim:
                    raise ConfigError(f"config.json: {lw}.vdim must equal dim (the values are the keys)")
                for name in ("decay_rank", "gate_rank"):
                    if name not in right:
                        raise ConfigError(f"config.json: {rw}.{name} is given neither by the dict nor by a stored "
                                          f"tensor's shape (l<i>.mix.right.a1 / .g1)")
                wr = DeltaSizes(heads=_get(right, "heads", int, rw), kv_heads=_get(right, "kv_heads", int, rw),
                                dim=_get(right, "dim", int, rw), vdim=_get(right, "vdim", int, rw),
                                taps=_get(right, "conv", int, rw), decay_rank=_get(right, "decay_rank", int, rw),
                                gate_rank=_get(right, "gate_rank", int, rw))
                mixer = SideBySideSizes(wl, wr, left_scale=_get(m, "left_scale", float, where + ".mixer"),
                                        right_scale=_get(m, "right_scale", float, where + ".mixer"))
                if wl.window < 0 or wr.taps < 1:
                    raise ConfigError(f"config.json: {where}.mixer: mask.size must not be negative, conv at least 1")
                for s in (wl, wr):
                    if s.kv_heads < 1 or s.heads % s.kv_heads:
                        raise ConfigError(f"config.json: {where}.mixer: heads must be a multiple of kv_heads")
                sizes = (wl.heads, wl.dim, wr.heads, wr.dim, wr.vdim, wr.decay_rank, wr.gate_rank)
            else:
                raise NotImplementedError(f"kasovik: {where} has mixer type {kind!r}; known: retention, parallel")
            if min(sizes) < 1:
                raise ConfigError(f"config.json: {where}.mixer: every size must be positive")
            mlp = entry.get("mlp")
            unit = None
            if mlp is not None:
                mkind = _get(mlp, "kind", str, where + ".mlp")
                if mkind != "dense":
                    raise NotImplementedError(f"kasovik: {where}.mlp.kind {mkind!r}; known: dense")
                unit = GatedUnit(ff=_get(mlp, "ff", int, where + ".mlp"), limit=_get(mlp, "limit", float, where + ".mlp"))
            shared = entry.get("weights_of")
            if shared is not None and (not isinstance(shared, int) or isinstance(shared, bool)
                                       or not 0 <= shared < len(listed) or shared == i):
                raise ConfigError(f"config.json: {where}.weights_of must name another layer")
            layers.append(KasovikLayer(kind, mixer, unit, shared))
        for i, layer in enumerate(layers):
            j, steps = i, 0
            while layers[j].weights_of is not None:
                j, steps = layers[j].weights_of, steps + 1
                if steps > len(layers):
                    raise ConfigError(f"config.json: layers[{i}].weights_of leads in a circle")
            if (layers[j].kind, layers[j].mixer, layers[j].mlp) != (layer.kind, layer.mixer, layer.mlp):
                raise ConfigError(f"config.json: layers[{i}] runs with layer {j}'s tensors but differs from it")
        e = _get(c, "embedding", Mapping, "config")
        b = e.get("bigram")
        pairs = None
        if b is not None:
            pairs = PairTable(buckets=_get(b, "buckets", int, "embedding.bigram"),
                              mul_prev=_get(b, "mul_prev", int, "embedding.bigram"),
                              mul_cur=_get(b, "mul_cur", int, "embedding.bigram"))
            if pairs.buckets < 1:
                raise ConfigError("config.json: embedding.bigram.buckets must be positive")
        eos = c.get("eos_token_id", ())
        eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
        cfg = KasovikConfig(width=_get(c, "width", int, "config"), vocab=_get(c, "vocab", int, "config"),
                            eps=_get(_get(c, "norm", Mapping, "config"), "eps", float, "norm"),
                            embed_scale=_get(e, "scale", float, "embedding"), pairs=pairs, layers=tuple(layers),
                            eos_token_ids=eos)
        if cfg.width < 1 or cfg.vocab < 1:
            raise ConfigError("config.json: 'width' and 'vocab' must be positive")
        return cfg


def complete(c: Mapping[str, Any], shapes: Mapping[str, tuple]) -> dict[str, Any]:
    """config.json with `right.decay_rank` and `right.gate_rank` entered from the stored tensors' shapes."""
    c = copy.deepcopy(dict(c))
    listed = c.get("layers")
    if not isinstance(listed, list):
        return c
    for i, entry in enumerate(listed):
        if not isinstance(entry, dict) or entry.get("type") != "parallel":
            continue
        j, steps = i, 0
        while isinstance(listed[j].get("weights_of"), int) and 0 <= listed[j]["weights_of"] < len(listed) and steps <= len(listed):
            j, steps = listed[j]["weights_of"], steps + 1
        right = entry.get("mixer", {}).get("right")
        if isinstance(right, dict):
            for key, stored in (("decay_rank", f"l{j}.mix.right.a1"), ("gate_rank", f"l{j}.mix.right.g1")):
                if key not in right and stored in shapes:
                    right[key] = int(shapes[stored][0])
    return c


WEIGHT_RULES = (
    WeightRule("embed", "embed.weight"),
    WeightRule("bigram", "embed.pair"),
    WeightRule("final.norm", "norm.weight"),
    WeightRule("l{i}.norm1", "layers.{i}.norm.weight"),
    WeightRule("l{i}.mix.{rest}", "layers.{i}.mixer.{rest}"),
    WeightRule("l{i}.mlp.{rest}", "layers.{i}.ffn.{rest}"),
)


def recipe(cfg: KasovikConfig) -> ModelSpec:
    norm = PartRef.of("norm", "rmsnorm", eps=cfg.eps)
    block = PartRef.of("block", "parallel")
    layers, order = [], []
    for i, layer in enumerate(cfg.layers):
        order.append(Run(cfg.owner(i), i))
        if layer.weights_of is not None:
            layers.append(None)
            continue
        m = layer.mixer
        if layer.kind == "retention":
            mixer = PartRef.of("mixer", "retention", heads=m.heads, dim=m.dim, vdim=m.vdim, decay=m.decay, eps=cfg.eps,
                               position=PartRef.of("position", "rope", theta=m.rot_base, rotary_dim=m.rot_dims)
                               if m.rot_dims else None)
        else:
            left = PartRef.of("mixer", "gqa", heads=m.left.heads, kv_heads=m.left.kv_heads, head_dim=m.left.dim,
                              position=None, window=m.left.window, scale=m.left.scale, unit_norm_eps=cfg.eps,
                              values_are_keys=True, sink=True,
                              names=(("q_proj.weight", "q"), ("k_proj.weight", "k"), ("o_proj.weight", "o")))
            right = PartRef.of("mixer", "gated_delta", heads=m.right.heads, kv_heads=m.right.kv_heads, dim=m.right.dim,
                               vdim=m.right.vdim, taps=m.right.taps, decay_rank=m.right.decay_rank,
                               gate_rank=m.right.gate_rank, eps=cfg.eps)
            mixer = PartRef.of("mixer", "side_by_side", left=left, right=right, left_scale=m.left_scale,
                               right_scale=m.right_scale)
        ffn = PartRef.of("ffn", "clamped_glu", inter=layer.mlp.ff, limit=layer.mlp.limit) if layer.mlp else None
        layers.append(LayerSpec(block, mixer, ffn, norm))
    p = cfg.pairs
    embed = PartRef.of("embed", "pair", scale=cfg.embed_scale, buckets=p.buckets if p else None,
                       mul_prev=p.mul_prev if p else 0, mul_cur=p.mul_cur if p else 0)
    return ModelSpec(hidden=cfg.width, vocab=cfg.vocab, layers=tuple(layers), order=tuple(order), embed=embed, norm=norm,
                     head=PartRef.of("head", "linear", tied=True), weight_rules=WEIGHT_RULES)


register_architecture("Kasovik", KasovikConfig.from_dict, recipe, complete=complete)
