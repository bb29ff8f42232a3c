"""Rulorax: its typed configuration and its recipe.

A decoder whose layers are listed one by one in config.json (`layers`: each with its mixer's sizes and its
feed-forward, or none). The mixer is latent attention: keys and values of all heads are made from one low-rank
latent per token plus one rotated key part that the heads share, and only those two are cached; a layer may read
the latent of an earlier layer instead of making its own (`kv_from`), which here is a run that reads another run's
cache entry. Feed-forwards are SwiGLU or routed experts (softmax router, top-k, squared-relu experts, an optional
gated shared expert). With `streams` the residual is kept in that many copies mixed by learned coefficients
(hyper-connections, block `hyper`); without, blocks are plain pre-norm ones. Every size and constant is read from
config.json; the stored tensor names are `embed`, `head`, `final.norm` and `l<i>.{norm1,norm2,mix.*,mlp.*,hc1.*,hc2.*}`.
"""
from __future__ import annotations

import dataclasses
from collections.abc import Mapping
from typing import Any

from ..config.registry import ConfigError, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartRef, Run, WeightRule


def _get(c: Mapping[str, Any], key: str, kind, where: str):
    if not isinstance(c, Mapping) or key not in c:
        raise ConfigError(f"config.json: {where} lacks {key!r}")
    value = c[key]
    if kind is float and isinstance(value, int) and not isinstance(value, bool):
        value = float(value)
    if not isinstance(value, kind) or isinstance(value, bool):
        raise ConfigError(f"config.json: {where}.{key} must be {kind.__name__}, not {value!r}")
    return value


@dataclasses.dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int                      # unrotated query/key dimensions per head
    rot_dim: int                  # rotated ones (the key's are shared by all heads)
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int                 # how many of the rot_dim entries turn (the first ones)
    kv_from: int | None = None


@dataclasses.dataclass(frozen=True)
class Experts:
    experts: int
    top: int
    scale: float
    ff: int
    shared_ff: int | None = None


@dataclasses.dataclass(frozen=True)
class RuloraxLayer:
    mixer: LatentMixer
    dense_ff: int | None = None
    experts: Experts | None = None


@dataclasses.dataclass(frozen=True)
class RuloraxConfig:
    width: int
    vocab: int
    eps: float
    streams: int | None
    layers: tuple[RuloraxLayer, ...]
    eos_token_ids: tuple[int, ...] = ()

    @staticmethod
    def from_dict(c: Mapping[str, Any]) -> "RuloraxConfig":
        layers = []
        listed = c.get("layers")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("config.json: 'layers' must list the layers")
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = _get(entry, "type", str, where)
            if kind != "latent_attention":
                raise NotImplementedError(f"rulorax: {where} has mixer type {kind!r}; known: latent_attention")
            m = _get(entry, "mixer", Mapping, where)
            rot = _get(m, "rot", Mapping, where + ".mixer")
            mixer = LatentMixer(
                heads=_get(m, "heads", int, where), dim=_get(m, "dim", int, where), rot_dim=_get(m, "rot_dim", int, where),
                vdim=_get(m, "vdim", int, where), kv_rank=_get(m, "kv_rank", int, where),
                scale=_get(m, "scale", float, where), rot_base=_get(rot, "base", float, where + ".mixer.rot"),
                rot_dims=_get(rot, "dims", int, where + ".mixer.rot"),
                kv_from=_get(m, "kv_from", int, where) if m.get("kv_from") is not None else None)
            for name in ("heads", "dim", "vdim", "kv_rank"):
                if getattr(mixer, name) < 1:
                    raise ConfigError(f"config.json: {where}.mixer.{name} must be positive")
            if mixer.rot_dims % 2 or not 0 <= mixer.rot_dims <= mixer.rot_dim:
                raise ConfigError(f"config.json: {where}.mixer.rot.dims must be even and at most rot_dim")
            if mixer.kv_from is not None:
                if not 0 <= mixer.kv_from < i or layers[mixer.kv_from].mixer.kv_from is not None:
                    raise ConfigError(f"config.json: {where}.mixer.kv_from must name an earlier layer that makes its own latent")
                src = layers[mixer.kv_from].mixer
                if (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims) != (mixer.kv_rank, mixer.rot_dim, mixer.rot_base, mixer.rot_dims):
                    raise ConfigError(f"config.json: {where}.mixer reads layer {mixer.kv_from}'s latent but differs in kv_rank, rot_dim or rot")
            mlp = entry.get("mlp")
            dense_ff = experts = None
            if mlp is not None:
                mkind = _get(mlp, "kind", str, where + ".mlp")
                if mkind == "dense":
                    dense_ff = _get(mlp, "ff", int, where + ".mlp")
                elif mkind == "moe":
                    r = _get(mlp, "router", Mapping, where + ".mlp")
                    shared = mlp.get("shared")
                    experts = Experts(
                        experts=_get(r, "experts", int, where + ".mlp.router"), top=_get(r, "top", int, where + ".mlp.router"),
                        scale=_get(r, "scale", float, where + ".mlp.router"),
                        ff=_get(_get(mlp, "expert", Mapping, where + ".mlp"), "ff", int, where + ".mlp.expert"),
                        shared_ff=_get(shared, "ff", int, where + ".mlp.shared") if shared is not None else None)
                    if not 1 <= experts.top <= experts.experts:
                        raise ConfigError(f"config.json: {where}.mlp.router.top must be between 1 and experts")
                else:
                    raise NotImplementedError(f"rulorax: {where}.mlp.kind {mkind!r}; known: dense, moe")
            layers.append(RuloraxLayer(mixer, dense_ff, experts))
        streams = c.get("streams")
        if streams is not None and (not isinstance(streams, int) or isinstance(streams, bool) or streams < 1):
            raise ConfigError("config.json: 'streams' must be a positive integer")
        eos = c.get("eos_token_id", ())
        eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
        cfg = RuloraxConfig(width=_get(c, "width", int, "config"), vocab=_get(c, "vocab", int, "config"),
                            eps=_get(_get(c, "norm", Mapping, "config"), "eps", float, "norm"), streams=streams,
                            layers=tuple(layers), eos_token_ids=eos)
        if cfg.width < 1 or cfg.vocab < 1:
            raise ConfigError("config.json: 'width' and 'vocab' must be positive")
        return cfg


WEIGHT_RULES = (
    WeightRule("embed", "embed.weight"),
    WeightRule("final.norm", "norm.weight"),
    WeightRule("head", "head.weight"),
    WeightRule("l{i}.norm1", "layers.{i}.input_norm.weight"),
    WeightRule("l{i}.norm2", "layers.{i}.post_norm.weight"),
    WeightRule("l{i}.mix.{rest}", "layers.{i}.mixer.{rest}"),
    WeightRule("l{i}.mlp.gate", "layers.{i}.ffn.gate_proj.weight"),
    WeightRule("l{i}.mlp.up", "layers.{i}.ffn.up_proj.weight"),
    WeightRule("l{i}.mlp.down", "layers.{i}.ffn.down_proj.weight"),
    WeightRule("l{i}.mlp.{rest}", "layers.{i}.ffn.{rest}"),
    WeightRule("l{i}.hc1.{rest}", "layers.{i}.hc1.{rest}"),
    WeightRule("l{i}.hc2.{rest}", "layers.{i}.hc2.{rest}"),
)


def recipe(cfg: RuloraxConfig) -> ModelSpec:
    norm = PartRef.of("norm", "rmsnorm", eps=cfg.eps)
    block = PartRef.of("block", "hyper", streams=cfg.streams) if cfg.streams else PartRef.of("block", "prenorm")
    layers, order = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        mixer = PartRef.of("mixer", "latent", heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, rank=m.kv_rank,
                           scale=m.scale, own_latent=m.kv_from is None, norm=norm,
                           position=PartRef.of("position", "rope", theta=m.rot_base, rotary_dim=m.rot_dims))
        if layer.dense_ff is not None:
            ffn = PartRef.of("ffn", "swiglu", inter=layer.dense_ff)
        elif layer.experts is not None:
            e = layer.experts
            ffn = PartRef.of("ffn", "experts", experts=e.experts, top=e.top, scale=e.scale, inter=e.ff,
                             shared_inter=e.shared_ff, activation="relu2", renormalize=False)
        else:
            ffn = None
        layers.append(LayerSpec(block, mixer, ffn, norm))
        order.append(Run(i, i) if m.kv_from is None else Run(i, m.kv_from, fills=False))
    return ModelSpec(hidden=cfg.width, vocab=cfg.vocab, layers=tuple(layers), order=tuple(order),
                     embed=PartRef.of("embed", "table"), norm=norm, head=PartRef.of("head", "linear", tied=False),
                     weight_rules=WEIGHT_RULES)


register_architecture("Rulorax", RuloraxConfig.from_dict, recipe)
