"""Typed configuration of the ``Vepevik`` architecture.

``config.json`` gives ``vocab``, ``width``, ``norm.eps`` and a list ``layers``; every entry names its
mixer (``type``: ``"retention"``, ``"channel_delta"`` or ``"attention"``), the mixer's sizes and constants
(``mixer``) and its feed-forward (``mlp``: ``kind`` ``"dense"`` or ``"moe"``, or null for none).  Layers may
differ from one another in everything.  Nothing here has a default that stands for a size: a
missing key is an error.  (The ranks of the two low-rank products of a ``channel_delta`` mixer are
sizes that the checkpoint's tensors give; ``mixer.ranks`` may name them for random weights.)
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .registry import ConfigError


def _need(m: Mapping[str, Any], key: str, where: str):
    if not isinstance(m, Mapping) or key not in m or m[key] is None:
        raise ConfigError(f"config.json: {where} lacks {key!r}")
    return m[key]


def _positive(m: Mapping[str, Any], key: str, where: str) -> int:
    v = _need(m, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]
    rot: Rotation | None


@dataclass(frozen=True)
class ChannelDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int | None = None
    gate_rank: int | None = None


@dataclass(frozen=True)
class ChunkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int | None
    rot: Rotation | None
    v_mix: bool


@dataclass(frozen=True)
class DenseConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    ff: int
    groups: int            # 0: no groups
    keep_groups: int
    scale: float


@dataclass(frozen=True)
class VepevikLayer:
    type: str
    mixer: RetentionConfig | ChannelDeltaConfig | ChunkAttentionConfig
    mlp: DenseConfig | ExpertsConfig | None


@dataclass(frozen=True)
class VepevikConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple[VepevikLayer, ...]

    @classmethod
    def from_json(cls, raw: Mapping[str, Any]) -> "VepevikConfig":
        layers = _need(raw, "layers", "the top level")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        return cls(
            vocab=_positive(raw, "vocab", "the top level"),
            width=_positive(raw, "width", "the top level"),
            eps=float(_need(_need(raw, "norm", "the top level"), "eps", "norm")),
            layers=tuple(_layer(l, f"layers[{i}]") for i, l in enumerate(layers)),
        )


def _rotation(m: Mapping[str, Any], dim: int, where: str) -> Rotation | None:
    rot = m.get("rot")
    if not rot:
        return None
    r = Rotation(base=float(_need(rot, "base", where + ".rot")), dims=_positive(rot, "dims", where + ".rot"))
    if r.dims % 2 or r.dims > dim:
        raise ConfigError(f"config.json: {where}.rot.dims={r.dims} must be even and at most dim={dim}")
    return r


def _layer(raw: Mapping[str, Any], where: str) -> VepevikLayer:
    kind = _need(raw, "type", where)
    m = _need(raw, "mixer", where)
    w = where + ".mixer"
    if kind == "retention":
        heads, dim = _positive(m, "heads", w), _positive(m, "dim", w)
        decay = _need(m, "decay", w)
        if not isinstance(decay, (list, tuple)) or len(decay) != heads:
            raise ConfigError(f"config.json: {w}.decay must list one decay per head ({heads})")
        mixer = RetentionConfig(heads=heads, dim=dim, vdim=_positive(m, "vdim", w),
                                decay=tuple(float(a) for a in decay), rot=_rotation(m, dim, w))
    elif kind == "channel_delta":
        ranks = m.get("ranks") or {}
        mixer = ChannelDeltaConfig(heads=_positive(m, "heads", w), kv_heads=_positive(m, "kv_heads", w),
                                   dim=_positive(m, "dim", w), vdim=_positive(m, "vdim", w),
                                   conv=_positive(m, "conv", w),
                                   decay_rank=_positive(ranks, "decay", w + ".ranks") if ranks.get("decay") else None,
                                   gate_rank=_positive(ranks, "gate", w + ".ranks") if ranks.get("gate") else None)
        if mixer.heads % mixer.kv_heads:
            raise ConfigError(f"config.json: {w}: {mixer.heads} heads cannot share {mixer.kv_heads} query/key heads")
    elif kind == "attention":
        dim = _positive(m, "dim", w)
        mask = m.get("mask")
        mixer = ChunkAttentionConfig(heads=_positive(m, "heads", w), kv_heads=_positive(m, "kv_heads", w), dim=dim,
                                     vdim=_positive(m, "vdim", w), scale=float(_need(m, "scale", w)),
                                     chunk=_positive(mask, "size", w + ".mask") if mask else None,
                                     rot=_rotation(m, dim, w), v_mix=bool(m.get("v_mix", False)))
        if mixer.heads % mixer.kv_heads:
            raise ConfigError(f"config.json: {w}: {mixer.heads} heads cannot share {mixer.kv_heads} key/value heads")
    else:
        raise ConfigError(f"config.json: {where}.type {kind!r} is none of 'retention', 'channel_delta', 'attention'")
    mlp = raw.get("mlp")
    ff: DenseConfig | ExpertsConfig | None = None
    if mlp is not None:
        w = where + ".mlp"
        mk = _need(mlp, "kind", w)
        if mk == "dense":
            ff = DenseConfig(ff=_positive(mlp, "ff", w), limit=float(_need(mlp, "limit", w)))
        elif mk == "moe":
            router, expert = _need(mlp, "router", w), _need(mlp, "expert", w)
            groups = router.get("groups")
            ff = ExpertsConfig(
                experts=_positive(router, "experts", w + ".router"), top=_positive(router, "top", w + ".router"),
                ff=_positive(expert, "ff", w + ".expert"),
                groups=_positive(groups, "count", w + ".router.groups") if groups else 0,
                keep_groups=_positive(groups, "keep", w + ".router.groups") if groups else 0,
                scale=float(router.get("scale", 1.0)),
            )
            if ff.top > ff.experts:
                raise ConfigError(f"config.json: {w}.router: top={ff.top} of {ff.experts} experts")
            if ff.groups:
                if ff.experts % ff.groups or ff.keep_groups > ff.groups:
                    raise ConfigError(f"config.json: {w}.router.groups: {ff.experts} experts in {ff.groups} groups, "
                                      f"{ff.keep_groups} kept")
                if ff.keep_groups * (ff.experts // ff.groups) < ff.top:
                    raise ConfigError(f"config.json: {w}.router: the kept groups hold fewer than top={ff.top} experts")
        else:
            raise ConfigError(f"config.json: {w}.kind {mk!r} is neither 'dense' nor 'moe'")
    return VepevikLayer(kind, mixer, ff)
