"""Typed configuration of the ``Ruburax`` architecture.

``config.json`` gives ``vocab``, ``width``, ``norm.eps``, ``residual_mult``, ``logit_scale``, optionally
``token_side.dim`` and a list ``layers``; every entry names its mixer (``type``: ``"rglru"``,
``"attention"`` or ``"parallel"``), the mixer's sizes (``mixer``) and its feed-forward (``mlp``: dense, a
mixture of experts, or null for none).  Layers may differ from one another in everything.  Nothing here
has a default that stands for a size: a missing key is an error.
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
class RecurrentUnitConfig:
    width: int
    blocks: int
    conv: int


@dataclass(frozen=True)
class FrequencyScaling:
    factor: float
    low: float
    high: float
    original: int


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int                       # 0: no rotation
    rot_scaling: FrequencyScaling | None
    kv_from: int | None = None          # the layer whose keys and values this one reads


@dataclass(frozen=True)
class MatrixMemoryConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: AttentionConfig
    right: MatrixMemoryConfig
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class DenseConfig:
    ff: int


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    ff: int
    scale: float
    groups: int               # 0: no groups
    keep_groups: int
    shared_ff: int            # 0: no shared expert


@dataclass(frozen=True)
class RuburaxLayer:
    type: str
    mixer: RecurrentUnitConfig | AttentionConfig | ParallelMixerConfig
    mlp: DenseConfig | ExpertsConfig | None


@dataclass(frozen=True)
class RuburaxConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    logit_scale: float
    side_dim: int             # 0: no per-layer token input
    layers: tuple[RuburaxLayer, ...]

    @classmethod
    def from_json(cls, raw: Mapping[str, Any]) -> "RuburaxConfig":
        layers = _need(raw, "layers", "the top level")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        side = raw.get("token_side")
        parsed = tuple(_layer(l, f"layers[{i}]") for i, l in enumerate(layers))
        for i, layer in enumerate(parsed):
            m = layer.mixer
            if isinstance(m, AttentionConfig) and m.kv_from is not None:
                j = m.kv_from
                o = parsed[j].mixer if 0 <= j < i else None
                if isinstance(o, ParallelMixerConfig):
                    o = o.left                  # a parallel layer's keys and values are its attention's
                if not isinstance(o, AttentionConfig) or o.kv_from is not None:
                    raise ConfigError(f"config.json: layers[{i}].mixer.kv_from={j} must name an earlier layer with "
                                      "an attention that has keys and values of its own")
                if (o.kv_heads, o.dim, o.vdim) != (m.kv_heads, m.dim, m.vdim):
                    raise ConfigError(f"config.json: layers[{i}] reads layer {j}'s keys and values, whose sizes differ")
        return cls(
            vocab=_positive(raw, "vocab", "the top level"),
            width=_positive(raw, "width", "the top level"),
            eps=float(_need(_need(raw, "norm", "the top level"), "eps", "norm")),
            residual_mult=float(_need(raw, "residual_mult", "the top level")),
            logit_scale=float(_need(raw, "logit_scale", "the top level")),
            side_dim=_positive(side, "dim", "token_side") if side else 0,
            layers=parsed,
        )


def _attention(m: Mapping[str, Any], where: str, shares: bool) -> AttentionConfig:
    rot = m.get("rot")
    dim = _positive(m, "dim", where)
    scaling = None
    if rot and rot.get("scaling"):
        sc = rot["scaling"]
        sw = where + ".rot.scaling"
        scaling = FrequencyScaling(float(_need(sc, "factor", sw)), float(_need(sc, "low", sw)),
                                   float(_need(sc, "high", sw)), _positive(sc, "original", sw))
        if scaling.high == scaling.low:
            raise ConfigError(f"config.json: {sw}: 'high' and 'low' must differ")
    kv_from = m.get("kv_from") if shares else None
    if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int)):
        raise ConfigError(f"config.json: {where}.kv_from must be a layer's index, got {kv_from!r}")
    a = AttentionConfig(
        heads=_positive(m, "heads", where), kv_heads=_positive(m, "kv_heads", where), dim=dim,
        vdim=_positive(m, "vdim", where), scale=float(_need(m, "scale", where)),
        rot_base=float(_need(rot, "base", where + ".rot")) if rot else 0.0,
        rot_dims=int(_need(rot, "dims", where + ".rot")) if rot else 0,
        rot_scaling=scaling, kv_from=kv_from,
    )
    if a.heads % a.kv_heads:
        raise ConfigError(f"config.json: {where}: {a.heads} heads cannot share {a.kv_heads} key/value heads")
    if a.rot_dims % 2 or not 0 <= a.rot_dims <= dim:
        raise ConfigError(f"config.json: {where}.rot.dims={a.rot_dims} must be even and at most dim={dim}")
    return a


def _layer(raw: Mapping[str, Any], where: str) -> RuburaxLayer:
    kind = _need(raw, "type", where)
    m = _need(raw, "mixer", where)
    mw = where + ".mixer"
    if kind == "rglru":
        mixer = RecurrentUnitConfig(width=_positive(m, "width", mw), blocks=_positive(m, "blocks", mw),
                                    conv=_positive(m, "conv", mw))
        if mixer.width % mixer.blocks:
            raise ConfigError(f"config.json: {where}: {mixer.width} channels are no {mixer.blocks} equal parts")
    elif kind == "attention":
        mixer = _attention(m, mw, shares=True)
    elif kind == "parallel":
        r = _need(m, "right", mw)
        rw = mw + ".right"
        right = MatrixMemoryConfig(heads=_positive(r, "heads", rw), dim=_positive(r, "dim", rw),
                                   vdim=_positive(r, "vdim", rw), gate_cap=float(_need(r, "gate_cap", rw)))
        if not right.gate_cap > 0:
            raise ConfigError(f"config.json: {rw}.gate_cap must be positive, got {right.gate_cap}")
        mixer = ParallelMixerConfig(_attention(_need(m, "left", mw), mw + ".left", shares=False), right,
                                    float(_need(m, "left_scale", mw)), float(_need(m, "right_scale", mw)))
    else:
        raise ConfigError(f"config.json: {where}.type {kind!r} is none of 'rglru', 'attention', 'parallel'")
    mlp = raw.get("mlp")
    ff: DenseConfig | ExpertsConfig | None = None
    if mlp is not None:
        fw = where + ".mlp"
        mlp_kind = _need(mlp, "kind", fw)
        if mlp_kind == "dense":
            ff = DenseConfig(_positive(mlp, "ff", fw))
        elif mlp_kind == "moe":
            router, expert = _need(mlp, "router", fw), _need(mlp, "expert", fw)
            groups, shared = router.get("groups"), mlp.get("shared")
            ff = ExpertsConfig(
                experts=_positive(router, "experts", fw + ".router"), top=_positive(router, "top", fw + ".router"),
                ff=_positive(expert, "ff", fw + ".expert"), scale=float(_need(router, "scale", fw + ".router")),
                groups=_positive(groups, "count", fw + ".router.groups") if groups else 0,
                keep_groups=_positive(groups, "keep", fw + ".router.groups") if groups else 0,
                shared_ff=_positive(shared, "ff", fw + ".shared") if shared else 0,
            )
            if ff.top > ff.experts:
                raise ConfigError(f"config.json: {fw}.router: top={ff.top} of {ff.experts} experts")
            if ff.groups:
                if ff.experts % ff.groups or ff.keep_groups > ff.groups:
                    raise ConfigError(f"config.json: {fw}.router.groups: {ff.experts} experts in {ff.groups} groups, "
                                      f"{ff.keep_groups} kept")
                if ff.keep_groups * (ff.experts // ff.groups) < ff.top:
                    raise ConfigError(f"config.json: {fw}.router.groups: {ff.keep_groups} groups of "
                                      f"{ff.experts // ff.groups} experts cannot give {ff.top}")
        else:
            raise ConfigError(f"config.json: {fw}.kind {mlp_kind!r} is neither 'dense' nor 'moe'")
    return RuburaxLayer(kind, mixer, ff)
