"""``Vepevik``: a pre-norm decoder (``x += mixer(norm1(x))``, then ``x += ff(norm2(x))``, RMS norms)
whose layers each have one of three mixers: retention (linear attention with a fixed decay per head),
the gated delta rule with a decay per key channel behind short convolutions, or softmax attention
over chunks of positions with normed queries and keys, values blended with those of the first
such layer, and a gate per head.  A layer's feed-forward is a dense clamped gated unit, a mixture of
experts whose router takes the softmax over all experts and chooses within the best groups, or
absent.  The embedding passes an RMS norm of its own before it starts the fp32 stream; the head is
the embedding table.

This file is the only place that knows the architecture: it turns a ``VepevikConfig`` into a
``ModelSpec`` of generic parts and names the checkpoint tensors (``embed``, ``embed.norm``,
``l{i}.norm1``, ``l{i}.norm2``, ``l{i}.mix.*``, ``l{i}.mlp.*``, ``final.norm``).
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.vepevik import (ChannelDeltaConfig, ChunkAttentionConfig, DenseConfig, ExpertsConfig, RetentionConfig,
                              VepevikConfig)
from ..parts.spec import LayerSpec, ModelSpec, PartSpec


def _rms(H: int, eps: float, name: str) -> PartSpec:
    return PartSpec("rmsnorm", {"hidden_size": H, "eps": eps}, rename={"weight": name})


def _rotary(rot, head_dim: int) -> PartSpec | None:
    if rot is None:
        return None
    return PartSpec("rotary", {"head_dim": head_dim, "theta": rot.base, "rotary_dim": rot.dims, "span": "rotated"})


def assemble(cfg: VepevikConfig) -> ModelSpec:
    H = cfg.width
    layers = []
    unread = []
    blending_seen = False
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        position = None
        if isinstance(m, RetentionConfig):
            mixer = PartSpec("retention", {"hidden_size": H, "num_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim,
                                           "decay": m.decay, "eps": cfg.eps}, prefix=p + "mix.")
            position = _rotary(m.rot, m.dim)
        elif isinstance(m, ChannelDeltaConfig):
            mixer = PartSpec("channel_delta_rule",
                             {"hidden_size": H, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "key_dim": m.dim,
                              "value_dim": m.vdim, "conv_taps": m.conv, "eps": cfg.eps, "unit_eps": 1e-6,
                              "decay_rank": m.decay_rank, "gate_rank": m.gate_rank}, prefix=p + "mix.")
        else:
            assert isinstance(m, ChunkAttentionConfig)
            blend = m.v_mix
            if m.v_mix and not blending_seen:
                # the first blending layer gives its values to the others; its own factor is never used
                blend, blending_seen = "source", True
                unread.append(p + "mix.vmix")
            mixer = PartSpec("chunk_attention",
                             {"hidden_size": H, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                              "value_dim": m.vdim, "scale": m.scale, "chunk": m.chunk, "qk_norm": True, "eps": cfg.eps,
                              "value_blend": blend, "head_gate": True}, prefix=p + "mix.")
            position = _rotary(m.rot, m.dim)
        e = layer.mlp
        if e is None:
            feed_forward, ff_norm = PartSpec("no_feed_forward"), PartSpec("no_norm")
            unread.append(p + "norm2")      # a layer without a feed-forward has nothing behind a second norm
        elif isinstance(e, DenseConfig):
            feed_forward = PartSpec("clamped_glu_mlp", {"hidden_size": H, "intermediate_size": e.ff, "limit": e.limit,
                                                        "alpha": 1.702, "up_offset": 1.0}, prefix=p + "mlp.")
            ff_norm = _rms(H, cfg.eps, p + "norm2")
        else:
            assert isinstance(e, ExpertsConfig)
            feed_forward = PartSpec("routed_experts",
                                    {"hidden_size": H, "experts": e.experts, "top": e.top, "expert_ff": e.ff,
                                     "activation": "silu", "scores": "all", "route_scale": e.scale,
                                     "groups": e.groups, "keep_groups": e.keep_groups}, prefix=p + "mlp.")
            ff_norm = _rms(H, cfg.eps, p + "norm2")
        layers.append(LayerSpec(mixer=mixer, feed_forward=feed_forward, mixer_norm=_rms(H, cfg.eps, p + "norm1"),
                                feed_forward_norm=ff_norm, position=position, arrangement="prenorm"))
    return ModelSpec(
        hidden_size=H,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": H, "norm_eps": cfg.eps},
                           rename={"weight": "embed", "norm": "embed.norm"}),
        layers=tuple(layers),
        final_norm=_rms(H, cfg.eps, "final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": H, "tied": True},
                      rename={"weight": "head"}),
        max_positions=None,
        ignorable=tuple(unread),
    )


register_architecture("Vepevik", VepevikConfig.from_json, assemble, replace=True)
