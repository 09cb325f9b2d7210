"""``Ruburax``: a decoder whose branches read the residual stream itself and whose norms stand behind
the branches: ``x += m * norm1(mixer(x))``, then ``x += m * norm2(ff(x))``, then a per-layer input from
the token itself, ``x += m * norm(W_proj (gelu_tanh(W_gate x) * e))`` with ``e`` the layer's columns of
the token's row of a side table.  A layer's mixer is a real-gated linear recurrent unit, softmax
attention (biases, normed queries and keys, rotary positions with a frequency rescale, a learned sink
per head; a layer may read an earlier layer's keys and values), or, side by side, such an attention
without biases and sink and a matrix memory with scalar gates.  The feed-forward is a dense SiLU-gated
unit, a mixture of experts (sigmoid scores, a correction of the choice, groups ranked by their two best,
a gated shared expert), or absent.  The head is the embedding table times a factor.

This file is the only place that knows the architecture: it turns a ``RuburaxConfig`` into a
``ModelSpec`` of generic parts and names the checkpoint tensors (``embed``, ``side.embed``, ``l{i}.norm1``,
``l{i}.norm2``, ``l{i}.mix.*``, ``l{i}.mlp.*``, ``l{i}.side.*``, ``final.norm``).
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.ruburax import (AttentionConfig, DenseConfig, ExpertsConfig, ParallelMixerConfig, RecurrentUnitConfig,
                              RuburaxConfig)
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _branch_norm(H: int, eps: float, mult: float, name: str) -> PartSpec:
    return PartSpec("branch_rmsnorm", {"hidden_size": H, "eps": eps, "mult": mult}, rename={"weight": name})


def _rotary(a: AttentionConfig) -> PartSpec | None:
    if not a.rot_dims:
        return None
    scaling = None
    if a.rot_scaling is not None:
        sc = a.rot_scaling
        scaling = {"factor": sc.factor, "low_freq_factor": sc.low, "high_freq_factor": sc.high,
                   "original_max_position_embeddings": sc.original}
    return PartSpec("rotary", {"head_dim": a.dim, "theta": a.rot_base, "rotary_dim": a.rot_dims, "span": "rotated",
                               "scaling": scaling})


def _attention(a: AttentionConfig, H: int, eps: float, prefix: str, *, bias: bool, sink: bool) -> PartSpec:
    return PartSpec("normed_attention",
                    {"hidden_size": H, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim,
                     "value_dim": a.vdim, "scale": a.scale, "qk_norm": True, "eps": eps, "bias": bias,
                     "sink": "learned" if sink else None, "own_kv": a.kv_from is None}, prefix=prefix)


def assemble(cfg: RuburaxConfig) -> ModelSpec:
    H, eps, mult = cfg.width, cfg.eps, cfg.residual_mult
    layers, schedule = [], []
    cache_of: dict[int, int] = {}       # layer -> the cache layer it writes
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        position = None
        if isinstance(m, RecurrentUnitConfig):
            mixer = PartSpec("rglru", {"hidden_size": H, "width": m.width, "blocks": m.blocks, "conv_taps": m.conv,
                                       "decay_scale": 8.0}, prefix=p + "mix.")
        elif isinstance(m, AttentionConfig):
            mixer = _attention(m, H, eps, p + "mix.", bias=True, sink=True)
            position = _rotary(m)
        else:
            assert isinstance(m, ParallelMixerConfig)
            R = m.right
            right = PartSpec("matrix_memory", {"hidden_size": H, "num_heads": R.heads, "key_dim": R.dim,
                                               "value_dim": R.vdim, "gate_cap": R.gate_cap, "eps": eps,
                                               "den_eps": 1e-6}, prefix="right.")
            mixer = PartSpec("side_by_side", {"left": _attention(m.left, H, eps, "left.", bias=False, sink=False),
                                              "right": right, "left_scale": m.left_scale,
                                              "right_scale": m.right_scale}, prefix=p + "mix.")
            position = _rotary(m.left)
        e = layer.mlp
        if e is None:
            feed_forward, ff_norm = PartSpec("no_feed_forward"), PartSpec("no_norm")
        elif isinstance(e, DenseConfig):
            feed_forward = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": e.ff, "activation": "silu"},
                                    rename={"gate_proj.weight": p + "mlp.gate", "up_proj.weight": p + "mlp.up",
                                            "down_proj.weight": p + "mlp.down"})
            ff_norm = _branch_norm(H, eps, mult, p + "norm2")
        else:
            assert isinstance(e, ExpertsConfig)
            feed_forward = PartSpec("routed_experts",
                                    {"hidden_size": H, "experts": e.experts, "top": e.top, "expert_ff": e.ff,
                                     "activation": "silu", "scores": "sigmoid", "correction": True,
                                     "route_scale": e.scale, "groups": e.groups, "keep_groups": e.keep_groups,
                                     "group_score": "top2", "shared_ff": e.shared_ff,
                                     "shared_gate": "sigmoid" if e.shared_ff else None}, prefix=p + "mlp.")
            ff_norm = _branch_norm(H, eps, mult, p + "norm2")
        layers.append(LayerSpec(mixer=mixer, feed_forward=feed_forward, mixer_norm=_branch_norm(H, eps, mult, p + "norm1"),
                                feed_forward_norm=ff_norm, position=position, arrangement="branch_norm"))
        after = None
        if cfg.side_dim:
            after = PartSpec("token_side_input",
                             {"hidden_size": H, "vocab_size": cfg.vocab, "dim": cfg.side_dim, "index": i,
                              "table_width": cfg.side_dim * len(cfg.layers), "eps": eps, "mult": mult},
                             prefix=p + "side.", rename={"table": "side.embed"})
        reads = m.kv_from if isinstance(m, AttentionConfig) else None
        if reads is None:
            cache_of[i] = len(cache_of)
            schedule.append(ScheduleEntry(layer=i, cache=cache_of[i], writes_cache=True, after=after))
        else:
            schedule.append(ScheduleEntry(layer=i, cache=cache_of[reads], writes_cache=False, after=after))
    return ModelSpec(
        hidden_size=H,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": H, "scale": 1.0},
                           rename={"weight": "embed"}),
        layers=tuple(layers),
        final_norm=PartSpec("rmsnorm", {"hidden_size": H, "eps": eps}, rename={"weight": "final.norm"}),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": H, "tied": True,
                                      "scale": cfg.logit_scale}, rename={"weight": "head"}),
        schedule=tuple(schedule),
        max_positions=None,
    )


register_architecture("Ruburax", RuburaxConfig.from_json, assemble, replace=True)
