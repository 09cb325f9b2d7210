"""The parts that ship with the package: RMS norm, rotary position encoding, grouped-query
attention, SwiGLU feed-forward, token embedding, output head, the pre-norm arrangement.

Each class takes its sizes and constants from its ``PartSpec.params`` and its tensors from
``bind``.  The formulas follow the reference's blocks, cited per class.
"""

from __future__ import annotations

import math

import torch

from ..csrc import ops
from .base import (
    Arrangement,
    BranchSum,
    DeferredNorm,
    FeedForward,
    KVNeed,
    LayerCache,
    Mixer,
    Norm,
    ParamDecl,
    Part,
    PlanNeeds,
    Position,
    StepContext,
    StreamCopy,
    StreamPart,
    StreamSink,
    register_arrangement,
    register_embedding,
    register_feed_forward,
    register_head,
    register_mixer,
    register_norm,
    register_position,
    register_stream_part,
)


def _as_compute(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """A matrix operand in the compute dtype (a no-op when it is stored that way)."""
    return t if t.dtype == dtype else t.to(dtype)


class Linear:
    """``y = x W^T`` with ``W [out, in]`` kept in the compute dtype.

    ``x`` may be a ``DeferredNorm`` whose statistics are row sums of squares (the product then
    finishes the norm in its epilogue), and ``into_stream`` adds the product to a sink's stream;
    ``fusable`` says whether this matrix and row count have those forms."""

    def __init__(self, weight: torch.Tensor) -> None:
        if weight.dim() != 2 or not weight.is_contiguous():
            raise ValueError("Linear needs a contiguous [out, in] matrix")
        self.weight = weight

    def __call__(self, x, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        if isinstance(x, DeferredNorm):
            if x.kind != "rms":
                raise ValueError(f"this product cannot finish a norm of kind {x.kind!r}")
            return ops.linear(x.x, self.weight, out_dtype, row_stats=x.stats)
        return ops.linear(x, self.weight, out_dtype)

    def fusable(self, n_rows: int, kind: str = "rms") -> bool:
        return kind == "rms" and ops.linear_fusable(n_rows, self.weight)

    def into_stream(self, x: torch.Tensor, sink: StreamSink) -> DeferredNorm:
        if sink.kind != "rms":
            raise ValueError(f"this product cannot finish a norm of kind {sink.kind!r}")
        gain, eps = sink.payload
        y, stats = ops.linear_into_stream(x, self.weight, sink.residual, gain, eps)
        return DeferredNorm(sink.norm, sink.kind, y, stats, sink.residual)


# ----------------------------------------------------------------------------- norm


class RMSNorm(Norm):
    """``w * r * rsqrt(mean(r^2) + eps)`` with ``r = x + residual`` in fp32
    (reference ``models/blocks/rmsnorm.py:63-93``; the residual sum is kept in fp32 here
    instead of being rounded to the model dtype).

    params: ``hidden_size``, ``eps``.  tensors: ``weight [hidden_size]``.
    """

    deferred_kind = "rms"

    def param_decls(self):
        return {"weight": ParamDecl((int(self.param("hidden_size")),), "gain")}

    def bind(self, tensors, dtype, device):
        w = tensors["weight"]
        # a gain stored in 32-bit stays 32-bit; anything else follows the compute dtype
        self.weight = w if w.dtype == torch.float32 else w.to(dtype)
        self.eps = float(self.param("eps"))
        self.dtype = dtype
        self._gain32 = None

    def stream_sink(self, residual, n_rows):
        if (not ops.fused_norms_enabled() or residual is None
                or n_rows > ops.TMA_GEMM_FUSED_ROWS or not residual.is_cuda):
            return None
        if getattr(self, "_gain32", None) is None:
            self._gain32 = self.weight.to(torch.float32).contiguous()   # the products' epilogues read fp32
        return StreamSink(self, self.deferred_kind, residual, (self._gain32, self.eps))

    def forward(self, x, residual, rows=None):
        if isinstance(x, DeferredNorm):
            if x.norm is not self or rows is not None:
                raise ValueError("a deferred norm was handed to another norm than the one it was made for")
            return x, x.residual
        if isinstance(x, BranchSum) or (residual is None and x.dtype == torch.float32 and self.dtype != torch.float32):
            return self._forward_sum(x, residual, rows)
        if rows is not None:
            return ops.add_rmsnorm(x, self.weight, self.eps, residual_in=residual, rows=rows), None
        new_residual = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        out = ops.add_rmsnorm(x, self.weight, self.eps, residual_in=residual,
                              residual_out=new_residual)
        return out, new_residual

    def _forward_sum(self, x, residual, rows):
        """Several addends at once, none of them rounded on the way: the outputs of parallel
        branches (compute dtype), an fp32 tensor and an fp32 row that a stream part left
        (``BranchSum.stream_add``, ``row_add``); before the first layer an fp32 ``x`` is the stream
        itself.  The stream that comes in is left as it is; a new one is returned."""
        if getattr(self, "_gain32", None) is None:
            self._gain32 = self.weight.to(torch.float32).contiguous()
        adds, add32, row_add = (), None, None
        if isinstance(x, BranchSum):
            adds, add32, row_add = tuple(x), x.stream_add, x.row_add
        elif residual is None and x.dtype == torch.float32:
            residual = x
        else:
            adds = (x,)
        return ops.add_rmsnorm_multi(residual, adds, self._gain32, self.eps, self.dtype, add32=add32,
                                     row_add=row_add, rows=rows)


class SameNorm(Norm):
    """The place of a feed-forward's norm in a layer whose two branches read one norm's output."""

    def forward(self, x, residual, rows=None):
        raise RuntimeError("this layer's feed-forward reads the mixer's norm")


class LayerNorm(Norm):
    """``(r - mean(r)) / sqrt(var(r) + eps) * w + b`` with ``r = x + residual`` in fp32, the variance
    being the mean of the squared deviations.  ``x`` may be a ``BranchSum``: its parts are added to
    the stream one by one in fp32.  The stream is updated in place.

    params: ``hidden_size``, ``eps``.  tensors: ``weight [hidden_size]``, ``bias [hidden_size]``.
    """

    def param_decls(self):
        H = int(self.param("hidden_size"))
        return {"weight": ParamDecl((H,), "gain"), "bias": ParamDecl((H,), "table")}

    def bind(self, tensors, dtype, device):
        self.weight = tensors["weight"].to(torch.float32).contiguous()
        self.bias = tensors["bias"].to(torch.float32).contiguous()
        self.eps = float(self.param("eps"))
        self.dtype = dtype

    @staticmethod
    def stream_and_addends(x, residual):
        """The fp32 stream and what is still to be added to it, from a layer's ``(x, residual)``:
        before the first layer ``x`` is the embedding and becomes the stream."""
        if residual is None:
            if isinstance(x, BranchSum):
                x = x.total()
            return (x if x.dtype == torch.float32 else x.to(torch.float32)).contiguous(), ()
        return residual, (tuple(x) if isinstance(x, BranchSum) else (x,))

    def forward(self, x, residual, rows=None):
        stream, adds = self.stream_and_addends(x, residual)
        out, = ops.add_layernorm(stream, adds, [(self.weight, self.bias)], self.eps, self.dtype, rows=rows)
        return out, (None if rows is not None else stream)

    def forward_with(self, other: "LayerNorm", x, residual):
        """This norm and ``other`` of the same stream in one pass: ``(out_self, out_other, stream)``."""
        stream, adds = self.stream_and_addends(x, residual)
        a, b = ops.add_layernorm(stream, adds, [(self.weight, self.bias), (other.weight, other.bias)],
                                 self.eps, self.dtype)
        return a, b, stream


class BranchRMSNorm(Norm):
    """An RMS norm that stands behind a branch instead of in front of it: the branch reads the stream
    itself, and the stream takes ``mult * w * y * rsqrt(mean(y^2) + eps)`` of the branch's output ``y``
    (``add_branch``).  The statistics, the product with the gain and the sum are fp32.

    params: ``hidden_size``, ``eps``, optional ``mult`` (default 1).  tensors: ``weight [hidden_size]``.
    """

    def param_decls(self):
        return {"weight": ParamDecl((int(self.param("hidden_size")),), "gain")}

    def bind(self, tensors, dtype, device):
        self.weight = tensors["weight"].to(torch.float32).contiguous()
        self.eps = float(self.param("eps"))
        self.mult = float(self.spec.params.get("mult", 1.0))
        self.dtype = dtype

    def add_branch(self, stream: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        """Adds the normed branch to the fp32 ``stream`` in place; returns the stream's copy in the
        compute dtype (the stream itself for float32)."""
        if isinstance(y, BranchSum):
            y = y.total()
        return ops.scaled_norm_add(stream, y, self.weight, self.eps, self.mult, self.dtype)

    def forward(self, x, residual, rows=None):
        raise RuntimeError("this norm stands behind a branch; the arrangement calls add_branch")


def stream_and_copy(x, residual, dtype: torch.dtype):
    """``(fp32 stream, its copy in the compute dtype)`` from what a layer is handed: a ``StreamCopy`` beside
    the stream, the embedding's output before the first layer, or addends that are still to be added."""
    if isinstance(x, StreamCopy) and residual is not None and x.rounded is not None:
        return residual, x.rounded
    if residual is None:
        if isinstance(x, BranchSum):
            x = x.total()
        stream = x if x.dtype == torch.float32 else x.to(torch.float32)
        return stream, (x if x.dtype == dtype else ops.scaled_norm_add(stream, None, None, 0.0, 1.0, dtype))
    if isinstance(x, BranchSum):
        x = x.total() if len(x) or x.stream_add is not None or x.row_add is not None else None
    if x is not None:
        residual = residual + x.to(torch.float32)
    return residual, ops.scaled_norm_add(residual, None, None, 0.0, 1.0, dtype)


class NoNorm(Norm):
    """The place of a norm in a layer that has nothing behind it (a layer without a feed-forward)."""

    def forward(self, x, residual, rows=None):
        raise RuntimeError("a layer asked the norm of a branch it does not have")


# ----------------------------------------------------------------------------- position


def rotary_inv_freq(head_dim: int, theta: float, rotary_dim: int | None = None,
                    scaling: dict | None = None) -> torch.Tensor:
    """fp32 rotation frequencies ``theta^(-2i/d)``, optionally with the llama3 rescale.

    The rescale sorts frequencies by wavelength into three bands: short waves (below
    ``L / high_freq_factor``, ``L`` the original context length) are kept, long waves (above
    ``L / low_freq_factor``) are slowed down by ``factor``, and the band between is a blend of
    both that is linear in ``L / wavelength``.  Every intermediate is fp32 and the
    operations run in the order of the reference's ``models/blocks/rope.py:200-225``, so
    the table comes out bit-equal to the reference's (a test compares them).
    """
    width = head_dim if rotary_dim is None else rotary_dim
    exponent = torch.arange(0, width, 2, dtype=torch.float32) / head_dim
    freq = 1.0 / (theta ** exponent)
    if scaling is None:
        return freq
    slow_down = float(scaling["factor"])
    low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    context = int(scaling["original_max_position_embeddings"])
    wave = 2 * math.pi / freq
    is_long, is_short = wave > context / low, wave < context / high
    slowed = torch.where(is_long, freq / slow_down, freq)
    blend = (context / wave - low) / (high - low)          # 0 at the long edge, 1 at the short edge
    blended = (1 - blend) * slowed / slow_down + blend * slowed
    in_between = ~is_short * ~is_long
    return torch.where(in_between, blended, slowed)


def rotary_freq64(over: int, theta: float, rotary_dim: int, scaling: dict | None) -> torch.Tensor:
    """The same frequencies in float64 from end to end (``theta^(-2i / over)`` for ``i < rotary_dim / 2``, with
    the three bands of the rescale where ``scaling`` is given), for kernels that form the angle in double
    precision."""
    out = []
    for i in range(rotary_dim // 2):
        f = float(theta) ** (-2.0 * i / over)
        if scaling is not None:
            slow_down = float(scaling["factor"])
            low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
            context = float(scaling["original_max_position_embeddings"])
            wave = 2.0 * math.pi / f
            if wave > context / low:
                f = f / slow_down
            elif not wave < context / high:
                blend = (context / wave - low) / (high - low)
                f = (1.0 - blend) * f / slow_down + blend * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64)


class RotaryPosition(Position):
    """Rotary encoding, half layout: dim ``j`` pairs with ``j + rotary_dim/2``
    (reference ``models/blocks/rope.py:392-431``).  Angles ``p * inv_freq`` and their sine
    and cosine are fp32 and computed in the kernel; each rotated value is rounded once.

    params: ``head_dim``, ``theta``, optional ``rotary_dim`` (default ``head_dim``),
    optional ``scaling`` (the llama3 mapping), optional ``span`` (``"head"``, the default: dimension
    ``i`` turns with ``theta^(-2i / head_dim)``; ``"rotated"``: with ``theta^(-2i / rotary_dim)``).

    A mixer whose own kernel rotates reads ``rotary_dim`` and ``freq64`` (the frequencies in float64:
    such a kernel forms the angle in double precision).
    """

    def bind(self, tensors, dtype, device):
        d = int(self.param("head_dim"))
        self.rotary_dim = int(self.spec.params.get("rotary_dim") or d)
        span = self.spec.params.get("span", "head")
        if span not in ("head", "rotated"):
            raise ValueError(f"unknown span {span!r} of the rotation's frequencies: 'head' or 'rotated'")
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= d:
            raise ValueError(f"{self.rotary_dim} rotated dimensions of a head of {d}")
        over = d if span == "head" else self.rotary_dim
        self.inv_freq = rotary_inv_freq(
            over, float(self.param("theta")), self.rotary_dim, self.spec.params.get("scaling")
        ).to(device)
        self.freq64 = rotary_freq64(over, float(self.param("theta")), self.rotary_dim,
                                    self.spec.params.get("scaling")).to(device)
        # layers with the same frequencies share one table per step
        self._table_key = (d, self.rotary_dim, float(self.param("theta")), repr(self.spec.params.get("scaling")), span)

    def encode(self, qkv, nq, nkv, head_dim, ctx):
        ops.rope_write(qkv, nq, nkv, head_dim, positions=ctx.positions, inv_freq=self.inv_freq,
                       rotary_dim=self.rotary_dim)

    def step_table(self, ctx, head_dim):
        """Sines and cosines of this step's positions for a mixer that rotates by itself, or
        None where that is not possible (a rotary width below the head size).  Layers share one
        table per step: it depends on the positions and the frequencies only."""
        if self.rotary_dim != head_dim:
            return None
        key = ("rope_table", self._table_key)
        table = ctx.scratch.get(key)
        if table is None:
            table = ctx.scratch[key] = ops.rope_table(ctx.positions, self.inv_freq)
        return table

    def rotate_and_store(self, qkv, nq, nkv, head_dim, ctx, cache):
        if cache.writes and cache.k is not None:
            ops.rope_write(qkv, nq, nkv, head_dim, positions=ctx.positions,
                           inv_freq=self.inv_freq, rotary_dim=self.rotary_dim,
                           slots=ctx.groups[cache.group].slots, kcache=cache.k, vcache=cache.v)
        else:
            self.encode(qkv, nq, nkv, head_dim, ctx)


class InterleavedRotary(Position):
    """Rotary encoding, interleaved layout: on the first ``rotary_dim`` dimensions of a head,
    dimension ``2i`` pairs with ``2i + 1`` and the pair ``(u, v)`` at position ``p`` becomes
    ``(u cos a - v sin a, v cos a + u sin a)``, ``a = p * theta^(-2i / rotary_dim)``; the other
    dimensions pass.  The frequencies are rounded once from float64; angles, sines and cosines are
    fp32 in the kernel.  A mixer with a fused kernel reads ``inv_freq`` and ``rotary_dim`` itself.

    params: ``head_dim``, ``theta``, optional ``rotary_dim`` (default ``head_dim``).
    """

    def bind(self, tensors, dtype, device):
        d = int(self.param("head_dim"))
        self.rotary_dim = int(self.spec.params.get("rotary_dim") or d)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= d:
            raise ValueError(f"{self.rotary_dim} rotated dimensions of a head of {d}")
        theta = float(self.param("theta"))
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        self.inv_freq = (theta ** (-2.0 * i / self.rotary_dim)).to(torch.float32).to(device)

    def encode(self, qkv, nq, nkv, head_dim, ctx):
        ops.rope_norm_store(qkv, 0, nq * head_dim, (nq + nkv) * head_dim, nq, nkv, head_dim, head_dim,
                            positions=ctx.positions, inv_freq=self.inv_freq, rot=self.rotary_dim,
                            unit_norm=False, eps=0.0)


# ----------------------------------------------------------------------------- mixer


class GroupedQueryAttention(Mixer):
    """Causal attention with ``num_heads`` query heads sharing ``num_kv_heads`` key/value
    heads over the paged cache (reference ``models/blocks/gqa.py:111-155`` and
    ``cache/packed_attention.py:242-340``): one merged q/k/v projection, position encoding
    of q and k, k/v written to pages, softmax(q k^T * scale + causal [+ window]) v in fp32,
    output projection.

    params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``; optional
    ``window`` (keys older than ``window - 1`` positions are not seen), ``scale``
    (default ``head_dim ** -0.5``).
    tensors: ``q_proj.weight``, ``k_proj.weight``, ``v_proj.weight``, ``o_proj.weight``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.nq = int(self.param("num_heads"))
        self.nkv = int(self.param("num_kv_heads"))
        self.d = int(self.param("head_dim"))
        w = self.spec.params.get("window")
        self.window = int(w) if w else None
        s = self.spec.params.get("scale")
        self.scale = float(s) if s else self.d ** -0.5
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads cannot share {self.nkv} key/value heads")
        if self.d % 16 or not 16 <= self.d <= 256:
            raise ValueError(f"head_dim {self.d} is not a multiple of 16 in [16, 256]")

    def param_decls(self):
        H, nq, nkv, d = self.hidden, self.nq, self.nkv, self.d
        return {
            "q_proj.weight": ParamDecl((nq * d, H)),
            "k_proj.weight": ParamDecl((nkv * d, H)),
            "v_proj.weight": ParamDecl((nkv * d, H)),
            "o_proj.weight": ParamDecl((H, nq * d)),
        }

    def cache_need(self):
        return KVNeed(self.nkv, self.d, self.window)

    def plan_needs(self):
        return PlanNeeds(ops.attention_tile_sizes(self.nq // self.nkv))

    def bind(self, tensors, dtype, device):
        qkv = torch.cat(
            [_as_compute(tensors[n], dtype) for n in ("q_proj.weight", "k_proj.weight", "v_proj.weight")],
            dim=0,
        ).contiguous()
        self.qkv_proj = Linear(qkv)
        self.o_proj = Linear(_as_compute(tensors["o_proj.weight"], dtype).contiguous())

    def takes_deferred_norm(self, n_rows, kind):
        return self.qkv_proj.fusable(n_rows, kind)

    def adds_to_stream(self, n_rows, kind):
        return self.o_proj.fusable(n_rows, kind)

    def forward(self, x, ctx: StepContext, cache: LayerCache, position, into=None):
        nq, nkv, d = self.nq, self.nkv, self.d
        qkv = self.qkv_proj(x)
        table = None
        if (position is not None and cache.k is not None
                and ops.decode_rope_fusable(x.dtype, d, ctx.decode_only, ctx.n_requests)):
            table = position.step_table(ctx, d)   # the decode kernel rotates q and stores the new k, v itself
        if table is not None:
            pass
        elif position is not None:
            position.rotate_and_store(qkv, nq, nkv, d, ctx, cache)
        elif cache.writes:
            ops.rope_write(qkv, nq, nkv, d, slots=ctx.groups[cache.group].slots,
                           kcache=cache.k, vcache=cache.v)
        out = torch.empty((ctx.n_tokens, nq * d), dtype=x.dtype, device=x.device)
        ops.attention(qkv, qkv.stride(0), out, cache, ctx, nq, nkv, d, self.scale, self.window or 0,
                      rope_table=table)
        return self.o_proj(out) if into is None else self.o_proj.into_stream(out, into)


# ----------------------------------------------------------------------------- feed-forward


class SwiGLU(FeedForward):
    """``down(silu(gate(x)) * up(x))``, no biases (reference ``models/blocks/swiglu.py:35-46``,
    ``models/blocks/activations.py:36-45``).  gate and up are one merged product whose rows
    alternate (gate 0, up 0, gate 1, up 1, ...), so that the activation can run in the
    product's epilogue, where both halves of a pair sit side by side; SiLU and the product
    are fp32 per element.

    params: ``hidden_size``, ``intermediate_size``, optional ``activation`` (``"silu"``, the default,
    or ``"gelu_tanh"``: ``0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))`` in the SiLU's place).
    tensors: ``gate_proj.weight``, ``up_proj.weight``, ``down_proj.weight``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        self.activation = str(self.spec.params.get("activation", "silu"))
        if self.activation not in ops.GLU_ACT:
            raise ValueError(f"unknown activation {self.activation!r}; known: {sorted(ops.GLU_ACT)}")

    def param_decls(self):
        H, I = int(self.param("hidden_size")), int(self.param("intermediate_size"))
        return {
            "gate_proj.weight": ParamDecl((I, H)),
            "up_proj.weight": ParamDecl((I, H)),
            "down_proj.weight": ParamDecl((H, I)),
        }

    def bind(self, tensors, dtype, device):
        gate, up = _as_compute(tensors["gate_proj.weight"], dtype), _as_compute(tensors["up_proj.weight"], dtype)
        gate_up = torch.stack([gate, up], dim=1).reshape(2 * gate.shape[0], gate.shape[1]).contiguous()
        self.gate_up_proj = Linear(gate_up)
        self.down_proj = Linear(_as_compute(tensors["down_proj.weight"], dtype).contiguous())

    def takes_deferred_norm(self, n_rows, kind):
        return self.gate_up_proj.fusable(n_rows, kind)

    def adds_to_stream(self, n_rows, kind):
        return self.down_proj.fusable(n_rows, kind)

    def forward(self, x, ctx, into=None):
        if isinstance(x, DeferredNorm):
            if x.kind != "rms":
                raise ValueError(f"this product cannot finish a norm of kind {x.kind!r}")
            h = ops.linear_swiglu(x.x, self.gate_up_proj.weight, row_stats=x.stats, act=self.activation)
        else:
            h = ops.linear_swiglu(x, self.gate_up_proj.weight, act=self.activation)
        return self.down_proj(h) if into is None else self.down_proj.into_stream(h, into)


class ClampedGLU(FeedForward):
    """``down(g' * sigmoid(alpha g') * (u' + up_offset))`` with ``g' = min(gate(x), limit)`` and
    ``u' = clamp(up(x), -limit, limit)``, no biases: the dense form of the routed experts' clamped
    activation.  gate and up are one merged product (gate rows, then up rows).

    params: ``hidden_size``, ``intermediate_size``, ``limit``, optional ``alpha`` (default 1.702),
    ``up_offset`` (default 1).  tensors: ``gate``, ``up``, ``down``.
    """

    def param_decls(self):
        H, I = int(self.param("hidden_size")), int(self.param("intermediate_size"))
        return {"gate": ParamDecl((I, H)), "up": ParamDecl((I, H)), "down": ParamDecl((H, I))}

    def bind(self, tensors, dtype, device):
        self.limit = float(self.param("limit"))
        self.alpha = float(self.spec.params.get("alpha", 1.702))
        self.up_offset = float(self.spec.params.get("up_offset", 1.0))
        self.gate_up = Linear(torch.cat([_as_compute(tensors["gate"], dtype), _as_compute(tensors["up"], dtype)],
                                        dim=0).contiguous())
        self.down = Linear(_as_compute(tensors["down"], dtype).contiguous())

    def forward(self, x, ctx):
        return self.down(ops.clamped_glu(self.gate_up(x), self.limit, self.alpha, self.up_offset))


# ----------------------------------------------------------------------------- embedding / head


class TokenEmbedding(Part):
    """``h0 = E[token]`` (reference ``models/llama/llama.py:104,159``), or with ``scale``
    ``h0 = float(E[token]) * scale``, or with ``norm_eps`` ``h0 = x / sqrt(mean(x^2) + norm_eps) * w``
    (``x = float(E[token])``, an RMS norm of the embedding's own); the latter two are then the fp32
    residual stream itself.

    params: ``vocab_size``, ``hidden_size``, optional ``scale``, optional ``norm_eps``.
    tensors: ``weight [vocab, hidden]`` and, with ``norm_eps``, ``norm [hidden]``.
    """

    def param_decls(self):
        decls = {"weight": ParamDecl((int(self.param("vocab_size")), int(self.param("hidden_size"))))}
        if self.spec.params.get("norm_eps") is not None:
            if self.spec.params.get("scale") is not None:
                raise ValueError("an embedding is scaled or normalised, not both")
            decls["norm"] = ParamDecl((int(self.param("hidden_size")),), "gain")
        return decls

    def bind(self, tensors, dtype, device):
        self.weight = _as_compute(tensors["weight"], dtype).contiguous()
        self.norm_gain = None
        if self.spec.params.get("norm_eps") is not None:
            self.norm_gain = tensors["norm"].to(torch.float32).contiguous()

    def forward(self, ctx: StepContext) -> torch.Tensor:
        if self.norm_gain is not None:
            return ops.embedding_rmsnorm(self.weight, ctx.token_ids, self.norm_gain, float(self.spec.params["norm_eps"]))
        scale = self.spec.params.get("scale")
        if scale is not None:
            return ops.embedding_scaled(self.weight, ctx.token_ids, float(scale))
        return ops.embedding(self.weight, ctx.token_ids)


class OutputHead(Part):
    """``logits = z W^T`` in fp32 (reference ``models/llama/llama.py:169-172``).  With
    ``tied`` the embedding's table is the weight and no tensor of its own is expected.

    params: ``vocab_size``, ``hidden_size``, ``tied``, optional ``scale`` (the logits are multiplied by it,
    in fp32).  tensors: ``weight`` unless tied.
    """

    @property
    def tied(self) -> bool:
        return bool(self.spec.params.get("tied", False))

    def param_decls(self):
        if self.tied:
            return {}
        return {"weight": ParamDecl((int(self.param("vocab_size")), int(self.param("hidden_size"))))}

    def bind(self, tensors, dtype, device, tied_weight: torch.Tensor | None = None):
        if self.tied:
            if tied_weight is None:
                raise ValueError("a tied head needs the embedding's table")
            self.proj = Linear(tied_weight)
        else:
            self.proj = Linear(_as_compute(tensors["weight"], dtype).contiguous())

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        logits = self.proj(z, out_dtype=torch.float32)
        scale = self.spec.params.get("scale")
        if scale is not None and float(scale) != 1.0:
            ops.scale_(logits, float(scale))
        return logits


# ----------------------------------------------------------------------------- arrangement


class PreNormBlock(Arrangement):
    """``h += mixer(norm1(h)); h += ffn(norm2(h))`` with every addition folded into the
    following norm (reference ``models/blocks/transformer_block.py:107-120,140-153``): the
    block receives the previous branch output ``x`` and the fp32 stream ``residual``, and
    returns its feed-forward output with the stream that does not yet include it.

    Where the parts on both sides of a norm say they can (few rows, bfloat16), the branch's last
    product adds its result to the stream itself and the product after the norm finishes the
    norm in its epilogue, so that the norm launches nothing: within the block for the second
    norm, and across blocks when the layer that follows gave its ``entry``.

    A layer without a feed-forward (``no_feed_forward``) is ``h += mixer(norm1(h))`` alone.
    """

    def entry(self):
        return self.mixer_norm, self.mixer

    @staticmethod
    def _sink(producer, norm, consumer, residual, n_rows):
        kind = norm.deferred_kind
        if (kind is None or residual is None or not producer.adds_to_stream(n_rows, kind)
                or not consumer.takes_deferred_norm(n_rows, kind)):
            return None
        return norm.stream_sink(residual, n_rows)

    def forward(self, x, residual, ctx, cache, following=None):
        n = ctx.n_tokens
        a, residual = self.mixer_norm.forward(x, residual)
        if isinstance(self.feed_forward, NoFeedForward):
            return self.mixer.forward(a, ctx, cache, self.position), residual
        sink = self._sink(self.mixer, self.feed_forward_norm, self.feed_forward, residual, n)
        if sink is None:
            h = self.mixer.forward(a, ctx, cache, self.position)
        else:
            h = self.mixer.forward(a, ctx, cache, self.position, into=sink)
        b, residual = self.feed_forward_norm.forward(h, residual)
        sink = self._sink(self.feed_forward, following[0], following[1], residual, n) if following else None
        if sink is None:
            f = self.feed_forward.forward(b, ctx)
        else:
            f = self.feed_forward.forward(b, ctx, into=sink)
        return f, residual


class ParallelBlock(Arrangement):
    """``h += mixer(norm1(h)) + ffn(norm2(h))``: both branches read the same stream.  The block
    receives the previous layer's branch outputs (a ``BranchSum``, or the embedding before the first
    layer) with the fp32 stream that does not yet include them, adds them while it normalises, and
    returns its own branch outputs unadded.  Two ``LayerNorm``s of one ``eps`` run as one kernel.
    A layer without a feed-forward (``no_feed_forward``) has the mixer's branch alone; with
    ``same_norm`` in the feed-forward norm's place both branches read the mixer norm's output
    (``h += mixer(n) + ffn(n)``, ``n = norm1(h)``)."""

    def forward(self, x, residual, ctx, cache):
        ff = None if isinstance(self.feed_forward, NoFeedForward) else self.feed_forward
        n1, n2 = self.mixer_norm, self.feed_forward_norm
        if ff is None:
            a, stream = n1.forward(x, residual)
            return self.mixer.forward(a, ctx, cache, self.position), stream
        if isinstance(n2, SameNorm):             # one norm, read by both branches
            a, stream = n1.forward(x, residual)
            m = self.mixer.forward(a, ctx, cache, self.position)
            return BranchSum((m, ff.forward(a, ctx))), stream
        if isinstance(n1, LayerNorm) and isinstance(n2, LayerNorm) and n1.eps == n2.eps:
            a, b, stream = n1.forward_with(n2, x, residual)
        else:
            a, stream = n1.forward(x, residual)
            zero = torch.zeros_like(a)          # any pair of norms: the second one sees the same stream
            b, _ = n2.forward(zero, stream.clone())
        m = self.mixer.forward(a, ctx, cache, self.position)
        f = ff.forward(b, ctx)
        return BranchSum((m, f)), stream


class BranchNormBlock(Arrangement):
    """``h += norm1(mixer(h)); h += norm2(ffn(h))``: both branches read the stream itself (its copy in
    the compute dtype) and each norm, a ``BranchRMSNorm`` with the residual factor in it, stands behind
    its branch.  The fp32 stream is updated in place; the block hands on a ``StreamCopy``.  A layer
    without a feed-forward (``no_feed_forward``) is the mixer's half alone."""

    def forward(self, x, residual, ctx, cache):
        stream, h = stream_and_copy(x, residual, ctx.dtype)
        h = self.mixer_norm.add_branch(stream, self.mixer.forward(h, ctx, cache, self.position))
        if not isinstance(self.feed_forward, NoFeedForward):
            h = self.feed_forward_norm.add_branch(stream, self.feed_forward.forward(h, ctx))
        return StreamCopy.of(h), stream


class TokenSideInput(StreamPart):
    """What a layer takes from the token itself, behind its branches: with ``e`` the columns ``[index *
    dim, (index + 1) * dim)`` of the token's row of a table shared by all layers, ``g = gelu_tanh(W_gate h)
    * e``, ``y = W_proj g``, and the stream takes ``mult * w * y * rsqrt(mean(y^2) + eps)``, an RMS norm
    with a plain gain (``h``: the stream's copy in the compute dtype; the gate's pre-activations, the
    norm and the sum are fp32).

    params: ``hidden_size``, ``vocab_size``, ``dim``, ``index``, ``table_width``, ``eps``, optional ``mult``.
    tensors: ``table [vocab_size, table_width]``, ``gate [dim, hidden_size]``, ``proj [hidden_size, dim]``,
    ``norm [hidden_size]``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden, self.dim = int(self.param("hidden_size")), int(self.param("dim"))
        self.col0 = int(self.spec.params.get("index", 0)) * self.dim
        self.table_width = int(self.param("table_width"))
        if self.dim <= 0 or self.col0 < 0 or self.col0 + self.dim > self.table_width:
            raise ValueError(f"columns {self.col0}..{self.col0 + self.dim} of a table row of {self.table_width}")

    def param_decls(self):
        return {"table": ParamDecl((int(self.param("vocab_size")), self.table_width)),
                "gate": ParamDecl((self.dim, self.hidden)), "proj": ParamDecl((self.hidden, self.dim)),
                "norm": ParamDecl((self.hidden,), "gain")}

    def bind(self, tensors, dtype, device):
        # this layer's columns only: the layers' copies together are one table
        self.table = _as_compute(tensors["table"], dtype)[:, self.col0:self.col0 + self.dim].contiguous()
        self.gate = Linear(_as_compute(tensors["gate"], dtype).contiguous())
        self.proj = Linear(_as_compute(tensors["proj"], dtype).contiguous())
        self.gain = tensors["norm"].to(torch.float32).contiguous()
        self.eps, self.mult = float(self.param("eps")), float(self.spec.params.get("mult", 1.0))
        self.dtype = dtype

    def forward(self, x, residual, ctx, embedded):
        stream, h = stream_and_copy(x, residual, self.dtype)
        g = ops.token_gate(self.gate(h, out_dtype=torch.float32), self.table, ctx.token_ids, 0)
        h = ops.scaled_norm_add(stream, self.proj(g), self.gain, self.eps, self.mult, self.dtype)
        return StreamCopy.of(h), stream


class NoFeedForward(FeedForward):
    """A layer without a feed-forward."""

    def forward(self, x, ctx):
        raise RuntimeError("this layer has no feed-forward")


register_norm("rmsnorm", RMSNorm, replace=True)
register_norm("layernorm", LayerNorm, replace=True)
register_norm("no_norm", NoNorm, replace=True)
register_norm("branch_rmsnorm", BranchRMSNorm, replace=True)
register_arrangement("branch_norm", BranchNormBlock, replace=True)
register_stream_part("token_side_input", TokenSideInput, replace=True)
register_norm("same_norm", SameNorm, replace=True)
register_position("rotary_interleaved", InterleavedRotary, replace=True)
register_feed_forward("no_feed_forward", NoFeedForward, replace=True)
register_arrangement("parallel", ParallelBlock, replace=True)
register_position("rotary", RotaryPosition, replace=True)
register_mixer("gqa_attention", GroupedQueryAttention, replace=True)
register_feed_forward("swiglu", SwiGLU, replace=True)
register_feed_forward("gated_mlp", SwiGLU, replace=True)
register_feed_forward("clamped_glu_mlp", ClampedGLU, replace=True)
register_embedding("token_embedding", TokenEmbedding, replace=True)
register_head("linear_head", OutputHead, replace=True)
register_arrangement("prenorm", PreNormBlock, replace=True)
