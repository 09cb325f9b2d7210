"""Mixers beyond plain grouped-query attention: a sliding-window attention with unit-norm queries
and keys and gated heads, an attention over chunks of positions with normed queries and keys,
blended values and a gate per head (also with biases, a learned sink per head, or another layer's keys
and values), five recurrent mixers that keep a state of fixed size per request (the real-gated linear
recurrent unit, gated linear attention, retention with a fixed decay per head, the gated delta rule
with a decay per key channel, and a matrix memory with scalar gates and a running maximum), and a
mixer that runs two of them side by side on the same input.

They share one shape (``ProjectedMixer``): everything a mixer projects from its input is one
stacked matrix, everything it hands to its output projection is one row of activations.  A mixer
alone runs ``input product -> mix -> output product``; side by side, the input matrices of both
are stacked into one product and the output matrices into another, and each mixer only fills its
columns.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from .base import KVNeed, LayerCache, Mixer, ParamDecl, PlanNeeds, StateNeed, StepContext, build_part, register_mixer
from .builtin import InterleavedRotary, Linear, RotaryPosition, _as_compute
from .spec import PartSpec


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).contiguous()


class ProjectedMixer(Mixer):
    """A mixer as ``W_out mix(W_in h)``.  Subclasses give ``in_width``/``out_width``, build
    ``self.w_in [in_width, H]`` and ``self.w_out [H, out_width]`` in ``bind``, and implement
    ``mix(proj, out, out_scale, ctx, cache, position)``, which reads the projected row ``proj
    [M, in_width]`` (a column range; it may be overwritten) and writes ``out [M, out_width]``
    (a column range) times ``out_scale``.  A mixer that needs some products of its input unrounded
    (the gates of a recurrence) builds ``self.w_in32 [in32_width, H]`` too; ``mix`` then gets them as
    ``proj32`` (fp32, a column range)."""

    in_width: int
    out_width: int
    w_in: torch.Tensor
    w_out: torch.Tensor
    in32_width: int = 0
    w_in32: torch.Tensor | None = None
    takes_position: bool = True       # side by side with another mixer: whether the layer's position part is for this one

    def mix(self, proj: torch.Tensor, out: torch.Tensor, out_scale: float, ctx: StepContext, cache: LayerCache,
            position) -> None:
        raise NotImplementedError

    def finish_bind(self) -> None:
        self._in, self._out = Linear(self.w_in), Linear(self.w_out)
        self._in32 = Linear(self.w_in32) if self.in32_width else None

    def forward(self, x, ctx, cache, position):
        proj = self._in(x)
        out = torch.empty((ctx.n_tokens, self.out_width), dtype=x.dtype, device=x.device)
        if self._in32 is None:
            self.mix(proj, out, 1.0, ctx, cache, position)
        else:
            self.mix(proj, out, 1.0, ctx, cache, position, proj32=self._in32(x, out_dtype=torch.float32))
        return self._out(out)


# ----------------------------------------------------------------------------- windowed attention


class GatedWindowAttention(ProjectedMixer):
    """Softmax attention over a sliding window (position ``i`` sees ``j`` with ``0 <= i - j <
    window``; no window: all of the past) with ``num_heads`` query heads sharing ``num_kv_heads``
    key/value heads, keys of ``head_dim`` and values of ``value_dim`` per head.  After the position
    encoding (an ``InterleavedRotary``, or none) queries and keys are divided by their root mean
    square over the head (``qk_unit_norm``); the score is ``q . k * scale``; the heads' outputs are
    multiplied by ``sigmoid(W_g h)`` (``gate``) before the output projection.  Scores, weights and
    sums are fp32 for either dtype.

    params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``; optional ``value_dim``
    (default ``head_dim``), ``window``, ``scale`` (default ``head_dim ** -0.5``), ``qk_unit_norm``
    (default False) with ``eps``, ``gate`` (None or ``"sigmoid"`` / ``"silu"``).
    tensors: ``q``, ``k``, ``v``, ``o`` and, with a gate, ``g``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        g = self.spec.params.get
        self.hidden = int(self.param("hidden_size"))
        self.nq, self.nkv = int(self.param("num_heads")), int(self.param("num_kv_heads"))
        self.d = int(self.param("head_dim"))
        self.dv = int(g("value_dim") or self.d)
        self.window = int(g("window")) if g("window") else None
        self.scale = float(g("scale")) if g("scale") is not None else self.d ** -0.5
        self.unit_norm = bool(g("qk_unit_norm", False))
        self.eps = float(g("eps", 0.0))
        self.gate = g("gate")
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads cannot share {self.nkv} key/value heads")
        if not (0 < self.d <= 256 and 0 < self.dv <= 256):
            raise ValueError(f"head sizes {self.d} and {self.dv} must lie in [1, 256]")
        if self.gate not in (None, "sigmoid", "silu"):
            raise ValueError(f"unknown gate {self.gate!r}")
        self.q_off = 0
        self.k_off = self.nq * self.d
        self.v_off = self.k_off + self.nkv * self.d
        self.g_off = self.v_off + self.nkv * self.dv
        self.in_width = self.g_off + (self.nq * self.dv if self.gate else 0)
        self.out_width = self.nq * self.dv

    def param_decls(self):
        H, nq, nkv, d, dv = self.hidden, self.nq, self.nkv, self.d, self.dv
        decls = {"q": ParamDecl((nq * d, H)), "k": ParamDecl((nkv * d, H)), "v": ParamDecl((nkv * dv, H)),
                 "o": ParamDecl((H, nq * dv))}
        if self.gate:
            decls["g"] = ParamDecl((nq * dv, H))
        return decls

    def cache_need(self):
        return KVNeed(self.nkv, self.d, self.window, None if self.dv == self.d else self.dv)

    def plan_needs(self):
        tiles = {ops.ATTENTION_TILE_TOKENS}
        if self._tensor_core_sizes():
            tiles |= set(ops.attention_tile_sizes(self.nq // self.nkv))
        return PlanNeeds(frozenset(tiles))

    def _tensor_core_sizes(self) -> bool:
        """Sizes the tensor-core attention kernels take: keys and values of one size, a multiple of 16."""
        return self.d == self.dv and self.d % 16 == 0 and 16 <= self.d <= 256

    def _attend(self, q, heads, cache, ctx):
        """bfloat16 with sizes the tensor-core kernels take and aligned rows: those kernels (scores and
        softmax in fp32, as everywhere); else the CUDA-core kernel."""
        if (q.dtype == torch.bfloat16 and self._tensor_core_sizes() and self.scale > 0 and heads.is_contiguous()
                and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0):
            ops.attention(q, q.stride(0), heads, cache, ctx, self.nq, self.nkv, self.d, self.scale, self.window or 0)
        else:
            ops.attention_kv(q, heads, cache, ctx, self.nq, self.nkv, self.d, self.dv, self.scale, self.window or 0)

    def bind(self, tensors, dtype, device):
        names = ["q", "k", "v"] + (["g"] if self.gate else [])
        self.w_in = torch.cat([_as_compute(tensors[n], dtype) for n in names], dim=0).contiguous()
        self.w_out = _as_compute(tensors["o"], dtype).contiguous()
        self.finish_bind()

    def mix(self, proj, out, out_scale, ctx, cache, position):
        nq, nkv, d, dv = self.nq, self.nkv, self.d, self.dv
        if position is not None and not isinstance(position, InterleavedRotary):
            raise ValueError("this attention takes an interleaved rotary encoding or none")
        group = ctx.groups[cache.group]
        ops.rope_norm_store(
            proj, self.q_off, self.k_off, self.v_off, nq, nkv, d, dv,
            positions=ctx.positions if position is not None else None,
            inv_freq=position.inv_freq if position is not None else None,
            rot=position.rotary_dim if position is not None else 0,
            unit_norm=self.unit_norm, eps=self.eps,
            slots=group.slots if cache.writes else None,
            kcache=cache.k if cache.writes else None, vcache=cache.v if cache.writes else None)
        q = proj[:, self.q_off:self.q_off + nq * d]
        if self.gate:
            heads = torch.empty((ctx.n_tokens, nq * dv), dtype=proj.dtype, device=proj.device)
            self._attend(q, heads, cache, ctx)
            ops.gate_mul(heads, proj[:, self.g_off:self.g_off + nq * dv], out, self.gate, out_scale)
        elif out_scale == 1.0:
            self._attend(q, out, cache, ctx)
        else:
            raise ValueError("an ungated attention cannot scale its output")



# ----------------------------------------------------------------------------- attention over chunks of positions


def _half_rotation(position, d: int):
    """``(rotated dimensions, float64 frequencies)`` of a mixer whose own kernel rotates in the half layout."""
    if position is None:
        return 0, None
    if not isinstance(position, RotaryPosition):
        raise ValueError("this mixer takes a rotary encoding of the half layout or none")
    if position.rotary_dim > d:
        raise ValueError(f"{position.rotary_dim} rotated dimensions of a head of {d}")
    return position.rotary_dim, position.freq64


class ChunkAttention(ProjectedMixer):
    """Softmax attention with ``num_heads`` query heads sharing ``num_kv_heads`` key/value heads, keys of
    ``head_dim`` and values of ``value_dim`` per head, in which position ``i`` sees ``j <= i`` of its own
    chunk of positions only (``i // chunk == j // chunk``, chunks counted from position 0; no ``chunk``:
    all of the past).  Queries and keys get an RMS norm over the head with a gain shared by the heads
    (``qk_norm``), then the position encoding (a ``RotaryPosition``, half layout, or none); the score is
    ``q . k * scale``.  With ``value_blend`` the values of every such layer of a model but the first to
    run become ``(1 - lam) v + lam v_first`` (``lam`` the layer's ``vmix``, ``v_first`` the first such
    layer's values of the same token); the blended values are what is cached; ``value_blend: "source"`` marks a layer that
    only gives its values away and has no ``vmix``.  With ``head_gate`` head
    ``h``'s output is multiplied by ``sigmoid(W_g x)_h``, one number per head.  With ``bias`` q, k and v
    have biases (added in fp32 before the norm).  With ``sink`` ``"learned"`` the softmax's denominator of head
    ``h`` also holds ``exp(sink_h)``: a logit of the head's own that enters the normaliser alone (no score scale).  With
    ``own_kv`` False the layer has no keys and values of its own (no ``k``, ``v``, ``k.norm``, no biases of
    theirs): it reads the cache layer that another layer with the same head counts wrote, with its own
    queries.  Scores, weights and sums are fp32 for either dtype.

    params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale``; optional ``value_dim``
    (default ``head_dim``), ``chunk``, ``qk_norm`` (default False) with ``eps``, ``value_blend``,
    ``head_gate``, ``bias`` (default False), ``sink`` (None or ``"learned"``) and ``own_kv`` (default True).
    tensors: ``q``, ``k``, ``v``, ``o`` and, as asked, ``q.norm``, ``k.norm``, ``vmix``, ``g``, ``q.b``, ``k.b``,
    ``v.b``, ``sink``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        g = self.spec.params.get
        self.hidden = int(self.param("hidden_size"))
        self.nq, self.nkv = int(self.param("num_heads")), int(self.param("num_kv_heads"))
        self.d = int(self.param("head_dim"))
        self.dv = int(g("value_dim") or self.d)
        self.scale = float(self.param("scale"))
        self.chunk = int(g("chunk")) if g("chunk") else None
        self.qk_norm = bool(g("qk_norm", False))
        self.eps = float(g("eps", 0.0))
        blend = g("value_blend", False)
        if blend not in (False, True, "source"):
            raise ValueError(f"value_blend is true, false or 'source', not {blend!r}")
        self.value_blend = blend is True            # takes ``vmix`` and blends (unless it is the first to run)
        self.value_source = bool(blend)             # may leave its values for the layers behind it
        self.head_gate = bool(g("head_gate", False))
        self.bias = bool(g("bias", False))
        self.sink = g("sink")
        self.own_kv = bool(g("own_kv", True))
        if self.sink not in (None, "learned"):
            raise ValueError(f"unknown sink {self.sink!r}: 'learned' or none")
        if not self.own_kv and (self.value_source or self.chunk):
            raise ValueError("a layer without keys and values of its own neither blends values nor has chunks")
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads cannot share {self.nkv} key/value heads")
        if not (0 < self.d <= 1024 and 0 < self.dv <= 512):
            raise ValueError(f"head sizes {self.d} (keys, up to 1024) and {self.dv} (values, up to 512)")
        own = self.nkv if self.own_kv else 0           # key/value heads that this layer projects
        self.q_off, self.k_off = 0, self.nq * self.d
        self.v_off = self.k_off + own * self.d
        self.g_off = self.v_off + own * self.dv
        self.in_width = self.g_off + (self.nq if self.head_gate else 0)
        self.out_width = self.nq * self.dv

    def param_decls(self):
        H, nq, nkv, d, dv = self.hidden, self.nq, self.nkv, self.d, self.dv
        decls = {"q": ParamDecl((nq * d, H)), "o": ParamDecl((H, nq * dv))}
        if self.own_kv:
            decls["k"], decls["v"] = ParamDecl((nkv * d, H)), ParamDecl((nkv * dv, H))
        if self.qk_norm:
            decls["q.norm"] = ParamDecl((d,), "gain")
            if self.own_kv:
                decls["k.norm"] = ParamDecl((d,), "gain")
        if self.bias:
            decls["q.b"] = ParamDecl((nq * d,), "table")
            if self.own_kv:
                decls["k.b"], decls["v.b"] = ParamDecl((nkv * d,), "table"), ParamDecl((nkv * dv,), "table")
        if self.sink:
            decls["sink"] = ParamDecl((nq,), "table")
        if self.value_blend:
            decls["vmix"] = ParamDecl((), "table")
        if self.head_gate:
            decls["g"] = ParamDecl((nq, H))
        return decls

    def cache_need(self):
        return KVNeed(self.nkv, self.d, None, None if self.dv == self.d else self.dv, self.chunk)

    def plan_needs(self):
        tiles = {ops.ATTENTION_TILE_TOKENS} | ops.rows_attention_tile_sizes(self.nq, self.nkv, self.d, self.dv, False)
        if self._tensor_core_sizes():
            tiles |= set(ops.attention_tile_sizes(self.nq // self.nkv))
        return PlanNeeds(frozenset(tiles))

    def _tensor_core_sizes(self) -> bool:
        """Sizes the tensor-core attention kernels take: keys and values of one size, a multiple of 16."""
        return self.d == self.dv and self.d % 16 == 0 and 16 <= self.d <= 256

    def _attend(self, q, heads, cache, ctx):
        """bfloat16 with sizes the tensor-core kernels take and aligned rows: those kernels (the balanced
        decode kernel, tcgen05 or mma.sync for prompt portions; scores and softmax in fp32, as everywhere);
        else the kernel for keys and values of two sizes or the CUDA-core kernel."""
        tensor_cores = (q.dtype == torch.bfloat16 and self._tensor_core_sizes() and self.scale > 0
                        and heads.is_contiguous() and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)
        if tensor_cores and self.sinks is None:
            ops.attention(q, q.stride(0), heads, cache, ctx, self.nq, self.nkv, self.d, self.scale,
                          chunk=self.chunk or 0)
        elif tensor_cores and ctx.decode_only and not self.chunk:
            # single tokens with sinks: the balanced decode kernel, the sink joining the last merge
            group = ctx.groups[cache.group]
            ops.attention_decode_balanced(q, q.stride(0), heads, cache.k, cache.v, group.block_table, group.page_size,
                                          ctx.q_start, ctx.kv_len, ctx.n_requests, self.nq, self.nkv, self.d, self.scale,
                                          0, table_rows=group.table_rows, sinks=self.sinks)
        else:
            ops.attention_ext(q, heads, cache, ctx, self.nq, self.nkv, self.d, self.dv, self.scale,
                              chunk=self.chunk or 0, sinks=self.sinks)

    def bind(self, tensors, dtype, device):
        names = ["q"] + (["k", "v"] if self.own_kv else []) + (["g"] if self.head_gate else [])
        self.w_in = torch.cat([_as_compute(tensors[n], dtype) for n in names], dim=0).contiguous()
        self.w_out = _as_compute(tensors["o"], dtype).contiguous()
        self.q_gain = _f32(tensors["q.norm"]) if self.qk_norm else None
        self.k_gain = _f32(tensors["k.norm"]) if self.qk_norm and self.own_kv else None
        self.sinks = _f32(tensors["sink"]) if self.sink else None
        self.in_bias = None
        if self.bias:        # one number per packed column of q, k and v
            self.in_bias = torch.cat([_f32(tensors[n + ".b"]) for n in (["q", "k", "v"] if self.own_kv else ["q"])])
        self.blend = _f32(tensors["vmix"]).reshape(1) if self.value_blend else None
        self.finish_bind()

    def mix(self, proj, out, out_scale, ctx, cache, position):
        nq, nkv, d, dv = self.nq, self.nkv, self.d, self.dv
        rot, freq = _half_rotation(position, d)
        v_other = None
        if self.value_source:
            # the first blending layer to run in a step leaves its values for the others
            values = proj[:, self.v_off:self.v_off + nkv * dv]
            first = ctx.scratch.get("value_blend_source")
            if first is None:
                ctx.scratch["value_blend_source"] = values
            elif not self.value_blend:
                raise ValueError("a layer that only gives its values away runs before the blending ones")
            elif first.shape != values.shape:
                raise ValueError(f"blended values of {tuple(values.shape)} and a first layer's of {tuple(first.shape)}")
            else:
                v_other = first
        group = ctx.groups[cache.group]
        if self.own_kv != bool(cache.writes):
            raise ValueError("a layer with keys and values of its own writes its cache layer; one without reads another's")
        own = nkv if self.own_kv else 0
        ops.qk_norm_rope_store(proj, self.q_off, self.k_off, self.v_off if own else None, nq, own, d, dv,
                               q_gain=self.q_gain, k_gain=self.k_gain, eps=self.eps, rot=rot, positions=ctx.positions,
                               freq=freq, v_other=v_other, blend=self.blend if v_other is not None else None,
                               slots=group.slots if cache.writes else None,
                               kcache=cache.k if cache.writes else None, vcache=cache.v if cache.writes else None,
                               bias=self.in_bias)
        q = proj[:, self.q_off:self.q_off + nq * d]
        if not self.head_gate and out_scale == 1.0:
            self._attend(q, out, cache, ctx)
            return
        heads = torch.empty((ctx.n_tokens, nq * dv), dtype=proj.dtype, device=proj.device)
        self._attend(q, heads, cache, ctx)
        if self.head_gate:
            ops.gate_mul(heads, proj[:, self.g_off:self.g_off + nq], out, "sigmoid", out_scale, per=dv)
        else:
            ops.gate_mul(heads, None, out, None, out_scale)

# ----------------------------------------------------------------------------- gated linear attention


class GatedLinearAttention(ProjectedMixer):
    """Per head a matrix state ``S [key_dim, value_dim]`` in fp32, carried from token to token:
    ``S_t = diag(alpha_t) S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` with ``q = W_q h * key_dim^-0.5``
    and a decay per key channel ``alpha = sigmoid(W_a2 (W_a1 h) + b)^(1 / tau)``.  Each head's ``o``
    gets an RMS norm over ``value_dim`` with one gain shared by the heads; the heads are multiplied by
    ``silu(W_g h)`` and projected.

    params: ``hidden_size``, ``num_heads``, ``key_dim``, ``value_dim``, ``tau``, ``eps``, ``decay_rank``
    (None: the rank is the one the checkpoint's ``a1`` has).
    tensors: ``q``, ``k``, ``v``, ``g``, ``o``, ``norm``, ``a1``, ``a2``, ``a2.b``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.heads = int(self.param("num_heads"))
        self.dk, self.dv = int(self.param("key_dim")), int(self.param("value_dim"))
        self.tau = float(self.param("tau"))
        rank = self.spec.params.get("decay_rank")
        self.rank = int(rank) if rank else None
        self.eps = float(self.param("eps"))
        if not 0 < self.dk <= 256:
            raise ValueError(f"key size {self.dk} must lie in [1, 256]")
        hk, hv = self.heads * self.dk, self.heads * self.dv
        self.q_off, self.k_off, self.v_off = 0, hk, 2 * hk
        self.g_off = 2 * hk + hv
        self.a_off = self.g_off + hv
        self.out_width = hv

    @property
    def in_width(self) -> int:
        return self.a_off + self.rank

    def param_decls(self):
        H, hk, hv = self.hidden, self.heads * self.dk, self.heads * self.dv
        return {"q": ParamDecl((hk, H)), "k": ParamDecl((hk, H)), "v": ParamDecl((hv, H)), "g": ParamDecl((hv, H)),
                "o": ParamDecl((H, hv)), "norm": ParamDecl((self.dv,), "gain"),
                "a1": ParamDecl((self.rank, H)), "a2": ParamDecl((hk, self.rank)), "a2.b": ParamDecl((hk,), "table")}

    def state_need(self):
        return StateNeed((self.heads, self.dk, self.dv), torch.float32)

    def bind(self, tensors, dtype, device):
        self.rank = int(tensors["a1"].shape[0])
        self.w_in = torch.cat([_as_compute(tensors[n], dtype) for n in ("q", "k", "v", "g", "a1")], dim=0).contiguous()
        self.w_out = _as_compute(tensors["o"], dtype).contiguous()
        self.a2 = Linear(_as_compute(tensors["a2"], dtype).contiguous())
        self.a2_bias = _f32(tensors["a2.b"])
        self.norm_gain = _f32(tensors["norm"])
        self.finish_bind()

    def mix(self, proj, out, out_scale, ctx, cache, position):
        hk, hv = self.heads * self.dk, self.heads * self.dv
        low = proj[:, self.a_off:self.a_off + self.rank]
        z = self.a2(low if low.data_ptr() % 16 == 0 else low.contiguous(), out_dtype=torch.float32)
        o = ops.gla_scan(proj[:, self.q_off:self.q_off + hk], proj[:, self.k_off:self.k_off + hk],
                         proj[:, self.v_off:self.v_off + hv], z, self.a2_bias, self.tau, self.dk ** -0.5,
                         self.heads, self.dk, self.dv, cache.state, ctx)
        ops.headnorm_gate(o, self.norm_gain, proj[:, self.g_off:self.g_off + hv], out, self.heads, self.dv,
                          self.eps, "silu", out_scale)



# ----------------------------------------------------------------------------- retention


class Retention(ProjectedMixer):
    """Linear attention with one fixed decay per head and neither softmax nor denominator: per head a
    matrix state ``S [key_dim, value_dim]`` in fp32, ``S_t = decay_h S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t``.
    Queries and keys are rotated by the position (a ``RotaryPosition``, half layout, or none) and the
    keys multiplied by ``key_dim^-1/2`` afterwards.  Each head's ``o`` is divided by its root mean square
    over ``value_dim``; the heads are multiplied by ``silu(W_g h)`` and projected.

    params: ``hidden_size``, ``num_heads``, ``key_dim``, ``value_dim``, ``decay`` (one number per head), ``eps``.
    tensors: ``q``, ``k``, ``v``, ``g``, ``o``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.heads = int(self.param("num_heads"))
        self.dk, self.dv = int(self.param("key_dim")), int(self.param("value_dim"))
        self.decay = [float(a) for a in self.param("decay")]
        self.eps = float(self.param("eps"))
        if len(self.decay) != self.heads:
            raise ValueError(f"{len(self.decay)} decays for {self.heads} heads")
        if not 0 < self.dk <= 256:
            raise ValueError(f"key size {self.dk} must lie in [1, 256]")
        hk, hv = self.heads * self.dk, self.heads * self.dv
        self.q_off, self.k_off, self.v_off, self.g_off = 0, hk, 2 * hk, 2 * hk + hv
        self.in_width = 2 * hk + 2 * hv
        self.out_width = hv

    def param_decls(self):
        H, hk, hv = self.hidden, self.heads * self.dk, self.heads * self.dv
        return {"q": ParamDecl((hk, H)), "k": ParamDecl((hk, H)), "v": ParamDecl((hv, H)), "g": ParamDecl((hv, H)),
                "o": ParamDecl((H, hv))}

    def state_need(self):
        return StateNeed((self.heads, self.dk, self.dv), torch.float32)

    def bind(self, tensors, dtype, device):
        self.w_in = torch.cat([_as_compute(tensors[n], dtype) for n in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_out = _as_compute(tensors["o"], dtype).contiguous()
        self.head_decay = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(device)
        self.unit_gain = torch.ones(self.dv, dtype=torch.float32, device=device)
        self.finish_bind()

    def mix(self, proj, out, out_scale, ctx, cache, position):
        hk, hv = self.heads * self.dk, self.heads * self.dv
        rot, freq = _half_rotation(position, self.dk)
        q, k = proj[:, self.q_off:self.q_off + hk], proj[:, self.k_off:self.k_off + hk]
        if rot:
            # what enters the recurrence stays in fp32: the rotated q and k are not rounded to bfloat16 again
            qk = torch.empty((ctx.n_tokens, 2 * hk), dtype=torch.float32, device=proj.device) \
                if proj.dtype != torch.float32 else None
            ops.qk_norm_rope_store(proj, self.q_off, self.k_off, None, self.heads, self.heads, self.dk, self.dv,
                                   rot=rot, positions=ctx.positions, freq=freq, qk_out=qk)
            if qk is not None:
                q, k = qk[:, :hk], qk[:, hk:]
        # the keys' factor rides on the queries: o is linear in both
        o = ops.gla_scan(q, k, proj[:, self.v_off:self.v_off + hv], None, None, 1.0, self.dk ** -0.5, self.heads,
                         self.dk, self.dv, cache.state, ctx, head_decay=self.head_decay)
        ops.headnorm_gate(o, self.unit_gain, proj[:, self.g_off:self.g_off + hv], out, self.heads, self.dv, self.eps,
                          "silu", out_scale)


# ----------------------------------------------------------------------------- gated delta rule


class ChannelDeltaRule(ProjectedMixer):
    """The gated delta rule with a decay per head and key channel.  ``q = W_q h`` and ``k = W_k h``
    (``num_kv_heads`` heads of ``key_dim``; head ``h`` uses q/k head ``h // (num_heads / num_kv_heads)``)
    and ``v = W_v h`` (``num_heads`` heads of ``value_dim``) each pass a causal convolution per channel over
    ``conv_taps`` tokens (the last tap meets the current token; zeros before the start) and SiLU; q and k
    become unit vectors per head (``x / sqrt(sum x^2 + unit_eps)``), q also times ``key_dim^-1/2``.  With
    ``beta = sigmoid(W_b h)`` per head and ``g = exp(-exp(A_log) * softplus(W_a2 (W_a1 h) + dt_bias))`` per
    head and key channel, per head on its fp32 state ``S [key_dim, value_dim]``:
    ``S <- diag(g) S``, ``u = beta (v - S^T k)``, ``S <- S + k u^T``, ``o = S^T q``.  Each head's ``o`` gets an RMS
    norm over ``value_dim`` with one gain shared by the heads, times ``sigmoid(W_g2 (W_g1 h))``; then ``W_o``.
    The state (fp32, per request) is the convolution's last ``conv_taps - 1`` inputs, then ``S``.

    params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``key_dim``, ``value_dim``, ``conv_taps``, ``eps``;
    optional ``unit_eps`` (default 1e-6), ``decay_rank`` and ``gate_rank`` (None: what the checkpoint has).
    tensors: ``q``, ``q.conv``, ``k``, ``k.conv``, ``v``, ``v.conv``, ``b``, ``A_log``, ``norm``, ``a1``, ``a2``,
    ``dt_bias``, ``g1``, ``g2``, ``o``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        g = self.spec.params.get
        self.hidden = int(self.param("hidden_size"))
        self.heads, self.kv_heads = int(self.param("num_heads")), int(self.param("num_kv_heads"))
        self.dk, self.dv = int(self.param("key_dim")), int(self.param("value_dim"))
        self.taps = int(self.param("conv_taps"))
        self.eps = float(self.param("eps"))
        self.unit_eps = float(g("unit_eps", 1e-6))
        self.rank_a = int(g("decay_rank")) if g("decay_rank") else None
        self.rank_g = int(g("gate_rank")) if g("gate_rank") else None
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} heads cannot share {self.kv_heads} query/key heads")
        if not 0 < self.dk <= 256:
            raise ValueError(f"key size {self.dk} must lie in [1, 256]")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"{self.taps} convolution taps (1 to 16 are taken)")
        gk, hv = self.kv_heads * self.dk, self.heads * self.dv
        self.q_off, self.k_off, self.v_off = 0, gk, 2 * gk
        self.conv_width = 2 * gk + hv                  # the channels that pass the convolution: q, k, v
        self.b_off = self.conv_width
        self.a_off = self.b_off + self.heads
        self.out_width = hv
        self.state_offset = (self.taps - 1) * self.conv_width

    @property
    def in_width(self) -> int:
        return self.a_off + self.rank_a + self.rank_g

    def param_decls(self):
        H, gk, hv, hk = self.hidden, self.kv_heads * self.dk, self.heads * self.dv, self.heads * self.dk
        return {"q": ParamDecl((gk, H)), "q.conv": ParamDecl((gk, self.taps), "table"),
                "k": ParamDecl((gk, H)), "k.conv": ParamDecl((gk, self.taps), "table"),
                "v": ParamDecl((hv, H)), "v.conv": ParamDecl((hv, self.taps), "table"),
                "b": ParamDecl((self.heads, H)), "A_log": ParamDecl((self.heads,), "table"),
                "norm": ParamDecl((self.dv,), "gain"),
                "a1": ParamDecl((self.rank_a, H)), "a2": ParamDecl((hk, self.rank_a)),
                "dt_bias": ParamDecl((hk,), "table"),
                "g1": ParamDecl((self.rank_g, H)), "g2": ParamDecl((hv, self.rank_g)),
                "o": ParamDecl((H, hv))}

    def state_need(self):
        return StateNeed((self.state_offset + self.heads * self.dk * self.dv,), torch.float32)

    def bind(self, tensors, dtype, device):
        self.rank_a, self.rank_g = int(tensors["a1"].shape[0]), int(tensors["g1"].shape[0])
        self.w_in = torch.cat([_as_compute(tensors[n], dtype) for n in ("q", "k", "v", "b", "a1", "g1")],
                              dim=0).contiguous()
        self.w_out = _as_compute(tensors["o"], dtype).contiguous()
        self.conv_w = torch.cat([_f32(tensors[n]) for n in ("q.conv", "k.conv", "v.conv")], dim=0).contiguous()
        self.a2 = Linear(_as_compute(tensors["a2"], dtype).contiguous())
        self.g2 = Linear(_as_compute(tensors["g2"], dtype).contiguous())
        self.dt_bias, self.a_log = _f32(tensors["dt_bias"]), _f32(tensors["A_log"])
        self.norm_gain = _f32(tensors["norm"])
        self.finish_bind()

    @staticmethod
    def _aligned(t: torch.Tensor) -> torch.Tensor:
        return t if (t.data_ptr() % 16 == 0 and t.stride(0) % 8 == 0) else t.contiguous()

    def mix(self, proj, out, out_scale, ctx, cache, position):
        if position is not None:
            raise ValueError("this mixer takes no position part: the order of the tokens is in its state")
        gk, hv, C = self.kv_heads * self.dk, self.heads * self.dv, self.conv_width
        x = proj[:, :C]
        u = torch.empty((ctx.n_tokens, C), dtype=proj.dtype, device=proj.device)
        ops.causal_conv(x, None, self.conv_w, None, cache.state, ctx, u, act="silu")
        z = self.a2(self._aligned(proj[:, self.a_off:self.a_off + self.rank_a]), out_dtype=torch.float32)
        gate = self.g2(self._aligned(proj[:, self.a_off + self.rank_a:self.a_off + self.rank_a + self.rank_g]))
        o = ops.delta_scan(u[:, self.q_off:self.q_off + gk], u[:, self.k_off:self.k_off + gk],
                           u[:, self.v_off:self.v_off + hv], z, self.dt_bias, self.a_log,
                           proj[:, self.b_off:self.b_off + self.heads], self.dk ** -0.5, self.unit_eps, self.heads,
                           self.kv_heads, self.dk, self.dv, cache.state, self.state_offset, ctx, conv_in=x,
                           taps=self.taps)
        ops.headnorm_gate(o, self.norm_gain, gate, out, self.heads, self.dv, self.eps, "sigmoid", out_scale)

# ----------------------------------------------------------------------------- matrix memory with scalar gates


class MatrixMemory(ProjectedMixer):
    """A matrix memory with an input and a forget gate per head and a running maximum that keeps their
    exponentials in range.  ``q = W_q h * key_dim^-1/2``, ``k = W_k h``, ``v = W_v h``; per head the log gates
    ``i = cap tanh((W_i h + b_i) / cap)`` and ``f = logsigmoid(cap tanh((W_f h + b_f) / cap))``.  From ``S = 0``,
    ``n = 0``, ``m = 0``:  ``m' = max(f + m, i)``,  ``S' = exp(f + m - m') S + exp(i - m') k v^T``,  ``n'`` likewise
    with ``k`` alone,  ``o = S'^T q / (max(|n' . q|, exp(-m')) + den_eps)``.  Each head's ``o`` is divided by its
    root mean square over ``value_dim``; the heads are multiplied by a gain (one number per head and
    channel) and by ``sigmoid(W_g h)``, and projected.  The state (fp32, per request) is ``[S | n]`` as
    ``[heads, key_dim, value_dim + 1]``, then ``m [heads]``; gates, exponentials and the state are fp32 and
    the gates' pre-activations come from a product of their own with an fp32 result.

    params: ``hidden_size``, ``num_heads``, ``key_dim``, ``value_dim``, ``gate_cap``, ``eps``, optional
    ``den_eps`` (default 1e-6).
    tensors: ``q``, ``k``, ``v``, ``g``, ``o``, ``norm``, ``i``, ``i.b``, ``f``, ``f.b``.
    """

    takes_position = False

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.heads = int(self.param("num_heads"))
        self.dk, self.dv = int(self.param("key_dim")), int(self.param("value_dim"))
        self.cap = float(self.param("gate_cap"))
        self.eps = float(self.param("eps"))
        self.den_eps = float(self.spec.params.get("den_eps", 1e-6))
        if not 0 < self.dk <= 256:
            raise ValueError(f"key size {self.dk} must lie in [1, 256]")
        if not self.cap > 0:
            raise ValueError(f"the gates' cap must be positive, got {self.cap}")
        hk, hv = self.heads * self.dk, self.heads * self.dv
        self.q_off, self.k_off, self.v_off, self.g_off = 0, hk, 2 * hk, 2 * hk + hv
        self.in_width = 2 * hk + 2 * hv
        self.in32_width = 2 * self.heads
        self.out_width = hv
        self.m_offset = self.heads * self.dk * (self.dv + 1)

    def param_decls(self):
        H, hk, hv, n = self.hidden, self.heads * self.dk, self.heads * self.dv, self.heads
        return {"q": ParamDecl((hk, H)), "k": ParamDecl((hk, H)), "v": ParamDecl((hv, H)), "g": ParamDecl((hv, H)),
                "o": ParamDecl((H, hv)), "norm": ParamDecl((hv,), "gain"),
                "i": ParamDecl((n, H)), "i.b": ParamDecl((n,), "table"),
                "f": ParamDecl((n, H)), "f.b": ParamDecl((n,), "table")}

    def state_need(self):
        return StateNeed((self.m_offset + self.heads,), torch.float32)

    def bind(self, tensors, dtype, device):
        self.w_in = torch.cat([_as_compute(tensors[n], dtype) for n in ("q", "k", "v", "g")], dim=0).contiguous()
        self.w_in32 = torch.cat([_as_compute(tensors["i"], dtype), _as_compute(tensors["f"], dtype)], dim=0).contiguous()
        self.w_out = _as_compute(tensors["o"], dtype).contiguous()
        self.bias_i, self.bias_f = _f32(tensors["i.b"]), _f32(tensors["f.b"])
        self.norm_gain = _f32(tensors["norm"])
        self.finish_bind()

    def mix(self, proj, out, out_scale, ctx, cache, position, proj32=None):
        if position is not None:
            raise ValueError("this mixer takes no position part: the order of the tokens is in its state")
        hk, hv = self.heads * self.dk, self.heads * self.dv
        gates = ops.mlstm_gates(proj32, self.bias_i, self.bias_f, self.cap, self.heads, cache.state, self.m_offset, ctx)
        o = ops.gla_scan(proj[:, self.q_off:self.q_off + hk], proj[:, self.k_off:self.k_off + hk],
                         proj[:, self.v_off:self.v_off + hv], None, None, 1.0, self.dk ** -0.5, self.heads, self.dk,
                         self.dv, cache.state, ctx, tok_gates=gates, extra_col=True)
        ops.headnorm_gate(o, self.norm_gain, proj[:, self.g_off:self.g_off + hv], out, self.heads, self.dv, self.eps,
                          "sigmoid", out_scale, tok_gates=gates, den_eps=self.den_eps)


# ----------------------------------------------------------------------------- real-gated linear recurrent unit


class RealGatedLinearRecurrence(ProjectedMixer):
    """Two branches of ``width`` channels: ``y = gelu_tanh(W_y h + b_y)`` and ``u = conv(W_x h + b_x)``,
    a causal convolution per channel over ``conv_taps`` tokens (the last tap meets the current
    token).  ``u`` is cut into ``blocks`` parts; in each, ``r = sigmoid(A_r u + b_r)`` and ``i =
    sigmoid(A_i u + b_i)`` with square matrices.  Then ``a = exp(-decay_scale * r * softplus(lam))``
    and ``S_t = a S_(t-1) + sqrt(1 - a^2) * i * u`` from ``S = 0``; the output is ``W_o (S * y)``.
    The state (fp32, per request) is ``S`` and the convolution's last ``conv_taps - 1`` inputs.

    params: ``hidden_size``, ``width``, ``blocks``, ``conv_taps``, optional ``decay_scale`` (default 8).
    tensors: ``y``, ``y.b``, ``x``, ``x.b``, ``conv``, ``conv.b``, ``ra``, ``ra.b``, ``ri``, ``ri.b``, ``lam``, ``o``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.width = int(self.param("width"))
        self.blocks = int(self.param("blocks"))
        self.taps = int(self.param("conv_taps"))
        self.decay_scale = float(self.spec.params.get("decay_scale", 8.0))
        if self.blocks <= 0 or self.width % self.blocks:
            raise ValueError(f"{self.width} channels cannot be cut into {self.blocks} equal parts")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"{self.taps} convolution taps (1 to 16 are taken)")
        self.in_width = 2 * self.width
        self.out_width = self.width

    def param_decls(self):
        H, C, B = self.hidden, self.width, self.blocks
        bw = C // B
        return {"y": ParamDecl((C, H)), "y.b": ParamDecl((C,), "table"), "x": ParamDecl((C, H)),
                "x.b": ParamDecl((C,), "table"), "conv": ParamDecl((C, self.taps), "table"),
                "conv.b": ParamDecl((C,), "table"), "ra": ParamDecl((B, bw, bw)), "ra.b": ParamDecl((B, bw), "table"),
                "ri": ParamDecl((B, bw, bw)), "ri.b": ParamDecl((B, bw), "table"), "lam": ParamDecl((C,), "table"),
                "o": ParamDecl((H, C))}

    def state_need(self):
        return StateNeed((self.taps, self.width), torch.float32)

    def bind(self, tensors, dtype, device):
        self.w_in = torch.cat([_as_compute(tensors["y"], dtype), _as_compute(tensors["x"], dtype)], dim=0).contiguous()
        self.w_out = _as_compute(tensors["o"], dtype).contiguous()
        self.y_bias, self.x_bias = _f32(tensors["y.b"]), _f32(tensors["x.b"])
        self.conv_w, self.conv_b = _f32(tensors["conv"]), _f32(tensors["conv.b"])
        self.gates_w = torch.cat([_as_compute(tensors["ra"], dtype), _as_compute(tensors["ri"], dtype)],
                                 dim=1).contiguous()                       # [blocks, 2 bw, bw]
        self.gate_bias_r, self.gate_bias_i = _f32(tensors["ra.b"]).reshape(-1), _f32(tensors["ri.b"]).reshape(-1)
        self.lam = _f32(tensors["lam"])
        self.finish_bind()

    def mix(self, proj, out, out_scale, ctx, cache, position):
        if out_scale != 1.0:
            raise ValueError("this mixer cannot scale its output")
        C = self.width
        y, x = proj[:, :C], proj[:, C:2 * C]
        u = torch.empty((ctx.n_tokens, C), dtype=proj.dtype, device=proj.device)
        ops.causal_conv(x, self.x_bias, self.conv_w, self.conv_b, cache.state, ctx, u)
        gates = ops.block_diagonal_gates(u, self.gates_w)
        ops.rglru_scan(gates, self.gate_bias_r, self.gate_bias_i, self.lam, self.decay_scale, u, y, self.y_bias,
                       x, self.x_bias, self.taps, cache.state, ctx, out)


# ----------------------------------------------------------------------------- two mixers side by side


class SideBySide(Mixer):
    """Two mixers that read the same input: ``left_scale * left(h) + right_scale * right(h)``.  Both
    are ``ProjectedMixer``s, so their input matrices are stacked into one product and their output
    matrices, side by side, into another; the scales ride on what each writes for that product.  At
    most one of them keeps keys and values and at most one a state (a layer's cache holds one of each).

    params: ``left``, ``right`` (each a ``PartSpec`` of a registered mixer, its ``prefix`` relative to
    this part's), ``left_scale``, ``right_scale``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        self.children: list[ProjectedMixer] = []
        self.scales: list[float] = []
        for side in ("left", "right"):
            child: PartSpec = self.param(side)
            part = build_part("mixer", PartSpec(child.kind, child.params, prefix=child.prefix, rename=child.rename))
            if not isinstance(part, ProjectedMixer):
                raise ValueError(f"mixer {child.kind!r} cannot run side by side with another")
            self.children.append(part)
            self.scales.append(float(self.spec.params.get(side + "_scale", 1.0)))
        if sum(c.cache_need() is not None for c in self.children) > 1 or \
                sum(c.state_need() is not None for c in self.children) > 1:
            raise ValueError("side by side, at most one mixer may keep keys and values and one a state")

    def param_decls(self):
        return {c.spec.prefix + local: decl for c in self.children for local, decl in c.param_decls().items()}

    def cache_need(self):
        return next((n for n in (c.cache_need() for c in self.children) if n is not None), None)

    def state_need(self):
        return next((n for n in (c.state_need() for c in self.children) if n is not None), None)

    def plan_needs(self):
        return PlanNeeds(frozenset().union(*(c.plan_needs().q_tile_tokens for c in self.children)))

    def bind(self, tensors, dtype, device):
        for c in self.children:
            c.bind({local: tensors[c.spec.prefix + local] for local in c.param_decls()}, dtype, device)
        self._in = Linear(torch.cat([c.w_in for c in self.children], dim=0).contiguous())
        self._out = Linear(torch.cat([c.w_out for c in self.children], dim=1).contiguous())
        rows32 = [c.w_in32 for c in self.children if c.in32_width]
        self._in32 = Linear(torch.cat(rows32, dim=0).contiguous()) if rows32 else None
        for c in self.children:      # the stacked copies are the ones that run
            c.w_in = c.w_out = c._in = c._out = c.w_in32 = c._in32 = None

    def forward(self, x, ctx, cache, position):
        proj = self._in(x)
        proj32 = self._in32(x, out_dtype=torch.float32) if self._in32 is not None else None
        out = torch.empty((ctx.n_tokens, sum(c.out_width for c in self.children)), dtype=x.dtype, device=x.device)
        i0 = o0 = p0 = 0
        for c, scale in zip(self.children, self.scales):
            kw = {}
            if c.in32_width:
                kw["proj32"] = proj32[:, p0:p0 + c.in32_width]
                p0 += c.in32_width
            c.mix(proj[:, i0:i0 + c.in_width], out[:, o0:o0 + c.out_width], scale, ctx, cache,
                  position if c.takes_position else None, **kw)
            i0 += c.in_width
            o0 += c.out_width
        return self._out(out)


register_mixer("gated_window_attention", GatedWindowAttention, replace=True)
register_mixer("gated_linear_attention", GatedLinearAttention, replace=True)
register_mixer("rglru", RealGatedLinearRecurrence, replace=True)
register_mixer("chunk_attention", ChunkAttention, replace=True)
register_mixer("retention", Retention, replace=True)
register_mixer("channel_delta_rule", ChannelDeltaRule, replace=True)
register_mixer("matrix_memory", MatrixMemory, replace=True)
register_mixer("normed_attention", ChunkAttention, replace=True)
register_mixer("side_by_side", SideBySide, replace=True)
