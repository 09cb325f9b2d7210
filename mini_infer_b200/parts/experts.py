"""Routed experts: a feed-forward of which every token uses a few experts out of many, chosen by a
router, and optionally one shared expert that every token uses.
"""

from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, ParamDecl, register_feed_forward
from .builtin import Linear, _as_compute


class RoutedExperts(FeedForward):
    """Router logits ``z = W_r h`` in fp32; a token's ``top`` experts are those with the largest
    logits and their weights the softmax over those logits alone (``scores`` ``"chosen"``, the
    default), or their scores under the softmax over all experts, divided by the sum of these
    (+ 1e-20) and multiplied by ``route_scale`` (``scores`` ``"all"``), or (``scores`` ``"sigmoid"``) the
    scores are ``s = sigmoid(z)``, the choice goes by ``s + correction`` (``correction``: a tensor, one number
    per expert) and the weights are the chosen ``s`` times ``route_scale`` (no division by their sum).  With
    ``groups`` > 1 the experts form that many equal groups of neighbours, a group counts as its best
    expert (``group_score`` ``"best"``, the default) or as the sum of its two best choice scores
    (``"top2"``), and only experts of the ``keep_groups`` best groups can be chosen.  The output is the
    weighted sum of the chosen experts' outputs, plus the shared expert's where there is one, which
    ``shared_gate`` ``"sigmoid"`` multiplies by ``sigmoid(w_sg . h)``, one number per token.  An expert is
    ``W_down (g' * sigmoid(alpha g') * (u' + 1))`` with ``g' = min(W_gate h, limit)`` and
    ``u' = clamp(W_up h, -limit, limit)`` (``activation`` ``"clamped"``, the default), or
    ``W_down (silu(W_gate h) * W_up h)`` (``"silu"``), no biases.

    params: ``hidden_size``, ``experts``, ``top``, ``expert_ff``, ``limit`` (with the clamped activation),
    optional ``alpha`` (default 1.702), ``shared_ff`` (0 or absent: no shared expert), ``shared_limit``,
    ``activation``, ``scores``, ``route_scale`` (default 1), ``groups``, ``keep_groups``, ``group_score``,
    ``correction`` (default False) and ``shared_gate``.
    tensors: ``router``, ``e{i}.gate``, ``e{i}.up``, ``e{i}.down``, with a correction ``correction`` and, with a
    shared expert, ``shared.gate``, ``shared.up``, ``shared.down`` and, with its gate, ``shared.sg``.
    """

    def __init__(self, spec):
        super().__init__(spec)
        g = self.spec.params.get
        self.hidden = int(self.param("hidden_size"))
        self.experts, self.top = int(self.param("experts")), int(self.param("top"))
        self.ff = int(self.param("expert_ff"))
        self.activation = str(g("activation", "clamped"))
        if self.activation == "clamped":
            self.limit, self.alpha, self.up_offset = float(self.param("limit")), float(g("alpha", 1.702)), 1.0
        elif self.activation == "silu":     # the clamped form without a limit, with alpha 1 and no offset
            self.limit, self.alpha, self.up_offset = float("inf"), 1.0, 0.0
        else:
            raise ValueError(f"unknown activation {self.activation!r} of the experts: 'clamped' or 'silu'")
        self.scores = str(g("scores", "chosen"))
        if self.scores not in ops.ROUTE_MODES:
            raise ValueError(f"unknown scores {self.scores!r} of the router: one of {sorted(ops.ROUTE_MODES)}")
        self.correction = bool(g("correction", False))
        if self.correction and self.scores != "sigmoid":
            raise ValueError("a correction of the choice goes with sigmoid scores")
        self.group_score = str(g("group_score", "best"))
        if self.group_score not in ("best", "top2"):
            raise ValueError(f"unknown group_score {self.group_score!r}: 'best' or 'top2'")
        self.shared_gate = g("shared_gate")
        if self.shared_gate not in (None, "sigmoid"):
            raise ValueError(f"unknown shared_gate {self.shared_gate!r}: 'sigmoid' or none")
        self.route_scale = float(g("route_scale", 1.0))
        self.groups, self.keep_groups = int(g("groups") or 0), int(g("keep_groups") or 0)
        self.shared_ff = int(g("shared_ff") or 0)
        self.shared_limit = float(g("shared_limit", self.limit))
        if self.shared_gate and not self.shared_ff:
            raise ValueError("a gate of the shared expert without a shared expert")
        if not 0 < self.top <= self.experts:
            raise ValueError(f"{self.top} of {self.experts} experts per token")
        if self.groups > 1:
            if self.experts % self.groups or not 0 < self.keep_groups <= self.groups:
                raise ValueError(f"{self.experts} experts in {self.groups} groups of which {self.keep_groups} are kept")
            if self.keep_groups * (self.experts // self.groups) < self.top:
                raise ValueError(f"{self.keep_groups} groups of {self.experts // self.groups} experts cannot give {self.top}")

    def param_decls(self):
        H, ff = self.hidden, self.ff
        decls = {"router": ParamDecl((self.experts, H))}
        for e in range(self.experts):
            decls[f"e{e}.gate"] = ParamDecl((ff, H))
            decls[f"e{e}.up"] = ParamDecl((ff, H))
            decls[f"e{e}.down"] = ParamDecl((H, ff))
        if self.shared_ff:
            decls["shared.gate"] = ParamDecl((self.shared_ff, H))
            decls["shared.up"] = ParamDecl((self.shared_ff, H))
            decls["shared.down"] = ParamDecl((H, self.shared_ff))
            if self.shared_gate:
                decls["shared.sg"] = ParamDecl((1, H))
        if self.correction:
            decls["correction"] = ParamDecl((self.experts,), "table")
        return decls

    def bind(self, tensors, dtype, device):
        E = range(self.experts)
        self.router = _as_compute(tensors["router"], dtype).contiguous()
        if self.shared_gate:     # the gate's row rides in the router's product: its logit comes out in fp32 beside theirs
            rows = [self.router, _as_compute(tensors["shared.sg"], dtype).reshape(1, -1)]
            pad = -(self.experts + 1) % 8      # rows of zeros up to a multiple of 8: the library's aligned products
            if pad:
                rows.append(torch.zeros((pad, self.hidden), dtype=self.router.dtype, device=self.router.device))
            self.router = torch.cat(rows).contiguous()
        self.choice_correction = tensors["correction"].to(torch.float32).contiguous() if self.correction else None
        # per expert its gate rows, then its up rows: one operand for a grouped product, two for the own kernels
        self.w_gate_up = torch.stack([torch.cat([_as_compute(tensors[f"e{e}.gate"], dtype),
                                                 _as_compute(tensors[f"e{e}.up"], dtype)]) for e in E]).contiguous()
        self.w_down = torch.stack([_as_compute(tensors[f"e{e}.down"], dtype) for e in E]).contiguous()
        self.shared_in = self.shared_out = None
        self.shared_pairs = None
        if self.shared_ff:
            gate, up = _as_compute(tensors["shared.gate"], dtype), _as_compute(tensors["shared.up"], dtype)
            if self.activation == "silu":
                # the plain SiLU unit: gate and up rows alternate, so that the activation rides in the product's epilogue
                self.shared_pairs = torch.stack([gate, up], dim=1).reshape(2 * gate.shape[0], gate.shape[1]).contiguous()
            else:
                self.shared_in = Linear(torch.cat([gate, up], dim=0).contiguous())
            self.shared_out = Linear(_as_compute(tensors["shared.down"], dtype).contiguous())

    def forward(self, x, ctx):
        shared = None
        if self.shared_pairs is not None:
            shared = self.shared_out(ops.linear_swiglu(x, self.shared_pairs, act="silu"))
        elif self.shared_in is not None:
            shared = self.shared_out(ops.clamped_glu(self.shared_in(x), self.shared_limit, self.alpha, self.up_offset))
        ids, weights, logits = ops.moe_route(x, self.router, self.top, scores=self.scores, groups=self.groups,
                                             keep_groups=self.keep_groups, scale=self.route_scale,
                                             correction=self.choice_correction, group_top2=self.group_score == "top2",
                                             experts=self.experts, return_logits=True)
        gate = logits[:, self.experts:self.experts + 1] if self.shared_gate else None
        return ops.moe_experts(x, ids, weights, self.w_gate_up, self.w_down, self.limit, self.alpha, shared,
                               up_offset=self.up_offset, shared_gate=gate)


register_feed_forward("routed_experts", RoutedExperts, replace=True)
