"""A decoder built from a :class:`~.spec.ModelSpec`.

``DecoderModel`` owns the built parts, knows the full checkpoint name of every tensor
they declared, hands loaded tensors to them, and runs one step: embedding, the schedule
of layers, final norm and output head on the wanted rows only.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .base import (
    Arrangement,
    KVNeed,
    LayerCache,
    ParamDecl,
    Part,
    PlanNeeds,
    StateNeed,
    StepContext,
    build_part,
    lookup,
)
from .spec import ModelSpec, PartSpec


@dataclass(frozen=True)
class ExpectedTensor:
    name: str            # full checkpoint name
    decl: ParamDecl
    part: Part
    local: str


@dataclass(frozen=True)
class CacheLayerNeed:
    """What cache layer ``index`` must hold (from the mixer of the entry that writes it)."""

    index: int
    kv: KVNeed | None
    state: StateNeed | None


class DecoderModel:
    def __init__(self, spec: ModelSpec) -> None:
        self.spec = spec
        self.embedding = build_part("embedding", spec.embedding)
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head)
        self.blocks: list[Arrangement] = []
        for layer in spec.layers:
            position = build_part("position", layer.position) if layer.position else None
            block = lookup("arrangement", layer.arrangement)(
                build_part("mixer", layer.mixer),
                build_part("feed_forward", layer.feed_forward),
                build_part("norm", layer.mixer_norm),
                build_part("norm", layer.feed_forward_norm),
                position,
            )
            self.blocks.append(block)
        self.schedule = spec.schedule
        # stream parts that run before a schedule entry (None where an entry has none)
        self.before: list[Part | None] = [build_part("stream", e.before) if e.before is not None else None
                                          for e in spec.schedule]
        self.after: list[Part | None] = [build_part("stream", e.after) if e.after is not None else None
                                         for e in spec.schedule]
        self._keeps_embedding = any(getattr(p, "needs_embedding", False) for p in self.before + self.after
                                    if p is not None)
        self._bound = False

    # ------------------------------------------------------------------ declarations

    def all_parts(self) -> list[Part]:
        parts: list[Part] = [self.embedding]
        for b in self.blocks:
            parts.extend(b.parts())
        parts.extend(p for p in self.before if p is not None)
        parts.extend(p for p in self.after if p is not None)
        parts.extend([self.final_norm, self.head])
        return parts

    def expected_tensors(self) -> list[ExpectedTensor]:
        out: list[ExpectedTensor] = []
        seen: dict[str, ExpectedTensor] = {}
        for part in self.all_parts():
            for local, decl in part.param_decls().items():
                name = part.spec.tensor_name(local)
                if name in seen:
                    if seen[name].decl.shape != decl.shape:
                        raise ValueError(
                            f"tensor {name!r} is declared twice with shapes "
                            f"{seen[name].decl.shape} and {decl.shape}"
                        )
                    continue
                e = ExpectedTensor(name, decl, part, local)
                seen[name] = e
                out.append(e)
        return out

    def ignorable_tensors(self) -> set[str]:
        """Names a checkpoint may carry although nothing reads them (a tied head's copy)."""
        head = self.head
        names = set(self.spec.ignorable)
        if getattr(head, "tied", False):
            names.add(head.spec.tensor_name("weight"))
        return names

    def cache_needs(self) -> list[CacheLayerNeed]:
        needs: dict[int, CacheLayerNeed] = {}
        for e in self.schedule:
            mixer = self.blocks[e.layer].mixer
            kv, st = mixer.cache_need(), mixer.state_need()
            if e.writes_cache:
                needs[e.cache] = CacheLayerNeed(e.cache, kv, st)
        for e in self.schedule:
            if not e.writes_cache:
                mixer = self.blocks[e.layer].mixer
                kv, owner = mixer.cache_need(), needs[e.cache].kv
                if kv is None or owner is None or (kv.kv_heads, kv.head_dim) != (owner.kv_heads, owner.head_dim):
                    raise ValueError(
                        f"layer {e.layer} reads cache layer {e.cache} whose key/value shape "
                        f"{owner} does not fit its own {kv}"
                    )
        out = [needs[i] for i in range(self.spec.num_cache_layers)]
        # an embedding that keeps something per request gets a state arena behind the cache layers'
        emb_state = getattr(self.embedding, "state_need", lambda: None)()
        if emb_state is not None:
            out.append(CacheLayerNeed(self.embedding_state_index, None, emb_state))
        return out

    @property
    def embedding_state_index(self) -> int:
        """The index under which the cache manager keeps the embedding's per-request state."""
        return self.spec.num_cache_layers

    def plan_needs(self) -> PlanNeeds:
        tiles: set[int] = set()
        for b in self.blocks:
            tiles |= set(b.mixer.plan_needs().q_tile_tokens)
        return PlanNeeds(frozenset(tiles))

    def graph_safe(self) -> bool:
        """Whether a step of this model may be captured as a CUDA graph (every part says so)."""
        return all(p.graph_safe for p in self.all_parts())

    # ------------------------------------------------------------------ binding

    def bind(self, tensors, dtype: torch.dtype, device: torch.device) -> None:
        """Give every part its tensors.  ``tensors`` is anything indexed by full checkpoint
        name: a dict, or a source that fetches a tensor when it is asked for (parts are bound
        one after the other, so such a source keeps peak memory at the model plus one part)."""
        def local_view(part: Part) -> dict[str, torch.Tensor]:
            return {local: tensors[part.spec.tensor_name(local)] for local in part.param_decls()}

        self.embedding.bind(local_view(self.embedding), dtype, device)
        for b in self.blocks:
            for part in b.parts():
                part.bind(local_view(part), dtype, device)
        for part in self.before + self.after:
            if part is not None:
                part.bind(local_view(part), dtype, device)
        self.final_norm.bind(local_view(self.final_norm), dtype, device)
        if getattr(self.head, "tied", False):
            self.head.bind({}, dtype, device, tied_weight=self.embedding.weight)
        else:
            self.head.bind(local_view(self.head), dtype, device)
        self.dtype, self.device = dtype, device
        self._bound = True

    # ------------------------------------------------------------------ one step

    def forward(self, ctx: StepContext, caches: list[LayerCache], want_rows: torch.Tensor | None,
                n_want: int) -> torch.Tensor:
        """fp32 logits ``[n_want, vocab]`` at the packed rows ``want_rows`` (int32)."""
        if not self._bound:
            raise RuntimeError("the model has no weights yet")
        if len(caches) > len(self.schedule):     # the embedding's own per-request state
            x = self.embedding.forward(ctx, caches[len(self.schedule)])
        else:
            x = self.embedding.forward(ctx)
        embedded = x if self._keeps_embedding else None
        residual = None
        for i, (entry, cache) in enumerate(zip(self.schedule, caches)):
            if self.before[i] is not None:
                x, residual = self.before[i].forward(x, residual, ctx, embedded)
            block = self.blocks[entry.layer]
            if block.entry() is None:
                x, residual = block.forward(x, residual, ctx, cache)
            else:
                # a layer that takes part in the hand-over of norms is told how the next one begins
                # (not across a stream part behind this layer, which wants a plain stream)
                nxt = None
                if i + 1 < len(self.schedule) and self.after[i] is None:
                    nxt = self.blocks[self.schedule[i + 1].layer].entry()
                x, residual = block.forward(x, residual, ctx, cache, following=nxt)
            if self.after[i] is not None:
                x, residual = self.after[i].forward(x, residual, ctx, embedded)
        if n_want == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=ctx.device)
        z, _ = self.final_norm.forward(x, residual, rows=want_rows)
        return self.head.forward(z)
