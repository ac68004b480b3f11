"""A decoder model put together from a :class:`ModelSpec`.

The model owns its parts and the order they run in; it does not own the cache.
``cache_plan`` says which run of which layer needs what, and the engine gives
``forward`` one :class:`CacheView` per schedule entry.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping, Optional

import torch

from ..config.specs import ModelSpec, PartSpec, TensorSpec
from .base import (
    CacheView, PagedKVNeed, PagesAndState, Runtime, StateNeed, StepContext, build_part, checkpoint_name, part_class,
    pages_of, state_of, walk_part_specs,
)
from .block import build_block


def _part_specs(model_spec: ModelSpec):
    """Every (category, PartSpec) of the model, with the parts that parts of any category nest."""
    yield from walk_part_specs("embedding", model_spec.embedding)
    for layer in model_spec.layers:
        block_class = part_class("block", layer.block)
        for role, category in block_class.part_categories().items():
            if role in layer.parts or role not in getattr(block_class, "optional_roles", ()):
                yield from walk_part_specs(category, layer.parts[role])
    yield from walk_part_specs("norm", model_spec.final_norm)
    yield from walk_part_specs("head", model_spec.head)


def expected_tensors(model_spec: ModelSpec) -> tuple[dict[str, TensorSpec], dict[str, TensorSpec]]:
    """Checkpoint tensors the model needs, and those it tolerates (a stored copy of a tied matrix)."""
    expected: dict[str, TensorSpec] = {}
    for category, spec in _part_specs(model_spec):
        for name, tensor_spec in part_class(category, spec.kind).tensor_specs(spec).items():
            expected[checkpoint_name(spec, name)] = tensor_spec
    optional: dict[str, TensorSpec] = {}
    head = model_spec.head
    if head.get("tied_to"):
        optional[checkpoint_name(head, "weight")] = TensorSpec((head["vocab_size"], head["hidden_size"]))
    return expected, optional


def kernel_libraries(model_spec: ModelSpec, runtime: Runtime) -> tuple[str, ...]:
    names: list[str] = []
    for category, spec in _part_specs(model_spec):
        names.extend(part_class(category, spec.kind).kernel_libraries(spec, runtime))
    return tuple(dict.fromkeys(names))


@dataclass(frozen=True)
class EntryCache:
    """Cache of one schedule entry: ``owner`` is the entry whose storage it uses."""

    need: PagedKVNeed | StateNeed | PagesAndState | None
    owner: int
    group: int = -1   # page group of a paged need


@dataclass(frozen=True)
class CachePlan:
    entries: tuple[EntryCache, ...]
    #: window of each page group (None: all keys are kept)
    group_windows: tuple[Optional[int], ...]
    #: per page group: the first positions of a sequence its window keeps (0: none)
    group_keeps: tuple[int, ...] = ()

    @property
    def has_state(self) -> bool:
        return any(state_of(e.need) is not None for e in self.entries)


class DecoderModel:
    def __init__(self, model_spec: ModelSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.spec = model_spec
        self.runtime = runtime
        self.embedding = build_part("embedding", model_spec.embedding, tensors, runtime)
        self.blocks = [build_block(layer, tensors, runtime) for layer in model_spec.layers]
        self.final_norm = build_part("norm", model_spec.final_norm, tensors, runtime)
        head_spec = model_spec.head
        head_class = part_class("head", head_spec.kind)
        tied = None
        if head_spec.get("tied_to"):
            if head_spec["tied_to"] != checkpoint_name(model_spec.embedding, "weight"):
                raise ValueError(f"head is tied to {head_spec['tied_to']!r}, which is not the embedding table")
            tied = self.embedding.table
            self.head = head_class(head_spec, {}, runtime, tied=tied)
        else:
            self.head = build_part("head", head_spec, tensors, runtime)
        self.schedule = model_spec.schedule
        self.cache_plan = self._plan_cache()

    def _plan_cache(self) -> CachePlan:
        windows: list[tuple[Optional[int], int]] = []
        entries: list[EntryCache] = []
        for index, entry in enumerate(self.schedule):
            block = self.blocks[entry.layer]
            # a block that keeps something of its own beside its mixer's cache says so itself
            need = block.cache_need() if hasattr(block, "cache_need") else block.mixer.cache_need()
            owner = index if entry.cache_from is None else entry.cache_from
            if owner != index:
                owner_need = entries[owner].need
                if isinstance(need, PagesAndState):
                    raise ValueError(f"schedule entry {index} carries a state row and cannot read another entry's cache")
                if type(owner_need) is not type(need) or (
                    isinstance(need, PagedKVNeed)
                    and (need.num_kv_heads, need.head_size, need.value_size)
                    != (owner_need.num_kv_heads, owner_need.head_size, owner_need.value_size)
                ):
                    raise ValueError(
                        f"schedule entry {index} cannot read the cache of entry {owner}: {need} vs {owner_need}"
                    )
            group = -1
            paged = pages_of(need)
            if paged is not None:
                if owner != index:
                    group = entries[owner].group
                else:
                    # a group is a window and the first positions it keeps
                    key = (paged.window, paged.keep_first if paged.window else 0)
                    if key not in windows:
                        windows.append(key)
                    group = windows.index(key)
            entries.append(EntryCache(need, owner, group))
        if not windows:
            windows.append((None, 0))  # the manager always has one page group
        return CachePlan(tuple(entries), tuple(w for w, _ in windows), tuple(k for _, k in windows))

    def forward(self, ctx: StepContext, caches: list[CacheView]) -> torch.Tensor:
        """Run the step's tokens through every schedule entry; float logits ``[S, vocab]``
        at ``ctx.logit_rows``."""
        residual = self.embedding.forward(ctx)
        # the stream is updated in place: entries that take the embedding output again get a copy of it
        first = residual.clone() if any(entry.add_embedding for entry in self.schedule) else None
        pending = None
        for index, entry in enumerate(self.schedule):
            if entry.add_embedding:
                # one more float32 term of the pending output, which the entry's first norm adds up
                terms = [first[None]]
                if pending is not None:
                    terms.insert(0, (pending if pending.dim() == 3 else pending[None]).to(torch.float32))
                pending = torch.cat(terms, dim=0) if len(terms) > 1 else terms[0]
            pending = self.blocks[entry.layer].forward(residual, pending, ctx, caches[index])
        if getattr(self.final_norm, "takes_status", False):
            x = self.final_norm.forward(pending, residual, rows=ctx.logit_rows, status=ctx.status)
        else:
            x = self.final_norm.forward(pending, residual, rows=ctx.logit_rows)
        return self.head.forward(x, ctx.status)
