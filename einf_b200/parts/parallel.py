"""Several mixers side by side on one input.

``side_by_side`` nests ``mixers`` (a tuple of mixer specs).  All read the same normalised input;
the result is the sum of their outputs, each already multiplied by its own ``output_scale`` where
the design has one (a mixer applies it in 32-bit before its last rounding).  The sum is not formed
here: the outputs travel on as float32 terms (split-K partial sums included) that the next kernel
of the block adds up in a fixed order.  At most one of the mixers may keep pages; the state rows
of the others lie end to end in the layer's state row.
"""
from __future__ import annotations

import torch

from .base import CacheView, Mixer, StepContext, build_nested, join_needs, register_part, state_of


@register_part("mixer", "side_by_side")
class SideBySide(Mixer):
    @classmethod
    def nested_parts(cls, spec):
        return {"mixers": "mixer"}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.mixers = [build_nested("mixer", nested, tensors, runtime) for nested in spec["mixers"]]
        if not self.mixers:
            raise ValueError("side_by_side needs at least one mixer")
        self._need, self._offsets = join_needs(*[mixer.cache_need() for mixer in self.mixers])
        self._state_sizes = [
            None if offset is None else state_of(mixer.cache_need()).shape[0]
            for mixer, offset in zip(self.mixers, self._offsets)
        ]

    def cache_need(self):
        return self._need

    def launch_key(self, ctx: StepContext, page_size: int) -> tuple:
        return tuple(mixer.launch_key(ctx, page_size) for mixer in self.mixers)

    def launch_group(self):
        return ("side_by_side",) + tuple(mixer.launch_group() for mixer in self.mixers)

    def forward_terms(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> list:
        """Every mixer's output, ``[T, hidden]`` or partial sums ``[splits, T, hidden]``, in the order of the spec."""
        terms = []
        for mixer, offset, size in zip(self.mixers, self._offsets, self._state_sizes):
            state = None if offset is None else cache.state[:, offset:offset + size]
            view = CacheView(cache.group, cache.k, cache.v, state, cache.writes, cache.page_size)
            terms.append(mixer.forward(x, ctx, view))
        return terms

    def forward(self, x, ctx, cache):
        terms = self.forward_terms(x, ctx, cache)
        return torch.cat([(t if t.dim() == 3 else t[None]).to(torch.float32) for t in terms], dim=0)
