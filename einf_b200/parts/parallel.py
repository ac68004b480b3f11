"""Several mixers side by side on one input.

``side_by_side`` nests ``mixers`` (a tuple of mixer specs).  All read the same normalised input;
the result is the sum of their outputs, each already multiplied by its own ``output_scale`` where
the design has one (a mixer applies it in 32-bit before its last rounding).  The sum is not formed
here: the outputs travel on as float32 terms (split-K partial sums included) that the next kernel
of the block adds up in a fixed order.  At most one of the mixers may keep pages; the state rows
of the others lie end to end in the layer's state row.

With ``join_norm`` (``eps``, ``scale``) the result is instead ``scale * sum_i w_i * o_i / rms(o_i)``:
every mixer's output divided by its root mean square over the model width and multiplied by a
stored weight of its own (``out.<i>``, plain), the sum times a constant (one half for the mean of
two).  One kernel reads the outputs, partial sums included, and leaves the result as a float32 term.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.specs import TensorSpec
from .base import CacheView, Mixer, StepContext, build_nested, join_needs, register_part, state_of


@register_part("mixer", "side_by_side")
class SideBySide(Mixer):
    @classmethod
    def nested_parts(cls, spec):
        return {"mixers": "mixer"}

    @classmethod
    def tensor_specs(cls, spec):
        if not spec.get("join_norm"):
            return {}
        return {f"out.{i}": TensorSpec((spec["hidden_size"],), "scale") for i in range(len(spec["mixers"]))}

    @classmethod
    def kernel_libraries(cls, spec, runtime):
        return ("pointwise",) if spec.get("join_norm") else ()

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.join_norm = spec.get("join_norm")
        self.join_weights = None
        if self.join_norm:
            self.join_weights = [runtime.vector(tensors[f"out.{i}"]) for i in range(len(spec["mixers"]))]
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
        if self.join_norm:
            out = torch.empty((1, x.shape[0], int(self.spec["hidden_size"])), dtype=torch.float32, device=x.device)
            ops.norm_join(terms, self.join_weights, float(self.join_norm["eps"]), out[0],
                          float(self.join_norm.get("scale", 1.0)))
            return out
        return torch.cat([(t if t.dim() == 3 else t[None]).to(torch.float32) for t in terms], dim=0)
