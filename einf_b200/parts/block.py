"""Arrangements of parts in one layer.

``prenorm``: ``h += mixer(norm1(h)); h += feed_forward(norm2(h))``.  The
residual stream ``h`` is a 32-bit tensor; a sublayer's output stays *pending*
until the next norm adds it, so each add is fused with the norm that follows
(``src/einf/executors/torch/qwen.py:526-563``).  ``prenorm_mixer`` has no feed-forward, ``parallel``
feeds mixer and feed-forward from one norm, ``prenorm_stream`` adds a residual multiplier,
convolutions in front of the sublayers, a per-layer token input and a weighted sum over the depth.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import CacheView, Part, StepContext, build_part, join_needs, part_class, register_part


class Block(Part):
    mixer: Part

    @classmethod
    def part_categories(cls) -> dict[str, str]:
        """Role name in :class:`LayerSpec.parts` -> part category."""
        raise NotImplementedError

    def forward(
        self, residual: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext, cache: CacheView
    ) -> torch.Tensor:
        """Consume ``pending`` into ``residual`` and return the new pending output."""
        raise NotImplementedError


@register_part("block", "prenorm")
class PreNormBlock(Block):
    @classmethod
    def part_categories(cls):
        return {
            "mixer_norm": "norm",
            "mixer": "mixer",
            "feed_forward_norm": "norm",
            "feed_forward": "feed_forward",
        }

    def __init__(self, layer_spec, tensors, runtime):
        self.runtime = runtime
        self.spec = layer_spec
        for role, category in self.part_categories().items():
            setattr(self, role, build_part(category, layer_spec.parts[role], tensors, runtime))

    @staticmethod
    def _normalise(norm, pending, residual, ctx):
        # a norm that declares ``takes_status`` gets the step's status word as well
        if getattr(norm, "takes_status", False):
            return norm.forward(pending, residual, status=ctx.status)
        return norm.forward(pending, residual)

    def forward(self, residual, pending, ctx, cache):
        x = self._normalise(self.mixer_norm, pending, residual, ctx)
        mixed = self.mixer.forward(x, ctx, cache)
        x = self._normalise(self.feed_forward_norm, mixed, residual, ctx)
        return self.feed_forward.forward(x, ctx)


@register_part("block", "prenorm_mixer")
class PreNormMixerBlock(PreNormBlock):
    """``h += mixer(norm1(h))`` and nothing else: a layer without a feed-forward."""

    @classmethod
    def part_categories(cls):
        return {"mixer_norm": "norm", "mixer": "mixer"}

    def forward(self, residual, pending, ctx, cache):
        x = self._normalise(self.mixer_norm, pending, residual, ctx)
        return self.mixer.forward(x, ctx, cache)


@register_part("block", "parallel")
class ParallelBlock(PreNormBlock):
    """``h += mixer(n) + feed_forward(n)`` with one norm ``n = norm(h)`` that both sublayers read.
    A feed-forward that takes an addend sums both in its last kernel, in 32-bit; otherwise the
    pending value is the stack of both as float32 terms, which the next norm adds up."""

    @classmethod
    def part_categories(cls):
        return {"mixer_norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}

    def forward(self, residual, pending, ctx, cache):
        x = self._normalise(self.mixer_norm, pending, residual, ctx)
        mixed = self.mixer.forward(x, ctx, cache)
        if getattr(self.feed_forward, "takes_addend", False):
            return self.feed_forward.forward(x, ctx, add=mixed)   # its last kernel adds the two up
        terms = [mixed if mixed.dim() == 3 else mixed[None], self.feed_forward.forward(x, ctx)[None]]
        return torch.cat([term.to(torch.float32) for term in terms], dim=0)


def build_block(layer_spec, tensors, runtime) -> Block:
    return part_class("block", layer_spec.block)(layer_spec, tensors, runtime)


@register_part("block", "prenorm_stream")
class PreNormStreamBlock(Block):
    """``h += m mixer(c1(norm1(h))); h += m ff(c2(norm2(h)))`` with a residual multiplier m and, each
    optional: a short causal convolution ``c(x) = x + conv(x)`` in front of a sublayer (run in the
    launch of the norm before it, continued from and into the request's state row), no feed-forward,
    a per-layer token input added after the feed-forward, and a weighted sum over the results of
    all layers so far in place of the layer's own result.  The layer's last kernel adds the pending
    sublayer output, the token input and the weighted sum in one pass over the row, so the block
    hands nothing pending to the next one.  The block's state row holds the convolutions' inputs
    in front of whatever state its mixer keeps."""

    optional_roles = ("mixer_conv", "feed_forward_norm", "feed_forward_conv", "feed_forward", "token_input",
                      "depth_mix")

    @classmethod
    def part_categories(cls):
        return {
            "mixer_norm": "norm",
            "mixer_conv": "stream",
            "mixer": "mixer",
            "feed_forward_norm": "norm",
            "feed_forward_conv": "stream",
            "feed_forward": "feed_forward",
            "token_input": "stream",
            "depth_mix": "stream",
        }

    def __init__(self, layer_spec, tensors, runtime):
        self.runtime = runtime
        self.spec = layer_spec
        self.residual_mult = float(layer_spec.params.get("residual_mult", 1.0))
        for role, category in self.part_categories().items():
            part = None
            if role in layer_spec.parts:
                part = build_part(category, layer_spec.parts[role], tensors, runtime)
            elif role not in self.optional_roles:
                raise KeyError(f"a prenorm_stream layer needs the part {role!r}")
            setattr(self, role, part)
        if (self.feed_forward is None) != (self.feed_forward_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        if self.feed_forward is None and self.feed_forward_conv is not None:
            raise ValueError("a convolution in front of a feed-forward that is not there")
        needs = [conv.state_need() if conv is not None else None for conv in (self.mixer_conv, self.feed_forward_conv)]
        self._need, offsets = join_needs(*needs, self.mixer.cache_need())
        self._conv_offsets, self._mixer_offset = offsets[:2], offsets[2]

    def cache_need(self):
        return self._need

    def _conv_state(self, which: int, cache: CacheView):
        conv = (self.mixer_conv, self.feed_forward_conv)[which]
        if conv is None or conv.taps == 1:
            return None
        offset = self._conv_offsets[which]
        rows = cache.state[:, offset:offset + (conv.taps - 1) * conv.size]
        return rows.unflatten(1, (conv.taps - 1, conv.size))

    def _normalise(self, which: int, pending, residual, ctx, cache):
        norm = (self.mixer_norm, self.feed_forward_norm)[which]
        conv = (self.mixer_conv, self.feed_forward_conv)[which]
        out = torch.empty(residual.shape, dtype=self.runtime.dtype, device=residual.device)
        ops.norm_conv(
            pending, self.residual_mult, residual, norm.weight, norm.eps, None if conv is None else conv.weight,
            self._conv_state(which, cache), ctx.seq_of_token, ctx.q_start, ctx.state_slots, out,
            single_tokens=ctx.decode_only,
        )
        return out

    def forward(self, residual, pending, ctx, cache):
        if pending is not None:
            raise ValueError("a prenorm_stream layer follows one that left its output pending")
        depth = self.depth_mix
        history = None
        if depth is not None:
            history = depth.history(ctx, residual)
            if depth.index == 0:
                history[0].copy_(residual)      # the embedding output, before this layer changes the stream
        x = self._normalise(0, None, residual, ctx, cache)
        view = cache
        if self._mixer_offset is not None:
            view = CacheView(cache.group, cache.k, cache.v, cache.state[:, self._mixer_offset:], cache.writes,
                             cache.page_size)
        terms = self.mixer.forward_terms(x, ctx, view) if hasattr(self.mixer, "forward_terms") \
            else [self.mixer.forward(x, ctx, view)]
        if self.feed_forward is not None:
            x = self._normalise(1, terms, residual, ctx, cache)
            terms = [self.feed_forward.forward(x, ctx)]
        side = self.token_input
        ops.stream_tail(
            residual, terms, self.residual_mult, ctx.token_ids,
            None if side is None else (side.table, side.gate, side.proj, side.norm, side.eps),
            None if depth is None else (history, depth.index, depth.weight),
        )
        return None
