"""What a block does to the residual stream and to a sublayer's input besides norms.

``causal_conv_input``: what a sublayer reads, h, becomes ``h + conv(h)``: a causal convolution over
time on each channel, ``conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j)`` with zeros before the
sequence's start and no bias.  The last ``taps - 1`` inputs are per-request state (32-bit).  The
block runs it in the same launch as the norm in front of it.

``token_side_input``: a second embedding per token and layer.  ``e`` is the token's row of the
layer's slice of a table; ``g = gelu(W_gate x) * e`` with x the residual stream; ``y = W_proj g``;
the stream gets ``y / sqrt(mean(y^2) + eps) * w`` added (times the block's residual multiplier).

``depth_average``: with X_0 the embedding output and X_(i+1) the result of layer i, what leaves
layer i is ``sum_(j <= i + 1) w[j] X_j``.  The results of all layers of the step are kept in one
32-bit buffer in ``ctx.extras``.

The parts hold tensors and sizes; the block that arranges them (``prenorm_stream``) launches one
kernel for the end of a layer: pending sublayer output, token input and weighted sum together.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.specs import TensorSpec
from .base import Part, StateNeed, register_part


@register_part("stream", "causal_conv_input")
class CausalConvInput(Part):
    @classmethod
    def tensor_specs(cls, spec):
        return {"weight": TensorSpec((spec["size"], spec["taps"]), "conv")}

    @classmethod
    def kernel_libraries(cls, spec, runtime):
        return ("stream",)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.size, self.taps = int(spec["size"]), int(spec["taps"])
        if not 1 <= self.taps <= ops.MAX_CONV_TAPS:
            raise ops.UnsupportedSize(f"{self.taps} taps: the convolution kernels take 1 to {ops.MAX_CONV_TAPS}")
        self.weight = runtime.vector(tensors["weight"])

    def state_need(self) -> StateNeed:
        """The last ``taps - 1`` inputs, oldest first, ``[taps - 1, size]`` floats in one row."""
        return StateNeed(((self.taps - 1) * self.size,), torch.float32)


@register_part("stream", "token_side_input")
class TokenSideInput(Part):
    @classmethod
    def tensor_specs(cls, spec):
        hidden, size = spec["hidden_size"], spec["size"]
        return {
            "table": TensorSpec((spec["vocab_size"], spec["table_width"])),
            "gate.weight": TensorSpec((size, hidden)),
            "proj.weight": TensorSpec((hidden, size)),
            "norm.weight": TensorSpec((hidden,), "scale"),
        }

    @classmethod
    def kernel_libraries(cls, spec, runtime):
        return ("stream",)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        if self.size > ops.MAX_SIDE_SIZE:
            raise ops.UnsupportedSize(f"a token input of {self.size} values: the kernel takes up to {ops.MAX_SIDE_SIZE}")
        offset = int(spec.get("table_offset", 0))
        # this layer's columns of the table only: the layers together hold the table once
        self.table = runtime.matrix(tensors["table"][:, offset:offset + self.size].contiguous())
        self.gate = runtime.matrix(tensors["gate.weight"])
        self.proj = runtime.matrix(tensors["proj.weight"].t().contiguous())     # [size, hidden]: rows are read along the stream
        self.norm = runtime.vector(tensors["norm.weight"])


@register_part("stream", "depth_average")
class DepthAverage(Part):
    @classmethod
    def tensor_specs(cls, spec):
        return {"weight": TensorSpec((spec["index"] + 2,), "depth")}

    @classmethod
    def kernel_libraries(cls, spec, runtime):
        return ("stream",)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.index, self.layers = int(spec["index"]), int(spec["layers"])
        if not 0 <= self.index < self.layers:
            raise ValueError(f"layer {self.index} of {self.layers}")
        self.weight = runtime.vector(tensors["weight"])

    def history(self, ctx, residual: torch.Tensor) -> torch.Tensor:
        """The step's buffer ``[layers + 1, tokens, hidden]``: made by the first layer, which also puts
        the embedding output into its first row."""
        if self.index == 0:
            history = torch.empty((self.layers + 1, *residual.shape), dtype=torch.float32, device=residual.device)
            ctx.extras["depth_history"] = history
            return history
        history = ctx.extras.get("depth_history")
        if history is None or history.shape[1:] != residual.shape:
            raise RuntimeError("a depth average runs before the first layer of the step has made the history")
        return history
