"""Mixers with a state of fixed size per request instead of keys and values.

Both run the same recurrence kernel (``ops.linear_recurrence``): per head a
32-bit state ``S [dim, vdim]`` with ``S <- a_t S + k_t (s_t v_t)^T`` and
``y_t = S^T q_t + skip v_t``, token after token in each request, read from and
written back to the request's state slot, so a prompt cut into portions and a
token decoded alone continue where the step before stopped.

``lightning``: linear attention with a constant decay per head.  ``q, k, v =
silu(W h)``; the heads of ``y`` are normalised together (RMS, weight), multiplied
by ``sigmoid(W_g h)`` and projected.  One matrix product for q, k, v and the gate.

``mamba2``: the state-space layer of Mamba-2 in its recurrent form.  One product
gives ``[z | x | B | C | dt]``; x, B and C pass a short causal convolution per
channel with bias and SiLU (its last ``taps - 1`` inputs are part of the
request's state); ``dt = softplus(dt + dt_bias)``, ``a_t = exp(-exp(A_log) dt)``,
``s_t = dt``, ``k = B``, ``q = C`` (shared by the heads of a group), ``v = x``,
``skip = D``; ``y * silu(z)`` is normalised in ``norm_groups`` parts (RMS, weight)
and projected.  Decays, step sizes, state, gates and norms are 32-bit.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.specs import TensorSpec
from .base import CacheView, Mixer, StateNeed, StepContext, register_part


class _RecurrentMixer(Mixer):
    @classmethod
    def kernel_libraries(cls, spec, runtime):
        return ("pointwise", "recurrence", "gemm_simt") + (
            ("gemm_tcgen05",) if runtime.dtype == torch.bfloat16 else ()
        )

    #: (heads, rows, columns) of the recurrent state, set by the subclasses
    state_shape: tuple[int, int, int] = (0, 0, 0)

    def launch_key(self, ctx: StepContext, page_size: int) -> tuple:
        """Long portions are cut into segments by the step's longest portion, a host-side figure."""
        return ops.recurrence_plan(ctx.num_requests, ctx.max_q_len, *self.state_shape)

    def launch_group(self):
        return ("recurrence",) + self.state_shape

    def _state(self, cache: CacheView) -> torch.Tensor:
        if cache.state is None or not cache.writes:
            raise ValueError(f"a {self.kind} mixer needs a state of its own")
        return cache.state


@register_part("mixer", "lightning")
class LightningAttention(_RecurrentMixer):
    @classmethod
    def tensor_specs(cls, spec):
        hidden, heads, dim, vdim = spec["hidden_size"], spec["num_heads"], spec["head_size"], spec["value_head_size"]
        return {
            "q_proj.weight": TensorSpec((heads * dim, hidden)),
            "k_proj.weight": TensorSpec((heads * dim, hidden)),
            "v_proj.weight": TensorSpec((heads * vdim, hidden)),
            "g_proj.weight": TensorSpec((heads * vdim, hidden)),
            "o_proj.weight": TensorSpec((hidden, heads * vdim)),
            "norm.weight": TensorSpec((heads * vdim,), "scale"),
        }

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.heads = int(spec["num_heads"])
        self.dim = int(spec["head_size"])
        self.vdim = int(spec["value_head_size"])
        self.eps = float(spec["eps"])
        decay = [float(d) for d in spec["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"{len(decay)} decays for {self.heads} heads")
        if self.dim > ops.MAX_STATE_ROWS:
            raise ops.UnsupportedSize(f"head size {self.dim}: the recurrence kernel takes up to {ops.MAX_STATE_ROWS}")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=runtime.device)
        matrices = [tensors[n + "_proj.weight"] for n in ("q", "k", "v", "g")]
        if len({m.dtype for m in matrices}) > 1:
            matrices = [m.to(torch.float32) for m in matrices]
        self.in_weight = runtime.matrix(torch.cat(matrices, dim=0))
        self.out_weight = runtime.matrix(tensors["o_proj.weight"])
        self.norm_weight = runtime.vector(tensors["norm.weight"])
        self.state_shape = (self.heads, self.dim, self.vdim)

    def cache_need(self):
        return StateNeed((self.heads * self.dim * self.vdim,), torch.float32)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        tokens = x.shape[0]
        keys, values = self.heads * self.dim, self.heads * self.vdim
        proj = ops.project(x, self.in_weight, ctx.status, allow_partial=False)
        q, k = proj[:, :keys], proj[:, keys:2 * keys]
        v, gate = proj[:, 2 * keys:2 * keys + values], proj[:, 2 * keys + values:]
        state = self._state(cache)
        y = torch.empty((tokens, values), dtype=torch.float32, device=x.device)
        ops.linear_recurrence(
            q, k, v, state.view(state.shape[0], self.heads, self.dim, self.vdim), ctx.q_start, ctx.state_slots, y,
            self.heads, self.heads, self.dim, self.vdim, head_decay=self.decay, silu_inputs=True,
            max_q_len=ctx.max_q_len,
        )
        out = torch.empty((tokens, values), dtype=self.runtime.dtype, device=x.device)
        ops.gated_norm(y, gate, self.norm_weight, out, 1, self.eps, gate_first=False, gate_kind="sigmoid")
        return ops.project(out, self.out_weight, ctx.status)


@register_part("mixer", "mamba2")
class Mamba2(_RecurrentMixer):
    @classmethod
    def _sizes(cls, spec):
        heads, vdim, state, groups = spec["num_heads"], spec["value_head_size"], spec["state_size"], spec["num_groups"]
        inner = heads * vdim
        return heads, vdim, state, groups, inner, inner + 2 * groups * state

    @classmethod
    def tensor_specs(cls, spec):
        heads, vdim, state, groups, inner, channels = cls._sizes(spec)
        hidden, taps = spec["hidden_size"], spec["conv_taps"]
        return {
            "in_proj.weight": TensorSpec((inner + channels + heads, hidden)),
            "conv.weight": TensorSpec((channels, taps), "conv"),
            "conv.bias": TensorSpec((channels,), "bias"),
            "dt_bias": TensorSpec((heads,), "dt_bias"),
            "A_log": TensorSpec((heads,), "a_log"),
            "D": TensorSpec((heads,), "scale"),
            "norm.weight": TensorSpec((inner,), "scale"),
            "o_proj.weight": TensorSpec((hidden, inner)),
        }

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.heads, self.vdim, self.state_size, self.groups, self.inner, self.channels = self._sizes(spec)
        self.taps = int(spec["conv_taps"])
        self.norm_groups = int(spec.get("norm_groups", 1))
        self.eps = float(spec["eps"])
        if self.heads % self.groups:
            raise ValueError(f"{self.heads} heads are not a multiple of {self.groups} groups")
        if self.inner % self.norm_groups:
            raise ValueError(f"an inner width of {self.inner} cannot be normalised in {self.norm_groups} equal parts")
        if not 1 <= self.taps <= ops.MAX_CONV_TAPS:
            raise ops.UnsupportedSize(f"{self.taps} taps: the convolution kernel takes 1 to {ops.MAX_CONV_TAPS}")
        if self.state_size > ops.MAX_STATE_ROWS:
            raise ops.UnsupportedSize(f"state size {self.state_size}: the kernel takes up to {ops.MAX_STATE_ROWS}")
        self.in_weight = runtime.matrix(tensors["in_proj.weight"])
        self.out_weight = runtime.matrix(tensors["o_proj.weight"])
        self.conv_weight = runtime.vector(tensors["conv.weight"])
        self.conv_bias = runtime.vector(tensors["conv.bias"])
        self.dt_bias = runtime.vector(tensors["dt_bias"])
        self.a_log = runtime.vector(tensors["A_log"])
        self.skip = runtime.vector(tensors["D"])
        self.norm_weight = runtime.vector(tensors["norm.weight"])
        self.state_floats = self.heads * self.state_size * self.vdim
        self.state_shape = (self.heads, self.state_size, self.vdim)

    def cache_need(self):
        # the recurrent state, then the convolution's last taps-1 inputs [taps-1, channels]
        return StateNeed((self.state_floats + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        tokens, device = x.shape[0], x.device
        inner, channels, heads = self.inner, self.channels, self.heads
        proj = ops.project(x, self.in_weight, ctx.status, allow_partial=False)
        z, xbc, dt_raw = proj[:, :inner], proj[:, inner:inner + channels], proj[:, inner + channels:]
        state = self._state(cache)
        slots = state.shape[0]
        recurrent = state[:, :self.state_floats].view(slots, heads, self.state_size, self.vdim)
        conv_state = state[:, self.state_floats:].view(slots, self.taps - 1, channels)
        conv = torch.empty((tokens, channels), dtype=proj.dtype, device=device)
        dt = torch.empty((tokens, heads), dtype=torch.float32, device=device)
        decay = torch.empty_like(dt)
        ops.conv_silu(
            xbc, self.conv_weight, self.conv_bias, conv_state, ctx.seq_of_token, ctx.q_start, ctx.state_slots, conv,
            dt_raw, self.dt_bias, self.a_log, dt, decay,
        )
        width = self.groups * self.state_size
        xs, b, c = conv[:, :inner], conv[:, inner:inner + width], conv[:, inner + width:]
        y = torch.empty((tokens, inner), dtype=torch.float32, device=device)
        ops.linear_recurrence(
            c, b, xs, recurrent, ctx.q_start, ctx.state_slots, y, heads, self.groups, self.state_size, self.vdim,
            token_decay=decay, token_scale=dt, skip=self.skip, max_q_len=ctx.max_q_len,
        )
        out = torch.empty((tokens, inner), dtype=self.runtime.dtype, device=device)
        ops.gated_norm(y, z, self.norm_weight, out, self.norm_groups, self.eps, gate_first=True, gate_kind="silu")
        return ops.project(out, self.out_weight, ctx.status)


@register_part("mixer", "gated_linear_recurrence")
class GatedLinearRecurrence(Mixer):
    """A recurrent block with a real-gated linear recurrent unit: a state of one float per channel.

    Two branches of ``width`` channels: ``y = gelu(W_y h + b_y)`` and ``u = conv(W_x h + b_x)``, a causal
    convolution per channel with bias and no activation (its last ``taps - 1`` inputs are state).  u
    is cut into ``blocks`` equal parts; in part b ``r = sigmoid(A_b u_b + a_b)`` and ``i = sigmoid(I_b
    u_b + i_b)`` with square matrices.  ``log a = -c r softplus(lam)`` with the constant c
    (``decay_constant``), ``S <- a S + sqrt(1 - a^2) i u`` from ``S = 0``, output ``W_o (S y)`` times
    ``output_scale``.  One product for both branches, one batched product for both gates; gates,
    decays and the state are 32-bit."""

    @classmethod
    def tensor_specs(cls, spec):
        hidden, width, blocks, taps = spec["hidden_size"], spec["width"], spec["blocks"], spec["conv_taps"]
        part = width // blocks
        return {
            "y_proj.weight": TensorSpec((width, hidden)),
            "y_proj.bias": TensorSpec((width,), "bias"),
            "x_proj.weight": TensorSpec((width, hidden)),
            "x_proj.bias": TensorSpec((width,), "bias"),
            "conv.weight": TensorSpec((width, taps), "conv"),
            "conv.bias": TensorSpec((width,), "bias"),
            "gate_a.weight": TensorSpec((blocks, part, part)),
            "gate_a.bias": TensorSpec((blocks, part), "bias"),
            "gate_i.weight": TensorSpec((blocks, part, part)),
            "gate_i.bias": TensorSpec((blocks, part), "bias"),
            "lam": TensorSpec((width,), "rate"),
            "o_proj.weight": TensorSpec((hidden, width)),
        }

    @classmethod
    def kernel_libraries(cls, spec, runtime):
        return ("pointwise", "recurrence", "gemm_simt") + (("gemm_tcgen05",) if runtime.dtype == torch.bfloat16 else ())

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.width, self.blocks, self.taps = int(spec["width"]), int(spec["blocks"]), int(spec["conv_taps"])
        if self.width % self.blocks:
            raise ValueError(f"a width of {self.width} is not a multiple of {self.blocks} blocks")
        if not 1 <= self.taps <= ops.MAX_CONV_TAPS:
            raise ops.UnsupportedSize(f"{self.taps} taps: the convolution kernel takes 1 to {ops.MAX_CONV_TAPS}")
        self.part = self.width // self.blocks
        self.output_scale = float(spec.get("output_scale", 1.0))
        matrices = [tensors["y_proj.weight"], tensors["x_proj.weight"]]
        if len({m.dtype for m in matrices}) > 1:
            matrices = [m.to(torch.float32) for m in matrices]
        self.in_weight = runtime.matrix(torch.cat(matrices, dim=0))
        self.in_bias = runtime.vector(torch.cat([tensors["y_proj.bias"].float(), tensors["x_proj.bias"].float()]))
        self.conv_weight = runtime.vector(tensors["conv.weight"])
        self.conv_bias = runtime.vector(tensors["conv.bias"])
        gates = [tensors["gate_a.weight"], tensors["gate_i.weight"]]
        if len({m.dtype for m in gates}) > 1:
            gates = [m.to(torch.float32) for m in gates]
        # per block the rows of the recurrence gate, then those of the input gate
        self.gate_weight = runtime.matrix(torch.cat(gates, dim=1))                       # [blocks, 2 part, part]
        self.gate_bias = runtime.vector(torch.cat([tensors["gate_a.bias"].float(), tensors["gate_i.bias"].float()], dim=1))
        # log a = rate * r with rate = -c softplus(lam), made once in 64-bit
        rate = -float(spec["decay_constant"]) * torch.nn.functional.softplus(tensors["lam"].to(torch.float64))
        self.rate = runtime.vector(rate)
        self.out_weight = runtime.matrix(tensors["o_proj.weight"])

    def cache_need(self):
        # the recurrent state, then the convolution's last taps-1 inputs [taps-1, width]
        return StateNeed((self.width * self.taps,), torch.float32)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        if cache.state is None or not cache.writes:
            raise ValueError("a gated linear recurrence needs a state of its own")
        tokens, width, device = x.shape[0], self.width, x.device
        proj = ops.project(x, self.in_weight, ctx.status, allow_partial=False)           # [T, y | x], bias not yet added
        state = cache.state
        recurrent = state[:, :width]
        conv_state = state[:, width:width * self.taps].unflatten(1, (self.taps - 1, width))
        u = torch.empty((tokens, width), dtype=proj.dtype, device=device)
        ops.conv_silu(
            proj[:, width:], self.conv_weight, self.conv_bias, conv_state, ctx.seq_of_token, ctx.q_start,
            ctx.state_slots, u, activation=False, input_bias=self.in_bias[width:],
        )
        gates = torch.empty((tokens, self.blocks, 2 * self.part), dtype=torch.float32, device=device)
        ops.per_head_project(u.view(tokens, self.blocks, self.part), self.gate_weight, gates)
        out = torch.empty((tokens, width), dtype=self.runtime.dtype, device=device)
        ops.gated_scan(
            gates, self.gate_bias, u, proj[:, :width], self.in_bias[:width], self.rate, recurrent, ctx.q_start,
            ctx.state_slots, out, self.output_scale, max_q_len=ctx.max_q_len,
        )
        return ops.project(out, self.out_weight, ctx.status)


@register_part("mixer", "matrix_memory")
class MatrixMemory(_RecurrentMixer):
    """A matrix memory with exponential gates (the mLSTM of xLSTM: Beck et al., "xLSTM: Extended Long
    Short-Term Memory").  Per head a state ``S [dim, vdim]``, a normaliser ``n [dim]`` and the running
    maximum m of the gates' logarithms, which starts at zero::

        i_t = c tanh((W_i h + b_i) / c)            f_t = logsigmoid(c tanh((W_f h + b_f) / c))
        m_t = max(f_t + m_(t-1), i_t)
        S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T          (n_t likewise, with k_t alone)
        o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + denominator_eps)

    with ``q = query_scale W_q h`` and the cap c (``gate_cap``).  Every head's o is divided by its root mean
    square, the heads together are multiplied by a stored weight and by ``sigmoid(W_g h)`` and
    projected.  The normaliser rides along as one more value column (a column of ones behind every
    head's values), so S and n pass through the recurrence kernel of the other mixers as one state
    ``[dim, columns]``; a kernel before it turns the raw gates into the recurrence's per-token decay and
    scale, a kernel behind it divides, normalises and gates.  Gates, maximum, state, the division
    and the norm are 32-bit; the two gate projections leave 32-bit values in both precisions."""

    @classmethod
    def tensor_specs(cls, spec):
        hidden, heads, dim, vdim = spec["hidden_size"], spec["num_heads"], spec["head_size"], spec["value_head_size"]
        return {
            "q_proj.weight": TensorSpec((heads * dim, hidden)),
            "k_proj.weight": TensorSpec((heads * dim, hidden)),
            "v_proj.weight": TensorSpec((heads * vdim, hidden)),
            "g_proj.weight": TensorSpec((heads * vdim, hidden)),
            "i_proj.weight": TensorSpec((heads, hidden)),
            "i_proj.bias": TensorSpec((heads,), "bias"),
            "f_proj.weight": TensorSpec((heads, hidden)),
            "f_proj.bias": TensorSpec((heads,), "forget_bias"),
            "norm.weight": TensorSpec((heads * vdim,), "scale"),
            "o_proj.weight": TensorSpec((hidden, heads * vdim)),
        }

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.heads = int(spec["num_heads"])
        self.dim = int(spec["head_size"])
        self.vdim = int(spec["value_head_size"])
        self.eps = float(spec["eps"])
        self.gate_cap = float(spec["gate_cap"])
        self.query_scale = float(spec.get("query_scale", self.dim ** -0.5))
        self.denominator_eps = float(spec["denominator_eps"])
        if not self.gate_cap > 0:
            raise ValueError(f"gate_cap must be positive, got {self.gate_cap}")
        if self.dim > ops.MAX_STATE_ROWS:
            raise ops.UnsupportedSize(f"head size {self.dim}: the recurrence kernel takes up to {ops.MAX_STATE_ROWS}")
        self.columns = ops.memory_value_columns(self.vdim)
        matrices = [tensors[n + "_proj.weight"] for n in ("q", "k", "v", "g")]
        if len({m.dtype for m in matrices}) > 1:
            matrices = [m.to(torch.float32) for m in matrices]
        self.in_weight = runtime.matrix(torch.cat(matrices, dim=0))
        gates = [tensors["i_proj.weight"], tensors["f_proj.weight"]]
        if len({m.dtype for m in gates}) > 1:
            gates = [m.to(torch.float32) for m in gates]
        self.gate_weight = runtime.matrix(torch.cat(gates, dim=0))                        # [2 heads, hidden]: input gates, forget gates
        self.gate_bias = runtime.vector(torch.cat([tensors["i_proj.bias"].float(), tensors["f_proj.bias"].float()]))
        self.out_weight = runtime.matrix(tensors["o_proj.weight"])
        self.norm_weight = runtime.vector(tensors["norm.weight"])
        self.state_floats = self.heads * self.dim * self.columns
        self.state_shape = (self.heads, self.dim, self.columns)

    def cache_need(self):
        # S with the normaliser as one of its columns, then the running maximum of every head; rows of
        # whole 16-byte pieces, which the streaming recurrence kernel wants
        return StateNeed(((self.state_floats + self.heads + 3) // 4 * 4,), torch.float32)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        tokens, device = x.shape[0], x.device
        heads, keys, values = self.heads, self.heads * self.dim, self.heads * self.vdim
        proj = ops.project(x, self.in_weight, ctx.status, allow_partial=False)
        q, k = proj[:, :keys], proj[:, keys:2 * keys]
        v, gate = proj[:, 2 * keys:2 * keys + values], proj[:, 2 * keys + values:]
        raw_gates = ops.project(x, self.gate_weight, ctx.status, out_dtype=torch.float32)   # [T, 2 heads], or partial sums
        state = self._state(cache)
        slots = state.shape[0]
        memory = state[:, :self.state_floats].view(slots, heads, self.dim, self.columns)
        top = state[:, self.state_floats:self.state_floats + heads]
        decay = torch.empty((tokens, heads), dtype=torch.float32, device=device)
        scale = torch.empty_like(decay)
        floor = torch.empty_like(decay)
        v_wide = torch.empty((tokens, heads * self.columns), dtype=proj.dtype, device=device)
        ops.memory_gates(raw_gates, self.gate_bias, self.gate_cap, v, top, ctx.q_start, ctx.state_slots, decay, scale,
                         floor, v_wide, heads, self.vdim, max_q_len=ctx.max_q_len)
        # a step of single tokens with few requests: several CTAs share a head's rows and leave parts of y
        parts = 1
        if ctx.max_q_len == 1:
            parts = ops.recurrence_step_splits(ctx.num_requests, heads, self.dim, self.columns, memory)
        shape = (tokens, heads * self.columns) if parts == 1 else (parts, tokens, heads * self.columns)
        y = torch.empty(shape, dtype=torch.float32, device=device)
        ops.linear_recurrence(
            q, k, v_wide, memory, ctx.q_start, ctx.state_slots, y, heads, heads, self.dim, self.columns,
            token_decay=decay, token_scale=scale, max_q_len=ctx.max_q_len,
        )
        out = torch.empty((tokens, values), dtype=self.runtime.dtype, device=device)
        ops.memory_output(y, floor, gate, self.norm_weight, out, heads, self.vdim, self.query_scale, self.eps,
                          self.denominator_eps)
        return ops.project(out, self.out_weight, ctx.status)
