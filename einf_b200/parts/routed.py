"""A routed feed-forward: many small gated feed-forwards (experts) of which each token uses a few.

``routed_mlp``: router logits ``z = W_router x`` in 32-bit; the ``top_k`` experts with the largest
scores (``score``: ``sigmoid`` or ``softmax`` over all experts; ``renormalise`` divides the chosen
weights by their sum); an expert is ``down(silu(gate(u)) * up(u))`` without biases.  With
``weight_on: "input"`` the expert sees ``u = w x`` and its output is added as it is; with ``"output"``
it sees x and its output is multiplied by w.

Optional, each from the spec.  ``correction``: a stored number per router output that is added to the
scores for the choice alone (the weights stay the scores).  ``groups`` (``count``, ``keep``): the router's
outputs form equal groups of neighbours, and only those of the ``keep`` groups whose best choice score
is largest can be chosen.  ``num_identity``: the router has that many outputs beyond the experts;
one of those, when chosen, hands the token through unchanged (times its weight) and has no tensors.
They count in the softmax, in the groups and in ``top_k`` like any expert.  ``shared`` (an
``intermediate_size``): one more gated feed-forward that every token takes, added to the sum; with
``shared_gate`` its output is multiplied by ``sigmoid(w . x)``, one stored row and one number per token
(the row rides along in the router's product).

The tokens never go through the host: the (token, choice) pairs are sorted by expert on the device,
the two products run over the sorted rows expert by expert in one launch each, and one kernel adds
a token's expert outputs up in 32-bit, together with another branch's output when the layer runs
its mixer and its feed-forward side by side (``forward(..., add=...)``).
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.specs import TensorSpec
from .base import FeedForward, register_part


@register_part("feed_forward", "routed_mlp")
class RoutedMLP(FeedForward):
    #: ``forward`` takes ``add``: a tensor (or split-K partial sums) that joins the sum over the experts
    takes_addend = True

    @classmethod
    def tensor_specs(cls, spec):
        hidden, inter, experts = spec["hidden_size"], spec["intermediate_size"], spec["num_experts"]
        outputs = experts + int(spec.get("num_identity") or 0)
        specs = {"router.weight": TensorSpec((outputs, hidden))}
        if spec.get("correction"):
            specs["router.correction"] = TensorSpec((outputs,), "small")
        if spec.get("shared"):
            shared = int(spec["shared"])
            specs["shared.gate_proj.weight"] = TensorSpec((shared, hidden))
            specs["shared.up_proj.weight"] = TensorSpec((shared, hidden))
            specs["shared.down_proj.weight"] = TensorSpec((hidden, shared))
            if spec.get("shared_gate"):
                specs["shared.gate.weight"] = TensorSpec((1, hidden))
        for e in range(experts):
            specs[f"experts.{e}.gate_proj.weight"] = TensorSpec((inter, hidden))
            specs[f"experts.{e}.up_proj.weight"] = TensorSpec((inter, hidden))
            specs[f"experts.{e}.down_proj.weight"] = TensorSpec((hidden, inter))
        return specs

    @classmethod
    def kernel_libraries(cls, spec, runtime):
        return ("pointwise", "routed", "gemm_simt") + (("gemm_tcgen05",) if runtime.dtype == torch.bfloat16 else ())

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.hidden_size = int(spec["hidden_size"])
        self.intermediate_size = int(spec["intermediate_size"])
        self.num_experts = int(spec["num_experts"])
        self.top_k = int(spec["top_k"])
        self.score = str(spec.get("score", "softmax"))
        if self.score not in ops.ROUTER_SCORES:
            raise ValueError(f"router score must be one of {sorted(ops.ROUTER_SCORES)}, got {self.score!r}")
        self.renormalise = bool(spec.get("renormalise", False))
        weight_on = str(spec.get("weight_on", "output"))
        if weight_on not in ("input", "output"):
            raise ValueError(f"weight_on must be input or output, got {weight_on!r}")
        self.weight_on_input = weight_on == "input"
        self.num_identity = int(spec.get("num_identity") or 0)
        self.num_outputs = self.num_experts + self.num_identity
        if not 0 < self.top_k <= self.num_outputs:
            raise ValueError(f"top_k {self.top_k} of {self.num_outputs} router outputs")
        if self.num_identity and self.weight_on_input:
            raise ValueError("experts that hand their input through take their weight on the output")
        self.groups = None
        if spec.get("groups"):
            self.groups = (int(spec["groups"]["count"]), int(spec["groups"]["keep"]))
            count, keep = self.groups
            if count <= 0 or self.num_outputs % count or not 0 < keep <= count or \
                    self.top_k > keep * (self.num_outputs // count):
                raise ValueError(f"{self.num_outputs} router outputs in {count} groups of which {keep} are kept "
                                 f"cannot give {self.top_k} choices")
        self.correction = runtime.vector(tensors["router.correction"]) if spec.get("correction") else None
        self.shared_size = int(spec.get("shared") or 0)
        self.shared_gated = bool(self.shared_size and spec.get("shared_gate"))
        router_rows = [tensors["router.weight"]]
        if self.shared_gated:
            router_rows.append(tensors["shared.gate.weight"])
        if len({m.dtype for m in router_rows}) > 1:
            router_rows = [m.to(torch.float32) for m in router_rows]
        # the shared expert's gate is one more row of the router's product
        self.router_weight = runtime.matrix(torch.cat(router_rows, dim=0))
        if self.shared_size:
            self.shared_gate_up = runtime.matrix(torch.cat(
                [tensors["shared.gate_proj.weight"], tensors["shared.up_proj.weight"]], dim=0))
            self.shared_down = runtime.matrix(tensors["shared.down_proj.weight"])
        names = range(self.num_experts)
        self.gate_up_weight = runtime.matrix(torch.stack([
            torch.cat([tensors[f"experts.{e}.gate_proj.weight"], tensors[f"experts.{e}.up_proj.weight"]], dim=0)
            for e in names
        ]))
        self.down_weight = runtime.matrix(torch.stack([tensors[f"experts.{e}.down_proj.weight"] for e in names]))

    def forward(self, x, ctx, add=None):
        tokens = x.shape[0]
        dtype, device = self.runtime.dtype, x.device
        experts, top_k = self.num_experts, self.top_k
        logits = ops.project(x, self.router_weight, ctx.status, out_dtype=torch.float32)   # [T, E], or partial sums
        expert_ids = torch.empty((tokens, top_k), dtype=torch.int32, device=device)
        weights = torch.empty((tokens, top_k), dtype=torch.float32, device=device)
        ops.router_topk(logits, top_k, self.score, self.renormalise, expert_ids, weights, self.num_outputs,
                        self.correction, self.groups)
        addend_gate = None
        if self.shared_size:
            if add is not None:
                raise ValueError("a routed feed-forward with a shared expert takes no other addend")
            gate_up = ops.project(x, self.shared_gate_up, ctx.status)
            inner = torch.empty((tokens, self.shared_size), dtype=dtype, device=device)
            ops.silu_mul(gate_up, inner)
            add = ops.project(inner, self.shared_down, ctx.status)      # [T, hidden], or partial sums
            if self.shared_gated:
                addend_gate = (logits, self.num_outputs)
        work = torch.empty((3 * experts + 1,), dtype=torch.int32, device=device)
        place = torch.empty((tokens, top_k), dtype=torch.int32, device=device)
        rows = tokens * top_k
        sorted_x = torch.empty((rows, self.hidden_size), dtype=dtype, device=device)
        offsets = ops.moe_dispatch(x, expert_ids, weights, experts, self.weight_on_input, work, place, sorted_x)
        gate_up = torch.empty((rows, 2 * self.intermediate_size), dtype=dtype, device=device)
        ops.moe_gemm(sorted_x, self.gate_up_weight, offsets, gate_up, ctx.status)
        hidden = torch.empty((rows, self.intermediate_size), dtype=dtype, device=device)
        ops.silu_mul(gate_up, hidden)
        splits = 1
        if ops.moe_gemm_on_tensor_cores(hidden, self.down_weight):
            splits = ops.moe_gemm_splits(rows, experts, self.hidden_size, self.intermediate_size)
        if splits > 1:      # a few rows against a matrix of few row tiles: K is cut, the combine adds up
            y = torch.empty((splits, rows, self.hidden_size), dtype=torch.float32, device=device)
        else:
            y = torch.empty((rows, self.hidden_size), dtype=dtype, device=device)
        ops.moe_gemm(hidden, self.down_weight, offsets, y, ctx.status)
        out = torch.empty((tokens, self.hidden_size), dtype=torch.float32, device=device)
        ops.moe_combine(y, expert_ids, place, weights, not self.weight_on_input, add, out, experts,
                        identity_input=x if self.num_identity else None, num_identity=self.num_identity,
                        addend_gate=addend_gate)
        return out
