"""Grouped-query attention over the paged cache.

One matrix product for Q, K and V on the concatenated weight
(``src/einf/executors/torch/packed_qkv.py:70-107,135-153``); bias, position
encoding and the cache write in one kernel; every token of the step attends to
the keys of its own request through the block table, so a prompt portion sees
itself through the cache (``qwen.py:405-411``); query head ``h`` uses key/value
head ``h // (heads / kv_heads)``; scores are scaled by ``scale`` and masked
lower-right causal (``model_runner.py:145``), optionally to the last ``window``
keys; then the output projection (``qwen.py:360,489``).

Optional, each from the spec: heads of unit root mean square, a soft cap on the scores, a chunked
mask, keys of another layer, values of another size than keys, a window that also keeps the first
``keep_first`` positions of the sequence, a rotation with neighbouring dimensions paired, and
``value_mix``: the first such layer of a model ("source") leaves its values of the step in
``ctx.extras``, every later one ("blend") caches ``(1 - m) v + m v_source`` with its stored scalar.

A layer may also mix its heads' scores before the softmax.  ``distance_slopes`` (one number per
head) takes ``slope_h (i - j)`` off the score of query i and key j; ``talking_heads`` then replaces
the heads' scores by ``sum_g talk[h, g] score_g`` (a stored matrix over all query heads, whatever
their key/value head); ``sink`` puts ``exp(sink_h)`` of a stored number per head into the softmax's
denominator, with no key and no value; ``output_scale`` multiplies the mixed values before they are
rounded for the output projection.  A layer with slopes or a mixing matrix runs a kernel of its
own, which computes all heads of a query together (``ops.paged_attention_mixed``); a sink alone is
taken by the general kernels.

``qk_norm_weight`` (with ``qk_unit_eps``): the normalised queries and keys are multiplied by stored
weights before any rotation: ``"head"``, one weight of the head's size for all query heads and one
for all key heads; ``"row"``, weights over all heads, and the root mean square is taken over the
whole projection at once instead of head by head.  ``values: "keys"``: the layer has no value
projection; a token's values are its keys as projected, before norm and rotation.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.specs import TensorSpec
from .base import CacheView, Mixer, PagedKVNeed, StepContext, build_nested, register_part


@register_part("mixer", "attention")
class PagedAttention(Mixer):
    @classmethod
    def tensor_specs(cls, spec):
        hidden, heads, kv_heads, size = (
            spec["hidden_size"], spec["num_heads"], spec["num_kv_heads"], spec["head_size"],
        )
        value_size = spec.get("value_head_size") or size
        own_kv = not spec.get("shared_kv", False)
        specs = {"q_proj.weight": TensorSpec((heads * size, hidden))}
        if own_kv:
            specs["k_proj.weight"] = TensorSpec((kv_heads * size, hidden))
            if spec.get("values", "projected") != "keys":
                specs["v_proj.weight"] = TensorSpec((kv_heads * value_size, hidden))
        if spec.get("qk_norm_weight"):
            rows = spec["qk_norm_weight"] == "row"
            specs["q_norm.weight"] = TensorSpec((heads * size if rows else size,), "scale")
            if own_kv:
                specs["k_norm.weight"] = TensorSpec((kv_heads * size if rows else size,), "scale")
        specs["o_proj.weight"] = TensorSpec((hidden, heads * value_size))
        if spec.get("qkv_bias", False):
            specs["q_proj.bias"] = TensorSpec((heads * size,), "bias")
            if own_kv:
                specs["k_proj.bias"] = TensorSpec((kv_heads * size,), "bias")
                specs["v_proj.bias"] = TensorSpec((kv_heads * value_size,), "bias")
        if spec.get("out_bias", False):
            specs["o_proj.bias"] = TensorSpec((hidden,), "bias")
        if spec.get("value_mix"):
            specs["value_mix"] = TensorSpec((), "fraction")   # stored by the source layer too, unused there
        if spec.get("talking_heads"):
            specs["talk"] = TensorSpec((heads, heads), "near_identity")
        if spec.get("sink"):
            specs["sink"] = TensorSpec((heads,), "bias")
        return specs

    @staticmethod
    def _mixes_scores(spec) -> bool:
        """Whether the heads' scores meet before the softmax (a kernel of its own computes them)."""
        return bool(spec.get("distance_slopes") or spec.get("talking_heads"))

    @staticmethod
    def _is_general(spec) -> bool:
        """Whether the layer asks for something only the general kernels compute."""
        return bool(
            spec.get("qk_unit_eps") is not None or spec.get("softcap") or spec.get("chunk")
            or spec.get("shared_kv", False)
            or (spec.get("value_head_size") or spec["head_size"]) != spec["head_size"]
            or spec.get("keep_first") or spec.get("value_mix")
            or spec["position"].get("layout", "halves") != "halves"
            or PagedAttention._mixes_scores(spec) or spec.get("output_scale") is not None
            or spec.get("sink") or spec.get("values", "projected") != "projected"
        )

    @staticmethod
    def _general_on_tensor_cores(spec, dtype) -> bool:
        """A general layer still runs the tcgen05 attention kernels (which know the chunked mask and
        the soft cap) when its keys and values have one size that those kernels take."""
        size = int(spec["head_size"])
        return dtype == torch.bfloat16 and (spec.get("value_head_size") or size) == size and size in (64, 128)

    @classmethod
    def kernel_libraries(cls, spec, runtime):
        if cls._mixes_scores(spec):
            tiled = ()
            if int(spec["num_heads"]) <= ops.MIXED_MAX_HEADS:
                tiled = ("attention_mixed_tiled:" + ops.mixed_tiled_variant(int(spec["num_heads"])),)
            return ("pointwise", "attention_mixed", "gemm_simt") + tiled + cls._product_libraries(runtime)
        if cls._is_general(spec):
            fast = (f"attention_tcgen05:HEAD_SIZE={int(spec['head_size'])}",) \
                if cls._general_on_tensor_cores(spec, runtime.dtype) else ()
            return ("pointwise", "attention_generic", "gemm_simt") + cls._product_libraries(runtime) + fast
        if ops.has_fast_attention(runtime.dtype, int(spec["head_size"])):
            # the page size is the engine's choice: ask for both prefill kernels of this head size
            libraries = ops.attention_libraries(int(spec["head_size"]), 16)
            return ("pointwise", "gemm_simt", "gemm_tcgen05") + libraries
        return ("pointwise", "attention_generic", "gemm_simt") + cls._product_libraries(runtime)

    @staticmethod
    def _product_libraries(runtime):
        return ("gemm_tcgen05",) if runtime.dtype == torch.bfloat16 else ()

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.hidden_size = int(spec["hidden_size"])
        self.num_heads = int(spec["num_heads"])
        self.num_kv_heads = int(spec["num_kv_heads"])
        self.head_size = int(spec["head_size"])
        self.scale = float(spec["scale"])
        self.window = spec.get("window")
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"{self.num_heads} heads are not a multiple of {self.num_kv_heads} key/value heads")
        self.value_size = int(spec.get("value_head_size") or self.head_size)
        self.qk_unit_eps = None if spec.get("qk_unit_eps") is None else float(spec["qk_unit_eps"])
        self.softcap = float(spec["softcap"]) if spec.get("softcap") else None
        self.chunk = int(spec["chunk"]) if spec.get("chunk") else None
        self.shared_kv = bool(spec.get("shared_kv", False))
        self.general = self._is_general(spec)
        if self.general:
            if max(self.head_size, self.value_size) > ops.MAX_HEAD_SIZE:
                raise ops.UnsupportedSize(
                    f"head sizes {self.head_size}, {self.value_size}: the attention kernels take up to {ops.MAX_HEAD_SIZE}"
                )
            if spec["position"].kind not in ("none", "rope"):
                raise ValueError(
                    "the general attention layer rotates or leaves its heads as they are; it does not know the "
                    f"position encoding {spec['position'].kind!r}"
                )
        elif self.head_size % 16 or self.head_size > ops.MAX_HEAD_SIZE:
            raise ops.UnsupportedSize(
                f"head size {self.head_size}: the attention kernels take multiples of 16 up to {ops.MAX_HEAD_SIZE}"
            )
        if self.window is not None and self.window <= 0:
            raise ValueError(f"window must be positive, got {self.window}")
        if self.chunk is not None and self.chunk <= 0:
            raise ValueError(f"chunk must be positive, got {self.chunk}")
        self.values_from_keys = spec.get("values", "projected") == "keys"
        if spec.get("values", "projected") not in ("projected", "keys"):
            raise ValueError(f"values must be projected or keys, got {spec.get('values')!r}")
        if self.values_from_keys and (self.shared_kv or self.value_size != self.head_size or spec.get("value_mix")
                                      or spec.get("qkv_bias", False)):
            raise ValueError("a layer whose values are its keys has keys of its own, of the values' size, unmixed, no bias")
        self.qk_norm_weight = spec.get("qk_norm_weight")
        if self.qk_norm_weight not in (None, "head", "row"):
            raise ValueError(f"qk_norm_weight must be head or row, got {self.qk_norm_weight!r}")
        if self.qk_norm_weight and self.qk_unit_eps is None:
            raise ValueError("qk_norm_weight needs qk_unit_eps")
        self.q_norm_weight = self.k_norm_weight = None
        if self.qk_norm_weight:
            self.q_norm_weight = runtime.vector(tensors["q_norm.weight"])
            if not self.shared_kv:
                self.k_norm_weight = runtime.vector(tensors["k_norm.weight"])
        if self.shared_kv:
            names = ["q_proj"]
        elif self.values_from_keys:
            names = ["q_proj", "k_proj"]
        else:
            names = ["q_proj", "k_proj", "v_proj"]
        matrices = [tensors[n + ".weight"] for n in names]
        if len({m.dtype for m in matrices}) > 1:
            matrices = [m.to(torch.float32) for m in matrices]
        self.qkv_weight = runtime.matrix(torch.cat(matrices, dim=0))
        self.qkv_bias = None
        if spec.get("qkv_bias", False):
            self.qkv_bias = runtime.vector(torch.cat([tensors[n + ".bias"].float() for n in names]))
        self.out_weight = runtime.matrix(tensors["o_proj.weight"])
        self.out_bias = runtime.vector(tensors["o_proj.bias"]) if spec.get("out_bias", False) else None
        self.position = build_nested("position", spec["position"], tensors, runtime)
        self.keep_first = int(spec.get("keep_first") or 0)
        if self.keep_first and self.window is None:
            raise ValueError("keep_first needs a window")
        self.value_mix = spec.get("value_mix")
        if self.value_mix not in (None, "source", "blend"):
            raise ValueError(f"value_mix must be source or blend, got {self.value_mix!r}")
        self.mix = runtime.vector(tensors["value_mix"].reshape(1)) if self.value_mix else None
        self.mixes_scores = self._mixes_scores(spec)
        self.output_scale = float(spec["output_scale"]) if spec.get("output_scale") is not None else 1.0
        self.slopes = self.talk = self.sink = None
        if self.mixes_scores:
            if self.softcap or self.chunk or self.keep_first or self.shared_kv:
                raise ValueError("a layer that mixes its heads' scores has no soft cap, chunks, kept positions or shared keys")
            if self.num_heads > ops.MIXED_MAX_HEADS:
                raise ops.UnsupportedSize(f"{self.num_heads} heads: the score-mixing kernel takes up to {ops.MIXED_MAX_HEADS}")
            if spec.get("distance_slopes"):
                slopes = [float(v) for v in spec["distance_slopes"]]
                if len(slopes) != self.num_heads:
                    raise ValueError(f"{len(slopes)} distance slopes for {self.num_heads} heads")
                self.slopes = torch.tensor(slopes, dtype=torch.float64).to(torch.float32).to(runtime.device)
            if spec.get("talking_heads"):
                self.talk = runtime.vector(tensors["talk"])
            if self.qk_norm_weight or self.values_from_keys:
                raise ValueError("a layer that mixes its heads' scores has no weighted norm and values of its own")
        elif self.output_scale != 1.0:
            raise ValueError("output_scale is applied by the score-mixing kernel only")
        if spec.get("sink"):
            if self.softcap or self.chunk or self.keep_first:
                raise ValueError("a sink comes without a soft cap, chunks or kept positions")
            self.sink = runtime.vector(tensors["sink"])
        self.fast = not self.general and ops.has_fast_attention(runtime.dtype, self.head_size)
        self.general_fast = self.general and not self.mixes_scores and self._general_on_tensor_cores(spec, runtime.dtype)

    def cache_need(self):
        value = self.value_size if self.value_size != self.head_size else None
        return PagedKVNeed(self.num_kv_heads, self.head_size, self.window, value, self.keep_first)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        tokens = x.shape[0]
        dtype, device = self.runtime.dtype, x.device
        qkv = ops.project(x, self.qkv_weight, ctx.status)   # [T, width], or split-K partial sums
        q = torch.empty((tokens, self.num_heads, self.head_size), dtype=dtype, device=device)
        if self.general:
            writes = cache.writes and cache.k is not None and not self.shared_kv
            shared_values = None
            if self.value_mix == "source":
                shared_values = torch.empty((tokens, self.num_kv_heads * self.value_size), dtype=torch.float32,
                                            device=device)
                ctx.extras["mixed_values"] = shared_values
            elif self.value_mix == "blend":
                shared_values = ctx.extras.get("mixed_values")
                if shared_values is None:
                    raise RuntimeError("a layer blends its values before any layer of the step has left its own")
            ops.qkv_norm_store(
                qkv, self.qkv_bias, ctx.slots[cache.group] if writes else None, q,
                cache.k if writes else None, cache.v if writes else None, self.num_heads,
                0 if self.shared_kv else self.num_kv_heads, self.head_size, self.value_size, self.qk_unit_eps,
                ctx.status, positions=ctx.positions, inv_freq=self.position.inv_freq,
                interleaved=getattr(self.position, "interleaved", False), value_mix=self.value_mix,
                shared_values=shared_values, mix=self.mix, q_norm_weight=self.q_norm_weight,
                k_norm_weight=self.k_norm_weight, norm_rows=self.qk_norm_weight == "row",
                values_from_keys=self.values_from_keys,
            )
        else:
            self.position.encode_and_store(
                qkv, self.qkv_bias, ctx, cache, q, self.num_heads, self.num_kv_heads, self.head_size
            )
        mixed = torch.empty((tokens, self.num_heads, self.value_size), dtype=dtype, device=device)
        self.attend(q, ctx, cache, mixed)
        if self.out_bias is None:
            return ops.project(mixed.view(tokens, -1), self.out_weight, ctx.status)
        out = torch.empty((tokens, self.hidden_size), dtype=dtype, device=device)
        ops.linear(mixed.view(tokens, -1), self.out_weight, self.out_bias, out)
        return out

    def launch_key(self, ctx: StepContext, page_size: int) -> tuple:
        """The decode attention cuts a token's keys by the number of single tokens and the bucket
        of the longest context: kernel, cluster size and clusters per token."""
        singles = int(ctx.single_tokens.shape[0])
        if self.mixes_scores:
            # the tiled kernel splits the keys of single tokens by their number and the longest context
            return ("mixed", ops.mixed_tiled_splits(singles, 1, self.window, ctx.max_context_len)) if singles else ()
        if not (self.fast or (self.general_fast and ops.has_tcgen05_attention(self.head_size, page_size))) or not singles:
            return ()
        context = ctx.max_context_len
        for bound in (self.window, self.chunk):
            if bound:
                context = min(context, bound)
        return ops.decode_plan(singles, self.num_heads, self.num_kv_heads, self.head_size, page_size, context)

    def launch_group(self):
        return ("attention", self.num_heads, self.num_kv_heads, self.head_size, self.window, self.fast, self.general,
                self.mixes_scores)

    def attend(self, q, ctx: StepContext, cache: CacheView, out) -> None:
        """bfloat16 with a head size up to 128 (a layer with a chunked mask, a soft cap or unit-norm
        heads: head sizes 64 and 128 with values as large as keys): the tensor-core kernels, cluster decode for the
        requests that bring one token, tiled prefill for the others, side by side in a mixed batch.  Everything else (the 32-bit path,
        larger heads): the generic kernel."""
        table = ctx.block_tables[cache.group]
        if self.mixes_scores:
            ops.paged_attention_mixed(
                q, cache.k, cache.v, table, ctx.seq_of_token, ctx.positions, out, self.scale, self.window,
                self.slopes, self.talk, self.sink, self.output_scale, ctx.status,
                q_tiles=ctx.q_tiles, single_tokens=None if ctx.decode_only else ctx.single_tokens,
                num_singles=int(ctx.single_tokens.shape[0]), max_context=ctx.max_context_len,
            )
            return
        if self.fast or (self.general_fast and ops.has_tcgen05_attention(self.head_size, cache.k.shape[2])):
            singles = ctx.single_tokens.shape[0]
            if singles:
                ops.paged_decode_attention_auto(
                    q, cache.k, cache.v, table, ctx.seq_of_token, ctx.positions, out, self.scale,
                    self.window, ctx.status, None if ctx.decode_only else ctx.single_tokens,
                    max_context=ctx.max_context_len, chunk=self.chunk, softcap=self.softcap,
                    keep_first=self.keep_first, sink=self.sink,
                )
            if ctx.q_tiles.shape[0]:
                ops.paged_prefill_attention(
                    q, cache.k, cache.v, table, ctx.q_tiles, out, self.scale, self.window, ctx.status,
                    cached_before=ctx.max_portion_start, chunk=self.chunk, softcap=self.softcap,
                    keep_first=self.keep_first, sink=self.sink,
                )
            return
        ops.paged_attention_generic(
            q, cache.k, cache.v, ctx.block_tables[cache.group], ctx.seq_of_token, ctx.positions,
            out, self.scale, self.window, ctx.status, chunk=self.chunk, softcap=self.softcap,
            keep_first=self.keep_first, sink=self.sink,
        )
