"""Python entry points of the hand-written sm_100a kernels.

Every function takes CUDA tensors, checks what the kernel assumes (dtype,
contiguity, the sizes it can take) and launches on the current stream.  There
is no other backend: a tensor that is not on a CUDA device, a size a kernel
cannot take, or a kernel library that cannot be built raises an error.

The plain PyTorch statement of each function lives beside the tests
(``tests/kernel_references.py``), where it is compared with the kernel.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional, Tuple

import torch

from . import _library
from ._library import KernelLibraryError, ensure_built

FLOAT32, BFLOAT16 = 0, 1
_DTYPE_CODES = {torch.float32: FLOAT32, torch.bfloat16: BFLOAT16}

STATUS_BAD_TOKEN = 1
STATUS_BAD_PAGE = 2
STATUS_WAIT_EXPIRED = 4

MAX_HEAD_SIZE = 256
#: the general attention kernel alone takes larger heads (a latent cache row)
MAX_GENERIC_HEAD_SIZE = 640


class KernelError(RuntimeError):
    """A launch returned a CUDA error."""


class UnsupportedSize(ValueError):
    """A kernel was asked for a size it does not take."""


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODES[t.dtype]
    except KeyError:
        raise TypeError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}") from None


def _dev(t: torch.Tensor, name: str) -> int:
    if not t.is_cuda:
        raise KernelError(
            f"{name} is on {t.device}: the kernels run on a CUDA device only and have no CPU path"
        )
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t.data_ptr()


def _opt(t: Optional[torch.Tensor], name: str, dtype: torch.dtype) -> int:
    if t is None:
        return 0
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    return _dev(t, name)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  Asked for at every launch, so by the short road where torch
    has one (the public ``current_stream()`` builds an object: 7 us, more than a launch costs)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


_stream_objects: dict[tuple[int, int], "torch.cuda.Stream"] = {}


def current_stream() -> "torch.cuda.Stream":
    """The current stream as an object (for events and synchronisation), cached per handle."""
    if _raw_stream is None:
        return torch.cuda.current_stream()
    device = torch.cuda.current_device()
    handle = _raw_stream(device)
    stream = _stream_objects.get((device, handle))
    if stream is None:
        stream = torch.cuda.current_stream()
        _stream_objects[(device, handle)] = stream
    return stream


#: launches of this package's own kernels since import (library matrix products are not counted)
launch_count = 0


def _check(code: int, what: str) -> None:
    global launch_count
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code}")
    launch_count += 1


_bound: dict[str, object] = {}


def _fn(symbol: str, argtypes, variant: str = ""):
    function = _bound.get((symbol, variant))
    if function is None:
        function = _library.launcher(symbol, argtypes, variant)
        _bound[(symbol, variant)] = function
    return function


# ---------------------------------------------------------------------------
def embed(tokens: torch.Tensor, table: torch.Tensor, residual: torch.Tensor, status: torch.Tensor,
          positions: Optional[torch.Tensor] = None, position_table: Optional[torch.Tensor] = None,
          scale: float = 1.0) -> None:
    """``residual[t] = scale * table[tokens[t]]`` as float (the product in 32-bit); a token outside the
    table sets the status word.
    With ``position_table [max_positions, hidden]`` (the table's dtype) the row ``position_table[positions[t]]``
    is added in 32-bit, unscaled; a position beyond it sets the status word too."""
    vocab, hidden = table.shape
    max_positions, pos_ptr, table_ptr = 0, 0, 0
    if position_table is not None:
        if positions is None or position_table.dtype != table.dtype or position_table.shape[1] != hidden:
            raise ValueError("a position table needs positions, the embedding's dtype and its width")
        max_positions = position_table.shape[0]
        pos_ptr, table_ptr = _opt(positions, "positions", torch.int32), _dev(position_table, "position_table")
    if tokens.dtype != torch.int32 or residual.dtype != torch.float32:
        raise TypeError("embed takes int32 tokens and a float32 residual")
    if residual.shape != (tokens.shape[0], hidden):
        raise ValueError(f"residual is {tuple(residual.shape)}, expected {(tokens.shape[0], hidden)}")
    fn = _fn("einf_embed", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                            c_int, c_float, c_void_p])
    _check(
        fn(_dev(tokens, "tokens"), _dev(table, "table"), _code(table), _dev(residual, "residual"),
           tokens.shape[0], hidden, vocab, _dev(status, "status"), pos_ptr, table_ptr, max_positions, float(scale),
           _stream()),
        "embed",
    )


def add_rmsnorm(
    x: Optional[torch.Tensor],
    residual: torch.Tensor,
    weight: torch.Tensor,
    eps: float,
    out: torch.Tensor,
    rows: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
) -> None:
    """``residual += x`` (summing a leading split dimension of ``x`` if it has one), then
    ``out = weight * residual * rsqrt(mean(residual^2) + eps)``.

    ``x`` may be None.  With ``rows`` (int32 indices), ``out[r]`` is computed from
    row ``rows[r]`` and the residual is not written.  With ``status`` (the step's status word) a
    handful of rows of split-K partial sums may take the kernel that fetches them by TMA, whose
    bounded wait reports there.
    """
    hidden = residual.shape[-1]
    if residual.dtype != torch.float32 or weight.dtype != torch.float32:
        raise TypeError("the residual stream and norm weights are float32")
    if weight.shape != (hidden,):
        raise ValueError(f"norm weight is {tuple(weight.shape)}, expected {(hidden,)}")
    if hidden > 50_000:
        raise UnsupportedSize(f"add_rmsnorm keeps a row in shared memory; width {hidden} > 50000")
    splits, stride, x_code, x_ptr = 1, 0, FLOAT32, 0
    if x is not None:
        if x.dim() == 3:
            splits, stride = x.shape[0], x.shape[1] * x.shape[2]
        if x.shape[-2:] != residual.shape:
            raise ValueError(f"x is {tuple(x.shape)}, residual {tuple(residual.shape)}")
        x_code, x_ptr = _code(x), _dev(x, "x")
    num_rows = rows.shape[0] if rows is not None else residual.shape[0]
    if out.shape != (num_rows, hidden):
        raise ValueError(f"out is {tuple(out.shape)}, expected {(num_rows, hidden)}")
    fn = _fn(
        "einf_add_rmsnorm",
        [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_float, c_void_p, c_int, c_void_p,
         c_int, c_int, c_int, c_void_p, c_void_p],
    )
    _check(
        fn(x_ptr, x_code, splits, stride, _dev(residual, "residual"), _dev(weight, "weight"), float(eps),
           _dev(out, "out"), _code(out), _opt(rows, "rows", torch.int32), num_rows, hidden,
           0 if rows is not None else 1, _opt(status, "status", torch.int32), _stream()),
        "add_rmsnorm",
    )


ADVANCE_MAX_GROUPS = 4


def advance_decode(
    token_ids: torch.Tensor,
    positions: torch.Tensor,
    context_lens: torch.Tensor,
    sampled: torch.Tensor,
    slots: list,
    block_tables: list,
    page_size: int,
) -> None:
    """One decode step on, in place, for a step of single tokens: ``token_ids[i] = sampled[i]`` for
    the first ``len(sampled)`` requests, ``positions += 1``, ``context_lens += 1`` and, per cache
    group, ``slots[i] = table[i, position // page] * page + position % page``.  Requests beyond
    ``sampled`` (padding of a graph bucket) and requests that write nothing keep what they have."""
    groups = len(slots)
    if groups > ADVANCE_MAX_GROUPS or groups != len(block_tables):
        raise UnsupportedSize(f"advance_decode takes up to {ADVANCE_MAX_GROUPS} cache groups")
    pointers = []
    for g in range(ADVANCE_MAX_GROUPS):
        if g < groups:
            pointers += [_opt(slots[g], "slots", torch.int32), _opt(block_tables[g], "block_table", torch.int32)]
        else:
            pointers += [0, 0]
    width = block_tables[0].shape[1] if groups else 0
    fn = _fn("einf_advance_decode", [c_void_p] * 4 + [c_int] + [c_void_p] * 8 + [c_int, c_int, c_int, c_void_p])
    _check(
        fn(_opt(token_ids, "token_ids", torch.int32), _opt(positions, "positions", torch.int32),
           _opt(context_lens, "context_lens", torch.int32), _opt(sampled, "sampled", torch.int32), sampled.shape[0],
           *pointers, groups, width, int(page_size), _stream()),
        "advance_decode",
    )


def zero_fresh_state(state: torch.Tensor, state_slots: torch.Tensor, q_start: torch.Tensor,
                     positions: torch.Tensor) -> None:
    """``state[state_slots[r]] = 0`` for every request ``r`` of the step whose first token stands at
    position 0 (``positions[q_start[r]] == 0``); requests without a slot (-1) are skipped.  ``state``
    is ``[slots, ...]`` of any dtype; the index tensors are the step's own inputs, so the launch
    can be captured in a CUDA graph."""
    num_requests = state_slots.shape[0]
    if q_start.shape[0] != num_requests + 1:
        raise ValueError("q_start must hold one more entry than state_slots")
    num_slots = state.shape[0]
    row_bytes = (state.numel() // num_slots) * state.element_size() if num_slots else 0
    fn = _fn("einf_zero_fresh_state", [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(
        fn(_dev(state, "state"), row_bytes, num_slots, _opt(state_slots, "state_slots", torch.int32),
           _opt(q_start, "q_start", torch.int32), _opt(positions, "positions", torch.int32), num_requests, _stream()),
        "zero_fresh_state",
    )


def _maybe_split(x: torch.Tensor, rows: int, width: int, name: str) -> tuple[int, int]:
    """``x`` is ``[rows, width]``, or float32 partial sums ``[splits, rows, width]``: (splits, stride)."""
    if x.dim() == 3:
        if x.dtype != torch.float32 or x.shape[1:] != (rows, width):
            raise ValueError(f"{name}: partial sums must be float32 [splits, {rows}, {width}], got {tuple(x.shape)}")
        return x.shape[0], rows * width
    if x.shape != (rows, width):
        raise ValueError(f"{name} is {tuple(x.shape)}, expected {(rows, width)}")
    return 1, 0


def rope_kv_write(
    qkv: torch.Tensor,
    bias: Optional[torch.Tensor],
    positions: torch.Tensor,
    inv_freq: torch.Tensor,
    slots: Optional[torch.Tensor],
    q_out: torch.Tensor,
    k_cache: Optional[torch.Tensor],
    v_cache: Optional[torch.Tensor],
    num_heads: int,
    num_kv_heads: int,
    head_size: int,
    status: torch.Tensor,
) -> None:
    """Add the QKV bias, rotate Q and K by their positions, write Q to ``q_out`` and
    K, V into the pages at ``slots``.  ``qkv`` is ``[tokens, width]``, or the float32 partial
    sums ``[splits, tokens, width]`` of a split-K product.  Caches are
    ``[pages, kv_heads, page_size, head_size]``; ``slots`` None (with no caches) computes Q only."""
    tokens = qkv.shape[-2]
    width = (num_heads + 2 * num_kv_heads) * head_size
    splits, stride = _maybe_split(qkv, tokens, width, "qkv")
    rotary_dim = 2 * inv_freq.shape[0]
    if rotary_dim > head_size or inv_freq.dtype != torch.float32:
        raise ValueError("inv_freq must be float32 with at most head_size / 2 entries")
    if q_out.numel() != tokens * num_heads * head_size:
        raise ValueError("q_out must hold [tokens, heads, head_size]")
    page_size = num_pages = 0
    k_ptr = v_ptr = 0
    if slots is not None:
        if k_cache is None or v_cache is None:
            raise ValueError("slots given without caches")
        num_pages, kvh, page_size, size = k_cache.shape
        if (kvh, size) != (num_kv_heads, head_size) or v_cache.shape != k_cache.shape:
            raise ValueError(f"cache is {tuple(k_cache.shape)}, expected [pages, {num_kv_heads}, page, {head_size}]")
        if k_cache.dtype != q_out.dtype or v_cache.dtype != q_out.dtype:
            raise TypeError("cache dtype differs from q_out")
        k_ptr, v_ptr = _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache")
    fn = _fn(
        "einf_rope_kv_write",
        [c_void_p, c_int, c_int, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    )
    _check(
        fn(_dev(qkv, "qkv"), _code(qkv), splits, stride, _code(q_out), _opt(bias, "bias", torch.float32),
           _opt(positions, "positions", torch.int32), _dev(inv_freq, "inv_freq"),
           _opt(slots, "slots", torch.int32), _dev(q_out, "q_out"), k_ptr, v_ptr, tokens, num_heads,
           num_kv_heads, head_size, rotary_dim, page_size, num_pages, _dev(status, "status"), _stream()),
        "rope_kv_write",
    )


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """``out = silu(gate_up[:, :I]) * gate_up[:, I:]``; ``gate_up`` may be float32 partial sums
    ``[splits, tokens, 2 I]`` of a split-K product."""
    tokens, inter = out.shape
    splits, stride = _maybe_split(gate_up, tokens, 2 * inter, "gate_up")
    fn = _fn("einf_silu_mul", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_longlong, c_int, c_void_p])
    _check(
        fn(_dev(gate_up, "gate_up"), _code(gate_up), splits, stride, _dev(out, "out"), _code(out), tokens, inter,
           _stream()),
        "silu_mul",
    )


#: activations of a gated feed-forward's gate branch (``silu`` has launches of its own, :func:`silu_mul`)
GATE_ACTIVATIONS = {"silu": 2, "gelu_tanh": 1}


def act_mul(gate_up: torch.Tensor, out: torch.Tensor, kind: str) -> None:
    """``out = act(gate_up[:, :I]) * gate_up[:, I:]`` with ``act`` one of :data:`GATE_ACTIVATIONS`;
    ``gate_up`` may be float32 partial sums ``[splits, tokens, 2 I]`` of a split-K product."""
    tokens, inter = out.shape
    splits, stride = _maybe_split(gate_up, tokens, 2 * inter, "gate_up")
    if kind not in GATE_ACTIVATIONS:
        raise ValueError(f"unknown gate activation {kind!r}; known: {sorted(GATE_ACTIVATIONS)}")
    fn = _fn("einf_act_mul", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_longlong, c_int, c_int, c_void_p])
    _check(
        fn(_dev(gate_up, "gate_up"), _code(gate_up), splits, stride, _dev(out, "out"), _code(out), tokens, inter,
           GATE_ACTIVATIONS[kind], _stream()),
        "act_mul",
    )


def gemm_simt(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """``out = x @ weight.T (+ bias)`` with 32-bit FMA accumulation; x rows may be strided."""
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape != (n, k) or out.shape != (m, n):
        raise ValueError(f"gemm: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if x.stride(1) != 1 or out.stride(1) != 1:
        raise ValueError("gemm operands must have unit stride in their last dimension")
    if not (x.is_cuda and out.is_cuda):
        raise KernelError("gemm operands must be on a CUDA device: there is no CPU path")
    fn = _fn(
        "einf_gemm_simt",
        [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong,
         c_longlong, c_void_p],
    )
    _check(
        fn(x.data_ptr(), _code(x), _dev(weight, "weight"), _code(weight), _opt(bias, "bias", torch.float32),
           out.data_ptr(), _code(out), m, n, k, x.stride(0), out.stride(0), _stream()),
        "gemm_simt",
    )


def tcgen05_takes(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the tensor-core kernel can take these operands (TMA needs 16-byte aligned rows)."""
    return (
        x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
        and x.stride(1) == 1 and weight.is_contiguous() and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
        and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
    )


def gemm_tcgen05_splits(k: int, splits: int) -> int:
    """The number of K ranges a request for ``splits`` really yields (no range is empty)."""
    fn = _fn("einf_gemm_tcgen05_splits", [c_int, c_int])
    return int(fn(k, splits))


def gemm_tcgen05(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    out: torch.Tensor,
    status: torch.Tensor,
    splits: int = 1,
) -> None:
    """``out = x @ weight.T (+ bias)`` on the tcgen05 tensor cores (bfloat16 operands, 32-bit
    accumulation).  ``out`` is ``[tokens, n]`` bfloat16 or float32; with ``splits`` > 1 it is
    float32 ``[splits, tokens, n]`` partial sums over K ranges, which the consumer adds up
    (``splits`` must then be what :func:`gemm_tcgen05_splits` returns)."""
    global launch_count
    tokens, k = x.shape
    n = weight.shape[0]
    if not tcgen05_takes(x, weight):
        raise UnsupportedSize(
            "gemm_tcgen05 takes bfloat16 operands whose rows are 16-byte aligned (K a multiple of 8)"
        )
    if weight.shape != (n, k):
        raise ValueError(f"weight is {tuple(weight.shape)}, expected {(n, k)}")
    if splits > 1:
        if out.dtype != torch.float32 or out.shape != (splits, tokens, n) or not out.is_contiguous():
            raise ValueError(f"split-K output must be contiguous float32 {(splits, tokens, n)}")
        if gemm_tcgen05_splits(k, splits) != splits:
            raise ValueError(f"K = {k} cannot be cut into {splits} non-empty ranges of 64-wide blocks")
        ldo = n
    else:
        if out.shape != (tokens, n) or out.stride(1) != 1:
            raise ValueError(f"out is {tuple(out.shape)}, expected {(tokens, n)}")
        ldo = out.stride(0)
    fn = _fn(
        "einf_gemm_tcgen05",
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_int,
         c_void_p, c_void_p],
    )
    if not x.is_cuda:
        raise KernelError("gemm operands must be on a CUDA device: there is no CPU path")
    _check(
        fn(x.data_ptr(), _dev(weight, "weight"), _opt(bias, "bias", torch.float32), out.data_ptr(), _code(out),
           tokens, n, k, x.stride(0), ldo, splits, _dev(status, "status"), _stream()),
        "gemm_tcgen05",
    )


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> None:
    rows, n = out.shape
    fn = _fn("einf_add_bias", [c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p])
    _check(fn(_dev(out, "out"), _code(out), _opt(bias, "bias", torch.float32), rows, n, _stream()), "add_bias")


def linear(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    out: torch.Tensor,
) -> None:
    """``out = x @ weight.T (+ bias)``.

    bfloat16 activations against a bfloat16 matrix go to the tensor cores through
    the library matrix product (as the reference's ``F.linear`` does,
    ``src/einf/executors/torch/packed_qkv.py:148``); everything else, the whole
    32-bit path included, runs the FMA kernel, which rounds no input.
    """
    if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.is_contiguous():
        if not x.is_cuda:
            raise KernelError("linear operands must be on a CUDA device: there is no CPU path")
        if out.dtype == torch.bfloat16:
            torch.mm(x, weight.t(), out=out)
        else:
            torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
        if bias is not None:
            add_bias(out, bias)
        return
    gemm_simt(x, weight, bias, out)


#: up to this many tokens every bfloat16 product runs on this package's tcgen05 kernel with split-K
#: that fills the GPU.  (Measured at 64 tokens, 0.5B sizes, kernel alone: QKV 2.9 against 3.8 us for
#: the library, O 2.7 against 3.3, down 4.3 against 8.8, gate/up 6.3 against 5.9; but with every
#: product cut 14 to 19 ways the consumers add up that many partial sums for 64 rows each, and
#: the step as a whole was slower: 1.63 against 1.57 ms.  See ``TCGEN05_MID_TOKENS``.)
TCGEN05_MAX_TOKENS = 32
#: K is cut at most this many ways: the consumers hold sixteen loads in flight, so up to sixteen partial
#: sums cost them one round trip to L2 and every further batch another (0.5B sizes, decode step at
#: 8 / 16 / 32 tokens: 0.807 / 0.935 / 1.175 ms with 16, 0.839 / 0.958 / 1.227 with 32 / 20 / 10,
#: 0.843 / 1.069 / 1.445 with 8 / 4 / 2).
MAX_SPLITS = 16


#: Between ``TCGEN05_MAX_TOKENS`` and this many tokens the tcgen05 kernel still takes the matrices
#: with few row tiles (at most ``MID_MAX_TILES`` of 128 rows: QKV, O and the down projection of the
#: small models, which as library products are grids of 7 to 9 CTAs), with K cut at most
#: ``MID_MAX_SPLITS`` ways; the gate/up matrix and the output matrix stay with the library.  Measured,
#: whole decode steps of 64 requests at contexts of 1,024 / 4,096 tokens: 0.5B sizes 1.116 -> 1.055 /
#: 1.505 -> 1.443 ms, 1.5B sizes 1.924 -> 1.762 / 2.773 -> 2.620 ms, 7B sizes 4.29 -> 4.15 / 5.85 ->
#: 5.74 ms (2 or 4 ways lose to the library, 16 ways lose to 12: the consumers' many rows).
TCGEN05_MID_TOKENS = 64
MID_MAX_TILES = 40
MID_MAX_SPLITS = 12


def _tcgen05_splits(tokens: int, n: int, k: int) -> int:
    """How many ways to split K, or 0 for the library product."""
    tiles = -(-n // 128)
    if tokens > TCGEN05_MAX_TOKENS:
        if tokens > TCGEN05_MID_TOKENS or tiles > MID_MAX_TILES:
            return 0
        return max(1, min(-(-_sm_count() // tiles), MID_MAX_SPLITS))
    slots = 2 * _sm_count()                     # two CTAs per SM
    fill = -(-slots // tiles)
    # A grid a little larger than one wave is fine while a CTA's share of the weights is small (at
    # 0.5B sizes more, shorter CTAs win: gate/up 4.6 us with 304 CTAs against 5.3 us with 228); when
    # it is hundreds of KB the few CTAs of a second wave cost a whole CTA's time (7B down projection:
    # 308 CTAs of 440 KB), so the grid then stays within the wave.
    if fill > 1 and fill * tiles > slots and 128 * k * 2 // fill > 64 * 1024:
        fill -= 1
    return max(1, min(fill, MAX_SPLITS))


def project(
    x: torch.Tensor,
    weight: torch.Tensor,
    status: torch.Tensor,
    out_dtype: Optional[torch.dtype] = None,
    allow_partial: bool = True,
) -> torch.Tensor:
    """``x @ weight.T`` for a consumer that can add up partial sums.

    Returns ``[tokens, n]`` in ``out_dtype`` (default: x's dtype), or, when the tcgen05 kernel
    splits K to fill the GPU at small token counts, float32 partial sums ``[splits, tokens, n]``
    which :func:`add_rmsnorm`, :func:`rope_kv_write` and :func:`silu_mul` add up themselves.
    """
    tokens, k = x.shape
    n = weight.shape[0]
    out_dtype = out_dtype or x.dtype
    splits = _tcgen05_splits(tokens, n, k) if tcgen05_takes(x, weight) else 0
    if splits and not allow_partial:
        splits = 1
    if splits:
        splits = gemm_tcgen05_splits(k, splits)
        if splits > 1:
            out = torch.empty((splits, tokens, n), dtype=torch.float32, device=x.device)
        else:
            out = torch.empty((tokens, n), dtype=out_dtype, device=x.device)
        gemm_tcgen05(x, weight, None, out, status, splits)
        return out
    out = torch.empty((tokens, n), dtype=out_dtype, device=x.device)
    linear(x, weight, None, out)
    return out


def paged_attention_generic(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: Optional[torch.Tensor],
    block_table: torch.Tensor,
    seq_of_token: torch.Tensor,
    positions: torch.Tensor,
    out: torch.Tensor,
    scale: float,
    window: Optional[int],
    status: torch.Tensor,
    chunk: Optional[int] = None,
    softcap: Optional[float] = None,
    keep_first: int = 0,
    values_in_keys: Optional[int] = None,
    sink: Optional[torch.Tensor] = None,
) -> None:
    """Causal attention of every token of the batch over the pages of its request.

    ``q`` is ``[tokens, heads, head_size]``, ``out`` ``[tokens, heads, value_size]``; the caches
    ``[pages, kv_heads, page_size, head_size]`` and ``[pages, kv_heads, page_size, value_size]``;
    ``block_table`` ``[requests, width]`` maps a request's logical page to a physical one.
    ``window``: only the last that many keys, and with ``keep_first`` n also the first n positions
    of the sequence; ``chunk``: only the keys of the token's own block of
    that many positions (blocks counted from position 0); ``softcap`` z: scores become
    ``z * tanh(score / z)`` before the softmax.  ``values_in_keys`` n (with ``v_cache`` None): a
    token's value is the first n elements of its key row (one cached row serves as both).
    ``sink`` (float32 ``[heads]``): the softmax's denominator of head h also holds ``exp(sink[h])``,
    unscaled, with no key and no value.
    """
    tokens, num_heads, head_size = q.shape
    if sink is not None and (sink.dtype != torch.float32 or sink.shape != (num_heads,)):
        raise ValueError(f"sink must be float32 [{num_heads}]")
    num_pages, num_kv_heads, page_size, size = k_cache.shape
    if values_in_keys is not None:
        if v_cache is not None or not 0 < values_in_keys <= size:
            raise ValueError("values_in_keys takes no value cache and at most the key size")
        v_cache, value_size, value_stride = k_cache, int(values_in_keys), size
    else:
        value_size = value_stride = v_cache.shape[3]
        if v_cache.shape[:3] != k_cache.shape[:3]:
            raise ValueError("key and value caches differ in pages, heads or page size")
    if size != head_size:
        raise ValueError("cache head size differs from q")
    if max(head_size, value_size) > MAX_GENERIC_HEAD_SIZE:
        raise UnsupportedSize(
            f"paged attention takes head sizes up to {MAX_GENERIC_HEAD_SIZE}, got {head_size}, {value_size}")
    if num_heads % num_kv_heads:
        raise UnsupportedSize(f"{num_heads} query heads are not a multiple of {num_kv_heads} key/value heads")
    if not (q.dtype == k_cache.dtype == v_cache.dtype == out.dtype):
        raise TypeError("q, caches and out must share one dtype")
    if out.shape != (tokens, num_heads, value_size):
        raise ValueError(f"out must be {(tokens, num_heads, value_size)}, got {tuple(out.shape)}")
    fn = _fn(
        "einf_paged_attention_generic",
        [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
         c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p],
    )
    _check(
        fn(_dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"), _code(q),
           _opt(block_table, "block_table", torch.int32), _opt(seq_of_token, "seq_of_token", torch.int32),
           _opt(positions, "positions", torch.int32), _dev(out, "out"), tokens, num_heads, num_kv_heads,
           head_size, value_size, value_stride, page_size, num_pages, block_table.shape[1], float(scale),
           int(window) if window else 0, int(keep_first) if window else 0, int(chunk) if chunk else 0,
           float(softcap) if softcap else 0.0, _opt(sink, "sink", torch.float32), _dev(status, "status"), _stream()),
        "paged_attention_generic",
    )


LATENT_DECODE_MAX_SPLITS = 32


def latent_decode_splits(num_tokens: int, num_heads: int, max_context: Optional[int]) -> int:
    """Shares of a token's keys in :func:`latent_decode_attention`: enough CTAs for two a multiprocessor,
    at least 128 keys a share."""
    ctas = max(1, num_tokens * -(-num_heads // 16))
    wanted = -(-2 * _sm_count() // ctas)
    most = max(1, (max_context or 1) // 128)
    return max(1, min(wanted, most, LATENT_DECODE_MAX_SPLITS))


_latent_decode_scratch: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


def latent_decode_attention(
    q: torch.Tensor,
    cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_of_token: torch.Tensor,
    positions: torch.Tensor,
    out: torch.Tensor,
    scale: float,
    splits: int,
    status: torch.Tensor,
) -> None:
    """Causal attention of single tokens over rows that all query heads share: ``q [tokens, heads, row]``,
    ``cache [pages, 1, page_size, row]`` whose first ``out.shape[2]`` elements are the values.  A CTA stages
    32 rows at a time in shared memory for sixteen heads; ``splits`` CTAs share a token's keys and a
    second kernel adds their results up in order (the workspace is kept per shape)."""
    tokens, heads, row = q.shape
    pages, kv_heads, page_size, size = cache.shape
    value_size = out.shape[2]
    if kv_heads != 1 or size != row or out.shape[:2] != (tokens, heads) or not 0 < value_size <= row:
        raise ValueError(f"latent_decode_attention: q {tuple(q.shape)}, cache {tuple(cache.shape)}, out {tuple(out.shape)}")
    if row > MAX_GENERIC_HEAD_SIZE:
        raise UnsupportedSize(f"rows up to {MAX_GENERIC_HEAD_SIZE} elements, got {row}")
    if not (q.dtype == cache.dtype == out.dtype):
        raise TypeError("q, cache and out must share one dtype")
    if not 1 <= splits <= LATENT_DECODE_MAX_SPLITS:
        raise UnsupportedSize(f"1 to {LATENT_DECODE_MAX_SPLITS} shares, not {splits}")
    acc_ptr = ml_ptr = 0
    if splits > 1:
        key = (str(q.device), tokens, heads, splits, value_size)
        scratch = _latent_decode_scratch.get(key)
        if scratch is None:
            scratch = (torch.empty((tokens, heads, splits, value_size), dtype=torch.float32, device=q.device),
                       torch.empty((tokens, heads, splits, 2), dtype=torch.float32, device=q.device))
            if len(_latent_decode_scratch) > 16:
                _latent_decode_scratch.clear()
            _latent_decode_scratch[key] = scratch
        acc_ptr, ml_ptr = scratch[0].data_ptr(), scratch[1].data_ptr()
    fn = _fn(
        "einf_latent_decode_attention",
        [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
         c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    )
    _check(
        fn(_dev(q, "q"), _dev(cache, "cache"), _code(q), _opt(block_table, "block_table", torch.int32),
           _opt(seq_of_token, "seq_of_token", torch.int32), _opt(positions, "positions", torch.int32), _dev(out, "out"),
           acc_ptr, ml_ptr, tokens, heads, row, value_size, page_size, pages, block_table.shape[1], float(scale),
           int(splits), _dev(status, "status"), _stream()),
        "latent_decode_attention",
    )


#: activations of :func:`activation` by name
ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2, "relu": 3}


def activation(x: torch.Tensor, out: torch.Tensor, kind: str) -> None:
    """``out = act(x)`` elementwise (``relu2``: the square of ReLU; ``gelu_tanh``; ``silu``; ``relu``);
    ``x`` may be float32 partial sums ``[splits, tokens, width]`` of a split-K product."""
    tokens, width = out.shape
    splits, stride = _maybe_split(x, tokens, width, "x")
    if kind not in ACTIVATIONS:
        raise ValueError(f"unknown activation {kind!r}; known: {sorted(ACTIVATIONS)}")
    fn = _fn("einf_activation", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_longlong, c_int, c_void_p])
    _check(
        fn(_dev(x, "x"), _code(x), splits, stride, _dev(out, "out"), _code(out), tokens * width, ACTIVATIONS[kind],
           _stream()),
        "activation",
    )


def qkv_norm_store(
    qkv: torch.Tensor,
    bias: Optional[torch.Tensor],
    slots: Optional[torch.Tensor],
    q_out: torch.Tensor,
    k_cache: Optional[torch.Tensor],
    v_cache: Optional[torch.Tensor],
    num_heads: int,
    num_kv_heads: int,
    key_size: int,
    value_size: int,
    unit_eps: Optional[float],
    status: torch.Tensor,
    positions: Optional[torch.Tensor] = None,
    inv_freq: Optional[torch.Tensor] = None,
    interleaved: bool = False,
    value_mix: Optional[str] = None,
    shared_values: Optional[torch.Tensor] = None,
    mix: Optional[torch.Tensor] = None,
    q_norm_weight: Optional[torch.Tensor] = None,
    k_norm_weight: Optional[torch.Tensor] = None,
    norm_rows: bool = False,
    values_from_keys: bool = False,
) -> None:
    """The general form of bias, position encoding and cache write.  With ``inv_freq`` (float32,
    n entries; needs ``positions``) the first 2n dimensions of every query and key head are rotated
    by ``position * inv_freq[i]``, pair i being dimensions (i, i + n), or (2i, 2i + 1) with
    ``interleaved``.  ``value_mix`` "source" also leaves the layer's values in ``shared_values``
    (float32 ``[tokens, kv_heads * value_size]``); "blend" caches ``(1 - m) v + m shared_values``
    with the one-element float32 tensor ``mix``.  Without these: add the bias, divide every query and key head by
    its root mean square (``unit_eps`` inside the root; None: leave them), write the queries to
    ``q_out [tokens, heads, key_size]`` and keys and values into the pages at ``slots``.  A row of
    ``qkv`` (or of its float32 split-K partial sums) is ``[heads * key_size | kv_heads * key_size |
    kv_heads * value_size]``; ``num_kv_heads`` 0 means the row holds queries only (the layer reads
    another layer's pages); ``slots`` None writes no keys or values.  Caches are ``[pages, kv_heads, page, key_size]`` and ``[..., value_size]``.
    ``q_norm_weight`` / ``k_norm_weight`` (float32; need ``unit_eps``): the normalised queries and keys
    are multiplied by a weight before any rotation, ``[key_size]`` shared by all heads, or, with
    ``norm_rows``, ``[heads * key_size]`` and ``[kv_heads * key_size]`` while the root mean square is taken
    over all heads of the row at once instead of head by head.  ``values_from_keys``: the row holds no
    values (``[queries | keys]``); a token's cached values are its keys as projected (with bias),
    before norm and rotation, so ``value_size`` is ``key_size``."""
    tokens = qkv.shape[-2]
    width = (num_heads + num_kv_heads) * key_size + (0 if values_from_keys else num_kv_heads * value_size)
    if values_from_keys and (value_size != key_size or value_mix is not None):
        raise ValueError("values taken from the keys have the keys' size and are not mixed across layers")
    norm_mode = 0 if unit_eps is None else (2 if norm_rows else 1)
    for name, weight, heads in (("q_norm_weight", q_norm_weight, num_heads), ("k_norm_weight", k_norm_weight, num_kv_heads)):
        if weight is None:
            continue
        if not norm_mode:
            raise ValueError(f"{name} needs unit_eps")
        wanted = heads * key_size if norm_rows else key_size
        if weight.dtype != torch.float32 or weight.shape != (wanted,):
            raise ValueError(f"{name} must be float32 [{wanted}]")
    splits, stride = _maybe_split(qkv, tokens, width, "qkv")
    if q_out.numel() != tokens * num_heads * key_size:
        raise ValueError("q_out must hold [tokens, heads, key_size]")
    if max(key_size, value_size) > MAX_HEAD_SIZE:
        raise UnsupportedSize(f"head sizes up to {MAX_HEAD_SIZE}, got {key_size}, {value_size}")
    page_size = num_pages = 0
    k_ptr = v_ptr = 0
    if num_kv_heads and slots is not None:
        if k_cache is None or v_cache is None:
            raise ValueError("slots given without caches")
        num_pages, kvh, page_size, size = k_cache.shape
        if (kvh, size) != (num_kv_heads, key_size) or v_cache.shape != (num_pages, kvh, page_size, value_size):
            raise ValueError(
                f"caches are {tuple(k_cache.shape)} and {tuple(v_cache.shape)}, expected "
                f"[pages, {num_kv_heads}, page, {key_size}] and [..., {value_size}]"
            )
        if k_cache.dtype != q_out.dtype or v_cache.dtype != q_out.dtype:
            raise TypeError("cache dtype differs from q_out")
        k_ptr, v_ptr = _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache")
    pairs = 0
    if inv_freq is not None and inv_freq.shape[0]:
        pairs = inv_freq.shape[0]
        if positions is None or 2 * pairs > key_size:
            raise ValueError("a rotation needs positions and at most key_size / 2 frequencies")
    mix_code = {None: 0, "source": 1, "blend": 2}[value_mix]
    if mix_code:
        if shared_values is None or shared_values.dtype != torch.float32 or \
                shared_values.numel() != tokens * num_kv_heads * value_size:
            raise ValueError("value mixing needs float32 shared_values [tokens, kv_heads * value_size]")
        if mix_code == 2 and (mix is None or mix.numel() != 1):
            raise ValueError("value_mix 'blend' needs the one-element tensor mix")
    fn = _fn(
        "einf_qkv_norm_store",
        [c_void_p, c_int, c_int, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
         c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    )
    _check(
        fn(_dev(qkv, "qkv"), _code(qkv), splits, stride, _code(q_out), _opt(bias, "bias", torch.float32),
           _opt(slots, "slots", torch.int32) if k_ptr else 0, _dev(q_out, "q_out"), k_ptr, v_ptr, tokens,
           num_heads, num_kv_heads, key_size, value_size, norm_mode,
           float(unit_eps or 0.0), page_size, num_pages,
           _opt(positions, "positions", torch.int32) if pairs else 0,
           _opt(inv_freq, "inv_freq", torch.float32) if pairs else 0, pairs, 1 if interleaved else 0, mix_code,
           _opt(shared_values, "shared_values", torch.float32) if mix_code else 0,
           _opt(mix, "mix", torch.float32) if mix_code == 2 else 0, FLOAT32,
           _opt(q_norm_weight, "q_norm_weight", torch.float32), _opt(k_norm_weight, "k_norm_weight", torch.float32),
           1 if values_from_keys else 0, _dev(status, "status"), _stream()),
        "qkv_norm_store",
    )


# ---------------------------------------------------------------------------
# Latent attention
def latent_down_store(
    down: torch.Tensor,
    q_rank: int,
    kv_rank: int,
    rot_dim: int,
    q_norm_weight: Optional[torch.Tensor],
    kv_norm_weight: torch.Tensor,
    eps: float,
    positions: torch.Tensor,
    inv_freq: torch.Tensor,
    interleaved: bool,
    slots: Optional[torch.Tensor],
    q_latent_out: Optional[torch.Tensor],
    cache: Optional[torch.Tensor],
    status: torch.Tensor,
) -> None:
    """From a token's product row ``[query latent q_rank | kv latent kv_rank | key part rot_dim]`` (or its
    float32 split-K partial sums): the RMS-normed query latent into ``q_latent_out [tokens, q_rank]``, and
    the cache row ``[normed kv latent | rotated key part]`` into the page slot of the token (``cache``
    ``[pages, 1, page_size, kv_rank + rot_dim]``; ``slots`` None writes none).  Norms carry a weight and
    ``eps`` inside the root; everything is computed in 32-bit and rounded once."""
    tokens = down.shape[-2]
    width = q_rank + kv_rank + rot_dim
    splits, stride = _maybe_split(down, tokens, width, "down")
    if inv_freq.shape[0] * 2 != rot_dim:
        raise ValueError(f"{rot_dim} rotated dimensions need {rot_dim // 2} frequencies, got {inv_freq.shape[0]}")
    if width * 4 > 48 * 1024:
        raise UnsupportedSize(f"latent rows of {width} values exceed the kernel's shared memory")
    page_size = num_pages = 0
    cache_ptr = 0
    dtype_of = q_latent_out if q_latent_out is not None else cache
    if slots is not None:
        if cache is None or cache.shape[1] != 1 or cache.shape[3] != kv_rank + rot_dim:
            raise ValueError(f"the latent cache must be [pages, 1, page, {kv_rank + rot_dim}]")
        num_pages, _, page_size, _ = cache.shape
        cache_ptr = _dev(cache, "cache")
    if q_rank and (q_latent_out is None or q_latent_out.shape != (tokens, q_rank) or q_norm_weight is None):
        raise ValueError("a query latent needs its norm weight and q_latent_out [tokens, q_rank]")
    fn = _fn(
        "einf_latent_down_store",
        [c_void_p, c_int, c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p,
         c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    )
    _check(
        fn(_dev(down, "down"), _code(down), splits, stride, _code(dtype_of), tokens, q_rank, kv_rank, rot_dim,
           _opt(q_norm_weight, "q_norm_weight", torch.float32) if q_rank else 0,
           _opt(kv_norm_weight, "kv_norm_weight", torch.float32), float(eps),
           _opt(positions, "positions", torch.int32), _opt(inv_freq, "inv_freq", torch.float32),
           1 if interleaved else 0, _opt(slots, "slots", torch.int32) if cache_ptr else 0,
           _dev(q_latent_out, "q_latent_out") if q_rank else 0, cache_ptr, page_size, num_pages,
           _dev(status, "status"), _stream()),
        "latent_down_store",
    )


def latent_q_store(
    q: torch.Tensor,
    positions: torch.Tensor,
    inv_freq: torch.Tensor,
    interleaved: bool,
    q_plain: torch.Tensor,
    q_full: torch.Tensor,
) -> None:
    """Queries ``[tokens, heads * (dim + rot_dim)]`` (or partial sums), head by head ``[dim plain | rot_dim
    to rotate]``: the plain part into ``q_plain [tokens, heads, dim]``, the rotated part into the last
    ``rot_dim`` elements of every head of ``q_full [tokens, heads, kv_rank + rot_dim]``."""
    tokens, heads, dim = q_plain.shape
    rot_dim = 2 * inv_freq.shape[0]
    kv_rank = q_full.shape[2] - rot_dim
    if q_full.shape[:2] != (tokens, heads) or kv_rank <= 0 or q_full.dtype != q_plain.dtype:
        raise ValueError(f"q_full {tuple(q_full.shape)} does not fit q_plain {tuple(q_plain.shape)}")
    splits, stride = _maybe_split(q, tokens, heads * (dim + rot_dim), "q")
    fn = _fn(
        "einf_latent_q_store",
        [c_void_p, c_int, c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
         c_void_p, c_void_p, c_void_p],
    )
    _check(
        fn(_dev(q, "q"), _code(q), splits, stride, _code(q_plain), tokens, heads, dim, rot_dim, kv_rank,
           _opt(positions, "positions", torch.int32), _opt(inv_freq, "inv_freq", torch.float32),
           1 if interleaved else 0, _dev(q_plain, "q_plain"), _dev(q_full, "q_full"), _stream()),
        "latent_q_store",
    )


def per_head_project(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """``out[t, h] = weight[h] @ x[t, h]`` for every head: ``x`` and ``out`` are ``[tokens, heads, *]`` views
    with unit stride in their last dimension (slices of wider rows are fine), ``weight`` is
    ``[heads, out, in]``.  bfloat16 goes to the library's batched product (``out`` bfloat16, or float32
    for a consumer that wants the sums unrounded), everything else to the FMA kernel head by head."""
    tokens, heads, size_in = x.shape
    if weight.shape[0] != heads or weight.shape[2] != size_in or out.shape != (tokens, heads, weight.shape[1]):
        raise ValueError(f"per_head_project: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and out.dtype == torch.bfloat16:
        if not x.is_cuda:
            raise KernelError("per_head_project operands must be on a CUDA device: there is no CPU path")
        torch.bmm(x.transpose(0, 1), weight.transpose(1, 2), out=out.transpose(0, 1))
        return
    if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and out.dtype == torch.float32:
        if not x.is_cuda:
            raise KernelError("per_head_project operands must be on a CUDA device: there is no CPU path")
        torch.bmm(x.transpose(0, 1), weight.transpose(1, 2), out_dtype=torch.float32, out=out.transpose(0, 1))
        return
    for head in range(heads):
        gemm_simt(x[:, head], weight[head], None, out[:, head])


# ---------------------------------------------------------------------------
# Routed feed-forward
ROUTER_SCORES = {"sigmoid": 0, "softmax": 1}


def router_topk(logits: torch.Tensor, top_k: int, score: str, renormalise: bool, expert_ids: torch.Tensor,
                weights: torch.Tensor, num_experts: Optional[int] = None, correction: Optional[torch.Tensor] = None,
                groups: Optional[Tuple[int, int]] = None) -> None:
    """Per row of float32 ``logits [tokens, width]`` (or split-K partial sums ``[splits, tokens, width]``,
    added up here): the ``top_k`` experts with the largest scores
    (ties to the lower index) into ``expert_ids`` (int32) and their weights into ``weights`` (float32),
    both ``[tokens, top_k]``, best first.  A weight is ``sigmoid(z)`` or the softmax over all experts;
    ``renormalise`` divides the chosen weights by their sum.  The experts are the first ``num_experts``
    columns of a row (default: all of them; further columns belong to someone else).  With
    ``correction`` (float32 ``[num_experts]``) the choice goes by ``score + correction`` while the weights
    stay the scores.  With ``groups = (count, keep)`` the experts form ``count`` equal groups of
    neighbours and only those of the ``keep`` groups whose best choice score is largest can be chosen."""
    tokens, width = logits.shape[-2:]
    experts = width if num_experts is None else int(num_experts)
    splits, stride = _maybe_split(logits, tokens, width, "logits")
    if logits.dtype != torch.float32 or weights.dtype != torch.float32 or expert_ids.dtype != torch.int32:
        raise TypeError("router_topk takes float32 logits and weights and int32 expert ids")
    if expert_ids.shape != (tokens, top_k) or weights.shape != (tokens, top_k):
        raise ValueError("expert_ids and weights must be [tokens, top_k]")
    if not 0 < top_k <= experts <= width or experts > 1024:
        raise UnsupportedSize(f"top_k {top_k} of {experts} experts (at most 1024) in rows of {width}")
    if correction is not None and (correction.dtype != torch.float32 or correction.shape != (experts,)):
        raise ValueError(f"correction must be float32 [{experts}]")
    count, keep = (0, 0) if groups is None else (int(groups[0]), int(groups[1]))
    if groups is not None:
        if count <= 0 or experts % count or not 0 < keep <= count or top_k > keep * (experts // count):
            raise ValueError(f"{experts} experts in {count} groups of which {keep} are kept cannot give {top_k} choices")
    fn = _fn("einf_router_topk", [c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                  c_int, c_void_p, c_void_p, c_void_p])
    _check(
        fn(_dev(logits, "logits"), splits, stride, tokens, width, experts, top_k, ROUTER_SCORES[score],
           1 if renormalise else 0, _opt(correction, "correction", torch.float32), count, keep,
           _dev(expert_ids, "expert_ids"), _dev(weights, "weights"), _stream()),
        "router_topk",
    )


def moe_dispatch(x: torch.Tensor, expert_ids: torch.Tensor, weights: torch.Tensor, num_experts: int,
                 scale_rows: bool, work: torch.Tensor, place: torch.Tensor, sorted_x: torch.Tensor) -> torch.Tensor:
    """Sort the (token, choice) pairs by expert.  ``work`` (int32 ``[3 experts + 1]``) gets counts, running
    cursors and offsets; ``place [tokens, top_k]`` the row of each pair in the sorted order; ``sorted_x
    [tokens * top_k, hidden]`` the tokens' rows in that order, times the pair's weight with
    ``scale_rows``.  Returns the offsets ``[experts + 1]`` (a view of ``work``)."""
    tokens, hidden = x.shape
    top_k = expert_ids.shape[1]
    if work.dtype != torch.int32 or work.numel() != 3 * num_experts + 1 or place.dtype != torch.int32:
        raise ValueError("work must be int32 [3 experts + 1] and place int32")
    if place.shape != (tokens, top_k) or sorted_x.shape != (tokens * top_k, hidden) or sorted_x.dtype != x.dtype:
        raise ValueError("place must be [tokens, top_k] and sorted_x [tokens * top_k, hidden] of x's dtype")
    fn = _fn(
        "einf_moe_dispatch",
        [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    )
    _check(
        fn(_dev(x, "x"), _code(x), _opt(expert_ids, "expert_ids", torch.int32), _opt(weights, "weights", torch.float32),
           tokens, top_k, num_experts, hidden, 1 if scale_rows else 0, _dev(work, "work"), _dev(place, "place"),
           _dev(sorted_x, "sorted_x"), _stream()),
        "moe_dispatch",
    )
    return work[2 * num_experts:]


def moe_gemm_on_tensor_cores(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def moe_gemm_splits(rows: int, experts: int, n: int, k: int) -> int:
    """How many ways the tcgen05 routed product cuts K: 1 unless a decode step's few rows and the
    matrix's few row tiles leave most of the GPU idle."""
    if rows > 64:
        return 1
    ctas = -(-n // 128) * min(experts, rows)
    wanted = max(1, min(8, (2 * _sm_count()) // max(ctas, 1)))
    return gemm_tcgen05_splits(k, wanted)


def moe_gemm(x: torch.Tensor, weight: torch.Tensor, offsets: torch.Tensor, out: torch.Tensor,
             status: Optional[torch.Tensor] = None) -> None:
    """``out[p] = weight[e] @ x[p]`` for the rows ``offsets[e] <= p < offsets[e + 1]`` of every expert e:
    ``x [rows, k]`` sorted by expert, ``weight [experts, n, k]``, ``out [rows, n]``.  bfloat16 operands
    (with ``status`` for the bounded waits, k a multiple of 8) run on the tcgen05 kernel whose token
    tiles never cross an expert; everything else, the 32-bit path included, on the FMA kernel.  ``out`` may
    be float32 ``[splits, rows, n]`` (``splits`` from :func:`moe_gemm_splits`): the tcgen05 kernel then cuts
    K and leaves partial sums for :func:`moe_combine` to add up."""
    rows, k = x.shape
    experts, n, k2 = weight.shape
    splits = out.shape[0] if out.dim() == 3 else 1
    if k2 != k or out.shape[-2:] != (rows, n) or offsets.numel() != experts + 1 or offsets.dtype != torch.int32:
        raise ValueError(f"moe_gemm: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if not offsets.is_cuda:
        raise KernelError("moe_gemm operands must be on a CUDA device: there is no CPU path")
    if moe_gemm_on_tensor_cores(x, weight) and status is not None:
        if out.dim() == 3 and (out.dtype != torch.float32 or splits != gemm_tcgen05_splits(k, splits)):
            raise ValueError("partial sums must be float32 [splits, rows, n] with splits from moe_gemm_splits")
        fn = _fn("einf_gemm_grouped_tcgen05", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                               c_int, c_void_p, c_void_p])
        _check(
            fn(_dev(x, "x"), _dev(weight, "weight"), offsets.data_ptr(), _dev(out, "out"), _code(out), rows, experts,
               n, k, splits, _dev(status, "status"), _stream()),
            "gemm_grouped_tcgen05",
        )
        return
    if out.dim() == 3:
        raise UnsupportedSize("only the tcgen05 routed product cuts K")
    fn = _fn("einf_moe_gemm", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                               c_void_p])
    _check(
        fn(_dev(x, "x"), _code(x), _dev(weight, "weight"), _code(weight), offsets.data_ptr(), _dev(out, "out"),
           _code(out), rows, experts, n, k, _stream()),
        "moe_gemm",
    )


def moe_combine(y: torch.Tensor, expert_ids: torch.Tensor, place: torch.Tensor, weights: torch.Tensor,
                scale_outputs: bool, addend: Optional[torch.Tensor], out: torch.Tensor, num_experts: int,
                identity_input: Optional[torch.Tensor] = None, num_identity: int = 0,
                addend_gate: Optional[Tuple[torch.Tensor, int]] = None) -> None:
    """``out[t] = addend[t] + sum_j y[place[t, j]]`` (times ``weights[t, j]`` with ``scale_outputs``) as
    float32: the experts' outputs of every token added up in the order of its choices, after the
    ``addend`` (``[tokens, hidden]`` or float32 partial sums ``[splits, tokens, hidden]``; may be None).
    A choice ``num_experts <= e < num_experts + num_identity`` is an expert that hands its input
    through: it adds ``weights[t, j] * identity_input[t]`` (``[tokens, hidden]``).  ``addend_gate``
    ``(logits, column)``: the addend is multiplied by ``sigmoid(logits[t, column])``, one number per
    token, with ``logits`` float32 ``[tokens, width]`` or split-K partial sums of it."""
    tokens, hidden = out.shape
    top_k = expert_ids.shape[1]
    y_splits = y.shape[0] if y.dim() == 3 else 1
    if out.dtype != torch.float32 or y.shape[-2:] != (tokens * top_k, hidden) or (y.dim() == 3 and y.dtype != torch.float32):
        raise ValueError("moe_combine: out must be float32 [tokens, hidden] and y [tokens * top_k, hidden] "
                         "(or float32 partial sums of it)")
    splits, stride, addend_code, addend_ptr = 1, 0, FLOAT32, 0
    if addend is not None:
        splits, stride = _maybe_split(addend, tokens, hidden, "addend")
        splits = max(splits, 1)
        addend_code, addend_ptr = _code(addend), _dev(addend, "addend")
    identity_ptr, identity_code = 0, FLOAT32
    if num_identity:
        if identity_input is None or identity_input.shape != (tokens, hidden):
            raise ValueError("experts that hand their input through need identity_input [tokens, hidden]")
        identity_ptr, identity_code = _dev(identity_input, "identity_input"), _code(identity_input)
    gate_ptr, gate_width, gate_column, gate_splits, gate_stride = 0, 0, 0, 1, 0
    if addend_gate is not None:
        gate, gate_column = addend_gate
        if addend is None or gate.dtype != torch.float32 or gate.shape[-2] != tokens or \
                not 0 <= gate_column < gate.shape[-1]:
            raise ValueError("addend_gate needs an addend and float32 logits [tokens, width] with the column inside")
        gate_width = gate.shape[-1]
        gate_splits, gate_stride = _maybe_split(gate, tokens, gate_width, "addend_gate")
        gate_splits = max(gate_splits, 1)
        gate_ptr = _dev(gate, "addend_gate")
    fn = _fn(
        "einf_moe_combine",
        [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_longlong, c_void_p, c_int,
         c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_longlong, c_void_p],
    )
    _check(
        fn(_dev(y, "y"), _code(y), _opt(expert_ids, "expert_ids", torch.int32), _opt(place, "place", torch.int32),
           _opt(weights, "weights", torch.float32), 1 if scale_outputs else 0, addend_ptr, addend_code, splits, stride,
           _dev(out, "out"), tokens, int(num_experts), top_k, hidden, y_splits, identity_ptr, identity_code,
           int(num_identity), gate_ptr, gate_width, int(gate_column), gate_splits, gate_stride, _stream()),
        "moe_combine",
    )


def softcap(values: torch.Tensor, cap: Optional[float], scale: float = 1.0) -> None:
    """``values = cap * tanh(scale * values / cap)`` in place (float32); without a cap (None)
    ``values = scale * values``."""
    if values.dtype != torch.float32:
        raise TypeError("softcap takes float32 values")
    fn = _fn("einf_softcap", [c_void_p, c_longlong, c_float, c_float, c_void_p])
    _check(fn(_dev(values, "values"), values.numel(), float(cap or 0.0), float(scale), _stream()), "softcap")


def _rows_of(x: torch.Tensor, name: str) -> int:
    """Row stride of a two-dimensional view whose rows are contiguous (a slice of columns of a wider matrix)."""
    if x.dim() != 2 or x.stride(1) != 1:
        raise ValueError(f"{name} must be a matrix with unit stride along its rows")
    if not x.is_cuda:
        raise KernelError(f"{name} is on {x.device}: the kernels run on a CUDA device only")
    return x.stride(0)


#: most taps of the short convolution
MAX_CONV_TAPS = 16
#: most rows (key size) of a recurrent state
MAX_STATE_ROWS = 512


def conv_silu(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    conv_state: torch.Tensor,
    seq_of_token: torch.Tensor,
    q_start: torch.Tensor,
    state_slots: torch.Tensor,
    out: torch.Tensor,
    dt_raw: Optional[torch.Tensor] = None,
    dt_bias: Optional[torch.Tensor] = None,
    a_log: Optional[torch.Tensor] = None,
    dt_out: Optional[torch.Tensor] = None,
    decay_out: Optional[torch.Tensor] = None,
    activation: bool = True,
    input_bias: Optional[torch.Tensor] = None,
) -> None:
    """Causal convolution per channel, bias and SiLU (``activation`` false: none) over the tokens of
    every request, continued from and into the requests' convolution states.  With ``input_bias``
    (float32 ``[channels]``) the convolution's input is ``x + input_bias`` (the state holds it so).

    ``x [tokens, channels]`` (columns of a wider matrix are fine), ``weight [channels, taps]`` with
    the current token's tap last, ``conv_state [slots, taps - 1, channels]`` float32 (a view whose
    slot stride may be larger): a request's last ``taps - 1`` inputs, oldest first.  ``out
    [tokens, channels]``.  With ``dt_raw [tokens, heads]`` (columns of the same wide matrix as
    ``x``) the launch also writes ``dt_out = softplus(dt_raw + dt_bias)`` and ``decay_out =
    exp(-exp(a_log) * dt_out)``, both float32 ``[tokens, heads]``."""
    tokens, channels = x.shape
    taps = weight.shape[1]
    if weight.shape != (channels, taps) or weight.dtype != torch.float32 or not weight.is_contiguous():
        raise ValueError(f"conv weight must be contiguous float32 {(channels, taps)}")
    if not 1 <= taps <= MAX_CONV_TAPS:
        raise UnsupportedSize(f"the convolution kernel takes 1 to {MAX_CONV_TAPS} taps, not {taps}")
    if conv_state.dtype != torch.float32 or conv_state.shape[1:] != (taps - 1, channels) or \
            (taps > 1 and (conv_state.stride(2) != 1 or conv_state.stride(1) != channels)):
        raise ValueError(f"conv_state must be float32 [slots, {taps - 1}, {channels}] with contiguous slots")
    if out.shape != (tokens, channels) or out.dtype != x.dtype:
        raise ValueError("out must have x's shape and dtype")
    stride = _rows_of(x, "x")
    heads, dt_ptr = 0, 0
    if dt_raw is not None:
        heads = dt_raw.shape[1]
        if _rows_of(dt_raw, "dt_raw") != stride or dt_raw.dtype != x.dtype or dt_raw.shape[0] != tokens:
            raise ValueError("dt_raw must be columns of the matrix x comes from")
        for name, t in (("dt_bias", dt_bias), ("a_log", a_log)):
            if t is None or t.dtype != torch.float32 or t.shape != (heads,):
                raise ValueError(f"{name} must be float32 [{heads}]")
        for name, t in (("dt_out", dt_out), ("decay_out", decay_out)):
            if t is None or t.dtype != torch.float32 or t.shape != (tokens, heads) or not t.is_contiguous():
                raise ValueError(f"{name} must be contiguous float32 {(tokens, heads)}")
        dt_ptr = dt_raw.data_ptr()
    fn = _fn(
        "einf_conv_silu",
        [c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int,
         c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
         c_void_p, c_void_p],
    )
    if input_bias is not None and (input_bias.dtype != torch.float32 or input_bias.shape != (channels,)):
        raise ValueError(f"input_bias must be float32 [{channels}]")
    _check(
        fn(x.data_ptr(), _code(x), stride, _dev(weight, "weight"), _opt(bias, "bias", torch.float32),
           conv_state.data_ptr(), conv_state.stride(0), _opt(seq_of_token, "seq_of_token", torch.int32),
           _opt(q_start, "q_start", torch.int32), _opt(state_slots, "state_slots", torch.int32), conv_state.shape[0],
           state_slots.shape[0], _dev(out, "out"), channels, taps, tokens, dt_ptr,
           _opt(dt_bias, "dt_bias", torch.float32), _opt(a_log, "a_log", torch.float32),
           0 if dt_out is None else dt_out.data_ptr(), 0 if decay_out is None else decay_out.data_ptr(), heads,
           1 if activation else 0, 0 if input_bias is None else input_bias.data_ptr(), _stream()),
        "conv_silu",
    )


#: tokens of a segment when a long portion is cut so that its segments run side by side
SEGMENT_TOKENS = 128
#: most segments of one request
MAX_SEGMENTS = 64


def recurrence_plan(num_requests: int, max_q_len: Optional[int], heads: int, dim: int, vdim: int,
                    sms: Optional[int] = None) -> tuple[int, int]:
    """``(segments, segment_len)`` of a recurrence launch: portions longer than ``SEGMENT_TOKENS`` are
    cut into segments that run side by side (at one and a half times the arithmetic) when the
    requests and heads alone would leave most of the GPU's schedulers without a warp."""
    if not max_q_len or max_q_len <= SEGMENT_TOKENS:
        return 1, max(1, max_q_len or 1)
    lanes = 1
    while lanes * 16 < dim:
        lanes *= 2
    warps = num_requests * heads * vdim * lanes // 32
    if warps >= (sms or _sm_count()) * 16:
        return 1, max_q_len
    limit = max(1, min(MAX_SEGMENTS, 65535 // max(1, num_requests)))
    segment_len = SEGMENT_TOKENS
    if -(-max_q_len // segment_len) > limit:
        segment_len = -(-(-(-max_q_len // limit)) // 16) * 16
    return -(-max_q_len // segment_len), segment_len


#: most CTAs that share one head's rows in a step of single tokens
RECURRENCE_STEP_MAX_SPLITS = 8


def recurrence_step_splits(num_requests: int, heads: int, dim: int, vdim: int, state: torch.Tensor) -> int:
    """How many CTAs share a head's rows when :func:`linear_recurrence` runs a step of single tokens:
    1 unless the requests and heads alone leave most multiprocessors without a CTA and the streaming
    kernel takes the sizes; then enough for about two CTAs a multiprocessor, at least 16 rows each.
    ``y`` is then ``[splits, tokens, heads * vdim]`` and its consumer adds the parts up."""
    if vdim % 4 or vdim // 4 > 128 or state.stride(0) % 4 or state.data_ptr() % 16:
        return 1
    ctas = max(1, num_requests * heads)
    wanted = (2 * _sm_count()) // ctas
    return max(1, min(RECURRENCE_STEP_MAX_SPLITS, wanted, dim // 16))


def linear_recurrence(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    state: torch.Tensor,
    q_start: torch.Tensor,
    state_slots: torch.Tensor,
    y: torch.Tensor,
    heads: int,
    groups: int,
    dim: int,
    vdim: int,
    head_decay: Optional[torch.Tensor] = None,
    token_decay: Optional[torch.Tensor] = None,
    token_scale: Optional[torch.Tensor] = None,
    skip: Optional[torch.Tensor] = None,
    silu_inputs: bool = False,
    max_q_len: Optional[int] = None,
    rows: int = 0,
    segment_len: Optional[int] = None,
    columns: int = 0,
) -> None:
    """Per request and head, over its tokens in order, with a float32 state ``S [dim, vdim]``::

        S <- a_t S + k_t (s_t v_t)^T        y_t = S^T q_t + skip_h v_t

    ``q``, ``k`` are ``[tokens, groups * dim]``, ``v`` ``[tokens, heads * vdim]`` (columns of wider
    matrices are fine); head ``h`` reads group ``h // (heads // groups)``.  ``a_t`` is
    ``head_decay [heads]`` or ``token_decay [tokens, heads]``; ``s_t`` is ``token_scale [tokens,
    heads]`` or 1; ``skip [heads]`` or 0; all float32.  ``silu_inputs``: q, k and v pass SiLU as
    they are read.  ``state [slots, heads, dim, vdim]`` float32 (slot stride may be larger) is read
    at the start of each request's portion and written at its end; ``y [tokens, heads * vdim]``
    float32, or, in a step of single tokens (``max_q_len`` 1), ``[splits, tokens, heads * vdim]`` with
    ``splits`` from :func:`recurrence_step_splits`: the parts of that many CTAs per head, for the
    consumer to add up.  ``max_q_len`` is the longest portion of the step as the host knows it (None: unknown,
    no portion is cut into segments); ``rows`` (0, 4, 8, 16), ``columns`` (0, 1, 2) and ``segment_len``
    override the launch's own choices (:func:`recurrence_plan`), for tests and measurements."""
    tokens = v.shape[0]
    if q.shape != (tokens, groups * dim) or k.shape != q.shape or v.shape != (tokens, heads * vdim):
        raise ValueError(f"q, k must be [{tokens}, {groups * dim}] and v [{tokens}, {heads * vdim}]")
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError("q, k and v must share one dtype")
    if heads % groups:
        raise UnsupportedSize(f"{heads} heads are not a multiple of {groups} groups")
    if dim > MAX_STATE_ROWS:
        raise UnsupportedSize(f"the recurrence kernel takes states of up to {MAX_STATE_ROWS} rows, not {dim}")
    if state.dtype != torch.float32 or state.shape[1:] != (heads, dim, vdim) or \
            state[0].stride() != (dim * vdim, vdim, 1):
        raise ValueError(f"state must be float32 [slots, {heads}, {dim}, {vdim}] with contiguous slots")
    y_splits = 1
    if y.dim() == 3:
        y_splits = y.shape[0]
        if max_q_len != 1 or y_splits != recurrence_step_splits(state_slots.shape[0], heads, dim, vdim, state):
            raise ValueError("y in parts is for a step of single tokens, with splits from recurrence_step_splits")
    if y.dtype != torch.float32 or y.shape[-2:] != (tokens, heads * vdim) or not y.is_contiguous():
        raise ValueError(f"y must be contiguous float32 {(tokens, heads * vdim)}")
    if (head_decay is None) == (token_decay is None):
        raise ValueError("give head_decay or token_decay")
    for name, t, shape in (("head_decay", head_decay, (heads,)), ("token_decay", token_decay, (tokens, heads)),
                           ("token_scale", token_scale, (tokens, heads)), ("skip", skip, (heads,))):
        if t is not None and (t.dtype != torch.float32 or t.shape != shape or not t.is_contiguous()):
            raise ValueError(f"{name} must be contiguous float32 {shape}")
    requests = state_slots.shape[0]
    if tokens == 0 or requests == 0:
        return
    if segment_len is not None:
        longest = max_q_len or tokens
        segments, segment_len = -(-longest // int(segment_len)), int(segment_len)
    else:
        segments, segment_len = recurrence_plan(requests, max_q_len, heads, dim, vdim)
        if max_q_len is None:
            segment_len = tokens
    segment_state = segment_decay = None
    if segments > 1:
        segment_state = torch.empty((requests * segments, heads, dim, vdim), dtype=torch.float32, device=y.device)
        segment_decay = torch.empty((requests * segments, heads), dtype=torch.float32, device=y.device)
    fn = _fn(
        "einf_linear_recurrence",
        [c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
         c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_longlong, c_void_p],
    )
    _check(
        fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), _code(q), _rows_of(q, "q"), _rows_of(k, "k"), _rows_of(v, "v"),
           _opt(head_decay, "head_decay", torch.float32), _opt(token_decay, "token_decay", torch.float32),
           _opt(token_scale, "token_scale", torch.float32), _opt(skip, "skip", torch.float32),
           state.data_ptr(), state.stride(0), state.shape[0], _opt(q_start, "q_start", torch.int32),
           _opt(state_slots, "state_slots", torch.int32), requests, _dev(y, "y"), heads, groups, dim,
           vdim, 1 if silu_inputs else 0, int(rows), int(columns), segments, segment_len,
           _opt(segment_state, "segment_state", torch.float32), _opt(segment_decay, "segment_decay", torch.float32),
           y_splits, tokens * heads * vdim, _stream()),
        "linear_recurrence",
    )
    if segments > 1:
        global launch_count
        launch_count += 2      # the first pass and the walk over the segments


def gated_norm(
    y: torch.Tensor,
    gate: torch.Tensor,
    weight: torch.Tensor,
    out: torch.Tensor,
    parts: int,
    eps: float,
    gate_first: bool,
    gate_kind: str,
) -> None:
    """The gate and RMS norm behind a recurrence, in 32-bit: ``y [tokens, width]`` float32 is cut
    into ``parts`` equal parts, each divided by its own root mean square.  ``gate_first``: ``u = y *
    g(gate)``, ``out = u / rms(u) * weight``; otherwise ``out = y / rms(y) * weight * g(gate)``.
    ``g`` is ``"silu"`` or ``"sigmoid"``; ``gate [tokens, width]`` may be columns of a wider matrix."""
    tokens, width = y.shape
    if y.dtype != torch.float32 or not y.is_contiguous():
        raise TypeError("y must be contiguous float32")
    if gate.shape != (tokens, width) or out.shape != (tokens, width) or gate.dtype != out.dtype:
        raise ValueError("gate and out must be [tokens, width] of one dtype")
    if weight.shape != (width,) or weight.dtype != torch.float32:
        raise ValueError(f"weight must be float32 [{width}]")
    if parts <= 0 or width % parts:
        raise ValueError(f"a row of {width} cannot be cut into {parts} equal parts")
    kinds = {"silu": 0, "sigmoid": 1}
    if gate_kind not in kinds:
        raise ValueError(f"gate_kind must be one of {sorted(kinds)}")
    fn = _fn(
        "einf_gated_norm",
        [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int,
         c_void_p],
    )
    _check(
        fn(_dev(y, "y"), gate.data_ptr(), _code(gate), _rows_of(gate, "gate"), _dev(weight, "weight"), _dev(out, "out"),
           tokens, width, parts, float(eps), 1 if gate_first else 0, kinds[gate_kind], _stream()),
        "gated_norm",
    )


def memory_value_columns(vdim: int) -> int:
    """Columns of a matrix memory's state that carries its normaliser beside its ``vdim`` value columns:
    one more, filled up to a multiple of four (what the streaming recurrence kernel's 16-byte accesses take)."""
    return (vdim + 1 + 3) // 4 * 4


def memory_gates(
    gates: torch.Tensor,
    bias: torch.Tensor,
    cap: float,
    v: torch.Tensor,
    top_state: torch.Tensor,
    q_start: torch.Tensor,
    state_slots: torch.Tensor,
    decay: torch.Tensor,
    scale: torch.Tensor,
    floor: torch.Tensor,
    v_wide: torch.Tensor,
    heads: int,
    vdim: int,
    max_q_len: Optional[int] = None,
) -> None:
    """The exponential gates of a matrix memory, stabilised by a running maximum, in 32-bit.
    ``gates`` float32 ``[tokens, 2 heads]`` (or split-K partial sums of it) holds per head the raw
    input gate, then the raw forget gate; with ``bias [2 heads]`` and the cap c::

        i_t = c tanh((z_i + b_i) / c)          f_t = logsigmoid(c tanh((z_f + b_f) / c))
        m_t = max(f_t + m_(t-1), i_t)          decay_t = exp(f_t + m_(t-1) - m_t)
        scale_t = exp(i_t - m_t)               floor_t = exp(-m_t)

    over each request's tokens in order; ``m`` is read from and written back to ``top_state
    [slots, heads]`` (float32, slot stride may be larger; a fresh request's row is zero).  ``decay``,
    ``scale``, ``floor``: float32 ``[tokens, heads]``.  The same launch widens the values for the
    recurrence: ``v_wide [tokens, heads * columns]`` (v's dtype) is ``v [tokens, heads * vdim]``
    (columns of a wider matrix are fine) with a column of ones behind every head's values and zeros
    up to ``columns``.  ``max_q_len``: the longest portion of the step as the host knows it (it sizes the
    launch; None: all tokens)."""
    tokens = v.shape[0]
    columns = v_wide.shape[1] // max(heads, 1)
    splits, stride = _maybe_split(gates, tokens, 2 * heads, "gates")
    if gates.dtype != torch.float32 or bias.dtype != torch.float32 or bias.shape != (2 * heads,):
        raise ValueError(f"gates must be float32 [tokens, {2 * heads}] and bias float32 [{2 * heads}]")
    for name, t in (("decay", decay), ("scale", scale), ("floor", floor)):
        if t.dtype != torch.float32 or t.shape != (tokens, heads) or not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous float32 {(tokens, heads)}")
    if v.shape != (tokens, heads * vdim) or v_wide.shape != (tokens, heads * columns) or columns <= vdim or \
            v_wide.dtype != v.dtype or not v_wide.is_contiguous():
        raise ValueError("v must be [tokens, heads * vdim] and v_wide contiguous [tokens, heads * columns], columns > vdim")
    if top_state.dtype != torch.float32 or top_state.shape[1] != heads or top_state.stride(1) != 1:
        raise ValueError(f"top_state must be float32 [slots, {heads}]")
    requests = state_slots.shape[0]
    if tokens == 0 or requests == 0:
        return
    fn = _fn(
        "einf_memory_gates",
        [c_void_p, c_int, c_longlong, c_void_p, c_float, c_void_p, c_int, c_longlong, c_void_p, c_longlong, c_int,
         c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    )
    _check(
        fn(_dev(gates, "gates"), splits, stride, _dev(bias, "bias"), float(cap), v.data_ptr(), _code(v), _rows_of(v, "v"),
           top_state.data_ptr(), top_state.stride(0), top_state.shape[0], _opt(q_start, "q_start", torch.int32),
           _opt(state_slots, "state_slots", torch.int32), requests, _dev(decay, "decay"), _dev(scale, "scale"),
           _dev(floor, "floor"), _dev(v_wide, "v_wide"), tokens, heads, vdim, columns, int(max_q_len or 0), _stream()),
        "memory_gates",
    )


def memory_output(
    y: torch.Tensor,
    floor: torch.Tensor,
    gate: torch.Tensor,
    weight: torch.Tensor,
    out: torch.Tensor,
    heads: int,
    vdim: int,
    query_scale: float,
    eps: float,
    denominator_eps: float,
) -> None:
    """What a matrix memory hands on, in 32-bit.  ``y`` float32 ``[tokens, heads * columns]`` is the
    recurrence's output on the widened values: per head ``vdim`` numerators, then the normaliser's
    product with the query.  With ``c = query_scale`` (the queries' factor, applied here)::

        o = c y[:vdim] / (max(|c y[vdim]|, floor) + denominator_eps)
        out = o / sqrt(mean(o^2) + eps) * weight * sigmoid(gate)

    head by head; ``floor`` float32 ``[tokens, heads]``, ``weight`` float32 ``[heads * vdim]``, ``gate`` and
    ``out`` ``[tokens, heads * vdim]`` of one dtype (``gate`` may be columns of a wider matrix).  ``y`` may be
    the stacked parts ``[splits, tokens, heads * columns]`` that a step of single tokens leaves: added up here."""
    tokens = y.shape[-2]
    columns = y.shape[-1] // max(heads, 1)
    y_splits = y.shape[0] if y.dim() == 3 else 1
    if y.dtype != torch.float32 or not y.is_contiguous() or y.shape[-2:] != (tokens, heads * columns) or columns <= vdim:
        raise ValueError("y must be contiguous float32 [tokens, heads * columns] (or parts of it, stacked) with columns > vdim")
    if floor.dtype != torch.float32 or floor.shape != (tokens, heads) or not floor.is_contiguous():
        raise ValueError(f"floor must be contiguous float32 {(tokens, heads)}")
    if gate.shape != (tokens, heads * vdim) or out.shape != gate.shape or gate.dtype != out.dtype:
        raise ValueError("gate and out must be [tokens, heads * vdim] of one dtype")
    if weight.dtype != torch.float32 or weight.shape != (heads * vdim,):
        raise ValueError(f"weight must be float32 [{heads * vdim}]")
    if vdim > MAX_STATE_ROWS * 2:
        raise UnsupportedSize(f"value heads of up to {MAX_STATE_ROWS * 2} elements, not {vdim}")
    if tokens == 0:
        return
    fn = _fn(
        "einf_memory_output",
        [c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
         c_float, c_float, c_int, c_longlong, c_void_p],
    )
    _check(
        fn(_dev(y, "y"), _dev(floor, "floor"), gate.data_ptr(), _code(gate), _rows_of(gate, "gate"),
           _dev(weight, "weight"), _dev(out, "out"), tokens, heads, vdim, columns, float(query_scale), float(eps),
           float(denominator_eps), y_splits, tokens * heads * columns, _stream()),
        "memory_output",
    )


def norm_join(terms, weights, eps: float, out: torch.Tensor, scale: float = 1.0) -> None:
    """``out = scale * sum_i weights[i] * terms[i] / sqrt(mean(terms[i]^2) + eps)``, row by row in
    32-bit: several branches' outputs, each RMS-normed over the row with a weight of its own, added
    up.  A term is ``[tokens, width]`` (float32 or bfloat16) or float32 split-K partial sums
    ``[splits, tokens, width]``; ``weights`` float32 ``[width]`` each; ``out`` float32 ``[tokens, width]``.
    Up to four terms."""
    tokens, width = out.shape
    if out.dtype != torch.float32 or not out.is_contiguous():
        raise TypeError("out must be contiguous float32")
    if not 0 < len(terms) <= 4 or len(weights) != len(terms):
        raise UnsupportedSize(f"one to four terms with a weight each, got {len(terms)} and {len(weights)}")
    packed = []
    for term, weight in zip(terms, weights):
        splits, stride = _maybe_split(term, tokens, width, "term")
        if weight.dtype != torch.float32 or weight.shape != (width,):
            raise ValueError(f"a weight must be float32 [{width}]")
        packed.append((_dev(term, "term"), _code(term), max(splits, 1), stride, _dev(weight, "weight")))
    while len(packed) < 4:
        packed.append((0, FLOAT32, 0, 0, 0))
    if tokens == 0:
        return
    fn = _fn("einf_norm_join", [c_int] + [c_void_p, c_int, c_int, c_longlong, c_void_p] * 4 +
             [c_float, c_float, c_void_p, c_int, c_int, c_void_p])
    flat = [value for term in packed for value in term]
    _check(fn(len(terms), *flat, float(eps), float(scale), _dev(out, "out"), tokens, width, _stream()), "norm_join")


#: head sizes the tensor-core attention kernels take (one build per size)
# ---------------------------------------------------------------------------
# The residual stream between sublayers
MAX_SIDE_SIZE = 256
#: most terms (tensors of pending sublayer output) one launch adds to the stream
MAX_PENDING_TERMS = 2


def _pending_terms(terms, rows: int, width: int) -> list:
    """Up to two pending outputs, each ``[rows, width]`` or partial sums ``[splits, rows, width]``, as
    the launchers' (pointer, dtype code, splits, stride) quadruples."""
    terms = [t for t in (terms or []) if t is not None]
    if len(terms) > MAX_PENDING_TERMS:
        raise UnsupportedSize(f"{len(terms)} pending terms: the kernels add up to {MAX_PENDING_TERMS}")
    out = []
    for index in range(MAX_PENDING_TERMS):
        if index < len(terms):
            t = terms[index]
            splits, stride = _maybe_split(t, rows, width, "pending") if t.dim() == 3 else (1, 0)
            if t.dim() == 2 and t.shape != (rows, width):
                raise ValueError(f"pending is {tuple(t.shape)}, expected {(rows, width)}")
            out += [_dev(t, "pending"), _code(t), splits, stride]
        else:
            out += [0, FLOAT32, 0, 0]
    return out


def norm_conv(
    pending,
    pending_scale: float,
    residual: torch.Tensor,
    norm_weight: torch.Tensor,
    eps: float,
    conv_weight: Optional[torch.Tensor],
    conv_state: Optional[torch.Tensor],
    seq_of_token: torch.Tensor,
    q_start: torch.Tensor,
    state_slots: torch.Tensor,
    out: torch.Tensor,
    single_tokens: bool = False,
) -> None:
    """``residual += pending_scale * sum(pending)`` (a list of up to two tensors, each ``[T, H]`` or
    partial sums ``[S, T, H]``; None or empty: nothing is added), ``h = residual * rsqrt(mean(residual^2)
    + eps) * norm_weight`` and, with ``conv_weight [H, taps]`` (float32, the current token's tap last),
    ``out = h + conv(h)``: a causal convolution over the tokens of each request, continued from and
    into ``conv_state [slots, taps - 1, H]`` (float32, oldest first; a view whose slot stride may be
    larger; not needed with one tap).  Everything is 32-bit; ``out`` is rounded once.
    ``single_tokens``: every request brings one token, and one launch does it all."""
    tokens, hidden = residual.shape
    if residual.dtype != torch.float32 or norm_weight.dtype != torch.float32 or norm_weight.shape != (hidden,):
        raise TypeError("the residual stream and norm weights are float32 [.., hidden]")
    if out.shape != (tokens, hidden):
        raise ValueError(f"out is {tuple(out.shape)}, expected {(tokens, hidden)}")
    if hidden > 16384:
        raise UnsupportedSize(f"norm_conv keeps a row in shared memory; width {hidden} > 16384")
    taps, state_ptr, state_stride, num_slots, weight_ptr, scratch_ptr = 0, 0, 0, 0, 0, 0
    scratch = None
    if conv_weight is not None:
        taps = conv_weight.shape[1]
        if conv_weight.shape != (hidden, taps) or conv_weight.dtype != torch.float32 or not conv_weight.is_contiguous():
            raise ValueError(f"conv weight must be contiguous float32 {(hidden, taps)}")
        if not 1 <= taps <= MAX_CONV_TAPS:
            raise UnsupportedSize(f"the convolution kernels take 1 to {MAX_CONV_TAPS} taps, not {taps}")
        weight_ptr = conv_weight.data_ptr()
        if taps > 1:
            if conv_state is None or conv_state.dtype != torch.float32 or conv_state.shape[1:] != (taps - 1, hidden) \
                    or conv_state.stride(2) != 1 or conv_state.stride(1) != hidden:
                raise ValueError(f"conv_state must be float32 [slots, {taps - 1}, {hidden}] with contiguous slots")
            state_ptr, state_stride, num_slots = conv_state.data_ptr(), conv_state.stride(0), conv_state.shape[0]
            if not single_tokens:
                scratch = torch.empty((tokens, hidden), dtype=torch.float32, device=residual.device)
                scratch_ptr = scratch.data_ptr()
    fn = _fn(
        "einf_norm_conv",
        [c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_int, c_longlong, c_float, c_void_p, c_void_p, c_float,
         c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
         c_int, c_int, c_int, c_void_p],
    )
    _check(
        fn(*_pending_terms(pending, tokens, hidden), float(pending_scale), _dev(residual, "residual"),
           _dev(norm_weight, "norm_weight"), float(eps), weight_ptr, taps, state_ptr, state_stride, num_slots,
           _opt(seq_of_token, "seq_of_token", torch.int32), _opt(q_start, "q_start", torch.int32),
           _opt(state_slots, "state_slots", torch.int32), state_slots.shape[0], _dev(out, "out"), _code(out),
           scratch_ptr, tokens, hidden, 1 if single_tokens else 0, _stream()),
        "norm_conv",
    )


def stream_tail(
    residual: torch.Tensor,
    pending,
    pending_scale: float,
    token_ids: torch.Tensor,
    side: Optional[tuple],
    depth: Optional[tuple],
) -> None:
    """The end of a layer in one pass over every row of the stream, in 32-bit:
    ``x = residual + pending_scale * sum(pending)`` (as in :func:`norm_conv`); with ``side = (table
    [vocab, n], gate [n, H], proj_t [n, H], norm [H] float32, eps)``: ``g = gelu(gate x) * table[token]``,
    ``y = proj_t^T g``, ``x += pending_scale * y * rsqrt(mean(y^2) + eps) * norm``; with ``depth =
    (history [L + 1, T, H] float32, index, weight [index + 2] float32)``: ``history[index + 1] = x`` and
    ``x = sum_(j <= index + 1) weight[j] history[j]``.  The result replaces ``residual``."""
    tokens, hidden = residual.shape
    if residual.dtype != torch.float32:
        raise TypeError("the residual stream is float32")
    if hidden > 16384:
        raise UnsupportedSize(f"stream_tail keeps a row in shared memory; width {hidden} > 16384")
    side_args = [0, 0, 0, FLOAT32, 0, 0, 0, 0.0]
    if side is not None:
        table, gate, proj_t, norm, eps = side
        size = table.shape[1]
        if gate.shape != (size, hidden) or proj_t.shape != (size, hidden) or norm.shape != (hidden,) or \
                norm.dtype != torch.float32 or not (table.dtype == gate.dtype == proj_t.dtype):
            raise ValueError("side input: table [vocab, n], gate [n, H], proj_t [n, H] of one dtype, norm float32 [H]")
        if size > MAX_SIDE_SIZE:
            raise UnsupportedSize(f"a token input of {size} values: the kernel takes up to {MAX_SIDE_SIZE}")
        side_args = [_dev(table, "table"), _dev(gate, "gate"), _dev(proj_t, "proj_t"), _code(table), _dev(norm, "norm"),
                     size, table.shape[0], float(eps)]
    depth_args = [0, 0, 0, 0]
    if depth is not None:
        history, index, weight = depth
        if history.dtype != torch.float32 or history.shape[1:] != (tokens, hidden) or not history.is_contiguous() or \
                not 0 <= index < history.shape[0] - 1 or weight.shape != (index + 2,) or weight.dtype != torch.float32:
            raise ValueError("depth average: history float32 [L + 1, T, H], weight float32 [index + 2]")
        depth_args = [history.data_ptr(), int(index), _dev(weight, "depth weight"), tokens * hidden]
    fn = _fn(
        "einf_stream_tail",
        [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_int, c_longlong, c_float, c_void_p,
         c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_int, c_void_p, c_longlong,
         c_int, c_int, c_void_p],
    )
    _check(
        fn(_dev(residual, "residual"), *_pending_terms(pending, tokens, hidden), float(pending_scale),
           _opt(token_ids, "token_ids", torch.int32), *side_args, *depth_args, tokens, hidden, _stream()),
        "stream_tail",
    )


# ---------------------------------------------------------------------------
# Attention whose heads' scores meet before the softmax
MIXED_MAX_HEADS = 32


NUM_SMS = 148
MIXED_KEYS_PER_SPLIT = 64       # a CTA that shares a block's keys takes at least one 64-key tile
_mixed_join_scratch: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


def mixed_tiled_variant(heads: int) -> str:
    """The build of the tiled score-mixing kernel for ``heads`` query heads."""
    return "HEADS_PAD=" + str(next(n for n in (4, 8, 16, 32) if n >= heads))


def mixed_tiled_rows(heads: int, kv_heads: int, key_size: int, value_size: int, single: bool,
                     dtype: torch.dtype = torch.float32) -> int:
    """Queries a CTA of the tiled score-mixing kernels takes for these sizes (0: they do not take them); 16
    for the bfloat16 prompt portions that the tensor-core kernel takes."""
    if heads > MIXED_MAX_HEADS:
        return 0
    fn = _fn("einf_paged_attention_mixed_tiled_rows", [c_int, c_int, c_int, c_int, c_int, c_int], mixed_tiled_variant(heads))
    return int(fn(heads, kv_heads, key_size, value_size, int(single), BFLOAT16 if dtype == torch.bfloat16 else FLOAT32))


def mixed_tiled_splits(blocks: int, rows: int, window: Optional[int], max_context: int, per_sm: int = 2) -> int:
    """CTAs that share the keys of one block of ``rows`` queries: as many as still run at once
    (``per_sm`` CTAs an SM) when the launch has few blocks, and no more than the 64-key tiles a query can see."""
    if not max_context and not window:
        return 1
    keys = max_context or (1 << 30)
    if window:
        keys = min(keys, int(window) + rows - 1)
    return max(1, min(-(-keys // MIXED_KEYS_PER_SPLIT), (NUM_SMS * per_sm) // max(1, blocks), 64))


def _mixed_tiled(q, k_cache, v_cache, block_table, seq_of_token, positions, out, scale, window, slopes, talk, sink,
                 out_scale, status, q_tiles, single_tokens, num_singles, max_context) -> bool:
    tokens, heads, key_size = q.shape
    num_pages, kv_heads, page_size, _ = k_cache.shape
    value_size = v_cache.shape[3]
    num_tiles = q_tiles.shape[0]
    if q_tiles.dtype != torch.int32 or q_tiles.dim() != 2 or q_tiles.shape[1] != 4:
        raise ValueError("q_tiles must be int32 [tiles, 4]")
    launches = []
    if num_singles:
        launches.append((single_tokens, num_singles, 1, mixed_tiled_rows(heads, kv_heads, key_size, value_size, True, q.dtype)))
    if num_tiles:
        launches.append((q_tiles, num_tiles, 0, mixed_tiled_rows(heads, kv_heads, key_size, value_size, False, q.dtype)))
    if not launches or any(rows == 0 for _, _, _, rows in launches):
        return False
    variant = mixed_tiled_variant(heads)
    fn = _fn(
        "einf_paged_attention_mixed_tiled",
        [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
         c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p, c_float, c_int,
         c_void_p, c_void_p, c_void_p, c_void_p],
        variant,
    )
    global launch_count
    for items, count, single, rows in launches:
        per_sm = 2
        if not single and q.dtype == torch.bfloat16:      # the tensor-core kernel runs one or two CTAs an SM
            ctas = _fn("einf_paged_attention_mixed_mma_ctas", [c_int, c_int, c_int, c_int, c_int], variant)
            per_sm = int(ctas(heads, kv_heads, key_size, value_size, BFLOAT16)) or 2
        splits = mixed_tiled_splits(count * (1 if single else -(-128 // rows)), rows, window, max_context, per_sm)
        part_acc = part_ml = None
        if splits > 1:
            # Buffers by power-of-two size and never given back: a captured graph keeps the address it saw.
            need = splits * tokens * heads * value_size
            bucket = max(1 << 16, 1 << (need - 1).bit_length())
            key = (str(q.device), bucket)
            scratch = _mixed_join_scratch.get(key)
            if scratch is None:
                scratch = (torch.empty(bucket, dtype=torch.float32, device=q.device),
                           torch.empty(2 * bucket, dtype=torch.float32, device=q.device))
                _mixed_join_scratch[key] = scratch
            part_acc, part_ml = scratch
        _check(
            fn(_dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"), _code(q),
               _opt(block_table, "block_table", torch.int32), block_table.shape[1],
               _opt(seq_of_token, "seq_of_token", torch.int32), _opt(positions, "positions", torch.int32),
               _opt(items, "items", torch.int32), count, single, _dev(out, "out"), tokens, heads, kv_heads, key_size,
               value_size, page_size, num_pages, float(scale), int(window or 0),
               _opt(slopes, "slopes", torch.float32), _opt(talk, "talk", torch.float32),
               _opt(sink, "sink", torch.float32), float(out_scale), splits,
               _opt(part_acc, "part_acc", torch.float32), _opt(part_ml, "part_ml", torch.float32),
               _dev(status, "status"), _stream()),
            "paged_attention_mixed_tiled",
        )
        if splits > 1:
            launch_count += 1      # the kernel that joins the splits
    return True


def paged_attention_mixed(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_of_token: torch.Tensor,
    positions: torch.Tensor,
    out: torch.Tensor,
    scale: float,
    window: Optional[int],
    slopes: Optional[torch.Tensor],
    talk: Optional[torch.Tensor],
    sink: Optional[torch.Tensor],
    out_scale: float,
    status: torch.Tensor,
    q_tiles: Optional[torch.Tensor] = None,
    single_tokens: Optional[torch.Tensor] = None,
    num_singles: int = 0,
    max_context: int = 0,
) -> None:
    """Causal (optionally windowed) attention over the paged cache in which all heads of a query are
    computed together: ``s_h(i, j) = scale q_h(i).k_g(j) - slopes[h] (i - j)``, then ``s_h <- sum_g talk[h,
    g] s_g`` over all query heads, then a softmax over the visible keys whose denominator also holds
    ``exp(sink[h])``, then ``out_h = out_scale * sum_j p_h(j) v_g(j)``.  ``slopes``, ``talk`` and ``sink``
    (float32 ``[H]``, ``[H, H]``, ``[H]``) are each optional.  ``q [T, H, D]``, caches ``[pages, G, page,
    D]`` and ``[pages, G, page, V]``, ``out [T, H, V]``; scores, weights and sums are 32-bit.

    With the step's split into ``q_tiles`` (int32 ``[tiles, 4]``: request, first token, rows, first position
    of up to 128 rows of a request that brings several tokens) and ``num_singles`` requests that bring one
    token (``single_tokens``: their token indices, or None when every token is one), the tiled kernel runs:
    consecutive queries of a request share the keys and values they read, and the keys of few queries are
    split over several CTAs (``max_context`` bounds the keys a query sees).  Without the split, or for
    sizes the tiled kernel does not take, one CTA per token walks its keys alone."""
    tokens, heads, key_size = q.shape
    num_pages, kv_heads, page_size, size = k_cache.shape
    value_size = v_cache.shape[3]
    if size != key_size or v_cache.shape[:3] != k_cache.shape[:3] or heads % kv_heads:
        raise ValueError(f"q {tuple(q.shape)}, k_cache {tuple(k_cache.shape)}, v_cache {tuple(v_cache.shape)}")
    if out.shape != (tokens, heads, value_size) or out.dtype != q.dtype or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise ValueError("out must be [tokens, heads, value_size] and share q's dtype with the caches")
    if heads > MIXED_MAX_HEADS:
        raise UnsupportedSize(f"{heads} heads: the score-mixing kernel takes up to {MIXED_MAX_HEADS}")
    if max(key_size, value_size) > MAX_HEAD_SIZE:
        raise UnsupportedSize(f"head sizes up to {MAX_HEAD_SIZE}, got {key_size}, {value_size}")
    for name, t, shape in (("slopes", slopes, (heads,)), ("talk", talk, (heads, heads)), ("sink", sink, (heads,))):
        if t is not None and (t.dtype != torch.float32 or t.shape != shape):
            raise ValueError(f"{name} must be float32 {shape}")
    if q_tiles is not None and _mixed_tiled(q, k_cache, v_cache, block_table, seq_of_token, positions, out, scale,
                                            window, slopes, talk, sink, out_scale, status, q_tiles, single_tokens,
                                            num_singles, max_context):
        return
    fn = _fn(
        "einf_paged_attention_mixed",
        [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
         c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p],
    )
    _check(
        fn(_dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"), _code(q),
           _opt(block_table, "block_table", torch.int32), block_table.shape[1],
           _opt(seq_of_token, "seq_of_token", torch.int32), _opt(positions, "positions", torch.int32),
           _dev(out, "out"), tokens, heads, kv_heads, key_size, value_size, page_size, num_pages, float(scale),
           int(window or 0), _opt(slopes, "slopes", torch.float32), _opt(talk, "talk", torch.float32),
           _opt(sink, "sink", torch.float32), float(out_scale), _dev(status, "status"), _stream()),
        "paged_attention_mixed",
    )


GATED_SCAN_SEGMENT = 16      # tokens a thread of the gated scan takes, while that makes no more than 128 segments


def gated_scan_plan(longest: int) -> Tuple[int, int]:
    """(segments, tokens per segment) of the gated scan for a step whose longest portion has ``longest`` tokens."""
    segment_len = max(GATED_SCAN_SEGMENT, 8 * -(-longest // (8 * 128)))
    return max(1, -(-longest // segment_len)), segment_len


def gated_scan(
    gates: torch.Tensor,
    gate_bias: torch.Tensor,
    u: torch.Tensor,
    y_raw: torch.Tensor,
    y_bias: torch.Tensor,
    rate: torch.Tensor,
    state: torch.Tensor,
    q_start: torch.Tensor,
    state_slots: torch.Tensor,
    out: torch.Tensor,
    out_scale: float,
    max_q_len: Optional[int] = None,
) -> None:
    """A gated linear recurrence with one state value per channel, over the tokens of every request,
    continued from and into ``state [slots, width]`` (float32; a view whose slot stride may be larger).
    ``gates [T, blocks, 2 part]`` float32 holds per block the raw recurrence gates, then the raw input
    gates (``gate_bias [blocks, 2 part]`` is added); ``r, i = sigmoid(.)``, ``a = exp(rate r)`` with
    ``rate [width]`` (negative), ``S <- a S + sqrt(1 - a^2) i u``; ``out = out_scale * S * gelu(y_raw +
    y_bias)``.  ``u [T, width]`` and ``y_raw`` (columns of a wider matrix are fine) share a dtype with
    ``out``.  All arithmetic is 32-bit."""
    tokens, blocks, twice = gates.shape
    width = blocks * (twice // 2)
    if gates.dtype != torch.float32 or not gates.is_contiguous() or twice % 2:
        raise ValueError("gates must be contiguous float32 [tokens, blocks, 2 * part]")
    for name, t in (("gate_bias", gate_bias), ("y_bias", y_bias), ("rate", rate)):
        if t.dtype != torch.float32 or t.numel() != (2 * width if name == "gate_bias" else width):
            raise ValueError(f"{name} must be float32 of the layer's width")
    if u.shape != (tokens, width) or out.shape != (tokens, width) or y_raw.shape != (tokens, width) or \
            not (u.dtype == out.dtype == y_raw.dtype):
        raise ValueError("u, y_raw and out are [tokens, width] of one dtype")
    if state.dtype != torch.float32 or state.shape[1] != width or state.stride(1) != 1:
        raise ValueError(f"state must be float32 [slots, {width}]")
    requests = state_slots.shape[0]
    if tokens == 0 or requests == 0:
        return
    segments, segment_len = gated_scan_plan(max_q_len or tokens)
    segment_keep = segment_add = None
    if segments > 1:
        segment_keep = torch.empty((requests * segments, width), dtype=torch.float32, device=out.device)
        segment_add = torch.empty_like(segment_keep)
    fn = _fn(
        "einf_gated_scan",
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_int,
         c_void_p, c_void_p, c_int, c_void_p, c_float, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
    )
    _check(
        fn(_dev(gates, "gates"), _dev(gate_bias, "gate_bias"), _dev(u, "u"), y_raw.data_ptr(), _code(u),
           _rows_of(y_raw, "y_raw"), y_bias.data_ptr(), _dev(rate, "rate"), state.data_ptr(), state.stride(0),
           state.shape[0], _opt(q_start, "q_start", torch.int32), _opt(state_slots, "state_slots", torch.int32),
           requests, _dev(out, "out"), float(out_scale), width, blocks, segments, segment_len,
           _opt(segment_keep, "segment_keep", torch.float32), _opt(segment_add, "segment_add", torch.float32),
           _stream()),
        "gated_scan",
    )
    if segments > 1:
        global launch_count
        launch_count += 1      # the first pass over the segments


FAST_ATTENTION_MAX_HEAD_SIZE = 128
#: query rows per tile of the prefill attention kernel
Q_TILE = 128


def attention_library(head_size: int) -> str:
    return f"attention_bf16:HEAD_SIZE={head_size}"


def has_tcgen05_attention(head_size: int, page_size: int) -> bool:
    """The tcgen05 prefill kernel is built for head sizes 64 and 128 and pages of 8 to 128 tokens."""
    return head_size in (64, 128) and page_size in (8, 16, 32, 64, 128)


def attention_libraries(head_size: int, page_size: int) -> tuple[str, ...]:
    names = (attention_library(head_size),)
    if has_tcgen05_attention(head_size, page_size):
        names += (f"attention_tcgen05:HEAD_SIZE={head_size}",)
    return names


def has_fast_attention(dtype: torch.dtype, head_size: int) -> bool:
    return dtype == torch.bfloat16 and head_size % 16 == 0 and head_size <= FAST_ATTENTION_MAX_HEAD_SIZE


def _check_fast_attention(q, k_cache, v_cache, out):
    tokens, num_heads, head_size = q.shape
    num_pages, num_kv_heads, page_size, size = k_cache.shape
    if not has_fast_attention(q.dtype, head_size):
        raise UnsupportedSize(
            f"the tensor-core attention kernels take bfloat16 and head sizes in steps of 16 up to "
            f"{FAST_ATTENTION_MAX_HEAD_SIZE}, got {q.dtype} and {head_size}"
        )
    if size != head_size or v_cache.shape != k_cache.shape or out.shape != q.shape:
        raise ValueError("q, caches and out do not fit together")
    if num_heads % num_kv_heads:
        raise UnsupportedSize(f"{num_heads} query heads are not a multiple of {num_kv_heads} key/value heads")
    if not (k_cache.dtype == v_cache.dtype == out.dtype == torch.bfloat16):
        raise TypeError("q, caches and out must be bfloat16")
    return tokens, num_heads, head_size, num_pages, num_kv_heads, page_size


def decode_splits(num_tokens: int, num_heads: int, num_kv_heads: int) -> int:
    """How many ways the keys of one token are split so that a decode launch fills the GPU
    (the reference picks splits per request from its context, qwen.py:40-57; here the kernel
    shortens the splits of a short context itself, so the count depends on the batch only)."""
    head_blocks = (num_heads // num_kv_heads + 15) // 16
    ctas_per_split = max(1, num_tokens * num_kv_heads * head_blocks)
    return max(1, min(16, -(-_sm_count() // ctas_per_split)))


class DecodeWorkspace:
    """Scratch of the split decode kernel: partial outputs, (max, sum) pairs, arrival counters."""

    def __init__(self, tokens: int, num_heads: int, num_kv_heads: int, head_size: int, splits: int, device) -> None:
        self.tokens, self.splits = tokens, splits
        head_blocks = (num_heads // num_kv_heads + 15) // 16
        self.acc = torch.empty((tokens, num_heads, splits, head_size), dtype=torch.float32, device=device)
        self.ml = torch.empty((tokens, num_heads, splits, 2), dtype=torch.float32, device=device)
        self.counters = torch.zeros((tokens, num_kv_heads * head_blocks), dtype=torch.int32, device=device)

    def fits(self, tokens: int, splits: int) -> bool:
        return tokens <= self.tokens and splits <= self.splits


def paged_decode_attention(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_of_token: torch.Tensor,
    positions: torch.Tensor,
    out: torch.Tensor,
    scale: float,
    window: Optional[int],
    workspace: DecodeWorkspace,
    splits: int,
    status: torch.Tensor,
) -> None:
    """Tensor-core attention for tokens that each attend alone (decoding): every token
    attends to the keys of its request up to its own position, split ``splits`` ways."""
    tokens, num_heads, head_size, num_pages, num_kv_heads, page_size = _check_fast_attention(q, k_cache, v_cache, out)
    if not workspace.fits(tokens, splits):
        raise ValueError("the decode workspace is too small for this launch")
    if not 1 <= splits <= 64:
        raise UnsupportedSize(f"decode attention splits a token's keys 1 to 64 ways, not {splits}")
    fn = _fn(
        "einf_paged_decode_attention",
        [c_void_p] * 10 + [c_int] * 6 + [c_float, c_int, c_int, c_void_p, c_void_p],
        f"HEAD_SIZE={head_size}",
    )
    _check(
        fn(_dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
           _opt(block_table, "block_table", torch.int32), _opt(seq_of_token, "seq_of_token", torch.int32),
           _opt(positions, "positions", torch.int32), _dev(out, "out"), workspace.acc.data_ptr(),
           workspace.ml.data_ptr(), workspace.counters.data_ptr(), tokens, num_heads, num_kv_heads, page_size,
           num_pages, block_table.shape[1], float(scale), int(window) if window else 0, splits,
           _dev(status, "status"), _stream()),
        "paged_decode_attention",
    )


def decode_cluster_size(num_tokens: int, num_heads: int, num_kv_heads: int) -> int:
    """CTAs that share one (token, key/value head) in the cluster decode kernel.  Measured on a
    B200 at head size 64: about half the SMs is the sweet spot (more CTAs shorten each CTA's
    key range, but clusters of eight large-shared-memory CTAs are slow to place)."""
    head_blocks = (num_heads // num_kv_heads + 15) // 16
    pairs = max(1, num_tokens * num_kv_heads * head_blocks)
    for cluster in (8, 4, 2):
        if pairs * cluster <= (_sm_count() * 55) // 100:
            return cluster
    return 1


_sm_counts: dict[int, int] = {}


def _sm_count() -> int:
    device = torch.cuda.current_device()
    if device not in _sm_counts:
        _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_counts[device]


_decode_cluster_room: dict[tuple[int, int, int], int] = {}


def tcgen05_decode_cluster_room(head_size: int, cluster: int) -> int:
    """How many clusters of ``cluster`` CTAs of the tcgen05 decode kernel the device holds at once
    (asked of the CUDA occupancy calculator once per device)."""
    key = (torch.cuda.current_device(), head_size, cluster)
    if key not in _decode_cluster_room:
        fn = _fn("einf_paged_decode_attention_tcgen05_max_clusters", [c_int], f"HEAD_SIZE={head_size}")
        _decode_cluster_room[key] = int(fn(cluster))
    return _decode_cluster_room[key]


def decode_context_bucket(max_context: Optional[int]) -> int:
    """The only thing a decode launch takes from the step's contexts: the longest one, rounded up
    to a power of two from 4,096 on (unknown: 4,096).  Steps whose graphs are kept apart by this
    figure may split their keys differently."""
    bucket = 4096
    while max_context is not None and bucket < max_context:
        bucket *= 2
    return bucket


#: (cluster size, clusters per token) pairs ``decode_plan`` chooses from
DECODE_SHAPES = tuple((c, s) for s in (1, 2, 3, 4, 8) for c in (16, 8, 7, 6, 5, 4, 3, 2, 1))


def decode_plan(num_tokens: int, num_heads: int, num_kv_heads: int, head_size: int, page_size: int,
                max_context: Optional[int] = None) -> tuple[str, int, int]:
    """Which decode kernel serves ``num_tokens`` single tokens, with what cluster size and how
    many clusters per token: ``("tcgen05" | "mma", cluster, splits)``.

    The tcgen05 kernel wherever it takes the sizes (head sizes 64 and 128, pages of 8 to 128
    tokens), the ``mma.sync`` cluster kernel otherwise.  Measured on a B200 (16-token pages): 64
    requests of 4,096 tokens at head size 64 32 us against 50 us; head size 128, 8 requests: 21 us
    against 46 us.

    A token's keys are cut into cluster x splits ranges, one CTA each, all CTAs of the launch on
    the device at once (a grid in two waves costs the kernel twice; at head size 128 one CTA fills
    an SM and the GPCs place fewer clusters of eight than SMs / 8: 16 pairs as clusters of 8 took
    16.9 us, as clusters of 4 about 9).  Among the shapes that fit, the one with the least
    estimated time for the bucket of the longest context (``decode_context_bucket``): a CTA walks
    its 128-key tiles one after the other at 0.9 us each, or at the pace the memory delivers them
    to all CTAs together; a cluster above eight costs 0.6 us more (and 1.7 us more where its CTAs
    share SMs); clusters that meet in global memory cost 3.5 us and 0.2 us for each of them.
    Measured, one request of 32,768 tokens at head size 64 (14 query heads, 2 key/value heads):
    clusters of 8 30.7 us, of 16 17.7 us, four clusters of 16 12.2 us; 8 requests of 32,768
    tokens: 35.7 us as clusters of 8, 28.0 us as four clusters of 4 each; head size 128 (28 and 4
    heads), one request of 32,768 tokens: 32.8 us as clusters of 8, 21.0 us as clusters of 16."""
    key = (torch.cuda.current_device(), num_tokens, num_heads, num_kv_heads, head_size, page_size,
           decode_context_bucket(max_context), DECODE_SHAPES)
    plan = _decode_plans.get(key)
    if plan is None:
        plan = _decode_plans[key] = _plan_decode(num_tokens, num_heads, num_kv_heads, head_size, page_size, key[6])
    return plan


_decode_plans: dict[tuple, tuple[str, int, int]] = {}


def _plan_decode(num_tokens: int, num_heads: int, num_kv_heads: int, head_size: int, page_size: int,
                 context_bucket: int, room=None, sms: Optional[int] = None) -> tuple[str, int, int]:
    """``decode_plan`` without its memory.  ``room(head_size, cluster)`` (how many clusters of a
    size the device holds at once) and ``sms`` are asked of the device unless given: the choice
    itself is plain arithmetic and is tested without a GPU."""
    head_blocks = (num_heads // num_kv_heads + 15) // 16
    pairs = max(1, num_tokens * num_kv_heads * head_blocks)
    if not has_tcgen05_attention(head_size, page_size):
        return "mma", decode_cluster_size(num_tokens, num_heads, num_kv_heads), 1
    tiles = context_bucket // 128
    tile_bytes = 2 * 128 * head_size * 2
    room = room or tcgen05_decode_cluster_room
    sms = sms or _sm_count()
    best, best_us = (1, 1), None
    for cluster, splits in DECODE_SHAPES:
        if pairs * splits > room(head_size, cluster) or pairs * splits > DECODE_SPLIT_SHARES:
            continue
        ctas = pairs * cluster * splits
        per_tile_us = max(0.9, ctas * tile_bytes / 6.5e6)
        us = -(-tiles // (cluster * splits)) * per_tile_us
        us += (0.6 if cluster > 8 else 0.0) + (3.5 + 0.2 * splits if splits > 1 else 0.0)
        if cluster > 8 and ctas > sms:
            us += 1.7       # large clusters that share SMs: 14 pairs of 4,096 tokens 8.6 us as clusters of 16, 8.0 as clusters of 8
        if best_us is None or us < best_us - 1e-9:
            best, best_us = (cluster, splits), us
    return "tcgen05", best[0], best[1]


def windowed_attention(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_of_token: torch.Tensor,
    positions: torch.Tensor,
    q_tiles: Optional[torch.Tensor],
    single_tokens: Optional[torch.Tensor],
    out: torch.Tensor,
    scale: float,
    window: Optional[int],
    keep_first: int,
    status: torch.Tensor,
    max_context: Optional[int] = None,
    cached_before: Optional[int] = None,
    chunk: Optional[int] = None,
    softcap: Optional[float] = None,
) -> None:
    """Attention of a whole step with any of the masks (window, first positions kept, chunks) and a soft
    cap: bfloat16 heads of 64 or 128 with values as large as keys run the tcgen05 kernels, the single
    tokens (``single_tokens``: their packed indices, None when the step has nothing else) by the
    decode kernel and the 128-row tiles of prompt portions (``q_tiles``) by the prefill kernel, side by
    side; everything else the general kernel.  The kept positions widen what a token reads by
    ``keep_first`` keys at most, so the decode kernel's shape is planned for window + keep_first."""
    head_size, page_size = q.shape[2], k_cache.shape[2]
    if (q.dtype == torch.bfloat16 and v_cache is not None and v_cache.shape == k_cache.shape
            and has_tcgen05_attention(head_size, page_size)):
        tiles = q_tiles is not None and q_tiles.shape[0] > 0
        decode = single_tokens.shape[0] > 0 if single_tokens is not None else not tiles
        if decode:
            paged_decode_attention_auto(q, k_cache, v_cache, block_table, seq_of_token, positions, out, scale, window,
                                        status, single_tokens, max_context=max_context, chunk=chunk, softcap=softcap,
                                        keep_first=keep_first)
        if q_tiles is not None and q_tiles.shape[0]:
            paged_prefill_attention(q, k_cache, v_cache, block_table, q_tiles, out, scale, window, status,
                                    cached_before=cached_before, chunk=chunk, softcap=softcap, keep_first=keep_first)
        return
    paged_attention_generic(q, k_cache, v_cache, block_table, seq_of_token, positions, out, scale, window, status,
                            chunk=chunk, softcap=softcap, keep_first=keep_first)


def paged_decode_attention_auto(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_of_token: torch.Tensor,
    positions: torch.Tensor,
    out: torch.Tensor,
    scale: float,
    window: Optional[int],
    status: torch.Tensor,
    token_list: Optional[torch.Tensor] = None,
    max_context: Optional[int] = None,
    chunk: Optional[int] = None,
    softcap: Optional[float] = None,
    keep_first: int = 0,
    sink: Optional[torch.Tensor] = None,
) -> None:
    """Decode attention by the kernel, cluster size and number of clusters per token that
    ``decode_plan`` picks for this batch; ``max_context`` is the longest context among the
    tokens (a window or a chunk shortens it), as the host knows it.  ``chunk`` and ``softcap`` (see
    :func:`paged_attention_generic`) are the tcgen05 kernel's alone."""
    tokens = token_list.shape[0] if token_list is not None else q.shape[0]
    for bound in (window, chunk):
        if bound and max_context is not None:
            max_context = min(max_context, int(bound))
    kernel, cluster, splits = decode_plan(tokens, q.shape[1], k_cache.shape[1], q.shape[2], k_cache.shape[2], max_context)
    if kernel == "tcgen05":
        paged_decode_attention_tcgen05(q, k_cache, v_cache, block_table, seq_of_token, positions, out, scale, window,
                                       cluster, status, token_list, splits, chunk=chunk, softcap=softcap,
                                       keep_first=keep_first, sink=sink)
    elif chunk or softcap or (window and keep_first) or sink is not None:
        raise UnsupportedSize("a chunked mask, a soft cap, kept first positions or a sink need the tcgen05 decode "
                              "kernel (head size 64 or 128)")
    else:
        paged_decode_attention_cluster(q, k_cache, v_cache, block_table, seq_of_token, positions, out, scale, window,
                                       cluster, status, token_list)


def paged_decode_attention_cluster(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_of_token: torch.Tensor,
    positions: torch.Tensor,
    out: torch.Tensor,
    scale: float,
    window: Optional[int],
    cluster: int,
    status: torch.Tensor,
    token_list: Optional[torch.Tensor] = None,
) -> None:
    """Decode attention whose key splits are the CTAs of a thread-block cluster (1, 2, 4 or 8)
    that merge through distributed shared memory: no scratch in global memory.  With
    ``token_list`` (int32 packed indices) only those tokens are processed."""
    tokens, num_heads, head_size, num_pages, num_kv_heads, page_size = _check_fast_attention(q, k_cache, v_cache, out)
    if token_list is not None:
        tokens = token_list.shape[0]
    if cluster not in (1, 2, 4, 8):
        raise UnsupportedSize(f"the cluster decode kernel takes clusters of 1, 2, 4 or 8 CTAs, not {cluster}")
    fn = _fn(
        "einf_paged_decode_attention_cluster",
        [c_void_p] * 8 + [c_int] * 6 + [c_float, c_int, c_int, c_void_p, c_void_p],
        f"HEAD_SIZE={head_size}",
    )
    _check(
        fn(_dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
           _opt(block_table, "block_table", torch.int32), _opt(seq_of_token, "seq_of_token", torch.int32),
           _opt(positions, "positions", torch.int32), _opt(token_list, "token_list", torch.int32), _dev(out, "out"),
           tokens, num_heads, num_kv_heads, page_size,
           num_pages, block_table.shape[1], float(scale), int(window) if window else 0, cluster,
           _dev(status, "status"), _stream()),
        "paged_decode_attention_cluster",
    )


DECODE_MAX_SPLITS = 8
DECODE_SPLIT_SHARES = 512       # (token, key/value head, head block) pairs x splits of one launch, at most
_decode_split_scratch: dict[str, tuple[torch.Tensor, torch.Tensor]] = {}


def _decode_split_workspace(pairs: int, splits: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    """Where the clusters of a split decode launch meet, per device: their shares (16 heads of up
    to 128 + 2 floats per pair and split) and the arrival counters, which every launch leaves at
    zero.  Launches on one stream run one after the other, so they share it; it is made once and
    never grows, because captured graphs hold its address."""
    if pairs * splits > DECODE_SPLIT_SHARES:
        raise UnsupportedSize(
            f"a split decode launch takes up to {DECODE_SPLIT_SHARES} shares, not {pairs} x {splits}: "
            f"split fewer ways, many tokens fill the device without it"
        )
    key = str(device)
    scratch = _decode_split_scratch.get(key)
    if scratch is None:
        scratch = (
            torch.empty(DECODE_SPLIT_SHARES * 16 * (128 + 2), dtype=torch.float32, device=device),
            torch.zeros(DECODE_SPLIT_SHARES, dtype=torch.int32, device=device),
        )
        _decode_split_scratch[key] = scratch
    return scratch


def paged_decode_attention_tcgen05(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_of_token: torch.Tensor,
    positions: torch.Tensor,
    out: torch.Tensor,
    scale: float,
    window: Optional[int],
    cluster: int,
    status: torch.Tensor,
    token_list: Optional[torch.Tensor] = None,
    splits: int = 1,
    chunk: Optional[int] = None,
    softcap: Optional[float] = None,
    keep_first: int = 0,
    sink: Optional[torch.Tensor] = None,
) -> None:
    """Decode attention on the tcgen05 tensor cores with the keys as the 128-row operand
    (S^T = K Q^T, O^T = V^T P^T), so the tile is full at any number of query heads.  Key splits
    are the CTAs of a cluster (any size from 1 to 16), as in ``paged_decode_attention_cluster``,
    and, for a few requests with long contexts, ``splits`` such clusters per token whose shares
    the last CTA to finish adds up from global memory; head sizes 64 and 128, pages of 8 to 128
    tokens."""
    tokens, num_heads, head_size, num_pages, num_kv_heads, page_size = _check_fast_attention(q, k_cache, v_cache, out)
    if not has_tcgen05_attention(head_size, page_size):
        raise UnsupportedSize(
            f"the tcgen05 attention kernels take head sizes 64 and 128 and pages of 8 to 128 tokens, "
            f"got {head_size} and {page_size}"
        )
    if sink is not None and (sink.dtype != torch.float32 or sink.shape != (num_heads,)):
        raise ValueError(f"sink must be float32 [{num_heads}]")
    if token_list is not None:
        tokens = token_list.shape[0]
    if not 1 <= cluster <= 16:
        raise UnsupportedSize(f"the tcgen05 decode kernel takes clusters of 1 to 16 CTAs, not {cluster}")
    if not 1 <= splits <= DECODE_MAX_SPLITS:
        raise UnsupportedSize(f"the tcgen05 decode kernel takes 1 to {DECODE_MAX_SPLITS} clusters per token, not {splits}")
    head_blocks = (num_heads // num_kv_heads + 15) // 16
    shares, counters = (None, None)
    if splits > 1:
        shares, counters = _decode_split_workspace(tokens * num_kv_heads * head_blocks, splits, q.device)
    fn = _fn(
        "einf_paged_decode_attention_tcgen05",
        [c_void_p] * 8 + [c_int] * 6 + [c_float, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p,
         c_void_p, c_void_p],
        f"HEAD_SIZE={head_size}",
    )
    _check(
        fn(_dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
           _opt(block_table, "block_table", torch.int32), _opt(seq_of_token, "seq_of_token", torch.int32),
           _opt(positions, "positions", torch.int32), _opt(token_list, "token_list", torch.int32), _dev(out, "out"),
           tokens, num_heads, num_kv_heads, page_size,
           num_pages, block_table.shape[1], float(scale), int(window) if window else 0,
           int(keep_first) if window else 0,
           int(chunk) if chunk else 0, float(softcap) if softcap else 0.0, cluster,
           splits, shares.data_ptr() if splits > 1 else None, counters.data_ptr() if splits > 1 else None,
           _opt(sink, "sink", torch.float32), _dev(status, "status"), _stream()),
        "paged_decode_attention_tcgen05",
    )


def prefill_prefix_bucket(cached_before: Optional[int]) -> int:
    """The only thing a prefill launch takes from the step's contexts: the largest cluster (8, 4,
    else 1) worth trying for the longest prefix that a prompt portion of the step finds in the
    cache.  Steps with equal buckets launch alike.  A cluster costs a launch about 3 us flat
    (measured: 128 tokens at the start of a prompt 7.9 us alone, 10 to 11 us as any cluster), which
    512 cached tokens repay to clusters of four and 1,024 to clusters of eight."""
    if cached_before is None or cached_before < 512:
        return 1
    return 8 if cached_before >= 1024 else 4


_prefill_cluster_room: dict[tuple[int, int, int], int] = {}


def tcgen05_prefill_cluster_room(head_size: int, cluster: int) -> int:
    """How many clusters of ``cluster`` CTAs of the tcgen05 prefill kernel the device holds at once
    (asked of the CUDA occupancy calculator once per device)."""
    key = (torch.cuda.current_device(), head_size, cluster)
    if key not in _prefill_cluster_room:
        fn = _fn("einf_paged_prefill_attention_tcgen05_max_clusters", [c_int], f"HEAD_SIZE={head_size}")
        _prefill_cluster_room[key] = int(fn(cluster))
    return _prefill_cluster_room[key]


def prefill_cluster_size(ctas: int, head_size: int, cached_before: Optional[int]) -> int:
    """CTAs that share one (row tile, head) of the tcgen05 prefill kernel, each with a run of its
    key tiles: the largest cluster (up to the prefix bucket) of which the device holds ``ctas`` at
    once.  A few row tiles behind a long prefix (a portion of a long prompt) do not fill the GPU,
    and the walk over their keys is a chain of dependent tiles; a grid in two waves costs more than
    the split saves, and so does a split of a portion at the start of its prompt, whose rows see
    few keys.  Measured on a B200, 14 heads of 64, one launch in a chain: 64 tokens after 8,192
    100 us alone, 55 / 32 / 21 us as clusters of 2 / 4 / 8; 512 tokens (56 CTAs) after 4,096 40 us
    alone, 27 as clusters of two, 34 as clusters of four (224 CTAs: two waves); 64 tokens after
    512 12.0 us alone, 9.4 as clusters of four; 256 tokens after none 8.3 us alone, 11.2 as
    clusters of two."""
    for cluster in range(prefill_prefix_bucket(cached_before), 1, -1):
        if ctas <= tcgen05_prefill_cluster_room(head_size, cluster):
            return cluster
    return 1


def paged_prefill_attention(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_table: torch.Tensor,
    q_tiles: torch.Tensor,
    out: torch.Tensor,
    scale: float,
    window: Optional[int],
    status: torch.Tensor,
    use_tcgen05: Optional[bool] = None,
    prefill_cluster: int = 0,
    cached_before: Optional[int] = None,
    chunk: Optional[int] = None,
    softcap: Optional[float] = None,
    keep_first: int = 0,
    sink: Optional[torch.Tensor] = None,
) -> None:
    """Tensor-core causal attention for prompt portions.  ``q_tiles`` is int32 ``[tiles, 4]``:
    request, first token (packed index), rows (at most ``Q_TILE``), position of the first row.
    Head sizes 64 and 128 with pages of 8 to 128 tokens run the tcgen05 kernel (``use_tcgen05``
    None: whenever it can; measured on a B200, a 2,048-token prompt of 14 heads of size 64 takes
    26 us against 82 us, 28 heads of size 128 take 62 us against 266 us), everything else the
    ``mma.sync`` kernel.  ``prefill_cluster`` (1 to 8; 0: ``prefill_cluster_size`` of the number of
    row tiles and ``cached_before``, the most tokens that a portion of this step finds in the
    cache, if the caller knows it) is the number of CTAs that share a row tile's keys in the
    tcgen05 kernel.  ``chunk``, ``softcap`` and ``sink`` (see :func:`paged_attention_generic`) are the tcgen05
    kernel's alone."""
    tokens, num_heads, head_size, num_pages, num_kv_heads, page_size = _check_fast_attention(q, k_cache, v_cache, out)
    if sink is not None and (sink.dtype != torch.float32 or sink.shape != (num_heads,)):
        raise ValueError(f"sink must be float32 [{num_heads}]")
    if q_tiles.dtype != torch.int32 or q_tiles.dim() != 2 or q_tiles.shape[1] != 4:
        raise ValueError("q_tiles must be int32 [tiles, 4]")
    can = has_tcgen05_attention(head_size, page_size)
    if use_tcgen05 is None:
        use_tcgen05 = can
    if use_tcgen05:
        if not can:
            raise UnsupportedSize(
                f"the tcgen05 attention kernel takes head sizes 64 and 128 and pages of 8 to 128 tokens, "
                f"got {head_size} and {page_size}"
            )
        fn = _fn(
            "einf_paged_prefill_attention_tcgen05",
            [c_void_p] * 5 + [c_int, c_void_p] + [c_int] * 6 + [c_float, c_int, c_int, c_int, c_float, c_int, c_void_p,
                                                                 c_void_p, c_void_p],
            f"HEAD_SIZE={head_size}",
        )
        cluster = prefill_cluster
        if not cluster:
            for bound in (window, chunk):
                if cached_before is not None and bound:
                    cached_before = min(cached_before, int(bound))
            cluster = prefill_cluster_size(num_heads * q_tiles.shape[0], head_size, cached_before)
        if window and keep_first:
            cluster = 1       # the kept keys are tiles of their own ahead of the window's: one CTA walks both
        _check(
            fn(_dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
               _opt(block_table, "block_table", torch.int32), _dev(q_tiles, "q_tiles"), q_tiles.shape[0],
               _dev(out, "out"), tokens, num_heads, num_kv_heads, page_size, num_pages, block_table.shape[1],
               float(scale), int(window) if window else 0, int(keep_first) if window else 0,
               int(chunk) if chunk else 0,
               float(softcap) if softcap else 0.0, int(cluster), _opt(sink, "sink", torch.float32),
               _dev(status, "status"), _stream()),
            "paged_prefill_attention_tcgen05",
        )
        return
    if chunk or softcap or (window and keep_first) or sink is not None:
        raise UnsupportedSize("a chunked mask, a soft cap, kept first positions or a sink need the tcgen05 prefill "
                              "kernel (head size 64 or 128)")
    fn = _fn(
        "einf_paged_prefill_attention",
        [c_void_p] * 5 + [c_int, c_void_p] + [c_int] * 5 + [c_float, c_int, c_void_p, c_void_p],
        f"HEAD_SIZE={head_size}",
    )
    _check(
        fn(_dev(q, "q"), _dev(k_cache, "k_cache"), _dev(v_cache, "v_cache"),
           _opt(block_table, "block_table", torch.int32), _dev(q_tiles, "q_tiles"), q_tiles.shape[0],
           _dev(out, "out"), num_heads, num_kv_heads, page_size, num_pages, block_table.shape[1], float(scale),
           int(window) if window else 0, _dev(status, "status"), _stream()),
        "paged_prefill_attention",
    )


ARGMAX_CHUNKS = 32
_argmax_scratch: dict[str, tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}


def _argmax_workspace(rows: int, device) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Partial (value, index) pairs and arrival counters of the two-step argmax, per device;
    launches on one stream run one after the other, so they share it."""
    key = str(device)
    scratch = _argmax_scratch.get(key)
    if scratch is None or scratch[2].shape[0] < rows:
        capacity = max(rows, 64)
        scratch = (
            torch.empty((capacity, ARGMAX_CHUNKS), dtype=torch.float32, device=device),
            torch.empty((capacity, ARGMAX_CHUNKS), dtype=torch.int32, device=device),
            torch.zeros(capacity, dtype=torch.int32, device=device),
        )
        _argmax_scratch[key] = scratch
    return scratch


def argmax(logits: torch.Tensor, tokens: torch.Tensor) -> None:
    """``tokens[r]`` = first index of the largest logit of row ``r``."""
    rows, vocab = logits.shape
    if logits.dtype != torch.float32 or tokens.dtype != torch.int32 or tokens.shape[0] < rows:
        raise TypeError("argmax takes float32 logits and an int32 token buffer")
    values, indices, counters = _argmax_workspace(rows, logits.device)
    fn = _fn("einf_argmax", [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(
        fn(_dev(logits, "logits"), _dev(tokens, "tokens"), rows, vocab, values.data_ptr(), indices.data_ptr(),
           counters.data_ptr(), _stream()),
        "argmax",
    )


def report(tokens: torch.Tensor, count: int, status: torch.Tensor, host: torch.Tensor) -> None:
    """``host[:count] = tokens[:count]; host[count] = status[0]``, written by a kernel into the
    pinned host tensor ``host``; readable after the stream is synchronised."""
    if tokens.dtype != torch.int32 or status.dtype != torch.int32 or host.dtype != torch.int32:
        raise TypeError("report takes int32 tensors")
    if tokens.shape[0] < count or host.shape[0] < count + 1 or not host.is_pinned():
        raise ValueError("report needs count tokens and a pinned host tensor of count + 1 entries")
    fn = _fn("einf_report", [c_void_p, c_int, c_void_p, c_void_p, c_void_p])
    _check(fn(_dev(tokens, "tokens"), count, _dev(status, "status"), host.data_ptr(), _stream()), "report")


def sample(
    logits: torch.Tensor,
    tokens: torch.Tensor,
    temperature: torch.Tensor,
    top_k: torch.Tensor,
    top_p: torch.Tensor,
    min_p: torch.Tensor,
    seed: torch.Tensor,
    sample_index: torch.Tensor,
) -> None:
    """Draw one token per row; rows with temperature 0 take the argmax."""
    rows, vocab = logits.shape
    if logits.dtype != torch.float32 or tokens.dtype != torch.int32 or tokens.shape[0] < rows:
        raise TypeError("sample takes float32 logits and an int32 token buffer")
    if seed.dtype != torch.int64 or sample_index.dtype != torch.int64:
        raise TypeError("seed and sample_index are int64")
    fn = _fn(
        "einf_sample",
        [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    )
    _check(
        fn(_dev(logits, "logits"), _dev(tokens, "tokens"), rows, vocab,
           _opt(temperature, "temperature", torch.float32), _opt(top_k, "top_k", torch.int32),
           _opt(top_p, "top_p", torch.float32), _opt(min_p, "min_p", torch.float32),
           _dev(seed, "seed"), _dev(sample_index, "sample_index"), _stream()),
        "sample",
    )


__all__ = [
    "KernelError",
    "KernelLibraryError",
    "UnsupportedSize",
    "add_bias",
    "add_rmsnorm",
    "argmax",
    "embed",
    "ensure_built",
    "gemm_simt",
    "gemm_tcgen05",
    "gemm_tcgen05_splits",
    "linear",
    "paged_attention_generic",
    "paged_decode_attention",
    "decode_plan",
    "decode_context_bucket",
    "paged_decode_attention_auto",
    "paged_decode_attention_cluster",
    "paged_decode_attention_tcgen05",
    "paged_prefill_attention",
    "project",
    "rope_kv_write",
    "sample",
    "silu_mul",
    "zero_fresh_state",
]
