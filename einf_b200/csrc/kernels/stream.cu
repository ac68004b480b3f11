// The residual stream between sublayers, for blocks that do more to it than add and normalise:
//   - a residual multiplier on every sublayer's output,
//   - a short causal convolution over time in front of a sublayer, in the launch of the norm,
//   - a per-layer token input after the feed-forward,
//   - a weighted sum over the results of all layers so far in place of the layer's own result.
// The stream is 32-bit; pending sublayer outputs arrive as up to two terms, each a [T, H] matrix
// (float or bfloat16) or the float partial sums [S, T, H] of a split-K product, and are added in
// a fixed order: term a split by split, then term b, then scaled, then added to the row.  Every
// row is computed by one CTA from the row's own request alone.
#include <cstdint>

#include "common.cuh"

namespace einf {

constexpr int kMaxTaps = 16;

struct Pending {
  const void* a;
  int a_dtype, a_splits;
  long long a_stride;
  const void* b;
  int b_dtype, b_splits;
  long long b_stride;
};

__device__ __forceinline__ float pending_term(const void* p, int dtype, int splits, long long stride, size_t idx) {
  if (dtype == kBFloat16) {
    const __nv_bfloat16* q = (const __nv_bfloat16*)p + idx;
    float v = 0.f;
    for (int s = 0; s < splits; ++s) v += __bfloat162float(q[(size_t)s * stride]);
    return v;
  }
  const float* q = (const float*)p + idx;
  constexpr int kBatch = 8;             // the partial sums sit in L2: keep several loads in flight
  float v = 0.f;
  for (int s0 = 0; s0 < splits; s0 += kBatch) {
    float part[kBatch];
#pragma unroll
    for (int e = 0; e < kBatch; ++e) part[e] = s0 + e < splits ? q[(size_t)(s0 + e) * stride] : 0.f;
#pragma unroll
    for (int e = 0; e < kBatch; ++e) v += part[e];
  }
  return v;
}

__device__ __forceinline__ float pending_sum(const Pending& p, size_t idx) {
  float v = 0.f;
  if (p.a) v = pending_term(p.a, p.a_dtype, p.a_splits, p.a_stride, idx);
  if (p.b) v += pending_term(p.b, p.b_dtype, p.b_splits, p.b_stride, idx);
  return v;
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// ---------------------------------------------------------------------------
// residual[t] += scale * pending[t];  h = residual[t] * rsqrt(mean(residual[t]^2) + eps) * weight
// and then one of
//   mode 0  out[t] = h (no convolution), or h * (1 + w[:, 0]) (a convolution of one tap)
//   mode 1  every request brings one token: out[t] = h + sum_j w[:, j] line[j] with line = the
//           request's state rows followed by h; the state moves on by one row in the same launch
//   mode 2  h goes to `scratch` (floats) for the two kernels below, which see a request's other
//           tokens of the step
// One CTA per token; the row lives in shared memory between the two passes.
// ---------------------------------------------------------------------------
template <typename TOut>
__global__ void norm_row_kernel(const __grid_constant__ Pending pending, float scale, float* __restrict__ residual,
                                const float* __restrict__ weight, float eps, const float* __restrict__ conv_weight,
                                int taps, float* __restrict__ conv_state, long long state_stride, int num_slots,
                                const int* __restrict__ seq_of_token, const int* __restrict__ state_slots,
                                TOut* __restrict__ out, float* __restrict__ scratch, int hidden, int mode) {
  extern __shared__ float smem[];
  float* row = smem;
  float* red = smem + hidden;
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const size_t base = (size_t)t * hidden;
  const bool adds = pending.a != nullptr || pending.b != nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = residual[base + c];
    if (adds) {
      v += scale * pending_sum(pending, base + c);
      residual[base + c] = v;
    }
    row[c] = v;
    ss = fmaf(v, v, ss);
  }
  const float inv = rsqrtf(block_sum(ss, red) / (float)hidden + eps);
  if (mode == 2) {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) scratch[base + c] = row[c] * inv * weight[c];
    return;
  }
  if (mode == 0) {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      float h = row[c] * inv * weight[c];
      if (conv_weight) h = fmaf(conv_weight[c], h, h);
      out[base + c] = from_float<TOut>(h);
    }
    return;
  }
  const int slot = state_slots[seq_of_token[t]];
  float* state = (slot >= 0 && slot < num_slots) ? conv_state + (long long)slot * state_stride : nullptr;
  const int keep = taps - 1;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float h = row[c] * inv * weight[c];
    const float* w = conv_weight + (size_t)c * taps;
    float acc = h;
    float line[kMaxTaps];
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j)
      if (j < keep) line[j] = state ? state[(size_t)j * hidden + c] : 0.f;
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j)
      if (j < keep) acc = fmaf(w[j], line[j], acc);
    acc = fmaf(w[keep], h, acc);
    out[base + c] = from_float<TOut>(acc);
    if (state) {
#pragma unroll
      for (int j = 0; j < kMaxTaps; ++j)
        if (j + 1 < keep) state[(size_t)j * hidden + c] = line[j + 1];
      state[(size_t)(keep - 1) * hidden + c] = h;
    }
  }
}

// out[t, c] = h[t, c] + sum_j w[c, j] * h[t - (taps - 1) + j, c] over the tokens of t's request, with
// the request's state rows (its last taps - 1 inputs, oldest first) in front of its first token.
template <typename TOut>
__global__ void conv_rows_kernel(const float* __restrict__ h, const float* __restrict__ conv_weight, int taps,
                                 const float* __restrict__ conv_state, long long state_stride, int num_slots,
                                 const int* __restrict__ seq_of_token, const int* __restrict__ q_start,
                                 const int* __restrict__ state_slots, TOut* __restrict__ out, int hidden,
                                 int num_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = (long long)num_tokens * hidden;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / hidden);
    const int c = (int)(idx - (long long)t * hidden);
    const int r = seq_of_token[t];
    const int first = q_start[r];
    const int slot = state_slots[r];
    const float* state = (slot >= 0 && slot < num_slots) ? conv_state + (long long)slot * state_stride : nullptr;
    float acc = h[idx];
    for (int j = 0; j < taps; ++j) {
      const int src = t - (taps - 1) + j;
      float v;
      if (src >= first) v = h[(long long)src * hidden + c];
      else v = state ? state[(long long)(taps - 1 - (first - src)) * hidden + c] : 0.f;
      acc = fmaf(conv_weight[(long long)c * taps + j], v, acc);
    }
    out[idx] = from_float<TOut>(acc);
  }
}

// Afterwards the request's last taps - 1 inputs become its state (a portion shorter than that keeps
// the tail of the old state in front).  One thread per (request, channel).
__global__ void conv_rows_state_kernel(const float* __restrict__ h, float* __restrict__ conv_state,
                                       long long state_stride, int num_slots, const int* __restrict__ q_start,
                                       const int* __restrict__ state_slots, int hidden, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int slot = state_slots[r];
  if (c >= hidden || slot < 0 || slot >= num_slots) return;
  const int first = q_start[r], count = q_start[r + 1] - first;
  if (count <= 0) return;
  float* state = conv_state + (long long)slot * state_stride;
  const int keep = taps - 1;
  float fresh[kMaxTaps];
#pragma unroll
  for (int u = 0; u < kMaxTaps; ++u) {
    if (u < keep) {
      const int rel = count - keep + u;
      fresh[u] = rel >= 0 ? h[(long long)(first + rel) * hidden + c] : state[(long long)(u + count) * hidden + c];
    }
  }
#pragma unroll
  for (int u = 0; u < kMaxTaps; ++u)
    if (u < keep) state[(long long)u * hidden + c] = fresh[u];
}

// ---------------------------------------------------------------------------
// The end of a layer.  One CTA per token, the row x in shared memory:
//   x = residual[t] + scale * pending[t]
//   token input (table != null):  s = gate x  [n];  g = gelu(s) * table[token]  [n];  y = proj_t^T g  [H];
//                                 x += scale * y * rsqrt(mean(y^2) + eps) * norm
//   depth average (history != null):  history[index + 1][t] = x;
//                                 x = sum_(j <= index) w[j] history[j][t] + w[index + 1] x
//   residual[t] = x
// gate [n, H] and proj_t [n, H] are read along H, a warp per row of gate for s, a thread per
// column for y; the arithmetic is 32-bit whatever the matrices' type.
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void stream_tail_kernel(float* __restrict__ residual, const __grid_constant__ Pending pending, float scale,
                                   const int* __restrict__ token_ids, const TW* __restrict__ table,
                                   const TW* __restrict__ gate, const TW* __restrict__ proj_t,
                                   const float* __restrict__ norm, int side, int vocab, float eps,
                                   float* __restrict__ history, int depth_index, const float* __restrict__ depth_weight,
                                   long long history_stride, int hidden) {
  extern __shared__ float smem[];
  float* x = smem;                   // [hidden]
  float* y = x + hidden;             // [hidden]
  float* g = y + hidden;             // [side]
  float* red = g + side;             // [33]
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const size_t base = (size_t)t * hidden;
  const bool adds = pending.a != nullptr || pending.b != nullptr;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = residual[base + c];
    if (adds) v += scale * pending_sum(pending, base + c);
    x[c] = v;
  }
  __syncthreads();
  if (table) {
    int token = token_ids[t];
    token = token < 0 ? 0 : (token >= vocab ? vocab - 1 : token);     // a bad id was reported by the embedding
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int d = warp; d < side; d += warps) {
      const TW* w = gate + (size_t)d * hidden;
      float dot = 0.f;
      for (int c = lane; c < hidden; c += 32) dot = fmaf(to_float(w[c]), x[c], dot);
      dot = warp_sum(dot);
      if (lane == 0) g[d] = gelu_tanh_f(dot) * to_float(table[(size_t)token * side + d]);
    }
    __syncthreads();
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      float acc = 0.f;
      for (int d = 0; d < side; ++d) acc = fmaf(to_float(proj_t[(size_t)d * hidden + c]), g[d], acc);
      y[c] = acc;
      ss = fmaf(acc, acc, ss);
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)hidden + eps);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) x[c] = fmaf(scale * inv * norm[c], y[c], x[c]);
    // every thread reads back the columns it wrote itself: no barrier is needed before the next loop
  }
  if (history) {
    float* mine = history + (size_t)(depth_index + 1) * history_stride + base;
    const float newest = depth_weight[depth_index + 1];
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float v = x[c];
      mine[c] = v;
      float acc = 0.f;
      for (int j = 0; j <= depth_index; ++j) acc = fmaf(depth_weight[j], history[(size_t)j * history_stride + base + c], acc);
      residual[base + c] = fmaf(newest, v, acc);
    }
  } else {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) residual[base + c] = x[c];
  }
}

// The same end of a layer for TB tokens a CTA, so the two token-input matrices are read once for all of them,
// in 16-byte pieces (hidden a multiple of 8).  s = gate x: a warp per pair of rows of gate, its lanes over the
// row's pieces, the tokens' x from shared memory.  y = proj_t^T g: a warp per eight pieces of columns, four
// lanes per piece that share the rows of proj_t and add up by shuffles in a fixed order.
constexpr int kTailThreads = 512;

template <typename TW>
__device__ __forceinline__ void piece_to_floats(const uint4& raw, float (&w)[8]);
template <>
__device__ __forceinline__ void piece_to_floats<__nv_bfloat16>(const uint4& raw, float (&w)[8]) {
  const __nv_bfloat162* p = (const __nv_bfloat162*)&raw;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(p[e]);
    w[2 * e] = f.x;
    w[2 * e + 1] = f.y;
  }
}

// eight weights of row `row` from column c on
template <typename TW>
__device__ __forceinline__ void load_piece(const TW* __restrict__ m, size_t at, float (&w)[8]) {
  if (sizeof(TW) == 2) {
    const uint4 raw = *(const uint4*)(m + at);
    piece_to_floats<__nv_bfloat16>(raw, w);
  } else {
    const float4 lo = *(const float4*)((const float*)m + at), hi = *(const float4*)((const float*)m + at + 4);
    w[0] = lo.x; w[1] = lo.y; w[2] = lo.z; w[3] = lo.w; w[4] = hi.x; w[5] = hi.y; w[6] = hi.z; w[7] = hi.w;
  }
}

template <typename TW, int TB>
__global__ void __launch_bounds__(kTailThreads)
stream_tail_tokens_kernel(float* __restrict__ residual, const __grid_constant__ Pending pending, float scale,
                          const int* __restrict__ token_ids, const TW* __restrict__ table, const TW* __restrict__ gate,
                          const TW* __restrict__ proj_t, const float* __restrict__ norm, int side, int vocab, float eps,
                          float* __restrict__ history, int depth_index, const float* __restrict__ depth_weight,
                          long long history_stride, int hidden, int num_tokens) {
  extern __shared__ float4 smem4[];
  float* x = (float*)smem4;          // [TB, hidden]
  float* y = x + TB * hidden;        // [TB, hidden]
  float* g = y + TB * hidden;        // [TB, side]
  float* red = g + TB * side;        // [TB, warps]
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int kWarps = kTailThreads / 32;
  const int t0 = blockIdx.x * TB;
  const int count = min(TB, num_tokens - t0);
  const bool adds = pending.a != nullptr || pending.b != nullptr;
  for (int idx = tid; idx < TB * hidden; idx += kTailThreads) {
    const int i = idx / hidden;
    float v = 0.f;
    if (i < count) {
      const size_t at = (size_t)t0 * hidden + idx;
      v = residual[at];
      if (adds) v += scale * pending_sum(pending, at);
    }
    x[idx] = v;
  }
  __syncthreads();
  if (table) {
    const int pieces = hidden / 8;
    // s = gate x, two rows a warp at a time
    for (int d0 = 2 * warp; d0 < side; d0 += 2 * kWarps) {
      float dot[2][TB];
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int i = 0; i < TB; ++i) dot[r][i] = 0.f;
#pragma unroll 4
      for (int p = lane; p < pieces; p += 32) {
        float w[2][8];
        load_piece<TW>(gate, (size_t)d0 * hidden + 8 * p, w[0]);
        if (d0 + 1 < side) load_piece<TW>(gate, (size_t)(d0 + 1) * hidden + 8 * p, w[1]);
#pragma unroll
        for (int i = 0; i < TB; ++i) {
          const float4 a = *(const float4*)(x + i * hidden + 8 * p), b = *(const float4*)(x + i * hidden + 8 * p + 4);
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            float acc = dot[r][i];
            acc = fmaf(w[r][0], a.x, acc); acc = fmaf(w[r][1], a.y, acc); acc = fmaf(w[r][2], a.z, acc);
            acc = fmaf(w[r][3], a.w, acc); acc = fmaf(w[r][4], b.x, acc); acc = fmaf(w[r][5], b.y, acc);
            acc = fmaf(w[r][6], b.z, acc); acc = fmaf(w[r][7], b.w, acc);
            dot[r][i] = acc;
          }
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int i = 0; i < TB; ++i) {
          const float total = warp_sum(dot[r][i]);
          if (lane == 0 && d0 + r < side && i < count) {
            int token = token_ids[t0 + i];
            token = token < 0 ? 0 : (token >= vocab ? vocab - 1 : token);     // a bad id was reported by the embedding
            g[i * side + d0 + r] = gelu_tanh_f(total) * to_float(table[(size_t)token * side + d0 + r]);
          }
        }
    }
    __syncthreads();
    // y = proj_t^T g
    float ss[TB];
#pragma unroll
    for (int i = 0; i < TB; ++i) ss[i] = 0.f;
    const int part = lane >> 3;                       // which quarter of the rows of proj_t
    for (int p = 8 * warp + (lane & 7); p - (lane & 7) < pieces; p += 8 * kWarps) {
      float acc[TB][8];
#pragma unroll
      for (int i = 0; i < TB; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
      if (p < pieces) {
#pragma unroll 8
        for (int d = part; d < side; d += 4) {
          float w[8];
          load_piece<TW>(proj_t, (size_t)d * hidden + 8 * p, w);
#pragma unroll
          for (int i = 0; i < TB; ++i) {
            const float gi = g[i * side + d];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[i][e] = fmaf(w[e], gi, acc[i][e]);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < TB; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float v = acc[i][e];
          v += __shfl_xor_sync(0xffffffffu, v, 8);
          v += __shfl_xor_sync(0xffffffffu, v, 16);
          acc[i][e] = v;
        }
      if (part == 0 && p < pieces) {
#pragma unroll
        for (int i = 0; i < TB; ++i) {
          if (i >= count) continue;
          *(float4*)(y + i * hidden + 8 * p) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
          *(float4*)(y + i * hidden + 8 * p + 4) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
#pragma unroll
          for (int e = 0; e < 8; ++e) ss[i] = fmaf(acc[i][e], acc[i][e], ss[i]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < TB; ++i) {
      const float total = warp_sum(ss[i]);
      if (lane == 0) red[i * kWarps + warp] = total;
    }
    __syncthreads();
    for (int idx = tid; idx < count * hidden; idx += kTailThreads) {
      const int i = idx / hidden, c = idx - i * hidden;
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) total += red[i * kWarps + w];
      const float inv = rsqrtf(total / (float)hidden + eps);
      x[idx] = fmaf(scale * inv * norm[c], y[idx], x[idx]);
    }
    // every thread reads back the elements it wrote itself: no barrier is needed before the next loop
  }
  if (history) {
    const float newest = depth_weight[depth_index + 1];
    for (int idx = tid; idx < count * hidden; idx += kTailThreads) {
      const size_t at = (size_t)t0 * hidden + idx;
      const float v = x[idx];
      history[(size_t)(depth_index + 1) * history_stride + at] = v;
      float acc = 0.f;
      constexpr int kBatch = 8;                         // earlier layers' results: several loads in flight
      for (int j0 = 0; j0 <= depth_index; j0 += kBatch) {
        float earlier[kBatch];
#pragma unroll
        for (int e = 0; e < kBatch; ++e)
          earlier[e] = j0 + e <= depth_index ? history[(size_t)(j0 + e) * history_stride + at] : 0.f;
#pragma unroll
        for (int e = 0; e < kBatch; ++e)
          if (j0 + e <= depth_index) acc = fmaf(depth_weight[j0 + e], earlier[e], acc);
      }
      residual[at] = fmaf(newest, v, acc);
    }
  } else {
    for (int idx = tid; idx < count * hidden; idx += kTailThreads) residual[(size_t)t0 * hidden + idx] = x[idx];
  }
}

static int row_threads(int hidden) {
  int threads = 64;
  while (threads < hidden / 4 && threads < 512) threads <<= 1;
  return threads;
}

}  // namespace einf

using namespace einf;

extern "C" int einf_norm_conv(const void* pend_a, int a_dtype, int a_splits, long long a_stride, const void* pend_b,
                              int b_dtype, int b_splits, long long b_stride, float scale, float* residual,
                              const float* weight, float eps, const float* conv_weight, int taps, float* conv_state,
                              long long state_stride, int num_slots, const int* seq_of_token, const int* q_start,
                              const int* state_slots, int num_requests, void* out, int out_dtype, float* scratch,
                              int num_tokens, int hidden, int single_tokens, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (taps > kMaxTaps || hidden <= 0 || num_requests > 65535) return (int)cudaErrorInvalidValue;
  const Pending pending{pend_a, a_dtype, a_splits, a_stride, pend_b, b_dtype, b_splits, b_stride};
  const bool conv = conv_weight != nullptr && taps > 1;
  if (conv && (!conv_state || (!single_tokens && !scratch))) return (int)cudaErrorInvalidValue;
  const int mode = !conv ? 0 : (single_tokens ? 1 : 2);
  const int threads = row_threads(hidden);
  const size_t smem = (size_t)(hidden + 33) * sizeof(float);
  EINF_DISPATCH_2(out_dtype, T, {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(norm_row_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    cudaError_t e = launch_pdl(norm_row_kernel<T>, num_tokens, threads, smem, stream, pending, scale, residual, weight,
                               eps, conv_weight, taps, conv_state, state_stride, num_slots, seq_of_token, state_slots,
                               (T*)out, scratch, hidden, mode);
    if (e != cudaSuccess || mode != 2) return (int)e;
    const long long total = (long long)num_tokens * hidden;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    e = launch_pdl(conv_rows_kernel<T>, (int)blocks, 256, 0, stream, (const float*)scratch, conv_weight, taps,
                   (const float*)conv_state, state_stride, num_slots, seq_of_token, q_start, state_slots, (T*)out,
                   hidden, num_tokens);
    if (e != cudaSuccess) return (int)e;
    const dim3 grid((hidden + 127) / 128, num_requests);
    return (int)launch_pdl(conv_rows_state_kernel, grid, 128, 0, stream, (const float*)scratch, conv_state,
                           state_stride, num_slots, q_start, state_slots, hidden, taps);
  })
}

extern "C" int einf_stream_tail(float* residual, const void* pend_a, int a_dtype, int a_splits, long long a_stride,
                                const void* pend_b, int b_dtype, int b_splits, long long b_stride, float scale,
                                const int* token_ids, const void* table, const void* gate, const void* proj_t,
                                int weight_dtype, const float* norm, int side, int vocab, float eps, float* history,
                                int depth_index, const float* depth_weight, long long history_stride, int num_tokens,
                                int hidden, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (hidden <= 0 || side < 0) return (int)cudaErrorInvalidValue;
  const Pending pending{pend_a, a_dtype, a_splits, a_stride, pend_b, b_dtype, b_splits, b_stride};
  if (hidden % 8 == 0 && side > 0 && ((uintptr_t)gate | (uintptr_t)proj_t) % 16 == 0) {
    // tokens a CTA: eight for a long step where they fit beside a second CTA, else four; one while every token
    // still gets an SM of its own (the step is then bound by one CTA's instructions, not by the matrices' bytes)
    auto bytes = [&](int each) { return (size_t)(2 * each * hidden + each * side + each * (kTailThreads / 32)) * sizeof(float); };
    const int each = (num_tokens >= 1024 && bytes(8) <= 100 * 1024) ? 8 : (num_tokens <= 148 ? 1 : 4);
    if (bytes(each) <= 200 * 1024) {
      const int blocks = (num_tokens + each - 1) / each;
#define EINF_TAIL(TB)                                                                                                   \
  EINF_DISPATCH_2(weight_dtype, T, {                                                                                    \
    auto kernel = stream_tail_tokens_kernel<T, TB>;                                                                     \
    if (bytes(TB) > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes(TB));        \
      if (e != cudaSuccess) return (int)e;                                                                              \
    }                                                                                                                   \
    return (int)launch_pdl(kernel, blocks, kTailThreads, bytes(TB), stream, residual, pending, scale, token_ids,       \
                           (const T*)table, (const T*)gate, (const T*)proj_t, norm, side, vocab, eps, history,          \
                           depth_index, depth_weight, history_stride, hidden, num_tokens);                              \
  })
      if (each == 8) EINF_TAIL(8)
      if (each == 1) EINF_TAIL(1)
      EINF_TAIL(4)
#undef EINF_TAIL
    }
  }
  const int threads = row_threads(hidden);
  const size_t smem = (size_t)(2 * hidden + side + 33) * sizeof(float);
  EINF_DISPATCH_2(weight_dtype, T, {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(stream_tail_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    return (int)launch_pdl(stream_tail_kernel<T>, num_tokens, threads, smem, stream, residual, pending, scale,
                           token_ids, (const T*)table, (const T*)gate, (const T*)proj_t, norm, side, vocab, eps,
                           history, depth_index, depth_weight, history_stride, hidden);
  })
}
