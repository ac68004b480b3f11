// A routed feed-forward (mixture of experts) in five steps, all on the device so that a step
// never waits for the host to learn how many tokens an expert got:
//
//   einf_router_topk   per token: the `top_k` largest router logits (ties to the lower index),
//                      their weights sigmoid(z) or softmax(z) over all experts, optionally
//                      divided by their sum; 32-bit throughout.  With a correction the choice goes
//                      by score + correction (the weights stay the scores); with groups only the
//                      experts of the `keep` groups of neighbours whose best choice score is
//                      largest can be chosen
//   einf_moe_dispatch  counts per expert, offsets (experts in order), the place of every
//                      (token, choice) in the order sorted by expert, and the rows gathered into
//                      that order (times the router weight where the weight acts on the input);
//                      one CTA does all of it for a decode step's few pairs, four launches otherwise
//   einf_moe_gemm      out[p] = W[expert of p] x[p] for the sorted rows: a tiled product whose row
//                      tiles never cross an expert; 32-bit FMA, operands float32 or bfloat16
//   (the activation between the two products is the ordinary silu-and-multiply kernel)
//   einf_moe_combine   out[t] = sum_s addend[s][t] + sum_j (w_tj) y[place(t, j)], in 32-bit and in
//                      a fixed order: the experts' outputs of a token (or their split-K partial
//                      sums), and, for a parallel layer, the other branch's output (possibly
//                      partial sums too), in one pass; a choice beyond the experts hands the
//                      token's own row through (times its weight), and the addend may carry a
//                      sigmoid gate of one number per token
//
// A row's result depends on that row, its expert and its weight alone: which other tokens share
// the batch moves nothing.  (The place of a row inside its expert's range is first come, first
// served; no value depends on it.)
#include "common.cuh"

namespace einf {

enum RouterScore : int { kScoreSigmoid = 0, kScoreSoftmax = 1 };

constexpr int kMaxExpertsPerLane = 32;   // experts up to 1024

__global__ void router_topk_kernel(const float* __restrict__ logits, int splits, size_t split_stride, int num_tokens,
                                   int row_width, int num_experts, int top_k, int score, int renormalise,
                                   const float* __restrict__ correction, int group_count, int group_keep,
                                   int* __restrict__ expert_ids, float* __restrict__ weights) {
  // per warp of the CTA: [num_experts] what the choice goes by | [num_experts] the scores (with a correction) |
  // [group_count] 1 for a group that may be chosen from
  extern __shared__ float z_all[];
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (t >= num_tokens) return;
  const int per_warp = (correction ? 2 : 1) * num_experts + group_count;
  float* z = z_all + (threadIdx.x >> 5) * per_warp;
  float* s_all = correction ? z + num_experts : z;
  float* group_open = z + (correction ? 2 : 1) * num_experts;
  for (int e = lane; e < num_experts; e += 32) {
    float v = 0.f;
    for (int s = 0; s < splits; ++s) v += logits[(size_t)s * split_stride + (size_t)t * row_width + e];
    z[e] = v;
  }
  __syncwarp();
  float z_max = -INFINITY;
  for (int e = lane; e < num_experts; e += 32) z_max = fmaxf(z_max, z[e]);
  z_max = warp_max(z_max);
  float denominator = 1.f;
  if (score == kScoreSoftmax) {
    float sum = 0.f;
    for (int e = lane; e < num_experts; e += 32) sum += expf(z[e] - z_max);
    denominator = warp_sum(sum);
  }
  if (correction) {
    // the scores themselves, and what the choice goes by in their place
    __syncwarp();
    for (int e = lane; e < num_experts; e += 32) {
      const float w = score == kScoreSoftmax ? expf(z[e] - z_max) / denominator : 1.f / (1.f + expf(-z[e]));
      s_all[e] = w;
      z[e] = w + correction[e];
    }
    __syncwarp();
  }
  if (group_count > 0) {
    // a group's score is its best choice score; the `group_keep` best groups stay open (ties to the lower index)
    const int per_group = num_experts / group_count;
    for (int g = lane; g < group_count; g += 32) group_open[g] = 0.f;
    __syncwarp();
    for (int j = 0; j < group_keep; ++j) {
      float best = -INFINITY;
      int best_g = 0x7fffffff;
      for (int g = lane; g < group_count; g += 32) {
        if (group_open[g] != 0.f) continue;
        float top = -INFINITY;
        for (int i = 0; i < per_group; ++i) top = fmaxf(top, z[g * per_group + i]);
        if (top > best || best_g == 0x7fffffff) {
          best = top;
          best_g = g;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, best, o);
        const int other_g = __shfl_xor_sync(0xffffffffu, best_g, o);
        if (other_g != 0x7fffffff && (best_g == 0x7fffffff || other > best || (other == best && other_g < best_g))) {
          best = other;
          best_g = other_g;
        }
      }
      if (lane == 0 && best_g != 0x7fffffff) group_open[best_g] = 1.f;
      __syncwarp();
    }
  }
  uint32_t taken = 0;   // bit i: expert lane + 32 i is chosen already
  float chosen_sum = 0.f;
  for (int j = 0; j < top_k; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane, i = 0; e < num_experts; e += 32, ++i) {
      if (taken & (1u << i)) continue;
      if (group_count > 0 && group_open[e / (num_experts / group_count)] == 0.f) continue;
      const float v = z[e];
      if (v > best || (v == best && e < best_e) || best_e == 0x7fffffff) {
        best = v;
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_e = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (other_e != 0x7fffffff && (best_e == 0x7fffffff || other > best || (other == best && other_e < best_e))) {
        best = other;
        best_e = other_e;
      }
    }
    if ((best_e & 31) == lane) taken |= 1u << (best_e >> 5);
    float w;
    if (correction) w = s_all[best_e];
    else w = score == kScoreSoftmax ? expf(best - z_max) / denominator : 1.f / (1.f + expf(-best));
    chosen_sum += w;
    if (lane == 0) {
      expert_ids[(size_t)t * top_k + j] = best_e;
      weights[(size_t)t * top_k + j] = w;
    }
  }
  if (renormalise && lane == 0) {
    for (int j = 0; j < top_k; ++j) weights[(size_t)t * top_k + j] /= chosen_sum;
  }
}

// work: [counts E | cursor E | offsets E + 1] int32
__global__ void moe_count_kernel(const int* __restrict__ expert_ids, int assignments, int num_experts,
                                 int* __restrict__ work) {
  pdl_launch_dependents();
  pdl_wait();
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p < assignments) {
    const int e = expert_ids[p];
    if (e >= 0 && e < num_experts) atomicAdd(work + e, 1);
  }
}

__global__ void moe_zero_kernel(int* __restrict__ work, int n) {
  pdl_launch_dependents();
  pdl_wait();
  for (int i = threadIdx.x; i < n; i += blockDim.x) work[i] = 0;
}

__global__ void moe_scan_kernel(int* __restrict__ work, int num_experts) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    int* counts = work;
    int* cursor = work + num_experts;
    int* offsets = work + 2 * num_experts;
    int sum = 0;
    for (int e = 0; e < num_experts; ++e) {
      offsets[e] = sum;
      cursor[e] = sum;
      sum += counts[e];
    }
    offsets[num_experts] = sum;
  }
}

template <typename T>
__global__ void moe_place_kernel(const T* __restrict__ x, const int* __restrict__ expert_ids,
                                 const float* __restrict__ weights, int assignments, int top_k, int num_experts,
                                 int hidden, int scale_rows, int* __restrict__ work, int* __restrict__ place,
                                 T* __restrict__ sorted_x) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int p = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (p >= assignments) return;
  const int e = expert_ids[p];
  if (e < 0 || e >= num_experts) return;
  int at = 0;
  if (lane == 0) {
    at = atomicAdd(work + num_experts + e, 1);
    place[p] = at;
  }
  at = __shfl_sync(0xffffffffu, at, 0);
  const float w = scale_rows ? weights[p] : 1.f;
  const T* src = x + (size_t)(p / top_k) * hidden;
  T* dst = sorted_x + (size_t)at * hidden;
  for (int d = lane; d < hidden; d += 32) dst[d] = from_float<T>(to_float(src[d]) * w);
}

// The same four steps in one CTA, for the few hundred (token, choice) pairs of a decode step: counts and
// cursors live in shared memory, one thread scans them, every warp then copies rows.
constexpr int kSmallDispatchThreads = 256;
constexpr int kSmallDispatchPairs = 1024;     // pairs one CTA takes
constexpr int kSmallDispatchExperts = 1024;

template <typename T>
__global__ void __launch_bounds__(kSmallDispatchThreads)
moe_dispatch_small_kernel(const T* __restrict__ x, const int* __restrict__ expert_ids, const float* __restrict__ weights,
                          int assignments, int top_k, int num_experts, int hidden, int scale_rows,
                          int* __restrict__ work, int* __restrict__ place, T* __restrict__ sorted_x) {
  __shared__ int counts[kSmallDispatchExperts];
  __shared__ int at_s[kSmallDispatchPairs];
  pdl_launch_dependents();
  pdl_wait();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < assignments; p += blockDim.x) {
    const int e = expert_ids[p];
    if (e >= 0 && e < num_experts) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int* offsets = work + 2 * num_experts;
    int sum = 0;
    for (int e = 0; e < num_experts; ++e) {
      const int count = counts[e];
      offsets[e] = sum;
      counts[e] = sum;          // from here on: the expert's cursor
      sum += count;
    }
    offsets[num_experts] = sum;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < assignments; p += blockDim.x) {
    const int e = expert_ids[p];
    int at = -1;
    if (e >= 0 && e < num_experts) {
      at = atomicAdd(&counts[e], 1);
      place[p] = at;
    }
    at_s[p] = at;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int p = warp; p < assignments; p += kSmallDispatchThreads / 32) {
    const int at = at_s[p];
    if (at < 0) continue;
    const float w = scale_rows ? weights[p] : 1.f;
    const T* src = x + (size_t)(p / top_k) * hidden;
    T* dst = sorted_x + (size_t)at * hidden;
    for (int d = lane; d < hidden; d += 32) dst[d] = from_float<T>(to_float(src[d]) * w);
  }
}

// Tiled product over rows sorted by expert.  A CTA owns 32 rows of one expert and 64 output
// columns; which expert and which of its row tiles is found by walking the offsets.
constexpr int kTileRows = 32, kTileCols = 64, kTileK = 32;

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const TX* __restrict__ x, const TW* __restrict__ w, const int* __restrict__ offsets,
                TO* __restrict__ out, int num_experts, int n, int k) {
  __shared__ float xs[kTileRows][kTileK + 1];
  __shared__ float ws[kTileCols][kTileK + 1];
  pdl_launch_dependents();
  pdl_wait();
  int expert = -1, row0 = 0, rows = 0;
  {
    int tile = blockIdx.x;
    for (int e = 0; e < num_experts; ++e) {
      const int begin = offsets[e], count = offsets[e + 1] - begin;
      const int tiles = (count + kTileRows - 1) / kTileRows;
      if (tile < tiles) {
        expert = e;
        row0 = begin + tile * kTileRows;
        rows = min(kTileRows, count - tile * kTileRows);
        break;
      }
      tile -= tiles;
    }
  }
  if (expert < 0) return;
  const int col0 = blockIdx.y * kTileCols;
  const TW* we = w + (size_t)expert * n * k;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;   // rows ty*2 .. +1, columns tx*4 .. +3
  float acc[2][4] = {};
  for (int k0 = 0; k0 < k; k0 += kTileK) {
    for (int i = threadIdx.x; i < kTileRows * kTileK; i += 256) {
      const int r = i / kTileK, c = i - r * kTileK;
      xs[r][c] = (r < rows && k0 + c < k) ? to_float(x[(size_t)(row0 + r) * k + k0 + c]) : 0.f;
    }
    for (int i = threadIdx.x; i < kTileCols * kTileK; i += 256) {
      const int r = i / kTileK, c = i - r * kTileK;
      ws[r][c] = (col0 + r < n && k0 + c < k) ? to_float(we[(size_t)(col0 + r) * k + k0 + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < kTileK; ++c) {
      const float a0 = xs[ty * 2][c], a1 = xs[ty * 2 + 1][c];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b = ws[tx * 4 + j][c];
        acc[0][j] = fmaf(a0, b, acc[0][j]);
        acc[1][j] = fmaf(a1, b, acc[1][j]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = ty * 2 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col0 + tx * 4 + j;
      if (c < n) out[(size_t)(row0 + r) * n + c] = from_float<TO>(acc[i][j]);
    }
  }
}

// Sum of `count` values `stride` apart, added in order; the loads go out eight at a time.
template <typename T>
__device__ __forceinline__ float sum_strided(const T* __restrict__ p, int count, size_t stride) {
  float v = 0.f;
  int s = 0;
  for (; s + 8 <= count; s += 8) {
    float t[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) t[u] = to_float(p[(size_t)(s + u) * stride]);
#pragma unroll
    for (int u = 0; u < 8; ++u) v += t[u];
  }
  if (s < count) {
    float t[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) t[u] = s + u < count ? to_float(p[(size_t)(s + u) * stride]) : 0.f;
#pragma unroll
    for (int u = 0; u < 8; ++u) v += t[u];
  }
  return v;
}

// One thread a (token, column), so that a decode step's handful of tokens still spreads over the GPU;
// with hundreds of tokens a thread takes kColumns columns 128 apart (a quarter of the CTAs, and a
// token's places and experts are read once for four columns).
template <typename TY, typename TA, typename TX, int kColumns>
__global__ void __launch_bounds__(128)
moe_combine_kernel(const TY* __restrict__ y, const int* __restrict__ expert_ids,
                                   const int* __restrict__ place,
                                   const float* __restrict__ weights, int scale_outputs, const TA* __restrict__ addend,
                                   int splits, size_t split_stride, float* __restrict__ out, int num_experts,
                                   int top_k, int hidden, int y_splits, size_t y_stride,
                                   const TX* __restrict__ identity_x, int num_identity,
                                   const float* __restrict__ gate_logits, int gate_width, int gate_column,
                                   int gate_splits, size_t gate_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.y;
  const int d0 = blockIdx.x * (128 * kColumns) + threadIdx.x;
  float v[kColumns];
  float addend_gate = 1.f;
  if (gate_logits) {
    const float z = sum_strided(gate_logits + (size_t)t * gate_width + gate_column, gate_splits, gate_stride);
    addend_gate = 1.f / (1.f + expf(-z));
  }
#pragma unroll
  for (int c = 0; c < kColumns; ++c) {
    const int d = d0 + 128 * c;
    v[c] = (addend && d < hidden) ? sum_strided(addend + (size_t)t * hidden + d, splits, split_stride) : 0.f;
    if (gate_logits) v[c] *= addend_gate;
  }
  for (int j = 0; j < top_k; ++j) {
    const int p = t * top_k + j;
    const int e = expert_ids[p];
    if (e >= num_experts && e < num_experts + num_identity) {
      // an expert that hands the token through: its weight times the token's own row
      const float w = weights[p];
#pragma unroll
      for (int c = 0; c < kColumns; ++c) {
        const int d = d0 + 128 * c;
        if (d < hidden) v[c] += w * to_float(identity_x[(size_t)t * hidden + d]);
      }
      continue;
    }
    if (e < 0 || e >= num_experts) continue;
    const TY* row = y + (size_t)place[p] * hidden;
    const float w = scale_outputs ? weights[p] : 1.f;
#pragma unroll
    for (int c = 0; c < kColumns; ++c) {
      const int d = d0 + 128 * c;
      if (d < hidden) {
        const float term = sum_strided(row + d, y_splits, y_stride);
        v[c] += scale_outputs ? w * term : term;
      }
    }
  }
#pragma unroll
  for (int c = 0; c < kColumns; ++c) {
    const int d = d0 + 128 * c;
    if (d < hidden) out[(size_t)t * hidden + d] = v[c];
  }
}

}  // namespace einf

using namespace einf;

extern "C" int einf_router_topk(const float* logits, int splits, long long split_stride, int num_tokens,
                                int row_width, int num_experts, int top_k, int score, int renormalise,
                                const float* correction, int group_count, int group_keep, int* expert_ids,
                                float* weights, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (num_experts <= 0 || num_experts > 32 * kMaxExpertsPerLane || top_k <= 0 || top_k > num_experts ||
      row_width < num_experts)
    return (int)cudaErrorInvalidValue;
  if (group_count < 0 || (group_count > 0 && (num_experts % group_count || group_keep <= 0 || group_keep > group_count ||
                                              top_k > group_keep * (num_experts / group_count))))
    return (int)cudaErrorInvalidValue;
  const int threads = 128;
  const int blocks = (num_tokens * 32 + threads - 1) / threads;
  const size_t per_warp = (size_t)(correction ? 2 : 1) * num_experts + group_count;
  return (int)launch_pdl(router_topk_kernel, blocks, threads, (size_t)(threads / 32) * per_warp * sizeof(float), stream,
                         logits, splits < 1 ? 1 : splits, (size_t)split_stride, num_tokens, row_width, num_experts, top_k,
                         score, renormalise, correction, group_count, group_keep, expert_ids, weights);
}

// x: [T, hidden]; expert_ids, weights, place: [T * top_k]; work: [3 E + 1] int32 (offsets are its last
// E + 1 entries); sorted_x: [T * top_k, hidden].
extern "C" int einf_moe_dispatch(const void* x, int dtype, const int* expert_ids, const float* weights, int num_tokens,
                                 int top_k, int num_experts, int hidden, int scale_rows, int* work, int* place,
                                 void* sorted_x, cudaStream_t stream) {
  const int assignments = num_tokens * top_k;
  if (assignments == 0) return 0;
  if (assignments <= 64 && num_experts <= kSmallDispatchExperts) {   // beyond that one CTA's copying costs more than three launches
    EINF_DISPATCH_2(dtype, T, {
      return (int)launch_pdl(moe_dispatch_small_kernel<T>, 1, kSmallDispatchThreads, 0, stream, (const T*)x, expert_ids,
                             weights, assignments, top_k, num_experts, hidden, scale_rows, work, place, (T*)sorted_x);
    })
  }
  cudaError_t e = launch_pdl(moe_zero_kernel, 1, 256, 0, stream, work, 3 * num_experts + 1);
  if (e != cudaSuccess) return (int)e;
  e = launch_pdl(moe_count_kernel, (assignments + 255) / 256, 256, 0, stream, expert_ids, assignments, num_experts, work);
  if (e != cudaSuccess) return (int)e;
  e = launch_pdl(moe_scan_kernel, 1, 32, 0, stream, work, num_experts);
  if (e != cudaSuccess) return (int)e;
  const int threads = 128;
  const int blocks = (int)(((long long)assignments * 32 + threads - 1) / threads);
  EINF_DISPATCH_2(dtype, T, {
    return (int)launch_pdl(moe_place_kernel<T>, blocks, threads, 0, stream, (const T*)x, expert_ids, weights, assignments,
                           top_k, num_experts, hidden, scale_rows, work, place, (T*)sorted_x);
  })
}

// x: [rows, k] sorted by expert; w: [E, n, k]; offsets: [E + 1]; out: [rows, n].
extern "C" int einf_moe_gemm(const void* x, int x_dtype, const void* w, int w_dtype, const int* offsets, void* out,
                             int out_dtype, int rows, int num_experts, int n, int k, cudaStream_t stream) {
  if (rows == 0 || n == 0) return 0;
  const int most_tiles = (rows + kTileRows - 1) / kTileRows + (num_experts < rows ? num_experts : rows);
  dim3 grid(most_tiles, (n + kTileCols - 1) / kTileCols);
  EINF_DISPATCH_2(x_dtype, TX, {
    EINF_DISPATCH_2(w_dtype, TW, {
      EINF_DISPATCH_2(out_dtype, TO, {
        return (int)launch_pdl(moe_gemm_kernel<TX, TW, TO>, grid, dim3(256), 0, stream, (const TX*)x, (const TW*)w,
                               offsets, (TO*)out, num_experts, n, k);
      })
    })
  })
}

// y: [T * top_k, hidden] sorted by expert (or y_splits float32 partial sums of it, stacked); addend: null, [T, hidden] or `splits` partial sums of it; out: float32 [T, hidden].
extern "C" int einf_moe_combine(const void* y, int y_dtype, const int* expert_ids, const int* place,
                                const float* weights, int scale_outputs, const void* addend, int addend_dtype,
                                int splits, long long split_stride, float* out, int num_tokens, int num_experts,
                                int top_k, int hidden, int y_splits, const void* identity_x, int identity_dtype,
                                int num_identity, const float* gate_logits, int gate_width, int gate_column,
                                int gate_splits, long long gate_stride, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (num_tokens > 65535) return (int)cudaErrorInvalidValue;
  if (num_identity < 0 || (num_identity > 0 && (!identity_x || !weights))) return (int)cudaErrorInvalidValue;
  if (gate_logits && (!addend || gate_column < 0 || gate_column >= gate_width)) return (int)cudaErrorInvalidValue;
  const bool many = num_tokens >= 128;
  const dim3 grid(many ? (hidden + 511) / 512 : (hidden + 127) / 128, num_tokens);
  EINF_DISPATCH_2(y_dtype, TY, {
    EINF_DISPATCH_2(addend_dtype, TA, {
      EINF_DISPATCH_2(identity_dtype, TX, {
        return (int)launch_pdl(many ? moe_combine_kernel<TY, TA, TX, 4> : moe_combine_kernel<TY, TA, TX, 1>, grid,
                               dim3(128), 0, stream, (const TY*)y, expert_ids, place,
                               weights, scale_outputs, (const TA*)addend, splits, (size_t)split_stride, out,
                               num_experts, top_k, hidden, y_splits < 1 ? 1 : y_splits,
                               (size_t)num_tokens * top_k * hidden, (const TX*)identity_x, num_identity, gate_logits,
                               gate_width, gate_column, gate_splits < 1 ? 1 : gate_splits, (size_t)gate_stride);
      })
    })
  })
}
