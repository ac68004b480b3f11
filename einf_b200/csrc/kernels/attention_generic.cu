// Paged causal attention for any batch: prompt portions and single decoded
// tokens alike, float or bfloat16, any head size up to 256 (16-byte loads where
// the size allows them), any number of heads and groups, with an optional
// sliding window, chunked mask and soft cap on the scores.
//
// This is the 32-bit path's attention and the fallback of the bfloat16 path for
// sizes its tensor-core kernels do not cover.  One warp owns one (token, query
// head) row and walks the keys of its request 32 at a time straight from the
// pages named by the block table:
//   scores: lane j computes q . K[j] in 32-bit (q is pre-multiplied by scale)
//   online softmax in 32-bit across the warp (max, exp, sum)
//   output: lane d accumulates sum_j p_j V[j][d] in 32-bit
// (reference for the maths: src/einf/executors/torch/ops/csrc/paged_attention_cuda.cu:74-147
// and flash_attention_cuda.cu:126-195; lower-right causal mask model_runner.py:145.)
// A token at position p of request r sees keys lo..p of r, lo = max(0, p - window + 1); with a
// chunk size c (chunked attention) lo is also at least floor(p / c) * c, the first position of p's
// own chunk, counted from position 0 of the sequence.  With a soft cap z the scaled score s becomes
// z * tanh(s / z) before the softmax.  Keys and values may have different sizes per head.
// With `keep_first` n > 0 a windowed token also sees the first n positions of its sequence
// (j < n), at their true positions.  With `sink` (one float per query head) the softmax's
// denominator of head h also holds exp(sink[h]): a column with no key and no value, unscaled.
// `value_stride` is the distance between two value rows in
// elements: value_size for a cache of its own, the key size when the values are the leading
// elements of the key rows (a latent cache that holds one row per token for both).
// The kernel exists twice: for sizes up to 256 and for sizes up to 640 (more registers a lane).
#include "common.cuh"

namespace einf {

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxHeadSize = 640;

template <typename T>
struct Vec;  // 16-byte vector of T
template <>
struct Vec<float> {
  static constexpr int N = 4;
  float4 raw;
  __device__ __forceinline__ float get(int i) const { return (&raw.x)[i]; }
};
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ __forceinline__ float get(int i) const {
    const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(&raw);
    return __bfloat162float(p[i]);
  }
};

template <typename T, int kHeadLimit>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
paged_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_cache,
                               const T* __restrict__ v_cache, const int* __restrict__ block_table,
                               const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                               T* __restrict__ out, int num_rows, int num_heads, int num_kv_heads,
                               int head_size, int value_size, int value_stride, int page_size, int num_pages,
                               int table_width, float scale, int window, int keep_first, int chunk, float softcap,
                               const float* __restrict__ sink, int* status) {
  __shared__ float q_smem[kWarpsPerBlock][kHeadLimit];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerBlock + warp;
  if (row >= num_rows) return;
  const int t = row / num_heads;
  const int h = row - t * num_heads;
  const int kv_head = h / (num_heads / num_kv_heads);
  const int r = seq_of_token[t];
  const int pos = positions[t];
  int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  if (chunk > 0) lo = max(lo, (pos / chunk) * chunk);
  const bool vectors = head_size % Vec<T>::N == 0;
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  const int* table = block_table + (size_t)r * table_width;

  const T* q_row = q + (size_t)row * head_size;
  for (int d = lane; d < head_size; d += 32) q_smem[warp][d] = to_float(q_row[d]) * scale;
  __syncwarp();
  const float* qs = q_smem[warp];

  constexpr int kDimsPerLane = kHeadLimit / 32;
  float acc[kDimsPerLane];
#pragma unroll
  for (int i = 0; i < kDimsPerLane; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  bool bad_page = false;

  // Two ranges of keys: the kept first positions below the window (empty without them), then
  // the window itself.
  const int kept = (window > 0 && keep_first > 0) ? min(keep_first, lo) : 0;
  for (int range = kept > 0 ? 0 : 1; range < 2; ++range) {
  const int first = range == 0 ? 0 : lo;
  const int last = range == 0 ? kept - 1 : pos;
  for (int base = first; base <= last; base += 32) {
    const int j = base + lane;
    float s = -INFINITY;
    long long key_row = -1;  // index of the (page, kv_head, slot) row in the caches, or -1
    if (j <= last) {
      const int logical = j / page_size;
      const int page = table[logical];
      if (page < 0 || page >= num_pages) {
        bad_page = true;
      } else {
        key_row = ((long long)page * num_kv_heads + kv_head) * page_size + (j - logical * page_size);
        const T* k_row = k_cache + key_row * head_size;
        float dot = 0.f;
        if (vectors) {
          for (int d = 0; d < head_size; d += Vec<T>::N) {
            Vec<T> kv;
            kv.raw = *reinterpret_cast<const decltype(kv.raw)*>(k_row + d);
#pragma unroll
            for (int e = 0; e < Vec<T>::N; ++e) dot = fmaf(qs[d + e], kv.get(e), dot);
          }
        } else {
          for (int d = 0; d < head_size; ++d) dot = fmaf(qs[d], to_float(k_row[d]), dot);
        }
        s = softcap > 0.f ? softcap * tanhf(dot * inv_cap) : dot;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    // m_new is finite unless every key so far had a bad page (the kept range comes first, so
    // key `pos` itself may still be ahead): then nothing is added.
    const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
    const float correction = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * correction + warp_sum(p);
#pragma unroll
    for (int i = 0; i < kDimsPerLane; ++i) acc[i] *= correction;
    m = m_new;
    const int count = min(32, last - base + 1);
    for (int kk = 0; kk < count; ++kk) {
      const float pj = __shfl_sync(0xffffffffu, p, kk);
      const long long off = __shfl_sync(0xffffffffu, key_row, kk);
      if (off < 0) continue;
      const T* v_row = v_cache + off * value_stride;
#pragma unroll
      for (int i = 0; i < kDimsPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < value_size) acc[i] = fmaf(pj, to_float(v_row[d]), acc[i]);
      }
    }
  }
  }
  if (__any_sync(0xffffffffu, bad_page) && lane == 0) atomicOr(status, kStatusBadPage);
  float inv = l > 0.f ? 1.f / l : 0.f;
  if (sink) {
    // one more term of the denominator, against the larger of the two maxima
    const float s = sink[h];
    const float top = fmaxf(m, s);
    const float keys = (m == -INFINITY) ? 0.f : l * expf(m - top);
    inv = (m == -INFINITY) ? 0.f : expf(m - top) / (keys + expf(s - top));
  }
  T* o_row = out + (size_t)row * value_size;
#pragma unroll
  for (int i = 0; i < kDimsPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d < value_size) o_row[d] = from_float<T>(acc[i] * inv);
  }
}

// ---------------------------------------------------------------------------
// Decode steps over rows that all query heads share (one key/value head whose values are the
// leading `value_size` elements of its key rows: a latent cache).  The kernel above gives every
// (token, head) a warp that walks all keys alone and reads each key row once per head; here a CTA
// takes one token, up to sixteen of its heads and one share of its keys, stages 32 key rows at a
// time in shared memory (read once from global memory for all sixteen heads, 16 bytes per
// access), and its eight warps take two heads each: a lane owns one key of the tile for the
// scores and a stripe of value dimensions for the mixing.  The shares of a token's keys (grid x)
// leave unnormalised (accumulator, maximum, sum) triples in a workspace, which a second kernel
// adds up in share order; with one share the CTA writes the result itself.
// Arithmetic and order of additions are 32-bit and fixed per (token, head): nothing depends on
// what else the batch holds.
// ---------------------------------------------------------------------------
constexpr int kSharedWarps = 8;
constexpr int kSharedHeads = 2 * kSharedWarps;   // heads a CTA takes
constexpr int kSharedTile = 32;                  // keys per tile

template <typename T, int kDimsPerLane>
__global__ void __launch_bounds__(kSharedWarps * 32)
latent_decode_attention_kernel(const T* __restrict__ q, const T* __restrict__ cache, const int* __restrict__ block_table,
                               const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                               T* __restrict__ out, float* __restrict__ part_acc, float* __restrict__ part_ml,
                               int num_heads, int row_size, int value_size, int page_size, int num_pages,
                               int table_width, float scale, int* status) {
  extern __shared__ __align__(16) unsigned char shared_raw[];
  // rows start on 16-byte borders, 16 bytes off a multiple of the row's own length
  const int row_pad = (row_size + 16 / (int)sizeof(T) - 1) / (16 / (int)sizeof(T)) * (16 / (int)sizeof(T)) + 16 / (int)sizeof(T);
  float* q_s = reinterpret_cast<float*>(shared_raw);              // [kSharedHeads][row_size]
  T* k_s = reinterpret_cast<T*>(q_s + kSharedHeads * row_size);   // [kSharedTile][row_pad]
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.y, split = blockIdx.x, splits = gridDim.x;
  const int head0 = blockIdx.z * kSharedHeads;
  const int heads_here = min(kSharedHeads, num_heads - head0);
  const int pos = positions[t];
  const int* table = block_table + (size_t)seq_of_token[t] * table_width;
  int per = (pos + 1 + splits - 1) / splits;
  per = (per + kSharedTile - 1) / kSharedTile * kSharedTile;
  const int k_begin = min(pos + 1, split * per), k_end = min(pos + 1, k_begin + per);

  for (int i = threadIdx.x; i < heads_here * row_size; i += blockDim.x) {
    const int h = i / row_size, d = i - h * row_size;
    q_s[h * row_size + d] = to_float(q[((size_t)t * num_heads + head0 + h) * row_size + d]) * scale;
  }
  const int h_a = 2 * warp, h_b = 2 * warp + 1;                   // this warp's heads (within the CTA's)
  const bool has_a = h_a < heads_here, has_b = h_b < heads_here;
  float acc_a[kDimsPerLane], acc_b[kDimsPerLane];
#pragma unroll
  for (int i = 0; i < kDimsPerLane; ++i) acc_a[i] = acc_b[i] = 0.f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  bool bad_page = false;
  const bool vectors = (row_size * sizeof(T)) % 16 == 0;
  constexpr int kVec = 16 / sizeof(T);

  for (int key0 = k_begin; key0 < k_end; key0 += kSharedTile) {
    __syncthreads();                                             // the tile before is used up (and q_s is written)
    // eight threads a key row
    {
      const int j = threadIdx.x >> 3, part = threadIdx.x & 7;
      const int key = key0 + j;
      T* dst = k_s + j * row_pad;
      int page = key < k_end ? table[key / page_size] : -1;
      if (key < k_end && (page < 0 || page >= num_pages)) {
        bad_page = true;
        page = -1;
      }
      if (page >= 0) {
        const T* src = cache + ((size_t)page * page_size + key % page_size) * row_size;
        if (vectors) {
          for (int c = part; c * kVec < row_size; c += 8)
            *reinterpret_cast<uint4*>(dst + c * kVec) = *reinterpret_cast<const uint4*>(src + c * kVec);
        } else {
          for (int d = part; d < row_size; d += 8) dst[d] = src[d];
        }
      } else {
        for (int d = part; d < row_size; d += 8) dst[d] = from_float<T>(0.f);   // finite values for the mixing
      }
    }
    __syncthreads();
    if (!has_a) continue;
    // scores of this lane's key against the warp's two heads
    const bool visible = key0 + lane < k_end;
    float s_a = 0.f, s_b = 0.f;
    {
      const T* row = k_s + lane * row_pad;
      const float* qa = q_s + h_a * row_size;
      const float* qb = q_s + (has_b ? h_b : h_a) * row_size;
      if (vectors) {
        // 16 bytes of the row at a time: with rows 16 bytes off a multiple of the banks the lanes of a
        // quarter warp read disjoint banks
        for (int d = 0; d < row_size; d += kVec) {
          Vec<T> kv;
          kv.raw = *reinterpret_cast<const decltype(kv.raw)*>(row + d);
#pragma unroll
          for (int e = 0; e < kVec; ++e) {
            const float x = kv.get(e);
            s_a = fmaf(qa[d + e], x, s_a);
            s_b = fmaf(qb[d + e], x, s_b);
          }
        }
      } else {
        for (int d = 0; d < row_size; ++d) {
          const float kv = to_float(row[d]);
          s_a = fmaf(qa[d], kv, s_a);
          s_b = fmaf(qb[d], kv, s_b);
        }
      }
    }
    if (!visible) s_a = s_b = -INFINITY;
    const float m_a_new = fmaxf(m_a, warp_max(s_a)), m_b_new = fmaxf(m_b, warp_max(s_b));
    const float p_a = s_a == -INFINITY ? 0.f : expf(s_a - m_a_new);
    const float p_b = s_b == -INFINITY ? 0.f : expf(s_b - m_b_new);
    const float c_a = m_a == -INFINITY ? 0.f : expf(m_a - m_a_new);
    const float c_b = m_b == -INFINITY ? 0.f : expf(m_b - m_b_new);
    l_a = l_a * c_a + warp_sum(p_a);
    l_b = l_b * c_b + warp_sum(p_b);
    m_a = m_a_new;
    m_b = m_b_new;
#pragma unroll
    for (int i = 0; i < kDimsPerLane; ++i) {
      acc_a[i] *= c_a;
      acc_b[i] *= c_b;
    }
    const int count = min(kSharedTile, k_end - key0);
    for (int kk = 0; kk < count; ++kk) {
      const float pa = __shfl_sync(0xffffffffu, p_a, kk), pb = __shfl_sync(0xffffffffu, p_b, kk);
      const T* row = k_s + kk * row_pad;
      // (measured: two neighbouring dimensions a lane, one load for both, is slower: 1,160 against 820 us
      // for 64 requests of 4,096 rows of 576)
#pragma unroll
      for (int i = 0; i < kDimsPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < value_size) {
          const float v = to_float(row[d]);
          acc_a[i] = fmaf(pa, v, acc_a[i]);
          acc_b[i] = fmaf(pb, v, acc_b[i]);
        }
      }
    }
  }
  if (__syncthreads_or(bad_page ? 1 : 0) && threadIdx.x == 0) atomicOr(status, kStatusBadPage);
  auto finish = [&](int h, const float* acc, float m, float l) {
    const int head = head0 + h;
    if (splits == 1) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T* o = out + ((size_t)t * num_heads + head) * value_size;
#pragma unroll
      for (int i = 0; i < kDimsPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < value_size) o[d] = from_float<T>(acc[i] * inv);
      }
    } else {
      const size_t slot = ((size_t)t * num_heads + head) * splits + split;
      float* o = part_acc + slot * value_size;
#pragma unroll
      for (int i = 0; i < kDimsPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < value_size) o[d] = acc[i];
      }
      if (lane == 0) {
        part_ml[2 * slot] = m;
        part_ml[2 * slot + 1] = l;
      }
    }
  };
  if (has_a) finish(h_a, acc_a, m_a, l_a);
  if (has_b) finish(h_b, acc_b, m_b, l_b);
}

// out[t, h] = sum_s w_s acc_s / sum_s w_s l_s with w_s = exp(m_s - max m), the shares in order.
template <typename T>
__global__ void latent_decode_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                           T* __restrict__ out, int splits, int value_size) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;
  const float* ml = part_ml + 2 * row * splits;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, ml[2 * s]);
  float l = 0.f;
  for (int s = 0; s < splits; ++s) l += ml[2 * s] == -INFINITY ? 0.f : expf(ml[2 * s] - m) * ml[2 * s + 1];
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int d = threadIdx.x; d < value_size; d += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < splits; ++s)
      if (ml[2 * s] != -INFINITY) v += expf(ml[2 * s] - m) * part_acc[(row * splits + s) * value_size + d];
    out[row * value_size + d] = from_float<T>(v * inv);
  }
}

}  // namespace einf

using namespace einf;

extern "C" int einf_paged_attention_generic(const void* q, const void* k_cache, const void* v_cache,
                                            int dtype, const int* block_table, const int* seq_of_token,
                                            const int* positions, void* out, int num_tokens,
                                            int num_heads, int num_kv_heads, int head_size, int value_size,
                                            int value_stride, int page_size, int num_pages, int table_width,
                                            float scale, int window, int keep_first, int chunk, float softcap,
                                            const float* sink, int* status, cudaStream_t stream) {
  const int rows = num_tokens * num_heads;
  if (rows == 0) return 0;
  if (head_size > kMaxHeadSize || value_size > kMaxHeadSize || head_size <= 0 || value_size <= 0)
    return (int)cudaErrorInvalidValue;
  const int blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (value_stride < value_size) return (int)cudaErrorInvalidValue;
  EINF_DISPATCH_2(dtype, T, {
    if (head_size <= 256 && value_size <= 256) {
      paged_attention_generic_kernel<T, 256><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(
          (const T*)q, (const T*)k_cache, (const T*)v_cache, block_table, seq_of_token, positions, (T*)out,
          rows, num_heads, num_kv_heads, head_size, value_size, value_stride, page_size, num_pages, table_width,
          scale, window, keep_first, chunk, softcap, sink, status);
    } else {
      paged_attention_generic_kernel<T, kMaxHeadSize><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(
          (const T*)q, (const T*)k_cache, (const T*)v_cache, block_table, seq_of_token, positions, (T*)out,
          rows, num_heads, num_kv_heads, head_size, value_size, value_stride, page_size, num_pages, table_width,
          scale, window, keep_first, chunk, softcap, sink, status);
    }
  })
  return (int)cudaGetLastError();
}

// Decode over shared rows: q [tokens, heads, row_size], cache [pages, 1, page_size, row_size] whose first
// value_size elements are the values, out [tokens, heads, value_size]; one token per request row of the
// batch (positions[t] is its position).  `splits` shares of every token's keys; with more than one,
// part_acc [tokens, heads, splits, value_size] and part_ml [tokens, heads, splits, 2] are the workspace.
extern "C" int einf_latent_decode_attention(const void* q, const void* cache, int dtype, const int* block_table,
                                            const int* seq_of_token, const int* positions, void* out,
                                            float* part_acc, float* part_ml, int num_tokens, int num_heads,
                                            int row_size, int value_size, int page_size, int num_pages,
                                            int table_width, float scale, int splits, int* status,
                                            cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (row_size <= 0 || row_size > kMaxHeadSize || value_size <= 0 || value_size > row_size || splits < 1 ||
      (splits > 1 && (!part_acc || !part_ml)) || num_tokens > 65535)
    return (int)cudaErrorInvalidValue;
  const int head_groups = (num_heads + kSharedHeads - 1) / kSharedHeads;
  const dim3 grid(splits, num_tokens, head_groups);
  const bool wide = value_size > 256;
  cudaError_t e = cudaSuccess;
  EINF_DISPATCH_2(dtype, T, {
    const size_t per_vector = 16 / sizeof(T);
    const size_t row_pad = (row_size + per_vector - 1) / per_vector * per_vector + per_vector;
    const size_t smem = (size_t)kSharedHeads * row_size * sizeof(float) + (size_t)kSharedTile * row_pad * sizeof(T);
    auto kernel = wide ? latent_decode_attention_kernel<T, kMaxHeadSize / 32> : latent_decode_attention_kernel<T, 8>;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    e = launch_pdl(kernel, grid, dim3(kSharedWarps * 32), smem, stream, (const T*)q, (const T*)cache, block_table,
                   seq_of_token, positions, (T*)out, part_acc, part_ml, num_heads, row_size, value_size, page_size,
                   num_pages, table_width, scale, status);
    if (e != cudaSuccess) return (int)e;
    if (splits > 1)
      e = launch_pdl(latent_decode_merge_kernel<T>, dim3(num_tokens * num_heads), dim3(128), 0, stream,
                     (const float*)part_acc, (const float*)part_ml, (T*)out, splits, value_size);
  })
  return (int)e;
}
