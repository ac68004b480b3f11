// Causal attention over the paged cache for layers whose heads' scores meet before the softmax.
// For query i (position p_i of its request) and key j, with H query heads over G key/value heads
// (head h reads key/value head h / (H / G)):
//   s_h(i, j) = scale * q_h(i) . k_g(j) - slope_h * (p_i - p_j)         (slopes optional)
//   s_h(i, j) <- sum_g' talk[h, g'] * s_g'(i, j)   over all H query heads  (talk optional)
//   p_h(i, j) = exp(s_h(i, j)) / (exp(sink_h) + sum_j' exp(s_h(i, j')))   (sink optional: a term of
//                                                                        the denominator with no key and no value)
//   out_h(i) = out_scale * sum_j p_h(i, j) v_g(j)
// over the keys j <= i of the same request, the last `window` of them if window > 0.  Because of the
// mixing, all heads of a query are computed together: one CTA per query token walks the visible
// keys in tiles.  Per tile: keys and values into shared memory as floats; raw scores, one (head,
// key) pair per thread; the mixing, one pair per thread; the softmax statistics, one warp per head,
// against a running maximum that starts at the sink (so the sink is the first term of the sum);
// the values, each thread owning a few (head, dimension) outputs in registers.  Scores, weights and
// sums are 32-bit; the order of a query's additions depends on its position alone (tiles start at
// the first visible key), never on the batch.
// q [T, H, D], caches [pages, G, page, D] and [pages, G, page, V], out [T, H, V].
#include "common.cuh"

namespace einf {

constexpr int kMixedThreads = 256;
constexpr int kMixedMaxHeads = 32;

template <typename T, int OUTS>
__global__ void __launch_bounds__(kMixedThreads)
paged_attention_mixed_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                             const int* __restrict__ block_table, int table_width,
                             const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                             T* __restrict__ out, int heads, int kv_heads, int dim, int vdim, int page_size,
                             int num_pages, float scale, int window, const float* __restrict__ slopes,
                             const float* __restrict__ talk, const float* __restrict__ sink, float out_scale,
                             int tile, int* __restrict__ status) {
  extern __shared__ float smem[];
  const int kdim = kv_heads * dim, kvdim = kv_heads * vdim;
  const int krow = kdim | 1;                          // odd row stride: a warp's keys fall into different banks
  float* qs = smem;                                   // [heads * dim], scaled
  float* talk_s = qs + heads * dim;                   // [heads * heads]
  float* ks = talk_s + heads * heads;                 // [tile * krow]
  float* vs = ks + tile * krow;                       // [tile * kvdim]
  float* raw = vs + tile * kvdim;                     // [heads * tile]
  float* prob = raw + heads * tile;                   // [heads * tile]
  float* top = prob + heads * tile;                   // [heads] running maximum
  float* total = top + heads;                         // [heads] running sum
  float* rescale = total + heads;                     // [heads] factor of this tile
  float* slope_s = rescale + heads;                   // [heads]

  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int per = heads / kv_heads;
  const int request = seq_of_token[t];
  const int position = positions[t];
  const int lo = window > 0 ? max(0, position - window + 1) : 0;
  const int* table = block_table + (size_t)request * table_width;
  for (int i = tid; i < heads * heads; i += kMixedThreads) talk_s[i] = talk ? talk[i] : (i / heads == i % heads ? 1.f : 0.f);
  for (int h = tid; h < heads; h += kMixedThreads) {
    top[h] = sink ? sink[h] : -INFINITY;
    total[h] = sink ? 1.f : 0.f;
    slope_s[h] = slopes ? slopes[h] : 0.f;
  }
  pdl_wait();
  for (int i = tid; i < heads * dim; i += kMixedThreads) qs[i] = to_float(q[(size_t)t * heads * dim + i]) * scale;

  float acc[OUTS];
#pragma unroll
  for (int n = 0; n < OUTS; ++n) acc[n] = 0.f;
  const int outs = heads * vdim;

  for (int j0 = lo; j0 <= position; j0 += tile) {
    const int count = min(tile, position - j0 + 1);
    __syncthreads();                                  // the tile before is used up; qs and the statistics are set
    // keys and values of the tile, one (key, key/value head) row per group of threads
    for (int idx = tid; idx < count * kdim; idx += kMixedThreads) {
      const int key = idx / kdim, e = idx - key * kdim;
      const int g = e / dim, d = e - g * dim;
      const int j = j0 + key;
      const int page = table[j / page_size];
      float value = 0.f;
      if (page >= 0 && page < num_pages)
        value = to_float(k_cache[(((size_t)page * kv_heads + g) * page_size + j % page_size) * dim + d]);
      else if (e == 0) atomicOr(status, kStatusBadPage);
      ks[key * krow + e] = value;
    }
    for (int idx = tid; idx < count * kvdim; idx += kMixedThreads) {
      const int key = idx / kvdim, e = idx - key * kvdim;
      const int g = e / vdim, d = e - g * vdim;
      const int j = j0 + key;
      const int page = table[j / page_size];
      float value = 0.f;
      if (page >= 0 && page < num_pages)
        value = to_float(v_cache[(((size_t)page * kv_heads + g) * page_size + j % page_size) * vdim + d]);
      vs[key * kvdim + e] = value;
    }
    __syncthreads();
    // raw scores with the distance taken off
    for (int idx = tid; idx < heads * tile; idx += kMixedThreads) {
      const int h = idx / tile, key = idx - h * tile;
      float s = 0.f;
      if (key < count) {
        const float* qh = qs + h * dim;
        const float* kr = ks + key * krow + (h / per) * dim;
        for (int d = 0; d < dim; ++d) s = fmaf(qh[d], kr[d], s);
        s -= slope_s[h] * (float)(position - (j0 + key));
      }
      raw[idx] = s;
    }
    __syncthreads();
    // the heads' scores mixed; keys beyond the query get no weight
    for (int idx = tid; idx < heads * tile; idx += kMixedThreads) {
      const int h = idx / tile, key = idx - h * tile;
      float s = -INFINITY;
      if (key < count) {
        s = 0.f;
        for (int g = 0; g < heads; ++g) s = fmaf(talk_s[h * heads + g], raw[g * tile + key], s);
      }
      prob[idx] = s;
    }
    __syncthreads();
    // statistics, a warp per head
    for (int h = warp; h < heads; h += kMixedThreads / 32) {
      float best = -INFINITY;
      for (int key = lane; key < tile; key += 32) best = fmaxf(best, prob[h * tile + key]);
      best = warp_max(best);
      const float before = top[h];
      const float now = fmaxf(before, best);
      float sum = 0.f;
      for (int key = lane; key < tile; key += 32) {
        const float s = prob[h * tile + key];
        const float p = s == -INFINITY ? 0.f : expf(s - now);
        prob[h * tile + key] = p;
        sum += p;
      }
      sum = warp_sum(sum);
      if (lane == 0) {
        const float factor = before == -INFINITY ? 0.f : expf(before - now);
        rescale[h] = factor;
        total[h] = fmaf(total[h], factor, sum);
        top[h] = now;
      }
    }
    __syncthreads();
    // values
#pragma unroll
    for (int n = 0; n < OUTS; ++n) {
      const int o = tid + n * kMixedThreads;
      if (o < outs) {
        const int h = o / vdim, d = o - h * vdim;
        const float* p = prob + h * tile;
        const float* vr = vs + (h / per) * vdim + d;
        float a = acc[n] * rescale[h];
        for (int key = 0; key < count; ++key) a = fmaf(p[key], vr[key * kvdim], a);
        acc[n] = a;
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int n = 0; n < OUTS; ++n) {
    const int o = tid + n * kMixedThreads;
    if (o < outs) {
      const int h = o / vdim;
      out[(size_t)t * outs + o] = from_float<T>(acc[n] / total[h] * out_scale);
    }
  }
}

}  // namespace einf

using namespace einf;

template <typename T, int OUTS>
static int launch_mixed(const void* q, const void* k_cache, const void* v_cache, const int* block_table, int table_width,
                        const int* seq_of_token, const int* positions, void* out, int num_tokens, int heads,
                        int kv_heads, int dim, int vdim, int page_size, int num_pages, float scale, int window,
                        const float* slopes, const float* talk, const float* sink, float out_scale, int* status,
                        cudaStream_t stream) {
  const int kdim = kv_heads * dim, kvdim = kv_heads * vdim;
  const size_t fixed = (size_t)heads * dim + (size_t)heads * heads + 4 * (size_t)heads;
  int tile = 128;
  auto bytes = [&](int n) { return (fixed + (size_t)n * ((kdim | 1) + kvdim + 2 * heads)) * sizeof(float); };
  while (tile > 8 && bytes(tile) > 96 * 1024) tile >>= 1;        // two CTAs an SM where the rows allow it
  if (window > 0)
    while (tile > 32 && tile / 2 >= window) tile >>= 1;
  if (bytes(tile) > 200 * 1024) return (int)cudaErrorInvalidValue;
  auto kernel = paged_attention_mixed_kernel<T, OUTS>;
  if (bytes(tile) > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes(tile));
    if (e != cudaSuccess) return (int)e;
  }
  return (int)launch_pdl(kernel, num_tokens, kMixedThreads, bytes(tile), stream, (const T*)q, (const T*)k_cache,
                         (const T*)v_cache, block_table, table_width, seq_of_token, positions, (T*)out, heads, kv_heads,
                         dim, vdim, page_size, num_pages, scale, window, slopes, talk, sink, out_scale, tile, status);
}

extern "C" int einf_paged_attention_mixed(const void* q, const void* k_cache, const void* v_cache, int dtype,
                                          const int* block_table, int table_width, const int* seq_of_token,
                                          const int* positions, void* out, int num_tokens, int heads, int kv_heads,
                                          int dim, int vdim, int page_size, int num_pages, float scale, int window,
                                          const float* slopes, const float* talk, const float* sink, float out_scale,
                                          int* status, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (heads <= 0 || heads > kMixedMaxHeads || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0)
    return (int)cudaErrorInvalidValue;
  const int outs = (heads * vdim + kMixedThreads - 1) / kMixedThreads;
#define EINF_MIXED(OUTS)                                                                                              \
  EINF_DISPATCH_2(dtype, T, {                                                                                         \
    return launch_mixed<T, OUTS>(q, k_cache, v_cache, block_table, table_width, seq_of_token, positions, out,         \
                                 num_tokens, heads, kv_heads, dim, vdim, page_size, num_pages, scale, window, slopes, \
                                 talk, sink, out_scale, status, stream);                                              \
  })
  if (outs <= 1) EINF_MIXED(1)
  if (outs <= 4) EINF_MIXED(4)
  if (outs <= 8) EINF_MIXED(8)
  if (outs <= 32) EINF_MIXED(32)
  return (int)cudaErrorInvalidValue;
#undef EINF_MIXED
}
