// Memory-bound kernels between the matrix products: embedding gather,
// residual-add + RMSNorm, rotary encoding fused with the QKV bias and the paged
// key/value write, SiLU-and-multiply.
//
// Arithmetic is 32-bit throughout; a value is rounded once, when it is stored in
// the activation type.  The residual stream is a float tensor in both modes.
#include <cuda.h>

#include "common.cuh"

namespace einf {

// ---------------------------------------------------------------------------
// Embedding: residual[t, :] = table[token[t], :]   (reference: nn.Embedding,
// src/einf/executors/torch/qwen.py:744).  With a table of learned position vectors
// (pos_table [max_positions, hidden]) the row of the token's position is added, unscaled, in
// 32-bit; a position outside the table sets the same status bit as a bad token.  The token's row
// is multiplied by `scale` (1 for most models), in 32-bit.
// ---------------------------------------------------------------------------
template <typename TTable>
__global__ void embed_kernel(const int* __restrict__ tokens, const TTable* __restrict__ table,
                             float* __restrict__ residual, int hidden, int vocab, int* status,
                             const int* __restrict__ positions, const TTable* __restrict__ pos_table,
                             int max_positions, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int token = tokens[t];
  const int position = pos_table ? positions[t] : 0;
  float* out = residual + (size_t)t * hidden;
  if (token < 0 || token >= vocab || (pos_table && (position < 0 || position >= max_positions))) {
    if (threadIdx.x == 0) atomicOr(status, kStatusBadToken);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = 0.f;
    return;
  }
  const TTable* row = table + (size_t)token * hidden;
  if (pos_table) {
    const TTable* pos = pos_table + (size_t)position * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = to_float(row[i]) * scale + to_float(pos[i]);
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = to_float(row[i]) * scale;
  }
}

// The input of a consumer may be the partial sums of a split-K product, [splits, T, width].
template <typename TIn>
__device__ __forceinline__ float sum_splits(const TIn* __restrict__ p, int splits, size_t split_stride) {
  // Sixteen loads in flight at a time: the partial sums sit in L2, and a chain of dependent
  // loads would cost a round trip each.
  constexpr int kBatch = 16;
  float v = 0.f;
  int s = 0;
  for (; s + kBatch <= splits; s += kBatch) {
    float t[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) t[u] = to_float(p[(size_t)(s + u) * split_stride]);
#pragma unroll
    for (int u = 0; u < kBatch; ++u) v += t[u];
  }
  if (s < splits) {
    float t[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) t[u] = s + u < splits ? to_float(p[(size_t)(s + u) * split_stride]) : 0.f;
#pragma unroll
    for (int u = 0; u < kBatch; ++u) v += t[u];
  }
  return v;
}

// ---------------------------------------------------------------------------
// residual += sum_s x[s]; out = weight * (residual * rsqrt(mean(residual^2) + eps))
// (reference: fused_add_rmsnorm / rmsnorm, src/einf/executors/torch/fused_ops.py:41-68).
// x may be absent (first norm of the model), or hold `splits` partial sums of a
// split-K matrix product, stacked [splits, T, hidden].  With `rows`, output row r
// is computed from input row rows[r] and the residual is left untouched (used to
// normalise only the rows whose logits are wanted).
// ---------------------------------------------------------------------------
template <typename TX, typename TOut>
__global__ void add_rmsnorm_kernel(const TX* __restrict__ x, int splits, size_t split_stride,
                                   float* __restrict__ residual, const float* __restrict__ weight,
                                   float eps, TOut* __restrict__ out, const int* __restrict__ rows,
                                   int hidden, int write_residual, int vectorised) {
  extern __shared__ float smem[];
  float* row_buf = smem;                          // [hidden]
  float* scratch = smem + (hidden + 3) / 4 * 4;   // [33]
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* res = residual + (size_t)src * hidden;
  float ss = 0.f;
  if (vectorised) {
    // hidden is a multiple of 4 and there are no partial sums: 16-byte loads of the residual
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(res + i);
      if (x) {
        const TX* xp = x + (size_t)src * hidden + i;
        v.x += to_float(xp[0]);
        v.y += to_float(xp[1]);
        v.z += to_float(xp[2]);
        v.w += to_float(xp[3]);
      }
      *reinterpret_cast<float4*>(row_buf + i) = v;
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = res[i];
      if (x) v += sum_splits(x + (size_t)src * hidden + i, splits, split_stride);
      row_buf[i] = v;
      ss += v * v;
    }
  }
  const float total = block_sum(ss, scratch);
  const float rstd = rsqrtf(total / (float)hidden + eps);
  if (vectorised) {
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row_buf + i);
      if (write_residual && x) *reinterpret_cast<float4*>(res + i) = v;
      const float4 w = *reinterpret_cast<const float4*>(weight + i);
      TOut* o = out + (size_t)r * hidden + i;
      o[0] = from_float<TOut>(w.x * (v.x * rstd));
      o[1] = from_float<TOut>(w.y * (v.y * rstd));
      o[2] = from_float<TOut>(w.z * (v.z * rstd));
      o[3] = from_float<TOut>(w.w * (v.w * rstd));
    }
    return;
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = row_buf[i];
    if (write_residual && x) res[i] = v;
    out[(size_t)r * hidden + i] = from_float<TOut>(weight[i] * (v * rstd));
  }
}

// The same for few rows (decode), where one CTA per row would leave all but a few SMs idle while
// it adds up dozens of partial sums: the CTAs of a cluster split a row's columns and exchange
// their sums of squares through distributed shared memory.  Up to four elements per thread.
template <typename TX, typename TOut>
__global__ void add_rmsnorm_cluster_kernel(const TX* __restrict__ x, int splits, size_t split_stride,
                                           float* __restrict__ residual, const float* __restrict__ weight,
                                           float eps, TOut* __restrict__ out, const int* __restrict__ rows,
                                           int hidden, int write_residual) {
  __shared__ float sums[8 * 32];   // slot c * warps + w: the sum of squares of warp w of CTA c (clusters of up to 8)
  pdl_launch_dependents();
  const uint32_t rank = cluster_ctarank(), csize = cluster_nctarank();
  const int r = blockIdx.y;
  const int src = rows ? rows[r] : r;                 // rows: an input of the step
  const int slice = (hidden + (int)csize - 1) / (int)csize;
  const int begin = (int)rank * slice, end = min(hidden, begin + slice);
  float w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int i = begin + (int)threadIdx.x + k * (int)blockDim.x;
    w[k] = i < end ? weight[i] : 0.f;
  }
  pdl_wait();
  float* res = residual + (size_t)src * hidden;
  float v[4];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int i = begin + (int)threadIdx.x + k * (int)blockDim.x;
    v[k] = 0.f;
    if (i < end) {
      v[k] = res[i];
      if (x) v[k] += sum_splits(x + (size_t)src * hidden + i, splits, split_stride);
      ss += v[k] * v[k];
    }
  }
  // Every warp pushes its sum into every CTA of the cluster before the one barrier, so nothing is
  // read remotely after it and no CTA has to be held back from leaving; each warp then adds the
  // same values in the same order.
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  ss = warp_sum(ss);
  if (lane < (int)csize) st_cluster_peer(&sums[(int)rank * warps + warp], (uint32_t)lane, ss);
  cluster_barrier();
  float mine = 0.f;
  for (int s = lane; s < (int)csize * warps; s += 32) mine += sums[s];
  const float total = warp_sum(mine);
  const float rstd = rsqrtf(total / (float)hidden + eps);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int i = begin + (int)threadIdx.x + k * (int)blockDim.x;
    if (i < end) {
      if (write_residual && x) res[i] = v[k];
      out[(size_t)r * hidden + i] = from_float<TOut>(w[k] * (v[k] * rstd));
    }
  }
}

// The same for many rows without partial sums: one warp per row, the row in registers
// (kVec float4 per lane, hidden <= 128 * kVec), no shared memory and no block barrier.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&a);
  raw.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename TX, typename TOut, int kVec>
__global__ void add_rmsnorm_warp_kernel(const TX* __restrict__ x, float* __restrict__ residual,
                                        const float* __restrict__ weight, float eps, TOut* __restrict__ out,
                                        const int* __restrict__ rows, int hidden, int num_rows, int write_residual) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = (int)((blockIdx.x * blockDim.x + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= num_rows) return;
  const int src = rows ? rows[r] : r;
  float* res = residual + (size_t)src * hidden;
  // Loads first, without a branch between them (an index past the row is clamped, its value
  // unused), so that a whole row is in flight at once; a branch per vector would wait for each.
  float4 v[kVec];
#pragma unroll
  for (int j = 0; j < kVec; ++j) v[j] = load4(res + min((j * 32 + lane) * 4, hidden - 4));
  if (x) {
    const TX* xr = x + (size_t)src * hidden;
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
      const float4 a = load4(xr + min((j * 32 + lane) * 4, hidden - 4));
      v[j].x += a.x;
      v[j].y += a.y;
      v[j].z += a.z;
      v[j].w += a.w;
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kVec; ++j)
    if ((j * 32 + lane) * 4 < hidden) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
  const float rstd = rsqrtf(warp_sum(ss) / (float)hidden + eps);
#pragma unroll
  for (int j = 0; j < kVec; ++j) {
    const int i = (j * 32 + lane) * 4;
    if (i < hidden) {
      if (write_residual && x) store4(res + i, v[j]);
      const float4 w = load4(weight + i);
      store4(out + (size_t)r * hidden + i,
             make_float4(w.x * (v[j].x * rstd), w.y * (v[j].y * rstd), w.z * (v[j].z * rstd), w.w * (v[j].w * rstd)));
    }
  }
}

// The same for few rows with partial sums when a row fits one CTA at one float4 per thread
// (hidden <= 4096, a multiple of 4): every load of a thread is issued before the first is used
// (the partial sums of up to sixteen K ranges at a time: each batch is a round trip to L2), and
// one block barrier is all the synchronisation there is.
constexpr int kRowBatch = 16;
template <typename TX, typename TOut>
__global__ void add_rmsnorm_row_kernel(const TX* __restrict__ x, int splits, size_t split_stride,
                                       float* __restrict__ residual, const float* __restrict__ weight,
                                       float eps, TOut* __restrict__ out, const int* __restrict__ rows,
                                       int hidden, int write_residual) {
  __shared__ float warp_ss[32];
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const int i = (int)threadIdx.x * 4;
  const bool live = i < hidden;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  const float4 w = live ? load4(weight + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  const int src = rows ? rows[r] : r;                 // rows: an input of the step
  pdl_wait();
  float* res = residual + (size_t)src * hidden;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) {
    v = load4(res + i);
    if (x) {
      const TX* xp = x + (size_t)src * hidden + i;
      for (int s = 0; s < splits; s += kRowBatch) {
        float4 t[kRowBatch];
#pragma unroll
        for (int u = 0; u < kRowBatch; ++u) t[u] = load4(xp + (size_t)min(s + u, splits - 1) * split_stride);
#pragma unroll
        for (int u = 0; u < kRowBatch; ++u) {
          if (s + u < splits) {
            v.x += t[u].x;
            v.y += t[u].y;
            v.z += t[u].z;
            v.w += t[u].w;
          }
        }
      }
    }
  }
  const float ss = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
  if (lane == 0) warp_ss[warp] = ss;
  __syncthreads();
  const float total = warp_sum(lane < warps ? warp_ss[lane] : 0.f);   // the same order in every warp
  const float rstd = rsqrtf(total / (float)hidden + eps);
  if (live) {
    if (write_residual && x) store4(res + i, v);
    store4(out + (size_t)r * hidden + i,
           make_float4(w.x * (v.x * rstd), w.y * (v.y * rstd), w.z * (v.z * rstd), w.w * (v.w * rstd)));
  }
}

// The same with the partial sums fetched by TMA: a row's partial sums (up to sixteen K ranges of
// up to 1,536 columns: 98 KB) come into shared memory as a few boxes of one three-dimensional
// tensor map [split, row, column], and the threads add them up from there.  Through the load
// pipe of the one SM that owns a row the same bytes take several times as long (an SM keeps too
// few of its own loads in flight), and the norm of a decode step is 49 such kernels.
constexpr int kRowTmaCols = 256;        // columns per box (a box dimension is at most 256)
constexpr int kRowTmaPolls = 1 << 22;
__device__ __forceinline__ uint32_t pw_smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
template <typename TOut>
__global__ void add_rmsnorm_row_tma_kernel(const __grid_constant__ CUtensorMap map_x, int splits,
                                           float* __restrict__ residual, const float* __restrict__ weight, float eps,
                                           TOut* __restrict__ out, const int* __restrict__ rows, int hidden,
                                           int write_residual, int* status) {
  extern __shared__ __align__(128) unsigned char row_smem[];      // [box][split][256 columns] float, then the barrier
  __shared__ float warp_ss[32];
  __shared__ __align__(8) unsigned long long row_bar;
  const uint32_t bar = pw_smem_addr(&row_bar);
  const int boxes = (hidden + kRowTmaCols - 1) / kRowTmaCols;
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const int i = (int)threadIdx.x * 4;
  const bool live = i < hidden;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  const float4 w = live ? load4(weight + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  const int src = rows ? rows[r] : r;                 // rows: an input of the step
  __syncthreads();                                    // the barrier is initialised
  pdl_wait();
  if (threadIdx.x == 0) {
    const uint32_t bytes = (uint32_t)boxes * (uint32_t)splits * kRowTmaCols * 4u;   // a box is counted whole, also past the row's end
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    for (int b = 0; b < boxes; ++b) {
      const uint32_t dst = pw_smem_addr(row_smem) + (uint32_t)b * (uint32_t)splits * kRowTmaCols * 4u;
      asm volatile(
          "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
          ::"r"(dst), "l"(&map_x), "r"(b * kRowTmaCols), "r"(src), "r"(0), "r"(bar)
          : "memory");
    }
  }
  float* res = residual + (size_t)src * hidden;
  float4 v = live ? load4(res + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  bool arrived = false;
  for (int poll = 0; poll < kRowTmaPolls && !arrived; ++poll) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(0)
        : "memory");
    arrived = done != 0;
  }
  if (!arrived && threadIdx.x == 0) atomicOr(status, kStatusWaitExpired);
  if (live && arrived) {
    const float* box = reinterpret_cast<const float*>(row_smem) + (size_t)(i / kRowTmaCols) * splits * kRowTmaCols +
                       (i % kRowTmaCols);
    for (int s = 0; s < splits; ++s) {
      const float4 t = *reinterpret_cast<const float4*>(box + (size_t)s * kRowTmaCols);
      v.x += t.x;
      v.y += t.y;
      v.z += t.z;
      v.w += t.w;
    }
  }
  const float ss = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
  if (lane == 0) warp_ss[warp] = ss;
  __syncthreads();
  const float total = warp_sum(lane < warps ? warp_ss[lane] : 0.f);   // the same order in every warp
  const float rstd = rsqrtf(total / (float)hidden + eps);
  if (live) {
    if (write_residual) store4(res + i, v);
    store4(out + (size_t)r * hidden + i,
           make_float4(w.x * (v.x * rstd), w.y * (v.y * rstd), w.z * (v.z * rstd), w.w * (v.w * rstd)));
  }
}

// ---------------------------------------------------------------------------
// Rotary encoding (rotate-half layout) of Q and K after the bias, and the paged
// write of K and V.  qkv is [T, (Hq + 2 Hkv) * D]: Q heads, then K heads, then V.
//   x'[i]        = x[i] cos(a_i) - x[i + R/2] sin(a_i)
//   x'[i + R/2]  = x[i + R/2] cos(a_i) + x[i] sin(a_i),   a_i = position * inv_freq[i]
// for i < R/2 (R = rotary_dim <= D); dims >= R pass through.  (reference:
// src/einf/executors/torch/model_runner.py:42-78; cache write
// src/einf/executors/torch/ops/csrc/kv_cache_cuda.cu:14-58.)  inv_freq is a
// float table made on the host so that angles match a host computation exactly.
// Cache layout: [page, kv_head, slot_in_page, D]; slots[t] = page * page_size + offset,
// negative = do not write.
// ---------------------------------------------------------------------------
template <typename TIn, typename T>
__global__ void rope_kv_write_kernel(const TIn* __restrict__ qkv, int splits, size_t split_stride,
                                     const float* __restrict__ bias,
                                     const int* __restrict__ positions,
                                     const float* __restrict__ inv_freq, const int* __restrict__ slots,
                                     T* __restrict__ q_out, T* __restrict__ k_cache,
                                     T* __restrict__ v_cache, int num_heads, int num_kv_heads,
                                     int head_size, int rotary_dim, int page_size, int num_pages,
                                     int* status) {
  extern __shared__ float smem[];
  const int half = rotary_dim >> 1;
  float* cos_t = smem;          // [half]
  float* sin_t = smem + half;   // [half]
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const float pos = (float)positions[t];   // an input of the step, like inv_freq: no need to wait
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf(pos * inv_freq[i], &s, &c);
    cos_t[i] = c;
    sin_t[i] = s;
  }
  pdl_wait();
  __syncthreads();
  const int width = (num_heads + 2 * num_kv_heads) * head_size;
  const TIn* row = qkv + (size_t)t * width;
  const int slot = slots ? slots[t] : -1;
  int page = -1, offset = 0;
  if (slot >= 0) {
    page = slot / page_size;
    offset = slot - page * page_size;
    if (page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, kStatusBadPage);
      page = -1;
    }
  }
  // Work items: one per (head, dim pair) for rotated dims, one per dim beyond them.
  const int rot_heads = num_heads + num_kv_heads;
  const int per_head = half + (head_size - rotary_dim);
  const int rot_items = rot_heads * per_head;
  for (int item = threadIdx.x; item < rot_items; item += blockDim.x) {
    const int head = item / per_head;
    const int j = item - head * per_head;
    const int base = head * head_size;
    T* dst;
    if (head < num_heads) {
      dst = q_out + ((size_t)t * num_heads + head) * head_size;
    } else {
      if (page < 0) continue;
      dst = k_cache + (((size_t)page * num_kv_heads + (head - num_heads)) * page_size + offset) * head_size;
    }
    if (j < half) {
      float a = sum_splits(row + base + j, splits, split_stride);
      float b = sum_splits(row + base + j + half, splits, split_stride);
      if (bias) {
        a += bias[base + j];
        b += bias[base + j + half];
      }
      const float c = cos_t[j], s = sin_t[j];
      dst[j] = from_float<T>(a * c - b * s);
      dst[j + half] = from_float<T>(b * c + a * s);
    } else {
      const int d = rotary_dim + (j - half);
      float a = sum_splits(row + base + d, splits, split_stride);
      if (bias) a += bias[base + d];
      dst[d] = from_float<T>(a);
    }
  }
  if (page >= 0) {
    const int v_items = num_kv_heads * head_size;
    const int v_base = rot_heads * head_size;
    for (int item = threadIdx.x; item < v_items; item += blockDim.x) {
      const int head = item / head_size;
      const int d = item - head * head_size;
      float a = sum_splits(row + v_base + item, splits, split_stride);
      if (bias) a += bias[v_base + item];
      v_cache[(((size_t)page * num_kv_heads + head) * page_size + offset) * head_size + d] = from_float<T>(a);
    }
  }
}

// The same with one CTA per (token, head), for few tokens (decode): a CTA per token would
// leave the reading of the partial sums to a handful of SMs.  Each thread computes the angle of
// its own pair, before the wait for the kernel that produced qkv.
template <typename TIn, typename T>
__global__ void rope_kv_write_heads_kernel(const TIn* __restrict__ qkv, int splits, size_t split_stride,
                                           const float* __restrict__ bias, const int* __restrict__ positions,
                                           const float* __restrict__ inv_freq, const int* __restrict__ slots,
                                           T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                           int num_heads, int num_kv_heads, int head_size, int rotary_dim,
                                           int page_size, int num_pages, int* status) {
  pdl_launch_dependents();
  const int heads_total = num_heads + 2 * num_kv_heads;
  const int t = blockIdx.x / heads_total;
  const int head = blockIdx.x - t * heads_total;
  const int half = rotary_dim >> 1;
  const int j = threadIdx.x;
  const bool is_v = head >= num_heads + num_kv_heads;
  float c = 1.f, s = 0.f;
  if (!is_v && j < half) sincosf((float)positions[t] * inv_freq[j], &s, &c);
  const int slot = slots ? slots[t] : -1;
  int page = -1, offset = 0;
  if (slot >= 0) {
    page = slot / page_size;
    offset = slot - page * page_size;
    if (page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, kStatusBadPage);
      page = -1;
    }
  }
  // The bias is a weight: read before the wait as well, so that after it only the partial sums
  // are a round trip away.
  const float* head_bias = bias ? bias + (size_t)head * head_size : nullptr;
  const int extra = rotary_dim + (j - half);                  // the dim of a thread past the pairs
  float bias_a = 0.f, bias_b = 0.f;
  if (head_bias) {
    if (is_v) {
      if (j < head_size) bias_a = head_bias[j];
    } else if (j < half) {
      bias_a = head_bias[j];
      bias_b = head_bias[j + half];
    } else if (j < half + (head_size - rotary_dim)) {
      bias_a = head_bias[extra];
    }
  }
  pdl_wait();
  const int width = heads_total * head_size;
  const TIn* row = qkv + (size_t)t * width + (size_t)head * head_size;
  T* dst;
  if (head < num_heads) {
    dst = q_out + ((size_t)t * num_heads + head) * head_size;
  } else {
    if (page < 0) return;
    const int kv_head = is_v ? head - num_heads - num_kv_heads : head - num_heads;
    dst = (is_v ? v_cache : k_cache) + (((size_t)page * num_kv_heads + kv_head) * page_size + offset) * head_size;
  }
  if (is_v) {
    if (j < head_size) dst[j] = from_float<T>(sum_splits(row + j, splits, split_stride) + bias_a);
    return;
  }
  if (j < half) {
    const float a = sum_splits(row + j, splits, split_stride) + bias_a;
    const float b = sum_splits(row + j + half, splits, split_stride) + bias_b;
    dst[j] = from_float<T>(a * c - b * s);
    dst[j + half] = from_float<T>(b * c + a * s);
  } else if (j < half + (head_size - rotary_dim)) {
    dst[extra] = from_float<T>(sum_splits(row + extra, splits, split_stride) + bias_a);
  }
}

// The same for dense bfloat16 rows with the whole head rotated and a head size that is a
// multiple of 16: eight pairs per thread, 16-byte loads and stores.
__device__ __forceinline__ void load8(const __nv_bfloat16* p, const float* bias, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(h[e]);
    v[2 * e] = f.x;
    v[2 * e + 1] = f.y;
  }
  if (bias) {   // 16-byte aligned like the row (the launcher checks)
    const float4 b0 = *reinterpret_cast<const float4*>(bias), b1 = *reinterpret_cast<const float4*>(bias + 4);
    v[0] += b0.x;
    v[1] += b0.y;
    v[2] += b0.z;
    v[3] += b0.w;
    v[4] += b1.x;
    v[5] += b1.y;
    v[6] += b1.z;
    v[7] += b1.w;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// Several tokens per CTA: their angles are computed side by side before the one barrier, and the
// 16-byte items of all of them are spread over the threads.
constexpr int kRopeTokens = 4;

__global__ void rope_kv_write_bf16x8_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ bias,
                                            const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                            const int* __restrict__ slots, __nv_bfloat16* __restrict__ q_out,
                                            __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                            int num_tokens, int num_heads, int num_kv_heads, int head_size,
                                            int page_size, int num_pages, int* status) {
  extern __shared__ float smem[];
  const int half = head_size >> 1;
  float* cos_t = smem;                          // [kRopeTokens][half]
  float* sin_t = smem + kRopeTokens * half;
  __shared__ int pages[kRopeTokens], offsets[kRopeTokens];
  pdl_launch_dependents();
  const int t0 = blockIdx.x * kRopeTokens;
  const int here = min(kRopeTokens, num_tokens - t0);
  for (int i = threadIdx.x; i < here * half; i += blockDim.x) {
    const int tok = i / half, j = i - tok * half;
    float s, c;
    sincosf((float)positions[t0 + tok] * inv_freq[j], &s, &c);   // inputs of the step: no need to wait
    cos_t[i] = c;
    sin_t[i] = s;
  }
  if (threadIdx.x < here) {
    const int slot = slots ? slots[t0 + threadIdx.x] : -1;
    int page = -1, offset = 0;
    if (slot >= 0) {
      page = slot / page_size;
      offset = slot - page * page_size;
      if (page >= num_pages) {
        atomicOr(status, kStatusBadPage);
        page = -1;
      }
    }
    pages[threadIdx.x] = page;
    offsets[threadIdx.x] = offset;
  }
  pdl_wait();
  __syncthreads();
  const int width = (num_heads + 2 * num_kv_heads) * head_size;
  const int groups = half >> 3;                       // groups of eight pairs per head
  const int rot_items = (num_heads + num_kv_heads) * groups;
  const int v_items = num_kv_heads * (head_size >> 3);
  const int per_token = rot_items + v_items;
  for (int index = threadIdx.x; index < here * per_token; index += blockDim.x) {
    const int tok = index / per_token, item = index - tok * per_token;
    const int t = t0 + tok;
    const __nv_bfloat16* row = qkv + (size_t)t * width;
    const int page = pages[tok], offset = offsets[tok];
    if (item < rot_items) {
      const int head = item / groups;
      const int j = (item - head * groups) << 3;
      const int base = head * head_size;
      __nv_bfloat16* dst;
      if (head < num_heads) {
        dst = q_out + ((size_t)t * num_heads + head) * head_size;
      } else {
        if (page < 0) continue;
        dst = k_cache + (((size_t)page * num_kv_heads + (head - num_heads)) * page_size + offset) * head_size;
      }
      float a[8], b[8], ra[8], rb[8];
      load8(row + base + j, bias ? bias + base + j : nullptr, a);
      load8(row + base + half + j, bias ? bias + base + half + j : nullptr, b);
      const float* cs = cos_t + tok * half + j;
      const float* sn = sin_t + tok * half + j;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        ra[e] = a[e] * cs[e] - b[e] * sn[e];
        rb[e] = b[e] * cs[e] + a[e] * sn[e];
      }
      store8(dst + j, ra);
      store8(dst + half + j, rb);
    } else {
      if (page < 0) continue;
      const int v_item = item - rot_items;
      const int per_head = head_size >> 3;
      const int head = v_item / per_head;
      const int d = (v_item - head * per_head) << 3;
      const int source = (num_heads + num_kv_heads) * head_size + head * head_size + d;
      float a[8];
      load8(row + source, bias ? bias + source : nullptr, a);
      store8(v_cache + (((size_t)page * num_kv_heads + head) * page_size + offset) * head_size + d, a);
    }
  }
}

// ---------------------------------------------------------------------------
// out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i],  silu(z) = z / (1 + exp(-z))
// (reference: src/einf/executors/torch/fused_ops.py:71-77)
// ---------------------------------------------------------------------------
template <typename TIn, typename T>
__global__ void silu_mul_kernel(const TIn* __restrict__ gate_up, int splits, size_t split_stride,
                                T* __restrict__ out, int intermediate, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const size_t t = idx / intermediate;
    const int i = (int)(idx - t * intermediate);
    const float g = sum_splits(gate_up + t * 2 * intermediate + i, splits, split_stride);
    const float u = sum_splits(gate_up + t * 2 * intermediate + intermediate + i, splits, split_stride);
    out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
  }
}

// The same for dense bfloat16 rows whose width is a multiple of 8: 16-byte loads and stores, one
// vector per thread, block = (token, chunk of the row).  At thousands of tokens this kernel is
// bound by arithmetic, not by memory, if it divides and calls expf exactly; the result is
// rounded to bfloat16, so the hardware exponential and reciprocal (relative error about 1e-6)
// are enough here.  The generic kernel above, which the 32-bit path uses, stays exact.
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out,
                                       int intermediate, int chunks_per_row) {
  pdl_launch_dependents();
  pdl_wait();
  const unsigned t = blockIdx.x / (unsigned)chunks_per_row;
  const unsigned chunk = blockIdx.x - t * (unsigned)chunks_per_row;
  const int i = (int)(chunk * blockDim.x + threadIdx.x) << 3;
  if (i < intermediate) {
    const __nv_bfloat16* row = gate_up + (size_t)t * 2 * intermediate;
    const uint4 g = *reinterpret_cast<const uint4*>(row + i);
    const uint4 u = *reinterpret_cast<const uint4*>(row + intermediate + i);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 result;
    __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&result);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 gf = __bfloat1622float2(gp[e]);
      const float2 uf = __bfloat1622float2(up[e]);
      rp[e] = __floats2bfloat162_rn(__fdividef(gf.x, 1.f + __expf(-gf.x)) * uf.x,
                                    __fdividef(gf.y, 1.f + __expf(-gf.y)) * uf.y);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * intermediate + i) = result;
  }
}

// One decode step on, in place, for a step of single tokens (one thread per request): the sampled
// token becomes the input, position and context length grow by one, and the cache slot of every
// group follows the request's block table.  A request that writes nothing (slot < 0: padding of a
// graph bucket) keeps its slot.  Lets several decode steps run before the host looks.
struct AdvanceGroups {
  int* slots[4];
  const int* tables[4];
};

__global__ void advance_decode_kernel(int* __restrict__ token_ids, int* __restrict__ positions,
                                      int* __restrict__ context_lens, const int* __restrict__ sampled,
                                      int num_requests, AdvanceGroups groups, int num_groups, int table_width,
                                      int page_size) {
  // No early launch of the dependents here: this kernel writes what the kernels of the next step
  // read before their own dependency wait (positions, slots), so none of them may start before it
  // has ended; without the call the next kernel starts when this one is complete.
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= num_requests) return;
  token_ids[i] = sampled[i];
  const int position = positions[i] + 1;
  positions[i] = position;
  context_lens[i] += 1;
  for (int g = 0; g < num_groups; ++g) {
    if (groups.slots[g][i] < 0) continue;
    const int page = groups.tables[g][(size_t)i * table_width + position / page_size];
    groups.slots[g][i] = page * page_size + position % page_size;   // a missing page (-1) gives a negative slot: no write
  }
}

// Per-request state of fixed size is read before it is written, so the rows of requests that
// start at position 0 in this step are cleared first; on the device, from the step's own inputs,
// so that the clearing can sit inside a captured step.  Requests without a slot (-1: the padding
// requests of a graph bucket) and requests that go on from an earlier step are left alone.
template <typename Word>
__global__ void zero_fresh_state_kernel(Word* __restrict__ state, long long row_words, int num_slots,
                                        const int* __restrict__ state_slots, const int* __restrict__ q_start,
                                        const int* __restrict__ positions) {
  pdl_launch_dependents();
  pdl_wait();
  const int request = blockIdx.y;
  const int slot = state_slots[request];
  if (slot < 0 || slot >= num_slots || positions[q_start[request]] != 0) return;
  Word* row = state + (size_t)slot * row_words;
  Word zero;
  memset(&zero, 0, sizeof(Word));
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < row_words; i += (long long)gridDim.x * blockDim.x)
    row[i] = zero;
}

// ---------------------------------------------------------------------------
// out[t, i] = act(x[t, i]) for the feed-forwards without a gate.  kinds (ops.ACTIVATIONS):
//   0 squared ReLU      max(z, 0)^2
//   1 GELU, tanh form   0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
//   2 SiLU              z / (1 + exp(-z))
//   3 ReLU
// x may be the float32 partial sums of a split-K product.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float activate(float z, int kind) {
  switch (kind) {
    case 0: { const float r = fmaxf(z, 0.f); return r * r; }
    case 1: return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    case 2: return z / (1.f + expf(-z));
    default: return fmaxf(z, 0.f);
  }
}

template <typename TIn, typename T>
__global__ void activation_kernel(const TIn* __restrict__ x, int splits, size_t split_stride, T* __restrict__ out,
                                  int kind, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride)
    out[idx] = from_float<T>(activate(sum_splits(x + idx, splits, split_stride), kind));
}

// Dense bfloat16 rows, eight values per thread with 16-byte accesses.
__global__ void activation_bf16x8_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, int kind,
                                         size_t vectors) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= vectors) return;
  const uint4 raw = reinterpret_cast<const uint4*>(x)[idx];
  const __nv_bfloat162* in = reinterpret_cast<const __nv_bfloat162*>(&raw);
  uint4 result;
  __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&result);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = __bfloat1622float2(in[e]);
    rp[e] = __floats2bfloat162_rn(activate(f.x, kind), activate(f.y, kind));
  }
  reinterpret_cast<uint4*>(out)[idx] = result;
}

// ---------------------------------------------------------------------------
// out[t, i] = act(gate_up[t, i]) * gate_up[t, I + i] for the activations above: the gated
// feed-forward with another gate than SiLU.  The dense bfloat16 form computes the GELU's tanh as
// 1 - 2 / (exp(2 a) + 1) with the hardware exponential and reciprocal (the result is rounded to
// bfloat16); the generic form, which the 32-bit path uses, calls tanhf.
// ---------------------------------------------------------------------------
template <typename TIn, typename T>
__global__ void act_mul_kernel(const TIn* __restrict__ gate_up, int splits, size_t split_stride, T* __restrict__ out,
                               int intermediate, int kind, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const size_t t = idx / intermediate;
    const int i = (int)(idx - t * intermediate);
    const float g = sum_splits(gate_up + t * 2 * intermediate + i, splits, split_stride);
    const float u = sum_splits(gate_up + t * 2 * intermediate + intermediate + i, splits, split_stride);
    out[idx] = from_float<T>(activate(g, kind) * u);
  }
}

__device__ __forceinline__ float activate_fast(float z, int kind) {
  if (kind == 1) {
    const float a = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    const float th = 1.f - __fdividef(2.f, __expf(2.f * a) + 1.f);
    return 0.5f * z * (1.f + th);
  }
  if (kind == 2) return __fdividef(z, 1.f + __expf(-z));
  return activate(z, kind);
}

__global__ void act_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out,
                                      int intermediate, int chunks_per_row, int kind) {
  pdl_launch_dependents();
  pdl_wait();
  const unsigned t = blockIdx.x / (unsigned)chunks_per_row;
  const unsigned chunk = blockIdx.x - t * (unsigned)chunks_per_row;
  const int i = (int)(chunk * blockDim.x + threadIdx.x) << 3;
  if (i < intermediate) {
    const __nv_bfloat16* row = gate_up + (size_t)t * 2 * intermediate;
    const uint4 g = *reinterpret_cast<const uint4*>(row + i);
    const uint4 u = *reinterpret_cast<const uint4*>(row + intermediate + i);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 result;
    __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&result);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 gf = __bfloat1622float2(gp[e]);
      const float2 uf = __bfloat1622float2(up[e]);
      rp[e] = __floats2bfloat162_rn(activate_fast(gf.x, kind) * uf.x, activate_fast(gf.y, kind) * uf.y);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * intermediate + i) = result;
  }
}

// ---------------------------------------------------------------------------
// Bias, unit-RMS queries and keys, and the cache write of an attention layer without a rotation.
// One warp per (token, head): the row of the product is [H query heads of `key_size` | G key heads
// of `key_size` | G value heads of `value_size`] (G = 0: a layer that reads another layer's keys and
// values computes queries only).  With `normalise`, a query or key head x becomes
// x / sqrt(mean(x^2) + eps), in 32-bit, before it is rounded; values pass through.  Queries go to
// q_out [T, H, key_size], keys and values into the pages at slots[t] (negative: not written):
// k_cache [pages, G, page, key_size], v_cache [pages, G, page, value_size].
// With `rotary_pairs` n > 0 the first 2n dimensions of every query and key head are rotated by
// the token's position: pair i is (i, i + n) (`interleaved` 0) or (2i, 2i + 1) (`interleaved` 1),
// (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * inv_freq[i], in 32-bit.
// Value mixing across layers (`value_mix`): 1 = this layer is the source, its values are also
// left in `shared_values` [T, G * value_size] (32-bit); 2 = its values become
// (1 - m) v + m shared_values[t] with the scalar m = *mix, before they are cached.
// Norm weights: with `normalise` 1 and q_weight / k_weight [key_size], a normalised query or key
// head is multiplied by the weight (one for all query heads, one for all key heads) before the
// rotation.  With `normalise` 2 the root mean square is taken over all query heads of the row at
// once (and over all key heads at once) and the weights are [H * key_size] and [G * key_size].
// With `values_from_keys` the row holds no values, [H query heads | G key heads]: a token's
// cached value head is its key head as projected (bias added), before norm and rotation.
// ---------------------------------------------------------------------------
template <typename TIn, typename T>
__global__ void qkv_norm_store_kernel(const TIn* __restrict__ qkv, int splits, size_t split_stride,
                                      const float* __restrict__ bias, const int* __restrict__ slots,
                                      T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                      int num_tokens, int num_heads, int num_kv_heads, int key_size, int value_size,
                                      int normalise, float eps, int page_size, int num_pages,
                                      const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                      int rotary_pairs, int interleaved, int value_mix,
                                      float* __restrict__ shared_values, const void* __restrict__ mix, int mix_dtype,
                                      const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                                      int values_from_keys, int token_blocks, int* status) {
  // token_blocks: a CTA is one token, a warp per head of its row (at most 32); the heads of a section
  // then share their sums of squares through shared memory instead of each adding up the whole section
  __shared__ float head_squares[32];
  __shared__ float pair_cos[128], pair_sin[128];      // token_blocks: the token's angles, made once for all heads
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int per_token = num_heads + 2 * num_kv_heads;
  if (warp >= (long long)num_tokens * per_token) return;
  bool rotate = rotary_pairs > 0;
  int value_head = -1;
  const int t = (int)(warp / per_token);
  const int item = (int)(warp - (long long)t * per_token);
  const int width = (num_heads + num_kv_heads) * key_size + (values_from_keys ? 0 : num_kv_heads * value_size);
  int size, base;
  T* dst;
  bool unit = normalise != 0;
  bool live = true;                   // false: a key or value head of a token that is not cached
  const float* weight = nullptr;     // the norm's weight for this head, indexed by the dimension
  int section = 0, section_size = 0;  // normalise 2: the part of the row whose root mean square counts
  if (item < num_heads) {
    size = key_size;
    base = item * key_size;
    dst = q_out + ((size_t)t * num_heads + item) * key_size;
    if (q_weight) weight = normalise == 2 ? q_weight + base : q_weight;
    section_size = num_heads * key_size;
  } else {
    const int slot = slots ? slots[t] : -1;
    int page = 0, offset = 0;
    if (slot < 0) {
      live = false;
    } else {
      page = slot / page_size;
      offset = slot - page * page_size;
      if (page >= num_pages) {
        if (lane == 0) atomicOr(status, kStatusBadPage);
        live = false;
        page = 0;
      }
    }
    if (!live && !token_blocks) return;      // a warp of a token's CTA stays for the CTA's barrier
    if (item < num_heads + num_kv_heads) {
      const int head = item - num_heads;
      size = key_size;
      base = item * key_size;
      dst = k_cache + (((size_t)page * num_kv_heads + head) * page_size + offset) * key_size;
      if (k_weight) weight = normalise == 2 ? k_weight + head * key_size : k_weight;
      section = num_heads * key_size;
      section_size = num_kv_heads * key_size;
    } else {
      const int head = item - num_heads - num_kv_heads;
      size = value_size;
      base = values_from_keys ? (num_heads + head) * key_size
                              : (num_heads + num_kv_heads) * key_size + head * value_size;
      dst = v_cache + (((size_t)page * num_kv_heads + head) * page_size + offset) * value_size;
      unit = false;
      rotate = false;
      value_head = head;
    }
  }
  constexpr int kPerLane = 8;   // head sizes up to 256
  const TIn* row = qkv + (size_t)t * width + base;
  float v[kPerLane];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int d = lane + 32 * i;
    v[i] = 0.f;
    if (d < size) {
      v[i] = sum_splits(row + d, splits, split_stride);
      if (bias) v[i] += bias[base + d];
      ss += v[i] * v[i];
    }
  }
  float factor = 1.f;
  if (token_blocks) {
    const float mine = warp_sum(ss);
    if (lane == 0) head_squares[item] = mine;
    if (rotary_pairs > 0) {
      const float pos = (float)positions[t];
      for (int i = threadIdx.x; i < rotary_pairs; i += blockDim.x) sincosf(pos * inv_freq[i], &pair_sin[i], &pair_cos[i]);
    }
    __syncthreads();
    if (!live) return;
    if (unit) {
      // the section's heads in order: the same sum in every warp of the section
      const int head0 = section == 0 ? 0 : num_heads, count = section == 0 ? num_heads : num_kv_heads;
      float all = 0.f;
      for (int i = 0; i < count; ++i) all += head_squares[head0 + i];
      factor = rsqrtf(all / (float)section_size + eps);
    }
  } else if (unit && normalise == 2) {
    // every warp of the section adds up the same squares in the same order
    const TIn* whole = qkv + (size_t)t * width + section;
    float all = 0.f;
    for (int d = lane; d < section_size; d += 32) {
      float x = sum_splits(whole + d, splits, split_stride);
      if (bias) x += bias[section + d];
      all += x * x;
    }
    factor = rsqrtf(warp_sum(all) / (float)section_size + eps);
  } else if (unit) {
    factor = rsqrtf(warp_sum(ss) / (float)size + eps);
  }
  if (weight) {
    // the weight comes before the rotation: scale the head now, and its partners as they are fetched
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d < size) v[i] *= factor * weight[d];
    }
  }
  if (rotate) {
    const float pos = (float)positions[t];
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d < 2 * rotary_pairs) {
        // the other element of the pair comes from the product again (it lies in another lane)
        int pair, other;
        bool leads;
        if (interleaved) {
          pair = d >> 1; leads = (d & 1) == 0; other = d ^ 1;
        } else {
          leads = d < rotary_pairs; pair = leads ? d : d - rotary_pairs; other = leads ? d + rotary_pairs : pair;
        }
        float w = sum_splits(row + other, splits, split_stride);
        if (bias) w += bias[base + other];
        if (weight) w *= factor * weight[other];
        float sn, cs;
        if (token_blocks) {
          sn = pair_sin[pair];
          cs = pair_cos[pair];
        } else {
          sincosf(pos * inv_freq[pair], &sn, &cs);
        }
        v[i] = leads ? v[i] * cs - w * sn : v[i] * cs + w * sn;
      }
    }
  }
  if (value_head >= 0 && value_mix) {
    float* shared_row = shared_values + ((size_t)t * num_kv_heads + value_head) * value_size;
    const float m = value_mix == 2 ? (mix_dtype == kFloat32 ? *(const float*)mix : to_float(*(const __nv_bfloat16*)mix)) : 0.f;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d < size) {
        if (value_mix == 1) shared_row[d] = v[i];
        else v[i] = (1.f - m) * v[i] + m * shared_row[d];
      }
    }
  }
  if (weight) factor = 1.f;     // applied above
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d < size) dst[d] = from_float<T>(v[i] * factor);
  }
}

// The same store for rows of bfloat16 at prompt sizes: a CTA per token, a thread per 16-byte piece
// of the row (eight elements of one head), so every load and store is a whole piece.  Sums of
// squares meet in shared memory piece by piece, then head by head (and, for a norm over whole
// rows, section by section), always in index order; the token's angles are made once; a rotated
// piece finds its partner (the piece `rotary_pairs` elements on or back in the same head) in a copy
// of the normalised row in shared memory.  No bias, no partial sums, no value mixing, halves
// layout only, head sizes and rotated widths that are multiples of eight: the launcher sends
// everything else to the kernel above.
__global__ void qkv_norm_store_bf16x8_kernel(const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ slots,
                                             __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_cache,
                                             __nv_bfloat16* __restrict__ v_cache, int num_heads, int num_kv_heads,
                                             int key_size, int value_size, int normalise, float eps, int page_size,
                                             int num_pages, const int* __restrict__ positions,
                                             const float* __restrict__ inv_freq, int rotary_pairs,
                                             const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                                             int values_from_keys, int* status) {
  extern __shared__ float smem[];
  const int qk_heads = num_heads + num_kv_heads;
  const int qk_width = qk_heads * key_size;
  const int width = qk_width + (values_from_keys ? 0 : num_kv_heads * value_size);
  float* piece_squares = smem;                          // [qk_width / 8]
  float* head_squares = piece_squares + qk_width / 8;   // [qk_heads]
  float* cos_t = head_squares + qk_heads;               // [rotary_pairs]
  float* sin_t = cos_t + rotary_pairs;
  float* normed = sin_t + rotary_pairs;                 // [qk_width], only with a rotation
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int e0 = threadIdx.x * 8;
  const bool mine = e0 < width;
  const bool is_qk = mine && e0 < qk_width;
  const int item = is_qk ? e0 / key_size : 0;                       // query heads, then key heads
  const int d0 = is_qk ? e0 - item * key_size : 0;
  const bool is_key = is_qk && item >= num_heads;
  int page = -1, offset = 0;
  {
    const int slot = slots ? slots[t] : -1;
    if (slot >= 0) {
      page = slot / page_size;
      offset = slot - page * page_size;
      if (page >= num_pages) {
        if (threadIdx.x == 0) atomicOr(status, kStatusBadPage);
        page = -1;
      }
    }
  }
  float x[8];
  if (mine) load8(qkv + (size_t)t * width + e0, nullptr, x);
  if (is_key && values_from_keys && page >= 0) {
    // the values: the keys as they came, before anything is done to them
    const int head = item - num_heads;
    store8(v_cache + (((size_t)page * num_kv_heads + head) * page_size + offset) * value_size + d0, x);
  }
  if (mine && !is_qk) {
    if (page >= 0) {
      const int v0 = e0 - qk_width, head = v0 / value_size;
      store8(v_cache + (((size_t)page * num_kv_heads + head) * page_size + offset) * value_size + (v0 - head * value_size), x);
    }
  }
  if (is_qk && normalise) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
    piece_squares[threadIdx.x] = ss;
  }
  if (rotary_pairs > 0) {
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < rotary_pairs; i += blockDim.x) sincosf(pos * inv_freq[i], &sin_t[i], &cos_t[i]);
  }
  __syncthreads();
  const int pieces_per_head = key_size / 8;
  if (normalise) {
    if (is_qk && d0 == 0) {
      float all = 0.f;
      for (int i = 0; i < pieces_per_head; ++i) all += piece_squares[threadIdx.x + i];
      head_squares[item] = all;
    }
    __syncthreads();
  }
  if (is_qk) {
    float factor = 1.f;
    if (normalise == 1) {
      factor = rsqrtf(head_squares[item] / (float)key_size + eps);
    } else if (normalise == 2) {
      const int head0 = is_key ? num_heads : 0, count = is_key ? num_kv_heads : num_heads;
      float all = 0.f;
      for (int i = 0; i < count; ++i) all += head_squares[head0 + i];
      factor = rsqrtf(all / (float)(count * key_size) + eps);
    }
    const float* weight = is_key ? k_weight : q_weight;
    if (weight) {
      const float* w = weight + (normalise == 2 ? (is_key ? (item - num_heads) * key_size : item * key_size) : 0) + d0;
      const float4 w0 = *reinterpret_cast<const float4*>(w), w1 = *reinterpret_cast<const float4*>(w + 4);
      const float ws[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] *= factor * ws[i];
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] *= factor;
    }
    if (rotary_pairs > 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) normed[e0 + i] = x[i];
    }
  }
  if (rotary_pairs > 0) {
    __syncthreads();
    if (is_qk && d0 < 2 * rotary_pairs) {
      const bool leads = d0 < rotary_pairs;
      const int pair0 = leads ? d0 : d0 - rotary_pairs;
      const float* other = normed + (leads ? e0 + rotary_pairs : e0 - rotary_pairs);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float cs = cos_t[pair0 + i], sn = sin_t[pair0 + i];
        x[i] = leads ? x[i] * cs - other[i] * sn : x[i] * cs + other[i] * sn;
      }
    }
  }
  if (is_qk && !is_key) store8(q_out + ((size_t)t * num_heads + item) * key_size + d0, x);
  if (is_key && page >= 0) {
    const int head = item - num_heads;
    store8(k_cache + (((size_t)page * num_kv_heads + head) * page_size + offset) * key_size + d0, x);
  }
}

// out[m, n] += bias[n]: the bias of a matrix product that a library computed.
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ out, const float* __restrict__ bias, int n, size_t total) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    out[idx] = from_float<T>(to_float(out[idx]) + bias[idx % n]);
  }
}

// Several branches' outputs joined after a norm each: out = scale * sum_i w_i * x_i / rms(x_i), row
// by row in 32-bit, the root mean square over the row with eps inside the root.  A term may be the
// partial sums of a split-K product.  One CTA per row.  A row of up to kJoinKeep elements a thread
// stays in registers between the sums of squares and the output; a wider one is summed twice from
// global memory (the second read comes from the cache), so any width goes.
struct JoinTerm {
  const void* x; int dtype; int splits; long long stride; const float* weight;
};
struct JoinArgs {
  JoinTerm term[4];
  int terms;
};

__device__ __forceinline__ float join_value(const JoinTerm& term, size_t at) {
  if (term.dtype == kFloat32) return sum_splits((const float*)term.x + at, term.splits, (size_t)term.stride);
  return to_float(((const __nv_bfloat16*)term.x)[at]);
}

constexpr int kJoinKeep = 8;

__global__ void norm_join_kernel(const __grid_constant__ JoinArgs a, float eps, float scale, float* __restrict__ out,
                                 int width) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = (size_t)blockIdx.x * width;
  float factor[4];
  if (width <= (int)blockDim.x * kJoinKeep) {
    float total[kJoinKeep];
#pragma unroll
    for (int j = 0; j < kJoinKeep; ++j) total[j] = 0.f;
    for (int i = 0; i < a.terms; ++i) {
      float x[kJoinKeep];
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < kJoinKeep; ++j) {
        const int d = threadIdx.x + j * blockDim.x;
        x[j] = d < width ? join_value(a.term[i], row + d) : 0.f;
        ss += x[j] * x[j];
      }
      const float f = rsqrtf(block_sum(ss, scratch) / (float)width + eps);
#pragma unroll
      for (int j = 0; j < kJoinKeep; ++j) {
        const int d = threadIdx.x + j * blockDim.x;
        if (d < width) total[j] += a.term[i].weight[d] * (x[j] * f);
      }
    }
#pragma unroll
    for (int j = 0; j < kJoinKeep; ++j) {
      const int d = threadIdx.x + j * blockDim.x;
      if (d < width) out[row + d] = scale * total[j];
    }
    return;
  }
  for (int i = 0; i < a.terms; ++i) {
    float ss = 0.f;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
      const float x = join_value(a.term[i], row + d);
      ss += x * x;
    }
    factor[i] = rsqrtf(block_sum(ss, scratch) / (float)width + eps);
  }
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    float v = 0.f;
    for (int i = 0; i < a.terms; ++i) v += a.term[i].weight[d] * (join_value(a.term[i], row + d) * factor[i]);
    out[row + d] = scale * v;
  }
}

// The same for many rows whose width is a multiple of eight and one or two terms: a warp per row,
// a lane holds kChunks pieces of eight elements of either term (16-byte loads of bfloat16, two of
// floats), all of them asked for before the first sum of squares, and the row stays in registers up
// to the output.
template <int kChunks>
__device__ __forceinline__ void join_load_row(const JoinTerm& term, size_t base, int lane, int width, float (&x)[kChunks][8]) {
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int d = (c * 32 + lane) * 8;
    if (d < width) {
      if (term.dtype == kFloat32) {
        const float4 lo = load4((const float*)term.x + base + d), hi = load4((const float*)term.x + base + d + 4);
        x[c][0] = lo.x; x[c][1] = lo.y; x[c][2] = lo.z; x[c][3] = lo.w;
        x[c][4] = hi.x; x[c][5] = hi.y; x[c][6] = hi.z; x[c][7] = hi.w;
      } else {
        load8((const __nv_bfloat16*)term.x + base + d, nullptr, x[c]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) x[c][i] = 0.f;
    }
  }
}

template <int kChunks>
__global__ void norm_join_warp_kernel(const __grid_constant__ JoinArgs a, float eps, float scale,
                                      float* __restrict__ out, int rows, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const size_t base = (size_t)row * width;
  const bool two = a.terms > 1;
  float x0[kChunks][8], x1[kChunks][8];
  join_load_row<kChunks>(a.term[0], base, lane, width, x0);
  if (two) join_load_row<kChunks>(a.term[1], base, lane, width, x1);
  float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
  for (int c = 0; c < kChunks; ++c)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      ss0 += x0[c][i] * x0[c][i];
      if (two) ss1 += x1[c][i] * x1[c][i];
    }
  const float f0 = rsqrtf(warp_sum(ss0) / (float)width + eps);
  const float f1 = two ? rsqrtf(warp_sum(ss1) / (float)width + eps) : 0.f;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int d = (c * 32 + lane) * 8;
    if (d >= width) continue;
    float v[8];
    {
      const float4 w0 = load4(a.term[0].weight + d), w1 = load4(a.term[0].weight + d + 4);
      const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = w[i] * (x0[c][i] * f0);
    }
    if (two) {
      const float4 w0 = load4(a.term[1].weight + d), w1 = load4(a.term[1].weight + d + 4);
      const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += w[i] * (x1[c][i] * f1);
    }
    store4(out + base + d, make_float4(scale * v[0], scale * v[1], scale * v[2], scale * v[3]));
    store4(out + base + d + 4, make_float4(scale * v[4], scale * v[5], scale * v[6], scale * v[7]));
  }
}

// out = cap * tanh(scale * out / cap), in place: a constant factor and the soft cap on logits;
// cap 0: the factor alone.
__global__ void softcap_kernel(float* __restrict__ values, long long n, float cap, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const float inv = cap > 0.f ? 1.f / cap : 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = values[i] * scale;
    values[i] = cap > 0.f ? cap * tanhf(v * inv) : v;
  }
}

}  // namespace einf

using namespace einf;

static inline int pick_threads(int work) {
  int threads = 32;
  while (threads < work && threads < 256) threads <<= 1;
  return threads;
}

extern "C" int einf_embed(const int* tokens, const void* table, int table_dtype, float* residual,
                          int num_tokens, int hidden, int vocab, int* status, const int* positions,
                          const void* pos_table, int max_positions, float scale, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const int threads = pick_threads(hidden);
  EINF_DISPATCH_2(table_dtype, T, {
    return (int)launch_pdl(embed_kernel<T>, num_tokens, threads, 0, stream, tokens, (const T*)table, residual, hidden,
                           vocab, status, positions, (const T*)pos_table, max_positions, scale);
  })
}

typedef CUresult (*PwEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static PwEncodeTiledFn pw_encode_tiled() {
  static PwEncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess)
      return (PwEncodeTiledFn) nullptr;
    return (PwEncodeTiledFn)ptr;
  }();
  return fn;
}

// status: the step's status word (may be null: the TMA-fed kernel, whose wait is bounded, is then not used).
extern "C" int einf_add_rmsnorm(const void* x, int x_dtype, int splits, long long split_stride,
                                float* residual, const float* weight, float eps, void* out,
                                int out_dtype, const int* rows, int num_rows, int hidden,
                                int write_residual, int* status, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  // With partial sums to add up, one element per thread keeps the loads of a row in flight together.
  int threads = pick_threads(hidden);
  if (splits > 1 || num_rows <= 128)
    while (threads < hidden && threads < 1024) threads <<= 1;
  const size_t smem = (size_t)(hidden + 33 + 3) / 4 * 4 * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  const int vectorised = (splits == 1 && hidden % 4 == 0 && ((uintptr_t)residual & 15) == 0 &&
                          ((uintptr_t)weight & 15) == 0) ? 1 : 0;
  if (vectorised && num_rows > 128) {
    threads = 32;
    while (threads * 4 < hidden && threads < 256) threads <<= 1;
  }
  const bool few_rows = num_rows <= 16 || (splits > 1 && num_rows <= 64);
  const bool x_vector = !x || (((uintptr_t)x & 15) == 0 && split_stride % 4 == 0);
  // Partial sums of a split-K product for up to 64 rows: one CTA per row with the partial sums
  // brought in by TMA (see the kernel).  Measured, 0.5B sizes, decode steps of 1 / 8 / 16 / 32
  // requests: 0.732 -> 0.725, 0.803 -> 0.787, 0.917 -> 0.881, 1.175 -> 1.115 ms.
  if (status && x && x_dtype == kFloat32 && splits >= 2 && splits <= 16 && num_rows >= 1 && num_rows <= 64 &&
      hidden % 4 == 0 && hidden >= 128 && hidden <= 4096 &&
      (size_t)((hidden + kRowTmaCols - 1) / kRowTmaCols) * splits * kRowTmaCols * 4 <= 160 * 1024 && x_vector &&
      split_stride % hidden == 0 && split_stride / hidden >= num_rows &&
      ((uintptr_t)residual & 15) == 0 && ((uintptr_t)weight & 15) == 0 && ((uintptr_t)out & 15) == 0 && pw_encode_tiled()) {
    const long long x_rows = split_stride / hidden;
    CUtensorMap map_x;
    cuuint64_t dims[3] = {(cuuint64_t)hidden, (cuuint64_t)x_rows, (cuuint64_t)splits};
    cuuint64_t strides[2] = {(cuuint64_t)hidden * 4, (cuuint64_t)split_stride * 4};
    cuuint32_t box[3] = {(cuuint32_t)kRowTmaCols, 1, (cuuint32_t)splits};
    cuuint32_t element_strides[3] = {1, 1, 1};
    if (pw_encode_tiled()(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(x), dims, strides, box,
                          element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS) {
      const int row_threads = (hidden / 4 + 31) / 32 * 32;
      const int boxes = (hidden + kRowTmaCols - 1) / kRowTmaCols;
      const size_t row_bytes = (size_t)boxes * splits * kRowTmaCols * 4;
      EINF_DISPATCH_2(out_dtype, TOut, {
        auto kernel = add_rmsnorm_row_tma_kernel<TOut>;
        if (row_bytes > 48 * 1024) {
          cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)row_bytes);
          if (e != cudaSuccess) return (int)e;
        }
        return (int)launch_pdl(kernel, num_rows, row_threads, row_bytes, stream, map_x, splits, residual, weight, eps,
                               (TOut*)out, rows, hidden, write_residual, status);
      })
    }
  }
  // From five rows on one CTA per row; below that the cluster kernel, whose four CTAs per row pull
  // a row's partial sums through four SMs (0.5B sizes, decode step: 4 rows 0.803 against 0.826 ms,
  // 6 rows 0.857 against 0.843 ms).
  if (few_rows && num_rows >= 5 && hidden % 4 == 0 && hidden >= 128 && hidden <= 4096 && x_vector && ((uintptr_t)residual & 15) == 0 &&
      ((uintptr_t)weight & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    const int row_threads = (hidden / 4 + 31) / 32 * 32;
    EINF_DISPATCH_2(x_dtype, TX, {
      EINF_DISPATCH_2(out_dtype, TOut, {
        return (int)launch_pdl(add_rmsnorm_row_kernel<TX, TOut>, num_rows, row_threads, 0, stream, (const TX*)x, splits,
                               (size_t)split_stride, residual, weight, eps, (TOut*)out, rows, hidden, write_residual);
      })
    })
  }
  if (few_rows && hidden >= 256 && hidden <= 4 * 4 * 1024) {
    // few rows, or partial sums to add up: a cluster of four CTAs per row
    const int cluster = 4;
    const int slice = (hidden + cluster - 1) / cluster;
    int cluster_threads = 32;
    while (cluster_threads * 4 < slice) cluster_threads <<= 1;   // at most four elements per thread ...
    while (cluster_threads < slice && cluster_threads < 256) cluster_threads <<= 1;   // ... and one where it fits
    EINF_DISPATCH_2(x_dtype, TX, {
      EINF_DISPATCH_2(out_dtype, TOut, {
        return (int)launch_pdl_cluster(add_rmsnorm_cluster_kernel<TX, TOut>, dim3(cluster, num_rows), dim3(cluster_threads),
                                       0, cluster, stream, (const TX*)x, splits, (size_t)split_stride, residual, weight,
                                       eps, (TOut*)out, rows, hidden, write_residual);
      })
    })
  }
  const bool x_aligned = !x || ((uintptr_t)x & 15) == 0;
  if (vectorised && num_rows > 128 && hidden <= 4096 && x_aligned && ((uintptr_t)out & 15) == 0) {
    const int warps_per_block = 4;   // small blocks: rows spread evenly over the SMs even at a few hundred rows
    const int blocks = (num_rows + warps_per_block - 1) / warps_per_block;
    EINF_DISPATCH_2(x_dtype, TX, {
      EINF_DISPATCH_2(out_dtype, TOut, {
        if (hidden <= 1024)
          return (int)launch_pdl(add_rmsnorm_warp_kernel<TX, TOut, 8>, blocks, warps_per_block * 32, 0, stream,
                                 (const TX*)x, residual, weight, eps, (TOut*)out, rows, hidden, num_rows, write_residual);
        if (hidden <= 2048)
          return (int)launch_pdl(add_rmsnorm_warp_kernel<TX, TOut, 16>, blocks, warps_per_block * 32, 0, stream,
                                 (const TX*)x, residual, weight, eps, (TOut*)out, rows, hidden, num_rows, write_residual);
        return (int)launch_pdl(add_rmsnorm_warp_kernel<TX, TOut, 32>, blocks, warps_per_block * 32, 0, stream,
                               (const TX*)x, residual, weight, eps, (TOut*)out, rows, hidden, num_rows, write_residual);
      })
    })
  }
  EINF_DISPATCH_2(x_dtype, TX, {
    EINF_DISPATCH_2(out_dtype, TOut, {
      auto kernel = add_rmsnorm_kernel<TX, TOut>;
      if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
      }
      return (int)launch_pdl(kernel, num_rows, threads, smem, stream, (const TX*)x, splits, (size_t)split_stride,
                             residual, weight, eps, (TOut*)out, rows, hidden, write_residual, vectorised);
    })
  })
}

// in_dtype / splits / split_stride: qkv is [T, width] of the activation type (splits = 1), or
// the float partial sums [splits, T, width] of a split-K product.
extern "C" int einf_rope_kv_write(const void* qkv, int in_dtype, int splits, long long split_stride, int dtype,
                                  const float* bias, const int* positions, const float* inv_freq,
                                  const int* slots, void* q_out, void* k_cache, void* v_cache, int num_tokens,
                                  int num_heads, int num_kv_heads, int head_size, int rotary_dim, int page_size,
                                  int num_pages, int* status, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  const int work = (num_heads + num_kv_heads) * head_size / 2;
  int threads = pick_threads(work);
  if (splits > 1 || num_tokens <= 128)
    while (threads < work && threads < 1024) threads <<= 1;
  const size_t smem = (size_t)rotary_dim * sizeof(float);
  auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  if (splits == 1 && in_dtype == kBFloat16 && dtype == kBFloat16 && rotary_dim == head_size && head_size % 16 == 0 &&
      aligned(qkv) && aligned(q_out) && aligned(k_cache) && aligned(v_cache) && (!bias || aligned(bias))) {
    const int items = (num_heads + num_kv_heads) * (head_size / 16) + num_kv_heads * (head_size / 8);
    const int tokens_here = num_tokens < kRopeTokens ? num_tokens : kRopeTokens;
    return (int)launch_pdl(rope_kv_write_bf16x8_kernel, (num_tokens + kRopeTokens - 1) / kRopeTokens,
                           pick_threads(items * tokens_here), (size_t)kRopeTokens * head_size * sizeof(float), stream,
                           (const __nv_bfloat16*)qkv, bias, positions, inv_freq, slots, (__nv_bfloat16*)q_out,
                           (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, num_tokens, num_heads, num_kv_heads,
                           head_size, page_size, num_pages, status);
  }
  if (num_tokens <= 64 && head_size <= 1024) {
    // few tokens: one CTA per (token, head), a thread per pair (or per value of V)
    int head_threads = 32;
    while (head_threads < head_size) head_threads <<= 1;
    const long long blocks = (long long)num_tokens * (num_heads + 2 * num_kv_heads);
    EINF_DISPATCH_2(in_dtype, TIn, {
      EINF_DISPATCH_2(dtype, T, {
        return (int)launch_pdl(rope_kv_write_heads_kernel<TIn, T>, (int)blocks, head_threads, 0, stream,
                               (const TIn*)qkv, splits, (size_t)split_stride, bias, positions, inv_freq, slots,
                               (T*)q_out, (T*)k_cache, (T*)v_cache, num_heads, num_kv_heads, head_size, rotary_dim,
                               page_size, num_pages, status);
      })
    })
  }
  EINF_DISPATCH_2(in_dtype, TIn, {
    EINF_DISPATCH_2(dtype, T, {
      return (int)launch_pdl(rope_kv_write_kernel<TIn, T>, num_tokens, threads, smem, stream, (const TIn*)qkv, splits,
                             (size_t)split_stride, bias, positions, inv_freq, slots, (T*)q_out, (T*)k_cache,
                             (T*)v_cache, num_heads, num_kv_heads, head_size, rotary_dim, page_size, num_pages,
                             status);
    })
  })
}

extern "C" int einf_silu_mul(const void* gate_up, int in_dtype, int splits, long long split_stride, void* out,
                             int dtype, long long num_tokens, int intermediate, cudaStream_t stream) {
  const size_t total = (size_t)num_tokens * intermediate;
  if (total == 0) return 0;
  const int threads = 256;
  if (splits == 1 && in_dtype == kBFloat16 && dtype == kBFloat16 && intermediate % 8 == 0 &&
      ((uintptr_t)gate_up & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    const int vectors_per_row = intermediate >> 3;
    const int chunks = (vectors_per_row + threads - 1) / threads;
    if ((long long)chunks * num_tokens < (1ll << 31))
      return (int)launch_pdl(silu_mul_bf16x8_kernel, (int)(chunks * num_tokens), threads, 0, stream,
                             (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, intermediate, chunks);
  }
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  EINF_DISPATCH_2(in_dtype, TIn, {
    EINF_DISPATCH_2(dtype, T, {
      return (int)launch_pdl(silu_mul_kernel<TIn, T>, (int)blocks, threads, 0, stream, (const TIn*)gate_up, splits,
                             (size_t)split_stride, (T*)out, intermediate, total);
    })
  })
}

extern "C" int einf_act_mul(const void* gate_up, int in_dtype, int splits, long long split_stride, void* out,
                            int dtype, long long num_tokens, int intermediate, int kind, cudaStream_t stream) {
  const size_t total = (size_t)num_tokens * intermediate;
  if (total == 0) return 0;
  const int threads = 256;
  if (splits == 1 && in_dtype == kBFloat16 && dtype == kBFloat16 && intermediate % 8 == 0 &&
      ((uintptr_t)gate_up & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    const int vectors_per_row = intermediate >> 3;
    const int chunks = (vectors_per_row + threads - 1) / threads;
    if ((long long)chunks * num_tokens < (1ll << 31))
      return (int)launch_pdl(act_mul_bf16x8_kernel, (int)(chunks * num_tokens), threads, 0, stream,
                             (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, intermediate, chunks, kind);
  }
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  EINF_DISPATCH_2(in_dtype, TIn, {
    EINF_DISPATCH_2(dtype, T, {
      return (int)launch_pdl(act_mul_kernel<TIn, T>, (int)blocks, threads, 0, stream, (const TIn*)gate_up, splits,
                             (size_t)split_stride, (T*)out, intermediate, kind, total);
    })
  })
}

extern "C" int einf_advance_decode(int* token_ids, int* positions, int* context_lens, const int* sampled,
                                   int num_requests, int* slots0, const int* table0, int* slots1, const int* table1,
                                   int* slots2, const int* table2, int* slots3, const int* table3, int num_groups,
                                   int table_width, int page_size, cudaStream_t stream) {
  if (num_requests == 0) return 0;
  if (num_groups < 0 || num_groups > 4 || page_size <= 0) return (int)cudaErrorInvalidValue;
  AdvanceGroups groups = {{slots0, slots1, slots2, slots3}, {table0, table1, table2, table3}};
  return (int)launch_pdl(advance_decode_kernel, (num_requests + 127) / 128, 128, 0, stream, token_ids, positions,
                         context_lens, sampled, num_requests, groups, num_groups, table_width, page_size);
}

extern "C" int einf_zero_fresh_state(void* state, long long row_bytes, int num_slots, const int* state_slots,
                                     const int* q_start, const int* positions, int num_requests,
                                     cudaStream_t stream) {
  if (num_requests == 0 || row_bytes == 0 || num_slots == 0) return 0;
  if (row_bytes < 0 || num_requests > 65535) return (int)cudaErrorInvalidValue;
  const bool wide = row_bytes % 16 == 0 && (uintptr_t)state % 16 == 0;
  const bool words = row_bytes % 4 == 0 && (uintptr_t)state % 4 == 0;
  const long long row_words = wide ? row_bytes / 16 : words ? row_bytes / 4 : row_bytes;
  const int threads = 256;
  long long blocks = (row_words + threads - 1) / threads;
  if (blocks > 64) blocks = 64;
  const dim3 grid((unsigned)blocks, (unsigned)num_requests);
  if (wide)
    return (int)launch_pdl(zero_fresh_state_kernel<uint4>, grid, threads, 0, stream, (uint4*)state, row_words, num_slots,
                           state_slots, q_start, positions);
  if (words)
    return (int)launch_pdl(zero_fresh_state_kernel<uint32_t>, grid, threads, 0, stream, (uint32_t*)state, row_words,
                           num_slots, state_slots, q_start, positions);
  return (int)launch_pdl(zero_fresh_state_kernel<uint8_t>, grid, threads, 0, stream, (uint8_t*)state, row_words,
                         num_slots, state_slots, q_start, positions);
}

extern "C" int einf_activation(const void* x, int in_dtype, int splits, long long split_stride, void* out, int dtype,
                               long long total, int kind, cudaStream_t stream) {
  if (total <= 0) return 0;
  if (kind < 0 || kind > 3) return (int)cudaErrorInvalidValue;
  const int threads = 256;
  if (splits == 1 && in_dtype == kBFloat16 && dtype == kBFloat16 && total % 8 == 0 && ((uintptr_t)x & 15) == 0 &&
      ((uintptr_t)out & 15) == 0) {
    const size_t vectors = (size_t)total >> 3;
    const size_t blocks = (vectors + threads - 1) / threads;
    if (blocks < (1ull << 31))
      return (int)launch_pdl(activation_bf16x8_kernel, (int)blocks, threads, 0, stream, (const __nv_bfloat16*)x,
                             (__nv_bfloat16*)out, kind, vectors);
  }
  size_t blocks = ((size_t)total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  EINF_DISPATCH_2(in_dtype, TIn, {
    EINF_DISPATCH_2(dtype, T, {
      return (int)launch_pdl(activation_kernel<TIn, T>, (int)blocks, threads, 0, stream, (const TIn*)x, splits,
                             (size_t)split_stride, (T*)out, kind, (size_t)total);
    })
  })
}

extern "C" int einf_qkv_norm_store(const void* qkv, int in_dtype, int splits, long long split_stride, int dtype,
                                   const float* bias, const int* slots, void* q_out, void* k_cache, void* v_cache,
                                   int num_tokens, int num_heads, int num_kv_heads, int key_size, int value_size,
                                   int normalise, float eps, int page_size, int num_pages, const int* positions,
                                   const float* inv_freq, int rotary_pairs, int interleaved, int value_mix,
                                   float* shared_values, const void* mix, int mix_dtype, const float* q_weight,
                                   const float* k_weight, int values_from_keys, int* status,
                                   cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  // norms over whole rows: a CTA per token where its heads fit one (a warp each)
  const int token_blocks = normalise == 2 && num_heads + 2 * num_kv_heads <= 32 ? 1 : 0;
  if (normalise < 0 || normalise > 2 || ((q_weight || k_weight) && !normalise)) return (int)cudaErrorInvalidValue;
  if (values_from_keys && (value_size != key_size || value_mix)) return (int)cudaErrorInvalidValue;
  if (rotary_pairs < 0 || 2 * rotary_pairs > key_size || (rotary_pairs > 0 && (!positions || !inv_freq)))
    return (int)cudaErrorInvalidValue;
  if (value_mix && (!shared_values || (value_mix == 2 && !mix))) return (int)cudaErrorInvalidValue;
  if (key_size > 256 || value_size > 256 || key_size <= 0 || (num_kv_heads > 0 && value_size <= 0))
    return (int)cudaErrorInvalidValue;
  // rows of bfloat16 at prompt sizes: whole 16-byte pieces, a CTA per token
  {
    const int qk_width = (num_heads + num_kv_heads) * key_size;
    const int width = qk_width + (values_from_keys ? 0 : num_kv_heads * value_size);
    const bool aligned = (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache |
                           (uintptr_t)q_weight | (uintptr_t)k_weight) & 15) == 0;
    if (in_dtype == kBFloat16 && dtype == kBFloat16 && splits <= 1 && !bias && !value_mix && !interleaved &&
        num_tokens >= 64 && key_size % 8 == 0 && value_size % 8 == 0 && rotary_pairs % 8 == 0 && width <= 8192 &&
        num_kv_heads > 0 && aligned) {
      const int threads = (width / 8 + 31) / 32 * 32;
      const size_t bytes = (size_t)(qk_width / 8 + num_heads + num_kv_heads + 2 * rotary_pairs +
                                    (rotary_pairs > 0 ? qk_width : 0)) * sizeof(float);
      return (int)launch_pdl(qkv_norm_store_bf16x8_kernel, num_tokens, threads, bytes, stream,
                             (const __nv_bfloat16*)qkv, slots, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache,
                             (__nv_bfloat16*)v_cache, num_heads, num_kv_heads, key_size, value_size, normalise, eps,
                             page_size, num_pages, positions, inv_freq, rotary_pairs, q_weight, k_weight,
                             values_from_keys, status);
    }
  }
  const long long warps = (long long)num_tokens * (num_heads + 2 * num_kv_heads);
  const int threads = token_blocks ? 32 * (num_heads + 2 * num_kv_heads) : 128;
  const long long blocks = token_blocks ? num_tokens : (warps * 32 + threads - 1) / threads;
  if (blocks >= (1ll << 31)) return (int)cudaErrorInvalidValue;
  EINF_DISPATCH_2(in_dtype, TIn, {
    EINF_DISPATCH_2(dtype, T, {
      return (int)launch_pdl(qkv_norm_store_kernel<TIn, T>, (int)blocks, threads, 0, stream, (const TIn*)qkv, splits,
                             (size_t)split_stride, bias, slots, (T*)q_out, (T*)k_cache, (T*)v_cache, num_tokens,
                             num_heads, num_kv_heads, key_size, value_size, normalise, eps, page_size, num_pages,
                             positions, inv_freq, rotary_pairs, interleaved, value_mix, shared_values, mix, mix_dtype,
                             q_weight, k_weight, values_from_keys, token_blocks, status);
    })
  })
}

extern "C" int einf_add_bias(void* out, int dtype, const float* bias, long long rows, int n,
                             cudaStream_t stream) {
  const size_t total = (size_t)rows * n;
  if (total == 0) return 0;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  EINF_DISPATCH_2(dtype, T, {
    add_bias_kernel<T><<<(int)blocks, threads, 0, stream>>>((T*)out, bias, n, total);
  })
  return (int)cudaGetLastError();
}

extern "C" int einf_softcap(float* values, long long n, float cap, float scale, cudaStream_t stream) {
  if (n == 0) return 0;
  if (!(cap >= 0.f)) return (int)cudaErrorInvalidValue;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return (int)launch_pdl(softcap_kernel, (int)blocks, 256, 0, stream, values, n, cap, scale);
}

extern "C" int einf_norm_join(int terms,
                              const void* x0, int d0, int s0, long long st0, const float* w0,
                              const void* x1, int d1, int s1, long long st1, const float* w1,
                              const void* x2, int d2, int s2, long long st2, const float* w2,
                              const void* x3, int d3, int s3, long long st3, const float* w3,
                              float eps, float scale, float* out, int rows, int width, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (terms < 1 || terms > 4 || width <= 0) return (int)cudaErrorInvalidValue;
  JoinArgs a;
  a.terms = terms;
  a.term[0] = {x0, d0, s0, st0, w0};
  a.term[1] = {x1, d1, s1, st1, w1};
  a.term[2] = {x2, d2, s2, st2, w2};
  a.term[3] = {x3, d3, s3, st3, w3};
  for (int i = 0; i < terms; ++i)
    if (!a.term[i].x || !a.term[i].weight || (a.term[i].dtype != kFloat32 && a.term[i].splits > 1))
      return (int)cudaErrorInvalidValue;
  // many rows of whole 16-byte pieces, one or two terms: a warp per row, the row in registers
  bool pieces = rows >= 64 && terms <= 2 && width % 8 == 0 && width <= 32 * 8 * 8 && ((uintptr_t)out & 15) == 0;
  for (int i = 0; i < terms; ++i)
    pieces = pieces && a.term[i].splits <= 1 && ((uintptr_t)a.term[i].x & 15) == 0 && ((uintptr_t)a.term[i].weight & 15) == 0;
  if (pieces) {
    const int warps = 4;
    const int blocks = (rows + warps - 1) / warps;
    if (width <= 32 * 8 * 2)
      return (int)launch_pdl(norm_join_warp_kernel<2>, blocks, warps * 32, 0, stream, a, eps, scale, out, rows, width);
    if (width <= 32 * 8 * 4)
      return (int)launch_pdl(norm_join_warp_kernel<4>, blocks, warps * 32, 0, stream, a, eps, scale, out, rows, width);
    if (width <= 32 * 8 * 6)
      return (int)launch_pdl(norm_join_warp_kernel<6>, blocks, warps * 32, 0, stream, a, eps, scale, out, rows, width);
    return (int)launch_pdl(norm_join_warp_kernel<8>, blocks, warps * 32, 0, stream, a, eps, scale, out, rows, width);
  }
  return (int)launch_pdl(norm_join_kernel, rows, pick_threads(width), 0, stream, a, eps, scale, out, width);
}
