// Score-mixing attention over the paged cache (the statement is at the top of attention_mixed.cu), tiled:
// a CTA takes `rows` consecutive queries of one request with all their heads and walks the keys that
// any of them sees in tiles of 64, so a key or value row is read once for all of them.  Per tile and
// key/value head the keys go to shared memory as floats and every warp computes raw scores for a
// (head, four queries) task, a lane per pair of keys (lane and lane + 32: rows 4 floats apart in the
// padded tile, so a quarter warp's 16-byte reads fall into different banks).  Then a thread per
// (query, key pair) takes the distance off, mixes the heads' scores from registers (the mixing matrix
// is padded to HEADS_PAD columns, the unroll) and masks; then a warp per (head, query) row updates the
// running maximum and sum and leaves the weights; then, per key/value head again, the values go to
// shared memory and every warp adds its tasks' weighted values into registers, a lane per value column.
// Scores, weights, sums and the output are 32-bit.  With several splits (grid.y) each CTA takes a share
// of the key tiles and leaves (maximum, sum, unnormalised output); a second kernel joins them and the
// sink.  Queries that come alone (decoding) use the same kernel with one query a task.
// Compiled per HEADS_PAD (4, 8, 16 or 32 >= heads).
#include "common.cuh"

#ifndef HEADS_PAD
#error "compile with -DHEADS_PAD=<4|8|16|32>"
#endif

namespace einf {

constexpr int kTiledThreads = 256;
constexpr int kTiledWarps = kTiledThreads / 32;
constexpr int kKeyTile = 64;
constexpr int kHP = HEADS_PAD;

struct MixedTiledArgs {
  const void* q;
  const void* k_cache;
  const void* v_cache;
  const int* block_table;
  int table_width;
  const int* seq_of_token;
  const int* positions;
  const int* q_tiles;        // [tiles, 4]: request, first token, rows, first position (tasks of four queries)
  const int* single_tokens;  // token indices (tasks of one query); null: token = block
  void* out;
  int heads, kv_heads, dim, vdim, page_size, num_pages;
  float scale;
  int window;
  const float* slopes;
  const float* talk;
  const float* sink;
  float out_scale;
  int rows, blocks_per_tile, splits;
  int groups_at_once;        // key/value heads whose tiles are in shared memory together
  int values_shared;         // tensor-core kernel: the values' tile takes the keys' place after the first product
  float* part_acc;           // [splits, tokens, heads * vdim]
  float* part_ml;            // [splits, tokens, heads, 2]
  int num_tokens;
  int* status;
};

struct BlockPlace {
  int request, first_token, rows, first_position;
};

template <int QI>
__device__ __forceinline__ BlockPlace block_place(const MixedTiledArgs& a) {
  BlockPlace b;
  if (QI == 1) {
    const int t = a.single_tokens ? a.single_tokens[blockIdx.x] : (int)blockIdx.x;
    b.request = a.seq_of_token[t];
    b.first_token = t;
    b.rows = 1;
    b.first_position = a.positions[t];
  } else {
    const int tile = blockIdx.x / a.blocks_per_tile, sub = blockIdx.x - tile * a.blocks_per_tile;
    const int* item = a.q_tiles + 4 * tile;
    b.request = item[0];
    b.first_token = item[1] + sub * a.rows;
    b.rows = min(a.rows, item[2] - sub * a.rows);
    b.first_position = item[3] + sub * a.rows;
  }
  return b;
}

// Rows j0 .. j0 + 63 of `groups` key/value heads from g0 on, as floats: tile[(g * 64 + key) * ld + d]; rows from
// `count` on are zeros.  `pages` holds the tile's 64 page numbers.  16-byte loads, four in flight a thread,
// where the row width allows; a page outside the pool leaves zeros and sets the status word.
template <typename T>
__device__ __forceinline__ void load_tile(float* __restrict__ tile, int ld, const T* __restrict__ cache, int width,
                                          int g0, int groups, int kv_heads, int page_size, int num_pages,
                                          const int* __restrict__ pages, int j0, int count, int* status) {
  constexpr int kEach = 16 / (int)sizeof(T);
  const int tid = threadIdx.x;
  if (width % kEach == 0) {
    const int chunks = width / kEach, total = groups * kKeyTile * chunks;
    for (int base = tid; base < total; base += 4 * kTiledThreads) {
      uint4 raw[4];
      int at[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int idx = base + e * kTiledThreads;
        raw[e] = make_uint4(0u, 0u, 0u, 0u);
        at[e] = -1;
        if (idx < total) {
          const int row = idx / chunks, c = idx - row * chunks;
          const int g = row / kKeyTile, key = row - g * kKeyTile;
          at[e] = row * ld + c * kEach;
          if (key < count) {
            const int j = j0 + key, page = pages[key];
            if (page >= 0 && page < num_pages)
              raw[e] = *(const uint4*)(cache + (((size_t)page * kv_heads + g0 + g) * page_size + j % page_size) * width +
                                       c * kEach);
            else if (c == 0) atomicOr(status, kStatusBadPage);
          }
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (at[e] < 0) continue;
        const T* v = (const T*)&raw[e];
#pragma unroll
        for (int x = 0; x < kEach; x += 4)
          *(float4*)(tile + at[e] + x) = make_float4(to_float(v[x]), to_float(v[x + 1]), to_float(v[x + 2]), to_float(v[x + 3]));
      }
    }
    return;
  }
  const int total = groups * kKeyTile * width;
  for (int idx = tid; idx < total; idx += kTiledThreads) {
    const int row = idx / width, d = idx - row * width;
    const int g = row / kKeyTile, key = row - g * kKeyTile;
    float value = 0.f;
    if (key < count) {
      const int j = j0 + key, page = pages[key];
      if (page >= 0 && page < num_pages)
        value = to_float(cache[(((size_t)page * kv_heads + g0 + g) * page_size + j % page_size) * width + d]);
      else if (d == 0) atomicOr(status, kStatusBadPage);
    }
    tile[row * ld + d] = value;
  }
}

template <typename T, int QI, int VD>
__global__ void __launch_bounds__(kTiledThreads, 2) paged_attention_mixed_tiled_kernel(const __grid_constant__ MixedTiledArgs a) {
  constexpr int NT = QI == 1 ? 4 : 16 / VD;           // (head, query group) tasks a warp may hold
  extern __shared__ float4 smem4[];
  float* smem = (float*)smem4;
  const int heads = a.heads, dim = a.dim, vdim = a.vdim, QB = a.rows;
  const int per = heads / a.kv_heads;
  const int nq = QB / QI;                             // query groups
  const int ldk = dim + 4;
  float* qs = smem;                                   // [heads * QB, dim], scaled
  const int GB = a.groups_at_once;
  float* kv = qs + heads * QB * dim;                  // [GB * 64, ldk] keys, then [GB * 64, vdim] values
  float* sc = kv + GB * kKeyTile * max(ldk, vdim);    // [heads * QB, 64]
  float* talk_s = sc + heads * QB * kKeyTile;         // [heads, kHP]
  float* slope_s = talk_s + heads * kHP;              // [kHP]
  float* top = slope_s + kHP;                         // [heads * QB]
  float* total = top + heads * QB;
  float* factor = total + heads * QB;
  int* pages = (int*)(factor + heads * QB);           // [2, 64] page numbers of this tile and the next

  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* q = (const T*)a.q;
  const T* k_cache = (const T*)a.k_cache;
  const T* v_cache = (const T*)a.v_cache;
  const bool joins = a.splits > 1;
  for (int i = tid; i < heads * kHP; i += kTiledThreads) {
    const int h = i / kHP, g = i - h * kHP;
    talk_s[i] = g < heads ? (a.talk ? a.talk[h * heads + g] : (h == g ? 1.f : 0.f)) : 0.f;
  }
  for (int g = tid; g < kHP; g += kTiledThreads) slope_s[g] = (a.slopes && g < heads) ? a.slopes[g] : 0.f;
  for (int r = tid; r < heads * QB; r += kTiledThreads) {
    const bool with_sink = a.sink && !joins;
    top[r] = with_sink ? a.sink[r / QB] : -INFINITY;
    total[r] = with_sink ? 1.f : 0.f;
  }
  pdl_wait();
  const BlockPlace place = block_place<QI>(a);
  if (place.rows <= 0) return;
  const int rows = place.rows, p0 = place.first_position;
  for (int idx = tid; idx < heads * QB * dim; idx += kTiledThreads) {
    const int r = idx / dim, d = idx - r * dim;
    const int h = r / QB, i = r - h * QB;
    qs[idx] = i < rows ? to_float(q[((size_t)(place.first_token + i) * heads + h) * dim + d]) * a.scale : 0.f;
  }
  const int hi = p0 + rows - 1;
  const int lo = a.window > 0 ? max(0, p0 - a.window + 1) : 0;
  const int tiles_total = (hi - lo + kKeyTile) / kKeyTile;
  const int tiles_each = (tiles_total + a.splits - 1) / a.splits;
  const int tile_first = blockIdx.y * tiles_each, tile_last = min(tiles_total, tile_first + tiles_each);
  const int* table = a.block_table + (size_t)place.request * a.table_width;

  float acc[NT][QI][VD];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int qi = 0; qi < QI; ++qi)
#pragma unroll
      for (int dd = 0; dd < VD; ++dd) acc[n][qi][dd] = 0.f;

  if (tid < kKeyTile && tile_first < tile_last) {
    const int j = lo + tile_first * kKeyTile + tid;
    pages[(tile_first & 1) * kKeyTile + tid] = j <= hi ? table[j / a.page_size] : 0;
  }
  for (int tile = tile_first; tile < tile_last; ++tile) {
    const int j0 = lo + tile * kKeyTile;
    const int count = min(kKeyTile, hi - j0 + 1);
    const int* tile_pages = pages + (tile & 1) * kKeyTile;
    if (tid < kKeyTile && tile + 1 < tile_last) {     // read after the barriers below, written again two tiles on
      const int j = j0 + kKeyTile + tid;
      pages[((tile + 1) & 1) * kKeyTile + tid] = j <= hi ? table[j / a.page_size] : 0;
    }
    // ---- raw scores, a few key/value heads after the others
    for (int g0 = 0; g0 < a.kv_heads; g0 += GB) {
      const int groups = min(GB, a.kv_heads - g0);
      __syncthreads();                                // kv is free (and, the first time, qs and pages are written)
      load_tile(kv, ldk, k_cache, dim, g0, groups, a.kv_heads, a.page_size, a.num_pages, tile_pages, j0, count, a.status);
      __syncthreads();
      for (int task = warp; task < groups * per * nq; task += kTiledWarps) {
        const int h = g0 * per + task / nq, iq = task % nq;
        float s[QI][2];
#pragma unroll
        for (int qi = 0; qi < QI; ++qi) s[qi][0] = s[qi][1] = 0.f;
        const float* k0 = kv + ((h / per - g0) * kKeyTile + lane) * ldk;
        const float* k1 = k0 + 32 * ldk;
        const float* qr = qs + (size_t)(h * QB + iq * QI) * dim;
        for (int d = 0; d < dim; d += 4) {
          const float4 x0 = *(const float4*)(k0 + d), x1 = *(const float4*)(k1 + d);
#pragma unroll
          for (int qi = 0; qi < QI; ++qi) {
            const float4 y = *(const float4*)(qr + qi * dim + d);
            s[qi][0] = fmaf(y.x, x0.x, s[qi][0]); s[qi][0] = fmaf(y.y, x0.y, s[qi][0]);
            s[qi][0] = fmaf(y.z, x0.z, s[qi][0]); s[qi][0] = fmaf(y.w, x0.w, s[qi][0]);
            s[qi][1] = fmaf(y.x, x1.x, s[qi][1]); s[qi][1] = fmaf(y.y, x1.y, s[qi][1]);
            s[qi][1] = fmaf(y.z, x1.z, s[qi][1]); s[qi][1] = fmaf(y.w, x1.w, s[qi][1]);
          }
        }
#pragma unroll
        for (int qi = 0; qi < QI; ++qi) {
          float* row = sc + (size_t)(h * QB + iq * QI + qi) * kKeyTile;
          row[lane] = s[qi][0];
          row[lane + 32] = s[qi][1];
        }
      }
    }
    __syncthreads();
    // ---- distance, mixing and mask: a warp per query, a lane per pair of keys
    for (int i = warp; i < QB; i += kTiledWarps) {
      const int position = p0 + i;
      float raw0[kHP], raw1[kHP];
      const float away0 = (float)(position - (j0 + lane)), away1 = (float)(position - (j0 + lane + 32));
#pragma unroll
      for (int g = 0; g < kHP; ++g) {
        if (g < heads) {
          const float* row = sc + (size_t)(g * QB + i) * kKeyTile;
          raw0[g] = row[lane] - slope_s[g] * away0;
          raw1[g] = row[lane + 32] - slope_s[g] * away1;
        } else {
          raw0[g] = raw1[g] = 0.f;
        }
      }
      const int reach = a.window > 0 ? position - a.window : -1;       // the last key out of sight
      const bool see0 = i < rows && j0 + lane <= position && j0 + lane > reach;
      const bool see1 = i < rows && j0 + lane + 32 <= position && j0 + lane + 32 > reach;
      for (int h = 0; h < heads; ++h) {
        const float4* mix = (const float4*)(talk_s + h * kHP);
        float m0 = 0.f, m1 = 0.f;
#pragma unroll
        for (int g4 = 0; g4 < kHP / 4; ++g4) {
          const float4 w = mix[g4];
          m0 = fmaf(w.x, raw0[4 * g4], m0); m0 = fmaf(w.y, raw0[4 * g4 + 1], m0);
          m0 = fmaf(w.z, raw0[4 * g4 + 2], m0); m0 = fmaf(w.w, raw0[4 * g4 + 3], m0);
          m1 = fmaf(w.x, raw1[4 * g4], m1); m1 = fmaf(w.y, raw1[4 * g4 + 1], m1);
          m1 = fmaf(w.z, raw1[4 * g4 + 2], m1); m1 = fmaf(w.w, raw1[4 * g4 + 3], m1);
        }
        float* row = sc + (size_t)(h * QB + i) * kKeyTile;
        row[lane] = see0 ? m0 : -INFINITY;
        row[lane + 32] = see1 ? m1 : -INFINITY;
      }
    }
    __syncthreads();
    // ---- running maximum and sum, a warp per (head, query) row; the weights stay in place
    for (int r = warp; r < heads * QB; r += kTiledWarps) {
      float* row = sc + (size_t)r * kKeyTile;
      const float s0 = row[lane], s1 = row[lane + 32];
      const float best = warp_max(fmaxf(s0, s1));
      const float before = top[r];
      const float now = fmaxf(before, best);
      const float w0 = s0 == -INFINITY ? 0.f : expf(s0 - now);
      const float w1 = s1 == -INFINITY ? 0.f : expf(s1 - now);
      row[lane] = w0;
      row[lane + 32] = w1;
      const float sum = warp_sum(w0 + w1);
      if (lane == 0) {
        const float f = before == -INFINITY ? 0.f : expf(before - now);
        factor[r] = f;
        total[r] = fmaf(total[r], f, sum);
        top[r] = now;
      }
    }
    // ---- values, one key/value head after the other
    for (int g0 = 0; g0 < a.kv_heads; g0 += GB) {
      const int groups = min(GB, a.kv_heads - g0);
      __syncthreads();                                // weights and factors are written; kv is free
      load_tile(kv, vdim, v_cache, vdim, g0, groups, a.kv_heads, a.page_size, a.num_pages, tile_pages, j0, count, a.status);
      __syncthreads();
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int task = n * kTiledWarps + warp;
        if (task >= heads * nq) continue;
        const int h = task / nq, iq = task - h * nq;
        const int g = h / per - g0;
        if (g < 0 || g >= groups) continue;
        const float* values = kv + (size_t)g * kKeyTile * vdim;
        const int r0 = h * QB + iq * QI;
#pragma unroll
        for (int qi = 0; qi < QI; ++qi) {
          const float f = factor[r0 + qi];
#pragma unroll
          for (int dd = 0; dd < VD; ++dd) acc[n][qi][dd] *= f;
        }
        for (int key = 0; key < kKeyTile; key += 4) {
          float v[4][VD];
#pragma unroll
          for (int e = 0; e < 4; ++e)
#pragma unroll
            for (int dd = 0; dd < VD; ++dd) {
              const int d = lane + 32 * dd;
              v[e][dd] = d < vdim ? values[(key + e) * vdim + d] : 0.f;
            }
#pragma unroll
          for (int qi = 0; qi < QI; ++qi) {
            const float4 w = *(const float4*)(sc + (size_t)(r0 + qi) * kKeyTile + key);
#pragma unroll
            for (int dd = 0; dd < VD; ++dd) {
              float o = acc[n][qi][dd];
              o = fmaf(w.x, v[0][dd], o); o = fmaf(w.y, v[1][dd], o);
              o = fmaf(w.z, v[2][dd], o); o = fmaf(w.w, v[3][dd], o);
              acc[n][qi][dd] = o;
            }
          }
        }
      }
    }
  }
  __syncthreads();                                    // the statistics, also when there was no tile
  const int outs = heads * vdim;
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int task = n * kTiledWarps + warp;
    if (task >= heads * nq) continue;
    const int h = task / nq, iq = task - h * nq;
#pragma unroll
    for (int qi = 0; qi < QI; ++qi) {
      const int i = iq * QI + qi;
      if (i >= rows) continue;
      const int r = h * QB + i;
      const size_t t = (size_t)place.first_token + i;
#pragma unroll
      for (int dd = 0; dd < VD; ++dd) {
        const int d = lane + 32 * dd;
        if (d >= vdim) continue;
        if (joins) a.part_acc[((size_t)blockIdx.y * a.num_tokens + t) * outs + h * vdim + d] = acc[n][qi][dd];
        else ((T*)a.out)[t * outs + h * vdim + d] = from_float<T>(acc[n][qi][dd] / total[r] * a.out_scale);
      }
      if (joins && lane == 0) {
        float* ml = a.part_ml + (((size_t)blockIdx.y * a.num_tokens + t) * heads + h) * 2;
        ml[0] = top[r];
        ml[1] = total[r];
      }
    }
  }
}

#if HEADS_PAD <= 16
// ---------------------------------------------------------------------------
// The same for bfloat16 prompt portions with the two products on the tensor cores (mma.sync m16n8k16, 32-bit
// accumulators): 16 queries a CTA.  Queries, keys and values sit in shared memory as they are stored.  Raw
// scores: warp w takes keys 8w .. 8w + 7 of the tile for all heads, so a thread holds every head's score at
// its four (query, key) places and scales, takes the distance off and mixes in registers; the mixed scores go
// to shared memory as floats.  A warp per (head, query) row then updates maximum and sum and leaves each
// weight in the row's place as two bfloat16 terms (w = hi + lo, 16 bits of mantissa), and the weighted values
// are two products per (head, 32 value columns) task.
// ---------------------------------------------------------------------------
constexpr int kMmaRows = 16;
constexpr int kScoreStride = kKeyTile + 4;            // floats; rows 16 bytes apart in the banks

__device__ __forceinline__ void ldmatrix4(uint32_t (&r)[4], const void* p) {
  const uint32_t at = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(at));
}
__device__ __forceinline__ void ldmatrix4_transposed(uint32_t (&r)[4], const void* p) {
  const uint32_t at = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(at));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&x)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(x[0]), "r"(x[1]), "r"(x[2]), "r"(x[3]), "r"(b0), "r"(b1));
}

// rows j0 .. j0 + 63 of every key/value head as stored: tile[(g * 64 + key) * ld + d]; zeros from `count` on
__device__ __forceinline__ void load_tile_bf16(__nv_bfloat16* __restrict__ tile, int ld, const __nv_bfloat16* __restrict__ cache,
                                               int width, int kv_heads, int page_size, int num_pages,
                                               const int* __restrict__ pages, int j0, int count, int* status) {
  const int chunks = width / 8, total = kv_heads * kKeyTile * chunks;
  for (int base = threadIdx.x; base < total; base += 4 * kTiledThreads) {
    uint4 raw[4];
    int at[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = base + e * kTiledThreads;
      raw[e] = make_uint4(0u, 0u, 0u, 0u);
      at[e] = -1;
      if (idx < total) {
        const int row = idx / chunks, c = idx - row * chunks;
        const int g = row / kKeyTile, key = row - g * kKeyTile;
        at[e] = row * ld + c * 8;
        if (key < count) {
          const int j = j0 + key, page = pages[key];
          if (page >= 0 && page < num_pages)
            raw[e] = *(const uint4*)(cache + (((size_t)page * kv_heads + g) * page_size + j % page_size) * width + c * 8);
          else if (c == 0) atomicOr(status, kStatusBadPage);
        }
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (at[e] >= 0) *(uint4*)(tile + at[e]) = raw[e];
  }
}

template <int VB, int MINB>
__global__ void __launch_bounds__(kTiledThreads, MINB) paged_attention_mixed_mma_kernel(const __grid_constant__ MixedTiledArgs a) {
  constexpr int NT = (kHP * VB + kTiledWarps - 1) / kTiledWarps;      // (head, 32 value columns) tasks a warp may hold
  extern __shared__ float4 smem4[];
  const int heads = a.heads, dim = a.dim, vdim = a.vdim, kv_heads = a.kv_heads;
  const int per = heads / kv_heads;
  const int ldq = dim + 8, ldv = vdim + 8;
  __nv_bfloat16* qs = (__nv_bfloat16*)smem4;                          // [heads * 16, ldq]
  __nv_bfloat16* ks = qs + heads * kMmaRows * ldq;                    // [kv_heads * 64, ldq]
  const bool shared_kv = a.values_shared != 0;
  __nv_bfloat16* vs = shared_kv ? ks : ks + kv_heads * kKeyTile * ldq;      // [kv_heads * 64, ldv]
  float* sc = (float*)(ks + kv_heads * kKeyTile * (shared_kv ? max(ldq, ldv) : ldq + ldv));   // [heads * 16, kScoreStride]
  float* talk_s = sc + heads * kMmaRows * kScoreStride;               // [heads, kHP]
  float* slope_s = talk_s + heads * kHP;                              // [kHP]
  float* top = slope_s + kHP;                                         // [heads * 16]
  float* total = top + heads * kMmaRows;
  float* factor = total + heads * kMmaRows;
  int* pages = (int*)(factor + heads * kMmaRows);                     // [64]

  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gl = lane >> 2, tl = lane & 3;                            // the thread's row and column pair in a fragment
  const int mrow = (lane & 7) + ((lane >> 3) & 1) * 8, mcol = (lane >> 4) * 8;   // its row address for ldmatrix
  const __nv_bfloat16* q = (const __nv_bfloat16*)a.q;
  const bool joins = a.splits > 1;
  for (int i = tid; i < heads * kHP; i += kTiledThreads) {
    const int h = i / kHP, g = i - h * kHP;
    talk_s[i] = g < heads ? (a.talk ? a.talk[h * heads + g] : (h == g ? 1.f : 0.f)) : 0.f;
  }
  for (int g = tid; g < kHP; g += kTiledThreads) slope_s[g] = (a.slopes && g < heads) ? a.slopes[g] : 0.f;
  for (int r = tid; r < heads * kMmaRows; r += kTiledThreads) {
    const bool with_sink = a.sink && !joins;
    top[r] = with_sink ? a.sink[r / kMmaRows] : -INFINITY;
    total[r] = with_sink ? 1.f : 0.f;
  }
  pdl_wait();
  const BlockPlace place = block_place<4>(a);
  if (place.rows <= 0) return;
  const int rows = place.rows, p0 = place.first_position;
  {
    const int chunks = dim / 8;
    for (int idx = tid; idx < heads * kMmaRows * chunks; idx += kTiledThreads) {
      const int r = idx / chunks, c = idx - r * chunks;
      const int h = r / kMmaRows, i = r - h * kMmaRows;
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (i < rows) raw = *(const uint4*)(q + ((size_t)(place.first_token + i) * heads + h) * dim + c * 8);
      *(uint4*)(qs + r * ldq + c * 8) = raw;
    }
  }
  const int hi = p0 + rows - 1;
  const int lo = a.window > 0 ? max(0, p0 - a.window + 1) : 0;
  const int tiles_total = (hi - lo + kKeyTile) / kKeyTile;
  const int tiles_each = (tiles_total + a.splits - 1) / a.splits;
  const int tile_first = blockIdx.y * tiles_each, tile_last = min(tiles_total, tile_first + tiles_each);
  const int* table = a.block_table + (size_t)place.request * a.table_width;

  float acc[NT][4][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[n][b][e] = 0.f;

  if (tid < kKeyTile && tile_first < tile_last) {
    const int j = lo + tile_first * kKeyTile + tid;
    pages[tid] = j <= hi ? table[j / a.page_size] : 0;
  }
  for (int tile = tile_first; tile < tile_last; ++tile) {
    const int j0 = lo + tile * kKeyTile;
    const int count = min(kKeyTile, hi - j0 + 1);
    const int* tile_pages = pages;
    __syncthreads();                                  // the tile before is used up; qs and pages are written
    load_tile_bf16(ks, ldq, (const __nv_bfloat16*)a.k_cache, dim, kv_heads, a.page_size, a.num_pages, tile_pages, j0, count, a.status);
    if (!shared_kv)
      load_tile_bf16(vs, ldv, (const __nv_bfloat16*)a.v_cache, vdim, kv_heads, a.page_size, a.num_pages, tile_pages, j0, count, a.status);
    __syncthreads();
    {
      // ---- raw scores of keys 8 warp .. 8 warp + 7 for every head, then distance, mixing and mask in registers
      float s[kHP][4];
      const int n0 = warp * 8;
#pragma unroll
      for (int h = 0; h < kHP; ++h) {
#pragma unroll
        for (int e = 0; e < 4; ++e) s[h][e] = 0.f;
        if (h < heads) {
          const __nv_bfloat16* krow = ks + ((h / per) * kKeyTile + n0 + gl) * ldq + tl * 2;
          const __nv_bfloat16* qrow = qs + (h * kMmaRows + mrow) * ldq + mcol;
#pragma unroll 4
          for (int d = 0; d < dim; d += 16) {
            uint32_t x[4];
            ldmatrix4(x, qrow + d);
            mma_bf16(s[h], x, *(const uint32_t*)(krow + d), *(const uint32_t*)(krow + d + 8));
          }
        }
      }
      const int key0 = j0 + n0 + tl * 2;
      const int pos0 = p0 + gl, pos1 = p0 + gl + 8;
      const int reach0 = a.window > 0 ? pos0 - a.window : -1, reach1 = a.window > 0 ? pos1 - a.window : -1;
      bool see[4];
      see[0] = gl < rows && key0 <= pos0 && key0 > reach0;
      see[1] = gl < rows && key0 + 1 <= pos0 && key0 + 1 > reach0;
      see[2] = gl + 8 < rows && key0 <= pos1 && key0 > reach1;
      see[3] = gl + 8 < rows && key0 + 1 <= pos1 && key0 + 1 > reach1;
#pragma unroll
      for (int h = 0; h < kHP; ++h) {
        const float slope = slope_s[h];
        s[h][0] = s[h][0] * a.scale - slope * (float)(pos0 - key0);
        s[h][1] = s[h][1] * a.scale - slope * (float)(pos0 - key0 - 1);
        s[h][2] = s[h][2] * a.scale - slope * (float)(pos1 - key0);
        s[h][3] = s[h][3] * a.scale - slope * (float)(pos1 - key0 - 1);
      }
      for (int h = 0; h < heads; ++h) {
        const float4* mix = (const float4*)(talk_s + h * kHP);
        float m[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int g4 = 0; g4 < kHP / 4; ++g4) {
          const float4 w = mix[g4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            m[e] = fmaf(w.x, s[4 * g4][e], m[e]); m[e] = fmaf(w.y, s[4 * g4 + 1][e], m[e]);
            m[e] = fmaf(w.z, s[4 * g4 + 2][e], m[e]); m[e] = fmaf(w.w, s[4 * g4 + 3][e], m[e]);
          }
        }
        float* row0 = sc + (size_t)(h * kMmaRows + gl) * kScoreStride + n0 + tl * 2;
        *(float2*)row0 = make_float2(see[0] ? m[0] : -INFINITY, see[1] ? m[1] : -INFINITY);
        *(float2*)(row0 + 8 * kScoreStride) = make_float2(see[2] ? m[2] : -INFINITY, see[3] ? m[3] : -INFINITY);
      }
    }
    __syncthreads();
    if (shared_kv)                                    // the keys are used up: their place takes the values
      load_tile_bf16(vs, ldv, (const __nv_bfloat16*)a.v_cache, vdim, kv_heads, a.page_size, a.num_pages, tile_pages, j0, count, a.status);
    // ---- running maximum and sum, a warp per (head, query) row, four rows at a time so that their
    // reductions overlap; each weight stays in its row's place as two bfloat16 terms
    for (int r0 = warp; r0 < heads * kMmaRows; r0 += 4 * kTiledWarps) {
      float2 v[4];
      float best[4], sum[4], now[4], before[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = r0 + u * kTiledWarps;
        v[u] = r < heads * kMmaRows ? *(const float2*)(sc + (size_t)r * kScoreStride + 2 * lane) : make_float2(-INFINITY, -INFINITY);
        best[u] = fmaxf(v[u].x, v[u].y);
      }
#pragma unroll
      for (int step = 16; step > 0; step >>= 1)
#pragma unroll
        for (int u = 0; u < 4; ++u) best[u] = fmaxf(best[u], __shfl_xor_sync(0xffffffffu, best[u], step));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = r0 + u * kTiledWarps;
        before[u] = r < heads * kMmaRows ? top[r] : -INFINITY;
        now[u] = fmaxf(before[u], best[u]);
        v[u].x = v[u].x == -INFINITY ? 0.f : expf(v[u].x - now[u]);
        v[u].y = v[u].y == -INFINITY ? 0.f : expf(v[u].y - now[u]);
        sum[u] = v[u].x + v[u].y;
      }
#pragma unroll
      for (int step = 16; step > 0; step >>= 1)
#pragma unroll
        for (int u = 0; u < 4; ++u) sum[u] += __shfl_xor_sync(0xffffffffu, sum[u], step);
      __syncwarp();
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = r0 + u * kTiledWarps;
        if (r >= heads * kMmaRows) continue;
        const __nv_bfloat16 h0 = __float2bfloat16_rn(v[u].x), h1 = __float2bfloat16_rn(v[u].y);
        const __nv_bfloat16 l0 = __float2bfloat16_rn(v[u].x - __bfloat162float(h0));
        const __nv_bfloat16 l1 = __float2bfloat16_rn(v[u].y - __bfloat162float(h1));
        __nv_bfloat162* terms = (__nv_bfloat162*)(sc + (size_t)r * kScoreStride);
        terms[lane] = __halves2bfloat162(h0, h1);
        terms[32 + lane] = __halves2bfloat162(l0, l1);
        if (lane == 0) {
          const float f = before[u] == -INFINITY ? 0.f : expf(before[u] - now[u]);
          factor[r] = f;
          total[r] = fmaf(total[r], f, sum[u]);
          top[r] = now[u];
        }
      }
    }
    __syncthreads();
    if (tid < kKeyTile && tile + 1 < tile_last) {     // this tile's loads are done; the next tile's come after a barrier
      const int j = j0 + kKeyTile + tid;
      pages[tid] = j <= hi ? table[j / a.page_size] : 0;
    }
    // ---- weighted values
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      const int task = n * kTiledWarps + warp;
      if (task >= heads * VB) continue;
      const int h = task / VB, vb = task - h * VB;
      const float f0 = factor[h * kMmaRows + gl], f1 = factor[h * kMmaRows + gl + 8];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        acc[n][b][0] *= f0; acc[n][b][1] *= f0; acc[n][b][2] *= f1; acc[n][b][3] *= f1;
      }
      const __nv_bfloat16* weights = (const __nv_bfloat16*)(sc + (size_t)(h * kMmaRows + mrow) * kScoreStride) + mcol;
      const __nv_bfloat16* values = vs + ((h / per) * kKeyTile + mrow) * ldv + vb * 32 + mcol;
#pragma unroll
      for (int k0 = 0; k0 < kKeyTile; k0 += 16) {
        uint32_t whi[4], wlo[4];
        ldmatrix4(whi, weights + k0);
        ldmatrix4(wlo, weights + kKeyTile + k0);
#pragma unroll
        for (int pair = 0; pair < 2; ++pair) {
          const int col = vb * 32 + pair * 16;
          if (col >= vdim) continue;
          uint32_t y[4];
          ldmatrix4_transposed(y, values + (size_t)k0 * ldv + pair * 16);
          mma_bf16(acc[n][2 * pair], whi, y[0], y[1]);
          mma_bf16(acc[n][2 * pair], wlo, y[0], y[1]);
          if (col + 8 < vdim) {
            mma_bf16(acc[n][2 * pair + 1], whi, y[2], y[3]);
            mma_bf16(acc[n][2 * pair + 1], wlo, y[2], y[3]);
          }
        }
      }
    }
  }
  __syncthreads();
  const int outs = heads * vdim;
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int task = n * kTiledWarps + warp;
    if (task >= heads * VB) continue;
    const int h = task / VB, vb = task - h * VB;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int i = gl + 8 * half;
      if (i >= rows) continue;
      const int r = h * kMmaRows + i;
      const size_t t = (size_t)place.first_token + i;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int d = vb * 32 + b * 8 + tl * 2;
        if (d >= vdim) continue;
        const float o0 = acc[n][b][2 * half], o1 = acc[n][b][2 * half + 1];
        if (joins) {
          *(float2*)(a.part_acc + ((size_t)blockIdx.y * a.num_tokens + t) * outs + h * vdim + d) = make_float2(o0, o1);
        } else {
          const float inv = a.out_scale / total[r];
          *(__nv_bfloat162*)((__nv_bfloat16*)a.out + t * outs + h * vdim + d) = __floats2bfloat162_rn(o0 * inv, o1 * inv);
        }
      }
      if (joins && vb == 0 && tl == 0) {
        float* ml = a.part_ml + (((size_t)blockIdx.y * a.num_tokens + t) * heads + h) * 2;
        ml[0] = top[r];
        ml[1] = total[r];
      }
    }
  }
}
#endif  // HEADS_PAD <= 16

// out[t, h, :] = out_scale * sum_s acc_s exp(m_s - M) / (exp(sink_h - M) + sum_s l_s exp(m_s - M)) with M the
// largest of the splits' maxima and the sink, splits in order.  The same blocks as the kernel above.
template <typename T, int QI>
__global__ void __launch_bounds__(kTiledThreads) mixed_join_kernel(const __grid_constant__ MixedTiledArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const BlockPlace place = block_place<QI>(a);
  if (place.rows <= 0) return;
  const int outs = a.heads * a.vdim;
  constexpr int kBatch = 8;                           // loads in flight before they are used
  const int idx = blockIdx.y * kTiledThreads + threadIdx.x;
  if (idx >= place.rows * outs) return;
  const int i = idx / outs, o = idx - i * outs;
  const int h = o / a.vdim;
  const size_t t = (size_t)place.first_token + i;
  const size_t ml_step = (size_t)a.num_tokens * a.heads * 2, acc_step = (size_t)a.num_tokens * outs;
  const float* ml = a.part_ml + (t * a.heads + h) * 2;
  const float* part = a.part_acc + t * outs + o;
  float best = a.sink ? a.sink[h] : -INFINITY;
  for (int s0 = 0; s0 < a.splits; s0 += kBatch) {
    float m[kBatch];
#pragma unroll
    for (int e = 0; e < kBatch; ++e) m[e] = s0 + e < a.splits ? ml[(s0 + e) * ml_step] : -INFINITY;
#pragma unroll
    for (int e = 0; e < kBatch; ++e) best = fmaxf(best, m[e]);
  }
  float sum = a.sink ? expf(a.sink[h] - best) : 0.f;
  float value = 0.f;
  for (int s0 = 0; s0 < a.splits; s0 += kBatch) {
    float m[kBatch], l[kBatch], v[kBatch];
#pragma unroll
    for (int e = 0; e < kBatch; ++e) {
      const bool in = s0 + e < a.splits;
      m[e] = in ? ml[(s0 + e) * ml_step] : -INFINITY;
      l[e] = in ? ml[(s0 + e) * ml_step + 1] : 0.f;
      v[e] = in ? part[(s0 + e) * acc_step] : 0.f;
    }
#pragma unroll
    for (int e = 0; e < kBatch; ++e) {
      const float w = m[e] == -INFINITY ? 0.f : expf(m[e] - best);
      sum = fmaf(l[e], w, sum);
      value = fmaf(v[e], w, value);
    }
  }
  ((T*)a.out)[t * outs + o] = from_float<T>(value / sum * a.out_scale);
}

}  // namespace einf

using namespace einf;

static size_t tiled_bytes(int heads, int dim, int vdim, int rows, int groups) {
  const size_t floats = (size_t)heads * rows * dim + (size_t)groups * kKeyTile * (dim + 4 > vdim ? dim + 4 : vdim) +
                        (size_t)heads * rows * kKeyTile + (size_t)heads * kHP + kHP + 3 * (size_t)heads * rows +
                        2 * kKeyTile;
  return floats * sizeof(float);
}

struct TiledShape {
  int rows, groups;
};

// Queries a CTA takes and key/value heads it holds at once.  Tasks of four queries: the most rows of 16, 8, 4
// whose tasks fit a warp's registers, with all key/value heads at once or else one, that leaves room for two
// CTAs an SM; else the most that fits at all.  rows 0: none does.
static TiledShape tiled_shape(int heads, int kv_heads, int dim, int vdim, int single) {
  const size_t limits[2] = {(size_t)112 * 1024, (size_t)220 * 1024};
  const int value_lanes = (vdim + 31) / 32;
  const int tasks = kTiledWarps * (16 / (value_lanes <= 1 ? 1 : value_lanes <= 2 ? 2 : 4));
  for (size_t limit : limits)
    for (int rows : {16, 8, 4}) {
      if (single) rows = 1;
      for (int groups : {kv_heads, 1})
        if ((single || heads * (rows / 4) <= tasks) && tiled_bytes(heads, dim, vdim, rows, groups) <= limit)
          return {rows, groups};
    }
  return {0, 0};
}

static size_t mma_bytes(int heads, int kv_heads, int dim, int vdim, bool values_shared) {
  const int both = values_shared ? (dim > vdim ? dim + 8 : vdim + 8) : dim + 8 + vdim + 8;
  return (size_t)(heads * 16 * (dim + 8) + kv_heads * kKeyTile * both) * 2 +
         (size_t)(heads * 16 * (kKeyTile + 4) + heads * kHP + kHP + 3 * heads * 16 + kKeyTile) * sizeof(float);
}

// How the tensor-core kernel runs for these sizes: two CTAs an SM where the shared memory of two fits (with
// the values in a place of their own if that fits too, else in the keys' place), else one.  ctas 0: it does not fit.
struct MmaMode {
  int ctas, values_shared;
};
static MmaMode mma_mode(int heads, int kv_heads, int dim, int vdim) {
  const size_t half = (size_t)(228 - 2) * 1024 / 2, whole = (size_t)220 * 1024;
  if (mma_bytes(heads, kv_heads, dim, vdim, false) <= half) return {2, 0};
  if (mma_bytes(heads, kv_heads, dim, vdim, true) <= half) return {2, 1};
  if (mma_bytes(heads, kv_heads, dim, vdim, false) <= whole) return {1, 0};
  if (mma_bytes(heads, kv_heads, dim, vdim, true) <= whole) return {1, 1};
  return {0, 0};
}

// The tensor-core kernel takes bfloat16 prompt portions of up to 16 heads whose sizes fit its fragments.
static bool mma_takes(int dtype, int heads, int kv_heads, int dim, int vdim) {
  return kHP <= 16 && dtype == kBFloat16 && dim % 16 == 0 && vdim % 8 == 0 && vdim <= 128 &&
         mma_mode(heads, kv_heads, dim, vdim).ctas > 0;
}

#if HEADS_PAD <= 16
template <int VB, int MINB>
static int launch_mma_as(MixedTiledArgs a, int blocks, int values_shared, cudaStream_t stream) {
  auto kernel = paged_attention_mixed_mma_kernel<VB, MINB>;
  a.values_shared = values_shared;
  const size_t bytes = mma_bytes(a.heads, a.kv_heads, a.dim, a.vdim, values_shared != 0);
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
  }
  cudaError_t e = launch_pdl(kernel, dim3(blocks, a.splits), kTiledThreads, bytes, stream, a);
  if (e != cudaSuccess || a.splits == 1) return (int)e;
  return (int)launch_pdl(mixed_join_kernel<__nv_bfloat16, 4>, dim3(blocks, (a.rows * a.heads * a.vdim + kTiledThreads - 1) / kTiledThreads),
                         kTiledThreads, 0, stream, a);
}

template <int VB>
static int launch_mma(const MixedTiledArgs& a, int blocks, cudaStream_t stream) {
  const MmaMode mode = mma_mode(a.heads, a.kv_heads, a.dim, a.vdim);
  if (mode.ctas == 2) return launch_mma_as<VB, 2>(a, blocks, mode.values_shared, stream);
  return launch_mma_as<VB, 1>(a, blocks, mode.values_shared, stream);
}
#endif

template <typename T, int QI, int VD>
static int launch_tiled(const MixedTiledArgs& a, int blocks, cudaStream_t stream) {
  auto kernel = paged_attention_mixed_tiled_kernel<T, QI, VD>;
  const size_t bytes = tiled_bytes(a.heads, a.dim, a.vdim, a.rows, a.groups_at_once);
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
  }
  cudaError_t e = launch_pdl(kernel, dim3(blocks, a.splits), kTiledThreads, bytes, stream, a);
  if (e != cudaSuccess || a.splits == 1) return (int)e;
  return (int)launch_pdl(mixed_join_kernel<T, QI>, dim3(blocks, (a.rows * a.heads * a.vdim + kTiledThreads - 1) / kTiledThreads),
                         kTiledThreads, 0, stream, a);
}

// Rows per CTA for the given sizes (0: this kernel does not take them; 1 with `single`).
extern "C" int einf_paged_attention_mixed_tiled_rows(int heads, int kv_heads, int dim, int vdim, int single, int dtype) {
  if (heads <= 0 || heads > kHP || kv_heads <= 0 || heads % kv_heads || dim <= 0 || dim % 4 || vdim <= 0 || vdim > 128)
    return 0;
  if (!single && mma_takes(dtype, heads, kv_heads, dim, vdim)) return 16;
  return tiled_shape(heads, kv_heads, dim, vdim, single).rows;
}

// CTAs of the tensor-core kernel that share an SM for these sizes (0: it does not take them).
extern "C" int einf_paged_attention_mixed_mma_ctas(int heads, int kv_heads, int dim, int vdim, int dtype) {
  if (heads <= 0 || heads > kHP || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0) return 0;
  return mma_takes(dtype, heads, kv_heads, dim, vdim) ? mma_mode(heads, kv_heads, dim, vdim).ctas : 0;
}

// `items`: q_tiles [num_items, 4] with single == 0; token indices [num_items] (or null: tokens 0 .. num_items - 1)
// with single != 0.  `splits` > 1 needs part_acc [splits, num_tokens, heads * vdim] and part_ml [splits, num_tokens, heads, 2].
extern "C" int einf_paged_attention_mixed_tiled(const void* q, const void* k_cache, const void* v_cache, int dtype,
                                                const int* block_table, int table_width, const int* seq_of_token,
                                                const int* positions, const int* items, int num_items, int single,
                                                void* out, int num_tokens, int heads, int kv_heads, int dim, int vdim,
                                                int page_size, int num_pages, float scale, int window,
                                                const float* slopes, const float* talk, const float* sink,
                                                float out_scale, int splits, float* part_acc, float* part_ml,
                                                int* status, cudaStream_t stream) {
  if (num_items == 0) return 0;
  const int rows = einf_paged_attention_mixed_tiled_rows(heads, kv_heads, dim, vdim, single, dtype);
  if (rows == 0 || splits < 1 || splits > 65535 ||
      (splits > 1 && (!part_acc || !part_ml)))
    return (int)cudaErrorInvalidValue;
  MixedTiledArgs a;
  a.q = q; a.k_cache = k_cache; a.v_cache = v_cache; a.block_table = block_table; a.table_width = table_width;
  a.seq_of_token = seq_of_token; a.positions = positions;
  a.q_tiles = single ? nullptr : items; a.single_tokens = single ? items : nullptr;
  a.out = out; a.heads = heads; a.kv_heads = kv_heads; a.dim = dim; a.vdim = vdim; a.page_size = page_size;
  a.num_pages = num_pages; a.scale = scale; a.window = window; a.slopes = slopes; a.talk = talk; a.sink = sink;
  a.groups_at_once = tiled_shape(heads, kv_heads, dim, vdim, single).groups;
  a.values_shared = 0;
  a.out_scale = out_scale; a.rows = rows; a.blocks_per_tile = single ? 1 : (128 + rows - 1) / rows; a.splits = splits;
  a.part_acc = part_acc; a.part_ml = part_ml; a.num_tokens = num_tokens; a.status = status;
  const int blocks = num_items * a.blocks_per_tile;
  const int value_lanes = (vdim + 31) / 32;
#if HEADS_PAD <= 16
  if (!single && mma_takes(dtype, heads, kv_heads, dim, vdim)) {
    if (value_lanes <= 1) return launch_mma<1>(a, blocks, stream);
    if (value_lanes <= 2) return launch_mma<2>(a, blocks, stream);
    if (value_lanes <= 3) return launch_mma<3>(a, blocks, stream);
    return launch_mma<4>(a, blocks, stream);
  }
#endif
#define EINF_TILED(QI, VD) EINF_DISPATCH_2(dtype, T, { return launch_tiled<T, QI, VD>(a, blocks, stream); })
  if (single) {
    if (value_lanes <= 1) EINF_TILED(1, 1)
    if (value_lanes <= 2) EINF_TILED(1, 2)
    EINF_TILED(1, 4)
  }
  if (value_lanes <= 1) EINF_TILED(4, 1)
  if (value_lanes <= 2) EINF_TILED(4, 2)
  EINF_TILED(4, 4)
#undef EINF_TILED
}
