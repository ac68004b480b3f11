// Mixers that carry a state of fixed size per request instead of keys and values: a linear
// recurrence over outer products (linear attention with a decay per head; the state-space
// recurrence of Mamba-2 in its recurrent form), the short causal convolution in front of it, and
// the gated norm behind it.  State lives in 32-bit floats in a slot per request
// (state[slot * row_stride + ...]); a request without a slot (-1: padding of a decode graph) reads
// zeros and writes nothing.  The step's tokens are packed request by request, q_start[r] ..
// q_start[r + 1], so a prompt portion and a single decoded token take the same code and the same
// order of additions: what a position computes does not depend on how the prompt was cut.
#include <type_traits>

#include "common.cuh"

namespace einf {

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// ---------------------------------------------------------------------------
// Causal convolution per channel over the tokens of each request, bias, SiLU:
//   out[t, c] = silu(bias[c] + sum_j w[c, j] * in[t - (taps - 1) + j, c]),  j = 0 .. taps-1,
// where inputs before the portion come from the request's convolution state (its last taps-1
// inputs, oldest first, [taps-1, channels] floats; zeros after a fresh start).  `act` 0 leaves the
// SiLU out; with `input_bias` the convolution's input is in + input_bias[c] (a projection's bias
// that is added here instead of by a launch of its own; the state holds the sum).  The same launch
// turns the raw step sizes of `heads` further columns into
//   dt = softplus(raw + dt_bias[h])   and   decay = exp(-exp(a_log[h]) * dt)
// in 32-bit (columns channels .. channels+heads of the work; `in` holds them at dt_offset).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void conv_silu_kernel(const T* __restrict__ in, long long in_stride, const float* __restrict__ weight,
                                 const float* __restrict__ bias, const float* __restrict__ conv_state,
                                 long long state_stride, const int* __restrict__ seq_of_token,
                                 const int* __restrict__ q_start, const int* __restrict__ state_slots, int num_slots,
                                 T* __restrict__ out, int channels, int taps, int num_tokens,
                                 const T* __restrict__ dt_in, const float* __restrict__ dt_bias,
                                 const float* __restrict__ a_log, float* __restrict__ dt_out,
                                 float* __restrict__ decay_out, int heads, int act,
                                 const float* __restrict__ input_bias) {
  pdl_launch_dependents();
  pdl_wait();
  const int columns = channels + heads;
  const long long total = (long long)num_tokens * columns;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / columns);
    const int c = (int)(idx - (long long)t * columns);
    if (c >= channels) {
      const int h = c - channels;
      const float dt = softplus_f(to_float(dt_in[(long long)t * in_stride + h]) + dt_bias[h]);
      dt_out[(long long)t * heads + h] = dt;
      decay_out[(long long)t * heads + h] = expf(-expf(a_log[h]) * dt);
      continue;
    }
    const int r = seq_of_token[t];
    const int first = q_start[r];
    const int slot = state_slots[r];
    const float* state = (slot >= 0 && slot < num_slots) ? conv_state + (long long)slot * state_stride : nullptr;
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int u = t - (taps - 1) + j;       // packed index of the input, if it is in this step
      float v;
      if (u >= first) v = to_float(in[(long long)u * in_stride + c]) + (input_bias ? input_bias[c] : 0.f);
      else v = state ? state[(long long)(taps - 1 - (first - u)) * channels + c] : 0.f;
      acc = fmaf(weight[(long long)c * taps + j], v, acc);
    }
    out[(long long)t * channels + c] = from_float<T>(act ? silu_f(acc) : acc);
  }
}

// After the convolution: the request's last taps-1 inputs become its convolution state (a portion
// shorter than that keeps the tail of the old state in front).  One thread per (request, channel).
constexpr int kMaxTaps = 16;
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ in, long long in_stride, float* __restrict__ conv_state,
                                         long long state_stride, const int* __restrict__ q_start,
                                         const int* __restrict__ state_slots, int num_slots, int channels, int taps,
                                         const float* __restrict__ input_bias) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int slot = state_slots[r];
  if (c >= channels || slot < 0 || slot >= num_slots) return;
  const int first = q_start[r], count = q_start[r + 1] - first;
  float* state = conv_state + (long long)slot * state_stride;
  const int keep = taps - 1;
  float fresh[kMaxTaps];
#pragma unroll
  for (int u = 0; u < kMaxTaps; ++u) {
    if (u < keep) {
      const int rel = count - keep + u;      // index among the step's tokens of this request
      fresh[u] = rel >= 0 ? to_float(in[(long long)(first + rel) * in_stride + c]) + (input_bias ? input_bias[c] : 0.f)
                          : state[(long long)(u + count) * channels + c];
    }
  }
#pragma unroll
  for (int u = 0; u < kMaxTaps; ++u)
    if (u < keep) state[(long long)u * channels + c] = fresh[u];
}

// ---------------------------------------------------------------------------
// The recurrence.  Per request and head, with S a [dim, vdim] matrix of floats:
//   S <- a_t S + k_t (s_t v_t)^T,      y_t = S^T q_t + skip_h v_t
// a_t is a constant per head (head_decay) or a value per token and head (token_decay), s_t a
// value per token and head (token_scale) or 1; query and key head of head h is h / (heads /
// groups).  With `act` the inputs pass SiLU as they are read.  q, k, v are rows of some wider
// matrix: element (t, head, i) of q is q[t * q_stride + head * dim + i].
//
// A thread owns ROWS consecutive rows of one column of S; the 2^n lanes that share a column
// (lanes_per_column = dim_pad / ROWS) sit columns_per_warp apart in a warp, so that loads and
// stores of S are contiguous over the columns, and add their parts of y with shuffles.  The CTA
// brings the inputs of a batch of tokens into shared memory as floats, activated once (every
// column needs the same k_t and q_t), while it works on the batch before; tokens are then taken
// one after the other.
//
// A long portion is cut into segments of `segment_len` tokens that run side by side (a single
// request's prompt would otherwise keep a few warps busy, each waiting on itself): a first pass
// adds up every segment's own contribution B from a zero state together with the product P of
// its decays, a small kernel walks the segments (S_start of the next = P S_start + B) and writes
// the request's final state, and the emitting pass runs every segment from its start state.
// Portions of up to segment_len tokens (decoding among them) take the emitting pass alone, which
// then reads and writes the slot itself.
// ---------------------------------------------------------------------------
// Stores into the staging buffers by the shared-memory instruction itself.
__device__ __forceinline__ void sts32(uint32_t address, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(address), "f"(v) : "memory");
}

constexpr int kRecurrenceThreads = 128;
constexpr int kStageKQ = 8;      // k (and q) elements a thread stages per batch: batch * dim <= 8 * 128
constexpr int kStageV = 4;       // v elements a thread stages per batch: batch * columns of the CTA <= 4 * 128
constexpr int kMaxBatch = 16;

struct RecurrenceArgs {
  const void* q; const void* k; const void* v;
  long long q_stride, k_stride, v_stride;
  const float* head_decay; const float* token_decay; const float* token_scale; const float* skip;
  float* state; long long state_stride;
  const int* q_start; const int* state_slots;
  float* y;
  int y_splits;              // the streaming kernel alone: CTAs that share a head's rows, each leaving its part of y
  long long y_split_stride;  // floats between two parts of y
  float* segment_state;    // [requests * segments, heads, dim, vdim]: B after the first pass, start states after the walk
  float* segment_decay;    // [requests * segments, heads]
  int num_slots, heads, groups, dim, vdim, act, lanes_per_column, dim_pad, batch, segments, segment_len;
};

// kEmit false: the first pass (no queries, no output, state from zero into segment_state).
// COLS columns of the state per thread (COLS * ROWS registers of S): with two, the k and q a thread
// reads from shared memory for a token serve twice as many state elements.
template <typename T, int ROWS, int COLS, bool kEmit>
__global__ void __launch_bounds__(kRecurrenceThreads, COLS == 1 ? 4 : 3)
linear_recurrence_kernel(const __grid_constant__ RecurrenceArgs a) {
  extern __shared__ __align__(16) float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int lanes = a.lanes_per_column;          // a power of two, 1 .. 32
  const int columns_per_warp = 32 / lanes;
  const int thread_columns = (kRecurrenceThreads / 32) * columns_per_warp;   // columns side by side over the threads
  const int columns_per_block = COLS * thread_columns;                        // thread c-th column: + c * thread_columns
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int part = lane / columns_per_warp;       // which rows of the column
  const int local_column = warp * columns_per_warp + (lane % columns_per_warp);
  const int column0 = blockIdx.x * columns_per_block;
  const int head = blockIdx.y;
  const int r = blockIdx.z / a.segments, segment = blockIdx.z - r * a.segments;
  const int group = head / (a.heads / a.groups);
  const int request_first = a.q_start[r], request_last = a.q_start[r + 1];
  const int count = request_last - request_first;
  const int num_segments = (count + a.segment_len - 1) / a.segment_len;
  if (segment >= num_segments || (!kEmit && num_segments <= 1)) return;
  const int first = request_first + segment * a.segment_len;
  const int last = min(request_last, first + a.segment_len);
  const int slot = a.state_slots[r];
  bool live[COLS];
  int col[COLS];
#pragma unroll
  for (int c = 0; c < COLS; ++c) {
    live[c] = column0 + c * thread_columns + local_column < a.vdim;
    col[c] = live[c] ? column0 + c * thread_columns + local_column : a.vdim - 1;   // idle lanes follow along and write nothing
  }
  const int r0 = part * ROWS;
  const int dim = a.dim, dim_pad = a.dim_pad, batch = a.batch;

  // shared memory: two buffers of [k: batch x dim_pad | q: batch x dim_pad | v: batch x columns | a: batch | s: batch]
  const int kq_floats = batch * dim_pad;
  const int buffer_floats = ((kEmit ? 2 : 1) * kq_floats + batch * columns_per_block + 2 * batch + 3) & ~3;
  for (int i = threadIdx.x; i < 2 * buffer_floats; i += kRecurrenceThreads) smem[i] = 0.f;   // rows beyond dim stay zero

  const float* start_state = nullptr;
  float* end_state = nullptr;
  const long long in_head = ((long long)head * dim) * a.vdim;
  if (kEmit) {
    if (num_segments == 1) {
      if (slot >= 0 && slot < a.num_slots) start_state = a.state + (long long)slot * a.state_stride + in_head;
    } else {
      // the walk over the segments left every segment's start state there (the first one's too:
      // the slot itself already holds the request's final state)
      start_state = a.segment_state + ((long long)blockIdx.z * a.heads * dim) * a.vdim + in_head;
    }
    if (num_segments == 1 && slot >= 0 && slot < a.num_slots) end_state = a.state + (long long)slot * a.state_stride + in_head;
  } else {
    end_state = a.segment_state + ((long long)blockIdx.z * a.heads * dim) * a.vdim + in_head;
  }
  float S[COLS][ROWS];
#pragma unroll
  for (int c = 0; c < COLS; ++c)
#pragma unroll
    for (int i = 0; i < ROWS; ++i)
      S[c][i] = (start_state && r0 + i < dim) ? start_state[(long long)(r0 + i) * a.vdim + col[c]] : 0.f;

  const T* qg = (const T*)a.q + (long long)group * dim;
  const T* kg = (const T*)a.k + (long long)group * dim;
  const T* vg = (const T*)a.v + (long long)head * a.vdim + column0;
  const float constant_decay = a.head_decay ? a.head_decay[head] : 1.f;
  const float skip = a.skip ? a.skip[head] : 0.f;
  const bool act = a.act != 0;
  const long long k_stride = a.k_stride, q_stride = a.q_stride, v_stride = a.v_stride;
  const float* token_decay = a.token_decay;
  const float* token_scale = a.token_scale;
  const int heads = a.heads;

  // What this thread stages of a batch: element idx = threadIdx.x + j * 128 of [batch x dim] (k and q) and of
  // [batch x columns] (v); token and index inside the token, packed, -1 for none.
  int kq_where[kStageKQ], v_where[kStageV];
#pragma unroll
  for (int j = 0; j < kStageKQ; ++j) {
    const int idx = threadIdx.x + j * kRecurrenceThreads;
    const int tt = idx / dim;
    kq_where[j] = tt < batch ? (tt << 16) | (idx - tt * dim) : -1;
  }
#pragma unroll
  for (int j = 0; j < kStageV; ++j) {
    const int idx = threadIdx.x + j * kRecurrenceThreads;
    const int tt = idx / columns_per_block;
    const int c = idx - tt * columns_per_block;
    v_where[j] = (tt < batch && column0 + c < a.vdim) ? (tt << 16) | c : -1;
  }
  // staged as they come (converted when they are put into shared memory: a conversion right behind
  // its load would make the warp wait for the load before it starts on the batch at hand)
  T k_regs[kStageKQ], q_regs[kStageKQ], v_regs[kStageV];
  float a_reg = constant_decay, s_reg = 1.f;
  const T zero = from_float<T>(0.f);
  auto fetch = [&](int t0) {
    const int n = min(batch, last - t0);
#pragma unroll
    for (int j = 0; j < kStageKQ; ++j) {
      const int tt = kq_where[j] >> 16, i = kq_where[j] & 0xffff;
      const bool valid = kq_where[j] >= 0 && tt < n;
      k_regs[j] = valid ? kg[(long long)(t0 + tt) * k_stride + i] : zero;
      if (kEmit) q_regs[j] = valid ? qg[(long long)(t0 + tt) * q_stride + i] : zero;
    }
#pragma unroll
    for (int j = 0; j < kStageV; ++j) {
      const int tt = v_where[j] >> 16, c = v_where[j] & 0xffff;
      v_regs[j] = (v_where[j] >= 0 && tt < n) ? vg[(long long)(t0 + tt) * v_stride + c] : zero;
    }
    if (threadIdx.x < n) {
      if (token_decay) a_reg = token_decay[(long long)(t0 + threadIdx.x) * heads + head];
      if (token_scale) s_reg = token_scale[(long long)(t0 + threadIdx.x) * heads + head];
    }
  };
  const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int v_offset = (kEmit ? 2 : 1) * kq_floats;             // floats from a buffer's start
  const int a_offset = v_offset + batch * columns_per_block;
  auto stash = [&](uint32_t buffer) {                           // buffer: shared address of the buffer's start
#pragma unroll
    for (int j = 0; j < kStageKQ; ++j) {
      if (kq_where[j] < 0) continue;
      const uint32_t at = buffer + 4u * ((kq_where[j] >> 16) * dim_pad + (kq_where[j] & 0xffff));
      sts32(at, act ? silu_f(to_float(k_regs[j])) : to_float(k_regs[j]));
      if (kEmit) sts32(at + 4u * kq_floats, act ? silu_f(to_float(q_regs[j])) : to_float(q_regs[j]));
    }
#pragma unroll
    for (int j = 0; j < kStageV; ++j) {
      if (v_where[j] < 0) continue;
      sts32(buffer + 4u * (v_offset + (v_where[j] >> 16) * columns_per_block + (v_where[j] & 0xffff)),
            act ? silu_f(to_float(v_regs[j])) : to_float(v_regs[j]));
    }
    if (threadIdx.x < batch) {
      sts32(buffer + 4u * (a_offset + threadIdx.x), a_reg);
      sts32(buffer + 4u * (a_offset + batch + threadIdx.x), s_reg);
    }
  };

  __syncthreads();                 // the zeros are in place
  fetch(first);
  stash(smem_base);
  __syncthreads();
  float decay_product = 1.f;
  int turn = 0;
  float* y_out = a.y + ((long long)first * a.heads + head) * a.vdim;
  const long long y_step = (long long)a.heads * a.vdim;
  for (int t0 = first; t0 < last; t0 += batch, turn ^= 1) {
    const bool more = t0 + batch < last;
    if (more) fetch(t0 + batch);   // on its way while this batch is added
    const float* bf = smem + turn * buffer_floats;
    const float* kb = bf + r0;
    const float* qb = kb + kq_floats;
    const float* vb = bf + v_offset + local_column;
    const float* ab = bf + a_offset;
    const int n = min(batch, last - t0);
    // kTokens tokens in a row: the state is updated token after token, the lanes' parts of the kTokens
    // outputs are added across the lanes together (shuffles of different tokens overlap).
    auto tokens = [&](int tt, auto count_tag) {
      constexpr int kTokens = decltype(count_tag)::value;
      float yp[COLS][kTokens], vcs[COLS][kTokens];
#pragma unroll
      for (int u = 0; u < kTokens; ++u) {
        const float ac = ab[tt + u], scale = ab[batch + tt + u];
        const float4* k4 = reinterpret_cast<const float4*>(kb + (tt + u) * dim_pad);
        const float4* q4 = reinterpret_cast<const float4*>(qb + (tt + u) * dim_pad);
        float4 kc[ROWS / 4], qc[ROWS / 4];
#pragma unroll
        for (int i = 0; i < ROWS / 4; ++i) {
          kc[i] = k4[i];
          if (kEmit) qc[i] = q4[i];
        }
#pragma unroll
        for (int c = 0; c < COLS; ++c) {
          const float vc = vb[(tt + u) * columns_per_block + c * thread_columns];
          const float sv = scale * vc;
          float y4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int i = 0; i < ROWS / 4; ++i) {
            S[c][4 * i + 0] = fmaf(ac, S[c][4 * i + 0], kc[i].x * sv);
            S[c][4 * i + 1] = fmaf(ac, S[c][4 * i + 1], kc[i].y * sv);
            S[c][4 * i + 2] = fmaf(ac, S[c][4 * i + 2], kc[i].z * sv);
            S[c][4 * i + 3] = fmaf(ac, S[c][4 * i + 3], kc[i].w * sv);
            if (kEmit) {
              y4[0] = fmaf(S[c][4 * i + 0], qc[i].x, y4[0]);
              y4[1] = fmaf(S[c][4 * i + 1], qc[i].y, y4[1]);
              y4[2] = fmaf(S[c][4 * i + 2], qc[i].z, y4[2]);
              y4[3] = fmaf(S[c][4 * i + 3], qc[i].w, y4[3]);
            }
          }
          yp[c][u] = (y4[0] + y4[1]) + (y4[2] + y4[3]);
          vcs[c][u] = vc;
        }
        if (!kEmit) decay_product *= ac;
      }
      if (kEmit) {
        for (int o = columns_per_warp; o < 32; o <<= 1) {
#pragma unroll
          for (int c = 0; c < COLS; ++c)
#pragma unroll
            for (int u = 0; u < kTokens; ++u) yp[c][u] += __shfl_xor_sync(0xffffffffu, yp[c][u], o);
        }
        if (part == 0) {
#pragma unroll
          for (int c = 0; c < COLS; ++c)
            if (live[c]) {
#pragma unroll
              for (int u = 0; u < kTokens; ++u) y_out[u * y_step + col[c]] = yp[c][u] + skip * vcs[c][u];
            }
        }
        y_out += kTokens * y_step;
      }
    };
    int tt = 0;
    for (; tt + 4 <= n; tt += 4) tokens(tt, std::integral_constant<int, 4>{});
    for (; tt < n; ++tt) tokens(tt, std::integral_constant<int, 1>{});
    if (more) stash(smem_base + 4u * ((turn ^ 1) * buffer_floats));
    __syncthreads();
  }
  if (end_state) {
#pragma unroll
    for (int c = 0; c < COLS; ++c)
      if (live[c]) {
#pragma unroll
        for (int i = 0; i < ROWS; ++i)
          if (r0 + i < dim) end_state[(long long)(r0 + i) * a.vdim + col[c]] = S[c][i];
      }
  }
  if (!kEmit && blockIdx.x == 0 && threadIdx.x == 0) a.segment_decay[(long long)blockIdx.z * a.heads + head] = decay_product;
}

// Between the two passes: walk a request's segments, S_start(next) = P S_start + B, leave every
// segment's start state where its B was, and write the request's final state into its slot.
__global__ void recurrence_walk_kernel(const __grid_constant__ RecurrenceArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int head = blockIdx.y, r = blockIdx.z;
  const int count = a.q_start[r + 1] - a.q_start[r];
  const int num_segments = (count + a.segment_len - 1) / a.segment_len;
  if (num_segments <= 1) return;
  const int slot = a.state_slots[r];
  const long long per_head = (long long)a.dim * a.vdim;
  float* slot_state = (slot >= 0 && slot < a.num_slots) ? a.state + (long long)slot * a.state_stride + head * per_head : nullptr;
  constexpr int kAtOnce = 16;      // segments whose B and P are in registers before the chain of products starts
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < per_head; e += (long long)gridDim.x * blockDim.x) {
    float current = slot_state ? slot_state[e] : 0.f;
    for (int base = 0; base < num_segments; base += kAtOnce) {
      float b[kAtOnce], p[kAtOnce];
#pragma unroll
      for (int u = 0; u < kAtOnce; ++u) {
        const long long index = (long long)r * a.segments + min(base + u, num_segments - 1);
        b[u] = a.segment_state[(index * a.heads + head) * per_head + e];
        p[u] = a.segment_decay[index * a.heads + head];
      }
#pragma unroll
      for (int u = 0; u < kAtOnce; ++u) {
        if (base + u >= num_segments) break;
        const long long index = (long long)r * a.segments + base + u;
        a.segment_state[(index * a.heads + head) * per_head + e] = current;
        current = fmaf(p[u], current, b[u]);
      }
    }
    if (slot_state) slot_state[e] = current;
  }
}

// One token per request (a decode step): the state is streamed through once, four columns a
// thread with 16-byte loads and stores along the rows, S <- a S + k (s v)^T and the thread's part of
// y = S^T q in the same pass; the row groups' parts of y meet in shared memory.  vdim / 4 is at most
// the 128 threads (the launcher sends other sizes to the kernel above); where it does not divide
// them, the threads beyond the last whole row group sit the pass out.  With y_splits > 1 that many
// CTAs (grid z) share a head's rows, a run of rows each, and leave their parts of y one after the
// other (y_split_stride floats apart) for the consumer to add up: a few requests with few large
// heads would otherwise be a few CTAs.
template <typename T>
__global__ void __launch_bounds__(kRecurrenceThreads)
recurrence_step_kernel(const __grid_constant__ RecurrenceArgs a) {
  extern __shared__ __align__(16) float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int head = blockIdx.x, r = blockIdx.y;
  const int t = a.q_start[r];
  if (a.q_start[r + 1] - t != 1) return;
  const int dim = a.dim, vdim = a.vdim;
  const int slot = a.state_slots[r];
  const int group = head / (a.heads / a.groups);
  float* ks = smem;                    // [dim]
  float* qs = ks + dim;                // [dim]
  float* vs = qs + dim;                // [vdim], already times s_t
  float* parts = vs + vdim;            // [row groups][vdim]
  const bool act = a.act != 0;
  const T* kg = (const T*)a.k + (long long)t * a.k_stride + (long long)group * dim;
  const T* qg = (const T*)a.q + (long long)t * a.q_stride + (long long)group * dim;
  const T* vg = (const T*)a.v + (long long)t * a.v_stride + (long long)head * vdim;
  const float decay = a.token_decay ? a.token_decay[(long long)t * a.heads + head] : a.head_decay[head];
  const float scale = a.token_scale ? a.token_scale[(long long)t * a.heads + head] : 1.f;
  for (int i = threadIdx.x; i < dim; i += kRecurrenceThreads) {
    const float kv = to_float(kg[i]), qv = to_float(qg[i]);
    ks[i] = act ? silu_f(kv) : kv;
    qs[i] = act ? silu_f(qv) : qv;
  }
  for (int i = threadIdx.x; i < vdim; i += kRecurrenceThreads) {
    const float v = to_float(vg[i]);
    vs[i] = scale * (act ? silu_f(v) : v);
  }
  __syncthreads();
  const int quads = vdim >> 2;                       // at most 128
  const int cq = threadIdx.x % quads, row0 = threadIdx.x / quads, row_step = kRecurrenceThreads / quads;
  const bool works = row0 < row_step;                // false: a thread beyond the last whole row group
  const int rows_each = (dim + a.y_splits - 1) / a.y_splits;
  const int row_begin = (int)blockIdx.z * rows_each, row_end = min(dim, row_begin + rows_each);
  const float4 sv = *reinterpret_cast<const float4*>(vs + 4 * cq);
  float4* state = (slot >= 0 && slot < a.num_slots)
      ? reinterpret_cast<float4*>(a.state + (long long)slot * a.state_stride + ((long long)head * dim) * vdim) + cq : nullptr;
  float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
  constexpr int kInFlight = 8;
  for (int row = works ? row_begin + row0 : row_end; row < row_end; row += row_step * kInFlight) {
    float4 s[kInFlight];
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const int rr = row + u * row_step;
      s[u] = (state && rr < row_end) ? state[(long long)rr * quads] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const int rr = row + u * row_step;
      if (rr >= row_end) break;
      const float kv = ks[rr], qv = qs[rr];
      s[u].x = fmaf(decay, s[u].x, kv * sv.x);
      s[u].y = fmaf(decay, s[u].y, kv * sv.y);
      s[u].z = fmaf(decay, s[u].z, kv * sv.z);
      s[u].w = fmaf(decay, s[u].w, kv * sv.w);
      y.x = fmaf(s[u].x, qv, y.x);
      y.y = fmaf(s[u].y, qv, y.y);
      y.z = fmaf(s[u].z, qv, y.z);
      y.w = fmaf(s[u].w, qv, y.w);
      if (state) state[(long long)rr * quads] = s[u];
    }
  }
  if (works) *reinterpret_cast<float4*>(parts + row0 * vdim + 4 * cq) = y;
  __syncthreads();
  const float skip = (a.skip && blockIdx.z == 0) ? a.skip[head] : 0.f;      // the skip term once, in the first part
  float* y_part = a.y + (long long)blockIdx.z * a.y_split_stride;
  for (int c = threadIdx.x; c < vdim; c += kRecurrenceThreads) {
    float total = 0.f;
    for (int g = 0; g < row_step; ++g) total += parts[g * vdim + c];
    const float v = to_float(vg[c]);
    y_part[((long long)t * a.heads + head) * vdim + c] = total + skip * (act ? silu_f(v) : v);
  }
}

// ---------------------------------------------------------------------------
// Gate and norm behind a recurrence.  y [T, width] floats, gate rows of some wider matrix
// (gate[t * gate_stride + i]), weight [width] floats; the row is cut into `parts` equal parts,
// each divided by its own root mean square (eps inside the root), in 32-bit.
//   gate_first:  u = y * g(gate);  out = u / rms(u) * weight          (gate before the norm)
//   otherwise:   out = y / rms(y) * weight * g(gate)                  (gate after the norm)
// g is SiLU (gate_kind 0) or the logistic sigmoid (1).  One CTA per (token, part).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void gated_norm_kernel(const float* __restrict__ y, const T* __restrict__ gate, long long gate_stride,
                                  const float* __restrict__ weight, T* __restrict__ out, int width, int parts,
                                  float eps, int gate_first, int gate_kind) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x / parts, part = blockIdx.x - t * parts;
  const int size = width / parts, base = part * size;
  const float* row = y + (long long)t * width + base;
  const T* g_row = gate + (long long)t * gate_stride + base;
  float ss = 0.f;
  for (int i = threadIdx.x; i < size; i += blockDim.x) {
    float u = row[i];
    if (gate_first) {
      const float g = to_float(g_row[i]);
      u *= gate_kind == 0 ? silu_f(g) : 1.f / (1.f + expf(-g));
    }
    ss += u * u;
  }
  const float factor = rsqrtf(block_sum(ss, scratch) / (float)size + eps);
  for (int i = threadIdx.x; i < size; i += blockDim.x) {
    const float g = to_float(g_row[i]);
    const float gv = gate_kind == 0 ? silu_f(g) : 1.f / (1.f + expf(-g));
    float u = row[i];
    if (gate_first) u = (u * gv) * factor * weight[base + i];
    else u = u * factor * weight[base + i] * gv;
    out[(long long)t * width + base + i] = from_float<T>(u);
  }
}

// ---------------------------------------------------------------------------
// The gates of a matrix memory with exponential gating.  Per request and head, token after token:
//   i = cap tanh((z_i + b_i) / cap),  f = logsigmoid(cap tanh((z_f + b_f) / cap)),
//   m <- max(f + m, i),   decay = exp(f + m_before - m),   scale = exp(i - m),   floor = exp(-m)
// where z are the raw gates [T, 2 heads] (input gates, then forget gates; possibly split-K partial
// sums), m the running maximum that lives in top_state[slot * top_stride + head] (zero after a
// fresh start; a request without a slot starts from zero and stores nothing).  decay and scale are
// what the linear recurrence multiplies its state and its input by; they never exceed one.
// The CTAs (x >= heads, request) of a request each widen the values of a share of its tokens for
// the recurrence, v_wide[t, h] = [v[t, h] | 1 | 0 ...] of `columns` elements, so that the memory's
// normaliser (the same recurrence on the keys alone) is one more column of its state.  CTA h < heads
// of the request makes the gates of head h: a step m -> max(m + f, i) is a pair (f, i), and two
// steps in a row are the pair (f1 + f2, max(i1 + f2, i2)); a warp takes 32 tokens at a time, a
// lane each, a scan over the lanes' pairs gives every lane its token's maximum from the one the
// tile starts with, and the last lane's is the next tile's start.  A portion of more than 256 tokens
// is cut into a range per warp: every warp first folds its range into one pair, the pairs of the
// ranges before it give the maximum its range starts from, and it walks the range again.  Nothing
// passes through memory on the way.  The maximum only sets the scale that state, normaliser and floor share, so the
// order of these sums moves no result beyond the rounding of that scale.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }
constexpr int kGateWarps = 8;      // warps of a CTA of the gate kernel

template <typename T>
__global__ void __launch_bounds__(256)
memory_gates_kernel(const float* __restrict__ gates, int splits, size_t split_stride, const float* __restrict__ bias,
                    float cap, const T* __restrict__ v, long long v_stride, float* __restrict__ top_state,
                    long long top_stride, int num_slots, const int* __restrict__ q_start,
                    const int* __restrict__ state_slots, float* __restrict__ decay, float* __restrict__ scale,
                    float* __restrict__ floor, T* __restrict__ v_wide, int heads, int vdim, int columns) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.y;
  const int first = q_start[r], last = q_start[r + 1];
  const int count = last - first;
  if (count <= 0) return;
  if ((int)blockIdx.x >= heads) {
    // this CTA's share of the request's tokens, widened: a warp per (token, head) row
    const int shares = (int)gridDim.x - heads;
    const int per = (count + shares - 1) / shares;
    const int t0 = first + ((int)blockIdx.x - heads) * per, t1 = min(last, t0 + per);
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int rows = max(0, t1 - t0) * heads;
    for (int row = threadIdx.x >> 5; row < rows; row += warps) {
      const int t = t0 + row / heads, h = row % heads;
      const T* src = v + (long long)t * v_stride + h * vdim;
      T* dst = v_wide + ((size_t)t * heads + h) * columns;
      for (int d = lane; d < columns; d += 32)
        dst[d] = d < vdim ? src[d] : from_float<T>(d == vdim ? 1.f : 0.f);
    }
    return;
  }
  __shared__ float range_add[kGateWarps], range_least[kGateWarps];
  const int h = blockIdx.x;
  const int slot = state_slots[r];
  const bool kept = slot >= 0 && slot < num_slots;
  const float inv_cap = 1.f / cap;
  const int width = 2 * heads;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float bias_in = bias[h], bias_keep = bias[heads + h];
  // a tile's raw gates are fetched while the tile before it is scanned
  auto fetch = [&](int t, int t_end, float& zi, float& zf) {
    zi = bias_in;
    zf = bias_keep;
    if (t >= t_end) return;
    for (int s = 0; s < splits; ++s) {
      zi += gates[(size_t)s * split_stride + (size_t)t * width + h];
      zf += gates[(size_t)s * split_stride + (size_t)t * width + heads + h];
    }
  };
  // One tile: the capped logarithms of the lane's token, and the steps of the tile's tokens 0 .. lane in a row.
  // A token beyond the range is the step that changes nothing: (0, -inf).
  auto scan_tile = [&](bool in, float zi, float zf, float& log_in, float& log_keep, float& add, float& least) {
    add = 0.f;
    least = -INFINITY;
    if (in) {
      least = cap * tanhf(zi * inv_cap);
      add = log_sigmoid_f(cap * tanhf(zf * inv_cap));
    }
    log_in = least;
    log_keep = add;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float add_before = __shfl_up_sync(0xffffffffu, add, o);
      const float least_before = __shfl_up_sync(0xffffffffu, least, o);
      if (lane >= o) {
        least = fmaxf(least_before + add, least);
        add += add_before;
      }
    }
  };
  // A short portion is one warp's; a long one is cut into a range of whole tiles per warp, and every
  // warp first folds its range into one step so that each knows the maximum its range starts from.
  const bool ranges = count > 8 * 32;
  if (!ranges && warp > 0) return;
  int range_first = first, range_last = last;
  if (ranges) {
    const int per = ((count + kGateWarps - 1) / kGateWarps + 31) / 32 * 32;
    range_first = min(last, first + warp * per);
    range_last = min(last, range_first + per);
  }
  float carry = kept ? top_state[(long long)slot * top_stride + h] : 0.f;      // the maximum before the tile
  if (ranges) {
    float run_add = 0.f, run_least = -INFINITY;
    float zi_next, zf_next;
    fetch(range_first + lane, range_last, zi_next, zf_next);
    for (int t0 = range_first; t0 < range_last; t0 += 32) {
      const float zi = zi_next, zf = zf_next;
      fetch(t0 + lane + 32, range_last, zi_next, zf_next);
      float log_in, log_keep, add, least;
      scan_tile(t0 + lane < range_last, zi, zf, log_in, log_keep, add, least);
      const float tile_add = __shfl_sync(0xffffffffu, add, 31), tile_least = __shfl_sync(0xffffffffu, least, 31);
      run_least = fmaxf(run_least + tile_add, tile_least);
      run_add += tile_add;
    }
    if (lane == 0) {
      range_add[warp] = run_add;
      range_least[warp] = run_least;
    }
    __syncthreads();
    for (int w = 0; w < warp; ++w) carry = fmaxf(carry + range_add[w], range_least[w]);
  }
  float zi_next, zf_next;
  fetch(range_first + lane, range_last, zi_next, zf_next);
  for (int t0 = range_first; t0 < range_last; t0 += 32) {
    const int t = t0 + lane;
    const bool in = t < range_last;
    const float zi = zi_next, zf = zf_next;
    fetch(t + 32, range_last, zi_next, zf_next);
    float log_in, log_keep, add, least;
    scan_tile(in, zi, zf, log_in, log_keep, add, least);
    const float m = fmaxf(carry + add, least);                 // the maximum behind this token
    float before = __shfl_up_sync(0xffffffffu, m, 1);
    if (lane == 0) before = carry;
    if (in) {
      const size_t at = (size_t)t * heads + h;
      // neither exponent is positive; the scan's sums may leave one a rounding above zero
      decay[at] = expf(fminf(log_keep + before - m, 0.f));
      scale[at] = expf(fminf(log_in - m, 0.f));
      floor[at] = expf(-m);
    }
    carry = __shfl_sync(0xffffffffu, m, 31);
  }
  // the warp of the last range (of the whole portion, if it is one warp's) holds the request's last maximum
  const bool closes = ranges ? warp == kGateWarps - 1 : true;
  if (closes && lane == 0 && kept) top_state[(long long)slot * top_stride + h] = carry;
}

// ---------------------------------------------------------------------------
// What a matrix memory hands on.  y [T, heads * columns] floats is the recurrence's output on the
// widened values: per head `vdim` numerators and, at column vdim, the normaliser's product with the
// query.  With c the queries' factor (applied here, to numerators and normaliser alike):
//   o = c y[:vdim] / (max(|c y[vdim]|, floor) + denominator_eps)
//   out = o / sqrt(mean(o^2) + eps) * weight * sigmoid(gate)
// head by head, in 32-bit.  One warp per (token, head).
// ---------------------------------------------------------------------------
template <typename T, bool kParts>
__global__ void memory_output_kernel(const float* __restrict__ y, const float* __restrict__ floor,
                                     const T* __restrict__ gate, long long gate_stride,
                                     const float* __restrict__ weight, T* __restrict__ out, long long pairs, int heads,
                                     int vdim, int columns, float query_scale, float eps, float denominator_eps,
                                     int y_splits, long long y_split_stride) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long pair = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (pair >= pairs) return;
  const long long t = pair / heads;
  const int h = (int)(pair - t * heads);
  const float* row = y + (t * heads + h) * columns;
  // y may come as the parts of several CTAs that shared the head's rows: added up here, in order
  auto value = [&](int d) {
    if (!kParts) return row[d];
    // up to eight parts, all their loads in flight together, added in order (the launcher checks the count)
    float part[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) part[s] = s < y_splits ? row[(long long)s * y_split_stride + d] : 0.f;
    float total = 0.f;
#pragma unroll
    for (int s = 0; s < 8; ++s) total += part[s];
    return total;
  };
  const float below = fmaxf(fabsf(query_scale * value(vdim)), floor[pair]) + denominator_eps;
  const float factor = query_scale / below;
  float ss = 0.f;
  for (int d = lane; d < vdim; d += 32) {
    const float o = value(d) * factor;
    ss += o * o;
  }
  const float unit = rsqrtf(warp_sum(ss) / (float)vdim + eps);
  const T* g_row = gate + t * gate_stride + (long long)h * vdim;
  T* o_row = out + (t * heads + h) * vdim;
  for (int d = lane; d < vdim; d += 32) {
    const float g = to_float(g_row[d]);
    o_row[d] = from_float<T>(value(d) * factor * unit * weight[h * vdim + d] * (1.f / (1.f + expf(-g))));
  }
}

// ---------------------------------------------------------------------------
// A gated linear recurrence with one state value per channel (a real-gated linear recurrent
// unit).  Per request and channel c of block b = c / part, token after token:
//   r = sigmoid(gates[t, b, k] + gate_bias[b, k]),   i = sigmoid(gates[t, b, part + k] + gate_bias[b, part + k]),
//   a = exp(rate[c] * r),   S <- a S + sqrt(1 - a^2) i u[t, c],   out[t, c] = out_scale * S * gelu(y[t, c] + y_bias[c])
// with k = c % part, rate negative (so 0 < a <= 1) and the tanh form of GELU.  One thread per
// (request, segment, channel); everything that does not depend on S (gates, decay, input, the other
// branch's activation) is computed for kScanBatch tokens at a time before their chain of
// multiply-adds, so the loads and the transcendental functions of a batch overlap.  S comes from
// and returns to state[slot * state_stride + c]; a request without a slot starts from zero and
// stores nothing.  A channel that remembers for long has a within 1e-5 of 1, where a float keeps two or
// three digits of 1 - a; so the kernel carries d = 1 - a = -expm1(rate r) instead, steps S <- S - d S + input,
// and forms 1 - a^2 as d (2 - d): the decay keeps its digits however close to 1 it is.
// ---------------------------------------------------------------------------
constexpr int kScanBatch = 8;
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

// A long portion is cut into segments of `segment_len` tokens that run side by side, one thread per
// (request, segment, channel).  The first pass runs every segment but a request's last from a zero
// state and leaves the product P of its decays and its own contribution B; the emitting pass walks
// the segments before its own (S <- P S + B, from the slot's state) and then runs its tokens.  A
// request's last segment writes the state back.  With one segment the emitting pass is all there is.
struct ScanArgs {
  const float* gates;
  const float* gate_bias;
  const void* u;
  const void* y;
  long long y_stride;
  const float* y_bias;
  const float* rate;
  float* state;
  long long state_stride;
  int num_slots;
  const int* q_start;
  const int* state_slots;
  void* out;
  float out_scale;
  int width, part, segments, segment_len;
  float* segment_keep;      // [requests * segments, width]: P
  float* segment_add;       // [requests * segments, width]: B
};

template <typename T, bool kEmit>
__global__ void __launch_bounds__(128) gated_scan_kernel(const __grid_constant__ ScanArgs a) {
  pdl_launch_dependents();
  const int r = blockIdx.z, seg = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int width = a.width, part = a.part;
  const bool live = c < width;
  const int b = live ? c / part : 0, k = live ? c - b * part : 0;
  const long long gate_row = 2ll * width;
  const int ga = b * 2 * part + k, gi = ga + part;
  const float bias_a = live ? a.gate_bias[ga] : 0.f, bias_i = live ? a.gate_bias[gi] : 0.f;
  const float channel_rate = live ? a.rate[c] : 0.f, channel_bias = (live && kEmit) ? a.y_bias[c] : 0.f;
  const T* u = (const T*)a.u;
  const T* y = (const T*)a.y;
  T* out = (T*)a.out;
  pdl_wait();
  if (!live) return;
  const int begin = a.q_start[r], end = a.q_start[r + 1];
  const int first = begin + seg * a.segment_len;
  if (first >= end) return;
  const int last = min(end, first + a.segment_len);
  const bool closes = last == end;                       // the request's last segment
  if (!kEmit && closes) return;
  const int slot = a.state_slots[r];
  const bool kept = slot >= 0 && slot < a.num_slots;
  float s = 0.f, keep = 1.f;
  if (kEmit) {
    s = kept ? a.state[(long long)slot * a.state_stride + c] : 0.f;
    const size_t row0 = (size_t)r * a.segments;
    for (int j0 = 0; j0 < seg; j0 += kScanBatch) {
      float p[kScanBatch], q[kScanBatch];
#pragma unroll
      for (int e = 0; e < kScanBatch; ++e) {
        const bool in = j0 + e < seg;
        p[e] = in ? a.segment_keep[(row0 + j0 + e) * width + c] : 1.f;
        q[e] = in ? a.segment_add[(row0 + j0 + e) * width + c] : 0.f;
      }
#pragma unroll
      for (int e = 0; e < kScanBatch; ++e) s = fmaf(p[e], s, q[e]);
    }
  }
  for (int t0 = first; t0 < last; t0 += kScanBatch) {
    float d[kScanBatch], in[kScanBatch], other[kScanBatch];
#pragma unroll
    for (int e = 0; e < kScanBatch; ++e) {
      const int t = t0 + e;
      if (t < last) {
        const float gr = a.gates[t * gate_row + ga] + bias_a;
        const float gin = a.gates[t * gate_row + gi] + bias_i;
        const float log_a = channel_rate * sigmoid_f(gr);
        d[e] = -expm1f(log_a);
        in[e] = sqrtf(d[e] * (2.f - d[e])) * sigmoid_f(gin) * to_float(u[(long long)t * width + c]);
        if (kEmit) other[e] = a.out_scale * gelu_tanh_f(to_float(y[(long long)t * a.y_stride + c]) + channel_bias);
      }
    }
#pragma unroll
    for (int e = 0; e < kScanBatch; ++e) {
      const int t = t0 + e;
      if (t < last) {
        s = fmaf(-d[e], s, s) + in[e];
        if (kEmit) out[(long long)t * width + c] = from_float<T>(s * other[e]);
        else keep = fmaf(-d[e], keep, keep);
      }
    }
  }
  if (kEmit) {
    if (closes && kept) a.state[(long long)slot * a.state_stride + c] = s;
  } else {
    const size_t row = (size_t)r * a.segments + seg;
    a.segment_keep[row * width + c] = keep;
    a.segment_add[row * width + c] = s;
  }
}

}  // namespace einf

using namespace einf;

extern "C" int einf_conv_silu(const void* in, int dtype, long long in_stride, const float* weight, const float* bias,
                              float* conv_state, long long state_stride, const int* seq_of_token, const int* q_start,
                              const int* state_slots, int num_slots, int num_requests, void* out, int channels,
                              int taps, int num_tokens, const void* dt_in, const float* dt_bias, const float* a_log,
                              float* dt_out, float* decay_out, int heads, int act, const float* input_bias,
                              cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (taps < 1 || taps > kMaxTaps || channels <= 0 || num_requests > 65535) return (int)cudaErrorInvalidValue;
  const int threads = 256;
  const long long total = (long long)num_tokens * (channels + heads);
  long long blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  EINF_DISPATCH_2(dtype, T, {
    cudaError_t e = launch_pdl(conv_silu_kernel<T>, (int)blocks, threads, 0, stream, (const T*)in, in_stride, weight,
                               bias, (const float*)conv_state, state_stride, seq_of_token, q_start, state_slots,
                               num_slots, (T*)out, channels, taps, num_tokens, (const T*)dt_in, dt_bias, a_log, dt_out,
                               decay_out, heads, act, input_bias);
    if (e != cudaSuccess || taps == 1) return (int)e;
    const dim3 grid((channels + 127) / 128, num_requests);
    return (int)launch_pdl(conv_state_update_kernel<T>, grid, 128, 0, stream, (const T*)in, in_stride, conv_state,
                           state_stride, q_start, state_slots, num_slots, channels, taps, input_bias);
  })
}

// rows per thread: 0 lets the launcher choose among 16, 8 and 4; columns per thread: 0 (the launcher's
// choice), 1, or 2 (with 16 rows).  segments > 1 needs segment_state [requests * segments,
// heads, dim, vdim] and segment_decay [requests * segments, heads].
extern "C" int einf_linear_recurrence(const void* q, const void* k, const void* v, int dtype, long long q_stride,
                                      long long k_stride, long long v_stride, const float* head_decay,
                                      const float* token_decay, const float* token_scale, const float* skip,
                                      float* state, long long state_stride, int num_slots, const int* q_start,
                                      const int* state_slots, int num_requests, float* y, int heads, int groups,
                                      int dim, int vdim, int act, int rows, int columns, int segments,
                                      int segment_len, float* segment_state, float* segment_decay, int y_splits,
                                      long long y_split_stride, cudaStream_t stream) {
  if (num_requests == 0) return 0;
  if (y_splits < 1 || y_splits > 64) return (int)cudaErrorInvalidValue;
  if (heads <= 0 || groups <= 0 || heads % groups || dim <= 0 || vdim <= 0 || dim > 512 || heads > 65535 ||
      segments < 1 || segment_len < 1 || (long long)num_requests * segments > 65535 ||
      (segments > 1 && (!segment_state || !segment_decay)))
    return (int)cudaErrorInvalidValue;
  // Sixteen rows a thread wherever the state has that many: measured at every size tried (14 heads of
  // 64 x 64 and of 128 x 64, 12 of 128 x 128; one segment and sixteen), fewer rows, which are more and
  // lighter threads, were slower.
  if (rows == 0) rows = dim > 8 ? 16 : dim > 4 ? 8 : 4;
  if ((rows != 4 && rows != 8 && rows != 16) || 32 * rows < dim) return (int)cudaErrorInvalidValue;
  RecurrenceArgs a;
  a.q = q; a.k = k; a.v = v;
  a.q_stride = q_stride; a.k_stride = k_stride; a.v_stride = v_stride;
  a.head_decay = head_decay; a.token_decay = token_decay; a.token_scale = token_scale; a.skip = skip;
  a.state = state; a.state_stride = state_stride;
  a.q_start = q_start; a.state_slots = state_slots;
  a.y = y;
  a.y_splits = y_splits; a.y_split_stride = y_split_stride;
  a.segment_state = segment_state; a.segment_decay = segment_decay;
  a.num_slots = num_slots; a.heads = heads; a.groups = groups; a.dim = dim; a.vdim = vdim; a.act = act;
  a.segments = segments; a.segment_len = segment_len;
  // A step of single tokens (segment_len 1 says so): the streaming kernel, where it takes the sizes.
  if (segments == 1 && segment_len == 1 && vdim % 4 == 0 && vdim / 4 <= kRecurrenceThreads &&
      state_stride % 4 == 0 && ((uintptr_t)state & 15) == 0) {
    a.lanes_per_column = 0; a.dim_pad = dim; a.batch = 1;
    const int row_groups = kRecurrenceThreads / (vdim / 4);
    const size_t bytes = (size_t)(2 * dim + vdim + row_groups * vdim) * sizeof(float);
    const dim3 step_grid(heads, num_requests, y_splits);
    EINF_DISPATCH_2(dtype, T, {
      return (int)launch_pdl(recurrence_step_kernel<T>, step_grid, kRecurrenceThreads, bytes, stream, a);
    })
  }
  if (y_splits != 1) return (int)cudaErrorInvalidValue;      // parts of y are the streaming kernel's alone
  int lanes = 1;
  while (lanes * rows < dim) lanes <<= 1;
  a.lanes_per_column = lanes;
  a.dim_pad = lanes * rows;
  // Two columns a thread where the state is wide enough for it and the launch still has CTAs for
  // the whole GPU (or the caller says so).
  const int thread_columns = (kRecurrenceThreads / 32) * (32 / lanes);
  if (columns == 0) {
    const long long ctas = (long long)((vdim + 2 * thread_columns - 1) / (2 * thread_columns)) * heads * num_requests * segments;
    columns = (rows == 16 && vdim >= 2 * thread_columns && ctas >= 2 * 148) ? 2 : 1;
  }
  if (columns != 1 && !(columns == 2 && rows == 16)) return (int)cudaErrorInvalidValue;
  const int columns_per_block = columns * thread_columns;
  int batch = kStageKQ * kRecurrenceThreads / dim;
  if (batch > kStageV * kRecurrenceThreads / columns_per_block) batch = kStageV * kRecurrenceThreads / columns_per_block;
  if (batch > kMaxBatch) batch = kMaxBatch;
  if (batch < 1) return (int)cudaErrorInvalidValue;
  a.batch = batch;
  const dim3 grid((vdim + columns_per_block - 1) / columns_per_block, heads, num_requests * segments);
  auto buffer_bytes = [&](bool emit) {
    const int floats = ((emit ? 2 : 1) * batch * a.dim_pad + batch * columns_per_block + 2 * batch + 3) & ~3;
    return (size_t)2 * floats * sizeof(float);
  };
#define EINF_RECURRENCE_ROWS(ROWS_, COLS_)                                                                                   \
  {                                                                                                                   \
    if (segments > 1) {                                                                                               \
      cudaError_t e = launch_pdl(linear_recurrence_kernel<T, ROWS_, COLS_, false>, grid, kRecurrenceThreads,          \
                                 buffer_bytes(false), stream, a);                                                     \
      if (e != cudaSuccess) return (int)e;                                                                            \
      const long long per_head = (long long)dim * vdim;                                                               \
      const dim3 walk_grid((unsigned)((per_head + 255) / 256 > 64 ? 64 : (per_head + 255) / 256), heads, num_requests); \
      e = launch_pdl(recurrence_walk_kernel, walk_grid, 256, 0, stream, a);                                           \
      if (e != cudaSuccess) return (int)e;                                                                            \
    }                                                                                                                 \
    return (int)launch_pdl(linear_recurrence_kernel<T, ROWS_, COLS_, true>, grid, kRecurrenceThreads, buffer_bytes(true), \
                           stream, a);                                                                                \
  }
  EINF_DISPATCH_2(dtype, T, {
    if (rows == 16 && columns == 2) EINF_RECURRENCE_ROWS(16, 2)
    if (rows == 16) EINF_RECURRENCE_ROWS(16, 1)
    if (rows == 8) EINF_RECURRENCE_ROWS(8, 1)
    EINF_RECURRENCE_ROWS(4, 1)
  })
#undef EINF_RECURRENCE_ROWS
}

extern "C" int einf_gated_norm(const float* y, const void* gate, int dtype, long long gate_stride, const float* weight,
                               void* out, int num_tokens, int width, int parts, float eps, int gate_first,
                               int gate_kind, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (parts <= 0 || width % parts) return (int)cudaErrorInvalidValue;
  const int size = width / parts;
  int threads = 32;
  while (threads < size && threads < 256) threads <<= 1;
  const long long blocks = (long long)num_tokens * parts;
  if (blocks >= (1ll << 31)) return (int)cudaErrorInvalidValue;
  EINF_DISPATCH_2(dtype, T, {
    return (int)launch_pdl(gated_norm_kernel<T>, (int)blocks, threads, 0, stream, y, (const T*)gate, gate_stride, weight,
                           (T*)out, width, parts, eps, gate_first, gate_kind);
  })
}

extern "C" int einf_gated_scan(const float* gates, const float* gate_bias, const void* u, const void* y, int dtype,
                               long long y_stride, const float* y_bias, const float* rate, float* state,
                               long long state_stride, int num_slots, const int* q_start, const int* state_slots,
                               int num_requests, void* out, float out_scale, int width, int blocks, int segments,
                               int segment_len, float* segment_keep, float* segment_add, cudaStream_t stream) {
  if (num_requests == 0 || width == 0) return 0;
  if (blocks <= 0 || width % blocks || num_requests > 65535 || segments < 1 || segments > 65535 || segment_len < 1 ||
      (segments > 1 && (!segment_keep || !segment_add)))
    return (int)cudaErrorInvalidValue;
  ScanArgs a;
  a.gates = gates; a.gate_bias = gate_bias; a.u = u; a.y = y; a.y_stride = y_stride; a.y_bias = y_bias; a.rate = rate;
  a.state = state; a.state_stride = state_stride; a.num_slots = num_slots; a.q_start = q_start;
  a.state_slots = state_slots; a.out = out; a.out_scale = out_scale; a.width = width; a.part = width / blocks;
  a.segments = segments; a.segment_len = segment_len; a.segment_keep = segment_keep; a.segment_add = segment_add;
  const int threads = 128;
  const dim3 grid((width + threads - 1) / threads, segments, num_requests);
  EINF_DISPATCH_2(dtype, T, {
    if (segments > 1) {
      cudaError_t e = launch_pdl(gated_scan_kernel<T, false>, grid, threads, 0, stream, a);
      if (e != cudaSuccess) return (int)e;
    }
    return (int)launch_pdl(gated_scan_kernel<T, true>, grid, threads, 0, stream, a);
  })
}

extern "C" int einf_memory_gates(const float* gates, int splits, long long split_stride, const float* bias, float cap,
                                 const void* v, int dtype, long long v_stride, float* top_state, long long top_stride,
                                 int num_slots, const int* q_start, const int* state_slots, int num_requests,
                                 float* decay, float* scale, float* floor, void* v_wide, int num_tokens, int heads,
                                 int vdim, int columns, int longest, cudaStream_t stream) {
  if (num_requests == 0 || num_tokens == 0) return 0;
  if (heads <= 0 || vdim <= 0 || columns <= vdim || !(cap > 0.f) || num_requests > 65535)
    return (int)cudaErrorInvalidValue;
  // CTAs that share a request's tokens for the widening: about 16 tokens each, up to 128
  if (longest <= 0) longest = num_tokens;
  int shares = (longest + 15) / 16;
  shares = shares < 1 ? 1 : (shares > 128 ? 128 : shares);
  const dim3 grid(heads + shares, num_requests);  // a CTA per head of a request makes its gates, the others widen its values
  EINF_DISPATCH_2(dtype, T, {
    return (int)launch_pdl(memory_gates_kernel<T>, grid, dim3(32 * kGateWarps), 0, stream, gates, splits < 1 ? 1 : splits,
                           (size_t)split_stride, bias, cap, (const T*)v, v_stride, top_state, top_stride, num_slots,
                           q_start, state_slots, decay, scale, floor, (T*)v_wide, heads, vdim, columns);
  })
}

extern "C" int einf_memory_output(const float* y, const float* floor, const void* gate, int dtype, long long gate_stride,
                                  const float* weight, void* out, int num_tokens, int heads, int vdim, int columns,
                                  float query_scale, float eps, float denominator_eps, int y_splits,
                                  long long y_split_stride, cudaStream_t stream) {
  if (num_tokens == 0) return 0;
  if (heads <= 0 || vdim <= 0 || columns <= vdim || y_splits < 1 || y_splits > 8) return (int)cudaErrorInvalidValue;
  const long long pairs = (long long)num_tokens * heads;
  const int threads = 128;
  const long long blocks = (pairs * 32 + threads - 1) / threads;
  if (blocks >= (1ll << 31)) return (int)cudaErrorInvalidValue;
  EINF_DISPATCH_2(dtype, T, {
    if (y_splits == 1)
      return (int)launch_pdl(memory_output_kernel<T, false>, (int)blocks, threads, 0, stream, y, floor, (const T*)gate,
                             gate_stride, weight, (T*)out, pairs, heads, vdim, columns, query_scale, eps,
                             denominator_eps, y_splits, y_split_stride);
    return (int)launch_pdl(memory_output_kernel<T, true>, (int)blocks, threads, 0, stream, y, floor, (const T*)gate,
                           gate_stride, weight, (T*)out, pairs, heads, vdim, columns, query_scale, eps,
                           denominator_eps, y_splits, y_split_stride);
  })
}
