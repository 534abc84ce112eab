// The gated delta rule: a recurrent mixer whose state is one matrix S [dim, vdim] per head.
//
// Per token, from projections of the layer's input (query and key heads may be shared by
// several value heads):
//
//     q, k, v   <- silu(short causal convolution over time, per channel)
//     q, k      <- unit vectors per head (x / sqrt(sum x^2 + unit_eps)); q also times dim^-1/2
//     beta      =  sigmoid(b),   g = exp(-exp(A_log) * softplus(a + dt_bias))        (per head)
//     S <- g S;  w = beta (v - S^T k);  S <- S + k w^T;  o = S^T q                 (in this order)
//     out       =  o / rms(o) * norm_weight * silu(gate)                             (per head)
//
// What is carried from token to token per request lies in one float32 slot: the heads' matrices
// [heads, dim, vdim] followed by the last (taps - 1) inputs of the convolution [taps - 1, channels].
// All of the recurrence is float32: unit norms, decay, beta, the state, the read-out and its norm.
//
// Four kernels:
//   delta_prepare       one warp per (token, q/k/v head): convolution + silu (+ unit norm), and per
//                       token the heads' decay and beta, into float32 buffers
//   delta_conv_advance  per (row, channel): the slot's convolution inputs move on by the row's tokens
//   delta_recurrence    per (row, head, slice of vdim): walks the row's tokens in order; the columns
//                       of S are independent of each other, so a block owns COLS of them, a column's
//                       dim entries spread over P lanes that add up by shuffles
//   delta_gated_norm    one warp per (token, head): RMS norm of the read-out, weight, gate
// The order of every sum depends on the sizes only, so a token's result does not depend on how the
// step was cut or what else is in the batch.
#include "common.cuh"

namespace pylon {

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// proj: [T, ld] projections in T (columns [q | k | v | ...] from column 0; gate_a / gate_b name the columns of a and b).
// conv_w: float32 [channels, taps] in the same channel order.  state: float32 [slots, slot_floats]; the convolution
// inputs start at conv_offset.  qkv: float32 [T, channels] out.  gates: float32 [T, 2, heads] out (decay, beta).
template <typename T, int MAX_TAPS>
__global__ void delta_prepare_kernel(const T* __restrict__ proj, long long ld, const float* __restrict__ conv_w, int taps,
                                     const float* __restrict__ state, long long slot_floats, long long conv_offset,
                                     const int* __restrict__ token_row, const int* __restrict__ q_start, const int* __restrict__ slots,
                                     float* __restrict__ qkv, float* __restrict__ gates, const float* __restrict__ a_log,
                                     const float* __restrict__ dt_bias, int col_a, int col_b, int heads, int kv_heads, int dim, int vdim,
                                     float unit_eps, int num_tokens) {
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int units = 2 * kv_heads + heads + 1;   // q heads, k heads, v heads, and one unit for the token's gates
  const long long item = (long long)blockIdx.x * warps_per_block + warp;
  if (item >= (long long)num_tokens * units) return;
  const int t = (int)(item / units), unit = (int)(item % units);
  const int row = token_row[t];
  if (row < 0) return;
  const T* mine = proj + (long long)t * ld;
  if (unit == units - 1) {
    for (int h = lane; h < heads; h += 32) {
      const float a = to_float<T>(mine[col_a + h]), b = to_float<T>(mine[col_b + h]);
      gates[(long long)t * 2 * heads + h] = expf(-expf(a_log[h]) * softplus_f(a + dt_bias[h]));
      gates[(long long)t * 2 * heads + heads + h] = 1.f / (1.f + expf(-b));
    }
    return;
  }
  const int channels = 2 * kv_heads * dim + heads * vdim;
  const bool is_value = unit >= 2 * kv_heads;
  const int size = is_value ? vdim : dim;
  const int first = is_value ? 2 * kv_heads * dim + (unit - 2 * kv_heads) * vdim : unit * dim;
  const int index = t - q_start[row];        // the token's place among the row's tokens of this step
  const float* old = state + (long long)slots[row] * slot_floats + conv_offset;   // [taps - 1, channels]
  float sumsq = 0.f;
  for (int e = lane; e < size; e += 32) {
    const int c = first + e;
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_TAPS; ++j) {
      if (j < taps) {
        const int back = taps - 1 - j;       // how many tokens before this one
        float input;
        if (back <= index) input = to_float<T>(proj[(long long)(t - back) * ld + c]);
        else input = old[(long long)(taps - 1 - (back - index)) * channels + c];
        acc = fmaf(conv_w[(long long)c * taps + j], input, acc);
      }
    }
    acc = silu_f(acc);
    qkv[(long long)t * channels + c] = acc;   // values are done; queries and keys are scaled below
    sumsq = fmaf(acc, acc, sumsq);
  }
  if (is_value) return;
  sumsq = warp_sum(sumsq);
  float factor = rsqrtf(sumsq + unit_eps);
  if (unit < kv_heads) factor *= rsqrtf((float)dim);
  __syncwarp();
  for (int e = lane; e < size; e += 32) qkv[(long long)t * channels + first + e] *= factor;
}

// The last (taps - 1) convolution inputs of every row move on by the tokens the row brought.
template <typename T, int MAX_TAPS>
__global__ void delta_conv_advance_kernel(const T* __restrict__ proj, long long ld, int taps, float* __restrict__ state,
                                          long long slot_floats, long long conv_offset, const int* __restrict__ q_start,
                                          const int* __restrict__ slots, int channels, int num_rows) {
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= (long long)num_rows * channels) return;
  const int row = (int)(item / channels), c = (int)(item % channels);
  const int begin = q_start[row], count = q_start[row + 1] - begin;
  if (count <= 0) return;
  float* mine = state + (long long)slots[row] * slot_floats + conv_offset;
  float kept[MAX_TAPS];
#pragma unroll
  for (int m = 0; m < MAX_TAPS; ++m) {
    if (m < taps - 1) {
      const int rel = count - (taps - 1) + m;   // place among the row's tokens; negative: from the old inputs
      kept[m] = rel >= 0 ? to_float<T>(proj[(long long)(begin + rel) * ld + c]) : mine[(long long)(m + count) * channels + c];
    }
  }
#pragma unroll
  for (int m = 0; m < MAX_TAPS; ++m)
    if (m < taps - 1) mine[(long long)m * channels + c] = kept[m];
}

// grid (slices of vdim, heads, rows); block = COLS columns x P lanes.  PER >= ceil(dim / P).
template <int PER>
__global__ void delta_recurrence_kernel(const float* __restrict__ qkv, const float* __restrict__ gates, float* __restrict__ state,
                                        long long slot_floats, const int* __restrict__ q_start, const int* __restrict__ slots,
                                        float* __restrict__ out, int heads, int kv_heads, int dim, int vdim, int lanes, int cols) {
  const int P = lanes;
  const int p = threadIdx.x % P;
  const int j = blockIdx.x * cols + threadIdx.x / P;   // my column of the head's matrix
  const int head = blockIdx.y, row = blockIdx.z;
  const int begin = q_start[row], end = q_start[row + 1];
  if (end <= begin) return;
  const bool live = j < vdim && (int)threadIdx.x / P < cols;   // a block is padded to a whole warp: the lanes beyond its columns only keep the shuffles whole
  const int kv = head / (heads / kv_heads);
  const int channels = 2 * kv_heads * dim + heads * vdim;
  const int q_col = kv * dim, k_col = kv_heads * dim + kv * dim, v_col = 2 * kv_heads * dim + head * vdim + j;
  float* mine = state + (long long)slots[row] * slot_floats + ((long long)head * dim) * vdim + j;   // S[i, j] at mine[i * vdim]
  float s[PER];
#pragma unroll
  for (int n = 0; n < PER; ++n) {
    const int i = p + n * P;
    s[n] = (live && i < dim) ? mine[(long long)i * vdim] : 0.f;
  }
  float k_next[PER], q_next[PER];
  float g_next, beta_next, v_next;
  auto fetch = [&](int t) {
    const float* token = qkv + (long long)t * channels;
#pragma unroll
    for (int n = 0; n < PER; ++n) {
      const int i = p + n * P;
      k_next[n] = i < dim ? token[k_col + i] : 0.f;
      q_next[n] = i < dim ? token[q_col + i] : 0.f;
    }
    g_next = gates[(long long)t * 2 * heads + head];
    beta_next = gates[(long long)t * 2 * heads + heads + head];
    v_next = live ? token[v_col] : 0.f;
  };
  fetch(begin);
  for (int t = begin; t < end; ++t) {
    float k[PER], q[PER];
#pragma unroll
    for (int n = 0; n < PER; ++n) { k[n] = k_next[n]; q[n] = q_next[n]; }
    const float g = g_next, beta = beta_next, v = v_next;
    if (t + 1 < end) fetch(t + 1);
    float dot = 0.f;
#pragma unroll
    for (int n = 0; n < PER; ++n) {
      s[n] *= g;
      dot = fmaf(s[n], k[n], dot);
    }
    for (int offset = P >> 1; offset > 0; offset >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, offset);
    const float w = beta * (v - dot);
    float read = 0.f;
#pragma unroll
    for (int n = 0; n < PER; ++n) {
      s[n] = fmaf(k[n], w, s[n]);
      read = fmaf(s[n], q[n], read);
    }
    for (int offset = P >> 1; offset > 0; offset >>= 1) read += __shfl_xor_sync(0xffffffffu, read, offset);
    if (live && p == 0) out[((long long)t * heads + head) * vdim + j] = read;
  }
  if (live) {
#pragma unroll
    for (int n = 0; n < PER; ++n) {
      const int i = p + n * P;
      if (i < dim) mine[(long long)i * vdim] = s[n];
    }
  }
}

// o: float32 [T, heads, vdim]; gate: columns of proj from col_gate, [heads, vdim]; out [T, heads * vdim] in T.
template <typename T>
__global__ void delta_gated_norm_kernel(const float* __restrict__ o, const T* __restrict__ proj, long long ld, int col_gate,
                                        const float* __restrict__ weight, T* __restrict__ out, int heads, int vdim, float eps,
                                        int num_tokens) {
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * warps_per_block + warp;
  if (item >= (long long)num_tokens * heads) return;
  const int t = (int)(item / heads), head = (int)(item % heads);
  const float* mine = o + item * vdim;
  float sumsq = 0.f;
  for (int e = lane; e < vdim; e += 32) sumsq = fmaf(mine[e], mine[e], sumsq);
  sumsq = warp_sum(sumsq);
  const float inv = rsqrtf(sumsq / (float)vdim + eps);
  const T* gate = proj + (long long)t * ld + col_gate + head * vdim;
  T* dst = out + item * vdim;
  for (int e = lane; e < vdim; e += 32) dst[e] = from_float<T>(mine[e] * inv * weight[e] * silu_f(to_float<T>(gate[e])));
}

}  // namespace pylon

using namespace pylon;

constexpr int DELTA_MAX_TAPS = 8;

template <typename T>
static int launch_delta(const void* proj_v, long long ld, const float* conv_w, int taps, float* state, long long slot_floats,
                        const int* token_row, const int* q_start, const int* slots, float* qkv, float* gates, float* o, void* out_v,
                        const float* a_log, const float* dt_bias, const float* norm_weight, int col_a, int col_b, int col_gate,
                        int heads, int kv_heads, int dim, int vdim, float unit_eps, float norm_eps, int num_tokens, int num_rows,
                        cudaStream_t stream) {
  const T* proj = (const T*)proj_v;
  T* out = (T*)out_v;
  const int channels = 2 * kv_heads * dim + heads * vdim;
  const long long conv_offset = (long long)heads * dim * vdim;
  {
    const int warps = 4;
    const long long items = (long long)num_tokens * (2 * kv_heads + heads + 1);
    delta_prepare_kernel<T, DELTA_MAX_TAPS><<<(unsigned)((items + warps - 1) / warps), warps * 32, 0, stream>>>(
        proj, ld, conv_w, taps, state, slot_floats, conv_offset, token_row, q_start, slots, qkv, gates, a_log, dt_bias, col_a, col_b,
        heads, kv_heads, dim, vdim, unit_eps, num_tokens);
  }
  if (taps > 1) {
    const long long items = (long long)num_rows * channels;
    delta_conv_advance_kernel<T, DELTA_MAX_TAPS><<<(unsigned)((items + 127) / 128), 128, 0, stream>>>(
        proj, ld, taps, state, slot_floats, conv_offset, q_start, slots, channels, num_rows);
  }
  {
    // P lanes share a column: the fewest (a power of two, at least 4) that leave a lane at most 16 entries, so a block of
    // 128 threads owns 32 columns at most and the slices of vdim fill the device also with few heads.
    int lanes = 4;
    while (lanes < 32 && (dim + lanes - 1) / lanes > 16) lanes *= 2;
    const int per = (dim + lanes - 1) / lanes;
    int cols = 128 / lanes;
    while (cols > 1 && cols / 2 >= vdim) cols /= 2;
    dim3 grid((vdim + cols - 1) / cols, heads, num_rows);
    const int threads = cols * lanes;   // a multiple of 32 unless one warp holds all columns; shuffles stay inside groups of P lanes
#define PYLON_DELTA_RECURRENCE(N) \
    delta_recurrence_kernel<N><<<grid, threads < 32 ? 32 : threads, 0, stream>>>(qkv, gates, state, slot_floats, q_start, slots, o, heads, kv_heads, dim, vdim, lanes, cols)
    if (per <= 4) PYLON_DELTA_RECURRENCE(4);
    else if (per <= 8) PYLON_DELTA_RECURRENCE(8);
    else if (per <= 16) PYLON_DELTA_RECURRENCE(16);
    else PYLON_DELTA_RECURRENCE(32);
#undef PYLON_DELTA_RECURRENCE
  }
  {
    const int warps = 4;
    const long long items = (long long)num_tokens * heads;
    delta_gated_norm_kernel<T><<<(unsigned)((items + warps - 1) / warps), warps * 32, 0, stream>>>(
        o, proj, ld, col_gate, norm_weight, out, heads, vdim, norm_eps, num_tokens);
  }
  PYLON_CHECK_LAUNCH("gated_delta_rule");
}

// proj: [num_tokens, ld] with columns [q (kv_heads * dim) | k (kv_heads * dim) | v (heads * vdim) | ...] and the gate
// (heads * vdim), a and b (heads each) at the columns named.  state: float32 [slots, slot_floats], slot_floats >=
// heads * dim * vdim + (taps - 1) * channels.  qkv [T, channels], gates [T, 2 * heads], o [T, heads * vdim]: float32 work
// buffers.  out: [T, heads * vdim] in dtype.  Rows without tokens leave their slot as it is.
extern "C" int pylon_gated_delta_rule(const void* proj, long long ld, const float* conv_w, int taps, float* state,
                                      long long slot_floats, const int* token_row, const int* q_start, const int* slots, float* qkv,
                                      float* gates, float* o, void* out, const float* a_log, const float* dt_bias,
                                      const float* norm_weight, int col_a, int col_b, int col_gate, int heads, int kv_heads, int dim,
                                      int vdim, float unit_eps, float norm_eps, int num_tokens, int num_rows, int dtype,
                                      cudaStream_t stream) {
  if (num_tokens <= 0 || num_rows <= 0) return 0;
  if (heads < 1 || kv_heads < 1 || heads % kv_heads) PYLON_REFUSE("gated_delta_rule: %d heads over %d query/key heads", heads, kv_heads);
  if (dim < 1 || dim > 1024 || vdim < 1) PYLON_REFUSE("gated_delta_rule: dim %d (1 to 1024), vdim %d", dim, vdim);
  if (taps < 1 || taps > DELTA_MAX_TAPS) PYLON_REFUSE("gated_delta_rule: %d taps (1 to %d)", taps, DELTA_MAX_TAPS);
  if (heads > 65535 || num_rows > 65535) PYLON_REFUSE("gated_delta_rule: %d heads, %d rows", heads, num_rows);
  const long long needed = (long long)heads * dim * vdim + (long long)(taps - 1) * (2 * kv_heads * dim + heads * vdim);
  if (slot_floats < needed) PYLON_REFUSE("gated_delta_rule: a slot of %lld floats, %lld needed", slot_floats, needed);
#define PYLON_DELTA_ARGS proj, ld, conv_w, taps, state, slot_floats, token_row, q_start, slots, qkv, gates, o, out, a_log, dt_bias, \
    norm_weight, col_a, col_b, col_gate, heads, kv_heads, dim, vdim, unit_eps, norm_eps, num_tokens, num_rows, stream
  if (dtype == PYLON_DTYPE_F32) return launch_delta<float>(PYLON_DELTA_ARGS);
  if (dtype == PYLON_DTYPE_BF16) return launch_delta<__nv_bfloat16>(PYLON_DELTA_ARGS);
#undef PYLON_DELTA_ARGS
  PYLON_REFUSE("gated_delta_rule: unknown dtype %d", dtype);
}
