// Linear attention with a fixed decay per head ("lightning attention"), from its projections on.
//
// Per head, with q, k [dim] and v [vdim] of a token (silu of the projections, taken here in float32):
//   S <- decay * S + k v^T        (S [dim, vdim], float32, one per request and head, kept in the request's state slot)
//   o  = S^T q                    (the read-out sees the token's own write)
// and then, over the concatenated heads of a token: y = o / sqrt(mean(o^2) + eps) * weight * sigmoid(gate).
//
// The columns of S do not depend on each other, so a block owns a slice of the columns of one head of one request and
// walks the request's tokens of this step in order: prompt portions and single decoded tokens are the same kernel, and
// what a token reads does not depend on how the prompt was cut or what else is in the step.  A column's `dim` entries
// lie in the registers of P = 2^n lanes (32 entries each, entry i of lane p being d = i * P + p), which add up their
// parts of the read-out by shuffles.  Tokens come 16 at a time through shared memory, silu applied on the way.
#include "common.cuh"

namespace pylon {

constexpr int LIGHTNING_THREADS = 128;
constexpr int LIGHTNING_PER_LANE = 32;    // entries of a column in one lane's registers
constexpr int LIGHTNING_LANE_PITCH = 36;  // floats between two lanes' entries in shared memory: 16-byte reads without bank conflicts
constexpr int LIGHTNING_TOKENS = 16;      // tokens staged at a time
constexpr int LIGHTNING_MAX_DIM = 256;

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(LIGHTNING_THREADS) lightning_recurrence_kernel(
    const T* __restrict__ proj, long long ld, int q_col, int k_col, int v_col, float* __restrict__ state,
    long long slot_stride, const int* __restrict__ q_start, const int* __restrict__ slots, int num_slots,
    const float* __restrict__ decay, float* __restrict__ out, int heads, int dim, int vdim, int lanes) {
  __shared__ __align__(16) float qs[LIGHTNING_TOKENS][LIGHTNING_MAX_DIM / LIGHTNING_PER_LANE * LIGHTNING_LANE_PITCH];
  __shared__ __align__(16) float ks[LIGHTNING_TOKENS][LIGHTNING_MAX_DIM / LIGHTNING_PER_LANE * LIGHTNING_LANE_PITCH];
  __shared__ float vs[LIGHTNING_TOKENS][LIGHTNING_THREADS];
  const int row = blockIdx.z, head = blockIdx.y, tid = threadIdx.x;
  const int t0 = q_start[row], t1 = q_start[row + 1];
  if (t1 <= t0) return;   // a row without tokens (a step padded to a captured size): its slot stays as it is
  const int slot = slots[row];
  if (slot < 0 || slot >= num_slots) return;
  const int columns = LIGHTNING_THREADS / lanes;
  const int part = tid % lanes;
  const int column = blockIdx.x * columns + tid / lanes;
  const bool live = column < vdim;
  const float g = decay[head];
  float* s_head = state + (size_t)slot * slot_stride + (size_t)head * dim * vdim;

  float s[LIGHTNING_PER_LANE];
#pragma unroll
  for (int i = 0; i < LIGHTNING_PER_LANE; ++i) {
    const int d = i * lanes + part;
    s[i] = (live && d < dim) ? s_head[(size_t)d * vdim + column] : 0.f;
  }
  const int padded = lanes * LIGHTNING_PER_LANE;
  for (int c0 = t0; c0 < t1; c0 += LIGHTNING_TOKENS) {
    const int count = t1 - c0 < LIGHTNING_TOKENS ? t1 - c0 : LIGHTNING_TOKENS;
    __syncthreads();
    for (int e = tid; e < count * padded; e += LIGHTNING_THREADS) {
      const int tt = e / padded, d = e % padded;
      const T* src = proj + (size_t)(c0 + tt) * ld + (size_t)head * dim + d;
      const int where = (d % lanes) * LIGHTNING_LANE_PITCH + d / lanes;
      qs[tt][where] = d < dim ? silu_f(to_float<T>(src[q_col])) : 0.f;
      ks[tt][where] = d < dim ? silu_f(to_float<T>(src[k_col])) : 0.f;
    }
    for (int e = tid; e < count * columns; e += LIGHTNING_THREADS) {
      const int tt = e / columns, c = e % columns;
      const int col = blockIdx.x * columns + c;
      vs[tt][c] = col < vdim ? silu_f(to_float<T>(proj[(size_t)(c0 + tt) * ld + v_col + (size_t)head * vdim + col])) : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < count; ++tt) {
      const float v = vs[tt][tid / lanes];
      const float4* kq = reinterpret_cast<const float4*>(&ks[tt][part * LIGHTNING_LANE_PITCH]);
      const float4* qq = reinterpret_cast<const float4*>(&qs[tt][part * LIGHTNING_LANE_PITCH]);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < LIGHTNING_PER_LANE / 4; ++i) {
        const float4 k4 = kq[i], q4 = qq[i];
        s[4 * i + 0] = fmaf(g, s[4 * i + 0], k4.x * v);
        s[4 * i + 1] = fmaf(g, s[4 * i + 1], k4.y * v);
        s[4 * i + 2] = fmaf(g, s[4 * i + 2], k4.z * v);
        s[4 * i + 3] = fmaf(g, s[4 * i + 3], k4.w * v);
        acc[0] = fmaf(s[4 * i + 0], q4.x, acc[0]);
        acc[1] = fmaf(s[4 * i + 1], q4.y, acc[1]);
        acc[2] = fmaf(s[4 * i + 2], q4.z, acc[2]);
        acc[3] = fmaf(s[4 * i + 3], q4.w, acc[3]);
      }
      float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
      for (int offset = 1; offset < lanes; offset <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
      if (live && part == 0) out[(size_t)(c0 + tt) * heads * vdim + (size_t)head * vdim + column] = sum;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < LIGHTNING_PER_LANE; ++i) {
      const int d = i * lanes + part;
      if (d < dim) s_head[(size_t)d * vdim + column] = s[i];
    }
  }
}

// y[t] = o[t] / sqrt(mean(o[t]^2) + eps) * weight * sigmoid(gate[t]) over the `width` concatenated head outputs of a token.
template <typename T>
__global__ void __launch_bounds__(256) sigmoid_gated_rmsnorm_kernel(const float* __restrict__ o, const T* __restrict__ gate, long long gate_ld,
                                                                    const float* __restrict__ weight, T* __restrict__ out, int width, float eps) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const float* row = o + (size_t)t * width;
  float squares = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) squares = fmaf(row[i], row[i], squares);
  const float inv = rsqrtf(block_sum(squares, scratch) / width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float gv = to_float<T>(gate[(size_t)t * gate_ld + i]);
    out[(size_t)t * width + i] = from_float<T>(row[i] * inv * weight[i] / (1.f + expf(-gv)));
  }
}

}  // namespace pylon

using namespace pylon;

// proj [T, ld]: the columns [q | k | v | gate] of a token start at q_col, k_col, v_col, gate_col; q and k hold heads x dim
// numbers, v and gate heads x vdim.  state [num_slots, heads, dim, vdim] float32; rows: q_start [rows + 1], slots [rows].
// o [T, heads * vdim] float32 scratch; y [T, heads * vdim] in the activation dtype.
extern "C" int pylon_lightning_attention(const void* proj, long long ld, int q_col, int k_col, int v_col, int gate_col, float* state,
                                         long long slot_stride, int num_slots, const int* q_start, const int* slots, int rows,
                                         const float* decay, const float* norm_weight, float eps, float* o, void* y, int num_tokens,
                                         int heads, int dim, int vdim, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0 || rows <= 0) return 0;
  if (heads < 1 || dim < 1 || vdim < 1 || dim > LIGHTNING_MAX_DIM) PYLON_REFUSE("lightning_attention: %d heads of %d x %d (a head's dim is at most %d)", heads, dim, vdim, LIGHTNING_MAX_DIM);
  if (heads > 65535 || rows > 65535) PYLON_REFUSE("lightning_attention: %d heads, %d rows", heads, rows);
  int lanes = 1;
  while (lanes * LIGHTNING_PER_LANE < dim) lanes *= 2;
  const int columns = LIGHTNING_THREADS / lanes;
  dim3 grid((vdim + columns - 1) / columns, heads, rows);
  const int width = heads * vdim;
  const int norm_threads = width >= 1024 ? 256 : 128;
  if (dtype == PYLON_DTYPE_F32) {
    lightning_recurrence_kernel<float><<<grid, LIGHTNING_THREADS, 0, stream>>>((const float*)proj, ld, q_col, k_col, v_col, state, slot_stride, q_start,
                                                                                slots, num_slots, decay, o, heads, dim, vdim, lanes);
    sigmoid_gated_rmsnorm_kernel<float><<<num_tokens, norm_threads, 0, stream>>>(o, (const float*)proj + gate_col, ld, norm_weight, (float*)y, width, eps);
  } else if (dtype == PYLON_DTYPE_BF16) {
    lightning_recurrence_kernel<__nv_bfloat16><<<grid, LIGHTNING_THREADS, 0, stream>>>((const __nv_bfloat16*)proj, ld, q_col, k_col, v_col, state, slot_stride,
                                                                                        q_start, slots, num_slots, decay, o, heads, dim, vdim, lanes);
    sigmoid_gated_rmsnorm_kernel<__nv_bfloat16><<<num_tokens, norm_threads, 0, stream>>>(o, (const __nv_bfloat16*)proj + gate_col, ld, norm_weight,
                                                                                          (__nv_bfloat16*)y, width, eps);
  } else {
    PYLON_REFUSE("lightning_attention: unknown dtype %d", dtype);
  }
  PYLON_CHECK_LAUNCH("lightning_attention");
}
