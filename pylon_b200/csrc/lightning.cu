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
// lie in the registers of P = 2^n lanes (16 entries each, entry i of lane p being d = i * P + p), which add up their
// parts of the read-out by shuffles.  A first kernel takes silu of q, k and v of all tokens at once, in float32 and in the
// order the walk reads them, so that the walk itself only copies (cp.async, 16 tokens at a time, two buffers) and multiplies.
#include "common.cuh"

namespace pylon {

constexpr int LIGHTNING_THREADS = 128;
constexpr int LIGHTNING_PER_LANE = 16;    // entries of a column in one lane's registers
constexpr int LIGHTNING_LANE_PITCH = 20;  // floats between two lanes' entries in shared memory: 16-byte reads without bank conflicts
constexpr int LIGHTNING_TOKENS = 16;      // tokens staged at a time
constexpr int LIGHTNING_MAX_DIM = 512;    // 32 lanes of 16 entries

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }

__device__ __forceinline__ void lightning_copy_4(void* smem, const void* global, bool valid) {
  const unsigned address = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 4 : 0;   // 0: the word is filled with zeros
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(address), "l"(global), "r"(bytes));
}

__device__ __forceinline__ void lightning_copy_16(void* smem, const void* global) {
  const unsigned address = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(address), "l"(global));
}

// silu of a step's q, k and v in float32, laid out as the walk reads them: qk [T, heads, 2, lanes * PITCH] with entry d of a
// head at (d % lanes) * PITCH + d / lanes (zeros where d >= dim and in the padding), v [T, heads, vdim].  One block per (token, head).
template <typename T>
__global__ void __launch_bounds__(LIGHTNING_THREADS) lightning_prepare_kernel(const T* __restrict__ proj, long long ld, int q_col, int k_col, int v_col,
                                                                             float* __restrict__ qk, float* __restrict__ v, int heads, int dim, int vdim,
                                                                             int lanes) {
  const int t = blockIdx.x, head = blockIdx.y;
  const int row = lanes * LIGHTNING_LANE_PITCH;
  const T* src = proj + (size_t)t * ld + (size_t)head * dim;
  float* dst = qk + ((size_t)t * heads + head) * 2 * row;
  for (int e = threadIdx.x; e < row; e += LIGHTNING_THREADS) {
    const int lane = e / LIGHTNING_LANE_PITCH, i = e % LIGHTNING_LANE_PITCH;
    const int d = i * lanes + lane;
    const bool real = i < LIGHTNING_PER_LANE && d < dim;
    dst[e] = real ? silu_f(to_float<T>(src[q_col + d])) : 0.f;
    dst[row + e] = real ? silu_f(to_float<T>(src[k_col + d])) : 0.f;
  }
  const T* vsrc = proj + (size_t)t * ld + v_col + (size_t)head * vdim;
  float* vdst = v + ((size_t)t * heads + head) * vdim;
  for (int e = threadIdx.x; e < vdim; e += LIGHTNING_THREADS) vdst[e] = silu_f(to_float<T>(vsrc[e]));
}

// The walk.  A block owns 128 / lanes columns of one head of one request; `lanes` (a power of two) lanes share a column, each with
// 16 of its entries in registers.  Tokens come 16 at a time by cp.async into one of two buffers while the other is walked.
__global__ void __launch_bounds__(LIGHTNING_THREADS) lightning_recurrence_kernel(
    const float* __restrict__ qk, const float* __restrict__ v, float* __restrict__ state, long long slot_stride, const int* __restrict__ q_start,
    const int* __restrict__ slots, int num_slots, const float* __restrict__ decay, float* __restrict__ out, int heads, int dim, int vdim, int lanes) {
  extern __shared__ __align__(16) float lightning_shared[];
  const int row_floats = 2 * lanes * LIGHTNING_LANE_PITCH;              // q and k of one token and head
  const int columns = LIGHTNING_THREADS / lanes;
  const int token_floats = row_floats + columns;                        // plus the block's slice of v
  float* buffers[2] = {lightning_shared, lightning_shared + LIGHTNING_TOKENS * token_floats};
  const int row = blockIdx.z, head = blockIdx.y, tid = threadIdx.x;
  const int t0 = q_start[row], t1 = q_start[row + 1];
  if (t1 <= t0) return;   // a row without tokens (a step padded to a captured size): its slot stays as it is
  const int slot = slots[row];
  if (slot < 0 || slot >= num_slots) return;
  const int part = tid % lanes;
  const int first_column = blockIdx.x * columns;
  const int column = first_column + tid / lanes;
  const bool live = column < vdim;
  const float g = decay[head];
  float* s_head = state + (size_t)slot * slot_stride + (size_t)head * dim * vdim;

  auto stage = [&](int c0, float* buffer) {
    const int count = t1 - c0 < LIGHTNING_TOKENS ? t1 - c0 : LIGHTNING_TOKENS;
    const int chunks = row_floats / 4;
    for (int e = tid; e < count * chunks; e += LIGHTNING_THREADS) {
      const int tt = e / chunks, c = e % chunks;
      lightning_copy_16(buffer + tt * token_floats + c * 4, qk + ((size_t)(c0 + tt) * heads + head) * row_floats + c * 4);
    }
    for (int e = tid; e < count * columns; e += LIGHTNING_THREADS) {
      const int tt = e / columns, c = e % columns;
      const bool real = first_column + c < vdim;
      lightning_copy_4(buffer + tt * token_floats + row_floats + c, v + ((size_t)(c0 + tt) * heads + head) * vdim + (real ? first_column + c : 0), real);
    }
  };
  stage(t0, buffers[0]);
  asm volatile("cp.async.commit_group;\n" ::);

  float s[LIGHTNING_PER_LANE];
#pragma unroll
  for (int i = 0; i < LIGHTNING_PER_LANE; ++i) {
    const int d = i * lanes + part;
    s[i] = (live && d < dim) ? s_head[(size_t)d * vdim + column] : 0.f;
  }
  int turn = 0;
  for (int c0 = t0; c0 < t1; c0 += LIGHTNING_TOKENS, turn ^= 1) {
    const int count = t1 - c0 < LIGHTNING_TOKENS ? t1 - c0 : LIGHTNING_TOKENS;
    if (c0 + LIGHTNING_TOKENS < t1) stage(c0 + LIGHTNING_TOKENS, buffers[turn ^ 1]);
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group 1;\n" ::);
    __syncthreads();
    const float* buffer = buffers[turn];
    // unrolled: a token's shuffles and its store overlap the next tokens' products (the state is the only chain from token to token)
#pragma unroll 4
    for (int tt = 0; tt < count; ++tt) {
      const float* token = buffer + tt * token_floats;
      const float value = token[row_floats + tid / lanes];
      const float4* qq = reinterpret_cast<const float4*>(token + part * LIGHTNING_LANE_PITCH);
      const float4* kq = reinterpret_cast<const float4*>(token + lanes * LIGHTNING_LANE_PITCH + part * LIGHTNING_LANE_PITCH);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < LIGHTNING_PER_LANE / 4; ++i) {
        const float4 k4 = kq[i], q4 = qq[i];
        s[4 * i + 0] = fmaf(g, s[4 * i + 0], k4.x * value);
        s[4 * i + 1] = fmaf(g, s[4 * i + 1], k4.y * value);
        s[4 * i + 2] = fmaf(g, s[4 * i + 2], k4.z * value);
        s[4 * i + 3] = fmaf(g, s[4 * i + 3], k4.w * value);
        acc[0] = fmaf(s[4 * i + 0], q4.x, acc[0]);
        acc[1] = fmaf(s[4 * i + 1], q4.y, acc[1]);
        acc[2] = fmaf(s[4 * i + 2], q4.z, acc[2]);
        acc[3] = fmaf(s[4 * i + 3], q4.w, acc[3]);
      }
      float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
      for (int offset = 1; offset < lanes; offset <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
      if (live && part == 0) out[(size_t)(c0 + tt) * heads * vdim + (size_t)head * vdim + column] = sum;
    }
    __syncthreads();   // the buffer is free for the chunk after next
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
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
// o [T, heads * vdim] float32 scratch; work: float32 scratch of pylon_lightning_work_floats numbers; y [T, heads * vdim] in
// the activation dtype.
static int lightning_lanes(int dim) {
  int lanes = 1;
  while (lanes * LIGHTNING_PER_LANE < dim) lanes *= 2;
  return lanes;
}

extern "C" long long pylon_lightning_work_floats(int num_tokens, int heads, int dim, int vdim) {
  return (long long)num_tokens * heads * (2 * lightning_lanes(dim) * LIGHTNING_LANE_PITCH + vdim);
}

extern "C" int pylon_lightning_attention(const void* proj, long long ld, int q_col, int k_col, int v_col, int gate_col, float* state,
                                         long long slot_stride, int num_slots, const int* q_start, const int* slots, int rows,
                                         const float* decay, const float* norm_weight, float eps, float* o, float* work, void* y, int num_tokens,
                                         int heads, int dim, int vdim, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0 || rows <= 0) return 0;
  if (heads < 1 || dim < 1 || vdim < 1 || dim > LIGHTNING_MAX_DIM) PYLON_REFUSE("lightning_attention: %d heads of %d x %d (a head's dim is at most %d)", heads, dim, vdim, LIGHTNING_MAX_DIM);
  if (heads > 65535 || rows > 65535) PYLON_REFUSE("lightning_attention: %d heads, %d rows", heads, rows);
  if (dtype != PYLON_DTYPE_F32 && dtype != PYLON_DTYPE_BF16) PYLON_REFUSE("lightning_attention: unknown dtype %d", dtype);
  const int lanes = lightning_lanes(dim);
  const int columns = LIGHTNING_THREADS / lanes;
  float* qk = work;
  float* v = work + (size_t)num_tokens * heads * 2 * lanes * LIGHTNING_LANE_PITCH;
  const size_t smem = (size_t)2 * LIGHTNING_TOKENS * (2 * lanes * LIGHTNING_LANE_PITCH + columns) * sizeof(float);
  static bool configured[MAX_DEVICES] = {};
  bool& done = configured[current_device_slot()];
  if (!done) {
    if (cudaFuncSetAttribute(lightning_recurrence_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * LIGHTNING_TOKENS * (2 * 32 * LIGHTNING_LANE_PITCH + 4) * 4) != cudaSuccess)
      PYLON_REFUSE("lightning_attention: the shared memory of the widest head is not to be had");
    done = true;
  }
  dim3 prepare_grid(num_tokens, heads);
  dim3 grid((vdim + columns - 1) / columns, heads, rows);
  const int width = heads * vdim;
  const int norm_threads = width >= 1024 ? 256 : 128;
  if (dtype == PYLON_DTYPE_F32)
    lightning_prepare_kernel<float><<<prepare_grid, LIGHTNING_THREADS, 0, stream>>>((const float*)proj, ld, q_col, k_col, v_col, qk, v, heads, dim, vdim, lanes);
  else
    lightning_prepare_kernel<__nv_bfloat16><<<prepare_grid, LIGHTNING_THREADS, 0, stream>>>((const __nv_bfloat16*)proj, ld, q_col, k_col, v_col, qk, v, heads, dim, vdim, lanes);
  lightning_recurrence_kernel<<<grid, LIGHTNING_THREADS, smem, stream>>>(qk, v, state, slot_stride, q_start, slots, num_slots, decay, o, heads, dim, vdim, lanes);
  if (dtype == PYLON_DTYPE_F32)
    sigmoid_gated_rmsnorm_kernel<float><<<num_tokens, norm_threads, 0, stream>>>(o, (const float*)proj + gate_col, ld, norm_weight, (float*)y, width, eps);
  else
    sigmoid_gated_rmsnorm_kernel<__nv_bfloat16><<<num_tokens, norm_threads, 0, stream>>>(o, (const __nv_bfloat16*)proj + gate_col, ld, norm_weight,
                                                                                          (__nv_bfloat16*)y, width, eps);
  PYLON_CHECK_LAUNCH("lightning_attention");
}
