// Linear attention with a fixed decay per head ("lightning attention"), from its projections on.
//
// Per head, with q, k [dim] and v [vdim] of a token (silu of the projections, taken here in float32):
//   S <- decay * S + k v^T        (S [dim, vdim], float32, one per request and head, kept in the request's state slot,
//                                  column by column: entry (d, j) at j * dim + d, so that the lanes of a column read whole sectors)
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
//
// Long rows in segments (`segments` > 1: a row's tokens in runs of `seg_len`, each a block's walk of its own, so that a long prompt
// fills the device): segment 0 walks from the slot's state and leaves its end state there; a later segment g walks from zero and
// leaves what its own tokens wrote in parts[row, g - 1] (CARRY = false).  lightning_scan_kernel then chains the ends
// (S_g = decay^len_g S_(g-1) + part_g) and leaves in parts[row, g - 1] the state at the start of segment g; and the walk with
// CARRY = true adds to every token of a later segment what it reads of that state, decay^(i + 1) S^T q for the segment's token i.
template <bool CARRY>
__global__ void __launch_bounds__(LIGHTNING_THREADS, 4) lightning_recurrence_kernel(
    const float* __restrict__ qk, const float* __restrict__ v, float* __restrict__ state, long long slot_stride, const int* __restrict__ q_start,
    const int* __restrict__ slots, int num_slots, const float* __restrict__ decay, float* __restrict__ out, int heads, int dim, int vdim, int lanes,
    int seg_len, int segments, float* __restrict__ parts) {
  extern __shared__ __align__(16) float lightning_shared[];
  const int row_floats = 2 * lanes * LIGHTNING_LANE_PITCH;              // q and k of one token and head
  const int columns = LIGHTNING_THREADS / lanes;
  const int token_floats = row_floats + columns;                        // plus the block's slice of v
  float* buffers[2] = {lightning_shared, lightning_shared + LIGHTNING_TOKENS * token_floats};
  const int head = blockIdx.y, tid = threadIdx.x;
  const int walks = CARRY ? segments - 1 : segments;                     // blocks along z per row
  const int row = blockIdx.z / walks, segment = blockIdx.z % walks + (CARRY ? 1 : 0);
  int t0 = q_start[row], t1 = q_start[row + 1];
  if (segments > 1) {
    t0 += segment * seg_len;
    if (t1 > t0 + seg_len) t1 = t0 + seg_len;
  }
  if (t1 <= t0) return;   // a row without tokens (a step padded to a captured size), or a segment behind the row's end: nothing is touched
  const int slot = slots[row];
  if (slot < 0 || slot >= num_slots) return;
  const int part = tid % lanes;
  const int first_column = blockIdx.x * columns;
  const int column = first_column + tid / lanes;
  const bool live = column < vdim;
  const float g = decay[head];
  float* s_head = segment == 0 ? state + (size_t)slot * slot_stride + (size_t)head * dim * vdim
                               : parts + ((size_t)row * (segments - 1) + segment - 1) * ((size_t)heads * dim * vdim) + (size_t)head * dim * vdim;

  // a thread's units of a chunk's copies lie 128 apart: (token, unit) advance by fixed steps, no division in the loop
  const int chunks = row_floats / 4;
  const int qk_token_step = LIGHTNING_THREADS / chunks, qk_unit_step = LIGHTNING_THREADS % chunks;
  const int v_token_step = LIGHTNING_THREADS / columns;   // columns divides 128
  auto stage = [&](int c0, float* buffer) {
    const int count = t1 - c0 < LIGHTNING_TOKENS ? t1 - c0 : LIGHTNING_TOKENS;
    const float* from = qk + ((size_t)c0 * heads + head) * row_floats;
    for (int tt = tid / chunks, c = tid % chunks; tt < count;) {
      lightning_copy_16(buffer + tt * token_floats + c * 4, from + (size_t)tt * heads * row_floats + c * 4);
      tt += qk_token_step;
      c += qk_unit_step;
      if (c >= chunks) {
        c -= chunks;
        ++tt;
      }
    }
    const int c = tid % columns;
    const bool real = first_column + c < vdim;
    const float* v_from = v + ((size_t)c0 * heads + head) * vdim + (real ? first_column + c : 0);
    for (int tt = tid / columns; tt < count; tt += v_token_step)
      lightning_copy_4(buffer + tt * token_floats + row_floats + c, v_from + (size_t)tt * heads * vdim, real);
  };
  stage(t0, buffers[0]);
  asm volatile("cp.async.commit_group;\n" ::);

  float s[LIGHTNING_PER_LANE];
#pragma unroll
  for (int i = 0; i < LIGHTNING_PER_LANE; ++i) {
    const int d = i * lanes + part;
    s[i] = (live && d < dim && (CARRY || segment == 0)) ? s_head[(size_t)column * dim + d] : 0.f;   // a later segment's own walk starts from zero
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
      const float4* qq = reinterpret_cast<const float4*>(token + part * LIGHTNING_LANE_PITCH);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      if (CARRY) {
#pragma unroll
        for (int i = 0; i < LIGHTNING_PER_LANE / 4; ++i) {
          const float4 q4 = qq[i];
          s[4 * i + 0] *= g;
          s[4 * i + 1] *= g;
          s[4 * i + 2] *= g;
          s[4 * i + 3] *= g;
          acc[0] = fmaf(s[4 * i + 0], q4.x, acc[0]);
          acc[1] = fmaf(s[4 * i + 1], q4.y, acc[1]);
          acc[2] = fmaf(s[4 * i + 2], q4.z, acc[2]);
          acc[3] = fmaf(s[4 * i + 3], q4.w, acc[3]);
        }
      } else {
        const float value = token[row_floats + tid / lanes];
        const float4* kq = reinterpret_cast<const float4*>(token + lanes * LIGHTNING_LANE_PITCH + part * LIGHTNING_LANE_PITCH);
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
      }
      float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
      for (int offset = 1; offset < lanes; offset <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
      if (live && part == 0) out[(size_t)(c0 + tt) * heads * vdim + (size_t)head * vdim + column] = sum;   // CARRY: `out` is the buffer of what is carried in
    }
    __syncthreads();   // the buffer is free for the chunk after next
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
  if (live && !CARRY) {
#pragma unroll
    for (int i = 0; i < LIGHTNING_PER_LANE; ++i) {
      const int d = i * lanes + part;
      if (d < dim) s_head[(size_t)column * dim + d] = s[i];
    }
  }
}

// One thread per entry of a row's state: chains the segments' ends (see lightning_recurrence_kernel); the row's first threads also
// note for every token of the row which segment it is in.
__global__ void lightning_scan_kernel(float* __restrict__ state, long long slot_stride, const int* __restrict__ q_start, const int* __restrict__ slots,
                                      int num_slots, const float* __restrict__ decay, float* __restrict__ parts, int* __restrict__ token_segment, int heads,
                                      int dim, int vdim, int seg_len, int segments) {
  const int row = blockIdx.y;
  const int entries = heads * dim * vdim;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  const int t0 = q_start[row], tokens = q_start[row + 1] - t0;
  for (int t = e; t < tokens; t += gridDim.x * blockDim.x) token_segment[t0 + t] = t / seg_len;
  if (e >= entries) return;
  const int slot = slots[row];
  if (tokens <= seg_len || slot < 0 || slot >= num_slots) return;   // one segment: the walk left the end state in the slot
  const float g = decay[e / (dim * vdim)];
  const float whole = powf(g, (float)seg_len);
  float* mine = state + (size_t)slot * slot_stride + e;
  float s = *mine;
  for (int segment = 1; segment < segments && segment * seg_len < tokens; ++segment) {
    const int length = tokens - segment * seg_len;
    float* part = parts + ((size_t)row * (segments - 1) + segment - 1) * entries + e;
    const float own = *part;
    *part = s;
    s = fmaf(length >= seg_len ? whole : powf(g, (float)length), s, own);
  }
  *mine = s;
}

// y[t] = o[t] / sqrt(mean(o[t]^2) + eps) * weight * sigmoid(gate[t]) over the `width` concatenated head outputs of a token.
template <typename T>
__global__ void __launch_bounds__(512) sigmoid_gated_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ carried,
                                                                    const int* __restrict__ token_segment, const T* __restrict__ gate, long long gate_ld,
                                                                    const float* __restrict__ weight, T* __restrict__ out, int width, float eps) {
  // carried (optional): what a token of a later segment of a long row reads of the state before its segment, to be added to o;
  // token_segment[t] > 0 says that token t is such a token (only those rows of `carried` were written)
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const float* row = o + (size_t)t * width;
  const float* extra = carried != nullptr && token_segment[t] > 0 ? carried + (size_t)t * width : nullptr;
  float squares = 0.f;
#pragma unroll 4
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float x = row[i] + (extra ? extra[i] : 0.f);
    squares = fmaf(x, x, squares);
  }
  const float inv = rsqrtf(block_sum(squares, scratch) / width + eps);
#pragma unroll 4
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float gv = to_float<T>(gate[(size_t)t * gate_ld + i]);
    const float x = row[i] + (extra ? extra[i] : 0.f);
    out[(size_t)t * width + i] = from_float<T>(x * inv * weight[i] / (1.f + expf(-gv)));
  }
}

}  // namespace pylon

using namespace pylon;

// proj [T, ld]: the columns [q | k | v | gate] of a token start at q_col, k_col, v_col, gate_col; q and k hold heads x dim
// numbers, v and gate heads x vdim.  state [num_slots, heads, vdim, dim] float32 (a head's matrix column by column); rows: q_start [rows + 1], slots [rows].
// o [T, heads * vdim] float32 scratch; work: float32 scratch of pylon_lightning_work_floats numbers; y [T, heads * vdim] in
// the activation dtype.

constexpr int LIGHTNING_SEGMENT_FROM = 1024;    // rows from this many tokens on are cut into segments
constexpr int LIGHTNING_SEGMENT_LEAST = 128;    // of at least this many tokens
constexpr long long LIGHTNING_MAX_PART_FLOATS = 64LL << 20;

static int lightning_lanes(int dim) {
  int lanes = 1;
  while (lanes * LIGHTNING_PER_LANE < dim) lanes *= 2;
  return lanes;
}
static size_t lightning_shared_bytes(int lanes) {
  return (size_t)2 * LIGHTNING_TOKENS * (2 * lanes * LIGHTNING_LANE_PITCH + LIGHTNING_THREADS / lanes) * sizeof(float);
}
static bool lightning_configure() {
  static bool configured[MAX_DEVICES] = {};
  bool& done = configured[current_device_slot()];
  if (!done) {
    const int most = (int)lightning_shared_bytes(32);
    if (cudaFuncSetAttribute(lightning_recurrence_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) != cudaSuccess ||
        cudaFuncSetAttribute(lightning_recurrence_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, most) != cudaSuccess)
      return false;
    done = true;
  }
  return true;
}

// Into how many segments of how many tokens the longest row of a step is cut: as many as let one long row's walks fill the device
// once (what is resident at a time), each of at least 128 tokens.  In float32 the walk stays whole: there the order of every sum is
// to depend on the token's position only, not on where a step's portion starts.
static void lightning_segments(int rows, int max_q, int heads, int dim, int vdim, int dtype, int* segments, int* seg_len) {
  *segments = 1;
  *seg_len = max_q > 0 ? max_q : 1;
  if (dtype == PYLON_DTYPE_F32 || max_q < LIGHTNING_SEGMENT_FROM || !lightning_configure()) return;
  const int lanes = lightning_lanes(dim);
  const int columns = LIGHTNING_THREADS / lanes;
  int resident = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, lightning_recurrence_kernel<false>, LIGHTNING_THREADS, lightning_shared_bytes(lanes)) != cudaSuccess) return;
  const long long room = (long long)resident * multiprocessors();
  const long long walk_blocks = (long long)((vdim + columns - 1) / columns) * heads;
  long long count = room / walk_blocks;
  if (count > max_q / LIGHTNING_SEGMENT_LEAST) count = max_q / LIGHTNING_SEGMENT_LEAST;
  if (count < 2 || (long long)rows * (count - 1) * heads * dim * vdim > LIGHTNING_MAX_PART_FLOATS) return;
  *segments = (int)count;
  *seg_len = (int)(((max_q + count - 1) / count + LIGHTNING_TOKENS - 1) / LIGHTNING_TOKENS * LIGHTNING_TOKENS);
}

// work: silu of q, k, v of every token; behind it, for steps with long rows, what their later segments' tokens are handed from before
// their segment [T, heads * vdim], the later segments' states of every row, and the segment of every token (int32)
extern "C" long long pylon_lightning_work_floats(int num_tokens, int rows, int max_q, int heads, int dim, int vdim, int dtype) {
  int segments, seg_len;
  lightning_segments(rows, max_q, heads, dim, vdim, dtype, &segments, &seg_len);
  long long floats = (long long)num_tokens * heads * (2 * lightning_lanes(dim) * LIGHTNING_LANE_PITCH + vdim);
  if (segments > 1) floats += (long long)num_tokens * heads * vdim + (long long)rows * (segments - 1) * heads * dim * vdim + num_tokens;
  return floats;
}

extern "C" int pylon_lightning_attention(const void* proj, long long ld, int q_col, int k_col, int v_col, int gate_col, float* state,
                                         long long slot_stride, int num_slots, const int* q_start, const int* slots, int rows,
                                         const float* decay, const float* norm_weight, float eps, float* o, float* work, void* y, int num_tokens,
                                         int max_q, int heads, int dim, int vdim, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0 || rows <= 0) return 0;
  if (heads < 1 || dim < 1 || vdim < 1 || dim > LIGHTNING_MAX_DIM) PYLON_REFUSE("lightning_attention: %d heads of %d x %d (a head's dim is at most %d)", heads, dim, vdim, LIGHTNING_MAX_DIM);
  if (heads > 65535 || rows > 65535) PYLON_REFUSE("lightning_attention: %d heads, %d rows", heads, rows);
  if (dtype != PYLON_DTYPE_F32 && dtype != PYLON_DTYPE_BF16) PYLON_REFUSE("lightning_attention: unknown dtype %d", dtype);
  const int lanes = lightning_lanes(dim);
  const int columns = LIGHTNING_THREADS / lanes;
  if (!lightning_configure()) PYLON_REFUSE("lightning_attention: the shared memory of the widest head is not to be had");
  int segments, seg_len;
  lightning_segments(rows, max_q, heads, dim, vdim, dtype, &segments, &seg_len);
  if ((long long)rows * segments > 65535) PYLON_REFUSE("lightning_attention: %d rows in %d segments", rows, segments);
  const int width = heads * vdim;
  float* qk = work;
  float* v = work + (size_t)num_tokens * heads * 2 * lanes * LIGHTNING_LANE_PITCH;
  float* carried = v + (size_t)num_tokens * width;
  float* parts = carried + (size_t)num_tokens * width;
  int* token_segment = reinterpret_cast<int*>(parts + (size_t)rows * (segments - 1) * heads * dim * vdim);
  const size_t smem = lightning_shared_bytes(lanes);
  dim3 prepare_grid(num_tokens, heads);
  dim3 grid((vdim + columns - 1) / columns, heads, rows * segments);
  const int norm_threads = width >= 2048 ? 512 : (width >= 1024 ? 256 : 128);
  if (dtype == PYLON_DTYPE_F32)
    lightning_prepare_kernel<float><<<prepare_grid, LIGHTNING_THREADS, 0, stream>>>((const float*)proj, ld, q_col, k_col, v_col, qk, v, heads, dim, vdim, lanes);
  else
    lightning_prepare_kernel<__nv_bfloat16><<<prepare_grid, LIGHTNING_THREADS, 0, stream>>>((const __nv_bfloat16*)proj, ld, q_col, k_col, v_col, qk, v, heads, dim, vdim, lanes);
  lightning_recurrence_kernel<false><<<grid, LIGHTNING_THREADS, smem, stream>>>(qk, v, state, slot_stride, q_start, slots, num_slots, decay, o, heads, dim, vdim,
                                                                                 lanes, seg_len, segments, parts);
  if (segments > 1) {
    const int entries = heads * dim * vdim;
    lightning_scan_kernel<<<dim3((unsigned)((entries + 255) / 256), rows), 256, 0, stream>>>(state, slot_stride, q_start, slots, num_slots, decay, parts, token_segment,
                                                                                            heads, dim, vdim, seg_len, segments);
    grid.z = rows * (segments - 1);
    lightning_recurrence_kernel<true><<<grid, LIGHTNING_THREADS, smem, stream>>>(qk, v, state, slot_stride, q_start, slots, num_slots, decay, carried, heads, dim, vdim,
                                                                                  lanes, seg_len, segments, parts);
  }
  const float* extra = segments > 1 ? carried : nullptr;
  if (dtype == PYLON_DTYPE_F32)
    sigmoid_gated_rmsnorm_kernel<float><<<num_tokens, norm_threads, 0, stream>>>(o, extra, token_segment, (const float*)proj + gate_col, ld, norm_weight, (float*)y, width, eps);
  else
    sigmoid_gated_rmsnorm_kernel<__nv_bfloat16><<<num_tokens, norm_threads, 0, stream>>>(o, extra, token_segment, (const __nv_bfloat16*)proj + gate_col, ld, norm_weight,
                                                                                          (__nv_bfloat16*)y, width, eps);
  PYLON_CHECK_LAUNCH("lightning_attention");
}
