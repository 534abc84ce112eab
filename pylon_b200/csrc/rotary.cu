// What stands between an attention mixer's projections and its attention, for the forms the fused
// kernels of elementwise.cu are not written for: biases, rotation of part of a head, either layout of
// the rotated pairs, the per-head norm before or after the rotation and with or without a weight,
// values of another width than the keys, and a latent row per token in place of keys and values.
//
// A rotation turns the pair (u, v) of a head at position p into (u cos a - v sin a, v cos a + u sin a);
// a = p * f_i comes as float32 tables cos/sin [positions, rot / 2] (any scaling of the frequencies, and
// any factor on cos and sin, is in the tables).  Layout 0 pairs element i with i + rot / 2, layout 1
// element 2 i with 2 i + 1, i < rot / 2; elements from `rot` on pass unchanged.  All arithmetic is float32.
#include "common.cuh"

namespace pylon {

constexpr int ROTARY_THREADS = 128;
constexpr int ROTARY_WARPS = ROTARY_THREADS / 32;

// Rotates buf[0 .. rot) in place; one lane owns a pair.  The caller orders the warp before and after.
__device__ __forceinline__ void rotate_pairs(float* buf, const float* __restrict__ cos_row, const float* __restrict__ sin_row, int rot, int layout, int lane) {
  const int half = rot >> 1;
  for (int i = lane; i < half; i += 32) {
    const int a = layout ? 2 * i : i, b = layout ? 2 * i + 1 : i + half;
    const float c = cos_row[i], s = sin_row[i], u = buf[a], v = buf[b];
    buf[a] = u * c - v * s;
    buf[b] = v * c + u * s;
  }
}

// buf[0 .. n) divided by its root mean square, times weight (or 1).
__device__ __forceinline__ void unit_rms(float* buf, int n, const float* __restrict__ weight, float eps, int lane) {
  float squares = 0.f;
  for (int e = lane; e < n; e += 32) squares = fmaf(buf[e], buf[e], squares);
  const float inv = rsqrtf(warp_sum(squares) / n + eps);
  for (int e = lane; e < n; e += 32) buf[e] *= weight ? inv * weight[e] : inv;
}

// One warp per (token, head of q, k or v).  qkv [T, ld] holds [q: nq x d | k: nkv x d | v: nkv x dv] per token; q is
// written back in place, k and v go into the token's slot of its pages.  norm_mode 0: no norm of q and k; 1: before the
// rotation; 2: after it.
template <typename T>
__global__ void __launch_bounds__(ROTARY_THREADS) qkv_rotate_write_kernel(
    T* __restrict__ qkv, long long ld, const float* __restrict__ bias, const float* __restrict__ cos_table, const float* __restrict__ sin_table,
    int rot, int layout, int table_positions, int norm_mode, const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
    const int* __restrict__ positions, const int* __restrict__ token_row, const int* __restrict__ block_table, int table_width, int page_size,
    T* __restrict__ k_pages, T* __restrict__ v_pages, int num_pages, int nq, int nkv, int d, int dv, int num_tokens, int* __restrict__ error_word) {
  extern __shared__ float rotary_shared[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int widest = d > dv ? d : dv;
  float* buf = rotary_shared + (size_t)warp * widest;
  const int per_token = nq + 2 * nkv;
  const long long item = (long long)blockIdx.x * ROTARY_WARPS + warp;
  if (item >= (long long)num_tokens * per_token) return;
  const int t = (int)(item / per_token), hh = (int)(item % per_token);
  const int row = token_row[t];
  if (row < 0) return;   // a padding token: nothing of it is kept
  const int pos = positions[t];
  const bool is_q = hh < nq, is_v = hh >= nq + nkv;
  const int width = is_v ? dv : d;
  const int column = is_q ? hh * d : (is_v ? (nq + nkv) * d + (hh - nq - nkv) * dv : hh * d);
  T* src = qkv + (size_t)t * ld + column;
  for (int e = lane; e < width; e += 32) buf[e] = to_float<T>(src[e]) + (bias ? bias[column + e] : 0.f);
  __syncwarp();
  if (!is_v) {
    const float* weight = is_q ? q_weight : k_weight;
    if (norm_mode == 1) {
      unit_rms(buf, d, weight, eps, lane);
      __syncwarp();
    }
    if (rot > 0 && pos < table_positions) {
      rotate_pairs(buf, cos_table + (size_t)pos * (rot >> 1), sin_table + (size_t)pos * (rot >> 1), rot, layout, lane);
      __syncwarp();
    }
    if (norm_mode == 2) {
      unit_rms(buf, d, weight, eps, lane);
      __syncwarp();
    }
  }
  T* dst = src;
  if (!is_q) {
    const int logical = pos / page_size;
    const int page = logical < table_width ? block_table[(size_t)row * table_width + logical] : -1;
    if (page < 0 || page >= num_pages) {
      if (lane == 0 && error_word) atomicMax(error_word, PYLON_ERROR_BAD_PAGE);
      return;
    }
    const int head = is_v ? hh - nq - nkv : hh - nq;
    dst = (is_v ? v_pages : k_pages) + (((size_t)page * nkv + head) * page_size + pos % page_size) * width;
  }
  for (int e = lane; e < width; e += 32) dst[e] = from_float<T>(buf[e]);
}

// One block per token.  down [T, ld] holds [query latent: q_rank | key/value latent: kv_rank | shared rotated key part: rot_dim].
// cq [T, q_rank] = RMS norm of the query latent times q_weight; the token's one cache row [kv_rank + rot_dim] = RMS norm of the
// key/value latent times kv_weight, then the rotated key part (its first `rot` elements rotated, not normed).
template <typename T>
__global__ void __launch_bounds__(ROTARY_THREADS) latent_norm_rotate_write_kernel(
    const T* __restrict__ down, long long ld, T* __restrict__ cq, const float* __restrict__ q_weight, const float* __restrict__ kv_weight, float eps,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, int rot, int layout, int table_positions,
    const int* __restrict__ positions, const int* __restrict__ token_row, const int* __restrict__ block_table, int table_width, int page_size,
    T* __restrict__ pages, int num_pages, int q_rank, int kv_rank, int rot_dim, int* __restrict__ error_word) {
  extern __shared__ float rotary_shared[];
  float* scratch = rotary_shared;        // [34]
  float* staged = rotary_shared + 34;    // [q_rank + kv_rank + rot_dim]: the token's row, read from global memory once
  float* turned = staged + q_rank + kv_rank;
  const int t = blockIdx.x, tid = threadIdx.x;
  const int row = token_row[t];
  if (row < 0) return;
  const int pos = positions[t];
  const T* src = down + (size_t)t * ld;
  const int total = q_rank + kv_rank + rot_dim;
#pragma unroll 4
  for (int e = tid; e < total; e += ROTARY_THREADS) staged[e] = to_float<T>(src[e]);
  const int logical = pos / page_size;
  const int page = logical < table_width ? block_table[(size_t)row * table_width + logical] : -1;
  __syncthreads();
  float q_squares = 0.f, kv_squares = 0.f;
  for (int e = tid; e < q_rank; e += ROTARY_THREADS) q_squares = fmaf(staged[e], staged[e], q_squares);
  for (int e = tid; e < kv_rank; e += ROTARY_THREADS) kv_squares = fmaf(staged[q_rank + e], staged[q_rank + e], kv_squares);
  const float q_inv = rsqrtf(block_sum(q_squares, scratch) / (q_rank > 0 ? q_rank : 1) + eps);
  const float kv_inv = rsqrtf(block_sum(kv_squares, scratch) / kv_rank + eps);
  for (int e = tid; e < q_rank; e += ROTARY_THREADS) cq[(size_t)t * q_rank + e] = from_float<T>(staged[e] * q_inv * q_weight[e]);
  if (tid < 32 && rot > 0 && pos < table_positions)
    rotate_pairs(turned, cos_table + (size_t)pos * (rot >> 1), sin_table + (size_t)pos * (rot >> 1), rot, layout, tid);
  __syncthreads();
  if (page < 0 || page >= num_pages) {
    if (tid == 0 && error_word) atomicMax(error_word, PYLON_ERROR_BAD_PAGE);
    return;
  }
  T* dst = pages + ((size_t)page * page_size + pos % page_size) * (kv_rank + rot_dim);
  for (int e = tid; e < kv_rank; e += ROTARY_THREADS) dst[e] = from_float<T>(staged[q_rank + e] * kv_inv * kv_weight[e]);
  for (int e = tid; e < rot_dim; e += ROTARY_THREADS) dst[kv_rank + e] = from_float<T>(turned[e]);
}

// One warp per (token, head): dst[t, h, 0 .. width) = src[t, h, 0 .. width) with its first `rot` elements rotated.
template <typename T>
__global__ void __launch_bounds__(ROTARY_THREADS) rotate_heads_kernel(
    const T* __restrict__ src, long long src_token_stride, long long src_head_stride, T* __restrict__ dst, long long dst_token_stride,
    long long dst_head_stride, const float* __restrict__ cos_table, const float* __restrict__ sin_table, int rot, int layout, int table_positions,
    const int* __restrict__ positions, int heads, int width, int num_tokens) {
  extern __shared__ float rotary_shared[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* buf = rotary_shared + (size_t)warp * width;
  const long long item = (long long)blockIdx.x * ROTARY_WARPS + warp;
  if (item >= (long long)num_tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item % heads);
  const int pos = positions[t];
  const T* from = src + (size_t)t * src_token_stride + (size_t)h * src_head_stride;
  for (int e = lane; e < width; e += 32) buf[e] = to_float<T>(from[e]);
  __syncwarp();
  if (rot > 0 && pos >= 0 && pos < table_positions) rotate_pairs(buf, cos_table + (size_t)pos * (rot >> 1), sin_table + (size_t)pos * (rot >> 1), rot, layout, lane);
  __syncwarp();
  T* to = dst + (size_t)t * dst_token_stride + (size_t)h * dst_head_stride;
  for (int e = lane; e < width; e += 32) to[e] = from_float<T>(buf[e]);
}

}  // namespace pylon

using namespace pylon;

extern "C" int pylon_qkv_rotate_write(void* qkv, long long ld, const float* bias, const float* cos_table, const float* sin_table, int rot, int layout,
                                      int table_positions, int norm_mode, const float* q_weight, const float* k_weight, float eps, const int* positions,
                                      const int* token_row, const int* block_table, int table_width, int page_size, void* k_pages, void* v_pages,
                                      int num_pages, int nq, int nkv, int d, int dv, int num_tokens, int dtype, int* error_word, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (nq < 1 || nkv < 1 || d < 1 || dv < 1 || d > 2048 || dv > 2048) PYLON_REFUSE("qkv_rotate_write: %d / %d heads of %d and %d", nq, nkv, d, dv);
  if (rot < 0 || rot > d || rot % 2 || (rot > 0 && (!cos_table || !sin_table))) PYLON_REFUSE("qkv_rotate_write: %d rotated elements of %d", rot, d);
  if (norm_mode < 0 || norm_mode > 2 || page_size < 1 || table_width < 1) PYLON_REFUSE("qkv_rotate_write: norm mode %d, page size %d, table width %d", norm_mode, page_size, table_width);
  const long long items = (long long)num_tokens * (nq + 2 * nkv);
  const unsigned blocks = (unsigned)((items + ROTARY_WARPS - 1) / ROTARY_WARPS);
  const size_t smem = (size_t)ROTARY_WARPS * (d > dv ? d : dv) * sizeof(float);
  if (dtype == PYLON_DTYPE_F32)
    qkv_rotate_write_kernel<float><<<blocks, ROTARY_THREADS, smem, stream>>>(
        (float*)qkv, ld, bias, cos_table, sin_table, rot, layout, table_positions, norm_mode, q_weight, k_weight, eps, positions, token_row, block_table,
        table_width, page_size, (float*)k_pages, (float*)v_pages, num_pages, nq, nkv, d, dv, num_tokens, error_word);
  else if (dtype == PYLON_DTYPE_BF16)
    qkv_rotate_write_kernel<__nv_bfloat16><<<blocks, ROTARY_THREADS, smem, stream>>>(
        (__nv_bfloat16*)qkv, ld, bias, cos_table, sin_table, rot, layout, table_positions, norm_mode, q_weight, k_weight, eps, positions, token_row,
        block_table, table_width, page_size, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, num_pages, nq, nkv, d, dv, num_tokens, error_word);
  else
    PYLON_REFUSE("qkv_rotate_write: unknown dtype %d", dtype);
  PYLON_CHECK_LAUNCH("qkv_rotate_write");
}

extern "C" int pylon_latent_norm_rotate_write(const void* down, long long ld, void* cq, const float* q_weight, const float* kv_weight, float eps,
                                              const float* cos_table, const float* sin_table, int rot, int layout, int table_positions,
                                              const int* positions, const int* token_row, const int* block_table, int table_width, int page_size,
                                              void* pages, int num_pages, int q_rank, int kv_rank, int rot_dim, int num_tokens, int dtype,
                                              int* error_word, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (q_rank < 0 || kv_rank < 1 || rot_dim < 0 || rot_dim > 8192) PYLON_REFUSE("latent_norm_rotate_write: ranks %d / %d, %d rotated", q_rank, kv_rank, rot_dim);
  if (rot < 0 || rot > rot_dim || rot % 2 || (rot > 0 && (!cos_table || !sin_table))) PYLON_REFUSE("latent_norm_rotate_write: %d rotated elements of %d", rot, rot_dim);
  if (page_size < 1 || table_width < 1) PYLON_REFUSE("latent_norm_rotate_write: page size %d, table width %d", page_size, table_width);
  const size_t smem = (size_t)(34 + q_rank + kv_rank + rot_dim) * sizeof(float);
  if (smem > 48 * 1024) PYLON_REFUSE("latent_norm_rotate_write: a row of %d numbers is too wide", q_rank + kv_rank + rot_dim);
  if (dtype == PYLON_DTYPE_F32)
    latent_norm_rotate_write_kernel<float><<<num_tokens, ROTARY_THREADS, smem, stream>>>(
        (const float*)down, ld, (float*)cq, q_weight, kv_weight, eps, cos_table, sin_table, rot, layout, table_positions, positions, token_row,
        block_table, table_width, page_size, (float*)pages, num_pages, q_rank, kv_rank, rot_dim, error_word);
  else if (dtype == PYLON_DTYPE_BF16)
    latent_norm_rotate_write_kernel<__nv_bfloat16><<<num_tokens, ROTARY_THREADS, smem, stream>>>(
        (const __nv_bfloat16*)down, ld, (__nv_bfloat16*)cq, q_weight, kv_weight, eps, cos_table, sin_table, rot, layout, table_positions, positions,
        token_row, block_table, table_width, page_size, (__nv_bfloat16*)pages, num_pages, q_rank, kv_rank, rot_dim, error_word);
  else
    PYLON_REFUSE("latent_norm_rotate_write: unknown dtype %d", dtype);
  PYLON_CHECK_LAUNCH("latent_norm_rotate_write");
}

extern "C" int pylon_rotate_heads(const void* src, long long src_token_stride, long long src_head_stride, void* dst, long long dst_token_stride,
                                  long long dst_head_stride, const float* cos_table, const float* sin_table, int rot, int layout, int table_positions,
                                  const int* positions, int heads, int width, int num_tokens, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0 || heads <= 0 || width <= 0) return 0;
  if (width > 2048 || rot < 0 || rot > width || rot % 2 || (rot > 0 && (!cos_table || !sin_table))) PYLON_REFUSE("rotate_heads: %d rotated elements of %d", rot, width);
  const long long items = (long long)num_tokens * heads;
  const unsigned blocks = (unsigned)((items + ROTARY_WARPS - 1) / ROTARY_WARPS);
  const size_t smem = (size_t)ROTARY_WARPS * width * sizeof(float);
  if (dtype == PYLON_DTYPE_F32)
    rotate_heads_kernel<float><<<blocks, ROTARY_THREADS, smem, stream>>>((const float*)src, src_token_stride, src_head_stride, (float*)dst, dst_token_stride,
                                                                          dst_head_stride, cos_table, sin_table, rot, layout, table_positions, positions,
                                                                          heads, width, num_tokens);
  else if (dtype == PYLON_DTYPE_BF16)
    rotate_heads_kernel<__nv_bfloat16><<<blocks, ROTARY_THREADS, smem, stream>>>((const __nv_bfloat16*)src, src_token_stride, src_head_stride,
                                                                                  (__nv_bfloat16*)dst, dst_token_stride, dst_head_stride, cos_table, sin_table,
                                                                                  rot, layout, table_positions, positions, heads, width, num_tokens);
  else
    PYLON_REFUSE("rotate_heads: unknown dtype %d", dtype);
  PYLON_CHECK_LAUNCH("rotate_heads");
}
