// The residual stream kept as several copies ("hyper-connections"), and the norms that read it.
//
// A model may carry S >= 1 streams x_1 .. x_S per token, float32 [T, S, W].  A sublayer reads one
// combination of them, u = sum_s read[s] * x_s, through a norm, and its output y goes back into all
// of them at once, computed from the old ones:
//
//     x_t <- sum_s mix[s, t] * x_s + scale * out[t] * y            (mix is indexed [from, to])
//
// The plain residual sum is the case S = 1 with mix = out = read = 1, optionally with a factor on
// the sublayer's output.  One kernel does the pending update of the sublayer before and the read
// and norm of the sublayer after, so the streams are read and written once per sublayer:
//
//     update (optional)  ->  u = sum_s read[s] x_s  ->  norm(u) * weight  ->  out
//
// Norm kinds: 0 = layer norm without bias, (u - mean) / sqrt(var + eps) * w with var the mean of
// the squared deviations (two passes over the row, which lies in shared memory); 1 = RMS norm,
// u / sqrt(mean(u^2) + eps) * w.  Everything is float32 but the sublayer's output as it comes in
// and the normalised row as it goes out.  With a row selection the streams are not written: the
// selected rows are normalised from the updated values computed on the fly (final norm at the
// rows whose logits are wanted).
#include "common.cuh"

namespace pylon {

constexpr int MAX_STREAMS = 8;

template <typename TD, typename TO>
__global__ void streams_update_norm_kernel(float* __restrict__ x, const TD* __restrict__ delta, int delta_parts, long long part_stride,
                                           float scale, const float* __restrict__ mix, const float* __restrict__ outw,
                                           const float* __restrict__ read, const float* __restrict__ weight, const int* __restrict__ rows,
                                           TO* __restrict__ out, int streams, int width, float eps, int kind) {
  extern __shared__ float shared[];
  float* u_row = shared;                 // [width]
  float* scratch = u_row + width;        // [34]
  float* coef = scratch + 34;            // mix [S * S], out [S], read [S]
  const int S = streams;
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) coef[i] = mix ? mix[i] : (i / S == i % S ? 1.f : 0.f);
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    coef[S * S + i] = (outw ? outw[i] : 1.f) * scale;
    coef[S * S + S + i] = read ? read[i] : 1.f;
  }
  __syncthreads();
  const float* c_mix = coef;
  const float* c_out = coef + S * S;
  const float* c_read = c_out + S;
  const int n = blockIdx.x;
  const long long t = rows ? rows[n] : n;
  float* xt = x + t * (long long)S * width;
  const bool update = delta != nullptr || mix != nullptr;
  float local_sum = 0.f;
  for (int e = threadIdx.x; e < width; e += blockDim.x) {
    float old[MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < MAX_STREAMS; ++s) old[s] = s < S ? xt[(long long)s * width + e] : 0.f;
    float y = 0.f;
    if (delta) {
      for (int part = 0; part < delta_parts; ++part) y += to_float<TD>(delta[part * part_stride + t * width + e]);
    }
    float u = 0.f;
#pragma unroll
    for (int to = 0; to < MAX_STREAMS; ++to) {
      if (to < S) {
        float value = old[to];
        if (update) {
          value = 0.f;
#pragma unroll
          for (int from = 0; from < MAX_STREAMS; ++from)
            if (from < S) value = fmaf(c_mix[from * S + to], old[from], value);
          value = fmaf(c_out[to], y, value);
          if (!rows) xt[(long long)to * width + e] = value;
        }
        u = fmaf(c_read[to], value, u);
      }
    }
    u_row[e] = u;
    local_sum += u;
  }
  if (!out) return;
  float mean = 0.f;
  if (kind == 0) mean = block_sum(local_sum, scratch) / (float)width;
  float local_sq = 0.f;
  for (int e = threadIdx.x; e < width; e += blockDim.x) {   // each thread reads back what it wrote itself
    const float c = u_row[e] - mean;
    local_sq = fmaf(c, c, local_sq);
  }
  const float inv = rsqrtf(block_sum(local_sq, scratch) / (float)width + eps);
  TO* orow = out + (long long)n * width;
  for (int e = threadIdx.x; e < width; e += blockDim.x) orow[e] = from_float<TO>((u_row[e] - mean) * inv * weight[e]);
}

}  // namespace pylon

using namespace pylon;

// x: float32 [tokens, streams, width], updated in place unless `rows` selects.  delta: the sublayer's output [tokens, width] in
// delta_dtype, or float32 partial sums [delta_parts, tokens, width] whose sum it is, or null (nothing pending).  mix [S, S], outw [S],
// read [S]: float32 on the device, null = identity / ones / ones.  weight null: only the update (out is not written).
// out: [n_rows, width] in out_dtype.  n_rows: the selected rows, or all tokens.
extern "C" int pylon_streams_update_norm(float* x, const void* delta, int delta_parts, int delta_dtype, float scale, const float* mix,
                                         const float* outw, const float* read, const float* weight, const int* rows, void* out,
                                         int out_dtype, int n_rows, int tokens, int streams, int width, float eps, int kind,
                                         cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (streams < 1 || streams > MAX_STREAMS) PYLON_REFUSE("streams_update_norm: %d streams (1 to %d)", streams, MAX_STREAMS);
  if (width < 1 || width > 32768) PYLON_REFUSE("streams_update_norm: width %d", width);
  if (kind != 0 && kind != 1) PYLON_REFUSE("streams_update_norm: norm kind %d", kind);
  if ((weight == nullptr) != (out == nullptr)) PYLON_REFUSE("streams_update_norm: a norm weight and an output go together");
  if (!out && rows) PYLON_REFUSE("streams_update_norm: a row selection without an output does nothing");
  if (delta && delta_parts < 1) PYLON_REFUSE("streams_update_norm: %d parts", delta_parts);
  if (delta && delta_parts > 1 && delta_dtype != PYLON_DTYPE_F32) PYLON_REFUSE("streams_update_norm: partial sums are float32");
  const int threads = width >= 4096 ? 512 : (width >= 1024 ? 256 : 128);
  const size_t smem = (size_t)(width + 34 + streams * streams + 2 * streams) * sizeof(float);
  const long long part_stride = (long long)tokens * width;
#define PYLON_STREAMS_LAUNCH(TD, TO)                                                                                          \
  do {                                                                                                                        \
    static bool raised[MAX_DEVICES] = {};                                                                                     \
    if (smem > 48 * 1024 && !raised[current_device_slot()]) {                                                                 \
      cudaFuncSetAttribute(streams_update_norm_kernel<TD, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);      \
      raised[current_device_slot()] = true;                                                                                   \
    }                                                                                                                         \
    streams_update_norm_kernel<TD, TO><<<n_rows, threads, smem, stream>>>(x, (const TD*)delta, delta_parts, part_stride,      \
        scale, mix, outw, read, weight, rows, (TO*)out, streams, width, eps, kind);                                           \
  } while (0)
  const bool delta_f32 = !delta || delta_dtype == PYLON_DTYPE_F32;
  if (!delta_f32 && delta_dtype != PYLON_DTYPE_BF16) PYLON_REFUSE("streams_update_norm: unknown delta dtype %d", delta_dtype);
  if (out_dtype == PYLON_DTYPE_F32) {
    if (delta_f32) PYLON_STREAMS_LAUNCH(float, float); else PYLON_STREAMS_LAUNCH(__nv_bfloat16, float);
  } else if (out_dtype == PYLON_DTYPE_BF16) {
    if (delta_f32) PYLON_STREAMS_LAUNCH(float, __nv_bfloat16); else PYLON_STREAMS_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  } else {
    PYLON_REFUSE("streams_update_norm: unknown output dtype %d", out_dtype);
  }
#undef PYLON_STREAMS_LAUNCH
  PYLON_CHECK_LAUNCH("streams_update_norm");
}
