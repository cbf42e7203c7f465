// The step between two sublayers of a layer that norms a sublayer's OUTPUT (and nothing
// else) before it joins the fp32 residual stream:
//
//   x += y / sqrt(mean(y^2) + eps) * (add_offset + w_add)        (y: the sublayer's output)
//   out = x, in the type the next sublayer reads                  (w_out null)
//   out = x / sqrt(mean(x^2) + eps) * (out_offset + w_out)       (w_out given: a norm)
//
// one pass over the stream. Any of the three may be absent: without y nothing is added (the
// copy of the stream for a first layer, or a plain RMS norm with a weight stored around zero,
// `offset` 1, or around one, `offset` 0); without out only the stream is completed. With
// `rows` only those rows are normed or copied (the final norm of the wanted positions). Sums
// of squares, roots and products are fp32 with one rounding at the store; one block a row,
// the row in shared memory, so the order of the additions depends on the row's length alone.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float inverse_rms(const float* row, int hidden, float eps,
                                             float* scratch) {
  float q = 0.f;
  for (int i = threadIdx.x; i < hidden; i += kThreads) q = fmaf(row[i], row[i], q);
  return 1.f / sqrtf(block_sum(q, scratch) / static_cast<float>(hidden) + eps);
}

template <typename W, typename Out>
__global__ void __launch_bounds__(kThreads)
rms_update_kernel(float* __restrict__ x, const float* __restrict__ y,
                  const W* __restrict__ w_add, float add_offset,
                  const int32_t* __restrict__ rows, const W* __restrict__ w_out, float out_offset,
                  Out* __restrict__ out, int hidden, float eps) {
  extern __shared__ float row[];
  __shared__ float scratch[33];
  const long long src = rows ? rows[blockIdx.x] : blockIdx.x;
  float* in = x + src * hidden;
  if (y != nullptr) {
    const float* add = y + src * hidden;
    for (int i = threadIdx.x; i < hidden; i += kThreads) row[i] = add[i];
    __syncthreads();
    const float r = inverse_rms(row, hidden, eps, scratch);
    for (int i = threadIdx.x; i < hidden; i += kThreads) {
      const float v = in[i] + row[i] * r * (add_offset + widen(w_add[i]));
      in[i] = v;
      row[i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += kThreads) row[i] = in[i];
  }
  if (out == nullptr) return;
  Out* o = out + (long long)blockIdx.x * hidden;
  if (w_out == nullptr) {                   // (each thread reads back what it wrote itself)
    for (int i = threadIdx.x; i < hidden; i += kThreads) o[i] = narrow<Out>(row[i]);
    return;
  }
  __syncthreads();
  const float r = inverse_rms(row, hidden, eps, scratch);
  for (int i = threadIdx.x; i < hidden; i += kThreads)
    o[i] = narrow<Out>(row[i] * r * (out_offset + widen(w_out[i])));
}

template <typename W, typename Out>
int launch(float* x, const float* y, const void* w_add, float add_offset, const int32_t* rows,
           const void* w_out, float out_offset, void* out, int n, int hidden, float eps,
           cudaStream_t stream) {
  return launch_ordered(rms_update_kernel<W, Out>, dim3(n), dim3(kThreads),
                        (size_t)hidden * sizeof(float), stream, x, y, (const W*)w_add, add_offset,
                        rows, (const W*)w_out, out_offset, (Out*)out, hidden, eps);
}

}  // namespace

// x: fp32 [T, hidden], updated in place when `y` (fp32 [T, hidden]) is given. out (may be
// null): [n, hidden] of `out_dtype`, the rows `rows ? rows[r] : r`; `rows` only without `y`.
// Weights of `w_dtype`.
SAKV_EXPORT int sakv_rms_update(float* x, const float* y, const void* w_add, float add_offset,
                                const int32_t* rows, const void* w_out, float out_offset,
                                int w_dtype, void* out, int out_dtype, int n, int hidden,
                                float eps, cudaStream_t stream) {
  if (n < 0 || hidden <= 0 || hidden > 12000 || (y != nullptr && (rows != nullptr || !w_add)) ||
      (out == nullptr && y == nullptr))
    return cudaErrorInvalidValue;
  if (n == 0) return 0;
  if (w_dtype == SAKV_F32 && out_dtype == SAKV_F32)
    return launch<float, float>(x, y, w_add, add_offset, rows, w_out, out_offset, out, n, hidden,
                                eps, stream);
  if (w_dtype == SAKV_BF16 && out_dtype == SAKV_BF16)
    return launch<__nv_bfloat16, __nv_bfloat16>(x, y, w_add, add_offset, rows, w_out, out_offset,
                                                out, n, hidden, eps, stream);
  if (w_dtype == SAKV_BF16 && out_dtype == SAKV_F32)
    return launch<__nv_bfloat16, float>(x, y, w_add, add_offset, rows, w_out, out_offset, out, n,
                                        hidden, eps, stream);
  if (w_dtype == SAKV_F32 && out_dtype == SAKV_BF16)
    return launch<float, __nv_bfloat16>(x, y, w_add, add_offset, rows, w_out, out_offset, out, n,
                                        hidden, eps, stream);
  return cudaErrorInvalidValue;
}
