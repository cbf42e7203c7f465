// The small steps around attention over a cached latent.
//
// `latent_prepare`: one block a token takes the row of the fused down projection (fp32:
// [query latent | key/value latent | shared key part]) and
//   * divides the query latent by its root mean square (eps inside the root), multiplies by
//     its weight and stores it for the up projection,
//   * does the same to the key/value latent and writes it to the token's cache row,
//   * rotates the shared key part by the token's position (pairs (i, i + rot/2), or with
//     `interleaved` (2i, 2i + 1); table of cosines and sines that already carry the
//     rotation's magnitude) and writes it behind the latent in the same cache row.
// `rotate_heads`: rotates a slice of every head of a projection's output in place, with
// the same two ways of pairing.
// Sums of squares, norms and rotations are fp32 in both modes.
#include "common.cuh"

namespace {

constexpr int kThreads = 128;

template <typename W, typename T>
__global__ void __launch_bounds__(kThreads)
latent_prepare_kernel(const float* __restrict__ down, long long stride, int q_rank, int rank,
                      int rot, const W* __restrict__ q_weight, const W* __restrict__ kv_weight,
                      float eps, const int32_t* __restrict__ positions,
                      const int32_t* __restrict__ token_seq,
                      const int32_t* __restrict__ block_table, int max_blocks,
                      const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                      T* __restrict__ q_latent, T* __restrict__ cache, int write_cache,
                      int interleaved) {
  __shared__ float scratch[33];
  const long long t = blockIdx.x;
  const float* row = down + t * stride;
  if (q_rank > 0) {
    float s = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += kThreads) s = fmaf(row[i], row[i], s);
    const float r = rsqrtf(block_sum(s, scratch) / static_cast<float>(q_rank) + eps);
    for (int i = threadIdx.x; i < q_rank; i += kThreads)
      q_latent[t * q_rank + i] = narrow<T>(row[i] * r * widen(q_weight[i]));
  }
  if (!write_cache) return;
  const float* kv = row + q_rank;
  float s = 0.f;
  for (int i = threadIdx.x; i < rank; i += kThreads) s = fmaf(kv[i], kv[i], s);
  const float r = rsqrtf(block_sum(s, scratch) / static_cast<float>(rank) + eps);
  const int pos = positions[t];
  const int block = block_table[(long long)token_seq[t] * max_blocks + pos / kCacheBlock];
  T* to = cache + ((long long)block * kCacheBlock + pos % kCacheBlock) * (rank + rot);
  for (int i = threadIdx.x; i < rank; i += kThreads)
    to[i] = narrow<T>(kv[i] * r * widen(kv_weight[i]));
  const int half = rot / 2;
  const float* part = kv + rank;
  for (int i = threadIdx.x; i < half; i += kThreads) {
    const float c = cos_t[(long long)pos * half + i], sn = sin_t[(long long)pos * half + i];
    const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
    const float u = part[a], v = part[b];
    to[rank + a] = narrow<T>(u * c - v * sn);
    to[rank + b] = narrow<T>(v * c + u * sn);
  }
}

template <typename T>
__global__ void rotate_heads_kernel(T* __restrict__ x, long long stride, int head_stride,
                                    int offset, int heads, int rot,
                                    const int32_t* __restrict__ positions,
                                    const float* __restrict__ cos_t,
                                    const float* __restrict__ sin_t, long long count,
                                    int interleaved) {
  const int half = rot / 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x) {
    const int e = static_cast<int>(i % half);
    const long long rest = i / half;
    const int h = static_cast<int>(rest % heads);
    const long long t = rest / heads;
    const int pos = positions[t];
    const float c = cos_t[(long long)pos * half + e], sn = sin_t[(long long)pos * half + e];
    T* p = x + t * stride + (long long)h * head_stride + offset + (interleaved ? 2 * e : e);
    const int other = interleaved ? 1 : half;
    const float u = widen(p[0]), v = widen(p[other]);
    p[0] = narrow<T>(u * c - v * sn);
    p[other] = narrow<T>(v * c + u * sn);
  }
}

template <typename W, typename T>
int prepare(const float* down, long long stride, int q_rank, int rank, int rot,
            const void* q_weight, const void* kv_weight, float eps, const int32_t* positions,
            const int32_t* token_seq, const int32_t* block_table, int max_blocks,
            const float* cos_t, const float* sin_t, void* q_latent, void* cache, int write_cache,
            int interleaved, int tokens, cudaStream_t stream) {
  return launch_ordered(latent_prepare_kernel<W, T>, dim3(tokens), dim3(kThreads), 0, stream, down,
                        stride, q_rank, rank, rot, (const W*)q_weight, (const W*)kv_weight, eps,
                        positions, token_seq, block_table, max_blocks, cos_t, sin_t,
                        (T*)q_latent, (T*)cache, write_cache, interleaved);
}

}  // namespace

// down: fp32 [tokens, stride], columns [q_rank | rank | rot]. q_latent: [tokens, q_rank] and
// cache: [blocks, 1, 64, rank + rot], both of `dtype`; weights of `w_dtype`. cos_t, sin_t:
// fp32 [positions, rot / 2]. q_rank may be 0 (no query latent). interleaved: the rotation
// pairs (2i, 2i + 1) instead of (i, i + rot / 2).
SAKV_EXPORT int sakv_latent_prepare(const float* down, long long stride, int q_rank, int rank,
                                    int rot, const void* q_weight, const void* kv_weight,
                                    int w_dtype, float eps, const int32_t* positions,
                                    const int32_t* token_seq, const int32_t* block_table,
                                    int max_blocks, const float* cos_t, const float* sin_t,
                                    void* q_latent, void* cache, int dtype, int write_cache,
                                    int interleaved, int tokens, cudaStream_t stream) {
  if (tokens < 0 || q_rank < 0 || rank <= 0 || rot <= 0 || rot % 2 || max_blocks <= 0 ||
      stride < q_rank + rank + rot || w_dtype != dtype)
    return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  if (dtype == SAKV_F32)
    return prepare<float, float>(down, stride, q_rank, rank, rot, q_weight, kv_weight, eps,
                                 positions, token_seq, block_table, max_blocks, cos_t, sin_t,
                                 q_latent, cache, write_cache, interleaved, tokens, stream);
  if (dtype == SAKV_BF16)
    return prepare<__nv_bfloat16, __nv_bfloat16>(down, stride, q_rank, rank, rot, q_weight,
                                                 kv_weight, eps, positions, token_seq, block_table,
                                                 max_blocks, cos_t, sin_t, q_latent, cache,
                                                 write_cache, interleaved, tokens, stream);
  return cudaErrorInvalidValue;
}

// x: [tokens, stride] of `dtype`; in every head h the `rot` columns from h * head_stride +
// offset on are rotated in place by the token's position.
SAKV_EXPORT int sakv_rotate_heads(void* x, int dtype, long long stride, int head_stride,
                                  int offset, int heads, int rot, const int32_t* positions,
                                  const float* cos_t, const float* sin_t, int interleaved,
                                  int tokens, cudaStream_t stream) {
  if (tokens < 0 || heads <= 0 || rot <= 0 || rot % 2 || offset < 0 || offset + rot > head_stride ||
      (long long)heads * head_stride > stride)
    return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  const long long count = (long long)tokens * heads * (rot / 2);
  const dim3 grid(grid_for(count, 256)), block(256);
  if (dtype == SAKV_F32)
    return launch_ordered(rotate_heads_kernel<float>, grid, block, 0, stream, (float*)x, stride,
                          head_stride, offset, heads, rot, positions, cos_t, sin_t, count,
                          interleaved);
  if (dtype == SAKV_BF16)
    return launch_ordered(rotate_heads_kernel<__nv_bfloat16>, grid, block, 0, stream,
                          (__nv_bfloat16*)x, stride, head_stride, offset, heads, rot, positions,
                          cos_t, sin_t, count, interleaved);
  return cudaErrorInvalidValue;
}
