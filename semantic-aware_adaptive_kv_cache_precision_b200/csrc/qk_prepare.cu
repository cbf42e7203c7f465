// What lies between an attention mixer's fused projection and its attention when queries and
// keys are normed over the WHOLE projection before they are split into heads:
//
//   q <- q / sqrt(mean(q^2) + eps) * wq      (over all heads * dim numbers of the token at once)
//   k <- k / sqrt(mean(k^2) + eps) * wk      (over all kv_heads * dim numbers)
//   the first `rot` numbers of every head of q and k are turned by the token's position
//   (number i paired with i + rot / 2: (u, v) -> (u cos - v sin, v cos + u sin)); the rest pass
//   q goes to a tensor of its own, k and v into the token's place in the cache blocks.
//
// The projection's output is fp32 (its accumulator, unrounded); sums of squares, the norm and
// the rotation are fp32, and queries, keys and values are rounded once, at the store. Either
// norm may be absent (null weight), and so may the rotation (null tables). One block a token.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

template <typename W, typename C>
__global__ void __launch_bounds__(kThreads)
qk_prepare_kernel(const float* __restrict__ proj, long long stride, int q_off, int k_off,
                  int v_off, const W* __restrict__ wq, const W* __restrict__ wk, float eps,
                  const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
                  const int32_t* __restrict__ positions, const int32_t* __restrict__ token_seq,
                  const int32_t* __restrict__ block_table, int max_blocks, C* __restrict__ q_out,
                  C* __restrict__ k_cache, C* __restrict__ v_cache, int heads, int kv_heads,
                  int dim, int vdim, int write_cache) {
  __shared__ float scratch[33];
  const long long t = blockIdx.x;
  const float* row = proj + t * stride;
  const int pos = positions[t];
  const int half = rot / 2;
  const float* cs = cos_t ? cos_t + (long long)pos * half : nullptr;
  const float* sn = sin_t ? sin_t + (long long)pos * half : nullptr;
  long long slot_row = 0;
  if (write_cache) {
    const int block = block_table[(long long)token_seq[t] * max_blocks + pos / kCacheBlock];
    slot_row = (long long)block * kv_heads * kCacheBlock + pos % kCacheBlock;
  }
  // one projection at a time: queries (which = 0), then keys
  for (int which = 0; which < 2; ++which) {
    const int n_heads = which == 0 ? heads : kv_heads;
    const int count = n_heads * dim;
    const float* src = row + (which == 0 ? q_off : k_off);
    const W* w = which == 0 ? wq : wk;
    if (which == 1 && !write_cache) break;
    float r = 1.f;
    if (w != nullptr) {
      float ss = 0.f;
      for (int e = threadIdx.x; e < count; e += kThreads) ss = fmaf(src[e], src[e], ss);
      r = 1.f / sqrtf(block_sum(ss, scratch) / static_cast<float>(count) + eps);
    }
    for (int e = threadIdx.x; e < count; e += kThreads) {
      const int h = e / dim, i = e - h * dim;
      C* dst = which == 0
                   ? q_out + t * count + e
                   : k_cache + (slot_row + (long long)h * kCacheBlock) * dim + i;
      if (i >= rot || cs == nullptr) {
        *dst = narrow<C>(w ? src[e] * r * widen(w[e]) : src[e]);
      } else if (i < half) {
        const float u = w ? src[e] * r * widen(w[e]) : src[e];
        const float v = w ? src[e + half] * r * widen(w[e + half]) : src[e + half];
        const float c = cs[i], s = sn[i];
        dst[0] = narrow<C>(u * c - v * s);
        dst[half] = narrow<C>(v * c + u * s);
      }
    }
  }
  if (write_cache) {
    const int count = kv_heads * vdim;
    const float* src = row + v_off;
    for (int e = threadIdx.x; e < count; e += kThreads) {
      const int h = e / vdim, i = e - h * vdim;
      v_cache[(slot_row + (long long)h * kCacheBlock) * vdim + i] = narrow<C>(src[e]);
    }
  }
}

template <typename W, typename C>
int launch(const float* proj, long long stride, int q_off, int k_off, int v_off, const void* wq,
           const void* wk, float eps, const float* cos_t, const float* sin_t, int rot,
           const int32_t* positions, const int32_t* token_seq, const int32_t* block_table,
           int max_blocks, void* q_out, void* k_cache, void* v_cache, int tokens, int heads,
           int kv_heads, int dim, int vdim, int write_cache, cudaStream_t stream) {
  return launch_ordered(qk_prepare_kernel<W, C>, dim3(tokens), dim3(kThreads), 0, stream, proj,
                        stride, q_off, k_off, v_off, (const W*)wq, (const W*)wk, eps, cos_t,
                        sin_t, rot, positions, token_seq, block_table, max_blocks, (C*)q_out,
                        (C*)k_cache, (C*)v_cache, heads, kv_heads, dim, vdim, write_cache);
}

}  // namespace

// proj: fp32 [tokens, stride]; queries at column q_off (heads * dim), keys at k_off (kv_heads *
// dim), values at v_off (kv_heads * vdim). wq [heads * dim], wk [kv_heads * dim] of `w_dtype`
// (null: no norm). cos_t, sin_t: fp32 [positions, rot / 2] (null: no rotation). q_out: [tokens,
// heads * dim]; k_cache [blocks, kv_heads, 64, dim], v_cache [blocks, kv_heads, 64, vdim], all
// of `c_dtype`. write_cache 0: only the queries are made.
SAKV_EXPORT int sakv_qk_prepare(const float* proj, long long stride, int q_off, int k_off,
                                int v_off, const void* wq, const void* wk, int w_dtype, float eps,
                                const float* cos_t, const float* sin_t, int rot,
                                const int32_t* positions, const int32_t* token_seq,
                                const int32_t* block_table, int max_blocks, void* q_out,
                                void* k_cache, void* v_cache, int c_dtype, int tokens, int heads,
                                int kv_heads, int dim, int vdim, int write_cache,
                                cudaStream_t stream) {
  if (tokens < 0 || heads <= 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || rot < 0 || rot % 2 ||
      rot > dim || max_blocks <= 0 || (cos_t == nullptr) != (sin_t == nullptr))
    return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
#define SAKV_QK(W, C)                                                                            \
  return launch<W, C>(proj, stride, q_off, k_off, v_off, wq, wk, eps, cos_t, sin_t, rot,         \
                      positions, token_seq, block_table, max_blocks, q_out, k_cache, v_cache,    \
                      tokens, heads, kv_heads, dim, vdim, write_cache, stream)
  if (w_dtype == SAKV_F32 && c_dtype == SAKV_F32) SAKV_QK(float, float);
  if (w_dtype == SAKV_BF16 && c_dtype == SAKV_BF16) SAKV_QK(__nv_bfloat16, __nv_bfloat16);
  if (w_dtype == SAKV_F32 && c_dtype == SAKV_BF16) SAKV_QK(float, __nv_bfloat16);
  if (w_dtype == SAKV_BF16 && c_dtype == SAKV_F32) SAKV_QK(__nv_bfloat16, float);
#undef SAKV_QK
  return cudaErrorInvalidValue;
}
