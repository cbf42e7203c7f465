// Recurrent mixers whose state is decayed and added to, token by token, without any feedback
// from the state into its own update:
//
//   * the selective scan (a state of N numbers a channel, decay and input step chosen by the
//     token):   S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;   y_c = sum_n S[c, n] C_n + D_c x_c
//     with the pieces around it: the short causal convolution a channel with its running
//     inputs as state, the step size dt = softplus(Wdt low + b), the gate y * silu(z);
//   * attention without softmax whose state, a matrix a head, fades by a fixed factor a head:
//               S <- decay_h S + k v^T;   o = S^T q          (q, k, v after silu)
//     and the norm over all heads' outputs with its sigmoid gate.
//
// Everything that enters a recurrence is fp32: decays, exponentials, softplus, step sizes, the
// states and the sums over them. The projections' outputs come as fp32 (their accumulators,
// unrounded). A sequence's tokens are taken in order by the threads that own a piece of its
// state, so the result of a token does not depend on how its sequence was cut into steps or
// on what else is in the step.
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---------------------------------------------------------------------------------------
// The short causal convolution. Token i of a sequence's part in this step reads its own
// input and the taps - 1 before it: from the step while there are any, from the state (the
// sequence's last taps - 1 inputs, oldest first, zeros before its start) otherwise.
// ---------------------------------------------------------------------------------------
template <typename W, typename C>
__global__ void causal_conv_kernel(const float* __restrict__ in, long long stride,
                                   const W* __restrict__ w, const W* __restrict__ bias,
                                   const float* __restrict__ state,
                                   const int32_t* __restrict__ cu_seqlens,
                                   const int32_t* __restrict__ token_seq,
                                   const int32_t* __restrict__ slots, C* __restrict__ out,
                                   int channels, int taps, long long count) {
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < count;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / channels;
    const int c = static_cast<int>(idx - t * channels);
    const int b = token_seq[t];
    const int i = static_cast<int>(t - cu_seqlens[b]);           // place in this step's part
    const float* old = state + (long long)slots[b] * (taps - 1) * channels;
    float acc = bias ? widen(bias[c]) : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;                             // column j: `back` tokens ago
      const float v = back <= i ? in[(t - back) * stride + c]
                                : old[(long long)(taps - 1 - (back - i)) * channels + c];
      acc = fmaf(v, widen(w[(long long)c * taps + j]), acc);
    }
    out[t * channels + c] = narrow<C>(silu(acc));
  }
}

// The state after the step: the sequence's last taps - 1 inputs. One thread a (sequence,
// channel) reads what it needs of the old state before it writes.
__global__ void conv_state_kernel(const float* __restrict__ in, long long stride,
                                  float* __restrict__ state,
                                  const int32_t* __restrict__ cu_seqlens,
                                  const int32_t* __restrict__ slots, int channels, int taps,
                                  int sequences) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)sequences * channels) return;
  const int b = static_cast<int>(idx / channels), c = static_cast<int>(idx - (long long)b * channels);
  const int first = cu_seqlens[b], n = cu_seqlens[b + 1] - first, keep = taps - 1;
  float* mine = state + (long long)slots[b] * keep * channels + c;
  // new[j] is the input `keep - j` tokens before the step's end: from the step if there are
  // that many, else from the old state, which moves up by n places (ascending j reads ahead
  // of what it has written)
  for (int j = 0; j < keep; ++j) {
    const int back = keep - j;
    mine[(long long)j * channels] = back <= n ? in[(long long)(first + n - back) * stride + c]
                                              : mine[(long long)(j + n) * channels];
  }
}

// ---------------------------------------------------------------------------------------
// Step sizes: dt[t, c] = softplus(sum_r low[t, r] Wdt[c, r] + b[c]). A block a token.
// ---------------------------------------------------------------------------------------
template <typename W>
__global__ void step_size_kernel(const float* __restrict__ low, long long stride, int rank,
                                 const W* __restrict__ w, const W* __restrict__ bias,
                                 float* __restrict__ dt, int channels) {
  extern __shared__ float row[];
  const long long t = blockIdx.x;
  for (int r = threadIdx.x; r < rank; r += blockDim.x) row[r] = low[t * stride + r];
  __syncthreads();
  for (int c = threadIdx.x; c < channels; c += blockDim.x) {
    const W* wr = w + (long long)c * rank;
    float acc = 0.f;
    for (int r = 0; r < rank; ++r) acc = fmaf(row[r], widen(wr[r]), acc);
    dt[t * channels + c] = softplus(acc + (bias ? widen(bias[c]) : 0.f));
  }
}

// ---------------------------------------------------------------------------------------
// The selective scan. A channel's N states are dealt to G neighbouring lanes, NPT each
// (state n = g * NPT + k belongs to lane g); a lane keeps its states in registers for the
// whole step, the sum over the states ends with log2(G) shuffles. Blocks: (channels * G /
// blockDim, sequences). State in memory: [slots, channels, N].
// ---------------------------------------------------------------------------------------
template <int NPT, typename W, typename C>
__global__ void selective_scan_kernel(const C* __restrict__ x, const float* __restrict__ dt,
                                      const float* __restrict__ low, long long low_stride,
                                      int b_off, int c_off, const float* __restrict__ z,
                                      long long z_stride, const W* __restrict__ a_log,
                                      const W* __restrict__ d_skip, float* __restrict__ state,
                                      const int32_t* __restrict__ cu_seqlens,
                                      const int32_t* __restrict__ slots, C* __restrict__ out,
                                      int channels, int n_state, int lanes, int keep_state) {
  const int b = blockIdx.y;
  const long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const int c_raw = static_cast<int>(id / lanes), g = static_cast<int>(id % lanes);
  const bool live = c_raw < channels;                 // (idle lanes still join the shuffles)
  const int c = live ? c_raw : channels - 1;
  const int n0 = g * NPT;
  float a[NPT], s[NPT];
  float* mine = state + ((long long)slots[b] * channels + c) * n_state + n0;
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const bool has = n0 + k < n_state;
    a[k] = has ? -expf(widen(a_log[(long long)c * n_state + n0 + k])) : 0.f;
    s[k] = has ? mine[k] : 0.f;
  }
  const float skip = widen(d_skip[c]);
  const int first = cu_seqlens[b], last = cu_seqlens[b + 1];
  for (int t = first; t < last; ++t) {
    const float step = dt[(long long)t * channels + c];
    const float xv = widen(x[(long long)t * channels + c]);
    const float* bt = low + (long long)t * low_stride + b_off + n0;
    const float* ct = low + (long long)t * low_stride + c_off + n0;
    const float dx = step * xv;
    float y = 0.f;
#pragma unroll
    for (int k = 0; k < NPT; ++k) {
      const bool has = n0 + k < n_state;
      const float bv = has ? bt[k] : 0.f, cv = has ? ct[k] : 0.f;
      // S + (e^(dt A) - 1) S + dt x B: a decay close to 1 keeps its distance from 1 exactly
      s[k] += fmaf(expm1f(step * a[k]), s[k], dx * bv);
      y = fmaf(s[k], cv, y);
    }
    for (int o = lanes >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
    if (g == 0 && live) {
      y = fmaf(skip, xv, y);
      out[(long long)t * channels + c] = narrow<C>(y * silu(z[(long long)t * z_stride + c]));
    }
  }
  if (keep_state && live) {
#pragma unroll
    for (int k = 0; k < NPT; ++k)
      if (n0 + k < n_state) mine[k] = s[k];
  }
}

// ---------------------------------------------------------------------------------------
// Attention without softmax, a matrix of state a head that fades by a fixed factor. A block
// owns `cols` neighbouring value columns of one head of one sequence; a column's `dim` rows
// are dealt to RS neighbouring lanes, RP each (row i = r * RP + k belongs to lane r). The
// block brings a run of tokens' q, k (this head's) and v (its columns) into shared memory,
// silu applied once an element, and then walks them. State in memory: [slots, heads, vdim,
// dim] (a column's rows lie together).
// ---------------------------------------------------------------------------------------
constexpr int kRun = 16;          // tokens brought into shared memory at a time

template <int RP>
__global__ void decay_attention_kernel(const float* __restrict__ proj, long long stride,
                                       int q_off, int k_off, int v_off,
                                       const float* __restrict__ decay_less_one,
                                       float* __restrict__ state,
                                       const int32_t* __restrict__ cu_seqlens,
                                       const int32_t* __restrict__ slots, float* __restrict__ out,
                                       int heads, int dim, int vdim, int rs, int cols,
                                       int keep_state) {
  extern __shared__ __align__(16) float shared[];
  const int padded = rs * RP;                       // dim rounded up to whole lanes
  float* qs = shared;                               // [kRun, padded]
  float* ks = qs + kRun * padded;                   // [kRun, padded]
  float* vs = ks + kRun * padded;                   // [kRun, cols]
  const int b = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * cols;
  const int r = threadIdx.x % rs, j = threadIdx.x / rs;
  const int col = col0 + j;
  const bool live = col < vdim;
  const float fade = decay_less_one[h];        // decay - 1, rounded once from the exact number
  float s[RP];
  float* mine = state + (((long long)slots[b] * heads + h) * vdim + (live ? col : 0)) * dim + r * RP;
#pragma unroll
  for (int k = 0; k < RP; ++k) s[k] = (live && r * RP + k < dim) ? mine[k] : 0.f;
  const int first = cu_seqlens[b], last = cu_seqlens[b + 1];
  for (int t0 = first; t0 < last; t0 += kRun) {
    const int run = last - t0 < kRun ? last - t0 : kRun;
    __syncthreads();
    for (int e = threadIdx.x; e < run * padded; e += blockDim.x) {
      const int tt = e / padded, i = e - tt * padded;
      const float* row = proj + (long long)(t0 + tt) * stride + (long long)h * dim + i;
      qs[e] = i < dim ? silu(row[q_off]) : 0.f;
      ks[e] = i < dim ? silu(row[k_off]) : 0.f;
    }
    for (int e = threadIdx.x; e < run * cols; e += blockDim.x) {
      const int tt = e / cols, i = e - tt * cols;
      vs[e] = col0 + i < vdim
                  ? silu(proj[(long long)(t0 + tt) * stride + v_off + (long long)h * vdim + col0 + i])
                  : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < run; ++tt) {
      const float v = vs[tt * cols + j];
      float o = 0.f;
#pragma unroll
      for (int k = 0; k < RP; ++k) {
        s[k] += fmaf(fade, s[k], ks[tt * padded + r * RP + k] * v);
        o = fmaf(s[k], qs[tt * padded + r * RP + k], o);
      }
      for (int d = rs >> 1; d > 0; d >>= 1) o += __shfl_xor_sync(0xffffffffu, o, d);
      if (r == 0 && live) out[((long long)(t0 + tt) * heads + h) * vdim + col] = o;
    }
  }
  if (keep_state && live) {
#pragma unroll
    for (int k = 0; k < RP; ++k)
      if (r * RP + k < dim) mine[k] = s[k];
  }
}

// out[t] = y[t] / sqrt(mean(y[t]^2) + eps) * w * sigmoid(gate[t]) * scale over the whole row
// (all heads' outputs together). A block a token.
template <typename W, typename C>
__global__ void __launch_bounds__(256)
norm_gate_kernel(const float* __restrict__ y, const W* __restrict__ w,
                 const float* __restrict__ gate, long long gate_stride, C* __restrict__ out,
                 int width, float eps, float scale) {
  __shared__ float scratch[33];
  const long long t = blockIdx.x;
  const float* row = y + t * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
  const float r = 1.f / sqrtf(block_sum(ss, scratch) / static_cast<float>(width) + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = row[i] * r * widen(w[i]);
    if (gate) v *= 1.f / (1.f + expf(-gate[t * gate_stride + i]));
    out[t * width + i] = narrow<C>(v * scale);
  }
}

int lanes_for(int n, int per_lane) {          // a power of two of lanes that hold n numbers
  int lanes = 1;
  while (lanes * per_lane < n) lanes *= 2;
  return lanes;
}

}  // namespace

// in: fp32 [tokens, stride] (the first `channels` columns are the convolution's input); w:
// [channels, taps], bias [channels] (null: none) of `w_dtype`; state: fp32 [slots, taps - 1,
// channels], read here and replaced by `sakv_conv_state` afterwards. out: [tokens, channels]
// of `out_dtype` = silu(convolution).
SAKV_EXPORT int sakv_causal_conv(const float* in, long long stride, const void* w,
                                 const void* bias, int w_dtype, const float* state,
                                 const int32_t* cu_seqlens, const int32_t* token_seq,
                                 const int32_t* slots, void* out, int out_dtype, int tokens,
                                 int channels, int taps, cudaStream_t stream) {
  if (tokens < 0 || channels <= 0 || taps < 1 || taps > 64) return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  const long long count = (long long)tokens * channels;
  const dim3 grid(grid_for(count, 256)), block(256);
#define SAKV_CONV(W, C)                                                                          \
  return launch_ordered(causal_conv_kernel<W, C>, grid, block, 0, stream, in, stride,            \
                        (const W*)w, (const W*)bias, state, cu_seqlens, token_seq, slots,        \
                        (C*)out, channels, taps, count)
  if (w_dtype == SAKV_F32 && out_dtype == SAKV_F32) SAKV_CONV(float, float);
  if (w_dtype == SAKV_BF16 && out_dtype == SAKV_BF16) SAKV_CONV(__nv_bfloat16, __nv_bfloat16);
  if (w_dtype == SAKV_BF16 && out_dtype == SAKV_F32) SAKV_CONV(__nv_bfloat16, float);
  if (w_dtype == SAKV_F32 && out_dtype == SAKV_BF16) SAKV_CONV(float, __nv_bfloat16);
#undef SAKV_CONV
  return cudaErrorInvalidValue;
}

SAKV_EXPORT int sakv_conv_state(const float* in, long long stride, float* state,
                                const int32_t* cu_seqlens, const int32_t* slots, int sequences,
                                int channels, int taps, cudaStream_t stream) {
  if (sequences < 0 || channels <= 0 || taps < 1) return cudaErrorInvalidValue;
  if (sequences == 0 || taps == 1) return 0;
  const long long count = (long long)sequences * channels;
  return launch_ordered(conv_state_kernel, dim3((unsigned)((count + 255) / 256)), dim3(256), 0,
                        stream, in, stride, state, cu_seqlens, slots, channels, taps, sequences);
}

// low: fp32 [tokens, stride], its first `rank` columns; w: [channels, rank], bias [channels]
// of `w_dtype`; dt: fp32 [tokens, channels].
SAKV_EXPORT int sakv_step_size(const float* low, long long stride, int rank, const void* w,
                               const void* bias, int w_dtype, float* dt, int tokens, int channels,
                               cudaStream_t stream) {
  if (tokens < 0 || channels <= 0 || rank <= 0 || rank > 8192) return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  const size_t smem = (size_t)rank * sizeof(float);
  if (w_dtype == SAKV_F32)
    return launch_ordered(step_size_kernel<float>, dim3(tokens), dim3(256), smem, stream, low,
                          stride, rank, (const float*)w, (const float*)bias, dt, channels);
  if (w_dtype == SAKV_BF16)
    return launch_ordered(step_size_kernel<__nv_bfloat16>, dim3(tokens), dim3(256), smem, stream,
                          low, stride, rank, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias,
                          dt, channels);
  return cudaErrorInvalidValue;
}

// x: [tokens, channels] of `c_dtype` (the convolution's output); dt: fp32 [tokens, channels];
// low: fp32 [tokens, low_stride] with B at column b_off and C at c_off (n_state each); z: fp32
// rows `z_stride` apart (the gate's pre-activation); a_log [channels, n_state], d_skip
// [channels] of `w_dtype`; state: fp32 [slots, channels, n_state]. out: [tokens, channels] of
// `c_dtype` = (scan + d_skip x) * silu(z).
SAKV_EXPORT int sakv_selective_scan(const void* x, int c_dtype, const float* dt, const float* low,
                                    long long low_stride, int b_off, int c_off, const float* z,
                                    long long z_stride, const void* a_log, const void* d_skip,
                                    int w_dtype, float* state, const int32_t* cu_seqlens,
                                    const int32_t* slots, void* out, int tokens, int sequences,
                                    int channels, int n_state, int keep_state,
                                    cudaStream_t stream) {
  if (tokens < 0 || sequences < 0 || channels <= 0 || n_state <= 0 || n_state > 512)
    return cudaErrorInvalidValue;
  if (tokens == 0 || sequences == 0) return 0;
  const int per_lane = n_state <= 128 ? 4 : 16;
  const int lanes = lanes_for(n_state, per_lane);
  const long long threads = (long long)channels * lanes;
  // smaller blocks while the step's sequences and channels do not fill the GPU
  int block = 128;
  while (block > 32 && (threads + block - 1) / block * sequences < 2LL * sm_count()) block /= 2;
  const dim3 grid((unsigned)((threads + block - 1) / block), (unsigned)sequences);
#define SAKV_SCAN(NPT, W, C)                                                                     \
  return launch_ordered(selective_scan_kernel<NPT, W, C>, grid, dim3(block), 0, stream,          \
                        (const C*)x, dt, low, low_stride, b_off, c_off, z, z_stride,             \
                        (const W*)a_log, (const W*)d_skip, state, cu_seqlens, slots, (C*)out,    \
                        channels, n_state, lanes, keep_state)
#define SAKV_SCAN_T(NPT)                                                                         \
  do {                                                                                           \
    if (w_dtype == SAKV_F32 && c_dtype == SAKV_F32) SAKV_SCAN(NPT, float, float);                \
    if (w_dtype == SAKV_BF16 && c_dtype == SAKV_BF16) SAKV_SCAN(NPT, __nv_bfloat16, __nv_bfloat16); \
    if (w_dtype == SAKV_F32 && c_dtype == SAKV_BF16) SAKV_SCAN(NPT, float, __nv_bfloat16);       \
    if (w_dtype == SAKV_BF16 && c_dtype == SAKV_F32) SAKV_SCAN(NPT, __nv_bfloat16, float);       \
  } while (0)
  if (per_lane == 4) SAKV_SCAN_T(4);
  else SAKV_SCAN_T(16);
#undef SAKV_SCAN_T
#undef SAKV_SCAN
  return cudaErrorInvalidValue;
}

// proj: fp32 [tokens, stride] with the pre-activations of q at q_off (heads * dim), k at k_off
// (heads * dim) and v at v_off (heads * vdim); decay: fp32 [heads] holding `decay - 1` (the
// state moves by `(decay - 1) S + k v^T`, so a decay close to 1 loses nothing to rounding);
// state: fp32 [slots, heads, vdim, dim]. out: fp32 [tokens, heads * vdim] = S^T q after the
// token's update.
SAKV_EXPORT int sakv_decay_attention(const float* proj, long long stride, int q_off, int k_off,
                                     int v_off, const float* decay, float* state,
                                     const int32_t* cu_seqlens, const int32_t* slots, float* out,
                                     int tokens, int sequences, int heads, int dim, int vdim,
                                     int keep_state, cudaStream_t stream) {
  if (tokens < 0 || sequences < 0 || heads <= 0 || dim <= 0 || dim > 256 || vdim <= 0)
    return cudaErrorInvalidValue;
  if (tokens == 0 || sequences == 0) return 0;
  const int rp = dim <= 128 ? 4 : 8;
  const int rs = lanes_for(dim, rp);
  int cols = 256 / rs;                       // value columns a block
  // fewer columns a block while the step's heads and sequences do not fill the GPU
  while (cols > 1 && (long long)((vdim + cols - 1) / cols) * heads * sequences < 2LL * sm_count())
    cols /= 2;
  while (cols > 1 && cols / 2 >= vdim) cols /= 2;
  if (cols * rs < 32) cols = 32 / rs;        // whole warps
  const dim3 grid((unsigned)((vdim + cols - 1) / cols), (unsigned)heads, (unsigned)sequences);
  const size_t smem = (size_t)kRun * (2 * rs * rp + cols) * sizeof(float);
  if (rp == 4)
    return launch_ordered(decay_attention_kernel<4>, grid, dim3(cols * rs), smem, stream, proj,
                          stride, q_off, k_off, v_off, decay, state, cu_seqlens, slots, out, heads,
                          dim, vdim, rs, cols, keep_state);
  return launch_ordered(decay_attention_kernel<8>, grid, dim3(cols * rs), smem, stream, proj,
                        stride, q_off, k_off, v_off, decay, state, cu_seqlens, slots, out, heads,
                        dim, vdim, rs, cols, keep_state);
}

// y: fp32 [tokens, width]; w: [width] of `w_dtype`; gate: fp32 rows `gate_stride` apart (null:
// none). out: [tokens, width] of `out_dtype`.
SAKV_EXPORT int sakv_norm_gate(const float* y, const void* w, int w_dtype, const float* gate,
                               long long gate_stride, void* out, int out_dtype, int tokens,
                               int width, float eps, float scale, cudaStream_t stream) {
  if (tokens < 0 || width <= 0) return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
#define SAKV_NG(W, C)                                                                            \
  return launch_ordered(norm_gate_kernel<W, C>, dim3(tokens), dim3(256), 0, stream, y,           \
                        (const W*)w, gate, gate_stride, (C*)out, width, eps, scale)
  if (w_dtype == SAKV_F32 && out_dtype == SAKV_F32) SAKV_NG(float, float);
  if (w_dtype == SAKV_BF16 && out_dtype == SAKV_BF16) SAKV_NG(__nv_bfloat16, __nv_bfloat16);
  if (w_dtype == SAKV_BF16 && out_dtype == SAKV_F32) SAKV_NG(__nv_bfloat16, float);
  if (w_dtype == SAKV_F32 && out_dtype == SAKV_BF16) SAKV_NG(float, __nv_bfloat16);
#undef SAKV_NG
  return cudaErrorInvalidValue;
}
