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

// e^x - 1 for x <= 0, to about 1e-7 of ITSELF where x is small (what a decay close to 1 needs:
// its distance from 1) and to about 2e-7 absolutely elsewhere. EXACT: the library's expm1f
// (1 ulp, some thirty instructions); otherwise six terms of the series below 1/8 and the
// hardware exponential above (a dozen instructions), for the 16-bit mode, whose scan is bound
// by instruction issue.
template <bool EXACT>
__device__ __forceinline__ float exp_less_one(float x) {
  if (EXACT) return expm1f(x);
  const float series = x * fmaf(x, fmaf(x, fmaf(x, fmaf(x, fmaf(x, 1.f / 720.f, 1.f / 120.f),
                                                        1.f / 24.f), 1.f / 6.f), 0.5f), 1.f);
  return x > -0.125f ? series : __expf(x) - 1.f;
}

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

// Both of the above in one launch for a step in which every sequence brings one token: a
// thread a (sequence, channel) reads the running inputs, adds the products in the same order
// as the kernel above, and moves the running inputs up by one.
template <typename W, typename C>
__global__ void conv_step_kernel(const float* __restrict__ in, long long stride,
                                 const W* __restrict__ w, const W* __restrict__ bias,
                                 float* __restrict__ state, const int32_t* __restrict__ slots,
                                 C* __restrict__ out, int channels, int taps, long long count,
                                 int keep_state) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= count) return;
  const long long b = idx / channels;
  const int c = static_cast<int>(idx - b * channels);
  float* old = state + (long long)slots[b] * (taps - 1) * channels + c;
  const float now = in[b * stride + c];
  float acc = bias ? widen(bias[c]) : 0.f;
  for (int j = 0; j + 1 < taps; ++j)
    acc = fmaf(old[(long long)j * channels], widen(w[(long long)c * taps + j]), acc);
  acc = fmaf(now, widen(w[(long long)c * taps + taps - 1]), acc);
  out[idx] = narrow<C>(silu(acc));
  if (keep_state && taps > 1) {
    for (int j = 0; j + 2 < taps; ++j) old[(long long)j * channels] = old[(long long)(j + 1) * channels];
    old[(long long)(taps - 2) * channels] = now;
  }
}

// ---------------------------------------------------------------------------------------
// Step sizes: dt[t, c] = softplus(sum_r low[t, r] Wdt[c, r] + b[c]), a tiled fp32 product
// (plain FFMA): a block of 256 threads makes BM tokens x 64 channels, a thread TM x 4 of
// them, both operands staged through shared memory 16 numbers of the sum at a time. Every
// output adds its products in the order r = 0, 1, 2, ... whatever the tile.
// ---------------------------------------------------------------------------------------
constexpr int kStepN = 64, kStepK = 16;

template <int BM, typename W>
__global__ void __launch_bounds__(256)
step_size_kernel(const float* __restrict__ low, long long stride, int rank,
                 const W* __restrict__ w, const W* __restrict__ bias, float* __restrict__ dt,
                 int tokens, int channels) {
  constexpr int TM = BM / 16;
  __shared__ float As[kStepK][BM + 4];
  __shared__ float Ws[kStepK][kStepN + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * kStepN;
  float acc[TM][4];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < rank; k0 += kStepK) {
    for (int i = threadIdx.x; i < BM * kStepK; i += 256) {
      const int r = i / kStepK, c = i % kStepK;
      const int m = m0 + r, k = k0 + c;
      As[c][r] = (m < tokens && k < rank) ? low[(long long)m * stride + k] : 0.f;
    }
    for (int i = threadIdx.x; i < kStepN * kStepK; i += 256) {
      const int r = i / kStepK, c = i % kStepK;
      const int n = n0 + r, k = k0 + c;
      Ws[c][r] = (n < channels && k < rank) ? widen(w[(long long)n * rank + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kStepK; ++k) {
      float a[TM], b[4];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= tokens) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < channels)
        dt[(long long)m * channels + n] = softplus(acc[i][j] + (bias ? widen(bias[n]) : 0.f));
    }
  }
}

// ---------------------------------------------------------------------------------------
// The selective scan. A channel's N states are dealt to G neighbouring lanes, NPT each
// (state n = g * NPT + k belongs to lane g); a lane keeps its states in registers for the
// whole step, the sum over the states ends with log2(G) shuffles. Blocks: (channels * G /
// blockDim, sequences). State in memory: [slots, channels, N].
//
// A long prompt is cut into runs of `chunk_len` tokens that are walked side by side, in
// three launches. PHASE 1: every run starts from zero and leaves its end state and the sum of
// its step sizes in scratch memory ([sequences, max_chunks, channels, N] and [..., channels]).
// The carry kernel then walks a sequence's runs in order: the state a run starts from replaces
// what the run left, S <- exp(A sum dt) S + left. PHASE 2: every run starts from there and
// writes its outputs. PHASE 0 is the whole step by one walk (the sums then do not depend on
// how a sequence was cut into steps).
// ---------------------------------------------------------------------------------------
template <int NPT, int PHASE, typename W, typename C>
__global__ void selective_scan_kernel(const C* __restrict__ x, const float* __restrict__ dt,
                                      const float* __restrict__ low, long long low_stride,
                                      int b_off, int c_off, const float* __restrict__ z,
                                      long long z_stride, const W* __restrict__ a_log,
                                      const W* __restrict__ d_skip, float* __restrict__ state,
                                      const int32_t* __restrict__ cu_seqlens,
                                      const int32_t* __restrict__ slots, C* __restrict__ out,
                                      int channels, int n_state, int lanes, int keep_state,
                                      int chunk_len, int max_chunks, float* __restrict__ scratch,
                                      float* __restrict__ dt_sums, const W* __restrict__ w_dt,
                                      const W* __restrict__ b_dt, int rank) {
  const int b = PHASE == 0 ? blockIdx.y : blockIdx.y / max_chunks;
  const int run = PHASE == 0 ? 0 : blockIdx.y % max_chunks;
  int first = cu_seqlens[b], last = cu_seqlens[b + 1];
  if (PHASE != 0) {
    first += run * chunk_len;
    if (first >= last) return;                        // (the whole block: b and run are its own)
    if (last - first > chunk_len) last = first + chunk_len;
  }
  const long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const int c_raw = static_cast<int>(id / lanes), g = static_cast<int>(id % lanes);
  const bool live = c_raw < channels;                 // (idle lanes still join the shuffles)
  const int c = live ? c_raw : channels - 1;
  const int n0 = g * NPT;
  float a[NPT], s[NPT];
  float* mine = PHASE == 0
                    ? state + ((long long)slots[b] * channels + c) * n_state + n0
                    : scratch + (((long long)b * max_chunks + run) * channels + c) * n_state + n0;
#pragma unroll
  for (int k = 0; k < NPT; ++k) {
    const bool has = n0 + k < n_state;
    a[k] = has ? -expf(widen(a_log[(long long)c * n_state + n0 + k])) : 0.f;
    s[k] = (has && PHASE != 1) ? mine[k] : 0.f;
  }
  const float skip = widen(d_skip[c]);
  float dt_sum = 0.f;
  for (int t = first; t < last; ++t) {
    float step;
    if (PHASE == 0 && dt == nullptr) {
      // the step size made here (a step of few tokens): the same products in the same order
      // as the tiled kernel adds them
      const float* lt = low + (long long)t * low_stride;
      const W* wr = w_dt + (long long)c * rank;
      float acc = 0.f;
      for (int r = 0; r < rank; ++r) acc = fmaf(lt[r], widen(wr[r]), acc);
      step = softplus(acc + (b_dt ? widen(b_dt[c]) : 0.f));
    } else {
      step = dt[(long long)t * channels + c];
    }
    const float xv = widen(x[(long long)t * channels + c]);
    const float* bt = low + (long long)t * low_stride + b_off + n0;
    const float* ct = low + (long long)t * low_stride + c_off + n0;
    const float dx = step * xv;
    dt_sum += step;
    float y = 0.f;
#pragma unroll
    for (int k = 0; k < NPT; ++k) {
      const bool has = n0 + k < n_state;
      const float bv = has ? bt[k] : 0.f;
      // S + (e^(dt A) - 1) S + dt x B: a decay close to 1 keeps its distance from 1 exactly
      s[k] += fmaf(exp_less_one<sizeof(C) == 4>(step * a[k]), s[k], dx * bv);
      if (PHASE != 1) y = fmaf(s[k], has ? ct[k] : 0.f, y);
    }
    if (PHASE != 1) {
      for (int o = lanes >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (g == 0 && live) {
        y = fmaf(skip, xv, y);
        out[(long long)t * channels + c] = narrow<C>(y * silu(z[(long long)t * z_stride + c]));
      }
    }
  }
  if (live && (PHASE == 1 || (PHASE == 0 && keep_state))) {
#pragma unroll
    for (int k = 0; k < NPT; ++k)
      if (n0 + k < n_state) mine[k] = s[k];
  }
  if (PHASE == 1 && live && g == 0)
    dt_sums[((long long)b * max_chunks + run) * channels + c] = dt_sum;
}

// Between the two passes over a prompt's runs: one thread a (sequence, channel, state) walks
// the runs in order. What a run left (its end state from zero) is replaced by the state it
// starts from; the state after the last run goes back to the sequence's slot.
template <typename W>
__global__ void scan_carry_kernel(const W* __restrict__ a_log, float* __restrict__ state,
                                  float* __restrict__ scratch, const float* __restrict__ dt_sums,
                                  const int32_t* __restrict__ cu_seqlens,
                                  const int32_t* __restrict__ slots, int sequences, int channels,
                                  int n_state, int chunk_len, int max_chunks, int keep_state) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long per = (long long)channels * n_state;
  if (idx >= sequences * per) return;
  const int b = static_cast<int>(idx / per);
  const long long cn = idx - b * per;
  const int c = static_cast<int>(cn / n_state);
  const int runs = (cu_seqlens[b + 1] - cu_seqlens[b] + chunk_len - 1) / chunk_len;
  const float a = -expf(widen(a_log[cn]));
  float* home = state + (long long)slots[b] * per + cn;
  float s = *home;
  for (int j = 0; j < runs; ++j) {
    float* p = scratch + ((long long)b * max_chunks + j) * per + cn;
    const float left = *p;
    *p = s;
    s += fmaf(expm1f(a * dt_sums[((long long)b * max_chunks + j) * channels + c]), s, left);
  }
  if (keep_state) *home = s;
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

// What shapes q, k and v on their way into shared memory: `act` 1 is silu of each element
// (0: as projected); `rot` > 0 turns the first `rot` numbers of every head of q and k by the
// token's position (pairs (i, i + rot / 2), tables [positions, rot / 2] that carry the
// rotation's magnitude), after the activation; `k_scale` multiplies k after that.
struct FadeInput {
  int act;
  int rot;
  const int32_t* positions;
  const float* cos_t;
  const float* sin_t;
  float k_scale;
};

__device__ __forceinline__ float fade_act(float x, int act) { return act ? silu(x) : x; }

// One token's head of q or k from `head` (global) to `to` (shared), `padded` floats of which
// the first `dim` are real, times `scale`; element `i` is this thread's. A rotated pair is
// made by the thread of its lower half, which reads both numbers and the angle once.
__device__ __forceinline__ void fade_stage(const float* __restrict__ head, float* __restrict__ to,
                                           int i, int dim, int pos, float scale,
                                           const FadeInput& in) {
  const int half = in.rot >> 1;
  if (i >= half && i < in.rot) return;                 // its partner's thread writes it
  if (i >= dim) {
    to[i] = 0.f;
    return;
  }
  const float x = fade_act(head[i], in.act);
  if (i >= in.rot) {
    to[i] = x * scale;
    return;
  }
  const float y = fade_act(head[i + half], in.act);
  const float c = in.cos_t[(long long)pos * half + i], sn = in.sin_t[(long long)pos * half + i];
  to[i] = (x * c - y * sn) * scale;
  to[i + half] = (y * c + x * sn) * scale;
}

// PHASE as in the selective scan: 0 walks a sequence's whole part of the step from the state in
// its slot; 1 walks one run of `chunk_len` tokens from zero and leaves the end state in scratch
// memory ([sequences, max_chunks, heads, vdim, dim]), without outputs; 2 walks a run from the
// state that the carry kernel put there and writes the outputs.
template <int RP, int PHASE>
__global__ void decay_attention_kernel(const float* __restrict__ proj, long long stride,
                                       int q_off, int k_off, int v_off,
                                       const float* __restrict__ decay_less_one,
                                       float* __restrict__ state,
                                       const int32_t* __restrict__ cu_seqlens,
                                       const int32_t* __restrict__ slots, float* __restrict__ out,
                                       int heads, int dim, int vdim, int rs, int cols,
                                       int keep_state, int chunk_len, int max_chunks,
                                       float* __restrict__ scratch, const FadeInput in) {
  extern __shared__ __align__(16) float shared[];
  const int padded = rs * RP;                       // dim rounded up to whole lanes
  const int padded_shift = 31 - __clz(padded);
  float* qs = shared;                               // [kRun, padded]
  float* ks = qs + kRun * padded;                   // [kRun, padded]
  float* vs = ks + kRun * padded;                   // [kRun, cols]
  const int b = PHASE == 0 ? blockIdx.z : blockIdx.z / max_chunks;
  const int piece = PHASE == 0 ? 0 : blockIdx.z % max_chunks;
  int first = cu_seqlens[b], last = cu_seqlens[b + 1];
  if (PHASE != 0) {
    first += piece * chunk_len;
    if (first >= last) return;                      // (the whole block)
    if (last - first > chunk_len) last = first + chunk_len;
  }
  const int h = blockIdx.y, col0 = blockIdx.x * cols;
  const int r = threadIdx.x % rs, j = threadIdx.x / rs;
  const int col = col0 + j;
  const bool live = col < vdim;
  const float fade = decay_less_one[h];        // decay - 1, rounded once from the exact number
  float s[RP];
  const long long place = ((long long)h * vdim + (live ? col : 0)) * dim + r * RP;
  float* mine = PHASE == 0
                    ? state + (long long)slots[b] * heads * vdim * dim + place
                    : scratch + ((long long)b * max_chunks + piece) * heads * vdim * dim + place;
#pragma unroll
  for (int k = 0; k < RP; ++k) s[k] = (PHASE != 1 && live && r * RP + k < dim) ? mine[k] : 0.f;
  for (int t0 = first; t0 < last; t0 += kRun) {
    const int run = last - t0 < kRun ? last - t0 : kRun;
    __syncthreads();
    for (int e = threadIdx.x; e < run * padded; e += blockDim.x) {
      const int tt = e >> padded_shift, i = e & (padded - 1);     // (padded is a power of two)
      const float* row = proj + (long long)(t0 + tt) * stride + (long long)h * dim;
      const int pos = in.rot ? in.positions[t0 + tt] : 0;
      if (PHASE != 1) fade_stage(row + q_off, qs + tt * padded, i, dim, pos, 1.f, in);
      fade_stage(row + k_off, ks + tt * padded, i, dim, pos, in.k_scale, in);
    }
    for (int e = threadIdx.x; e < run * cols; e += blockDim.x) {
      const int tt = e / cols, i = e - tt * cols;
      float v = 0.f;
      if (col0 + i < vdim) {
        v = proj[(long long)(t0 + tt) * stride + v_off + (long long)h * vdim + col0 + i];
        if (in.act) v = silu(v);
      }
      vs[e] = v;
    }
    __syncthreads();
    for (int tt = 0; tt < run; ++tt) {
      const float v = vs[tt * cols + j];
      float o = 0.f;
      // a lane's rows of k and q lie together: four at a time (RP is 4 or 8; the offsets are
      // multiples of four floats); S + (decay - 1) S in one rounding, then k v added by the next
      const float4* k4 = reinterpret_cast<const float4*>(ks + tt * padded + r * RP);
      const float4* q4 = reinterpret_cast<const float4*>(qs + tt * padded + r * RP);
#pragma unroll
      for (int k = 0; k < RP; k += 4) {
        const float4 kk = k4[k >> 2];
        s[k] = fmaf(kk.x, v, fmaf(fade, s[k], s[k]));
        s[k + 1] = fmaf(kk.y, v, fmaf(fade, s[k + 1], s[k + 1]));
        s[k + 2] = fmaf(kk.z, v, fmaf(fade, s[k + 2], s[k + 2]));
        s[k + 3] = fmaf(kk.w, v, fmaf(fade, s[k + 3], s[k + 3]));
        if (PHASE != 1) {
          const float4 qq = q4[k >> 2];
          o = fmaf(s[k], qq.x, o);
          o = fmaf(s[k + 1], qq.y, o);
          o = fmaf(s[k + 2], qq.z, o);
          o = fmaf(s[k + 3], qq.w, o);
        }
      }
      if (PHASE != 1) {
        for (int d = rs >> 1; d > 0; d >>= 1) o += __shfl_xor_sync(0xffffffffu, o, d);
        if (r == 0 && live) out[((long long)(t0 + tt) * heads + h) * vdim + col] = o;
      }
    }
  }
  if (live && (PHASE == 1 || (PHASE == 0 && keep_state))) {
#pragma unroll
    for (int k = 0; k < RP; ++k)
      if (r * RP + k < dim) mine[k] = s[k];
  }
}

// Between the two passes over a prompt's runs: one thread a (sequence, head, column, row) walks
// the runs in order; a run of n tokens fades what came before by decay^n.
__global__ void decay_carry_kernel(const float* __restrict__ decay_less_one,
                                   float* __restrict__ state, float* __restrict__ scratch,
                                   const int32_t* __restrict__ cu_seqlens,
                                   const int32_t* __restrict__ slots, int sequences, int heads,
                                   long long per_head, int chunk_len, int max_chunks,
                                   int keep_state) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long per = heads * per_head;
  if (idx >= sequences * per) return;
  const int b = static_cast<int>(idx / per);
  const long long e = idx - b * per;
  const int n = cu_seqlens[b + 1] - cu_seqlens[b];
  const int runs = (n + chunk_len - 1) / chunk_len;
  const float log_fade = log1pf(decay_less_one[e / per_head]);
  float* home = state + (long long)slots[b] * per + e;
  float s = *home;
  for (int j = 0; j < runs; ++j) {
    float* p = scratch + ((long long)b * max_chunks + j) * per + e;
    const float left = *p;
    *p = s;
    const int len = n - j * chunk_len < chunk_len ? n - j * chunk_len : chunk_len;
    s += fmaf(expm1f(log_fade * static_cast<float>(len)), s, left);
  }
  if (keep_state) *home = s;
}

// out[t] = y[t] / sqrt(mean(y[t]^2) + eps) * w * sigmoid(gate[t]) * scale. A block a token.
// `group` == width: the mean over the whole row (all heads' outputs together); smaller: over
// each run of `group` numbers (a head's outputs), a warp a run. `w` null: no weight.
// `gate_silu`: the gate is `g * sigmoid(g)` instead of `sigmoid(g)`.
template <typename W, typename C>
__global__ void __launch_bounds__(256)
norm_gate_kernel(const float* __restrict__ y, const W* __restrict__ w,
                 const float* __restrict__ gate, long long gate_stride, C* __restrict__ out,
                 int width, int group, int gate_silu, float eps, float scale) {
  __shared__ float scratch[33];
  const long long t = blockIdx.x;
  const float* row = y + t * width;
  auto finish = [&](int i, float r) {
    float v = row[i] * r;
    if (w) v *= widen(w[i]);
    if (gate) {
      const float g = gate[t * gate_stride + i];
      v *= (gate_silu ? g : 1.f) / (1.f + expf(-g));
    }
    out[t * width + i] = narrow<C>(v * scale);
  };
  if (group == width) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
    const float r = 1.f / sqrtf(block_sum(ss, scratch) / static_cast<float>(width) + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) finish(i, r);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int g0 = warp * group; g0 < width; g0 += warps * group) {
    float ss = 0.f;
    for (int i = lane; i < group; i += 32) ss = fmaf(row[g0 + i], row[g0 + i], ss);
    const float r = 1.f / sqrtf(warp_sum(ss) / static_cast<float>(group) + eps);
    for (int i = lane; i < group; i += 32) finish(g0 + i, r);
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

// `sakv_causal_conv` and `sakv_conv_state` in one launch for a step in which each of `sequences`
// sequences brings one token (token b belongs to sequence b).
SAKV_EXPORT int sakv_conv_step(const float* in, long long stride, const void* w, const void* bias,
                               int w_dtype, float* state, const int32_t* slots, void* out,
                               int out_dtype, int sequences, int channels, int taps,
                               int keep_state, cudaStream_t stream) {
  if (sequences < 0 || channels <= 0 || taps < 1 || taps > 64) return cudaErrorInvalidValue;
  if (sequences == 0) return 0;
  const long long count = (long long)sequences * channels;
  const dim3 grid((unsigned)((count + 127) / 128)), block(128);
#define SAKV_CONV(W, C)                                                                          \
  return launch_ordered(conv_step_kernel<W, C>, grid, block, 0, stream, in, stride, (const W*)w, \
                        (const W*)bias, state, slots, (C*)out, channels, taps, count, keep_state)
  if (w_dtype == SAKV_F32 && out_dtype == SAKV_F32) SAKV_CONV(float, float);
  if (w_dtype == SAKV_BF16 && out_dtype == SAKV_BF16) SAKV_CONV(__nv_bfloat16, __nv_bfloat16);
  if (w_dtype == SAKV_BF16 && out_dtype == SAKV_F32) SAKV_CONV(__nv_bfloat16, float);
  if (w_dtype == SAKV_F32 && out_dtype == SAKV_BF16) SAKV_CONV(float, __nv_bfloat16);
#undef SAKV_CONV
  return cudaErrorInvalidValue;
}

// low: fp32 [tokens, stride], its first `rank` columns; w: [channels, rank], bias [channels]
// of `w_dtype`; dt: fp32 [tokens, channels].
SAKV_EXPORT int sakv_step_size(const float* low, long long stride, int rank, const void* w,
                               const void* bias, int w_dtype, float* dt, int tokens, int channels,
                               cudaStream_t stream) {
  if (tokens < 0 || channels <= 0 || rank <= 0) return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  const bool few = tokens <= 16;
  const dim3 grid((unsigned)((channels + kStepN - 1) / kStepN),
                  (unsigned)((tokens + (few ? 15 : 63)) / (few ? 16 : 64)));
#define SAKV_STEP(BM, W)                                                                         \
  return launch_ordered(step_size_kernel<BM, W>, grid, dim3(256), 0, stream, low, stride, rank,  \
                        (const W*)w, (const W*)bias, dt, tokens, channels)
  if (w_dtype == SAKV_F32) {
    if (few) SAKV_STEP(16, float);
    SAKV_STEP(64, float);
  }
  if (w_dtype == SAKV_BF16) {
    if (few) SAKV_STEP(16, __nv_bfloat16);
    SAKV_STEP(64, __nv_bfloat16);
  }
#undef SAKV_STEP
  return cudaErrorInvalidValue;
}

// x: [tokens, channels] of `c_dtype` (the convolution's output); dt: fp32 [tokens, channels];
// low: fp32 [tokens, low_stride] with B at column b_off and C at c_off (n_state each); z: fp32
// rows `z_stride` apart (the gate's pre-activation); a_log [channels, n_state], d_skip
// [channels] of `w_dtype`; state: fp32 [slots, channels, n_state]. out: [tokens, channels] of
// `c_dtype` = (scan + d_skip x) * silu(z). `dt` null: dt = softplus(low[:, :rank] w_dt^T + b_dt)
// is made in the kernel (w_dt [channels, rank], b_dt [channels] or null, of `w_dtype`).
SAKV_EXPORT int sakv_selective_scan(const void* x, int c_dtype, const float* dt, const float* low,
                                    long long low_stride, int b_off, int c_off, const float* z,
                                    long long z_stride, const void* a_log, const void* d_skip,
                                    int w_dtype, float* state, const int32_t* cu_seqlens,
                                    const int32_t* slots, void* out, int tokens, int sequences,
                                    int channels, int n_state, int keep_state, int chunk_len,
                                    int max_chunks, float* scratch, float* dt_sums,
                                    const void* w_dt, const void* b_dt, int rank,
                                    cudaStream_t stream) {
  if (tokens < 0 || sequences < 0 || channels <= 0 || n_state <= 0 || n_state > 512)
    return cudaErrorInvalidValue;
  // dt null: the step sizes are made in the kernel from low's first `rank` columns (one walk only)
  if (dt == nullptr && (w_dt == nullptr || rank <= 0 || chunk_len > 0)) return cudaErrorInvalidValue;
  if (tokens == 0 || sequences == 0) return 0;
  const bool runs = chunk_len > 0;
  if (runs && (max_chunks <= 0 || scratch == nullptr || dt_sums == nullptr ||
               (long long)sequences * max_chunks > 65535))
    return cudaErrorInvalidValue;
  const int per_lane = n_state <= 128 ? 4 : 16;
  const int lanes = lanes_for(n_state, per_lane);
  const long long threads = (long long)channels * lanes;
  const long long walks = runs ? (long long)sequences * max_chunks : sequences;
  // smaller blocks while the step's walks and channels do not fill the GPU
  int block = 128;
  while (block > 32 && (threads + block - 1) / block * walks < 2LL * sm_count()) block /= 2;
  const dim3 grid((unsigned)((threads + block - 1) / block), (unsigned)walks);
#define SAKV_SCAN(NPT, PHASE, W, C)                                                              \
  launch_ordered(selective_scan_kernel<NPT, PHASE, W, C>, grid, dim3(block), 0, stream,          \
                 (const C*)x, dt, low, low_stride, b_off, c_off, z, z_stride, (const W*)a_log,   \
                 (const W*)d_skip, state, cu_seqlens, slots, (C*)out, channels, n_state, lanes,  \
                 keep_state, chunk_len, max_chunks, scratch, dt_sums, (const W*)w_dt,            \
                 (const W*)b_dt, rank)
#define SAKV_SCAN_ALL(NPT, W, C)                                                                 \
  do {                                                                                           \
    if (!runs) return SAKV_SCAN(NPT, 0, W, C);                                                   \
    int code = SAKV_SCAN(NPT, 1, W, C);                                                          \
    if (code) return code;                                                                       \
    const long long count = (long long)sequences * channels * n_state;                           \
    code = launch_ordered(scan_carry_kernel<W>, dim3((unsigned)((count + 127) / 128)),           \
                          dim3(128), 0, stream, (const W*)a_log, state, scratch, dt_sums,        \
                          cu_seqlens, slots, sequences, channels, n_state, chunk_len,            \
                          max_chunks, keep_state);                                               \
    if (code) return code;                                                                       \
    return SAKV_SCAN(NPT, 2, W, C);                                                              \
  } while (0)
#define SAKV_SCAN_T(NPT)                                                                         \
  do {                                                                                           \
    if (w_dtype == SAKV_F32 && c_dtype == SAKV_F32) SAKV_SCAN_ALL(NPT, float, float);            \
    if (w_dtype == SAKV_BF16 && c_dtype == SAKV_BF16)                                            \
      SAKV_SCAN_ALL(NPT, __nv_bfloat16, __nv_bfloat16);                                          \
    if (w_dtype == SAKV_F32 && c_dtype == SAKV_BF16) SAKV_SCAN_ALL(NPT, float, __nv_bfloat16);   \
    if (w_dtype == SAKV_BF16 && c_dtype == SAKV_F32) SAKV_SCAN_ALL(NPT, __nv_bfloat16, float);   \
  } while (0)
  if (per_lane == 4) SAKV_SCAN_T(4);
  else SAKV_SCAN_T(16);
#undef SAKV_SCAN_T
#undef SAKV_SCAN_ALL
#undef SAKV_SCAN
  return cudaErrorInvalidValue;
}

// proj: fp32 [tokens, stride] with the pre-activations of q at q_off (heads * dim), k at k_off
// (heads * dim) and v at v_off (heads * vdim); decay: fp32 [heads] holding `decay - 1` (the
// state moves by `(decay - 1) S + k v^T`, so a decay close to 1 loses nothing to rounding);
// state: fp32 [slots, heads, vdim, dim]. out: fp32 [tokens, heads * vdim] = S^T q after the
// token's update. act: 1 = silu of q, k, v (0: as they are). rot > 0: the first `rot` numbers
// of every head of q and k are turned by positions[t] (int32 [tokens]) with the tables cos_t,
// sin_t (fp32 [positions, rot / 2]); k_scale multiplies k afterwards.
SAKV_EXPORT int sakv_decay_attention(const float* proj, long long stride, int q_off, int k_off,
                                     int v_off, const float* decay, float* state,
                                     const int32_t* cu_seqlens, const int32_t* slots, float* out,
                                     int tokens, int sequences, int heads, int dim, int vdim,
                                     int keep_state, int chunk_len, int max_chunks, float* scratch,
                                     int act, int rot, const int32_t* positions,
                                     const float* cos_t, const float* sin_t, float k_scale,
                                     cudaStream_t stream) {
  if (tokens < 0 || sequences < 0 || heads <= 0 || dim <= 0 || dim > 256 || vdim <= 0 ||
      rot < 0 || rot % 2 || rot > dim || (rot > 0 && (!positions || !cos_t || !sin_t)))
    return cudaErrorInvalidValue;
  if (tokens == 0 || sequences == 0) return 0;
  const FadeInput in = {act, rot, positions, cos_t, sin_t, k_scale};
  const bool runs = chunk_len > 0;
  if (runs && (max_chunks <= 0 || scratch == nullptr ||
               (long long)sequences * max_chunks > 65535))
    return cudaErrorInvalidValue;
  const long long walks = runs ? (long long)sequences * max_chunks : sequences;
  const int rp = dim < 128 ? 4 : 8;        // (rows a lane; 16 lanes a column from 128 rows on)
  const int rs = lanes_for(dim, rp);
  int cols = 256 / rs;                       // value columns a block
  // fewer columns a block while the step's heads and walks do not fill the GPU
  while (cols > 1 && (long long)((vdim + cols - 1) / cols) * heads * walks < 2LL * sm_count())
    cols /= 2;
  while (cols > 1 && cols / 2 >= vdim) cols /= 2;
  if (cols * rs < 32) cols = 32 / rs;        // whole warps
  const dim3 grid((unsigned)((vdim + cols - 1) / cols), (unsigned)heads, (unsigned)walks);
  const size_t smem = (size_t)kRun * (2 * rs * rp + cols) * sizeof(float);
#define SAKV_FADE(RP, PHASE)                                                                     \
  launch_ordered(decay_attention_kernel<RP, PHASE>, grid, dim3(cols * rs), smem, stream, proj,   \
                 stride, q_off, k_off, v_off, decay, state, cu_seqlens, slots, out, heads, dim,  \
                 vdim, rs, cols, keep_state, chunk_len, max_chunks, scratch, in)
#define SAKV_FADE_ALL(RP)                                                                        \
  do {                                                                                           \
    if (!runs) return SAKV_FADE(RP, 0);                                                          \
    int code = SAKV_FADE(RP, 1);                                                                 \
    if (code) return code;                                                                       \
    const long long per_head = (long long)vdim * dim;                                            \
    const long long count = (long long)sequences * heads * per_head;                             \
    code = launch_ordered(decay_carry_kernel, dim3((unsigned)((count + 127) / 128)), dim3(128),  \
                          0, stream, decay, state, scratch, cu_seqlens, slots, sequences, heads, \
                          per_head, chunk_len, max_chunks, keep_state);                          \
    if (code) return code;                                                                       \
    return SAKV_FADE(RP, 2);                                                                     \
  } while (0)
  if (rp == 4) SAKV_FADE_ALL(4);
  SAKV_FADE_ALL(8);
#undef SAKV_FADE_ALL
#undef SAKV_FADE
}

// y: fp32 [tokens, width]; w: [width] of `w_dtype` (null: no weight); gate: fp32 rows
// `gate_stride` apart (null: none), used as sigmoid(g), or g sigmoid(g) with `gate_silu`.
// group: how many numbers share a root mean square (width: the whole row; it divides width).
// out: [tokens, width] of `out_dtype`.
SAKV_EXPORT int sakv_norm_gate(const float* y, const void* w, int w_dtype, const float* gate,
                               long long gate_stride, void* out, int out_dtype, int tokens,
                               int width, int group, int gate_silu, float eps, float scale,
                               cudaStream_t stream) {
  if (tokens < 0 || width <= 0 || group <= 0 || width % group) return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
#define SAKV_NG(W, C)                                                                            \
  return launch_ordered(norm_gate_kernel<W, C>, dim3(tokens), dim3(256), 0, stream, y,           \
                        (const W*)w, gate, gate_stride, (C*)out, width, group, gate_silu, eps,     \
                        scale)
  if (w_dtype == SAKV_F32 && out_dtype == SAKV_F32) SAKV_NG(float, float);
  if (w_dtype == SAKV_BF16 && out_dtype == SAKV_BF16) SAKV_NG(__nv_bfloat16, __nv_bfloat16);
  if (w_dtype == SAKV_BF16 && out_dtype == SAKV_F32) SAKV_NG(__nv_bfloat16, float);
  if (w_dtype == SAKV_F32 && out_dtype == SAKV_BF16) SAKV_NG(float, __nv_bfloat16);
#undef SAKV_NG
  return cudaErrorInvalidValue;
}
