// A mixture of small gated feed-forwards, routed on the device.
//
//   route    a warp a token: the `top` largest router scores (ties: the lowest index), the
//            scores as weights, and the token's place among the rows of each chosen expert.
//            A score is the sigmoid of the logit, or the softmax over all the router's
//            outputs; a bias an output may be added for the choice only. Outputs beyond the
//            experts that have weights are identity experts: they take no rows, and combine
//            adds the token's own input times the weight for them
//   plan     one block: where each expert's rows begin and which (expert, first row) every
//            tile of `TM` rows of the grouped products covers (for a step of few tokens the
//            same block chooses for all of them first: one launch instead of two)
//   gather   the experts' input rows, sorted by expert: x * weight (the weight multiplies an
//            expert's INPUT) rounded once to the activations' type
//   products out = rows x W[e]^T for every tile, with the weights of the tile's expert:
//            the gated pair with the clamped activation in its epilogue
//              g = min(., limit), u = clamp(., -limit, limit), y = g * sigmoid(alpha g) * (u + 1)
//            and the plain product that leaves fp32
//   combine  a token's rows summed in the order of its choices, plus the shared expert's
//            output times sigmoid of its gate's logit
//
// Nothing is read back by the host: the grid of the products is sized for the most tiles
// there can be, and blocks beyond the planned count leave at once. A row's result does not
// depend on which other rows share its tile (every output adds its products for k = 0, 1,
// 2, ... in that order), so the unordered placement of rows inside an expert changes nothing.
#include "common.cuh"
#include "mma.cuh"

namespace {

constexpr int TM = 32;          // rows of a tile
constexpr int TN = 64;          // output columns of a tile
constexpr int TK = 32;          // K step

// Router logits in fp32: a warp a (token, output) walks the row; the order of the sums
// depends on the width alone.
template <typename T>
__global__ void logits_kernel(const T* __restrict__ h, const float* __restrict__ w,
                              float* __restrict__ out, int outputs, int width, long long count) {
  const long long item = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (item >= count) return;
  const long long t = item / outputs;
  const int o = static_cast<int>(item - t * outputs);
  const T* x = h + t * width;
  const float* row = w + (long long)o * width;
  float sum = 0.f;
  for (int i = lane; i < width; i += 32) sum = fmaf(widen(x[i]), row[i], sum);
  sum = warp_sum(sum);
  if (lane == 0) out[item] = sum;
}

// `experts`: the router's outputs; the first `real` of them have weights. softmax 0: the score
// is sigmoid(z); 1: exp(z - max) / sum over all outputs. bias (null: none): added to the score
// for the choice. Without a bias the sigmoid's order is the logits' own, and they are compared.
__device__ __forceinline__ void route_token(const float* __restrict__ z, int experts, int top,
                                            int32_t* __restrict__ chosen,
                                            float* __restrict__ weights,
                                            int32_t* counts, int32_t* __restrict__ rank,
                                            int real, int softmax,
                                            const float* __restrict__ bias, int lane) {
  float top_z = -INFINITY, total = 1.f;
  if (softmax) {
    for (int e = lane; e < experts; e += 32) top_z = fmaxf(top_z, z[e]);
    top_z = warp_max(top_z);
    float sum = 0.f;
    for (int e = lane; e < experts; e += 32) sum += expf(z[e] - top_z);
    total = warp_sum(sum);
  }
  auto score = [&](float logit) {
    return softmax ? expf(logit - top_z) / total : 1.f / (1.f + expf(-logit));
  };
  const bool by_logit = !softmax && bias == nullptr;
  uint32_t taken = 0;                              // bit i: this lane's i-th expert is chosen
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int i = 0, e = lane; e < experts; ++i, e += 32) {
      if (taken >> i & 1) continue;
      const float v = by_logit ? z[e] : score(z[e]) + (bias ? bias[e] : 0.f);
      if (v > best || (at == 0x7fffffff && !(v != v))) {
        best = v;
        at = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) {
        best = ob;
        at = oa;
      }
    }
    if (at == 0x7fffffff) at = k;                  // (a row without a finite logit)
    if ((at & 31) == lane) taken |= 1u << (at >> 5);
    if (lane == 0) {
      chosen[k] = at;
      weights[k] = score(z[at]);
      rank[k] = at < real ? atomicAdd(counts + at, 1) : -1;
    }
  }
}

__global__ void route_kernel(const float* __restrict__ logits, long long ld, int experts, int top,
                             int32_t* __restrict__ chosen, float* __restrict__ weights,
                             int32_t* __restrict__ counts, int32_t* __restrict__ rank,
                             int tokens, int real, int softmax, const float* __restrict__ bias) {
  const long long t = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  if (t >= tokens) return;
  route_token(logits + t * ld, experts, top, chosen + t * top, weights + t * top, counts,
              rank + t * top, real, softmax, bias, threadIdx.x & 31);
}

// Where each expert's rows begin and the tiles of the grouped products, from the experts'
// row counts; `base`: [experts + 1] ints of shared memory. The whole block calls it.
__device__ __forceinline__ void plan_tiles(const int32_t* counts, int32_t* __restrict__ offsets,
                                           int32_t* __restrict__ tile_expert,
                                           int32_t* __restrict__ tile_row,
                                           int32_t* __restrict__ n_tiles, int experts,
                                           int max_tiles, int32_t* base) {
  if (threadIdx.x == 0) {
    int rows = 0, tiles = 0;
    for (int e = 0; e < experts; ++e) {
      offsets[e] = rows;
      base[e] = tiles;
      rows += counts[e];
      tiles += (counts[e] + TM - 1) / TM;
    }
    offsets[experts] = rows;
    base[experts] = tiles;
    *n_tiles = tiles < max_tiles ? tiles : max_tiles;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    const int n = base[e + 1] - base[e];
    for (int i = 0; i < n; ++i) {
      if (base[e] + i >= max_tiles) break;
      tile_expert[base[e] + i] = e;
      tile_row[base[e] + i] = offsets[e] + i * TM;
    }
  }
}

// A step of few tokens: one block chooses for every token (a warp a token in turn, counting
// rows in shared memory) and then plans, in one launch.
__global__ void __launch_bounds__(256)
route_plan_kernel(const float* __restrict__ logits, long long ld, int experts, int top,
                  int32_t* __restrict__ chosen, float* __restrict__ weights,
                  int32_t* __restrict__ rank, int tokens, int real, int softmax,
                  const float* __restrict__ bias, int32_t* __restrict__ offsets,
                  int32_t* __restrict__ tile_expert, int32_t* __restrict__ tile_row,
                  int32_t* __restrict__ n_tiles, int max_tiles) {
  extern __shared__ int32_t shared_ints[];         // counts [real], then base [real + 1]
  int32_t* counts = shared_ints;
  for (int e = threadIdx.x; e < real; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int t = threadIdx.x >> 5; t < tokens; t += blockDim.x >> 5)
    route_token(logits + t * ld, experts, top, chosen + (long long)t * top,
                weights + (long long)t * top, counts, rank + (long long)t * top, real, softmax,
                bias, threadIdx.x & 31);
  __syncthreads();
  plan_tiles(counts, offsets, tile_expert, tile_row, n_tiles, real, max_tiles, counts + real);
}

__global__ void plan_kernel(int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                            int32_t* __restrict__ tile_expert, int32_t* __restrict__ tile_row,
                            int32_t* __restrict__ n_tiles, int experts, int max_tiles) {
  extern __shared__ int32_t base[];                // [experts + 1] first tile of each expert
  plan_tiles(counts, offsets, tile_expert, tile_row, n_tiles, experts, max_tiles, base);
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;     // for the next step
}

template <typename T>
__global__ void gather_kernel(const T* __restrict__ h, const int32_t* __restrict__ chosen,
                              const float* __restrict__ weights, const int32_t* __restrict__ rank,
                              const int32_t* __restrict__ offsets, T* __restrict__ rows,
                              int32_t* __restrict__ slot_of, int top, int width,
                              int weight_input) {
  const long long pair = blockIdx.x;                // token * top + k
  const long long t = pair / top;
  if (rank[pair] < 0) {                             // an identity expert: no row
    if (threadIdx.x == 0) slot_of[pair] = -1;
    return;
  }
  const int slot = offsets[chosen[pair]] + rank[pair];
  const float w = weight_input ? weights[pair] : 1.f;
  if (threadIdx.x == 0) slot_of[pair] = slot;
  const T* from = h + t * width;
  T* to = rows + (long long)slot * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) to[i] = narrow<T>(widen(from[i]) * w);
}

// One tile of a grouped product: rows [row0, row0 + TM) of `a` (those below `row_end`) times
// the expert's weights. DUAL: two weight matrices (gate and up) and the activation; else one
// and fp32 out. 256 threads; a thread owns 2 rows x 4 columns.
template <typename T, bool DUAL>
__global__ void __launch_bounds__(256)
grouped_kernel(const T* __restrict__ a, const T* __restrict__ w0, const T* __restrict__ w1,
               long long expert_stride, const int32_t* __restrict__ tile_expert,
               const int32_t* __restrict__ tile_row, const int32_t* __restrict__ offsets,
               const int32_t* __restrict__ n_tiles, void* __restrict__ out_v, int n, int k,
               float limit, float alpha) {
  __shared__ float as[TK][TM + 4];
  __shared__ float ws[DUAL ? 2 : 1][TK][TN + 4];
  if ((int)blockIdx.x >= *n_tiles) return;
  const int e = tile_expert[blockIdx.x], row0 = tile_row[blockIdx.x];
  const int row_end = offsets[e + 1];
  const int n0 = blockIdx.y * TN;
  const T* wa = w0 + (long long)e * expert_stride;
  const T* wb = DUAL ? w1 + (long long)e * expert_stride : nullptr;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[DUAL ? 2 : 1][2][4] = {};
  for (int k0 = 0; k0 < k; k0 += TK) {
    for (int i = threadIdx.x; i < TM * TK; i += 256) {
      const int r = i / TK, c = i % TK;
      as[c][r] = (row0 + r < row_end && k0 + c < k)
                     ? widen(a[(long long)(row0 + r) * k + k0 + c]) : 0.f;
    }
    for (int i = threadIdx.x; i < TN * TK; i += 256) {
      const int r = i / TK, c = i % TK;
      const bool ok = n0 + r < n && k0 + c < k;
      ws[0][c][r] = ok ? widen(wa[(long long)(n0 + r) * k + k0 + c]) : 0.f;
      if (DUAL) ws[1][c][r] = ok ? widen(wb[(long long)(n0 + r) * k + k0 + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < TK; ++c) {
      const float a0 = as[c][ty * 2], a1 = as[c][ty * 2 + 1];
#pragma unroll
      for (int m = 0; m < (DUAL ? 2 : 1); ++m) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float w = ws[m][c][tx * 4 + j];
          acc[m][0][j] = fmaf(a0, w, acc[m][0][j]);
          acc[m][1][j] = fmaf(a1, w, acc[m][1][j]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + ty * 2 + i;
    if (row >= row_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = n0 + tx * 4 + j;
      if (col >= n) continue;
      if constexpr (DUAL) {
        const float g = fminf(acc[0][i][j], limit);
        const float u = fminf(fmaxf(acc[1][i][j], -limit), limit);
        const float y = g / (1.f + expf(-alpha * g)) * (u + 1.f);
        static_cast<T*>(out_v)[(long long)row * n + col] = narrow<T>(y);
      } else {
        static_cast<float*>(out_v)[(long long)row * n + col] = acc[0][i][j];
      }
    }
  }
}

// The same tile on the tensor cores (bf16 operands, fp32 accumulators: `mma.sync` m16n8k16).
// 128 threads; warp w owns output columns [16 w, 16 w + 16) of the tile's 64 for all 32 rows.
// Rows and weights come through a ring of three or four shared-memory stages filled by 16-byte
// asynchronous copies, rows padded to 80 bytes so that the 8 x 16-byte reads of an `ldmatrix`
// fall into different banks. Rows beyond the expert's last and columns beyond n are zeros.
constexpr int kPad = 40;                 // bf16 elements in a padded row of TK = 32

__device__ __forceinline__ void copy16(void* dst, const void* src, bool real) {
  const uint32_t to = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  const int bytes = real ? 16 : 0;       // (0: the 16 bytes are filled with zeros)
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(to), "l"(src), "r"(bytes)
               : "memory");
}

template <bool DUAL>
__global__ void __launch_bounds__(128)
grouped_tc_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w0,
                  const __nv_bfloat16* __restrict__ w1, long long expert_stride,
                  const int32_t* __restrict__ tile_expert, const int32_t* __restrict__ tile_row,
                  const int32_t* __restrict__ offsets, const int32_t* __restrict__ n_tiles,
                  void* __restrict__ out_v, int n, int k, float limit, float alpha) {
  constexpr int kW = DUAL ? 2 : 1;
  constexpr int kStages = DUAL ? 3 : 4;          // (48 KB of static shared memory at most)
  __shared__ __align__(16) __nv_bfloat16 as[kStages][TM][kPad];
  __shared__ __align__(16) __nv_bfloat16 ws[kStages][kW][TN][kPad];
  if ((int)blockIdx.x >= *n_tiles) return;
  const int e = tile_expert[blockIdx.x], row0 = tile_row[blockIdx.x];
  const int row_end = offsets[e + 1];
  const int n0 = blockIdx.y * TN;
  const __nv_bfloat16* wsrc[2] = {w0 + (long long)e * expert_stride,
                                  DUAL ? w1 + (long long)e * expert_stride : nullptr};
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int steps = (k + TK - 1) / TK;

  auto fill = [&](int step) {
    const int stage = step % kStages, k0 = step * TK;
    // rows: TM x 4 pieces of 8 elements; weights: TN x 4 pieces a matrix
    {
      const int r = threadIdx.x >> 2, c = (threadIdx.x & 3) * 8;
      const bool real = row0 + r < row_end && k0 + c < k;
      copy16(&as[stage][r][c], real ? a + (long long)(row0 + r) * k + k0 + c : a, real);
    }
#pragma unroll
    for (int m = 0; m < kW; ++m)
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int idx = threadIdx.x + i * 128;
        const int r = idx >> 2, c = (idx & 3) * 8;
        const bool real = n0 + r < n && k0 + c < k;
        copy16(&ws[stage][m][r][c], real ? wsrc[m] + (long long)(n0 + r) * k + k0 + c : wsrc[m],
               real);
      }
  };

  float acc[kW][2][2][4] = {};           // [matrix][row tile of 16][column tile of 8][fragment]
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < steps) fill(s);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int step = 0; step < steps; ++step) {
    asm volatile("cp.async.wait_group %0;" ::"n"(kStages - 2) : "memory");
    __syncthreads();
    if (step + kStages - 1 < steps) fill(step + kStages - 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const int stage = step % kStages;
#pragma unroll
    for (int kk = 0; kk < TK; kk += 16) {
      uint32_t af[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(
            &as[stage][mt * 16 + (lane & 15)][kk + (lane >> 4) * 8]));
        mma::ldmatrix_x4(addr, af[mt][0], af[mt][1], af[mt][2], af[mt][3]);
      }
#pragma unroll
      for (int m = 0; m < kW; ++m) {
        uint32_t bf[4];                  // (b0, b1) of column tile 0, then of column tile 1
        const int nrow = warp * 16 + (lane >> 4) * 8 + (lane & 7);
        const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(
            &ws[stage][m][nrow][kk + ((lane >> 3) & 1) * 8]));
        mma::ldmatrix_x4(addr, bf[0], bf[1], bf[2], bf[3]);
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          mma::bf16_16816(acc[m][mt][0], af[mt], bf[0], bf[1]);
          mma::bf16_16816(acc[m][mt][1], af[mt], bf[2], bf[3]);
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        const int row = row0 + mt * 16 + (lane >> 2) + (f >> 1) * 8;
        const int col = n0 + warp * 16 + nt * 8 + (lane & 3) * 2 + (f & 1);
        if (row >= row_end || col >= n) continue;
        if constexpr (DUAL) {
          const float g = fminf(acc[0][mt][nt][f], limit);
          const float u = fminf(fmaxf(acc[1][mt][nt][f], -limit), limit);
          static_cast<__nv_bfloat16*>(out_v)[(long long)row * n + col] =
              __float2bfloat16_rn(g / (1.f + expf(-alpha * g)) * (u + 1.f));
        } else {
          static_cast<float*>(out_v)[(long long)row * n + col] = acc[0][mt][nt][f];
        }
      }
}

// The dense form of the same activation for the shared expert: gate_up [T, 2 ff] -> [T, ff].
template <typename T>
__global__ void clamped_act_kernel(const T* __restrict__ gate_up, T* __restrict__ out,
                                   long long count, int ff, float limit, float alpha) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / ff;
    const int c = static_cast<int>(i - t * ff);
    const float g = fminf(widen(gate_up[t * 2 * ff + c]), limit);
    const float u = fminf(fmaxf(widen(gate_up[t * 2 * ff + ff + c]), -limit), limit);
    out[i] = narrow<T>(g / (1.f + expf(-alpha * g)) * (u + 1.f));
  }
}

template <typename T>
__global__ void combine_kernel(const float* __restrict__ rows, const int32_t* __restrict__ slot_of,
                               const float* __restrict__ weights, int weight_output,
                               const float* __restrict__ shared, const float* __restrict__ gate,
                               long long gate_ld, float* __restrict__ out, int top, int width,
                               long long count, const T* __restrict__ h, int accumulate) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / width;
    const int c = static_cast<int>(i - t * width);
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
      const int slot = slot_of[t * top + k];
      if (slot < 0) {                               // an identity expert: the input itself
        sum = fmaf(widen(h[i]), weights[t * top + k], sum);
        continue;
      }
      const float v = rows[(long long)slot * width + c];
      sum += weight_output ? v * weights[t * top + k] : v;
    }
    if (shared) {
      const float s = gate ? 1.f / (1.f + expf(-gate[t * gate_ld])) : 1.f;
      sum = fmaf(shared[i], s, sum);
    }
    out[i] = accumulate ? out[i] + sum : sum;
  }
}

}  // namespace

SAKV_EXPORT int sakv_moe_tile_rows() { return TM; }

// logits: fp32 [tokens, ld] (the first `experts` columns, of which the first `real` belong to
// experts with weights and the rest to identity experts); counts: int32 [real], zero on entry
// (plan leaves it zero again). chosen, rank: int32 [tokens, top] (rank -1: an identity
// expert); weights: fp32. softmax: the score's kind; bias: fp32 [experts] or null.
SAKV_EXPORT int sakv_moe_route(const float* logits, long long ld, int experts, int top,
                               int32_t* chosen, float* weights, int32_t* counts, int32_t* rank,
                               int tokens, int real, int softmax, const float* bias,
                               cudaStream_t stream) {
  if (tokens < 0 || experts <= 0 || experts > 1024 || top <= 0 || top > experts || top > 32 ||
      ld < experts || real < 0 || real > experts)
    return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  const int threads = 128;
  const long long blocks = ((long long)tokens * 32 + threads - 1) / threads;
  return launch_ordered(route_kernel, dim3((unsigned)blocks), dim3(threads), 0, stream, logits, ld,
                        experts, top, chosen, weights, counts, rank, tokens, real, softmax, bias);
}

// `sakv_moe_route` and `sakv_moe_plan` in one launch of one block, for steps of few tokens
// (the rows' counts live in shared memory: no `counts` argument).
SAKV_EXPORT int sakv_moe_route_plan(const float* logits, long long ld, int experts, int top,
                                    int32_t* chosen, float* weights, int32_t* rank, int tokens,
                                    int real, int softmax, const float* bias, int32_t* offsets,
                                    int32_t* tile_expert, int32_t* tile_row, int32_t* n_tiles,
                                    int max_tiles, cudaStream_t stream) {
  if (tokens <= 0 || experts <= 0 || experts > 1024 || top <= 0 || top > experts || top > 32 ||
      ld < experts || real <= 0 || real > experts || max_tiles <= 0)
    return cudaErrorInvalidValue;
  return launch_ordered(route_plan_kernel, dim3(1), dim3(256), (size_t)(2 * real + 1) * 4, stream,
                        logits, ld, experts, top, chosen, weights, rank, tokens, real, softmax,
                        bias, offsets, tile_expert, tile_row, n_tiles, max_tiles);
}

// out[t, o] = sum_i h[t, i] w[o, i] in fp32: h [tokens, width] of `dtype`, w fp32 [outputs,
// width], out fp32 [tokens, outputs].
SAKV_EXPORT int sakv_moe_logits(const void* h, int dtype, const float* w, float* out, int tokens,
                                int outputs, int width, cudaStream_t stream) {
  if (tokens < 0 || outputs <= 0 || width <= 0) return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  const long long count = (long long)tokens * outputs;
  const long long blocks = (count * 32 + 255) / 256;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
  const dim3 grid((unsigned)blocks), block(256);
  if (dtype == SAKV_F32)
    return launch_ordered(logits_kernel<float>, grid, block, 0, stream, (const float*)h, w, out,
                          outputs, width, count);
  if (dtype == SAKV_BF16)
    return launch_ordered(logits_kernel<__nv_bfloat16>, grid, block, 0, stream,
                          (const __nv_bfloat16*)h, w, out, outputs, width, count);
  return cudaErrorInvalidValue;
}

SAKV_EXPORT int sakv_moe_plan(int32_t* counts, int32_t* offsets, int32_t* tile_expert,
                              int32_t* tile_row, int32_t* n_tiles, int experts, int max_tiles,
                              cudaStream_t stream) {
  if (experts <= 0 || experts > 1024 || max_tiles <= 0) return cudaErrorInvalidValue;
  return launch_ordered(plan_kernel, dim3(1), dim3(256), (size_t)(experts + 1) * 4, stream, counts,
                        offsets, tile_expert, tile_row, n_tiles, experts, max_tiles);
}

SAKV_EXPORT int sakv_moe_gather(const void* h, int dtype, const int32_t* chosen,
                                const float* weights, const int32_t* rank, const int32_t* offsets,
                                void* rows, int32_t* slot_of, int tokens, int top, int width,
                                int weight_input, cudaStream_t stream) {
  if (tokens < 0 || top <= 0 || width <= 0) return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  const dim3 grid((unsigned)((long long)tokens * top)), block(width >= 1024 ? 256 : 128);
  if (dtype == SAKV_F32)
    return launch_ordered(gather_kernel<float>, grid, block, 0, stream, (const float*)h, chosen,
                          weights, rank, offsets, (float*)rows, slot_of, top, width, weight_input);
  if (dtype == SAKV_BF16)
    return launch_ordered(gather_kernel<__nv_bfloat16>, grid, block, 0, stream,
                          (const __nv_bfloat16*)h, chosen, weights, rank, offsets,
                          (__nv_bfloat16*)rows, slot_of, top, width, weight_input);
  return cudaErrorInvalidValue;
}

// a: [rows, k] of `dtype`, sorted by expert. w0 (and w1 when `dual`): the experts' weights,
// expert e's [n, k] at w + e * expert_stride. dual: out [rows, n] of `dtype` = the clamped
// gated activation of (a w0^T, a w1^T); else out fp32 [rows, n] = a w0^T.
SAKV_EXPORT int sakv_moe_product(const void* a, int dtype, const void* w0, const void* w1,
                                 long long expert_stride, const int32_t* tile_expert,
                                 const int32_t* tile_row, const int32_t* offsets,
                                 const int32_t* n_tiles, int max_tiles, void* out, int n, int k,
                                 int dual, float limit, float alpha, cudaStream_t stream) {
  if (max_tiles <= 0 || n <= 0 || k <= 0 || (dual && !w1)) return cudaErrorInvalidValue;
  const dim3 grid(max_tiles, (n + TN - 1) / TN), block(256);
  if (grid.y > 65535) return cudaErrorInvalidValue;
#define SAKV_GROUPED(T, DUAL)                                                                    \
  return launch_ordered(grouped_kernel<T, DUAL>, grid, block, 0, stream, (const T*)a,          \
                        (const T*)w0, (const T*)w1, expert_stride, tile_expert, tile_row,        \
                        offsets, n_tiles, out, n, k, limit, alpha)
  if (dtype == SAKV_F32) {
    if (dual) SAKV_GROUPED(float, true);
    SAKV_GROUPED(float, false);
  }
  if (dtype == SAKV_BF16) {
    // the tensor-core tile wants 16-byte pieces: k a multiple of 8, aligned operands
    if (k % 8 == 0 && !(((uintptr_t)a | (uintptr_t)w0 | (uintptr_t)w1) & 15) &&
        expert_stride % 8 == 0) {
      const dim3 threads(128);
      if (dual)
        return launch_ordered(grouped_tc_kernel<true>, grid, threads, 0, stream,
                              (const __nv_bfloat16*)a, (const __nv_bfloat16*)w0,
                              (const __nv_bfloat16*)w1, expert_stride, tile_expert, tile_row,
                              offsets, n_tiles, out, n, k, limit, alpha);
      return launch_ordered(grouped_tc_kernel<false>, grid, threads, 0, stream,
                            (const __nv_bfloat16*)a, (const __nv_bfloat16*)w0,
                            (const __nv_bfloat16*)w1, expert_stride, tile_expert, tile_row,
                            offsets, n_tiles, out, n, k, limit, alpha);
    }
    if (dual) SAKV_GROUPED(__nv_bfloat16, true);
    SAKV_GROUPED(__nv_bfloat16, false);
  }
#undef SAKV_GROUPED
  return cudaErrorInvalidValue;
}

SAKV_EXPORT int sakv_clamped_act(const void* gate_up, void* out, int dtype, int tokens, int ff,
                                 float limit, float alpha, cudaStream_t stream) {
  if (tokens < 0 || ff <= 0) return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  const long long count = (long long)tokens * ff;
  const dim3 grid(grid_for(count, 256)), block(256);
  if (dtype == SAKV_F32)
    return launch_ordered(clamped_act_kernel<float>, grid, block, 0, stream, (const float*)gate_up,
                          (float*)out, count, ff, limit, alpha);
  if (dtype == SAKV_BF16)
    return launch_ordered(clamped_act_kernel<__nv_bfloat16>, grid, block, 0, stream,
                          (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, count, ff, limit,
                          alpha);
  return cudaErrorInvalidValue;
}

// out[t] = sum_k rows[slot_of[t, k]] (* weights[t, k] if weight_output) + shared[t] *
// sigmoid(gate[t * gate_ld]); shared and gate may be null. A choice with slot_of -1 (an
// identity expert) adds h[t] * weights[t, k]; h: [tokens, width] of `h_dtype`. accumulate:
// out += the sum (the residual stream itself) instead of out = the sum.
SAKV_EXPORT int sakv_moe_combine(const float* rows, const int32_t* slot_of, const float* weights,
                                 int weight_output, const float* shared, const float* gate,
                                 long long gate_ld, float* out, int tokens, int top, int width,
                                 const void* h, int h_dtype, int accumulate,
                                 cudaStream_t stream) {
  if (tokens < 0 || top <= 0 || width <= 0 || h == nullptr) return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  const long long count = (long long)tokens * width;
  const dim3 grid(grid_for(count, 256)), block(256);
  if (h_dtype == SAKV_F32)
    return launch_ordered(combine_kernel<float>, grid, block, 0, stream, rows, slot_of, weights,
                          weight_output, shared, gate, gate_ld, out, top, width, count,
                          (const float*)h, accumulate);
  if (h_dtype == SAKV_BF16)
    return launch_ordered(combine_kernel<__nv_bfloat16>, grid, block, 0, stream, rows, slot_of,
                          weights, weight_output, shared, gate, gate_ld, out, top, width, count,
                          (const __nv_bfloat16*)h, accumulate);
  return cudaErrorInvalidValue;
}
