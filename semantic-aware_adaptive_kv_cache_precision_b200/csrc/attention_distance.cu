// Causal grouped-query attention with a logarithmic distance penalty, an optional window,
// values of a width of their own and an optional gate a head:
//
//   s_ij = (q_i . k_j) * scale - slope[h] * ln(1 + rate[h] * (i - j))
//          for the keys j with 0 <= i - j (< window where there is one)
//   out_i = (sum_j softmax(s_i)_j v_j) * sigmoid(gate_i[h])
//
// Scores, the penalty, the softmax weights and the weighted sum of the values are fp32; keys
// and values are widened from the cache's type. One warp for each (token, head) walks the
// visible keys in the order of their positions with a running maximum and sum, so a token's
// result is the same to the bit whether it came in a prompt, in a piece of one, alone or
// beside other sequences. `kv_store` puts a step's keys and values (columns of the fused
// projection's output) into the cache blocks: keys [block, kv_head, 64, dim], values
// [block, kv_head, 64, vdim].
//
// The tiled form also takes what other kinds of cached attention need (`AttentionExtra`):
//   * queries in two pieces from two tensors (a head's first columns from one projection, the
//     rest from another), and heads that lie further apart than their width;
//   * key rows and value rows wider than what a head reads of them, and values that ARE the
//     first columns of the key rows (attention over one cached latent a position);
//   * a mask of chunks instead of a sliding window: query i sees key j <= i only if both lie
//     in the same run of `chunk` positions counted from the sequence's start;
//   * several softmax maps a head over the same values (MAPS = 2: the key row holds one key
//     a map, queries lie head by head as [map 1 | map 2]) combined as
//       o = a1 - lambda * a2;  out = o / sqrt(mean(o^2) + eps) * out_scale * sigmoid(gate)
//     with the gate taken element by element from the projection's output.
#include "common.cuh"

// What the tiled kernel needs beyond the plain grouped-query case; `attention_extra_plain`
// gives the values that leave it as it was.
struct AttentionExtra {
  const void* q2;            // second source of query columns (null: none)
  long long q2_stride;       // its row stride
  int q2_head_stride;        // distance between two heads in q2
  int q_split;               // query columns from here on come from q2
  int q_head_stride;         // distance between two (virtual) heads in qkv
  int k_row;                 // elements in a key row of the cache (>= maps * dim)
  int v_row;                 // elements in a value row of the cache (>= vdim)
  int v_in_k;                // values are the first vdim columns of the key rows
  int chunk;                 // > 0: the chunk mask (window must be 0)
  float lambda, out_scale, eps;   // the combination of two maps
  int gate_elem_off;         // column of the element-wise gate in qkv (-1: none)
  int no_trigger;            // the kernel after this one may be a library's: it starts only
                             // when this one has completed
  // A token's keys over `key_splits` blocks (grid y) as well as over a block's warps: every
  // block leaves its sums in `scratch`, takes a ticket, and the block that takes a token's
  // last ticket folds them in the order of the splits and writes the output.
  int key_splits;
  float* scratch;            // [items, key_splits, P, row_floats]
  long long scratch_floats;
  int* tickets;              // [items], zero on entry and on exit
  int warp_stage;            // decode: every warp copies its chunks into shared memory first
  // Decoded tokens, one warp a group of heads: the items run over a token's groups of heads
  // first, a block's warps are the groups of ONE token and key/value head, and they share every
  // chunk of its keys through shared memory as a prompt's consecutive tokens do (the rows are
  // read once for all of the token's heads); `key_splits` blocks take ranges of the chunks.
  int heads_first;
  // A window that keeps a sequence's first tokens: key j < keep is seen by every later query
  // whatever the window says (it keeps its own position). With `sink` (fp32, one number a
  // head) the softmax's denominator also holds exp(sink[h]): a logit without key or value.
  int keep;
  const float* sink;
  // A gate a head from a tensor of its own (queries that are not part of the projection the
  // gates came with): head h's output is multiplied by sigmoid(head_gate[t * stride + h]),
  // elements of the queries' type. Null: none (or `gate_off` inside qkv).
  const void* head_gate;
  long long head_gate_stride;
};

namespace {

inline AttentionExtra attention_extra_plain(int dim, int vdim) {
  AttentionExtra x = {};
  x.q2 = nullptr;
  x.q_split = dim;
  x.q_head_stride = dim;
  x.k_row = dim;
  x.v_row = vdim;
  x.gate_elem_off = -1;
  x.out_scale = 1.f;
  return x;
}

__device__ __forceinline__ int first_visible(int pos, int window, int chunk) {
  if (chunk > 0) return pos - pos % chunk;
  return (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
}

// The chunks of 32 positions that hold visible keys, as a list: the chunks of the kept first
// tokens that lie before the window's first chunk, then the window's chunks up to `last`.
struct ChunkList {
  int kept, from, count;
  __device__ __forceinline__ ChunkList(int first, int last, int keep) {
    from = first / 32;
    kept = (keep + 31) / 32 < from ? (keep + 31) / 32 : from;
    count = kept + last / 32 - from + 1;
  }
  __device__ __forceinline__ int at(int i) const { return i < kept ? i : from + i - kept; }
};

template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ qkv, long long stride, int k_off, int v_off,
                                const int32_t* __restrict__ positions,
                                const int32_t* __restrict__ token_seq,
                                const int32_t* __restrict__ block_table, int max_blocks,
                                T* __restrict__ k_cache, T* __restrict__ v_cache, int kv_heads,
                                int dim, int vdim, long long count) {
  let_next_kernel_start();
  wait_for_previous_kernel();
  const int per_token = kv_heads * (dim + vdim);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / per_token;
    int c = static_cast<int>(i - t * per_token);
    const int pos = positions[t];
    const int block = block_table[(long long)token_seq[t] * max_blocks + pos / kCacheBlock];
    const int at = pos % kCacheBlock;
    if (c < kv_heads * dim) {
      const int g = c / dim, e = c - g * dim;
      k_cache[(((long long)block * kv_heads + g) * kCacheBlock + at) * dim + e] =
          qkv[t * stride + k_off + c];
    } else {
      c -= kv_heads * dim;
      const int g = c / vdim, e = c - g * vdim;
      v_cache[(((long long)block * kv_heads + g) * kCacheBlock + at) * vdim + e] =
          qkv[t * stride + v_off + c];
    }
  }
}

template <int PER, typename T>
__global__ void distance_attention_kernel(
    const T* __restrict__ qkv, long long stride, int gate_off, T* __restrict__ out,
    const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_seq,
    const int32_t* __restrict__ block_table, int max_blocks, int tokens, int heads, int kv_heads,
    int dim, int vdim, float scale, int window, const float* __restrict__ slope,
    const float* __restrict__ rate) {
  let_next_kernel_start();
  wait_for_previous_kernel();
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (long long)tokens * heads) return;
  const int t = static_cast<int>(warp / heads);
  const int h = static_cast<int>(warp - (long long)t * heads);
  const int g = h / (heads / kv_heads);
  const int pos = positions[t];
  const int32_t* table = block_table + (long long)token_seq[t] * max_blocks;
  const float sl = slope ? slope[h] : 0.f, rt = rate ? rate[h] : 0.f;

  float qr[PER], acc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    qr[i] = e < dim ? widen(qkv[(long long)t * stride + (long long)h * dim + e]) : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  for (int j = first; j <= pos; ++j) {
    const int block = table[j / kCacheBlock];
    const long long at = ((long long)block * kv_heads + g) * kCacheBlock + j % kCacheBlock;
    const T* kp = k_cache + at * dim;
    const T* vp = v_cache + at * vdim;
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + 32 * i;
      if (e < dim) part = fmaf(qr[i], widen(kp[e]), part);
    }
    float s = warp_sum(part) * scale;
    if (slope) s -= sl * log1pf(rt * (float)(pos - j));
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new);
    const float p = expf(s - m_new);
    l = fmaf(l, corr, p);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + 32 * i;
      if (e < vdim) acc[i] = fmaf(acc[i], corr, p * widen(vp[e]));
    }
    m = m_new;
  }
  float gate = 1.f;
  if (gate_off >= 0) {
    const float z = widen(qkv[(long long)t * stride + gate_off + h]);
    gate = 1.f / (1.f + expf(-z));
  }
  const float inv = gate / l;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    if (e < vdim) out[((long long)t * heads + h) * vdim + e] = narrow<T>(acc[i] * inv);
  }
}

// The faster form for key and value widths up to 256. A warp takes up to P query heads of one
// token that share a key/value head and walks the visible keys in chunks of 32 positions
// (aligned to multiples of 32, so a chunk lies in one cache block): each lane scores ONE key
// against the P queries (the key's row is read once for all of them, the queries come from
// shared memory), the chunk's maxima and sums are taken across the lanes, and for the
// weighted sum of the values the lanes share out the value's columns while the weights go
// round by shuffle. `splits` warps may share one token's keys (a decoded token has few
// queries and many keys) and merge their running maxima, sums and partial outputs through
// shared memory. With one warp a token the sums have the same terms in the same order
// however the tokens are cut into steps.
__device__ __forceinline__ void copy16_async(void* dst, const void* src) {
  const uint32_t to = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(to), "l"(src) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void copies_wait_all_but_last() {
  asm volatile("cp.async.wait_group 1;" ::: "memory");
}

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

template <int P, int VPL, int MAPS, typename T>
__global__ void __launch_bounds__(VPL >= 16 ? 256 : 512)      // (wide values: more registers)
distance_attention_tiled_kernel(
    const T* __restrict__ qkv, long long stride, int gate_off, T* __restrict__ out,
    const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_seq,
    const int32_t* __restrict__ block_table, int max_blocks, int tokens, int heads, int kv_heads,
    int dim, int vdim, float scale, int window, const float* __restrict__ slope,
    const float* __restrict__ rate, int splits, int row_floats, int stage_ok,
    const AttentionExtra x) {
  static_assert(MAPS == 1 || P % MAPS == 0, "a head's maps stay in one warp");
  extern __shared__ __align__(16) float shared[];
  if (!x.no_trigger) let_next_kernel_start();
  wait_for_previous_kernel();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int hg = heads / kv_heads, per_group = (hg + P - 1) / P;
  const long long items = (long long)tokens * kv_heads * per_group;
  const long long item = (long long)blockIdx.x * (warps / splits) + warp / splits;
  const int split = warp % splits;
  const bool active = item < items;
  float* mine = shared + (long long)warp * P * row_floats;     // queries now, partials later
  int t = 0, g = 0, h0 = 0, np = 0, pos = 0, first = 0;
  float m[P], l[P], acc[P][VPL], sl[P], rt[P];
#pragma unroll
  for (int p = 0; p < P; ++p) {
    m[p] = -INFINITY;
    l[p] = 0.f;
    sl[p] = rt[p] = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) acc[p][i] = 0.f;
  }
  const int k_row = x.k_row, v_row = x.v_row;
  const bool wide_k = dim % 8 == 0 && k_row % 8 == 0 && !((uintptr_t)k_cache & 15);
  const bool wide_v = vdim % VPL == 0 && v_row % VPL == 0 && (v_row * sizeof(T)) % 16 == 0 &&
                      lane * VPL + VPL <= vdim && !((uintptr_t)v_cache & 15);
  // (the same for every thread of the block)
  bool staged = false;
  int block_first = 0, block_last = 0;
  const int groups = kv_heads * per_group;
  int key_part = 0, key_parts = 1;       // this block's range of the chunks, when they are split
  if (stage_ok == 1 && splits == 1 && x.heads_first) {
    const long long item0 = (long long)blockIdx.x * warps, last = item0 + warps - 1;
    if (last < items && item0 / groups == last / groups &&
        (item0 % groups) / per_group == (last % groups) / per_group) {
      staged = true;
      const int p0 = positions[item0 / groups];
      block_first = first_visible(p0, window, x.chunk);
      block_last = p0;
      key_part = x.key_splits > 1 ? (int)blockIdx.y : 0;
      key_parts = x.key_splits > 1 ? x.key_splits : 1;
    }
  } else if (stage_ok == 1 && splits == 1) {
    const long long item0 = (long long)blockIdx.x * warps, last = item0 + warps - 1;
    if (last < items && item0 / tokens == last / tokens) {
      const int t0 = static_cast<int>(item0 % tokens), t1 = t0 + warps - 1;
      if (token_seq[t0] == token_seq[t1] && positions[t1] == positions[t0] + warps - 1) {
        staged = true;
        const int p0 = positions[t0];
        block_first = first_visible(p0, window, x.chunk);
        block_last = positions[t1];
      }
    }
  }
  if (active) {
    t = static_cast<int>(x.heads_first ? item / groups : item % tokens);
    const int rest = static_cast<int>(x.heads_first ? item % groups : item / tokens);
    const int qi = rest % per_group;
    g = rest / per_group;
    h0 = g * hg + qi * P;
    np = hg - qi * P < P ? hg - qi * P : P;
    pos = positions[t];
    first = first_visible(pos, window, x.chunk);
    const T* q2 = static_cast<const T*>(x.q2);
#pragma unroll
    for (int p = 0; p < P; ++p) {
      if (p < np && slope) {
        sl[p] = slope[h0 + p];
        rt[p] = rate[h0 + p];
      }
      const T* qa = qkv + (long long)t * stride + (long long)(h0 + p) * x.q_head_stride;
      const T* qb = q2 ? q2 + (long long)t * x.q2_stride +
                             (long long)(h0 + p) * x.q2_head_stride - x.q_split
                       : qa;
      for (int e = lane; e < dim; e += 32)
        mine[p * row_floats + e] = p < np ? widen(e < x.q_split ? qa[e] : qb[e]) : 0.f;
    }
    __syncwarp();
    const int32_t* table = block_table + (long long)token_seq[t] * max_blocks;
    // chunk c: `kp` this lane's key's row, `vp` the chunk's first value row at this lane's
    // columns, rows `vstride` apart (in the cache, or in the block's copy of the chunk)
    auto chunk = [&](int c, const T* kp, const T* vp, int vstride) {
      const int j = c * 32 + lane;
      const bool valid = (j >= first || j < x.keep) && j <= pos;
      float s[P];
#pragma unroll
      for (int p = 0; p < P; ++p) s[p] = 0.f;
      if (valid) {
#pragma unroll
       for (int mm = 0; mm < MAPS; ++mm, kp += dim) {        // a map's key in the key row
        if (wide_k) {
          // four 16-byte pieces of the key's row are asked for before any is used (eight were
          // slower for the widest rows: 6.8 against 9.7 TFLOP/s over a prompt)
          constexpr int kAhead = 4;
          for (int e = 0; e < dim; e += 8 * kAhead) {
            float kv[kAhead][8];
#pragma unroll
            for (int i = 0; i < kAhead; ++i)
              if (e + 8 * i < dim) load8<T>(kp + e + 8 * i, kv[i]);
#pragma unroll
            for (int i = 0; i < kAhead; ++i) {
              if (e + 8 * i < dim) {
#pragma unroll
                for (int p = mm; p < P; p += MAPS) {
                  const float* q = mine + p * row_floats + e + 8 * i;
                  const float4 a = *reinterpret_cast<const float4*>(q);
                  const float4 b = *reinterpret_cast<const float4*>(q + 4);
                  s[p] = fmaf(a.x, kv[i][0], s[p]); s[p] = fmaf(a.y, kv[i][1], s[p]);
                  s[p] = fmaf(a.z, kv[i][2], s[p]); s[p] = fmaf(a.w, kv[i][3], s[p]);
                  s[p] = fmaf(b.x, kv[i][4], s[p]); s[p] = fmaf(b.y, kv[i][5], s[p]);
                  s[p] = fmaf(b.z, kv[i][6], s[p]); s[p] = fmaf(b.w, kv[i][7], s[p]);
                }
              }
            }
          }
        } else {
          for (int e = 0; e < dim; ++e) {
            const float kv = widen(kp[e]);
#pragma unroll
            for (int p = mm; p < P; p += MAPS) s[p] = fmaf(mine[p * row_floats + e], kv, s[p]);
          }
        }
       }
      }
      const float dist = (float)(pos - j);
      float w[P];
#pragma unroll
      for (int p = 0; p < P; ++p) {
        float sc = -INFINITY;
        if (valid) {
          sc = s[p] * scale;
          if (slope) sc -= sl[p] * log1pf(rt[p] * dist);
        }
        const float m_new = fmaxf(m[p], warp_max(sc));
        const float corr = expf(m[p] - m_new);
        w[p] = valid ? expf(sc - m_new) : 0.f;
        l[p] = fmaf(l[p], corr, warp_sum(w[p]));
        m[p] = m_new;
#pragma unroll
        for (int i = 0; i < VPL; ++i) acc[p][i] *= corr;
      }
      const int lo = (first - c * 32 > 0 && c * 32 >= x.keep) ? first - c * 32 : 0;
      const int hi = pos - c * 32 < 31 ? pos - c * 32 : 31;
      for (int k0 = lo; k0 <= hi; k0 += 4) {         // four values' rows in flight at a time
        alignas(16) T got[4][VPL];
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          const T* vr = vp + (long long)(k0 + n) * vstride;
          if (k0 + n > hi) continue;
          if (wide_v) {                    // a lane's columns in one access
            constexpr int kBytes = VPL * (int)sizeof(T);
            if constexpr (kBytes == 64) {
#pragma unroll
              for (int q = 0; q < 4; ++q)
                reinterpret_cast<uint4*>(got[n])[q] = reinterpret_cast<const uint4*>(vr)[q];
            } else if constexpr (kBytes == 32) {
              reinterpret_cast<uint4*>(got[n])[0] = reinterpret_cast<const uint4*>(vr)[0];
              reinterpret_cast<uint4*>(got[n])[1] = reinterpret_cast<const uint4*>(vr)[1];
            } else if constexpr (kBytes == 16) {
              *reinterpret_cast<uint4*>(got[n]) = *reinterpret_cast<const uint4*>(vr);
            } else if constexpr (kBytes == 8) {
              *reinterpret_cast<uint2*>(got[n]) = *reinterpret_cast<const uint2*>(vr);
            } else if constexpr (kBytes == 4) {
              *reinterpret_cast<uint32_t*>(got[n]) = *reinterpret_cast<const uint32_t*>(vr);
            } else {
#pragma unroll
              for (int i = 0; i < VPL; ++i) got[n][i] = vr[i];
            }
          } else {
#pragma unroll
            for (int i = 0; i < VPL; ++i)
              got[n][i] = lane * VPL + i < vdim ? vr[i] : narrow<T>(0.f);
          }
        }
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          if (k0 + n > hi) continue;
          float pk[P];
#pragma unroll
          for (int p = 0; p < P; ++p) pk[p] = __shfl_sync(0xffffffffu, w[p], k0 + n);
#pragma unroll
          for (int i = 0; i < VPL; ++i) {
            const float v = widen(got[n][i]);
#pragma unroll
            for (int p = 0; p < P; ++p) acc[p][i] = fmaf(pk[p], v, acc[p][i]);
          }
        }
      }
    };
    auto rows_of = [&](int c) {
      return ((long long)table[c >> 1] * kv_heads + g) * kCacheBlock + (c & 1) * 32;
    };
    if (!staged) {
      // (with split keys, whatever the form: block y takes every key_splits-th turn)
      const ChunkList list(first, pos, x.keep);
      const int i0 = (x.key_splits > 1 ? (int)blockIdx.y * splits : 0) + split;
      for (int ci = i0; ci < list.count; ci += splits * (x.key_splits > 1 ? x.key_splits : 1)) {
        const int c = list.at(ci);
        const long long rows = rows_of(c);
        if (stage_ok == 2) {
          // a decoded token: the warp copies its chunk's rows into shared memory with every
          // copy in flight at once (one trip to memory a chunk instead of one every few
          // pieces of a row), then scores from there
          constexpr int kPiece = 16 / (int)sizeof(T);
          const int kstride = k_row + kPiece;
          const int per_warp = 32 * (kstride + (x.v_in_k ? 0 : vdim));
          T* ks = reinterpret_cast<T*>(shared + (long long)warps * P * row_floats) +
                  (long long)warp * per_warp;
          T* vs = ks + 32 * kstride;
          const int kp16 = k_row / kPiece, vp16 = x.v_in_k ? 0 : vdim / kPiece;
          for (int i = lane; i < 32 * kp16; i += 32) {
            const int r = i / kp16, q = (i - r * kp16) * kPiece;
            copy16_async(ks + r * kstride + q, k_cache + (rows + r) * k_row + q);
          }
          for (int i = lane; i < 32 * vp16; i += 32) {
            const int r = i / vp16, q = (i - r * vp16) * kPiece;
            copy16_async(vs + r * vdim + q, v_cache + (rows + r) * v_row + q);
          }
          copies_commit();
          asm volatile("cp.async.wait_group 0;" ::: "memory");
          __syncwarp();
          if (x.v_in_k) chunk(c, ks + lane * kstride, ks + lane * VPL, kstride);
          else chunk(c, ks + lane * kstride, vs + lane * VPL, vdim);
          __syncwarp();
          continue;
        }
        chunk(c, k_cache + (rows + lane) * k_row, v_cache + rows * v_row + lane * VPL, v_row);
      }
    } else {
      // The block's four tokens follow one another in one sequence and see nearly the same
      // keys: every chunk is copied into shared memory once, a chunk ahead of its use, and
      // each warp scores the chunks of its own token's range from there.
      constexpr int kPiece = 16 / (int)sizeof(T);
      const int kstride = k_row + kPiece;            // padded: the lanes' rows hit different banks
      T* stage = reinterpret_cast<T*>(shared + (long long)warps * P * row_floats);
      const int per_buffer = 32 * (kstride + (x.v_in_k ? 0 : vdim));
      const ChunkList list(block_first, block_last, x.keep);
      int c_lo = 0, c_hi = list.count - 1;           // (places in the block's list of chunks)
      if (key_parts > 1) {               // a contiguous share of the chunks for this block
        const int share = (c_hi - c_lo + key_parts) / key_parts;
        c_lo += key_part * share;
        c_hi = c_hi < c_lo + share - 1 ? c_hi : c_lo + share - 1;
      }
      auto fetch = [&](int c, int buffer) {
        const long long rows = rows_of(c);
        T* ks = stage + buffer * per_buffer;
        T* vs = ks + 32 * kstride;
        const int kp16 = k_row / kPiece, vp16 = x.v_in_k ? 0 : vdim / kPiece;
        for (int i = threadIdx.x; i < 32 * kp16; i += blockDim.x) {
          const int r = i / kp16, q = (i - r * kp16) * kPiece;
          copy16_async(ks + r * kstride + q, k_cache + (rows + r) * k_row + q);
        }
        for (int i = threadIdx.x; i < 32 * vp16; i += blockDim.x) {
          const int r = i / vp16, q = (i - r * vp16) * kPiece;
          copy16_async(vs + r * vdim + q, v_cache + (rows + r) * v_row + q);
        }
        copies_commit();
      };
      if (c_lo <= c_hi) fetch(list.at(c_lo), 0);
      int buffer = 0;
      for (int ci = c_lo; ci <= c_hi; ++ci, buffer ^= 1) {
        const int c = list.at(ci);
        if (ci < c_hi) fetch(list.at(ci + 1), buffer ^ 1);
        else copies_commit();
        copies_wait_all_but_last();
        __syncthreads();
        if ((c >= first / 32 || c * 32 < x.keep) && c <= pos / 32) {
          const T* ks = stage + buffer * per_buffer;
          if (x.v_in_k) chunk(c, ks + lane * kstride, ks + lane * VPL, kstride);
          else chunk(c, ks + lane * kstride, ks + 32 * kstride + lane * VPL, vdim);
        }
        __syncthreads();
      }
    }
  }
  if (splits > 1) {                      // (uniform over the block)
    __syncwarp();
    if (active) {
#pragma unroll
      for (int p = 0; p < P; ++p) {
        float* row = mine + p * row_floats;
        if (lane == 0) {
          row[0] = m[p];
          row[1] = l[p];
        }
#pragma unroll
        for (int i = 0; i < VPL; ++i)
          if (lane * VPL + i < vdim) row[2 + lane * VPL + i] = acc[p][i];
      }
    }
    __syncthreads();
    if (!active || split != 0) return;
#pragma unroll
    for (int p = 0; p < P; ++p) {
      float top = -INFINITY;
      for (int w = 0; w < splits; ++w)
        top = fmaxf(top, shared[((long long)(warp + w) * P + p) * row_floats]);
      float total = 0.f, sum[VPL];
#pragma unroll
      for (int i = 0; i < VPL; ++i) sum[i] = 0.f;
      for (int w = 0; w < splits; ++w) {
        const float* row = shared + ((long long)(warp + w) * P + p) * row_floats;
        const float f = row[0] == -INFINITY ? 0.f : expf(row[0] - top);   // (a warp without keys)
        total = fmaf(row[1], f, total);
#pragma unroll
        for (int i = 0; i < VPL; ++i)
          if (lane * VPL + i < vdim) sum[i] = fmaf(row[2 + lane * VPL + i], f, sum[i]);
      }
      m[p] = top;
      l[p] = total;
#pragma unroll
      for (int i = 0; i < VPL; ++i) acc[p][i] = sum[i];
    }
  }
  if (!active) return;
  if (x.key_splits > 1) {              // (uniform over the grid; this warp is the item's)
    const int S = x.key_splits;
    float* part = x.scratch + ((item * S + blockIdx.y) * P) * (long long)row_floats;
#pragma unroll
    for (int p = 0; p < P; ++p) {
      float* row = part + (long long)p * row_floats;
      if (lane == 0) {
        row[0] = m[p];
        row[1] = l[p];
      }
#pragma unroll
      for (int i = 0; i < VPL; ++i)
        if (lane * VPL + i < vdim) row[2 + lane * VPL + i] = acc[p][i];
    }
    __threadfence();
    int ticket = 0;
    if (lane == 0) ticket = atomicAdd(x.tickets + item, 1);
    ticket = __shfl_sync(0xffffffffu, ticket, 0);
    if (ticket != S - 1) return;
    __threadfence();
    if (lane == 0) x.tickets[item] = 0;
    const float* all = x.scratch + (item * S * P) * (long long)row_floats;
#pragma unroll
    for (int p = 0; p < P; ++p) {
      float top = -INFINITY;
      for (int w = 0; w < S; ++w) top = fmaxf(top, __ldcg(all + ((long long)w * P + p) * row_floats));
      float total = 0.f, sum[VPL];
#pragma unroll
      for (int i = 0; i < VPL; ++i) sum[i] = 0.f;
#pragma unroll 4                    // (several splits' rows asked for before the first is used)
      for (int w = 0; w < S; ++w) {
        const float* row = all + ((long long)w * P + p) * row_floats;
        const float mw = __ldcg(row);
        const float f = mw == -INFINITY ? 0.f : expf(mw - top);
        total = fmaf(__ldcg(row + 1), f, total);
#pragma unroll
        for (int i = 0; i < VPL; ++i)
          if (lane * VPL + i < vdim) sum[i] = fmaf(__ldcg(row + 2 + lane * VPL + i), f, sum[i]);
      }
      m[p] = top;
      l[p] = total;
#pragma unroll
      for (int i = 0; i < VPL; ++i) acc[p][i] = sum[i];
    }
  }
  if (x.sink != nullptr) {             // one more logit in the denominator, counted once
#pragma unroll
    for (int p = 0; p < P; ++p) {
      if (p >= np) continue;
      const float s = x.sink[(h0 + p) / MAPS];
      const float m_new = fmaxf(m[p], s);
      const float corr = expf(m[p] - m_new);
      l[p] = fmaf(l[p], corr, expf(s - m_new));
#pragma unroll
      for (int i = 0; i < VPL; ++i) acc[p][i] *= corr;
    }
  }
  if constexpr (MAPS == 2) {
    // two maps a head over the same values: o = a1 - lambda a2, unit root mean square over
    // the head's values, the scale, and the gate element by element
#pragma unroll
    for (int p = 0; p < P; p += 2) {
      if (p >= np) continue;
      const float i1 = 1.f / l[p], i2 = x.lambda / l[p + 1];
      float o[VPL], ss = 0.f;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        o[i] = lane * VPL + i < vdim ? acc[p][i] * i1 - acc[p + 1][i] * i2 : 0.f;
        ss = fmaf(o[i], o[i], ss);
      }
      const float r = rsqrtf(warp_sum(ss) / (float)vdim + x.eps) * x.out_scale;
      const long long head = (long long)t * (heads / 2) + (h0 + p) / 2;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int col = lane * VPL + i;
        if (col >= vdim) continue;
        float gate = 1.f;
        if (x.gate_elem_off >= 0) {
          const float z = widen(qkv[(long long)t * stride + x.gate_elem_off +
                                    (long long)((h0 + p) / 2) * vdim + col]);
          gate = 1.f / (1.f + expf(-z));
        }
        out[head * vdim + col] = narrow<T>(o[i] * r * gate);
      }
    }
    return;
  }
#pragma unroll
  for (int p = 0; p < P; ++p) {
    if (p >= np) continue;
    float gate = 1.f;
    if (gate_off >= 0) {
      const float z = widen(qkv[(long long)t * stride + gate_off + h0 + p]);
      gate = 1.f / (1.f + expf(-z));
    } else if (x.head_gate != nullptr) {
      const float z = widen(static_cast<const T*>(x.head_gate)[(long long)t * x.head_gate_stride +
                                                                h0 + p]);
      gate = 1.f / (1.f + expf(-z));
    }
    const float inv = gate * x.out_scale / l[p];
#pragma unroll
    for (int i = 0; i < VPL; ++i)
      if (lane * VPL + i < vdim)
        out[((long long)t * heads + h0 + p) * vdim + lane * VPL + i] = narrow<T>(acc[p][i] * inv);
  }
}

template <int P, int VPL, int MAPS, typename T>
int launch_tiled(const void* qkv, long long stride, int gate_off, void* out, const void* k_cache,
                 const void* v_cache, const int32_t* positions, const int32_t* token_seq,
                 const int32_t* block_table, int max_blocks, int tokens, int heads, int kv_heads,
                 int dim, int vdim, float scale, int window, const float* slope,
                 const float* rate, int splits, const AttentionExtra& x, cudaStream_t stream) {
  constexpr int kBudget = 200 * 1024;
  static PerDeviceOnce configured;
  auto kernel = distance_attention_tiled_kernel<P, VPL, MAPS, T>;
  if (configured.needs()) {
    const cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBudget);
    if (e != cudaSuccess) return (int)e;
    configured.done();
  }
  const int hg = heads / kv_heads, per_group = (hg + P - 1) / P;
  int row_floats = (dim > vdim + 2 ? dim : vdim + 2);
  row_floats = (row_floats + 3) / 4 * 4;                     // rows stay 16-byte aligned
  int warps = splits > 1 ? splits : (tokens >= 64 ? 8 : 4);     // (a block's tokens share keys)
  if (VPL >= 16 && warps > 8) warps = 8;                        // (the kernel's launch bounds)
  if (x.heads_first && splits == 1) {
    // a block's warps are groups of heads of one token and key/value head: as many as divide
    // the groups there are, so that no block lies across two tokens
    const int cap = VPL >= 16 ? 8 : 16;
    warps = 1;
    for (int w = 1; w <= cap && w <= per_group; ++w)
      if (per_group % w == 0) warps = w;
  }
  while ((size_t)warps * P * row_floats * sizeof(float) > (size_t)kBudget && warps > 1) warps /= 2;
  if ((size_t)warps * P * row_floats * sizeof(float) > (size_t)kBudget) return cudaErrorInvalidValue;
  if (splits > 1) splits = warps;
  // prompts: room for two chunks of keys and values that a block's tokens share
  size_t smem = (size_t)warps * P * row_floats * sizeof(float);
  const size_t staging =
      (size_t)2 * 32 * (x.k_row + 16 / sizeof(T) + (x.v_in_k ? 0 : vdim)) * sizeof(T);
  const bool copies_fit = (x.k_row * sizeof(T)) % 16 == 0 && (vdim * sizeof(T)) % 16 == 0 &&
                          (x.v_row * sizeof(T)) % 16 == 0 && !((uintptr_t)k_cache & 15) &&
                          !((uintptr_t)v_cache & 15);
  int stage_ok = splits == 1 && copies_fit && smem + staging <= (size_t)kBudget &&
                 (x.heads_first || (warps >= 4 && tokens >= warps));
  if (stage_ok) smem += staging;
  // a decoded token's warps: a chunk's rows a warp (`stage_ok` 2), where the step asked for it
  if (splits > 1 && x.warp_stage && copies_fit &&
      smem + (staging / 2) * warps <= (size_t)kBudget) {
    stage_ok = 2;
    smem += (staging / 2) * warps;
  }
  const long long items = (long long)tokens * kv_heads * per_group;
  const long long blocks = (items + warps / splits - 1) / (warps / splits);
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
  unsigned across = 1;
  if (x.key_splits > 1) {
    if ((splits <= 1 && !x.heads_first) || x.key_splits > 64 || x.scratch == nullptr ||
        x.tickets == nullptr ||
        items * x.key_splits * P * row_floats > x.scratch_floats)
      return cudaErrorInvalidValue;
    across = (unsigned)x.key_splits;
  }
  return launch_overlapped(kernel, dim3((unsigned)blocks, across), dim3(warps * 32), smem, stream, 1,
                           (const T*)qkv, stride, gate_off, (T*)out, (const T*)k_cache,
                           (const T*)v_cache, positions, token_seq, block_table, max_blocks,
                           tokens, heads, kv_heads, dim, vdim, scale, window, slope, rate, splits,
                           row_floats, stage_ok, x);
}

template <typename T>
int pick_tiled(const void* qkv, long long stride, int gate_off, void* out, const void* k_cache,
               const void* v_cache, const int32_t* positions, const int32_t* token_seq,
               const int32_t* block_table, int max_blocks, int tokens, int heads, int kv_heads,
               int dim, int vdim, float scale, int window, const float* slope, const float* rate,
               int splits, int maps, const AttentionExtra& x, cudaStream_t stream) {
  const int hg = heads / kv_heads;       // (virtual heads: a head's maps count one each)
#define SAKV_TILED(P, VPL, MAPS)                                                                 \
  return launch_tiled<P, VPL, MAPS, T>(qkv, stride, gate_off, out, k_cache, v_cache, positions,  \
                                       token_seq, block_table, max_blocks, tokens, heads,        \
                                       kv_heads, dim, vdim, scale, window, slope, rate, splits,  \
                                       x, stream)
#define SAKV_TILED_P(VPL)                        \
  if (maps == 2) {                               \
    if (hg == 2) SAKV_TILED(2, VPL, 2);          \
    SAKV_TILED(4, VPL, 2);                       \
  }                                              \
  if (hg == 1) SAKV_TILED(1, VPL, 1);            \
  if (hg == 2) SAKV_TILED(2, VPL, 1);            \
  SAKV_TILED(4, VPL, 1)
  if (vdim <= 32) { SAKV_TILED_P(1); }
  if (vdim <= 64) { SAKV_TILED_P(2); }
  if (vdim <= 128) { SAKV_TILED_P(4); }
  if (vdim <= 256) { SAKV_TILED_P(8); }
  // (sixteen columns a lane: two heads a warp at most, for the registers' sake)
  if (maps == 2) SAKV_TILED(2, 16, 2);
  // (a decoded token's groups of heads share their rows through shared memory: one head a
  // warp costs no reads and gives a block twice the warps, which pays while the step's tokens
  // leave SMs idle: 8 tokens of 8 heads 598 against 714 us over six layers, 64 tokens 417
  // against 304 us a layer)
  if (hg == 1 || (x.heads_first && (long long)tokens * heads <= 2LL * sm_count()))
    SAKV_TILED(1, 16, 1);
  SAKV_TILED(2, 16, 1);
#undef SAKV_TILED_P
#undef SAKV_TILED
}

template <typename T>
int launch_attention(const void* qkv, long long stride, int gate_off, void* out,
                     const void* k_cache, const void* v_cache, const int32_t* positions,
                     const int32_t* token_seq, const int32_t* block_table, int max_blocks,
                     int tokens, int heads, int kv_heads, int dim, int vdim, float scale,
                     int window, const float* slope, const float* rate, cudaStream_t stream) {
  const int threads = 128;
  const long long blocks = ((long long)tokens * heads * 32 + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
  const int widest = dim > vdim ? dim : vdim;
#define SAKV_ATT(PER)                                                                            \
  return launch_overlapped(distance_attention_kernel<PER, T>, dim3((unsigned)blocks),            \
                           dim3(threads), 0, stream, 1, (const T*)qkv, stride, gate_off, (T*)out, \
                           (const T*)k_cache, (const T*)v_cache, positions, token_seq,           \
                           block_table, max_blocks, tokens, heads, kv_heads, dim, vdim, scale,   \
                           window, slope, rate)
  if (widest <= 32) SAKV_ATT(1);
  if (widest <= 64) SAKV_ATT(2);
  if (widest <= 128) SAKV_ATT(4);
  if (widest <= 256) SAKV_ATT(8);
  SAKV_ATT(16);
#undef SAKV_ATT
}

}  // namespace

SAKV_EXPORT int sakv_kv_store(const void* qkv, int dtype, long long stride, int k_off, int v_off,
                              const int32_t* positions, const int32_t* token_seq,
                              const int32_t* block_table, int max_blocks, void* k_cache,
                              void* v_cache, int tokens, int kv_heads, int dim, int vdim,
                              cudaStream_t stream) {
  if (tokens < 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || max_blocks <= 0)
    return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  const long long count = (long long)tokens * kv_heads * (dim + vdim);
  const dim3 grid(grid_for(count, 256)), block(256);
  if (dtype == SAKV_F32)
    return launch_overlapped(kv_store_kernel<float>, grid, block, 0, stream, 1, (const float*)qkv,
                             stride, k_off, v_off, positions, token_seq, block_table, max_blocks,
                             (float*)k_cache, (float*)v_cache, kv_heads, dim, vdim, count);
  if (dtype == SAKV_BF16)
    return launch_overlapped(kv_store_kernel<__nv_bfloat16>, grid, block, 0, stream, 1,
                             (const __nv_bfloat16*)qkv, stride, k_off, v_off, positions, token_seq,
                             block_table, max_blocks, (__nv_bfloat16*)k_cache,
                             (__nv_bfloat16*)v_cache, kv_heads, dim, vdim, count);
  return cudaErrorInvalidValue;
}

// qkv: [tokens, stride] with the queries in its first heads * dim columns and, if gate_off
// >= 0, the gates' pre-activations in columns gate_off .. gate_off + heads - 1. slope, rate:
// fp32 [heads] (null: no penalty). window 0: every earlier key. out: [tokens, heads * vdim].
// `splits`: 0 runs the plain form (a warp for each token and head, one key at a time); 1 the
// form that scores 32 keys at a time (widths up to 256); more than 1 lets that many warps
// (up to 16) share a token's keys.
SAKV_EXPORT int sakv_distance_attention(const void* qkv, int dtype, long long stride, int gate_off,
                                        void* out, const void* k_cache, const void* v_cache,
                                        const int32_t* positions, const int32_t* token_seq,
                                        const int32_t* block_table, int max_blocks, int tokens,
                                        int heads, int kv_heads, int dim, int vdim, float scale,
                                        int window, const float* slope, const float* rate,
                                        int splits, cudaStream_t stream) {
  if (tokens < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 ||
      dim > 512 || vdim > 512 || max_blocks <= 0 || window < 0 || splits < 0 || splits > 16)
    return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  if (splits > 0 && dim <= 256 && vdim <= 256) {
    const AttentionExtra x = attention_extra_plain(dim, vdim);
    if (dtype == SAKV_F32)
      return pick_tiled<float>(qkv, stride, gate_off, out, k_cache, v_cache, positions, token_seq,
                               block_table, max_blocks, tokens, heads, kv_heads, dim, vdim, scale,
                               window, slope, rate, splits, 1, x, stream);
    if (dtype == SAKV_BF16)
      return pick_tiled<__nv_bfloat16>(qkv, stride, gate_off, out, k_cache, v_cache, positions,
                                       token_seq, block_table, max_blocks, tokens, heads, kv_heads,
                                       dim, vdim, scale, window, slope, rate, splits, 1, x, stream);
    return cudaErrorInvalidValue;
  }
  if (dtype == SAKV_F32)
    return launch_attention<float>(qkv, stride, gate_off, out, k_cache, v_cache, positions,
                                   token_seq, block_table, max_blocks, tokens, heads, kv_heads,
                                   dim, vdim, scale, window, slope, rate, stream);
  if (dtype == SAKV_BF16)
    return launch_attention<__nv_bfloat16>(qkv, stride, gate_off, out, k_cache, v_cache,
                                           positions, token_seq, block_table, max_blocks, tokens,
                                           heads, kv_heads, dim, vdim, scale, window, slope, rate,
                                           stream);
  return cudaErrorInvalidValue;
}

// The tiled form with everything `AttentionExtra` describes. `heads` counts query heads;
// each has `maps` (1 or 2) queries of `dim` columns, `q_head_stride` apart in qkv. Query
// columns from `q_split` on are read from `q2` (null: all from qkv). Keys: rows of `k_row`
// elements, map m's key at column m * dim; values: the first `vdim` of rows of `v_row`
// elements in v_cache, or (v_cache null) of the key rows. `chunk` > 0 is the chunk mask;
// `window` and `chunk` exclude each other. With two maps: lambda, out_scale, eps and
// gate_elem_off (the element-wise gate's first column in qkv, -1 for none) shape the output;
// with one map `gate_off` is the gate a head as above. out: [tokens, heads * vdim].
// `splits` >= 1 as above. `key_splits` > 1 (with splits > 1): that many blocks share a token's
// keys as well; `scratch` (floats, at least tokens * kv_heads * (heads * maps / kv_heads + 3) *
// key_splits * (max(dim, vdim + 2) + 4)) holds their sums and `tickets` (int32 for every
// token, kv head and group of heads; zero on entry, left zero) tells which block came last.
// `heads_first` (with splits 1): the form for decoded tokens in which a block's warps are one
// token's groups of heads and share each chunk of keys through shared memory; `key_splits`
// blocks then take contiguous shares of the chunks.
SAKV_EXPORT int sakv_cached_attention(
    const void* qkv, int dtype, long long stride, int q_head_stride, const void* q2,
    long long q2_stride, int q2_head_stride, int q_split, int gate_off, void* out,
    const void* k_cache, int k_row, const void* v_cache, int v_row,
    const int32_t* positions, const int32_t* token_seq, const int32_t* block_table,
    int max_blocks, int tokens, int heads, int kv_heads, int maps, int dim, int vdim, float scale,
    int window, int chunk, float lambda, float out_scale, float eps, int gate_elem_off,
    int splits, int key_splits, float* scratch, long long scratch_floats, int* tickets,
    int warp_stage, int heads_first, int keep_first, const float* sink, const void* head_gate,
    long long head_gate_stride, cudaStream_t stream) {
  if (keep_first < 0 || (keep_first > 0 && chunk > 0)) return cudaErrorInvalidValue;
  if (head_gate != nullptr && (maps != 1 || gate_off >= 0)) return cudaErrorInvalidValue;
  if (tokens < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 ||
      dim > 640 || vdim > 512 || max_blocks <= 0 || window < 0 || chunk < 0 ||
      (window > 0 && chunk > 0) || splits < 1 || splits > 16 || (maps != 1 && maps != 2) ||
      k_row < maps * dim || (q2 != nullptr && (q_split < 0 || q_split > dim)) ||
      q_head_stride <= 0)
    return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  AttentionExtra x = {};
  x.q2 = q2;
  x.q2_stride = q2_stride;
  x.q2_head_stride = q2_head_stride;
  x.q_split = q2 ? q_split : dim;
  x.q_head_stride = q_head_stride;
  x.k_row = k_row;
  x.v_in_k = v_cache == nullptr;
  x.v_row = x.v_in_k ? k_row : v_row;
  if (x.v_row < vdim) return cudaErrorInvalidValue;
  x.chunk = chunk;
  x.lambda = lambda;
  x.out_scale = out_scale;
  x.eps = eps;
  x.gate_elem_off = gate_elem_off;
  x.no_trigger = 1;
  x.key_splits = key_splits > 1 ? key_splits : 1;
  x.scratch = scratch;
  x.scratch_floats = scratch_floats;
  x.tickets = tickets;
  x.warp_stage = warp_stage;
  x.heads_first = heads_first && splits == 1;
  x.keep = window > 0 ? keep_first : 0;
  x.sink = sink;
  x.head_gate = head_gate;
  x.head_gate_stride = head_gate_stride;
  const void* values = x.v_in_k ? k_cache : v_cache;
  if (dtype == SAKV_F32)
    return pick_tiled<float>(qkv, stride, gate_off, out, k_cache, values, positions, token_seq,
                             block_table, max_blocks, tokens, heads * maps, kv_heads, dim, vdim,
                             scale, window, nullptr, nullptr, splits, maps, x, stream);
  if (dtype == SAKV_BF16)
    return pick_tiled<__nv_bfloat16>(qkv, stride, gate_off, out, k_cache, values, positions,
                                     token_seq, block_table, max_blocks, tokens, heads * maps,
                                     kv_heads, dim, vdim, scale, window, nullptr, nullptr, splits,
                                     maps, x, stream);
  return cudaErrorInvalidValue;
}
