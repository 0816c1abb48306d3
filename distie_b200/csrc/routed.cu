// Kernels of a routed feed-forward: every token goes through `top` of `experts` small SwiGLU layers.
//
//   route_top     logits = x W_router^T in float32, scores = sigmoid(logits), the `top` largest per token
//                 (ties to the lower index) with their scores.  One block per token.
//   route_plan    (token, choice) pairs sorted by expert: for every slot of the sorted order the token it reads,
//                 the weight of the pair and the row of the output it writes; the list of row tiles (expert,
//                 first slot, rows) that the grouped products walk.  One block.
//   grouped products over the sorted slots, a tile of rows of one expert per block:
//                 hidden = silu(z Wg_e^T) * (z Wu_e^T) with z = weight * x[token] (or x[token]);
//                 out[choice, token, :] = hidden Wd_e^T (times the weight when it was not on the input).
//
// Nothing reads host-side batch data: counts, offsets and tiles stay on the device, so a captured decode step
// replays these kernels for whatever tokens it is given.  A row's result depends on its own token and expert
// only (the order of accumulation over K is fixed), never on what else was routed to the expert.
// Accumulation is float32; T (float or bfloat16) is the type of activations and weights.
#include "common.cuh"

#include <mma.h>

namespace distie {

__device__ __forceinline__ float routed_silu(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float routed_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
// The hidden activation of an expert: silu(g) * u, or with limit > 0 the capped form
// g' = min(g, limit), u' = clamp(u, -limit, limit), g' * sigmoid(1.702 g') * (u' + 1).
__device__ __forceinline__ float routed_glu(float g, float u, float limit) {
  if (limit > 0.f) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * routed_sigmoid(1.702f * g) * (u + 1.f);
  }
  return routed_silu(g) * u;
}

constexpr int kRouteThreads = 256;
constexpr int kMaxTop = 32;

// A warp picks for one token.  `mine` holds the token's `experts` scores in shared memory and `group_s` has room for
// `count` floats.  With count > 1 and keep < count the experts form `count` equal groups of neighbours; a group's
// score is the sum of its two largest scores (of its one score in groups of one) and only the experts of the `keep`
// best groups (ties to the lower group) stay eligible.  Then the `top` largest eligible scores, ties to the lower
// index; the weights are the scores times `weight_scale`.  `plain` holds the scores the weights are taken from: `mine`
// itself, or a second array when the choice runs on scores with a correction added (which may lie anywhere, so what
// is taken or not eligible is marked with -infinity).  `normalise`: the chosen scores are divided by their sum + 1e-20.
__device__ __forceinline__ void route_choose(float* mine, float* group_s, int experts, int top, int count, int keep,
                                             float weight_scale, int* __restrict__ ids, float* __restrict__ weights,
                                             int lane, const float* plain = nullptr, int normalise = 0) {
  if (plain == nullptr) plain = mine;
  if (count > 1 && keep < count) {
    const int size = experts / count;
    for (int g = lane; g < count; g += 32) {
      float first = -1.f, second = -1.f;
      for (int i = 0; i < size; ++i) {
        const float sc = mine[g * size + i];
        if (sc > first) { second = first; first = sc; }
        else if (sc > second) second = sc;
      }
      group_s[g] = size > 1 ? first + second : first;
    }
    __syncwarp();
    for (int j = 0; j < keep; ++j) {
      float best = -1.f;  // group scores lie in [0, 2]; a group kept is set to -3
      int at = count;
      for (int g = lane; g < count; g += 32) {
        const float sc = group_s[g];
        if (sc > best) { best = sc; at = g; }
      }
#pragma unroll
      for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, best, offset);
        const int other_at = __shfl_xor_sync(0xffffffffu, at, offset);
        if (other > best || (other == best && other_at < at)) { best = other; at = other_at; }
      }
      if (lane == 0 && at < count) group_s[at] = -3.f;
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
      if (group_s[e / size] != -3.f) mine[e] = -INFINITY;
    __syncwarp();
  }
  float total = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;  // a score taken or not eligible is -infinity
    int at = experts;
    for (int e = lane; e < experts; e += 32) {
      const float sc = mine[e];
      if (sc > best) { best = sc; at = e; }  // the first of equal scores within a lane: the lower index
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, offset);
      const int other_at = __shfl_xor_sync(0xffffffffu, at, offset);
      if (other > best || (other == best && other_at < at)) { best = other; at = other_at; }
    }
    if (lane == 0 && at < experts) {
      ids[j] = at;
      weights[j] = plain[at] * weight_scale;
      total += plain[at];
      mine[at] = -INFINITY;
    }
    __syncwarp();
  }
  if (normalise && lane == 0) {
    const float inv = 1.f / (total + 1e-20f);
    for (int j = 0; j < top; ++j) weights[j] *= inv;
  }
}

// What a warp does to a token's row of logits before it chooses: with `softmax` the scores become the softmax over
// the row (else the row already holds sigmoid scores); with a `correction` the plain scores are kept in `plain_s` and
// the row itself becomes score + correction.  Returns where the plain scores lie.
__device__ __forceinline__ const float* route_scores(float* mine, float* plain_s, int experts, int softmax,
                                                     const float* __restrict__ correction, int lane) {
  if (softmax) {
    float top = -INFINITY;
    for (int e = lane; e < experts; e += 32) top = fmaxf(top, mine[e]);
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, offset));
    float sum = 0.f;
    for (int e = lane; e < experts; e += 32) {
      const float ex = expf(mine[e] - top);
      mine[e] = ex;
      sum += ex;
    }
    sum = warp_sum(sum);
    for (int e = lane; e < experts; e += 32) mine[e] = mine[e] / sum;
    __syncwarp();
  }
  if (correction == nullptr) return mine;
  for (int e = lane; e < experts; e += 32) {
    plain_s[e] = mine[e];
    mine[e] += correction[e];
  }
  __syncwarp();
  return plain_s;
}

// TOK tokens a block: their rows wait in shared memory as floats and a warp takes an expert at a time for all of
// them, so a router row is read once per TOK tokens, in runs of VEC elements a lane.  Then a warp per token picks
// the `top` largest scores.  Dynamic shared memory: TOK * hidden floats (the rows), then TOK * experts (the scores).
template <typename T, int TOK, int VEC>
__global__ void __launch_bounds__(kRouteThreads)
route_top_kernel(const T* __restrict__ x, int x_stride, const T* __restrict__ router, int tokens, int hidden, int experts,
                 int top, int* __restrict__ ids, float* __restrict__ weights, int group_count, int group_keep,
                 float weight_scale, int extra, float* __restrict__ extra_out, int softmax,
                 const float* __restrict__ correction, int normalise) {
  extern __shared__ __align__(16) float route_s[];
  float* x_s = route_s;
  float* scores_s = route_s + (size_t)TOK * hidden;  // per token: experts scores, group_count floats, experts plain scores
  const int score_row = 2 * experts + group_count;
  const int t0 = blockIdx.x * TOK, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int live = min(TOK, tokens - t0);
  for (int r = 0; r < TOK; ++r) {
    const T* src = x + (size_t)(t0 + min(r, live - 1)) * x_stride;
    float* dst = x_s + (size_t)r * hidden;
    if (VEC > 1 && x_stride % VEC == 0 && ((uintptr_t)x & 15) == 0) {
      for (int k = threadIdx.x * VEC; k < hidden; k += kRouteThreads * VEC) {
        float v[VEC];
        if constexpr (VEC == 8) load8(src + k, v);
        else if constexpr (VEC == 4) { const float4 q = load4(src + k); v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w; }
        else v[0] = to_float(src[k]);
#pragma unroll
        for (int i = 0; i < VEC; ++i) dst[k + i] = v[i];
      }
    } else {
      for (int k = threadIdx.x; k < hidden; k += kRouteThreads) dst[k] = to_float(src[k]);
    }
  }
  __syncthreads();
  for (int e = warp; e < experts + extra; e += kRouteThreads / 32) {  // rows past the experts': logits handed out as they are
    const T* w = router + (size_t)e * hidden;
    float dot[TOK];
#pragma unroll
    for (int r = 0; r < TOK; ++r) dot[r] = 0.f;
    for (int k = lane * VEC; k < hidden; k += 32 * VEC) {
      float wv[VEC];
      if constexpr (VEC == 8) load8(w + k, wv);
      else if constexpr (VEC == 4) { const float4 q = load4(w + k); wv[0] = q.x; wv[1] = q.y; wv[2] = q.z; wv[3] = q.w; }
      else wv[0] = to_float(w[k]);
#pragma unroll
      for (int r = 0; r < TOK; ++r) {
        if constexpr (VEC >= 4) {  // (hidden and k are multiples of VEC: the runs are 16-byte aligned)
#pragma unroll
          for (int i = 0; i < VEC; i += 4) {
            const float4 q = *reinterpret_cast<const float4*>(x_s + (size_t)r * hidden + k + i);
            dot[r] += (q.x * wv[i] + q.y * wv[i + 1]) + (q.z * wv[i + 2] + q.w * wv[i + 3]);
          }
        } else {
          dot[r] += x_s[r * hidden + k] * wv[0];
        }
      }
    }
#pragma unroll
    for (int r = 0; r < TOK; ++r) {
      const float z = warp_sum(dot[r]);
      if (lane == 0) {
        if (e < experts) scores_s[r * score_row + e] = softmax ? z : routed_sigmoid(z);
        else if (r < live) extra_out[(size_t)(t0 + r) * extra + e - experts] = z;
      }
    }
  }
  __syncthreads();
  for (int r = warp; r < live; r += kRouteThreads / 32) {
    float* mine = scores_s + (size_t)r * score_row;
    const size_t t = t0 + r;
    const float* plain = route_scores(mine, mine + experts + group_count, experts, softmax, correction, lane);
    route_choose(mine, mine + experts, experts, top, group_count, group_keep, weight_scale, ids + t * top, weights + t * top, lane,
                 plain, normalise);
  }
}

// The choice alone, from float32 logits [tokens, experts] that a product left: a warp per token.
__global__ void __launch_bounds__(kRouteThreads)
route_pick_kernel(const float* __restrict__ logits, int logit_stride, int tokens, int experts, int top,
                  int* __restrict__ ids, float* __restrict__ weights, int group_count, int group_keep, float weight_scale,
                  int softmax, const float* __restrict__ correction, int normalise) {
  extern __shared__ float pick_s[];  // per warp: a row of scores, group_count floats, a row of plain scores
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (kRouteThreads / 32) + warp;
  if (t >= tokens) return;
  float* mine = pick_s + (size_t)warp * (2 * experts + group_count);
  for (int e = lane; e < experts; e += 32) {
    const float z = logits[(size_t)t * logit_stride + e];
    mine[e] = softmax ? z : routed_sigmoid(z);
  }
  __syncwarp();
  const float* plain = route_scores(mine, mine + experts + group_count, experts, softmax, correction, lane);
  route_choose(mine, mine + experts, experts, top, group_count, group_keep, weight_scale, ids + (size_t)t * top,
               weights + (size_t)t * top, lane, plain, normalise);
}

// plan layout (int32): [0] number of tiles; [1 .. 1 + experts] offsets of the experts' slots; then
// tile_expert[max_tiles], tile_first[max_tiles], tile_rows[max_tiles]; then per slot source[pairs], dest[pairs];
// scale[pairs] (float bits).  max_tiles = pairs / tile + experts (rounded up).
struct RoutePlan {
  int* num_tiles;
  int* offsets;
  int* tile_expert;
  int* tile_first;
  int* tile_rows;
  int* source;
  int* dest;
  float* scale;
};

__host__ __device__ inline RoutePlan plan_views(int* base, int pairs, int experts, int tile) {
  const int max_tiles = (pairs + tile - 1) / tile + experts;
  RoutePlan p;
  p.num_tiles = base;
  p.offsets = base + 1;
  p.tile_expert = p.offsets + experts + 1;
  p.tile_first = p.tile_expert + max_tiles;
  p.tile_rows = p.tile_first + max_tiles;
  p.source = p.tile_rows + max_tiles;
  p.dest = p.source + pairs;
  p.scale = reinterpret_cast<float*>(p.dest + pairs);
  return p;
}

// counts_s: 2 * experts ints of dynamic shared memory (counts, then cursors).
__global__ void __launch_bounds__(1024)
route_plan_kernel(const int* __restrict__ ids, const float* __restrict__ weights, int tokens, int top, int experts,
                  int tile, int* __restrict__ plan_base, int* __restrict__ error, int identity) {
  extern __shared__ int counts_s[];
  int* cursor_s = counts_s + experts;
  const int pairs = tokens * top;
  const RoutePlan plan = plan_views(plan_base, pairs, experts, tile);
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts_s[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e < 0 || e >= experts) {  // ids experts .. experts + identity - 1 return their input and are in no tile
      if ((e < 0 || e >= experts + identity) && error) atomicExch(error, 7);
      continue;
    }
    atomicAdd(&counts_s[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    for (int e = 0; e < experts; ++e) {
      const int count = counts_s[e];
      plan.offsets[e] = at;
      cursor_s[e] = at;
      for (int first = 0; first < count; first += tile) {
        plan.tile_expert[tiles] = e;
        plan.tile_first[tiles] = at + first;
        plan.tile_rows[tiles] = min(tile, count - first);
        ++tiles;
      }
      at += count;
    }
    plan.offsets[experts] = at;
    *plan.num_tiles = tiles;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e < 0 || e >= experts) continue;
    const int slot = atomicAdd(&cursor_s[e], 1);
    const int token = p / top, choice = p % top;
    plan.source[slot] = token;
    plan.dest[slot] = choice * tokens + token;
    plan.scale[slot] = weights[p];
  }
}

// ---- grouped products, float32 arithmetic on the FMA pipe ---------------------------------------------------------
constexpr int kTileM = 32, kTileN = 64, kTileK = 16, kGroupedThreads = 256;

// C[slot, n] = sum_k A[row(slot), k] * W[e][n, k] for the slots of one tile of one expert.
//   SWIGLU: W is [experts, 2 N, K]; C = silu(A Wg^T) * (A Wu^T), stored as T in `out` [pairs, N] by slot.
//   else:   W is [experts, N, K]; C stored as float32 in `out32` at row dest[slot] (times scale[slot] with scale_out).
// `gather`: A's row of a slot is source[slot] and is multiplied by scale[slot] when scale_in is set; otherwise the
// slot's own row.
template <typename T, bool SWIGLU>
__global__ void __launch_bounds__(kGroupedThreads)
grouped_product_kernel(const T* __restrict__ a, int a_stride, const T* __restrict__ w, int* __restrict__ plan_base,
                       int pairs, int experts, T* __restrict__ out, float* __restrict__ out32, int N, int K, int gather,
                       int scale_in, int scale_out, float limit) {
  const RoutePlan plan = plan_views(plan_base, pairs, experts, kTileM);
  const int tile = blockIdx.x;
  if (tile >= *plan.num_tiles) return;
  const int expert = plan.tile_expert[tile], first = plan.tile_first[tile], rows = plan.tile_rows[tile];
  const int n0 = blockIdx.y * kTileN;
  __shared__ float a_s[kTileK][kTileM + 1];
  __shared__ float w_s[SWIGLU ? 2 : 1][kTileK][kTileN + 1];
  __shared__ int src_s[kTileM];
  __shared__ float scale_s[kTileM];
  const int tid = threadIdx.x;
  if (tid < kTileM) {
    const int slot = first + min(tid, rows - 1);
    src_s[tid] = gather ? plan.source[slot] : slot;
    scale_s[tid] = plan.scale[slot];
  }
  __syncthreads();
  const int ty = tid / 16, tx = tid % 16;  // rows 2 ty, 2 ty + 1; columns 4 tx .. 4 tx + 3
  float acc[2][4] = {}, acc_up[2][4] = {};
  const size_t w_rows = SWIGLU ? 2 * (size_t)N : (size_t)N;
  const T* w_e = w + (size_t)expert * w_rows * K;
  for (int k0 = 0; k0 < K; k0 += kTileK) {
    for (int idx = tid; idx < kTileM * kTileK; idx += kGroupedThreads) {
      const int r = idx / kTileK, kk = idx % kTileK;
      float v = 0.f;
      if (r < rows && k0 + kk < K) {
        v = to_float(a[(size_t)src_s[r] * a_stride + k0 + kk]);
        if (scale_in) v = to_float(from_float<T>(v * scale_s[r]));  // the expert reads weight * x in the engine's type
      }
      a_s[kk][r] = v;
    }
    for (int idx = tid; idx < kTileN * kTileK; idx += kGroupedThreads) {
      const int n = idx / kTileK, kk = idx % kTileK;
      const bool live = n0 + n < N && k0 + kk < K;
      w_s[0][kk][n] = live ? to_float(w_e[(size_t)(n0 + n) * K + k0 + kk]) : 0.f;
      if (SWIGLU) w_s[1][kk][n] = live ? to_float(w_e[((size_t)N + n0 + n) * K + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTileK; ++kk) {
      const float a0 = a_s[kk][2 * ty], a1 = a_s[kk][2 * ty + 1];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float b = w_s[0][kk][4 * tx + c];
        acc[0][c] += a0 * b;
        acc[1][c] += a1 * b;
        if (SWIGLU) {
          const float u = w_s[1][kk][4 * tx + c];
          acc_up[0][c] += a0 * u;
          acc_up[1][c] += a1 * u;
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int local = 2 * ty + r;
    if (local >= rows) continue;
    const int slot = first + local;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int n = n0 + 4 * tx + c;
      if (n >= N) continue;
      if (SWIGLU) {
        out[(size_t)slot * N + n] = from_float<T>(routed_glu(acc[r][c], acc_up[r][c], limit));
      } else {
        const float v = scale_out ? acc[r][c] * scale_s[local] : acc[r][c];
        out32[(size_t)plan.dest[slot] * N + n] = v;
      }
    }
  }
}

// ---- grouped products on the tensor cores (bfloat16, float32 accumulation) ------------------------------------------
// The same tiles with 64 rows: a tile of A (gathered rows, scaled and rounded to bfloat16 where the weight is on the
// input) and a tile of W in shared memory, warp-level matrix products on 16 x 16 x 16 fragments, eight warps as
// 4 (rows) x 2 (columns) over a 64 x 64 tile (x 2 for gate and up).
constexpr int kMmaM = 64, kMmaN = 64, kMmaK = 32, kMmaThreads = 256, kMmaPad = 8;

template <bool SWIGLU>
__global__ void __launch_bounds__(kMmaThreads)
grouped_product_mma_kernel(const __nv_bfloat16* __restrict__ a, int a_stride, const __nv_bfloat16* __restrict__ w,
                           int* __restrict__ plan_base, int pairs, int experts, __nv_bfloat16* __restrict__ out,
                           float* __restrict__ out32, int N, int K, int gather, int scale_in, int scale_out, float limit) {
  using namespace nvcuda;
  const RoutePlan plan = plan_views(plan_base, pairs, experts, kMmaM);
  const int tile = blockIdx.x;
  if (tile >= *plan.num_tiles) return;
  const int expert = plan.tile_expert[tile], first = plan.tile_first[tile], rows = plan.tile_rows[tile];
  const int n0 = blockIdx.y * kMmaN;
  __shared__ __align__(32) __nv_bfloat16 a_s[kMmaM][kMmaK + kMmaPad];
  __shared__ __align__(32) __nv_bfloat16 w_s[SWIGLU ? 2 : 1][kMmaN][kMmaK + kMmaPad];
  __shared__ __align__(32) float c_s[kMmaThreads / 32][16][16 + 4];
  __shared__ int src_s[kMmaM];
  __shared__ float scale_s[kMmaM];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < kMmaM) {
    const int slot = first + min(tid, rows - 1);
    src_s[tid] = gather ? plan.source[slot] : slot;
    scale_s[tid] = plan.scale[slot];
  }
  __syncthreads();
  const int wr = warp >> 1, wc = warp & 1;  // the warp's 16 rows and 32 columns
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[2], acc_up[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) { wmma::fill_fragment(acc[i], 0.f); wmma::fill_fragment(acc_up[i], 0.f); }
  const size_t w_rows = SWIGLU ? 2 * (size_t)N : (size_t)N;
  const __nv_bfloat16* w_e = w + (size_t)expert * w_rows * K;
  for (int k0 = 0; k0 < K; k0 += kMmaK) {
    // eight elements (16 bytes) a thread: K is a multiple of 8 and rows are 16-byte aligned
    for (int idx = tid; idx < kMmaM * (kMmaK / 8); idx += kMmaThreads) {
      const int r = idx / (kMmaK / 8), kk = (idx % (kMmaK / 8)) * 8;
      uint4 raw = make_uint4(0, 0, 0, 0);
      if (r < rows && k0 + kk < K) {
        raw = *reinterpret_cast<const uint4*>(a + (size_t)src_s[r] * a_stride + k0 + kk);
        if (scale_in) {
          float v[8];
          load8(reinterpret_cast<const __nv_bfloat16*>(&raw), v);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] *= scale_s[r];
          store8(reinterpret_cast<__nv_bfloat16*>(&raw), v);
        }
      }
      *reinterpret_cast<uint4*>(&a_s[r][kk]) = raw;
    }
    for (int idx = tid; idx < kMmaN * (kMmaK / 8); idx += kMmaThreads) {
      const int n = idx / (kMmaK / 8), kk = (idx % (kMmaK / 8)) * 8;
      const bool live = n0 + n < N && k0 + kk < K;
      uint4 g = make_uint4(0, 0, 0, 0), u = make_uint4(0, 0, 0, 0);
      if (live) g = *reinterpret_cast<const uint4*>(w_e + (size_t)(n0 + n) * K + k0 + kk);
      *reinterpret_cast<uint4*>(&w_s[0][n][kk]) = g;
      if (SWIGLU) {
        if (live) u = *reinterpret_cast<const uint4*>(w_e + ((size_t)N + n0 + n) * K + k0 + kk);
        *reinterpret_cast<uint4*>(&w_s[1][n][kk]) = u;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kMmaK; kk += 16) {
      wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa;
      wmma::load_matrix_sync(fa, &a_s[wr * 16][kk], kMmaK + kMmaPad);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb;
        wmma::load_matrix_sync(fb, &w_s[0][wc * 32 + i * 16][kk], kMmaK + kMmaPad);
        wmma::mma_sync(acc[i], fa, fb, acc[i]);
        if (SWIGLU) {
          wmma::load_matrix_sync(fb, &w_s[1][wc * 32 + i * 16][kk], kMmaK + kMmaPad);
          wmma::mma_sync(acc_up[i], fa, fb, acc_up[i]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (SWIGLU) {
#pragma unroll
      for (int e = 0; e < acc[i].num_elements; ++e) acc[i].x[e] = routed_glu(acc[i].x[e], acc_up[i].x[e], limit);
    }
    wmma::store_matrix_sync(&c_s[warp][0][0], acc[i], 16 + 4, wmma::mem_row_major);
    __syncwarp();
    for (int idx = lane; idx < 256; idx += 32) {
      const int r = idx / 16, c = idx % 16;
      const int local = wr * 16 + r, n = n0 + wc * 32 + i * 16 + c;
      if (local < rows && n < N) {
        const int slot = first + local;
        const float v = c_s[warp][r][c];
        if (SWIGLU) out[(size_t)slot * N + n] = __float2bfloat16_rn(v);
        else out32[(size_t)plan.dest[slot] * N + n] = scale_out ? v * scale_s[local] : v;
      }
    }
    __syncwarp();
  }
}

// VEC consecutive elements as floats (16 bytes when VEC is 8 for bfloat16 or 4 for float; one element otherwise).
template <typename T, int VEC>
__device__ __forceinline__ void load_run(const T* p, float (&v)[VEC]) {
  if constexpr (VEC == 8) load8(p, v);
  else if constexpr (VEC == 4) { const float4 q = load4(p); v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w; }
  else v[0] = to_float(p[0]);
}

// ---- around the grouped product on the tcgen05 kernel (prompt portions in bfloat16) --------------------------------------
// gathered[slot, :] = x[source[slot], :] (* scale[slot]): the rows sorted by expert, as the product's A operand.
template <typename T>
__global__ void routed_gather_kernel(const T* __restrict__ x, int x_stride, int* __restrict__ plan_base, int pairs,
                                     int experts, int tile, T* __restrict__ gathered, int hidden, int scale_in) {
  const RoutePlan plan = plan_views(plan_base, pairs, experts, tile);
  const int slot = blockIdx.x;
  if (slot >= plan.offsets[experts]) return;  // fewer slots than pairs: some pairs go to no expert's product
  const T* src = x + (size_t)plan.source[slot] * x_stride;
  const float scale = scale_in ? plan.scale[slot] : 1.f;
  T* dst = gathered + (size_t)slot * hidden;
  constexpr int WIDE = sizeof(T) == 2 ? 8 : 4;
  if (hidden % WIDE == 0 && x_stride % WIDE == 0 && (((uintptr_t)x | (uintptr_t)gathered) & 15) == 0) {
    for (int c = threadIdx.x * WIDE; c < hidden; c += blockDim.x * WIDE) {  // 16 bytes a thread and round
      float v[WIDE];
      load_run<T, WIDE>(src + c, v);
#pragma unroll
      for (int i = 0; i < WIDE; ++i) v[i] *= scale;
      if constexpr (WIDE == 8) store8(dst + c, v);
      else store4(dst + c, make_float4(v[0], v[1], v[2], v[3]));
    }
    return;
  }
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = from_float<T>(to_float(src[c]) * scale);
}

// out[dest[slot], :] = y[slot, :] (* scale[slot]): the product's rows back in the order [choice, token].
__global__ void routed_scatter_kernel(const float* __restrict__ y, int* __restrict__ plan_base, int pairs, int experts,
                                      int tile, float* __restrict__ out, int hidden, int scale_out) {
  const RoutePlan plan = plan_views(plan_base, pairs, experts, tile);
  const int slot = blockIdx.x;
  if (slot >= plan.offsets[experts]) return;
  const float scale = scale_out ? plan.scale[slot] : 1.f;
  const float* src = y + (size_t)slot * hidden;
  float* dst = out + (size_t)plan.dest[slot] * hidden;
  if (hidden % 4 == 0 && (((uintptr_t)y | (uintptr_t)out) & 15) == 0) {
    for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(src + c);
      *reinterpret_cast<float4*>(dst + c) = make_float4(v.x * scale, v.y * scale, v.z * scale, v.w * scale);
    }
    return;
  }
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = src[c] * scale;
}

// Pairs whose id lies behind the experts' (experts .. experts + identity - 1) stand for an expert that returns its
// input: out[choice, token, :] = weight * x[token, :].  A block per pair; pairs of real experts are left alone.
template <typename T>
__global__ void routed_identity_kernel(const T* __restrict__ x, int x_stride, const int* __restrict__ ids,
                                       const float* __restrict__ weights, int tokens, int top, int experts,
                                       float* __restrict__ out, int hidden) {
  const int p = blockIdx.x;
  if (ids[p] < experts) return;
  const int token = p / top, choice = p % top;
  const float w = weights[p];
  const T* src = x + (size_t)token * x_stride;
  float* dst = out + ((size_t)choice * tokens + token) * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = w * to_float(src[c]);
}

// ---- grouped products of steps with few rows per expert: every weight row is streamed once per tile of eight rows -------
// A tile's rows of A (gathered, scaled) wait in shared memory; a warp takes two weight rows at a time (the gate and the up
// row of one output column, or two neighbouring columns of the down product), every lane a run of VEC elements of K per
// round, all loads of a round independent of one another; no barrier inside the walk over K.
constexpr int kRowsR = 8, kRowsWarps = 8;


template <typename T, bool SWIGLU, int VEC>
__global__ void __launch_bounds__(kRowsWarps * 32, 3)
grouped_rows_kernel(int rounds, const T* __restrict__ a, int a_stride, const T* __restrict__ w, int* __restrict__ plan_base, int pairs,
                    int experts, T* __restrict__ out, float* __restrict__ out32, int N, int K, int gather, int scale_in,
                    int scale_out, float limit) {
  extern __shared__ __align__(16) unsigned char rows_raw[];
  T* a_s = reinterpret_cast<T*>(rows_raw);  // [kRowsR][K]
  __shared__ int src_s[kRowsR];
  __shared__ float scale_s[kRowsR];
  const RoutePlan plan = plan_views(plan_base, pairs, experts, kRowsR);
  const int tile = blockIdx.x;
  if (tile >= *plan.num_tiles) return;
  const int expert = plan.tile_expert[tile], first = plan.tile_first[tile], rows = plan.tile_rows[tile];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < kRowsR) {
    const int slot = first + min(tid, rows - 1);
    src_s[tid] = gather ? plan.source[slot] : slot;
    scale_s[tid] = plan.scale[slot];
  }
  __syncthreads();
  for (int r = 0; r < rows; ++r) {  // the expert reads weight * x in the engine's type
    const T* src = a + (size_t)src_s[r] * a_stride;
    const float scale = scale_in ? scale_s[r] : 1.f;
    for (int k = tid * VEC; k < K; k += kRowsWarps * 32 * VEC) {
      float v[VEC];
      load_run<T, VEC>(src + k, v);
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[i] *= scale;
      if constexpr (VEC == 8) store8(a_s + (size_t)r * K + k, v);
      else if constexpr (VEC == 4) store4(a_s + (size_t)r * K + k, make_float4(v[0], v[1], v[2], v[3]));
      else a_s[(size_t)r * K + k] = from_float<T>(v[0]);
    }
  }
  __syncthreads();
  const size_t w_rows = SWIGLU ? 2 * (size_t)N : (size_t)N;
  const T* w_e = w + (size_t)expert * w_rows * K;
  constexpr int COLS = SWIGLU ? 1 : 2;  // output columns a warp finishes per round
  const int col0 = (blockIdx.y * kRowsWarps * rounds + warp * rounds) * COLS;  // `rounds` pairs of weight rows a warp
#pragma unroll 1
  for (int round = 0; round < rounds; ++round) {
    const int n = col0 + round * COLS;
    if (n >= N) break;
    const bool second = SWIGLU || n + 1 < N;
    const T* w0 = w_e + (size_t)n * K;
    const T* w1 = w_e + (SWIGLU ? (size_t)N + n : (second ? (size_t)n + 1 : (size_t)n)) * K;
    float acc0[kRowsR], acc1[kRowsR];
#pragma unroll
    for (int r = 0; r < kRowsR; ++r) acc0[r] = acc1[r] = 0.f;
    // Three rounds of K at a time: their six runs of the two weight rows are requested before any is used.
    constexpr int AHEAD = 3;
    for (int k0 = lane * VEC; k0 < K; k0 += AHEAD * 32 * VEC) {
      float x0[AHEAD][VEC], x1[AHEAD][VEC];
#pragma unroll
      for (int u = 0; u < AHEAD; ++u) {
        const int k = k0 + u * 32 * VEC;
        if (k < K) {
          load_run<T, VEC>(w0 + k, x0[u]);
          load_run<T, VEC>(w1 + k, x1[u]);
        } else {
#pragma unroll
          for (int i = 0; i < VEC; ++i) x0[u][i] = x1[u][i] = 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < AHEAD; ++u) {
        const int k = min(k0 + u * 32 * VEC, K - VEC);  // (a round past the end multiplies zeros)
#pragma unroll
        for (int r = 0; r < kRowsR; ++r) {
          if (r < rows) {
            float av[VEC];
            load_run<T, VEC>(a_s + (size_t)r * K + k, av);
#pragma unroll
            for (int i = 0; i < VEC; ++i) { acc0[r] += av[i] * x0[u][i]; acc1[r] += av[i] * x1[u][i]; }
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kRowsR; ++r) {
      if (r < rows) { acc0[r] = warp_sum(acc0[r]); acc1[r] = warp_sum(acc1[r]); }
    }
    if (lane < rows) {
      float v0 = 0.f, v1 = 0.f;
#pragma unroll
      for (int r = 0; r < kRowsR; ++r)
        if (r == lane) { v0 = acc0[r]; v1 = acc1[r]; }
      const int slot = first + lane;
      if (SWIGLU) {
        out[(size_t)slot * N + n] = from_float<T>(routed_glu(v0, v1, limit));
      } else {
        const float s = scale_out ? scale_s[lane] : 1.f;
        float* dst = out32 + (size_t)plan.dest[slot] * N + n;
        dst[0] = v0 * s;
        if (second) dst[1] = v1 * s;
      }
    }
  }
}

template <typename T, bool SWIGLU>
static int launch_grouped_rows(const T* a, int a_stride, const T* w, int* plan, int pairs, int experts, T* out, float* out32,
                               int N, int K, int gather, int scale_in, int scale_out, float limit, unsigned max_tiles, cudaStream_t stream) {
  constexpr int WIDE = sizeof(T) == 2 ? 8 : 4;
  const bool vec = K % WIDE == 0 && a_stride % WIDE == 0 && (((uintptr_t)a | (uintptr_t)w) & 15) == 0;
  const size_t shared = (size_t)kRowsR * K * sizeof(T);
  // Pairs of weight rows a warp takes in turn: fewer where the product has few columns, so that the grid stays large.
  const int rounds = (long long)N * (SWIGLU ? 2 : 1) >= 4096 ? 4 : 2;
  const int per_block = kRowsWarps * rounds * (SWIGLU ? 1 : 2);
  const dim3 grid(max_tiles, (N + per_block - 1) / per_block);
  auto run = [&](auto kernel) {
    if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    kernel<<<grid, kRowsWarps * 32, shared, stream>>>(rounds, a, a_stride, w, plan, pairs, experts, out, out32, N, K, gather, scale_in,
                                                     scale_out, limit);
  };
  if (vec) run(grouped_rows_kernel<T, SWIGLU, WIDE>);
  else run(grouped_rows_kernel<T, SWIGLU, 1>);
  DISTIE_LAUNCH_CHECK();
  return 0;
}

}  // namespace distie

using namespace distie;

// x [tokens, hidden] and router [experts, hidden] of one type; ids, weights [tokens, top].
extern "C" int distie_route_top(const void* x, int x_stride, const void* router, int tokens, int hidden, int experts,
                                int top, int* ids, float* weights, int group_count, int group_keep, float weight_scale,
                                int extra, float* extra_out, int softmax, const float* correction, int normalise,
                                int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (correction != nullptr && group_count > 1 && group_keep < group_count) return DISTIE_ERR_ARG;
  if (hidden < 1 || experts < 1 || top < 1 || top > experts || top > kMaxTop || experts > 8192 || group_count < 1 ||
      experts % group_count != 0 || group_keep < 1 || group_keep > group_count || extra < 0 || (extra > 0 && !extra_out) ||
      top > group_keep * (experts / group_count))
    return DISTIE_ERR_ARG;
  if (dtype != DISTIE_BF16 && dtype != DISTIE_F32) return DISTIE_ERR_UNSUPPORTED;
  const int wide = dtype == DISTIE_BF16 ? 8 : 4;
  const bool vec = hidden % wide == 0 && ((uintptr_t)router & 15) == 0;
  const int tok = tokens >= 64 && (size_t)4 * (hidden + 2 * experts + group_count) * sizeof(float) <= 96 * 1024 ? 4 : 1;
  const size_t shared = (size_t)tok * (hidden + 2 * experts + group_count) * sizeof(float);
  if (shared > 200 * 1024) return DISTIE_ERR_UNSUPPORTED;
  const unsigned blocks = (unsigned)((tokens + tok - 1) / tok);
  auto run = [&](auto kernel, auto xp, auto rp) {
    if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    kernel<<<blocks, kRouteThreads, shared, stream>>>(xp, x_stride, rp, tokens, hidden, experts, top, ids, weights, group_count,
                                                      group_keep, weight_scale, extra, extra_out, softmax, correction, normalise);
  };
#define DISTIE_ROUTE(T, VECV)                                                                             \
  do {                                                                                                    \
    if (tok == 4) run(route_top_kernel<T, 4, VECV>, (const T*)x, (const T*)router);                       \
    else run(route_top_kernel<T, 1, VECV>, (const T*)x, (const T*)router);                                \
  } while (0)
  if (dtype == DISTIE_BF16) { if (vec) DISTIE_ROUTE(__nv_bfloat16, 8); else DISTIE_ROUTE(__nv_bfloat16, 1); }
  else { if (vec) DISTIE_ROUTE(float, 4); else DISTIE_ROUTE(float, 1); }
#undef DISTIE_ROUTE
  DISTIE_LAUNCH_CHECK();
  return 0;
}

// Rows per tile of the grouped products for this type and these sizes (the plan is made for it): few rows per
// expert stream the weights past tiles of eight rows; more go to tiles of 64 (tensor cores) or 32 (FMA pipe).
extern "C" int distie_routed_tile(int dtype, int hidden, int ff, int pairs, int experts) {
  const int widest = hidden > ff ? hidden : ff;
  if (pairs <= 16 * experts && (size_t)kRowsR * widest * (dtype == DISTIE_BF16 ? 2 : 4) <= 160 * 1024) return kRowsR;
  return (dtype == DISTIE_BF16 && hidden % 8 == 0 && ff % 8 == 0) ? kMmaM : kTileM;
}

// int32 words of the plan for `pairs` (token, choice) pairs.
extern "C" long long distie_route_plan_words(int pairs, int experts, int tile) {
  const long long max_tiles = (pairs + tile - 1) / tile + experts;
  return 1 + (experts + 1) + 3 * max_tiles + 3LL * pairs;
}

// Rows of `out` [top, tokens, hidden] of the pairs whose id is experts or more: weight * x[token] (see
// routed_identity_kernel).
extern "C" int distie_routed_identity(const void* x, int x_stride, const int* ids, const float* weights, int tokens, int top,
                                      int experts, float* out, int hidden, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (dtype == DISTIE_BF16)
    routed_identity_kernel<<<tokens * top, threads, 0, stream>>>((const __nv_bfloat16*)x, x_stride, ids, weights, tokens, top,
                                                                experts, out, hidden);
  else if (dtype == DISTIE_F32)
    routed_identity_kernel<<<tokens * top, threads, 0, stream>>>((const float*)x, x_stride, ids, weights, tokens, top, experts,
                                                                out, hidden);
  else
    return DISTIE_ERR_UNSUPPORTED;
  DISTIE_LAUNCH_CHECK();
  return 0;
}

// x [tokens, hidden]; gate_up [experts, 2 ff, hidden]; down [experts, hidden, ff]; ids, weights [tokens, top];
// ids experts .. experts + identity - 1 stand for experts that return their input (weight on the output only).
// plan: distie_route_plan_words int32; mid [tokens * top, ff] of the type; out [top, tokens, hidden] float32.
// weight_on_input: the pair's weight multiplies the expert's input, else its output.
extern "C" int distie_routed_swiglu(const void* x, int x_stride, const int* ids, const float* weights, const void* gate_up,
                                    const void* down, int* plan, void* mid, float* out, int tokens, int top, int experts,
                                    int hidden, int ff, int weight_on_input, float limit, int identity, int dtype, int* error,
                                    cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (top < 1 || experts < 1 || hidden < 1 || ff < 1 || experts > 4096 || identity < 0 || (identity > 0 && weight_on_input))
    return DISTIE_ERR_ARG;
  if (dtype != DISTIE_BF16 && dtype != DISTIE_F32) return DISTIE_ERR_UNSUPPORTED;
  const int pairs = tokens * top;
  const int tile = distie_routed_tile(dtype, hidden, ff, pairs, experts);
  const bool mma = tile == kMmaM && x_stride % 8 == 0 &&
                   (((uintptr_t)x | (uintptr_t)gate_up | (uintptr_t)down | (uintptr_t)mid) & 15) == 0;
  if (tile == kMmaM && !mma) return DISTIE_ERR_UNSUPPORTED;
  route_plan_kernel<<<1, 1024, 2 * (size_t)experts * sizeof(int), stream>>>(ids, weights, tokens, top, experts, tile, plan,
                                                                           error, identity);
  DISTIE_LAUNCH_CHECK();
  if (identity > 0) {
    const int status = distie_routed_identity(x, x_stride, ids, weights, tokens, top, experts, out, hidden, dtype, stream);
    if (status != 0) return status;
  }
  const unsigned max_tiles = (unsigned)((pairs + tile - 1) / tile + experts);
  const int in = weight_on_input ? 1 : 0;
  if (tile == kRowsR) {
    int status;
    if (dtype == DISTIE_BF16) {
      status = launch_grouped_rows<__nv_bfloat16, true>((const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)gate_up, plan,
                                                        pairs, experts, (__nv_bfloat16*)mid, nullptr, ff, hidden, 1, in, 0,
                                                        limit, max_tiles, stream);
      if (status != 0) return status;
      return launch_grouped_rows<__nv_bfloat16, false>((const __nv_bfloat16*)mid, ff, (const __nv_bfloat16*)down, plan, pairs,
                                                       experts, nullptr, out, hidden, ff, 0, 0, 1 - in, 0.f, max_tiles, stream);
    }
    status = launch_grouped_rows<float, true>((const float*)x, x_stride, (const float*)gate_up, plan, pairs, experts,
                                              (float*)mid, nullptr, ff, hidden, 1, in, 0, limit, max_tiles, stream);
    if (status != 0) return status;
    return launch_grouped_rows<float, false>((const float*)mid, ff, (const float*)down, plan, pairs, experts, nullptr, out,
                                             hidden, ff, 0, 0, 1 - in, 0.f, max_tiles, stream);
  }
  if (mma) {
    const dim3 up_grid(max_tiles, (ff + kMmaN - 1) / kMmaN), down_grid(max_tiles, (hidden + kMmaN - 1) / kMmaN);
    grouped_product_mma_kernel<true><<<up_grid, kMmaThreads, 0, stream>>>(
        (const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)gate_up, plan, pairs, experts, (__nv_bfloat16*)mid,
        nullptr, ff, hidden, 1, in, 0, limit);
    DISTIE_LAUNCH_CHECK();
    grouped_product_mma_kernel<false><<<down_grid, kMmaThreads, 0, stream>>>(
        (const __nv_bfloat16*)mid, ff, (const __nv_bfloat16*)down, plan, pairs, experts, nullptr, out, hidden, ff, 0, 0,
        1 - in, 0.f);
    DISTIE_LAUNCH_CHECK();
    return 0;
  }
  const dim3 up_grid(max_tiles, (ff + kTileN - 1) / kTileN), down_grid(max_tiles, (hidden + kTileN - 1) / kTileN);
  if (dtype == DISTIE_BF16) {
    grouped_product_kernel<__nv_bfloat16, true><<<up_grid, kGroupedThreads, 0, stream>>>(
        (const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)gate_up, plan, pairs, experts, (__nv_bfloat16*)mid,
        nullptr, ff, hidden, 1, in, 0, limit);
    DISTIE_LAUNCH_CHECK();
    grouped_product_kernel<__nv_bfloat16, false><<<down_grid, kGroupedThreads, 0, stream>>>(
        (const __nv_bfloat16*)mid, ff, (const __nv_bfloat16*)down, plan, pairs, experts, nullptr, out, hidden, ff, 0, 0,
        1 - in, 0.f);
  } else {
    grouped_product_kernel<float, true><<<up_grid, kGroupedThreads, 0, stream>>>(
        (const float*)x, x_stride, (const float*)gate_up, plan, pairs, experts, (float*)mid, nullptr, ff, hidden, 1, in, 0, limit);
    DISTIE_LAUNCH_CHECK();
    grouped_product_kernel<float, false><<<down_grid, kGroupedThreads, 0, stream>>>(
        (const float*)mid, ff, (const float*)down, plan, pairs, experts, nullptr, out, hidden, ff, 0, 0, 1 - in, 0.f);
  }
  DISTIE_LAUNCH_CHECK();
  return 0;
}

// The plan alone (see route_plan_kernel), for callers that run the grouped products themselves; `tile` rows a tile.
extern "C" int distie_route_plan(const int* ids, const float* weights, int tokens, int top, int experts, int tile,
                                 int* plan, int* error, int identity, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (top < 1 || experts < 1 || experts > 4096 || tile < 1 || identity < 0) return DISTIE_ERR_ARG;
  route_plan_kernel<<<1, 1024, 2 * (size_t)experts * sizeof(int), stream>>>(ids, weights, tokens, top, experts, tile, plan,
                                                                           error, identity);
  DISTIE_LAUNCH_CHECK();
  return 0;
}

extern "C" int distie_routed_gather(const void* x, int x_stride, int* plan, int pairs, int experts, int tile, void* gathered,
                                    int hidden, int scale_in, int dtype, cudaStream_t stream) {
  if (pairs <= 0) return 0;
  if (dtype == DISTIE_BF16)
    routed_gather_kernel<<<pairs, 256, 0, stream>>>((const __nv_bfloat16*)x, x_stride, plan, pairs, experts, tile,
                                                   (__nv_bfloat16*)gathered, hidden, scale_in);
  else if (dtype == DISTIE_F32)
    routed_gather_kernel<<<pairs, 256, 0, stream>>>((const float*)x, x_stride, plan, pairs, experts, tile, (float*)gathered,
                                                   hidden, scale_in);
  else
    return DISTIE_ERR_UNSUPPORTED;
  DISTIE_LAUNCH_CHECK();
  return 0;
}

extern "C" int distie_routed_scatter(const float* y, int* plan, int pairs, int experts, int tile, float* out, int hidden,
                                     int scale_out, cudaStream_t stream) {
  if (pairs <= 0) return 0;
  routed_scatter_kernel<<<pairs, 256, 0, stream>>>(y, plan, pairs, experts, tile, out, hidden, scale_out);
  DISTIE_LAUNCH_CHECK();
  return 0;
}

// ids and weights from float32 logits [tokens, experts] (row stride logit_stride): see route_pick_kernel.
extern "C" int distie_route_pick(const float* logits, int logit_stride, int tokens, int experts, int top, int* ids,
                                 float* weights, int group_count, int group_keep, float weight_scale, int softmax,
                                 const float* correction, int normalise, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (correction != nullptr && group_count > 1 && group_keep < group_count) return DISTIE_ERR_ARG;
  if (experts < 1 || top < 1 || top > experts || top > kMaxTop || experts > 4096 || group_count < 1 ||
      experts % group_count != 0 || group_keep < 1 || group_keep > group_count || top > group_keep * (experts / group_count))
    return DISTIE_ERR_ARG;
  const int warps = kRouteThreads / 32;
  const size_t shared = (size_t)warps * (2 * experts + group_count) * sizeof(float);
  if (shared > 48 * 1024) cudaFuncSetAttribute(route_pick_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
  route_pick_kernel<<<(tokens + warps - 1) / warps, kRouteThreads, shared, stream>>>(logits, logit_stride, tokens, experts,
                                                                                    top, ids, weights, group_count, group_keep,
                                                                                    weight_scale, softmax, correction, normalise);
  DISTIE_LAUNCH_CHECK();
  return 0;
}
