// Kernels of an attention through a latent: every token stores ONE row [latent | rotated key part] that all
// heads share; queries are folded into the latent's space, the attention mixes stored latents, and the values'
// up-projection is applied to the mix.
//
//   latent_kv_write   float32 projection [q latent | kv latent | key part | ...] (or its slices) -> both RMS norms,
//                     the rotation of the key part, the token's row into its page, the normed query latent out.
//   latent_q_prepare  float32 query projection (per head [plain | to rotate]) -> plain part [heads, T, dim] and
//                     rotated part [T, heads, rot] in the engine's type.
//   latent_attention  (kernels below) causal softmax over the request's rows with a sink in the denominator.
//   latent_gate       [heads, T, vdim] -> [T, heads * vdim] times sigmoid(gate[t, head]).
//   glu_act           float32 [T, 2 ff] (gate columns, then up columns) -> SwiGLU or its capped form, optionally
//                     times sigmoid of a per-row logit; float32 [T, ff] -> squared ReLU.
//
// Arithmetic is float32 everywhere (norm statistics, angles, scores, softmax, the mix); T (float or bfloat16) is
// the type of what is stored.  Nothing reads host-side batch data.
#include "common.cuh"

namespace distie {

__device__ __forceinline__ float sum_slices(const float* p, int slices, long long slice_stride) {
  float v = p[0];
  for (int s = 1; s < slices; ++s) v += p[(size_t)s * slice_stride];
  return v;
}

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

// The pair (a, b) of a rotation of `rotary_dim` dimensions: neighbours (interleaved) or half a rotation apart.
__device__ __forceinline__ void rotary_pair(int i, int rotary_dim, int interleaved, int& a, int& b) {
  if (interleaved) { a = 2 * i; b = 2 * i + 1; }
  else { a = i; b = i + rotary_dim / 2; }
}

// One block per token.  Dynamic shared memory: q_rank + kv_rank + rot_dim floats.
template <typename T>
__global__ void __launch_bounds__(256)
latent_kv_write_kernel(const float* __restrict__ proj, int row_stride, int slices, long long slice_stride, int q_rank,
                       const float* __restrict__ q_norm, int kv_rank, const float* __restrict__ kv_norm, int rot_dim,
                       float eps, T* __restrict__ q_out, int q_out_stride, const int* __restrict__ positions,
                       const int* __restrict__ token_seq, const int* __restrict__ seq_seat,
                       const int* __restrict__ block_table, int table_width, const float* __restrict__ inv_freq,
                       float factor, int rotary_dim, int interleaved, T* __restrict__ k_cache, int page_size,
                       int num_pages, int write, int* __restrict__ error) {
  extern __shared__ float row_s[];
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int total = q_rank + (write ? kv_rank + rot_dim : 0);
  const float* src = proj + (size_t)t * row_stride;
  float sq_q = 0.f, sq_kv = 0.f;
  for (int c = threadIdx.x; c < total; c += blockDim.x) {
    const float v = sum_slices(src + c, slices, slice_stride);
    row_s[c] = v;
    if (c < q_rank) sq_q += v * v;
    else if (c < q_rank + kv_rank) sq_kv += v * v;
  }
  sq_q = block_sum(sq_q, scratch);
  const float inv_q = 1.f / sqrtf(sq_q / (float)q_rank + eps);
  for (int c = threadIdx.x; c < q_rank; c += blockDim.x)
    q_out[(size_t)t * q_out_stride + c] = from_float<T>(row_s[c] * inv_q * q_norm[c]);
  if (!write) return;
  sq_kv = block_sum(sq_kv, scratch);
  const float inv_kv = 1.f / sqrtf(sq_kv / (float)kv_rank + eps);
  const int pos = positions[t];
  const int seat = seq_seat[token_seq[t]];
  const int column = pos / page_size;
  const int page = column < table_width ? block_table[(size_t)seat * table_width + column] : -1;
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0 && error) atomicExch(error, 2);
    return;
  }
  T* dst = k_cache + ((size_t)page * page_size + pos % page_size) * (size_t)(kv_rank + rot_dim);
  for (int c = threadIdx.x; c < kv_rank; c += blockDim.x)
    dst[c] = from_float<T>(row_s[q_rank + c] * inv_kv * kv_norm[c]);
  const float* part = row_s + q_rank + kv_rank;
  for (int i = threadIdx.x; i < rotary_dim / 2; i += blockDim.x) {
    int a, b;
    rotary_pair(i, rotary_dim, interleaved, a, b);
    float sn, cs;
    sincosf((float)pos * inv_freq[i], &sn, &cs);
    sn *= factor; cs *= factor;
    const float u = part[a], v = part[b];
    dst[kv_rank + a] = from_float<T>(u * cs - v * sn);
    dst[kv_rank + b] = from_float<T>(v * cs + u * sn);
  }
  for (int c = rotary_dim + threadIdx.x; c < rot_dim; c += blockDim.x) dst[kv_rank + c] = from_float<T>(part[c]);
}

// One block per token: every head's plain columns to plain[head, t, :], its rotated columns to rotated[t, head, :].
template <typename T>
__global__ void __launch_bounds__(256)
latent_q_prepare_kernel(const float* __restrict__ q, int row_stride, int slices, long long slice_stride, int tokens,
                        int heads, int dim, int rot_dim, const int* __restrict__ positions,
                        const float* __restrict__ inv_freq, float factor, int rotary_dim, int interleaved,
                        T* __restrict__ plain, T* __restrict__ rotated) {
  const int t = blockIdx.x;
  const float* src = q + (size_t)t * row_stride;
  const int per_head = dim + rot_dim;
  for (int c = threadIdx.x; c < heads * dim; c += blockDim.x) {
    const int h = c / dim, d = c % dim;
    plain[((size_t)h * tokens + t) * dim + d] = from_float<T>(sum_slices(src + h * per_head + d, slices, slice_stride));
  }
  const int pos = positions[t];
  const int half = rotary_dim / 2, loose = rot_dim - rotary_dim;
  for (int c = threadIdx.x; c < heads * (half + loose); c += blockDim.x) {
    const int h = c / (half + loose), i = c % (half + loose);
    const float* part = src + h * per_head + dim;
    T* dst = rotated + ((size_t)t * heads + h) * rot_dim;
    if (i < half) {
      int a, b;
      rotary_pair(i, rotary_dim, interleaved, a, b);
      float sn, cs;
      sincosf((float)pos * inv_freq[i], &sn, &cs);
      sn *= factor; cs *= factor;
      const float u = sum_slices(part + a, slices, slice_stride), v = sum_slices(part + b, slices, slice_stride);
      dst[a] = from_float<T>(u * cs - v * sn);
      dst[b] = from_float<T>(v * cs + u * sn);
    } else {
      const int e = rotary_dim + i - half;
      dst[e] = from_float<T>(sum_slices(part + e, slices, slice_stride));
    }
  }
}

// y [heads, T, vdim] -> out [T, heads * vdim], head h of token t times sigmoid(gate[t, h]) (gate: float32 slices).
template <typename T>
__global__ void __launch_bounds__(256)
latent_gate_kernel(const T* __restrict__ y, int tokens, int heads, int vdim, const float* __restrict__ gate,
                   int gate_stride, int gate_slices, long long gate_slice_stride, T* __restrict__ out, int out_stride) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < heads * vdim; c += blockDim.x) {
    const int h = c / vdim, d = c % vdim;
    float v = to_float(y[((size_t)h * tokens + t) * vdim + d]);
    if (gate) v *= sigmoid_f(sum_slices(gate + (size_t)t * gate_stride + h, gate_slices, gate_slice_stride));
    out[(size_t)t * out_stride + c] = from_float<T>(v);
  }
}

// The hidden activation of a gated layer on float32 accumulators.  limit <= 0: silu(g) * u; limit > 0:
// g' = min(g, limit), u' = clamp(u, -limit, limit), g' * sigmoid(1.702 g') * (u' + 1).
__device__ __forceinline__ float glu_value(float g, float u, float limit) {
  if (limit > 0.f) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * sigmoid_f(1.702f * g) * (u + 1.f);
  }
  return g * sigmoid_f(g) * u;
}

// kind 0: gated (x is [T, 2 ff]); kind 1: squared ReLU (x is [T, ff]).
template <typename T>
__global__ void __launch_bounds__(256)
glu_act_kernel(const float* __restrict__ x, int row_stride, int slices, long long slice_stride, int tokens, int ff,
               int kind, float limit, const float* __restrict__ row_gate, int gate_stride, int gate_slices,
               long long gate_slice_stride, T* __restrict__ out, int out_stride) {
  const int t = blockIdx.y;
  const float* src = x + (size_t)t * row_stride;
  float row_scale = 1.f;
  if (row_gate) row_scale = sigmoid_f(sum_slices(row_gate + (size_t)t * gate_stride, gate_slices, gate_slice_stride));
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < ff; c += gridDim.x * blockDim.x) {
    float v;
    if (kind == 1) {
      const float z = fmaxf(sum_slices(src + c, slices, slice_stride), 0.f);
      v = z * z;
    } else {
      v = glu_value(sum_slices(src + c, slices, slice_stride), sum_slices(src + ff + c, slices, slice_stride), limit);
    }
    out[(size_t)t * out_stride + c] = from_float<T>(v * row_scale);
  }
}

// ---- attention over the stored rows: the size-agnostic kernel ----------------------------------------------------
// A block takes one token, HB of its heads and one of `splits` equal parts of the keys the token sees
// (positions 0 .. pos of its request).  A warp takes every fourth key of the part: it loads the key's row once
// (RMAX elements a lane) and uses it for all HB heads, as key (the whole row against [folded | rotated]) and as
// value (its first `rank` columns).  Online softmax per head in float32; the warps' results are merged through
// shared memory.  With one split the block divides by the sum, to which the head's sink adds exp(sink); with
// more it leaves (sum of weighted latents, maximum, sum) per split and latent_merge_kernel finishes.
// Which keys a token reads depends on its position and its request's block table only.
constexpr int kLatentWarps = 4;

template <typename T, int RMAX, int HB>
__global__ void __launch_bounds__(kLatentWarps * 32)
latent_attention_kernel(const T* __restrict__ folded, const T* __restrict__ rotated, T* __restrict__ out,
                        float* __restrict__ partial, int tokens, int heads, int rank, int rot,
                        const int* __restrict__ positions, const int* __restrict__ token_seq,
                        const int* __restrict__ seq_seat, const int* __restrict__ block_table, int table_width,
                        const T* __restrict__ k_cache, int page_size, int num_pages, float scale,
                        const float* __restrict__ sink, int splits, int first, int* __restrict__ error) {
  extern __shared__ float latent_s[];
  constexpr int kRow = RMAX * 32;
  float* q_s = latent_s;                                   // [HB][kRow], zero beyond the row
  float* acc_s = q_s + HB * kRow;                          // [warps][HB][rank]
  float* ml_s = acc_s + (size_t)kLatentWarps * HB * rank;  // [warps][HB][2]
  const int t = first + blockIdx.x, h0 = blockIdx.y * HB, split = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = rank + rot;
  const int live = min(HB, heads - h0);
  for (int c = threadIdx.x; c < HB * kRow; c += blockDim.x) {
    const int hb = c / kRow, e = c % kRow;
    float v = 0.f;
    if (hb < live) {
      if (e < rank) v = to_float(folded[((size_t)(h0 + hb) * tokens + t) * rank + e]);
      else if (e < row) v = to_float(rotated[((size_t)t * heads + h0 + hb) * rot + e - rank]);
    }
    q_s[c] = v;
  }
  __syncthreads();
  const int pos = positions[t];
  const int seat = seq_seat[token_seq[t]];
  const int* table = block_table + (size_t)seat * table_width;
  const int count = pos + 1;
  const int per = (count + splits - 1) / splits;
  const int begin = split * per, end = min(count, begin + per);

  float m[HB], l[HB], acc[HB][RMAX];
#pragma unroll
  for (int hb = 0; hb < HB; ++hb) {
    m[hb] = -INFINITY;
    l[hb] = 0.f;
#pragma unroll
    for (int i = 0; i < RMAX; ++i) acc[hb][i] = 0.f;
  }
  // A key's row is on its way while the one before it is used: the loop is a chain of dependent steps (the running
  // maximum), and a load issued inside it would be waited for in full at every key.
  auto fetch = [&](int key, float (&dst)[RMAX]) -> bool {
    const int column = key / page_size;
    const int page = column < table_width ? table[column] : -1;
    if (page < 0 || page >= num_pages) {
      if (lane == 0 && error) atomicExch(error, 3);
      return false;
    }
    const T* src = k_cache + ((size_t)page * page_size + key % page_size) * (size_t)row;
#pragma unroll
    for (int i = 0; i < RMAX; ++i) {
      const int e = lane + 32 * i;
      dst[i] = e < row ? to_float(src[e]) : 0.f;
    }
    return true;
  };
  float kr[RMAX];
  bool have = begin + warp < end && fetch(begin + warp, kr);
  for (int key = begin + warp; key < end; key += kLatentWarps) {
    float ahead[RMAX];
    const bool have_ahead = key + kLatentWarps < end && fetch(key + kLatentWarps, ahead);
    if (have) {
#pragma unroll
      for (int hb = 0; hb < HB; ++hb) {
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < RMAX; ++i) dot += q_s[hb * kRow + lane + 32 * i] * kr[i];
        const float s = warp_sum(dot) * scale;
        const float m_new = fmaxf(m[hb], s);
        const float corr = expf(m[hb] - m_new);
        const float p = expf(s - m_new);
        l[hb] = l[hb] * corr + p;
#pragma unroll
        for (int i = 0; i < RMAX; ++i) acc[hb][i] = acc[hb][i] * corr + p * kr[i];
        m[hb] = m_new;
      }
    }
    have = have_ahead;
#pragma unroll
    for (int i = 0; i < RMAX; ++i) kr[i] = ahead[i];
  }
#pragma unroll
  for (int hb = 0; hb < HB; ++hb) {
    if (lane == 0) {
      ml_s[(warp * HB + hb) * 2] = m[hb];
      ml_s[(warp * HB + hb) * 2 + 1] = l[hb];
    }
#pragma unroll
    for (int i = 0; i < RMAX; ++i) {
      const int e = lane + 32 * i;
      if (e < rank) acc_s[((size_t)warp * HB + hb) * rank + e] = acc[hb][i];
    }
  }
  __syncthreads();
  for (int hb = 0; hb < live; ++hb) {
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < kLatentWarps; ++w) m_all = fmaxf(m_all, ml_s[(w * HB + hb) * 2]);
    float weight[kLatentWarps], l_all = 0.f;
#pragma unroll
    for (int w = 0; w < kLatentWarps; ++w) {
      const float mw = ml_s[(w * HB + hb) * 2];
      weight[w] = mw == -INFINITY ? 0.f : expf(mw - m_all);
      l_all += ml_s[(w * HB + hb) * 2 + 1] * weight[w];
    }
    const int head = h0 + hb;
    if (splits == 1) {
      float top = m_all, extra = 0.f;
      if (sink) {
        top = fmaxf(m_all, sink[head]);
        extra = expf(sink[head] - top);
      }
      const float shrink = m_all == -INFINITY ? 0.f : expf(m_all - top);
      const float den = l_all * shrink + extra;
      const float inv = den > 0.f ? shrink / den : 0.f;
      T* dst = out + ((size_t)head * tokens + t) * rank;
      for (int e = threadIdx.x; e < rank; e += blockDim.x) {
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < kLatentWarps; ++w) total += acc_s[((size_t)w * HB + hb) * rank + e] * weight[w];
        dst[e] = from_float<T>(total * inv);
      }
    } else {
      float* dst = partial + (((size_t)split * tokens + t) * heads + head) * (size_t)(rank + 2);
      for (int e = threadIdx.x; e < rank; e += blockDim.x) {
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < kLatentWarps; ++w) total += acc_s[((size_t)w * HB + hb) * rank + e] * weight[w];
        dst[e] = total;
      }
      if (threadIdx.x == 0) { dst[rank] = m_all; dst[rank + 1] = l_all; }
    }
  }
}

// One block per (token, head): the splits' partial results into the final row.
template <typename T>
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* __restrict__ partial, T* __restrict__ out, int tokens, int heads, int rank, int splits,
                    const float* __restrict__ sink, int first) {
  const int t = first + blockIdx.x, head = blockIdx.y;
  __shared__ float weight_s[64], max_s[64], sum_s[64];  // the launchers take at most 64 splits
  const size_t stride = (size_t)tokens * heads * (rank + 2);
  const float* mine = partial + ((size_t)t * heads + head) * (size_t)(rank + 2);
  // One round trip for all the splits' maxima and sums, a thread each; the rest of the bookkeeping is on chip.
  for (int s = threadIdx.x; s < splits; s += blockDim.x) {
    max_s[s] = mine[s * stride + rank];
    sum_s[s] = mine[s * stride + rank + 1];
  }
  __syncthreads();
  float top = sink ? sink[head] : -INFINITY;
  for (int s = 0; s < splits; ++s) top = fmaxf(top, max_s[s]);
  float den = sink ? expf(sink[head] - top) : 0.f;
  for (int s = 0; s < splits; ++s)
    if (max_s[s] != -INFINITY) den += sum_s[s] * expf(max_s[s] - top);
  const float inv = den > 0.f ? 1.f / den : 0.f;
  for (int s = threadIdx.x; s < splits; s += blockDim.x)
    weight_s[s] = max_s[s] != -INFINITY ? expf(max_s[s] - top) * inv : 0.f;  // (a split without keys wrote zeros)
  __syncthreads();
  // A thread takes one column (the grid's z covers the row): its loads from the splits do not depend on one another.
  T* dst = out + ((size_t)head * tokens + t) * rank;
  const int e = blockIdx.z * blockDim.x + threadIdx.x;
  if (e < rank) {
    float total = 0.f;
#pragma unroll 16
    for (int s = 0; s < splits; ++s) total += mine[s * stride + e] * weight_s[s];
    dst[e] = from_float<T>(total);
  }
}

template <typename T, int RMAX, int HB>
static int launch_latent_attention(const void* folded, const void* rotated, void* out, float* partial, int tokens,
                                   int heads, int rank, int rot, const int* positions, const int* token_seq,
                                   const int* seq_seat, const int* block_table, int table_width, const void* k_cache,
                                   int page_size, int num_pages, float scale, const float* sink, int splits,
                                   int first, int count, int* error, cudaStream_t stream) {
  const size_t shared = ((size_t)HB * RMAX * 32 + (size_t)kLatentWarps * HB * rank + kLatentWarps * HB * 2) * sizeof(float);
  auto kernel = latent_attention_kernel<T, RMAX, HB>;
  if (shared > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return (int)err;
  }
  const dim3 grid(count, (heads + HB - 1) / HB, splits);
  kernel<<<grid, kLatentWarps * 32, shared, stream>>>((const T*)folded, (const T*)rotated, (T*)out, partial, tokens, heads,
                                                      rank, rot, positions, token_seq, seq_seat, block_table, table_width,
                                                      (const T*)k_cache, page_size, num_pages, scale, sink, splits, first, error);
  DISTIE_LAUNCH_CHECK();
  if (splits > 1) {
    latent_merge_kernel<T><<<dim3(count, heads, (rank + 127) / 128), 128, 0, stream>>>(partial, (T*)out, tokens, heads, rank, splits, sink, first);
    DISTIE_LAUNCH_CHECK();
  }
  return 0;
}

template <typename T>
static int latent_attention_any(const void* folded, const void* rotated, void* out, float* partial, int tokens, int heads,
                                int rank, int rot, const int* positions, const int* token_seq, const int* seq_seat,
                                const int* block_table, int table_width, const void* k_cache, int page_size,
                                int num_pages, float scale, const float* sink, int splits, int first, int count,
                                int* error, cudaStream_t stream) {
  const int row = rank + rot;
#define DISTIE_LATENT(RMAX, HB)                                                                                     \
  return launch_latent_attention<T, RMAX, HB>(folded, rotated, out, partial, tokens, heads, rank, rot, positions,  \
                                              token_seq, seq_seat, block_table, table_width, k_cache, page_size,   \
                                              num_pages, scale, sink, splits, first, count, error, stream)
  if (row <= 128) DISTIE_LATENT(4, 8);
  if (row <= 256) DISTIE_LATENT(8, 8);
  if (row <= 512) DISTIE_LATENT(16, 4);
  if (row <= 640) DISTIE_LATENT(20, 3);
  DISTIE_LATENT(32, 2);
#undef DISTIE_LATENT
}

}  // namespace distie

using namespace distie;

extern "C" int distie_latent_kv_write(const float* proj, int row_stride, int slices, long long slice_stride, int q_rank,
                                      const float* q_norm, int kv_rank, const float* kv_norm, int rot_dim, float eps,
                                      void* q_out, int q_out_stride, const int* positions, const int* token_seq,
                                      const int* seq_seat, const int* block_table, int table_width,
                                      const float* inv_freq, float factor, int rotary_dim, int interleaved,
                                      void* k_cache, int page_size, int num_pages, int write, int tokens, int dtype,
                                      int* error, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (q_rank < 1 || slices < 1 || (rotary_dim & 1) || rotary_dim < 0 || rotary_dim > rot_dim ||
      (write && (kv_rank < 1 || rot_dim < 0 || page_size < 1 || table_width < 1 || !k_cache || !kv_norm)) ||
      (write && rotary_dim > 0 && !inv_freq))
    return DISTIE_ERR_ARG;
  const size_t shared = (size_t)(q_rank + (write ? kv_rank + rot_dim : 0)) * sizeof(float);
  if (shared > 48 * 1024) return DISTIE_ERR_UNSUPPORTED;
  if (dtype == DISTIE_BF16)
    latent_kv_write_kernel<<<tokens, 256, shared, stream>>>(
        proj, row_stride, slices, slice_stride, q_rank, q_norm, kv_rank, kv_norm, rot_dim, eps, (__nv_bfloat16*)q_out,
        q_out_stride, positions, token_seq, seq_seat, block_table, table_width, inv_freq, factor, rotary_dim, interleaved,
        (__nv_bfloat16*)k_cache, page_size, num_pages, write, error);
  else if (dtype == DISTIE_F32)
    latent_kv_write_kernel<<<tokens, 256, shared, stream>>>(
        proj, row_stride, slices, slice_stride, q_rank, q_norm, kv_rank, kv_norm, rot_dim, eps, (float*)q_out,
        q_out_stride, positions, token_seq, seq_seat, block_table, table_width, inv_freq, factor, rotary_dim, interleaved,
        (float*)k_cache, page_size, num_pages, write, error);
  else
    return DISTIE_ERR_UNSUPPORTED;
  DISTIE_LAUNCH_CHECK();
  return 0;
}

extern "C" int distie_latent_q_prepare(const float* q, int row_stride, int slices, long long slice_stride, int tokens,
                                       int heads, int dim, int rot_dim, const int* positions, const float* inv_freq,
                                       float factor, int rotary_dim, int interleaved, void* plain, void* rotated,
                                       int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads < 1 || dim < 1 || rot_dim < 0 || slices < 1 || (rotary_dim & 1) || rotary_dim < 0 || rotary_dim > rot_dim ||
      (rotary_dim > 0 && !inv_freq))
    return DISTIE_ERR_ARG;
  if (dtype == DISTIE_BF16)
    latent_q_prepare_kernel<<<tokens, 256, 0, stream>>>(q, row_stride, slices, slice_stride, tokens, heads, dim, rot_dim,
                                                        positions, inv_freq, factor, rotary_dim, interleaved,
                                                        (__nv_bfloat16*)plain, (__nv_bfloat16*)rotated);
  else if (dtype == DISTIE_F32)
    latent_q_prepare_kernel<<<tokens, 256, 0, stream>>>(q, row_stride, slices, slice_stride, tokens, heads, dim, rot_dim,
                                                        positions, inv_freq, factor, rotary_dim, interleaved,
                                                        (float*)plain, (float*)rotated);
  else
    return DISTIE_ERR_UNSUPPORTED;
  DISTIE_LAUNCH_CHECK();
  return 0;
}

extern "C" long long distie_latent_attention_scratch_floats(int tokens, int heads, int rank, int splits) {
  return splits > 1 ? (long long)splits * tokens * heads * (rank + 2) : 0;
}

extern "C" int distie_latent_attention(const void* folded, const void* rotated, void* out, float* partial, int tokens,
                                       int heads, int rank, int rot, const int* positions, const int* token_seq,
                                       const int* seq_seat, const int* block_table, int table_width,
                                       const void* k_cache, int page_size, int num_pages, float scale,
                                       const float* sink, int splits, int first, int count, int dtype, int* error,
                                       cudaStream_t stream) {
  if (tokens <= 0 || count <= 0) return 0;
  if (first < 0 || first + count > tokens) return DISTIE_ERR_ARG;
  if (heads < 1 || rank < 1 || rot < 0 || page_size < 1 || table_width < 1 || splits < 1 || splits > 64 ||
      (splits > 1 && !partial) || (heads + 1) / 2 > 65535)
    return DISTIE_ERR_ARG;
  if (rank + rot > 1024) return DISTIE_ERR_UNSUPPORTED;
  if (dtype == DISTIE_BF16)
    return latent_attention_any<__nv_bfloat16>(folded, rotated, out, partial, tokens, heads, rank, rot, positions,
                                               token_seq, seq_seat, block_table, table_width, k_cache, page_size,
                                               num_pages, scale, sink, splits, first, count, error, stream);
  if (dtype == DISTIE_F32)
    return latent_attention_any<float>(folded, rotated, out, partial, tokens, heads, rank, rot, positions, token_seq,
                                       seq_seat, block_table, table_width, k_cache, page_size, num_pages, scale, sink,
                                       splits, first, count, error, stream);
  return DISTIE_ERR_UNSUPPORTED;
}

// The splits' partial results [splits, tokens, heads, rank + 2] of tokens first .. first + count - 1 into out
// [heads, tokens, rank]; the head's sink joins the denominator here.
extern "C" int distie_latent_merge(const float* partial, void* out, int tokens, int heads, int rank, int splits,
                                   const float* sink, int first, int count, int dtype, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (!partial || tokens < 1 || heads < 1 || heads > 65535 || rank < 1 || splits < 1 || splits > 64 || first < 0 ||
      first + count > tokens)
    return DISTIE_ERR_ARG;
  if (dtype == DISTIE_BF16)
    latent_merge_kernel<__nv_bfloat16><<<dim3(count, heads, (rank + 127) / 128), 128, 0, stream>>>(partial, (__nv_bfloat16*)out, tokens, heads,
                                                                              rank, splits, sink, first);
  else if (dtype == DISTIE_F32)
    latent_merge_kernel<float><<<dim3(count, heads, (rank + 127) / 128), 128, 0, stream>>>(partial, (float*)out, tokens, heads, rank, splits,
                                                                       sink, first);
  else
    return DISTIE_ERR_UNSUPPORTED;
  DISTIE_LAUNCH_CHECK();
  return 0;
}

extern "C" int distie_latent_gate(const void* y, int tokens, int heads, int vdim, const float* gate, int gate_stride,
                                  int gate_slices, long long gate_slice_stride, void* out, int out_stride, int dtype,
                                  cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads < 1 || vdim < 1 || (gate && gate_slices < 1)) return DISTIE_ERR_ARG;
  if (dtype == DISTIE_BF16)
    latent_gate_kernel<<<tokens, 256, 0, stream>>>((const __nv_bfloat16*)y, tokens, heads, vdim, gate, gate_stride,
                                                   gate_slices, gate_slice_stride, (__nv_bfloat16*)out, out_stride);
  else if (dtype == DISTIE_F32)
    latent_gate_kernel<<<tokens, 256, 0, stream>>>((const float*)y, tokens, heads, vdim, gate, gate_stride, gate_slices,
                                                   gate_slice_stride, (float*)out, out_stride);
  else
    return DISTIE_ERR_UNSUPPORTED;
  DISTIE_LAUNCH_CHECK();
  return 0;
}

extern "C" int distie_glu_act(const float* x, int row_stride, int slices, long long slice_stride, int tokens, int ff,
                              int kind, float limit, const float* row_gate, int gate_stride, int gate_slices,
                              long long gate_slice_stride, void* out, int out_stride, int dtype, cudaStream_t stream) {
  if (tokens <= 0 || ff <= 0) return 0;
  if (slices < 1 || kind < 0 || kind > 1 || (row_gate && gate_slices < 1) || tokens > 65535 * 32) return DISTIE_ERR_ARG;
  const dim3 grid((ff + 255) / 256 > 64 ? 64 : (ff + 255) / 256, tokens);
  if (dtype == DISTIE_BF16)
    glu_act_kernel<<<grid, 256, 0, stream>>>(x, row_stride, slices, slice_stride, tokens, ff, kind, limit, row_gate,
                                             gate_stride, gate_slices, gate_slice_stride, (__nv_bfloat16*)out, out_stride);
  else if (dtype == DISTIE_F32)
    glu_act_kernel<<<grid, 256, 0, stream>>>(x, row_stride, slices, slice_stride, tokens, ff, kind, limit, row_gate,
                                             gate_stride, gate_slices, gate_slice_stride, (float*)out, out_stride);
  else
    return DISTIE_ERR_UNSUPPORTED;
  DISTIE_LAUNCH_CHECK();
  return 0;
}
