// Kernels between a product's float32 accumulators and what reads them: of layers that norm a sublayer's output before
// it joins the residual and whose attention keeps a token's key as its value, and of layers that norm q and k before
// they rotate them:
//
//  * norm_add_rmsnorm: d = sum_j scale_j * term_j (float32); residual += d * rsqrt(mean(d^2) + eps_d) * w_d
//    (or += d when there is no w_d), written back; out = residual * rsqrt(mean(residual^2) + eps) * w, cast
//    once at the store.  One block per row; with a list of rows only those are made and the residual stays.
//  * qk_rope_norm_write: from the float32 projection [q | k] (a matrix or the slices of a split product) plus
//    bias: the key as projected is stored as the value; q and k are rotated over the first `rotary_dim`
//    elements of each head (angles pos * inv_freq in float32), then each head is divided by its root mean
//    square; k goes to its page and q to its buffer.  One block per token, a warp per head.
//  * qkv_norm_write: from the float32 projection [q | k | v] plus bias: every head of q and k divided by its root mean
//    square (and multiplied by a weight shared by the heads), THEN rotated; q times a temperature that grows with the
//    logarithm of the position; k and v (values of a size of their own) to their pages, q to its buffer.
//
// All arithmetic is float32; T is the type of what is stored for the next product or in the cache.
#include "common.cuh"

namespace distie {

constexpr int kResidualTerms = 24;
struct ResidualTerms {
  const float* ptr[kResidualTerms];
  float scale[kResidualTerms];
  int count;
};

template <typename T>
__global__ void __launch_bounds__(512)
norm_add_rmsnorm_kernel(ResidualTerms terms, const float* __restrict__ delta_weight, float delta_eps,
                        float* __restrict__ residual, const float* __restrict__ weight, float eps, T* __restrict__ out,
                        const int* __restrict__ rows_index, int hidden) {
  extern __shared__ __align__(16) float row_s[];  // the summed terms, then the new residual
  __shared__ float scratch[32];
  const int i = blockIdx.x;
  const size_t row = rows_index ? (size_t)rows_index[i] : (size_t)i;
  float* res = residual + row * hidden;
  float ss = 0.f;
  if (terms.count > 0) {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      float d = 0.f;
      for (int j = 0; j < terms.count; ++j) d += terms.scale[j] * terms.ptr[j][row * hidden + c];
      row_s[c] = d;
      ss += d * d;
    }
    float factor = 1.f;
    if (delta_weight) factor = rsqrtf(block_sum(ss, scratch) / (float)hidden + delta_eps);
    ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float r = res[c] + (delta_weight ? row_s[c] * factor * delta_weight[c] : row_s[c]);
      row_s[c] = r;
      if (!rows_index) res[c] = r;
      ss += r * r;
    }
  } else {
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float r = res[c];
      row_s[c] = r;
      ss += r * r;
    }
  }
  if (!out) return;
  const float unit = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps);
  T* out_row = out + (size_t)i * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) out_row[c] = from_float<T>(row_s[c] * unit * weight[c]);
}

// The same with four columns a thread and the row in registers: hidden a multiple of 4 and at most
// 4 * PIECES * blockDim.x, every pointer 16-byte aligned.  All loads of a row's terms are in flight together.
template <typename T, int PIECES>
__global__ void __launch_bounds__(512)
norm_add_rmsnorm_vec_kernel(ResidualTerms terms, const float* __restrict__ delta_weight, float delta_eps,
                            float* __restrict__ residual, const float* __restrict__ weight, float eps,
                            T* __restrict__ out, const int* __restrict__ rows_index, int hidden) {
  __shared__ float scratch[32];
  const int i = blockIdx.x;
  const size_t row = rows_index ? (size_t)rows_index[i] : (size_t)i;
  float* res = residual + row * hidden;
  float4 r[PIECES], d[PIECES];
  float ss = 0.f;
#pragma unroll
  for (int p = 0; p < PIECES; ++p) {
    const int c = (p * blockDim.x + threadIdx.x) * 4;
    d[p] = make_float4(0.f, 0.f, 0.f, 0.f);
    r[p] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < hidden) {
      r[p] = *reinterpret_cast<const float4*>(res + c);
      for (int j = 0; j < terms.count; ++j) {
        const float4 v = *reinterpret_cast<const float4*>(terms.ptr[j] + row * hidden + c);
        const float s = terms.scale[j];
        d[p].x += s * v.x; d[p].y += s * v.y; d[p].z += s * v.z; d[p].w += s * v.w;
      }
      ss += (d[p].x * d[p].x + d[p].y * d[p].y) + (d[p].z * d[p].z + d[p].w * d[p].w);
    }
  }
  if (terms.count > 0) {
    float factor = 1.f;
    if (delta_weight) factor = rsqrtf(block_sum(ss, scratch) / (float)hidden + delta_eps);
#pragma unroll
    for (int p = 0; p < PIECES; ++p) {
      const int c = (p * blockDim.x + threadIdx.x) * 4;
      if (c < hidden) {
        float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
        if (delta_weight) w = *reinterpret_cast<const float4*>(delta_weight + c);
        r[p].x += d[p].x * factor * w.x; r[p].y += d[p].y * factor * w.y;
        r[p].z += d[p].z * factor * w.z; r[p].w += d[p].w * factor * w.w;
        if (!rows_index) *reinterpret_cast<float4*>(res + c) = r[p];
      }
    }
  }
  if (!out) return;
  ss = 0.f;
#pragma unroll
  for (int p = 0; p < PIECES; ++p) ss += (r[p].x * r[p].x + r[p].y * r[p].y) + (r[p].z * r[p].z + r[p].w * r[p].w);
  const float unit = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps);
  T* out_row = out + (size_t)i * hidden;
#pragma unroll
  for (int p = 0; p < PIECES; ++p) {
    const int c = (p * blockDim.x + threadIdx.x) * 4;
    if (c < hidden) {
      const float4 w = *reinterpret_cast<const float4*>(weight + c);
      store4(out_row + c, make_float4(r[p].x * unit * w.x, r[p].y * unit * w.y, r[p].z * unit * w.z, r[p].w * unit * w.w));
    }
  }
}

struct SlicedRows {
  const float* p;
  int stride;
  int splits;
  long long split_stride;
  __device__ __forceinline__ float at(size_t row, int col) const {
    const float* q = p + row * stride + col;
    float v = q[0];
    for (int s = 1; s < splits; ++s) v += q[(size_t)s * split_stride];
    return v;
  }
};

constexpr int kRopeWarps = 8;

// A block per token, a warp per head (in turns): the head waits in the warp's own piece of shared memory between
// the load, the rotation of its pairs and the stores.
template <typename T>
__global__ void __launch_bounds__(kRopeWarps * 32)
qk_rope_norm_write_kernel(SlicedRows qk, const float* __restrict__ bias, T* __restrict__ q_out, int q_out_stride,
                          const int* __restrict__ positions, const int* __restrict__ token_seq,
                          const int* __restrict__ seq_seat, const int* __restrict__ block_table, int table_width,
                          const float* __restrict__ inv_freq, float factor, T* __restrict__ k_cache,
                          T* __restrict__ v_cache, int num_heads, int num_kv_heads, int head_dim, int rotary_dim,
                          int interleaved, int page_size, int num_pages, int write, int normed, float norm_eps,
                          int* __restrict__ error) {
  extern __shared__ __align__(16) float heads_s[];  // kRopeWarps pieces of head_dim floats, then cos and sin of the token
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* head_s = heads_s + (size_t)warp * head_dim;
  const int pos = positions[t];
  const int half = rotary_dim / 2;
  float* cos_s = heads_s + (size_t)kRopeWarps * head_dim;  // the token's angles serve all of its heads
  float* sin_s = cos_s + half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    sincosf((float)pos * inv_freq[i], &sn, &cs);
    cos_s[i] = cs * factor;
    sin_s[i] = sn * factor;
  }
  __syncthreads();
  int page = -1;
  if (write) {
    const int seat = seq_seat[token_seq[t]];
    const int column = pos / page_size;
    page = column < table_width ? block_table[(size_t)seat * table_width + column] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0 && error) atomicExch(error, 2);
      page = -1;
    }
  }
  const int heads_here = num_heads + (write ? num_kv_heads : 0);
  for (int head = blockIdx.y * kRopeWarps + warp; head < heads_here; head += gridDim.y * kRopeWarps) {
    const bool is_key = head >= num_heads;
    const int column0 = head * head_dim;
    for (int e = lane; e < head_dim; e += 32) head_s[e] = qk.at(t, column0 + e) + (bias ? bias[column0 + e] : 0.f);
    __syncwarp();
    size_t cache_row = 0;
    if (is_key && page >= 0) {
      cache_row = (((size_t)page * num_kv_heads + (head - num_heads)) * page_size + pos % page_size) * head_dim;
      for (int e = lane; e < head_dim; e += 32) v_cache[cache_row + e] = from_float<T>(head_s[e]);
    }
    float ss = 0.f;
    for (int i = lane; i < half; i += 32) {  // every pair is read and written by one lane
      const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
      const float sn = sin_s[i], cs = cos_s[i];
      const float u = head_s[a], v = head_s[b];
      const float ru = u * cs - v * sn, rv = v * cs + u * sn;
      head_s[a] = ru;
      head_s[b] = rv;
      ss += ru * ru + rv * rv;
    }
    for (int e = rotary_dim + lane; e < head_dim; e += 32) ss += head_s[e] * head_s[e];
    __syncwarp();
    const float unit = normed ? rsqrtf(warp_sum(ss) / (float)head_dim + norm_eps) : 1.f;
    if (!is_key || page >= 0) {
      T* dst = is_key ? k_cache + cache_row : q_out + (size_t)t * q_out_stride + column0;
      for (int e = lane; e < head_dim; e += 32) dst[e] = from_float<T>(head_s[e] * unit);
    }
    __syncwarp();  // before the next head overwrites the piece
  }
}

// From the float32 projection [q | k | v] (a matrix or the slices of a split product; columns behind these are not
// read) to q in its buffer and k and v in their pages.  A block per token, a warp per head in turns.  For q and k
// heads, in this order: bias; with `normed` the division by the head's root mean square (eps inside the root) and,
// where a weight is given, the multiplication by it (head_dim floats shared by the heads); the rotation of the
// first rotary_dim elements; for q the temperature 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1)
// (temp_every > 0; the quotient of two floats is exact wherever it is whole, for positions below 2^24).  v heads (value_dim elements, which may differ from head_dim) get their bias and are stored.
template <typename T>
__global__ void __launch_bounds__(kRopeWarps * 32)
qkv_norm_write_kernel(SlicedRows qkv, const float* __restrict__ bias, T* __restrict__ q_out, int q_out_stride,
                      const int* __restrict__ positions, const int* __restrict__ token_seq,
                      const int* __restrict__ seq_seat, const int* __restrict__ block_table, int table_width,
                      const float* __restrict__ inv_freq, float factor, T* __restrict__ k_cache, T* __restrict__ v_cache,
                      int num_heads, int num_kv_heads, int head_dim, int value_dim, int rotary_dim, int interleaved,
                      int page_size, int num_pages, int write, int normed, float norm_eps,
                      const float* __restrict__ q_weight, const float* __restrict__ k_weight, float temp_coef,
                      float temp_every, int* __restrict__ error) {
  extern __shared__ __align__(16) float heads_s[];  // kRopeWarps pieces of `piece` floats, then cos and sin of the token
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int piece = max(head_dim, value_dim);
  float* head_s = heads_s + (size_t)warp * piece;
  const int pos = positions[t];
  const int half = rotary_dim / 2;
  float* cos_s = heads_s + (size_t)kRopeWarps * piece;  // the token's angles serve all of its heads
  float* sin_s = cos_s + half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    sincosf((float)pos * inv_freq[i], &sn, &cs);
    cos_s[i] = cs * factor;
    sin_s[i] = sn * factor;
  }
  __syncthreads();
  int page = -1;
  if (write) {
    const int seat = seq_seat[token_seq[t]];
    const int column = pos / page_size;
    page = column < table_width ? block_table[(size_t)seat * table_width + column] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0 && error) atomicExch(error, 2);
      page = -1;
    }
  }
  const float temperature = temp_every > 0.f ? 1.f + temp_coef * logf(floorf((float)(pos + 1) / temp_every) + 1.f) : 1.f;
  const int k_column0 = num_heads * head_dim, v_column0 = (num_heads + num_kv_heads) * head_dim;
  const int heads_here = num_heads + (write ? 2 * num_kv_heads : 0);
  for (int head = blockIdx.y * kRopeWarps + warp; head < heads_here; head += gridDim.y * kRopeWarps) {
    const bool is_query = head < num_heads, is_value = head >= num_heads + num_kv_heads;
    if (is_value) {
      if (page < 0) continue;
      const int kv_head = head - num_heads - num_kv_heads;
      const int column0 = v_column0 + kv_head * value_dim;
      T* dst = v_cache + (((size_t)page * num_kv_heads + kv_head) * page_size + pos % page_size) * value_dim;
      for (int e = lane; e < value_dim; e += 32)
        dst[e] = from_float<T>(qkv.at(t, column0 + e) + (bias ? bias[column0 + e] : 0.f));
      continue;
    }
    const int column0 = is_query ? head * head_dim : k_column0 + (head - num_heads) * head_dim;
    float ss = 0.f;
    for (int e = lane; e < head_dim; e += 32) {
      const float value = qkv.at(t, column0 + e) + (bias ? bias[column0 + e] : 0.f);
      head_s[e] = value;
      ss += value * value;
    }
    const float unit = normed ? rsqrtf(warp_sum(ss) / (float)head_dim + norm_eps) : 1.f;
    const float* weight = is_query ? q_weight : k_weight;
    __syncwarp();
    if (normed)
      for (int e = lane; e < head_dim; e += 32) head_s[e] = head_s[e] * unit * (weight ? weight[e] : 1.f);
    __syncwarp();
    for (int i = lane; i < half; i += 32) {  // every pair is read and written by one lane
      const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
      const float sn = sin_s[i], cs = cos_s[i];
      const float u = head_s[a], v = head_s[b];
      head_s[a] = u * cs - v * sn;
      head_s[b] = v * cs + u * sn;
    }
    __syncwarp();
    if (is_query || page >= 0) {
      T* dst = is_query ? q_out + (size_t)t * q_out_stride + column0
                        : k_cache + (((size_t)page * num_kv_heads + (head - num_heads)) * page_size + pos % page_size) * head_dim;
      const float times = is_query ? temperature : 1.f;
      for (int e = lane; e < head_dim; e += 32) dst[e] = from_float<T>(head_s[e] * times);
    }
    __syncwarp();  // before the next head overwrites the piece
  }
}

}  // namespace distie

using namespace distie;

// terms: `num_terms` float32 matrices [rows of the residual, hidden] with a scale each (none: nothing is added).
// delta_weight null: the sum joins the residual as it is.  out null: only the residual is moved on.
extern "C" int distie_norm_add_rmsnorm(const float* const* term_ptrs, const float* term_scales, int num_terms,
                                       const float* delta_weight, float delta_eps, float* residual, const float* weight,
                                       float eps, void* out, const int* rows_index, int rows, int hidden, int dtype,
                                       cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden < 1 || num_terms < 0 || num_terms > kResidualTerms || residual == nullptr || (out && !weight))
    return DISTIE_ERR_ARG;
  ResidualTerms terms;
  terms.count = num_terms;
  for (int j = 0; j < num_terms; ++j) { terms.ptr[j] = term_ptrs[j]; terms.scale[j] = term_scales[j]; }
  uintptr_t low_bits = (uintptr_t)residual | (uintptr_t)weight | (uintptr_t)delta_weight | (uintptr_t)out;
  for (int j = 0; j < num_terms; ++j) low_bits |= (uintptr_t)term_ptrs[j];
  if (hidden % 4 == 0 && hidden <= 4 * 4 * 512 && (low_bits & 15) == 0 && (dtype == DISTIE_BF16 || dtype == DISTIE_F32)) {
    const int quads = hidden / 4;
    int vec_threads = 32;
    while (vec_threads < 512 && vec_threads < quads) vec_threads *= 2;
    const int pieces = (quads + vec_threads - 1) / vec_threads;
#define DISTIE_NORM_VEC(T, PIECESV)                                                                                       \
  norm_add_rmsnorm_vec_kernel<T, PIECESV><<<rows, vec_threads, 0, stream>>>(terms, delta_weight, delta_eps, residual, weight, \
                                                                            eps, (T*)out, rows_index, hidden)
    if (dtype == DISTIE_BF16) {
      if (pieces == 1) DISTIE_NORM_VEC(__nv_bfloat16, 1); else if (pieces == 2) DISTIE_NORM_VEC(__nv_bfloat16, 2);
      else DISTIE_NORM_VEC(__nv_bfloat16, 4);
    } else {
      if (pieces == 1) DISTIE_NORM_VEC(float, 1); else if (pieces == 2) DISTIE_NORM_VEC(float, 2);
      else DISTIE_NORM_VEC(float, 4);
    }
#undef DISTIE_NORM_VEC
    DISTIE_LAUNCH_CHECK();
    return 0;
  }
  const int threads = hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128);
  const size_t shared = (size_t)hidden * sizeof(float);
  if (shared > 200 * 1024) return DISTIE_ERR_UNSUPPORTED;
  if (dtype == DISTIE_BF16) {
    if (shared > 48 * 1024)
      cudaFuncSetAttribute(norm_add_rmsnorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    norm_add_rmsnorm_kernel<<<rows, threads, shared, stream>>>(terms, delta_weight, delta_eps, residual, weight, eps,
                                                               (__nv_bfloat16*)out, rows_index, hidden);
  } else if (dtype == DISTIE_F32) {
    if (shared > 48 * 1024)
      cudaFuncSetAttribute(norm_add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    norm_add_rmsnorm_kernel<<<rows, threads, shared, stream>>>(terms, delta_weight, delta_eps, residual, weight, eps,
                                                               (float*)out, rows_index, hidden);
  } else {
    return DISTIE_ERR_UNSUPPORTED;
  }
  DISTIE_LAUNCH_CHECK();
  return 0;
}

// qk: float32 [tokens, (heads + kv_heads) * head_dim] with row stride `qk_stride`, or `splits` such matrices
// `split_stride` floats apart whose sum it is.  write == 0: only q is made.  normed == 0: no division.
extern "C" int distie_qk_rope_norm_write(const float* qk, int qk_stride, int splits, long long split_stride,
                                         const float* bias, void* q_out, int q_out_stride, const int* positions,
                                         const int* token_seq, const int* seq_seat, const int* block_table,
                                         int table_width, const float* inv_freq, float factor, void* k_cache,
                                         void* v_cache, int tokens, int num_heads, int num_kv_heads, int head_dim,
                                         int rotary_dim, int interleaved, int page_size, int num_pages, int write,
                                         int normed, float norm_eps, int dtype, int* error, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (num_heads < 1 || num_kv_heads < 1 || head_dim < 1 || head_dim > 1024 || rotary_dim < 0 || rotary_dim > head_dim ||
      (rotary_dim & 1) || (rotary_dim > 0 && inv_freq == nullptr) || splits < 1 || page_size < 1 ||
      num_heads + num_kv_heads > 65535 || (write && (k_cache == nullptr || v_cache == nullptr)))
    return DISTIE_ERR_ARG;
  // Few tokens: the heads of a token spread over several blocks, so that the step fills more of the machine.
  const dim3 grid(tokens, tokens < 512 ? (num_heads + num_kv_heads + kRopeWarps - 1) / kRopeWarps : 1);
  const int threads = kRopeWarps * 32;
  const size_t shared = ((size_t)kRopeWarps * head_dim + rotary_dim) * sizeof(float);
  const SlicedRows rows{qk, qk_stride, splits, split_stride};
  if (dtype == DISTIE_BF16)
    qk_rope_norm_write_kernel<<<grid, threads, shared, stream>>>(
        rows, bias, (__nv_bfloat16*)q_out, q_out_stride, positions, token_seq, seq_seat, block_table, table_width,
        inv_freq, factor, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, num_heads, num_kv_heads, head_dim,
        rotary_dim, interleaved, page_size, num_pages, write, normed, norm_eps, error);
  else if (dtype == DISTIE_F32)
    qk_rope_norm_write_kernel<<<grid, threads, shared, stream>>>(
        rows, bias, (float*)q_out, q_out_stride, positions, token_seq, seq_seat, block_table, table_width, inv_freq,
        factor, (float*)k_cache, (float*)v_cache, num_heads, num_kv_heads, head_dim, rotary_dim, interleaved, page_size,
        num_pages, write, normed, norm_eps, error);
  else
    return DISTIE_ERR_UNSUPPORTED;
  DISTIE_LAUNCH_CHECK();
  return 0;
}

// qkv: float32 [tokens, heads * head_dim + kv_heads * (head_dim + value_dim) (+ columns that are not read)] with row
// stride `qkv_stride`, or `splits` such matrices `split_stride` floats apart whose sum it is.  write == 0: only q is
// made.  normed == 0: no norm; q_weight / k_weight null: no weight.  temp_every <= 0: no temperature.
extern "C" int distie_qkv_norm_write(const float* qkv, int qkv_stride, int splits, long long split_stride, const float* bias,
                                     void* q_out, int q_out_stride, const int* positions, const int* token_seq,
                                     const int* seq_seat, const int* block_table, int table_width, const float* inv_freq,
                                     float factor, void* k_cache, void* v_cache, int tokens, int num_heads, int num_kv_heads,
                                     int head_dim, int value_dim, int rotary_dim, int interleaved, int page_size,
                                     int num_pages, int write, int normed, float norm_eps, const float* q_weight,
                                     const float* k_weight, float temp_coef, float temp_every, int dtype, int* error,
                                     cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (num_heads < 1 || num_kv_heads < 1 || head_dim < 1 || head_dim > 1024 || value_dim < 1 || value_dim > 1024 ||
      rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1) || (rotary_dim > 0 && inv_freq == nullptr) || splits < 1 ||
      page_size < 1 || num_heads + 2 * num_kv_heads > 65535 || (write && (k_cache == nullptr || v_cache == nullptr)))
    return DISTIE_ERR_ARG;
  const int heads_all = num_heads + 2 * num_kv_heads;
  // Few tokens: the heads of a token spread over several blocks, so that the step fills more of the machine.
  const dim3 grid(tokens, tokens < 512 ? (heads_all + kRopeWarps - 1) / kRopeWarps : 1);
  const int threads = kRopeWarps * 32;
  const int piece = head_dim > value_dim ? head_dim : value_dim;
  const size_t shared = ((size_t)kRopeWarps * piece + rotary_dim) * sizeof(float);
  const SlicedRows rows{qkv, qkv_stride, splits, split_stride};
  if (dtype == DISTIE_BF16)
    qkv_norm_write_kernel<<<grid, threads, shared, stream>>>(
        rows, bias, (__nv_bfloat16*)q_out, q_out_stride, positions, token_seq, seq_seat, block_table, table_width,
        inv_freq, factor, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, num_heads, num_kv_heads, head_dim, value_dim,
        rotary_dim, interleaved, page_size, num_pages, write, normed, norm_eps, q_weight, k_weight, temp_coef, temp_every,
        error);
  else if (dtype == DISTIE_F32)
    qkv_norm_write_kernel<<<grid, threads, shared, stream>>>(
        rows, bias, (float*)q_out, q_out_stride, positions, token_seq, seq_seat, block_table, table_width, inv_freq,
        factor, (float*)k_cache, (float*)v_cache, num_heads, num_kv_heads, head_dim, value_dim, rotary_dim, interleaved,
        page_size, num_pages, write, normed, norm_eps, q_weight, k_weight, temp_coef, temp_every, error);
  else
    return DISTIE_ERR_UNSUPPORTED;
  DISTIE_LAUNCH_CHECK();
  return 0;
}
