// Kernels of layers that keep a state per request instead of (or beside) a cache of keys:
// the residual sum + LayerNorm over a weighted sum of terms, the paged key/value write of
// layers that rotate nothing, the sigmoid gate per head, the short causal convolution,
// the linear recurrence (gated delta rule, state-space duality, and plainly gated with an optional
// normaliser column), the gated RMS norm, and what a memory with exponential gates needs around its
// recurrence: an activation over a split product, the gates' scan under a running maximum, the stabilised read-out.
//
// Conventions.  Everything between a layer's projections and its output projection is
// float32 here: inputs are float32 matrices with a row stride (views into a projection's
// output), state is float32, and only what feeds the next product is stored as T.
// A step's tokens are ordered by request: `token_seq[t]` (the batch row of token t) never
// decreases, so the tokens of row b are the range `seq_bounds[b] .. seq_bounds[b + 1] - 1`
// (made once per step on the device, with `token_first[t]`, the first token of t's request in
// this step); `seq_seat[b]` is the request's slot in every state tensor.  Nothing here reads
// host-side batch data, so captured decode steps replay these kernels for whatever seats they
// are given.
#include "common.cuh"

namespace distie {

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return log1pf(expf(-fabsf(z))) + fmaxf(z, 0.f); }
__device__ __forceinline__ float gate_f(int sigmoid, float z) { return sigmoid ? sigmoid_f(z) : silu_f(z); }

// A float32 matrix that may still be the slices of a split product: `splits` matrices `split_stride` floats apart
// whose sum it is (splits == 1: the matrix itself).  Loads add the slices up, in their order.
struct Sliced {
  const float* p;
  int stride;  // of a row
  int splits;
  long long split_stride;
  const float* bias = nullptr;  // per column, added to the sum of the slices (a projection's bias); null: none
  __device__ __forceinline__ float at(size_t row, int col) const {
    const float* q = p + row * stride + col;
    float v = q[0];
    for (int s = 1; s < splits; ++s) v += q[(size_t)s * split_stride];
    return bias ? v + bias[col] : v;
  }
  __device__ __forceinline__ float4 at4(size_t row, int col) const {
    const float* q = p + row * stride + col;
    float4 v = *reinterpret_cast<const float4*>(q);
    for (int s = 1; s < splits; ++s) {
      const float4 w = *reinterpret_cast<const float4*>(q + (size_t)s * split_stride);
      v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
    }
    if (bias) {
      const float4 b = *reinterpret_cast<const float4*>(bias + col);
      v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
    }
    return v;
  }
};

// ---------------------------------------------------------------------------
// residual += sum_j scale_j * term_j (float32, written back), then
//   out = (residual - mean) / sqrt(var + eps) * weight + bias,  var = mean((residual - mean)^2).
// With `rows_index` only the listed rows are normalised and the residual stays as it is.
// One block per output row; the summed row waits in shared memory between the passes.
// ---------------------------------------------------------------------------
constexpr int kMaxTerms = 24;
struct SumTerms {
  const float* ptr[kMaxTerms];
  float scale[kMaxTerms];
  int count;
};

template <typename T>
__global__ void add_layernorm_kernel(SumTerms terms, float* __restrict__ residual, const float* __restrict__ weight,
                                     const float* __restrict__ bias, T* __restrict__ out,
                                     const int* __restrict__ rows_index, int hidden, float eps) {
  extern __shared__ float row_cache[];
  __shared__ float scratch[32];
  const int out_row = blockIdx.x;
  const int row = rows_index ? rows_index[out_row] : out_row;
  float* res = residual + (size_t)row * hidden;
  const bool write_back = terms.count > 0 && rows_index == nullptr;
  float sum = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float add = 0.f;
    for (int j = 0; j < terms.count; ++j) add += terms.scale[j] * terms.ptr[j][(size_t)row * hidden + i];
    const float v = res[i] + add;
    if (write_back) res[i] = v;
    row_cache[i] = v;
    sum += v;
  }
  const float mean = block_sum(sum, scratch) / (float)hidden;
  float sq = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float d = row_cache[i] - mean;
    sq += d * d;
  }
  const float var = block_sum(sq, scratch) / (float)hidden;
  const float inv = 1.f / sqrtf(var + eps);
  T* dst = out + (size_t)out_row * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    dst[i] = from_float<T>((row_cache[i] - mean) * inv * weight[i] + bias[i]);
}

// The same with four columns per thread and the row in registers: hidden a multiple of 4, at most
// 4 * kNormPieces * blockDim.x, every pointer 16-byte aligned.
constexpr int kNormPieces = 8;
template <typename T>
__global__ void __launch_bounds__(512) add_layernorm_vec_kernel(SumTerms terms, float* __restrict__ residual,
                                                                const float* __restrict__ weight,
                                                                const float* __restrict__ bias, T* __restrict__ out,
                                                                const int* __restrict__ rows_index, int hidden, float eps) {
  __shared__ float scratch[32];
  const int out_row = blockIdx.x;
  const int row = rows_index ? rows_index[out_row] : out_row;
  float* res = residual + (size_t)row * hidden;
  const bool write_back = terms.count > 0 && rows_index == nullptr;
  float4 v[kNormPieces];
  float sum = 0.f;
#pragma unroll
  for (int p = 0; p < kNormPieces; ++p) {
    const int i = (p * blockDim.x + threadIdx.x) * 4;
    v[p] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < hidden) {
      float4 add = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j < terms.count; ++j) {
        const float4 d = *reinterpret_cast<const float4*>(terms.ptr[j] + (size_t)row * hidden + i);
        const float sc = terms.scale[j];
        add.x += sc * d.x; add.y += sc * d.y; add.z += sc * d.z; add.w += sc * d.w;
      }
      const float4 r = *reinterpret_cast<const float4*>(res + i);
      v[p] = make_float4(r.x + add.x, r.y + add.y, r.z + add.z, r.w + add.w);
      if (write_back) *reinterpret_cast<float4*>(res + i) = v[p];
      sum += (v[p].x + v[p].y) + (v[p].z + v[p].w);
    }
  }
  const float mean = block_sum(sum, scratch) / (float)hidden;
  float sq = 0.f;
#pragma unroll
  for (int p = 0; p < kNormPieces; ++p) {
    const int i = (p * blockDim.x + threadIdx.x) * 4;
    if (i < hidden) {
      const float a = v[p].x - mean, b = v[p].y - mean, c = v[p].z - mean, d = v[p].w - mean;
      sq += (a * a + b * b) + (c * c + d * d);
    }
  }
  const float inv = 1.f / sqrtf(block_sum(sq, scratch) / (float)hidden + eps);
  T* dst = out + (size_t)out_row * hidden;
#pragma unroll
  for (int p = 0; p < kNormPieces; ++p) {
    const int i = (p * blockDim.x + threadIdx.x) * 4;
    if (i < hidden) {
      const float4 w = *reinterpret_cast<const float4*>(weight + i), b = *reinterpret_cast<const float4*>(bias + i);
      store4(dst + i, make_float4((v[p].x - mean) * inv * w.x + b.x, (v[p].y - mean) * inv * w.y + b.y,
                                  (v[p].z - mean) * inv * w.z + b.z, (v[p].w - mean) * inv * w.w + b.w));
    }
  }
}

// ---------------------------------------------------------------------------
// Keys and values of the new tokens into their pages, unrotated; a value may have another size
// than a key.  One block per token.
// ---------------------------------------------------------------------------
template <typename TIn, typename T>
__global__ void kv_write_kernel(const TIn* __restrict__ k, int k_stride, const TIn* __restrict__ v, int v_stride,
                                const int* __restrict__ positions, const int* __restrict__ token_seq,
                                const int* __restrict__ seq_seat, const int* __restrict__ block_table, int table_width,
                                T* __restrict__ k_cache, T* __restrict__ v_cache, int num_kv_heads, int head_dim,
                                int value_dim, int page_size, int num_pages, int* __restrict__ error) {
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int seat = seq_seat[token_seq[t]];
  const int column = pos / page_size;
  const int page = (pos >= 0 && column < table_width) ? block_table[(size_t)seat * table_width + column] : -1;
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0 && error) atomicExch(error, 2);
    return;
  }
  const int slot = pos % page_size;
  for (int e = threadIdx.x; e < num_kv_heads * head_dim; e += blockDim.x) {
    const int h = e / head_dim, d = e % head_dim;
    k_cache[(((size_t)page * num_kv_heads + h) * page_size + slot) * head_dim + d] =
        from_float<T>(to_float(k[(size_t)t * k_stride + e]));
  }
  for (int e = threadIdx.x; e < num_kv_heads * value_dim; e += blockDim.x) {
    const int h = e / value_dim, d = e % value_dim;
    v_cache[(((size_t)page * num_kv_heads + h) * page_size + slot) * value_dim + d] =
        from_float<T>(to_float(v[(size_t)t * v_stride + e]));
  }
}

// x[t, h, :] *= sigmoid(logits[t, h]).
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, Sliced logits, int num_heads, int dim, size_t total) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / ((size_t)num_heads * dim);
    const int h = (int)((i / dim) % num_heads);
    x[i] = from_float<T>(to_float(x[i]) * sigmoid_f(logits.at(t, h)));
  }
}

// Four elements a thread: dim a multiple of 4, x aligned to four elements.
template <typename T>
__global__ void head_gate_vec_kernel(T* __restrict__ x, Sliced logits, int num_heads, int dim, size_t quads) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += (size_t)gridDim.x * blockDim.x) {
    const size_t e = i * 4;
    const size_t t = e / ((size_t)num_heads * dim);
    const int h = (int)((e / dim) % num_heads);
    const float s = sigmoid_f(logits.at(t, h));
    float4 v = load4(x + e);
    v.x *= s; v.y *= s; v.z *= s; v.w *= s;
    store4(x + e, v);
  }
}

// The gate element by element (a "head" of one element each): four columns a thread, their four logits in one load.
template <typename T>
__global__ void element_gate_vec_kernel(T* __restrict__ x, Sliced logits, int columns, size_t quads) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += (size_t)gridDim.x * blockDim.x) {
    const size_t e = i * 4;
    const size_t t = e / (size_t)columns;
    const float4 g = logits.at4(t, (int)(e % (size_t)columns));
    float4 v = load4(x + e);
    v.x *= sigmoid_f(g.x); v.y *= sigmoid_f(g.y); v.z *= sigmoid_f(g.z); v.w *= sigmoid_f(g.w);
    store4(x + e, v);
  }
}

// ---------------------------------------------------------------------------
// Short causal convolution over time, per channel and per request.
//   y[t, c] = act(bias[c] + sum_j w[c, taps-1-j] * x_in(t - j)),  j = 0 .. taps-1
// where x_in reaches back into the request's state (its last taps-1 inputs, oldest first) for
// tokens before this step's portion.  A second kernel then moves the state on; in a step in which
// every request brings one token (`single` set) the thread that read a channel's state is the only
// one that does, and moves it on itself.
// ---------------------------------------------------------------------------
constexpr int kMaxTaps = 16;

__global__ void short_conv_kernel(Sliced x, const float* __restrict__ weight,
                                  const float* __restrict__ bias, float* __restrict__ state,
                                  const int* __restrict__ token_seq, const int* __restrict__ token_first,
                                  const int* __restrict__ seq_seat, int channels, int taps, int silu, int single,
                                  float* __restrict__ out) {
  const int t = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int first = single ? t : token_first[t];
  float* held = state ? state + (size_t)seq_seat[token_seq[t]] * (taps - 1) * channels : nullptr;
  float acc = bias ? bias[c] : 0.f;
  float carry = 0.f;  // single: what the slot of the input j places back held before this step (j >= 1)
  for (int j = 0; j < taps; ++j) {
    const int at = t - j;
    float v;
    if (at >= first) v = x.at(at, c);
    else if (single) v = carry;
    else v = held ? held[(size_t)(at - first + taps - 1) * channels + c] : 0.f;
    acc += weight[(size_t)c * taps + (taps - 1 - j)] * v;
    if (single && held && j < taps - 1) {
      // the input j places back moves to slot taps-2-j (the current one to the newest slot); what that slot held
      // is the input j+1 places back, used by the next round
      float* slot = held + (size_t)(taps - 2 - j) * channels + c;
      carry = *slot;
      *slot = v;
    }
  }
  out[(size_t)t * channels + c] = silu ? silu_f(acc) : acc;
}

// A step in which every request brings one token: the thread reads its channel's taps-1 held inputs at once,
// and writes them back one slot down with the current input behind them.
__global__ void short_conv_single_kernel(Sliced x, const float* __restrict__ weight, const float* __restrict__ bias,
                                         float* __restrict__ state, const int* __restrict__ token_seq,
                                         const int* __restrict__ seq_seat, int channels, int taps, int silu,
                                         float* __restrict__ out) {
  const int t = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  float* held = state + (size_t)seq_seat[token_seq[t]] * (taps - 1) * channels + c;
  float old[kMaxTaps - 1];
#pragma unroll
  for (int i = 0; i < kMaxTaps - 1; ++i) old[i] = i < taps - 1 ? held[(size_t)i * channels] : 0.f;
  const float now = x.at(t, c);
  float acc = (bias ? bias[c] : 0.f) + weight[(size_t)c * taps + taps - 1] * now;
#pragma unroll
  for (int i = 0; i < kMaxTaps - 1; ++i)
    if (i < taps - 1) acc += weight[(size_t)c * taps + i] * old[i];  // slot i holds the input taps-1-i places back
#pragma unroll
  for (int i = 0; i < kMaxTaps - 1; ++i)
    if (i < taps - 1) held[(size_t)i * channels] = i + 1 < taps - 1 ? old[i + 1] : now;
  out[(size_t)t * channels + c] = silu ? silu_f(acc) : acc;
}

// Where each request's tokens lie in the step: seq_bounds[b] .. seq_bounds[b + 1] - 1 are the tokens of batch row b
// and token_first[t] is the first token of t's row.  One block.
__global__ void seq_index_kernel(const int* __restrict__ token_seq, int tokens, int num_seqs, int* __restrict__ token_first,
                                 int* __restrict__ seq_bounds) {
  for (int b = threadIdx.x; b <= num_seqs; b += blockDim.x) seq_bounds[b] = tokens;
  __syncthreads();
  for (int t = threadIdx.x; t < tokens; t += blockDim.x) {
    const int row = token_seq[t];
    if (row >= 0 && row < num_seqs && (t == 0 || token_seq[t - 1] != row)) seq_bounds[row] = t;
  }
  __syncthreads();
  for (int t = threadIdx.x; t < tokens; t += blockDim.x) {
    const int row = token_seq[t];
    token_first[t] = (row >= 0 && row < num_seqs) ? seq_bounds[row] : t;
  }
}

// Four channels a thread for steps that bring portions of prompts: channels and x_stride multiples of 4, x, state
// and out aligned to 16 bytes.  TAPS > 0: the number of taps at compile time.
template <int TAPS>
__global__ void short_conv_vec_kernel(Sliced x, const float* __restrict__ weight,
                                      const float* __restrict__ bias, const float* __restrict__ state,
                                      const int* __restrict__ token_seq, const int* __restrict__ token_first,
                                      const int* __restrict__ seq_seat, int channels, int taps_runtime, int silu,
                                      float* __restrict__ out) {
  const int taps = TAPS > 0 ? TAPS : taps_runtime;
  const int t = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c >= channels) return;
  const int first = token_first[t];
  const float* held = state ? state + (size_t)seq_seat[token_seq[t]] * (taps - 1) * channels : nullptr;
  float4 acc = bias ? *reinterpret_cast<const float4*>(bias + c) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int j = 0; j < (TAPS > 0 ? TAPS : kMaxTaps); ++j) {
    if (j >= taps) break;
    const int at = t - j;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (at >= first) v = x.at4(at, c);
    else if (held) v = *reinterpret_cast<const float4*>(held + (size_t)(at - first + taps - 1) * channels + c);
    const int tap = taps - 1 - j;
    acc.x += weight[(size_t)c * taps + tap] * v.x;
    acc.y += weight[(size_t)(c + 1) * taps + tap] * v.y;
    acc.z += weight[(size_t)(c + 2) * taps + tap] * v.z;
    acc.w += weight[(size_t)(c + 3) * taps + tap] * v.w;
  }
  if (silu) acc = make_float4(silu_f(acc.x), silu_f(acc.y), silu_f(acc.z), silu_f(acc.w));
  *reinterpret_cast<float4*>(out + (size_t)t * channels + c) = acc;
}

// Four taps, four channels and a run of eight tokens a thread, the window of held inputs in registers: every input
// is loaded once instead of once per tap, and a block lives eight times as long.  A run that crosses from one
// request into the next falls back to the token-by-token form.
constexpr int kConvRun = 8;
__global__ void short_conv_run4_kernel(Sliced x, const float* __restrict__ weight, const float* __restrict__ bias,
                                       const float* __restrict__ state, const int* __restrict__ token_seq,
                                       const int* __restrict__ token_first, const int* __restrict__ seq_seat, int tokens,
                                       int channels, int silu, float* __restrict__ out) {
  const int t0 = blockIdx.y * kConvRun;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c >= channels) return;
  const int n = min(kConvRun, tokens - t0);
  float4 w[4];  // w[j]: tap j of the four channels (tap 3 multiplies the current token)
  {
    const float4 a = *reinterpret_cast<const float4*>(weight + (size_t)c * 4), b = *reinterpret_cast<const float4*>(weight + (size_t)(c + 1) * 4);
    const float4 d = *reinterpret_cast<const float4*>(weight + (size_t)(c + 2) * 4), e = *reinterpret_cast<const float4*>(weight + (size_t)(c + 3) * 4);
    w[0] = make_float4(a.x, b.x, d.x, e.x); w[1] = make_float4(a.y, b.y, d.y, e.y);
    w[2] = make_float4(a.z, b.z, d.z, e.z); w[3] = make_float4(a.w, b.w, d.w, e.w);
  }
  const float4 base = bias ? *reinterpret_cast<const float4*>(bias + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  auto input = [&](int at, int first, const float* held) {  // the input at token index `at` of a request that starts at `first`
    if (at >= first) return x.at4(at, c);
    if (held) return *reinterpret_cast<const float4*>(held + (size_t)(at - first + 3) * channels + c);
    return make_float4(0.f, 0.f, 0.f, 0.f);
  };
  auto finish = [&](int t, float4 acc) {
    if (silu) acc = make_float4(silu_f(acc.x), silu_f(acc.y), silu_f(acc.z), silu_f(acc.w));
    *reinterpret_cast<float4*>(out + (size_t)t * channels + c) = acc;
  };
  auto mac = [](float4 acc, float4 wj, float4 v) {
    return make_float4(acc.x + wj.x * v.x, acc.y + wj.y * v.y, acc.z + wj.z * v.z, acc.w + wj.w * v.w);
  };
  const int row0 = token_seq[t0];
  if (row0 == token_seq[t0 + n - 1]) {
    const int first = token_first[t0];
    const float* held = state ? state + (size_t)seq_seat[row0] * 3 * channels : nullptr;
    float4 back3 = input(t0 - 3, first, held), back2 = input(t0 - 2, first, held), back1 = input(t0 - 1, first, held);
#pragma unroll
    for (int k = 0; k < kConvRun; ++k) {
      if (k < n) {
        const float4 now = x.at4(t0 + k, c);
        finish(t0 + k, mac(mac(mac(mac(base, w[0], back3), w[1], back2), w[2], back1), w[3], now));
        back3 = back2; back2 = back1; back1 = now;
      }
    }
  } else {
    for (int k = 0; k < n; ++k) {
      const int t = t0 + k, first = token_first[t];
      const float* held = state ? state + (size_t)seq_seat[token_seq[t]] * 3 * channels : nullptr;
      finish(t, mac(mac(mac(mac(base, w[0], input(t - 3, first, held)), w[1], input(t - 2, first, held)), w[2],
                        input(t - 1, first, held)), w[3], x.at4(t, c)));
    }
  }
}

__global__ void short_conv_state_kernel(Sliced x, float* __restrict__ state,
                                        const int* __restrict__ seq_bounds, const int* __restrict__ seq_seat,
                                        int channels, int taps) {
  const int row = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int first = seq_bounds[row], n = seq_bounds[row + 1] - first;
  if (c >= channels || n <= 0) return;
  float* held = state + (size_t)seq_seat[row] * (taps - 1) * channels;
  float next[kMaxTaps];
  for (int i = 0; i < taps - 1; ++i) {
    const int rel = n + i - (taps - 1);  // index among this step's tokens of the request, negative: still the old state
    next[i] = rel >= 0 ? x.at(first + rel, c) : held[(size_t)(i + n) * channels + c];
  }
  for (int i = 0; i < taps - 1; ++i) held[(size_t)i * channels + c] = next[i];
}

// ---------------------------------------------------------------------------
// Linear recurrence with a matrix state per head and request, float32, token by token:
//   S <- g S;  S <- S + k u^T;  o = S^T q (+ skip * v)
//   kDelta: q, k unit vectors (q times key_dim^-1/2); g = exp(-exp(rate) softplus(decay + bias));
//           u = sigmoid(write) (v - S^T k) with the decayed S.
//   kSsd:   dt = softplus(write + bias); g = exp(-exp(rate) dt); u = dt v; read-out + skip * v.
// State layout: [seat, head, value_dim, key_dim] (S transposed: a column is contiguous).
//
// Two kernels.  The first is parallel over tokens: it makes what a token contributes without the state
// (per head g and the factor of u; per group k . q; for the delta rule q and k as unit vectors, in place).
// The second walks the tokens.  The columns of S (one per value element) never meet, so a column belongs
// to a group of 8, 16 or 32 lanes that share its key_dim entries (lane l of L holds i = 4 l + 4 L r + c), and a
// block of 64 threads owns 8, 4 or 2 columns of one head of one request.  The read-out is taken from the state before the
// write, o = g (S^T q) + u (k . q), which is the same number: both sums over the state then run side by side
// instead of one after the other.  Tokens come in tiles of 16 that cp.async brings into shared memory a tile
// ahead of the walk.
// ---------------------------------------------------------------------------
//   kGated: nothing is normalised; g = decay[t, h] as given (or the constant rate[h] when there is no decay);
//           u = write[t, h] v (or v when there is no write).  With a unit column (v_dim = value_dim - 1) the
//           last column of every head's state sees the value 1 for every token: it carries n <- g n + write k.
constexpr int kRuleDelta = 0, kRuleSsd = 1, kRuleGated = 2;
constexpr int kScanThreads = 64, kScanTile = 16;

struct ScanArgs {
  float *q, *k;  // the delta rule normalises them in place
  const float *v, *decay, *write;
  int q_stride, k_stride, v_stride, decay_stride, write_stride;
  int splits;              // decay and write may be slices of a split product
  long long split_stride;
  const float *rate, *bias, *skip;
  float* state;
  float* out;
  int out_stride;
  const int *seq_bounds, *seq_seat;
  int tokens, heads, groups, key_dim, value_dim;
  int v_dim;  // elements of v per head: value_dim, or value_dim - 1 when the state's last column is the unit column
  float* scalars;  // [tokens, heads, 2]: g and the factor of u
  float* kq;       // [tokens, groups]: k . q
};

template <int RULE>
__global__ void __launch_bounds__(128) recurrence_prepare_kernel(ScanArgs a) {
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int h = threadIdx.x; h < a.heads; h += blockDim.x) {
    float g, factor;
    if (RULE == kRuleGated) {
      g = a.decay ? Sliced{a.decay, a.decay_stride, a.splits, a.split_stride}.at(t, h) : a.rate[h];
      factor = a.write ? Sliced{a.write, a.write_stride, a.splits, a.split_stride}.at(t, h) : 1.f;
      a.scalars[((size_t)t * a.heads + h) * 2] = g;
      a.scalars[((size_t)t * a.heads + h) * 2 + 1] = factor;
      continue;
    }
    const float rate = expf(a.rate[h]), bias = a.bias ? a.bias[h] : 0.f;
    const float w = Sliced{a.write, a.write_stride, a.splits, a.split_stride}.at(t, h);
    if (RULE == kRuleDelta) {
      g = expf(-rate * softplus_f(Sliced{a.decay, a.decay_stride, a.splits, a.split_stride}.at(t, h) + bias));
      factor = sigmoid_f(w);
    } else {
      factor = softplus_f(w + bias);
      g = expf(-rate * factor);
    }
    a.scalars[((size_t)t * a.heads + h) * 2] = g;
    a.scalars[((size_t)t * a.heads + h) * 2 + 1] = factor;
  }
  for (int grp = warp; grp < a.groups; grp += 4) {
    float* q = a.q + (size_t)t * a.q_stride + (size_t)grp * a.key_dim;
    float* k = a.k + (size_t)t * a.k_stride + (size_t)grp * a.key_dim;
    float qq = 0.f, kk = 0.f, kq = 0.f;
    for (int i = lane; i < a.key_dim; i += 32) {
      const float x = q[i], y = k[i];
      qq += x * x; kk += y * y; kq += x * y;
    }
    kq = warp_sum(kq);
    if (RULE == kRuleDelta) {
      qq = warp_sum(qq);
      kk = warp_sum(kk);
      const float qs = rsqrtf((float)a.key_dim) / sqrtf(qq + 1e-6f), ks = 1.f / sqrtf(kk + 1e-6f);
      for (int i = lane; i < a.key_dim; i += 32) { q[i] *= qs; k[i] *= ks; }
      kq *= qs * ks;
    }
    if (lane == 0) a.kq[(size_t)t * a.groups + grp] = kq;
  }
}

__device__ __forceinline__ void cp_async_f4(float* dst, const float* src, bool live) {
  const int bytes = live ? 16 : 0;  // zero-fills when not live
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_f1(float* dst, const float* src, bool live) {
  const int bytes = live ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One stage of the ring: a tile of q, k (rows of KD floats, zero beyond key_dim), the block's columns of v, and
// per token g, the factor of u and k . q.
template <int KD>
struct ScanStage {
  float q[kScanTile][KD];
  float k[kScanTile][KD];
  float v[kScanTile][8];  // at most eight columns a block
  float scalars[kScanTile][4];  // per token: g, the factor of u, k . q, unused
};

// KD: key_dim rounded up (32, 64, 128, 256).  LANES: threads that share a column (8, 16 or 32; each holds
// KD / LANES entries of it).  Few lanes mean few instructions per token and suit a step with many requests; many
// lanes shorten each thread's chain of dependent instructions and fill the machine when one long prompt is all there is.
template <int KD, int LANES, int RULE, bool VEC>
__global__ void __launch_bounds__(kScanThreads) linear_recurrence_kernel(ScanArgs a) {
  constexpr int PER = KD / LANES;
  constexpr int kScanColumns = kScanThreads / LANES;
  static_assert(PER >= 4 && PER % 4 == 0, "a thread holds whole float4s of its column");
  extern __shared__ __align__(16) unsigned char scan_smem[];
  ScanStage<KD>* stages = reinterpret_cast<ScanStage<KD>*>(scan_smem);  // two
  const int row = blockIdx.x, head = blockIdx.y;
  const int tid = threadIdx.x, lane8 = tid % LANES, col_local = tid / LANES;
  const int j = blockIdx.z * kScanColumns + col_local;
  const bool valid = j < a.value_dim;
  const int grp = head / (a.heads / a.groups);
  const int first = a.seq_bounds[row], end = a.seq_bounds[row + 1];
  if (end <= first) return;

  auto stage_tile = [&](int tile, ScanStage<KD>& st) {
    const int count = min(kScanTile, end - tile);
    if (VEC) {
      for (int idx = tid; idx < count * (KD / 4); idx += kScanThreads) {  // rows past the tile's tokens are never read
        const int tok = idx / (KD / 4), i = (idx % (KD / 4)) * 4;
        const bool live = i < a.key_dim;  // columns past key_dim are: zeros, so that they add nothing
        const size_t t = tile + (live ? tok : 0);
        const int at = live ? i : 0;
        cp_async_f4(&st.q[tok][i], a.q + t * a.q_stride + grp * a.key_dim + at, live);
        cp_async_f4(&st.k[tok][i], a.k + t * a.k_stride + grp * a.key_dim + at, live);
      }
    } else {
      for (int idx = tid; idx < count * KD; idx += kScanThreads) {
        const int tok = idx / KD, i = idx % KD;
        const bool live = i < a.key_dim;
        const size_t t = tile + (live ? tok : 0);
        const int at = live ? i : 0;
        cp_async_f1(&st.q[tok][i], a.q + t * a.q_stride + grp * a.key_dim + at, live);
        cp_async_f1(&st.k[tok][i], a.k + t * a.k_stride + grp * a.key_dim + at, live);
      }
    }
    for (int idx = tid; idx < count * kScanColumns; idx += kScanThreads) {
      const int tok = idx / kScanColumns, c = idx % kScanColumns, cj = blockIdx.z * kScanColumns + c;
      const bool live = cj < a.v_dim;  // (the unit column has no element of v: the walk puts 1 in its place)
      cp_async_f1(&st.v[tok][c], a.v + (size_t)(tile + (live ? tok : 0)) * a.v_stride + head * a.v_dim + (live ? cj : 0), live);
    }
    if (tid < count) {
      const bool live = true;
      const size_t t = tile + tid;
      cp_async_f1(&st.scalars[tid][0], a.scalars + (t * a.heads + head) * 2, live);
      cp_async_f1(&st.scalars[tid][1], a.scalars + (t * a.heads + head) * 2 + 1, live);
      cp_async_f1(&st.scalars[tid][2], a.kq + t * a.groups + grp, live);
    }
    cp_async_commit();
  };

  stage_tile(first, stages[0]);
  float* column = a.state + (((size_t)a.seq_seat[row] * a.heads + head) * a.value_dim + (valid ? j : 0)) * a.key_dim;
  float S[PER];
#pragma unroll
  for (int r = 0; r < PER / 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int i = 4 * lane8 + 4 * LANES * r + c;
      S[4 * r + c] = (valid && i < a.key_dim) ? column[i] : 0.f;
    }
  const float skip = (RULE == kRuleSsd && a.skip) ? a.skip[head] : 0.f;
  const bool unit_column = RULE == kRuleGated && j >= a.v_dim;

  int buffer = 0;
  for (int tile = first; tile < end; tile += kScanTile, buffer ^= 1) {
    const int count = min(kScanTile, end - tile);
    const bool more = tile + kScanTile < end;
    if (more) stage_tile(tile + kScanTile, stages[buffer ^ 1]);  // its last readers passed the barrier below
    if (more) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();
    const ScanStage<KD>& st = stages[buffer];
    float* out_at = a.out + (size_t)tile * a.out_stride + head * a.value_dim + (valid ? j : 0);
#pragma unroll 4
    for (int tok = 0; tok < count; ++tok) {
      float kk[PER], qq[PER];
#pragma unroll
      for (int r = 0; r < PER / 4; ++r) {
        const float4 kv = *reinterpret_cast<const float4*>(&st.k[tok][4 * lane8 + 4 * LANES * r]);
        const float4 qv = *reinterpret_cast<const float4*>(&st.q[tok][4 * lane8 + 4 * LANES * r]);
        kk[4 * r] = kv.x; kk[4 * r + 1] = kv.y; kk[4 * r + 2] = kv.z; kk[4 * r + 3] = kv.w;
        qq[4 * r] = qv.x; qq[4 * r + 1] = qv.y; qq[4 * r + 2] = qv.z; qq[4 * r + 3] = qv.w;
      }
      const float4 per_token = *reinterpret_cast<const float4*>(st.scalars[tok]);
      const float g = per_token.x, factor = per_token.y, kq = per_token.z;
      const float vj = unit_column ? 1.f : st.v[tok][col_local];
      // S^T k and S^T q of this column before the write, four partial sums each
      float dk[4] = {0.f, 0.f, 0.f, 0.f}, dq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int e = 0; e < PER; ++e) {
        if (RULE == kRuleDelta) dk[e & 3] += S[e] * kk[e];
        dq[e & 3] += S[e] * qq[e];
      }
      float sum_k = (dk[0] + dk[1]) + (dk[2] + dk[3]), sum_q = (dq[0] + dq[1]) + (dq[2] + dq[3]);
#pragma unroll
      for (int offset = 1; offset < LANES; offset <<= 1) {
        if (RULE == kRuleDelta) sum_k += __shfl_xor_sync(0xffffffffu, sum_k, offset);
        sum_q += __shfl_xor_sync(0xffffffffu, sum_q, offset);
      }
      const float u = RULE == kRuleDelta ? factor * (vj - g * sum_k) : factor * vj;
#pragma unroll
      for (int e = 0; e < PER; ++e) S[e] = g * S[e] + kk[e] * u;
      if (lane8 == 0 && valid) out_at[(size_t)tok * a.out_stride] = g * sum_q + u * kq + skip * vj;
    }
    __syncthreads();  // everyone is done with this stage before the copies of the tile after next land in it
  }
  if (valid) {
#pragma unroll
    for (int r = 0; r < PER / 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int i = 4 * lane8 + 4 * LANES * r + c;
        if (i < a.key_dim) column[i] = S[4 * r + c];
      }
  }
}

template <int KD, int LANES, int RULE>
static cudaError_t launch_scan_sized(const ScanArgs& a, int num_seqs, bool vec, cudaStream_t stream) {
  constexpr int columns = kScanThreads / LANES;
  const dim3 grid(num_seqs, a.heads, (a.value_dim + columns - 1) / columns);
  const size_t shared = 2 * sizeof(ScanStage<KD>);
  auto run = [&](auto kernel) {
    if (shared > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    kernel<<<grid, kScanThreads, shared, stream>>>(a);
  };
  if (vec) run(linear_recurrence_kernel<KD, LANES, RULE, true>);
  else run(linear_recurrence_kernel<KD, LANES, RULE, false>);
  return cudaGetLastError();
}

template <int KD, int RULE>
static cudaError_t launch_scan_lanes(const ScanArgs& a, int num_seqs, bool vec, cudaStream_t stream) {
  // Lanes per column: as few as keep the machine in warps (about four to an SM), at most what leaves a thread a float4.
  const long long columns = (long long)num_seqs * a.heads * a.value_dim;
  int lanes = 8;
  while (lanes < 32 && KD / (2 * lanes) >= 4 && columns * lanes / 32 < 600) lanes *= 2;
  if constexpr (KD >= 128) {
    if (lanes == 32) return launch_scan_sized<KD, 32, RULE>(a, num_seqs, vec, stream);
  }
  if constexpr (KD >= 64) {
    if (lanes == 16) return launch_scan_sized<KD, 16, RULE>(a, num_seqs, vec, stream);
  }
  return launch_scan_sized<KD, 8, RULE>(a, num_seqs, vec, stream);
}

template <int RULE>
static cudaError_t launch_scan(const ScanArgs& a, int num_seqs, cudaStream_t stream) {
  recurrence_prepare_kernel<RULE><<<a.tokens, 128, 0, stream>>>(a);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return err;
  // 16-byte copies need rows of q and k that start on 16-byte boundaries
  const bool vec = a.key_dim % 4 == 0 && a.q_stride % 4 == 0 && a.k_stride % 4 == 0 &&
                   (((uintptr_t)a.q | (uintptr_t)a.k) & 15) == 0;
  if (a.key_dim <= 32) return launch_scan_lanes<32, RULE>(a, num_seqs, vec, stream);
  if (a.key_dim <= 64) return launch_scan_lanes<64, RULE>(a, num_seqs, vec, stream);
  if (a.key_dim <= 128) return launch_scan_lanes<128, RULE>(a, num_seqs, vec, stream);
  return launch_scan_lanes<256, RULE>(a, num_seqs, vec, stream);
}

// ---------------------------------------------------------------------------
// RMS norm over groups of `group` neighbouring columns with a SiLU gate, a warp per (token, group):
//   gate_first (bit 0 of the mode): norm(x * silu(gate)) * weight;   else: norm(x) * weight * silu(gate).
//   bit 1 of the mode: sigmoid(gate) stands where silu(gate) does.
// weight has `weight_len` elements and repeats along the row.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ x, int x_stride, Sliced gate,
                                     const float* __restrict__ weight, int weight_len, T* __restrict__ out,
                                     int out_stride, int tokens, int groups, int group, float eps, int gate_first) {
  const int lane = threadIdx.x & 31;
  const int gate_sigmoid = gate_first >> 1;  // bit 1 of the mode: the gate is sigmoid(gate) instead of silu(gate)
  gate_first &= 1;
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= (long long)tokens * groups) return;
  const int t = (int)(unit / groups), part = (int)(unit % groups);
  const float* xr = x + (size_t)t * x_stride + (size_t)part * group;
  float sq = 0.f;
  for (int i = lane; i < group; i += 32) {
    const float v = gate_first ? xr[i] * gate_f(gate_sigmoid, gate.at(t, part * group + i)) : xr[i];
    sq += v * v;
  }
  const float inv = 1.f / sqrtf(warp_sum(sq) / (float)group + eps);
  T* dst = out + (size_t)t * out_stride + (size_t)part * group;
  for (int i = lane; i < group; i += 32) {
    const float s = gate_f(gate_sigmoid, gate.at(t, part * group + i));
    const float w = weight[(part * group + i) % weight_len];
    dst[i] = from_float<T>(gate_first ? xr[i] * s * inv * w : xr[i] * inv * w * s);
  }
}

// Four columns at a time and the group in registers: group a multiple of 4 and at most 4 * LANES * PIECES,
// strides multiples of 4, pointers aligned to 16 bytes (out to four elements).  LANES threads share a
// (token, group): a warp (LANES = 32, four of them to a block) or a whole block (LANES = blockDim.x = 256).
template <typename T, int PIECES, int LANES>
__global__ void __launch_bounds__(LANES == 32 ? 128 : LANES)
gated_rmsnorm_vec_kernel(const float* __restrict__ x, int x_stride, Sliced gate, const float* __restrict__ weight,
                         int weight_len, T* __restrict__ out, int out_stride, int tokens, int groups, int group,
                         float eps, int gate_first) {
  __shared__ float scratch[32];
  const int gate_sigmoid = gate_first >> 1;
  gate_first &= 1;
  const int lane = threadIdx.x % LANES;
  const long long unit = LANES == 32 ? (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5) : blockIdx.x;
  const bool live = unit < (long long)tokens * groups;  // (a block is either wholly live or a warp per unit)
  if (LANES == 32 && !live) return;
  const int t = (int)(unit / groups), part = (int)(unit % groups);
  const float* xr = x + (size_t)t * x_stride + (size_t)part * group;
  float4 v[PIECES], s[PIECES];
  float sq = 0.f;
#pragma unroll
  for (int p = 0; p < PIECES; ++p) {
    const int i = (p * LANES + lane) * 4;
    if (i < group) {
      v[p] = *reinterpret_cast<const float4*>(xr + i);
      const float4 g = gate.at4(t, part * group + i);
      s[p] = make_float4(gate_f(gate_sigmoid, g.x), gate_f(gate_sigmoid, g.y), gate_f(gate_sigmoid, g.z), gate_f(gate_sigmoid, g.w));
      if (gate_first) v[p] = make_float4(v[p].x * s[p].x, v[p].y * s[p].y, v[p].z * s[p].z, v[p].w * s[p].w);
      sq += (v[p].x * v[p].x + v[p].y * v[p].y) + (v[p].z * v[p].z + v[p].w * v[p].w);
    }
  }
  const float total = LANES == 32 ? warp_sum(sq) : block_sum(sq, scratch);
  const float inv = 1.f / sqrtf(total / (float)group + eps);
  T* dst = out + (size_t)t * out_stride + (size_t)part * group;
#pragma unroll
  for (int p = 0; p < PIECES; ++p) {
    const int i = (p * LANES + lane) * 4;
    if (i < group) {
      const int at = (part * group + i) % weight_len;  // weight_len is a multiple of 4 here
      const float4 w = *reinterpret_cast<const float4*>(weight + at);
      float4 o = make_float4(v[p].x * inv * w.x, v[p].y * inv * w.y, v[p].z * inv * w.z, v[p].w * inv * w.w);
      if (!gate_first) o = make_float4(o.x * s[p].x, o.y * s[p].y, o.z * s[p].z, o.w * s[p].w);
      store4(dst + i, o);
    }
  }
}


// ---------------------------------------------------------------------------
// out[t, c] = act(x[t, c]) (* scale for c < scaled_columns), x a matrix or the slices of a split product.
// ---------------------------------------------------------------------------
// Four columns a thread: columns, scaled_columns and the strides multiples of 4, pointers 16-byte aligned.
__global__ void activation_vec_kernel(Sliced x, float* __restrict__ out, int tokens, int columns, int silu, float scale,
                                      int scaled_columns) {
  const int quads = columns / 4;
  const size_t total = (size_t)tokens * quads;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / quads;
    const int c = (int)(idx % quads) * 4;
    float4 v = x.at4(t, c);
    if (silu) v = make_float4(silu_f(v.x), silu_f(v.y), silu_f(v.z), silu_f(v.w));
    if (c < scaled_columns) v = make_float4(v.x * scale, v.y * scale, v.z * scale, v.w * scale);
    *reinterpret_cast<float4*>(out + t * columns + c) = v;
  }
}

__global__ void activation_kernel(Sliced x, float* __restrict__ out, int tokens, int columns, int silu, float scale,
                                  int scaled_columns) {
  const size_t total = (size_t)tokens * columns;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / columns;
    const int c = (int)(idx % columns);
    float v = x.at(t, c);
    if (silu) v = silu_f(v);
    if (c < scaled_columns) v *= scale;
    out[idx] = v;
  }
}

// ---------------------------------------------------------------------------
// Exponential gates under a running maximum:
//   i = cap tanh((x_i + b_i) / cap);  f = logsigmoid(cap tanh((x_f + b_f) / cap));  m_t = max(f_t + m_(t-1), i_t)
//   keep = exp(f + m_(t-1) - m_t);  take = exp(i - m_t);  floor = exp(-m_t);  m lives in state[seat, head].
// Three kernels.  The gates of all tokens side by side over the whole machine (f into `keep`, i into `take`).  Then
// a block per request walks its tokens: a tile of gates comes into shared memory, a thread per head runs the chain
// (an addition and a maximum per token, its operands on the chip; it reads two arrays and writes three others, so
// that later loads need not wait for earlier stores), and the exponents go back out.  Then the exponentials side
// by side.  The walk is the plain sequence of operations whatever the tile or the cutting of the prompt.
// ---------------------------------------------------------------------------
__global__ void exp_gates_kernel(Sliced log_in, Sliced log_forget, const float* __restrict__ in_bias,
                                 const float* __restrict__ forget_bias, float cap, int tokens, int heads,
                                 float* __restrict__ keep, float* __restrict__ take) {
  const size_t total = (size_t)tokens * heads;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / heads;
    const int h = (int)(idx % heads);
    take[idx] = cap * tanhf((log_in.at(t, h) + in_bias[h]) / cap);
    keep[idx] = -softplus_f(-(cap * tanhf((log_forget.at(t, h) + forget_bias[h]) / cap)));
  }
}

// gates_s: 5 * tile_tokens * heads floats of dynamic shared memory.
__global__ void __launch_bounds__(512)
exp_gate_scan_kernel(float* __restrict__ state, const int* __restrict__ seq_bounds, const int* __restrict__ seq_seat,
                     int heads, int tile_tokens, float* __restrict__ keep, float* __restrict__ take,
                     float* __restrict__ floor_out) {
  extern __shared__ float gates_s[];
  const size_t plane = (size_t)tile_tokens * heads;
  const float* __restrict__ f_in = gates_s;
  const float* __restrict__ i_in = gates_s + plane;
  float* __restrict__ keep_o = gates_s + 2 * plane;
  float* __restrict__ take_o = gates_s + 3 * plane;
  float* __restrict__ floor_o = gates_s + 4 * plane;
  const int row = blockIdx.x;
  const int first = seq_bounds[row], end = seq_bounds[row + 1];
  float m = 0.f;
  float* slot = nullptr;
  if (threadIdx.x < heads) {
    slot = state + (size_t)seq_seat[row] * heads + threadIdx.x;
    m = *slot;
  }
  for (int tile = first; tile < end; tile += tile_tokens) {
    const int count = min(tile_tokens, end - tile) * heads;
    const size_t base = (size_t)tile * heads;
    // (16 bytes a thread and round where the tile starts on a 16-byte boundary: all of a thread's loads in flight)
    const bool quads = (base & 3) == 0 && (count & 3) == 0 && (plane & 3) == 0 &&
                       (((uintptr_t)keep | (uintptr_t)take | (uintptr_t)floor_out) & 15) == 0;
    if (quads) {
#pragma unroll 4
      for (int idx = threadIdx.x * 4; idx < count; idx += blockDim.x * 4) {
        *reinterpret_cast<float4*>(gates_s + idx) = *reinterpret_cast<const float4*>(keep + base + idx);
        *reinterpret_cast<float4*>(gates_s + plane + idx) = *reinterpret_cast<const float4*>(take + base + idx);
      }
    } else {
      for (int idx = threadIdx.x; idx < count; idx += blockDim.x) {
        gates_s[idx] = keep[base + idx];
        gates_s[plane + idx] = take[base + idx];
      }
    }
    __syncthreads();
    if (threadIdx.x < heads) {
      const int steps = count / heads;
      int step = 0;
      // Whole batches of eight tokens: sixteen loads, the chain in registers, twenty-four stores.
      for (; step + 8 <= steps; step += 8) {
        const int at0 = step * heads + threadIdx.x;
        float f[8], i[8], a[8], b[8], c[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          f[u] = f_in[at0 + u * heads];
          i[u] = i_in[at0 + u * heads];
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float m_new = fmaxf(f[u] + m, i[u]);
          a[u] = f[u] + m - m_new;
          b[u] = i[u] - m_new;
          c[u] = -m_new;
          m = m_new;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          keep_o[at0 + u * heads] = a[u];
          take_o[at0 + u * heads] = b[u];
          floor_o[at0 + u * heads] = c[u];
        }
      }
      for (int at = step * heads + threadIdx.x; at < count; at += heads) {
        const float f = f_in[at], i = i_in[at];
        const float m_new = fmaxf(f + m, i);
        keep_o[at] = f + m - m_new;
        take_o[at] = i - m_new;
        floor_o[at] = -m_new;
        m = m_new;
      }
    }
    __syncthreads();
    if (quads) {
#pragma unroll 4
      for (int idx = threadIdx.x * 4; idx < count; idx += blockDim.x * 4) {
        *reinterpret_cast<float4*>(keep + base + idx) = *reinterpret_cast<const float4*>(keep_o + idx);
        *reinterpret_cast<float4*>(take + base + idx) = *reinterpret_cast<const float4*>(take_o + idx);
        *reinterpret_cast<float4*>(floor_out + base + idx) = *reinterpret_cast<const float4*>(floor_o + idx);
      }
    } else {
      for (int idx = threadIdx.x; idx < count; idx += blockDim.x) {
        keep[base + idx] = keep_o[idx];
        take[base + idx] = take_o[idx];
        floor_out[base + idx] = floor_o[idx];
      }
    }
    __syncthreads();
  }
  if (slot) *slot = m;
}

__global__ void exp_three_kernel(float* __restrict__ a, float* __restrict__ b, float* __restrict__ c, size_t total) {
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    a[idx] = expf(a[idx]);
    b[idx] = expf(b[idx]);
    c[idx] = expf(c[idx]);
  }
}

// out[t, h, c] = read[t, h, c] / (max(|read[t, h, value_dim]|, floor[t, h]) + 1e-6) for c < value_dim.
__global__ void stabilized_readout_kernel(const float* __restrict__ read, int read_stride, const float* __restrict__ floor_in,
                                          float* __restrict__ out, int tokens, int heads, int value_dim) {
  const size_t total = (size_t)tokens * heads * value_dim;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(idx % value_dim);
    const size_t th = idx / value_dim;
    const size_t t = th / heads;
    const int h = (int)(th % heads);
    const float* row = read + t * read_stride + (size_t)h * (value_dim + 1);
    out[idx] = row[c] / (fmaxf(fabsf(row[value_dim]), floor_in[th]) + 1e-6f);
  }
}

}  // namespace distie

using namespace distie;

extern "C" int distie_add_layernorm(const float* const* term_ptrs, const float* term_scales, int num_terms,
                                    float* residual, const float* weight, const float* bias, void* out,
                                    const int* rows_index, int rows, int hidden, float eps, int dtype,
                                    cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden < 1 || num_terms < 0 || num_terms > kMaxTerms) return DISTIE_ERR_ARG;
  SumTerms terms;
  terms.count = num_terms;
  for (int j = 0; j < num_terms; ++j) { terms.ptr[j] = term_ptrs[j]; terms.scale[j] = term_scales[j]; }
  uintptr_t low_bits = (uintptr_t)residual | (uintptr_t)weight | (uintptr_t)bias | (uintptr_t)out;
  for (int j = 0; j < num_terms; ++j) low_bits |= (uintptr_t)term_ptrs[j];
  if (hidden % 4 == 0 && hidden <= 4 * kNormPieces * 512 && (low_bits & 15) == 0 &&
      (dtype == DISTIE_BF16 || dtype == DISTIE_F32)) {
    int vec_threads = 32;
    while (vec_threads < 512 && vec_threads * 8 < hidden) vec_threads *= 2;  // about two pieces a thread
    while (4 * kNormPieces * vec_threads < hidden) vec_threads *= 2;
    if (dtype == DISTIE_BF16)
      add_layernorm_vec_kernel<<<rows, vec_threads, 0, stream>>>(terms, residual, weight, bias, (__nv_bfloat16*)out,
                                                                 rows_index, hidden, eps);
    else
      add_layernorm_vec_kernel<<<rows, vec_threads, 0, stream>>>(terms, residual, weight, bias, (float*)out,
                                                                 rows_index, hidden, eps);
    DISTIE_LAUNCH_CHECK();
    return 0;
  }
  const int threads = hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128);
  const size_t shared = (size_t)hidden * sizeof(float);
  if (shared > 200 * 1024) return DISTIE_ERR_UNSUPPORTED;
  if (dtype == DISTIE_BF16) {
    if (shared > 48 * 1024)
      cudaFuncSetAttribute(add_layernorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    add_layernorm_kernel<<<rows, threads, shared, stream>>>(terms, residual, weight, bias, (__nv_bfloat16*)out,
                                                            rows_index, hidden, eps);
  } else if (dtype == DISTIE_F32) {
    if (shared > 48 * 1024)
      cudaFuncSetAttribute(add_layernorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    add_layernorm_kernel<<<rows, threads, shared, stream>>>(terms, residual, weight, bias, (float*)out, rows_index,
                                                            hidden, eps);
  } else {
    return DISTIE_ERR_UNSUPPORTED;
  }
  DISTIE_LAUNCH_CHECK();
  return 0;
}

extern "C" int distie_kv_write(const void* k, int k_stride, const void* v, int v_stride, int in_dtype,
                               const int* positions, const int* token_seq, const int* seq_seat, const int* block_table,
                               int table_width, void* k_cache, void* v_cache, int tokens, int num_kv_heads, int head_dim,
                               int value_dim, int page_size, int num_pages, int dtype, int* error, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (num_kv_heads < 1 || head_dim < 1 || value_dim < 1 || page_size < 1 || table_width < 1) return DISTIE_ERR_ARG;
  const int threads = 128;
#define DISTIE_KV_WRITE(TIN, T)                                                                                      \
  kv_write_kernel<<<tokens, threads, 0, stream>>>((const TIN*)k, k_stride, (const TIN*)v, v_stride, positions,        \
                                                  token_seq, seq_seat, block_table, table_width, (T*)k_cache,         \
                                                  (T*)v_cache, num_kv_heads, head_dim, value_dim, page_size,          \
                                                  num_pages, error)
  if (in_dtype == DISTIE_F32 && dtype == DISTIE_F32) DISTIE_KV_WRITE(float, float);
  else if (in_dtype == DISTIE_F32 && dtype == DISTIE_BF16) DISTIE_KV_WRITE(float, __nv_bfloat16);
  else if (in_dtype == DISTIE_BF16 && dtype == DISTIE_BF16) DISTIE_KV_WRITE(__nv_bfloat16, __nv_bfloat16);
  else if (in_dtype == DISTIE_BF16 && dtype == DISTIE_F32) DISTIE_KV_WRITE(__nv_bfloat16, float);
  else return DISTIE_ERR_UNSUPPORTED;
#undef DISTIE_KV_WRITE
  DISTIE_LAUNCH_CHECK();
  return 0;
}

extern "C" int distie_head_gate(void* x, const float* logits_ptr, int logit_stride, int splits, long long split_stride,
                                int tokens, int num_heads, int dim, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (num_heads < 1 || dim < 1 || splits < 1) return DISTIE_ERR_ARG;
  const Sliced logits{logits_ptr, logit_stride, splits, split_stride};
  const size_t total = (size_t)tokens * num_heads * dim;
  const int threads = 256;
  if (dim == 1 && num_heads % 4 == 0 && logit_stride % 4 == 0 && (splits == 1 || split_stride % 4 == 0) &&
      (((uintptr_t)x | (uintptr_t)logits_ptr) & 15) == 0 && (dtype == DISTIE_BF16 || dtype == DISTIE_F32)) {
    const size_t quads = total / 4, want_vec = (quads + threads - 1) / threads;
    const int blocks_vec = (int)(want_vec < 148 * 32 ? want_vec : 148 * 32);
    if (dtype == DISTIE_BF16)
      element_gate_vec_kernel<<<blocks_vec, threads, 0, stream>>>((__nv_bfloat16*)x, logits, num_heads, quads);
    else
      element_gate_vec_kernel<<<blocks_vec, threads, 0, stream>>>((float*)x, logits, num_heads, quads);
    DISTIE_LAUNCH_CHECK();
    return 0;
  }
  if (dim % 4 == 0 && ((uintptr_t)x & 15) == 0 && (dtype == DISTIE_BF16 || dtype == DISTIE_F32)) {
    const size_t quads = total / 4, want_vec = (quads + threads - 1) / threads;
    const int blocks_vec = (int)(want_vec < 148 * 32 ? want_vec : 148 * 32);
    if (dtype == DISTIE_BF16)
      head_gate_vec_kernel<<<blocks_vec, threads, 0, stream>>>((__nv_bfloat16*)x, logits, num_heads, dim, quads);
    else
      head_gate_vec_kernel<<<blocks_vec, threads, 0, stream>>>((float*)x, logits, num_heads, dim, quads);
    DISTIE_LAUNCH_CHECK();
    return 0;
  }
  const size_t want = (total + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  if (dtype == DISTIE_BF16)
    head_gate_kernel<<<blocks, threads, 0, stream>>>((__nv_bfloat16*)x, logits, num_heads, dim, total);
  else if (dtype == DISTIE_F32)
    head_gate_kernel<<<blocks, threads, 0, stream>>>((float*)x, logits, num_heads, dim, total);
  else
    return DISTIE_ERR_UNSUPPORTED;
  DISTIE_LAUNCH_CHECK();
  return 0;
}

extern "C" int distie_seq_index(const int* token_seq, int tokens, int num_seqs, int* token_first, int* seq_bounds,
                                cudaStream_t stream) {
  if (tokens <= 0 || num_seqs < 1) return DISTIE_ERR_ARG;
  seq_index_kernel<<<1, 1024, 0, stream>>>(token_seq, tokens, num_seqs, token_first, seq_bounds);
  DISTIE_LAUNCH_CHECK();
  return 0;
}

// state may be null only when taps == 1.  `single`: every request of the step brings exactly one token (the
// caller knows from how the step was laid out); the state is then moved on by the convolution kernel itself.
extern "C" int distie_short_conv(const float* x_ptr, int x_stride, int splits, long long split_stride,
                                 const float* weight, const float* bias, float* state,
                                 const int* token_seq, const int* token_first, const int* seq_bounds,
                                 const int* seq_seat, int tokens, int num_seqs, int channels, int taps, int silu,
                                 int single, float* out, const float* input_bias, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (channels < 1 || taps < 1 || num_seqs < 1) return DISTIE_ERR_ARG;
  if (taps > kMaxTaps) return DISTIE_ERR_UNSUPPORTED;
  if (taps > 1 && state == nullptr) return DISTIE_ERR_ARG;
  if (splits < 1) return DISTIE_ERR_ARG;
  const Sliced x{x_ptr, x_stride, splits, split_stride, input_bias};  // input_bias [channels]: added to every input of the step
  const int threads = 128;
  const bool vec = !single && channels % 4 == 0 && x_stride % 4 == 0 && split_stride % 4 == 0 &&
                   (((uintptr_t)x_ptr | (uintptr_t)state | (uintptr_t)out | (uintptr_t)bias | (uintptr_t)input_bias) & 15) == 0;
  if (vec) {
    const dim3 grid((channels / 4 + threads - 1) / threads, tokens);
    if (taps == 4 && ((uintptr_t)weight & 15) == 0) {
      const dim3 grid_runs(grid.x, (tokens + kConvRun - 1) / kConvRun);
      short_conv_run4_kernel<<<grid_runs, threads, 0, stream>>>(x, weight, bias, state, token_seq, token_first, seq_seat,
                                                                tokens, channels, silu, out);
    } else if (taps == 4)
      short_conv_vec_kernel<4><<<grid, threads, 0, stream>>>(x, weight, bias, state, token_seq, token_first,
                                                             seq_seat, channels, taps, silu, out);
    else
      short_conv_vec_kernel<0><<<grid, threads, 0, stream>>>(x, weight, bias, state, token_seq, token_first,
                                                             seq_seat, channels, taps, silu, out);
  } else if (single && taps > 1) {
    const dim3 grid((channels + threads - 1) / threads, tokens);
    short_conv_single_kernel<<<grid, threads, 0, stream>>>(x, weight, bias, state, token_seq, seq_seat, channels, taps,
                                                           silu, out);
  } else {
    const dim3 grid((channels + threads - 1) / threads, tokens);
    short_conv_kernel<<<grid, threads, 0, stream>>>(x, weight, bias, state, token_seq, token_first, seq_seat,
                                                    channels, taps, silu, single, out);
  }
  DISTIE_LAUNCH_CHECK();
  if (taps > 1 && !single) {
    const dim3 grid_state((channels + threads - 1) / threads, num_seqs);
    short_conv_state_kernel<<<grid_state, threads, 0, stream>>>(x, state, seq_bounds, seq_seat, channels, taps);
    DISTIE_LAUNCH_CHECK();
  }
  return 0;
}

// rule 2 (gated): decay may be null (rate[h] is then the decay itself) and write may be null (1); with `unit_column`
// v has value_dim - 1 elements per head and the state's last column per head is fed the value 1.
// q and k are overwritten by their unit vectors under the delta rule.  scratch: tokens * (2 heads + groups) floats.
// decay and write may be slices of a split product (`splits` of them, `split_stride` floats apart).
extern "C" int distie_linear_recurrence(int rule, float* q, int q_stride, float* k, int k_stride,
                                        const float* v, int v_stride, const float* decay, int decay_stride,
                                        const float* write, int write_stride, int splits, long long split_stride,
                                        const float* rate, const float* bias,
                                        const float* skip, float* state, float* out, int out_stride,
                                        float* scratch, const int* seq_bounds, const int* seq_seat, int tokens,
                                        int num_seqs, int heads, int groups, int key_dim, int value_dim,
                                        int unit_column, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads < 1 || groups < 1 || heads % groups || key_dim < 1 || value_dim < 1 || num_seqs < 1 || heads > 65535)
    return DISTIE_ERR_ARG;
  if (key_dim > 256 || (value_dim + 1) / 2 > 65535) return DISTIE_ERR_UNSUPPORTED;
  if (state == nullptr || scratch == nullptr || (rule == kRuleDelta && decay == nullptr) ||
      (rule != kRuleGated && (rate == nullptr || write == nullptr || unit_column)) ||
      (rule == kRuleGated && rate == nullptr && decay == nullptr) || (unit_column && value_dim < 2))
    return DISTIE_ERR_ARG;
  ScanArgs a;
  a.q = q; a.k = k; a.v = v; a.decay = decay; a.write = write;
  a.q_stride = q_stride; a.k_stride = k_stride; a.v_stride = v_stride; a.decay_stride = decay_stride;
  a.write_stride = write_stride;
  a.splits = splits < 1 ? 1 : splits; a.split_stride = split_stride;
  a.rate = rate; a.bias = bias; a.skip = skip; a.state = state; a.out = out; a.out_stride = out_stride;
  a.seq_bounds = seq_bounds; a.seq_seat = seq_seat;
  a.tokens = tokens; a.heads = heads; a.groups = groups; a.key_dim = key_dim; a.value_dim = value_dim;
  a.v_dim = unit_column ? value_dim - 1 : value_dim;
  a.scalars = scratch;
  a.kq = scratch + (size_t)tokens * heads * 2;
  cudaError_t err;
  if (rule == kRuleDelta) err = launch_scan<kRuleDelta>(a, num_seqs, stream);
  else if (rule == kRuleSsd) err = launch_scan<kRuleSsd>(a, num_seqs, stream);
  else if (rule == kRuleGated) err = launch_scan<kRuleGated>(a, num_seqs, stream);
  else return DISTIE_ERR_ARG;
  return err == cudaSuccess ? 0 : (int)err;
}

extern "C" int distie_gated_rmsnorm(const float* x, int x_stride, const float* gate_ptr, int gate_stride, int splits,
                                    long long split_stride, const float* weight, int weight_len, void* out,
                                    int out_stride, int tokens, int n, int group, float eps, int gate_first, int dtype,
                                    cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (n < 1 || group < 1 || n % group || weight_len < 1 || splits < 1) return DISTIE_ERR_ARG;
  if (dtype != DISTIE_BF16 && dtype != DISTIE_F32) return DISTIE_ERR_UNSUPPORTED;
  const Sliced gate{gate_ptr, gate_stride, splits, split_stride};
  const int groups = n / group, warps = 4;
  const long long units = (long long)tokens * groups;
  const unsigned blocks = (unsigned)((units + warps - 1) / warps);
  const bool vec = group % 4 == 0 && group <= 4 * 256 * 8 && weight_len % 4 == 0 && x_stride % 4 == 0 &&
                   gate_stride % 4 == 0 && split_stride % 4 == 0 && out_stride % 4 == 0 &&
                   (((uintptr_t)x | (uintptr_t)gate_ptr | (uintptr_t)weight | (uintptr_t)out) & 15) == 0;
#define DISTIE_GATED(T)                                                                                                  \
  do {                                                                                                                   \
    if (!vec)                                                                                                            \
      gated_rmsnorm_kernel<<<blocks, warps * 32, 0, stream>>>(x, x_stride, gate, weight, weight_len, (T*)out, out_stride, \
                                                              tokens, groups, group, eps, gate_first);                   \
    else if (group <= 256)                                                                                               \
      gated_rmsnorm_vec_kernel<T, 2, 32><<<blocks, warps * 32, 0, stream>>>(x, x_stride, gate, weight, weight_len,        \
                                                                            (T*)out, out_stride, tokens, groups, group,   \
                                                                            eps, gate_first);                            \
    else if (group <= 2048)                                                                                              \
      gated_rmsnorm_vec_kernel<T, 2, 256><<<(unsigned)units, 256, 0, stream>>>(x, x_stride, gate, weight, weight_len,     \
                                                                               (T*)out, out_stride, tokens, groups,       \
                                                                               group, eps, gate_first);                  \
    else                                                                                                                 \
      gated_rmsnorm_vec_kernel<T, 8, 256><<<(unsigned)units, 256, 0, stream>>>(x, x_stride, gate, weight, weight_len,     \
                                                                               (T*)out, out_stride, tokens, groups,       \
                                                                               group, eps, gate_first);                  \
  } while (0)
  if (dtype == DISTIE_BF16) DISTIE_GATED(__nv_bfloat16);
  else DISTIE_GATED(float);
#undef DISTIE_GATED
  DISTIE_LAUNCH_CHECK();
  return 0;
}

extern "C" int distie_activation(const float* x, int x_stride, int splits, long long split_stride, float* out, int tokens,
                                 int columns, int silu, float scale, int scaled_columns, cudaStream_t stream) {
  if (tokens <= 0 || columns <= 0) return 0;
  if (splits < 1 || scaled_columns < 0 || scaled_columns > columns) return DISTIE_ERR_ARG;
  const size_t total = (size_t)tokens * columns;
  if (columns % 4 == 0 && scaled_columns % 4 == 0 && x_stride % 4 == 0 && split_stride % 4 == 0 &&
      (((uintptr_t)x | (uintptr_t)out) & 15) == 0) {
    const size_t quads = total / 4;
    const unsigned vec_blocks = (unsigned)((quads + 255) / 256 > 148 * 16 ? 148 * 16 : (quads + 255) / 256);
    activation_vec_kernel<<<vec_blocks, 256, 0, stream>>>(Sliced{x, x_stride, splits, split_stride}, out, tokens, columns,
                                                         silu, scale, scaled_columns);
    DISTIE_LAUNCH_CHECK();
    return 0;
  }
  const unsigned blocks = (unsigned)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
  activation_kernel<<<blocks, 256, 0, stream>>>(Sliced{x, x_stride, splits, split_stride}, out, tokens, columns, silu,
                                               scale, scaled_columns);
  DISTIE_LAUNCH_CHECK();
  return 0;
}

// log_in and log_forget [tokens, heads] (views of one projection: the same slices); keep, take, floor [tokens, heads]
// contiguous; state [seats, heads].
extern "C" int distie_exp_gate_scan(const float* log_in, const float* log_forget, int gate_stride, int splits,
                                    long long split_stride, const float* in_bias, const float* forget_bias, float cap,
                                    float* state, const int* seq_bounds, const int* seq_seat, int num_seqs, int tokens,
                                    int heads, float* keep, float* take, float* floor_out, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (heads < 1 || splits < 1 || !(cap > 0.f) || state == nullptr || in_bias == nullptr || forget_bias == nullptr)
    return DISTIE_ERR_ARG;
  if (heads > 512 || tokens < 1) return DISTIE_ERR_UNSUPPORTED;
  const size_t total = (size_t)tokens * heads;
  const unsigned blocks = (unsigned)((total + 255) / 256 > 148 * 8 ? 148 * 8 : (total + 255) / 256);
  exp_gates_kernel<<<blocks, 256, 0, stream>>>(Sliced{log_in, gate_stride, splits, split_stride},
                                              Sliced{log_forget, gate_stride, splits, split_stride}, in_bias, forget_bias,
                                              cap, tokens, heads, keep, take);
  DISTIE_LAUNCH_CHECK();
  // Tiles as long as 160 KB of shared memory allow (512 tokens up to 16 heads): a tile costs a round trip to memory
  // on either side of its walk, which only a long tile makes small beside the walk.
  int tile_tokens = 8192 / (heads < 16 ? 16 : heads);
  if (tile_tokens < 1) tile_tokens = 1;
  if (tile_tokens > tokens) tile_tokens = tokens;
  const size_t scan_shared = 5 * (size_t)tile_tokens * heads * sizeof(float);
  if (scan_shared > 48 * 1024)
    cudaFuncSetAttribute(exp_gate_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)scan_shared);
  exp_gate_scan_kernel<<<num_seqs, 512, scan_shared, stream>>>(
      state, seq_bounds, seq_seat, heads, tile_tokens, keep, take, floor_out);
  DISTIE_LAUNCH_CHECK();
  exp_three_kernel<<<blocks, 256, 0, stream>>>(keep, take, floor_out, total);
  DISTIE_LAUNCH_CHECK();
  return 0;
}

extern "C" int distie_stabilized_readout(const float* read, int read_stride, const float* floor_in, float* out, int tokens,
                                         int heads, int value_dim, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (heads < 1 || value_dim < 1) return DISTIE_ERR_ARG;
  const size_t total = (size_t)tokens * heads * value_dim;
  const unsigned blocks = (unsigned)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
  stabilized_readout_kernel<<<blocks, 256, 0, stream>>>(read, read_stride, floor_in, out, tokens, heads, value_dim);
  DISTIE_LAUNCH_CHECK();
  return 0;
}
