// Attention through a latent for portions of prompts, on the tensor cores (bfloat16).
//
// Every token of the cache is ONE row [latent (rank) | rotated key part (rot)] that all heads share; a query of a
// head is [its plain part folded into the latent's space (rank) | its rotated part (rot)].  The score of a query and
// a key is the product of the two rows, and the value of a key is the first `rank` columns of its row, so one tile
// of rows in shared memory serves both products.
//
// A portion is cut into tiles of 64 consecutive tokens of one request.  One CTA of 16 warps takes one tile and one
// head and walks the keys the tile can see in blocks of 64 (cp.async, two stages; rows past the last visible key
// are zero-filled; rows are located one by one through the block table, so any page size works):
//
//   S = Q K^T    warp (rg, kh), rg = 0..3, kh = 0..3: query rows 16 rg .. 16 rg + 15 against keys 16 kh .. 16 kh + 15
//                of the block, reduction over the whole row (even and odd steps of it into accumulators of their
//                own, so that twice as many products are in flight); mma.sync.m16n8k16, float32 accumulators
//   softmax      online, float32, base-2 exponentials; the four warps of a row group exchange their block maxima
//                through shared memory, so all keep the same running maximum, and each keeps the sum of its own
//                keys (the sums are added at the end)
//   P            bfloat16 into shared memory, [64 rows x 64 keys]
//   O += P V     warp (rg, ch): the same 16 rows, value columns ch VC/4 .. (ch + 1) VC/4 - 1, reduction over the
//                block's 64 keys; O stays in registers (VC/8 floats a thread)
//   end          O / (sum + exp(sink - max)): the sink of the head is a term of the denominator without a value
//
// Single tokens (SINGLE) run the same loop with the roles of the rows changed: the rows of a tile are the heads of
// ONE token (16 RG of them a CTA), which all see the same keys, and the keys are cut into `splits` ranges of whole
// blocks, a CTA each, so that a step of few tokens fills the machine.  With more than one split a CTA leaves, per
// (token, head), the unnormalised sum, its maximum (natural-log units) and its sum of weights, in the layout that
// the size-agnostic kernel's merge reads; the sink joins in the merge.
//
// Key j is visible to the row at position p iff j <= p.  It depends on positions only, so the result does not depend
// on how the prompt was cut.  rank and rot multiples of 8 (16-byte copies), rank <= VC, rank + rot <= ROW; other
// sizes are refused (-2) and the caller uses the size-agnostic kernel.
#include "common.cuh"

namespace distie {

constexpr int kLmParts = 4;              // warps of a row group: parts of a block's keys, and of the value columns
constexpr int kLmKeys = 64;

__device__ __forceinline__ uint32_t lm_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void lm_cp16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void lm_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void lm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
__device__ __forceinline__ void lm_ldmatrix(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lm_ldmatrix_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lm_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lm_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// The warps of row group `rg` meet (barrier 0 is __syncthreads).
__device__ __forceinline__ void lm_group_sync(int rg) {
  asm volatile("bar.sync %0, %1;" ::"r"(rg + 1), "n"(kLmParts * 32) : "memory");
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a tile of CHUNKS chunks a row (CHUNKS a multiple of 8); the
// chunk is XOR-ed with the row so that the eight rows of an ldmatrix hit different banks.
template <int CHUNKS>
__device__ __forceinline__ uint32_t lm_offset(int row, int chunk) {
  return (uint32_t)((row * CHUNKS + (chunk ^ (row & 7))) * 16);
}

template <int ROW, int VC, int RG, bool SINGLE>
__global__ void __launch_bounds__(RG * kLmParts * 32, 1)
latent_attention_mma_kernel(const __nv_bfloat16* __restrict__ folded, const __nv_bfloat16* __restrict__ rotated,
                            __nv_bfloat16* __restrict__ out, int tokens, int heads, int rank, int rot,
                            const int* __restrict__ q_tiles, const int* __restrict__ positions,
                            const int* __restrict__ token_seq, const int* __restrict__ seq_seat,
                            const int* __restrict__ block_table, int table_width,
                            const __nv_bfloat16* __restrict__ k_cache, int page_size, int page_shift, int num_pages,
                            float scale_log2, const float* __restrict__ sink, float* __restrict__ partial,
                            int first, int* __restrict__ error) {
  constexpr int kLmRows = 16 * RG;            // rows of a tile: tokens of a portion, or heads of a single token
  constexpr int kLmThreads = RG * kLmParts * 32;
  constexpr int CHUNKS = ROW / 8;
  constexpr int TILE_BYTES = kLmKeys * ROW * 2;
  constexpr int P_CHUNKS = kLmKeys / 8;
  constexpr int NT = VC / (8 * kLmParts);  // tiles of 8 value columns a warp owns
  static_assert(ROW % 64 == 0 && NT % 2 == 0 && VC <= ROW, "tile sizes");
  extern __shared__ __align__(128) unsigned char lm_s[];
  unsigned char* q_s = lm_s;
  unsigned char* k_s = q_s + kLmRows * ROW * 2;                // two stages
  unsigned char* p_s = k_s + 2 * TILE_BYTES;                   // [64][64] bfloat16
  float* stat_s = reinterpret_cast<float*>(p_s + kLmRows * kLmKeys * 2);  // [parts][64]

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rg = warp % RG, kh = warp / RG;  // row group; part of the keys and of the columns
  const int g = lane >> 2, c = lane & 3;
  // A portion's tile: `rows` consecutive tokens from t0, one head.  A single token: `rows` heads from h0, token t0.
  // Tiles late in a request see the most keys and take longest: start them first.  A tile of the list holds up to
  // 128 rows: two CTAs take its halves.
  int t0, rows, h0;
  if (SINGLE) {
    t0 = first + blockIdx.y;
    h0 = blockIdx.x * kLmRows;
    rows = min(kLmRows, heads - h0);
  } else {
    const int slot = gridDim.y - 1 - blockIdx.y;
    const int tile = slot >> 1, half = slot & 1;
    h0 = blockIdx.x;
    t0 = q_tiles[2 * tile] + half * kLmRows;
    rows = min(kLmRows, q_tiles[2 * tile + 1] - half * kLmRows);
  }
  if (rows <= 0) return;
  const int row_len = rank + rot;
  const int p0 = positions[t0];
  const int seat = seq_seat[token_seq[t0]];
  const int* table = block_table + (size_t)seat * table_width;
  const int p_last = SINGLE ? p0 : p0 + rows - 1;
  int block_begin = 0, block_end = p_last / kLmKeys + 1;
  if (SINGLE && gridDim.z > 1) {
    const int per = (block_end + gridDim.z - 1) / gridDim.z;
    block_begin = min(block_end, (int)blockIdx.z * per);
    block_end = min(block_end, block_begin + per);
  }
  const int live_chunks = row_len / 8;               // chunks of a row that hold data; the rest stay zero
  const int ksteps = (row_len + 15) / 16;

  auto load_q = [&]() {
    for (int idx = threadIdx.x; idx < kLmRows * CHUNKS; idx += kLmThreads) {
      const int r = idx / CHUNKS, ch = idx % CHUNKS;
      const int live = r < rows ? r : 0;
      const int t = SINGLE ? t0 : t0 + live, head = SINGLE ? h0 + live : h0;
      const __nv_bfloat16* src = folded;
      int bytes = 0;
      if (r < rows && ch < live_chunks) {
        bytes = 16;
        src = ch * 8 < rank ? folded + ((size_t)head * tokens + t) * rank + ch * 8
                            : rotated + ((size_t)t * heads + head) * rot + (ch * 8 - rank);
      }
      lm_cp16(lm_smem(q_s + lm_offset<CHUNKS>(r, ch)), src, bytes);
    }
  };
  // A warp copies whole rows: the row's page is looked up once, and the lanes take its 16-byte pieces in turn.
  auto load_k = [&](int block, int stage) {
    const int kb = block * kLmKeys;
    for (int r = warp; r < kLmKeys; r += kLmThreads / 32) {
      const int key = kb + r;
      const __nv_bfloat16* src = k_cache;
      bool ok = key <= p_last;
      if (ok) {
        const int column = page_shift >= 0 ? key >> page_shift : key / page_size;
        const int within = page_shift >= 0 ? key & (page_size - 1) : key % page_size;
        const int page = column < table_width ? table[column] : -1;
        if (page < 0 || page >= num_pages) {
          if (lane == 0 && error) atomicExch(error, 3);
          ok = false;
        } else {
          src = k_cache + ((size_t)page * page_size + within) * (size_t)row_len;
        }
      }
      const uint32_t dst = lm_smem(k_s + stage * TILE_BYTES) + r * (CHUNKS * 16);
#pragma unroll
      for (int ch = lane; ch < CHUNKS; ch += 32) {
        const bool live = ok && ch < live_chunks;
        lm_cp16(dst + ((ch ^ (r & 7)) * 16), live ? src + ch * 8 : k_cache, live ? 16 : 0);
      }
    }
  };

  load_q();
  if (block_begin < block_end) load_k(block_begin, 0);
  lm_commit();

  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int r = 0; r < 4; ++r) o[i][r] = 0.f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};
  const int pos_row[2] = {SINGLE ? p0 : p0 + rg * 16 + g, SINGLE ? p0 : p0 + rg * 16 + g + 8};
  const int a_row = rg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;  // the row this lane names in an A-operand ldmatrix
  const int key_row = kh * 16 + (lane & 7) + (lane >> 4) * 8;       // and in a B-operand ldmatrix of the scores
  const uint32_t q_base = lm_smem(q_s) + a_row * (CHUNKS * 16);
  uint32_t off_a[4], off_b[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    off_a[j] = ((2 * j + (lane >> 4)) ^ (a_row & 7)) * 16;
    off_b[j] = ((2 * j + ((lane >> 3) & 1)) ^ (key_row & 7)) * 16;
  }

  for (int block = block_begin; block < block_end; ++block) {
    const int stage = (block - block_begin) & 1;
    if (block + 1 < block_end) load_k(block + 1, stage ^ 1);
    lm_commit();
    lm_wait<1>();
    __syncthreads();
    const unsigned char* k_tile = k_s + stage * TILE_BYTES;

    // ---- S = Q K^T: 16 rows x 16 keys a warp ------------------------------------------------------------------
    float s[2][4], s_odd[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int r = 0; r < 4; ++r) s[i][r] = s_odd[i][r] = 0.f;
    // Four steps of the reduction span 128 bytes of a row; within them the piece a lane reads is the step's piece
    // XOR-ed with its row, which is the same for every four steps: the offsets are made once.
    const uint32_t k_base = lm_smem(k_tile) + key_row * (CHUNKS * 16);
    const int quads = ksteps >> 2;
    for (int quad = 0; quad < quads; ++quad) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t a[4], b[4];
        lm_ldmatrix(a, q_base + quad * 128 + off_a[j]);
        lm_ldmatrix(b, k_base + quad * 128 + off_b[j]);
        if (j & 1) {
          lm_mma(s_odd[0], a, b[0], b[1]);
          lm_mma(s_odd[1], a, b[2], b[3]);
        } else {
          lm_mma(s[0], a, b[0], b[1]);
          lm_mma(s[1], a, b[2], b[3]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      if (4 * quads + j < ksteps) {
        uint32_t a[4], b[4];
        lm_ldmatrix(a, q_base + quads * 128 + off_a[j]);
        lm_ldmatrix(b, k_base + quads * 128 + off_b[j]);
        if (j & 1) {
          lm_mma(s_odd[0], a, b[0], b[1]);
          lm_mma(s_odd[1], a, b[2], b[3]);
        } else {
          lm_mma(s[0], a, b[0], b[1]);
          lm_mma(s[1], a, b[2], b[3]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int r = 0; r < 4; ++r) s[i][r] += s_odd[i][r];

    // ---- mask and block maximum -------------------------------------------------------------------------------
    const int kb = block * kLmKeys + kh * 16;
    float tile_max[2] = {-INFINITY, -INFINITY};
    if (kb + 15 <= (SINGLE ? p0 : p0 + rg * 16)) {  // wholly visible to every row of the warp
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int r = 0; r < 4; ++r) tile_max[r >> 1] = fmaxf(tile_max[r >> 1], s[i][r]);
    } else {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int key = kb + i * 8 + 2 * c + (r & 1);
          s[i][r] = key <= pos_row[r >> 1] ? s[i][r] : -INFINITY;
          tile_max[r >> 1] = fmaxf(tile_max[r >> 1], s[i][r]);
        }
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float m = tile_max[h];
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      tile_max[h] = m;
      if (c == 0) stat_s[kh * kLmRows + rg * 16 + g + 8 * h] = m;
    }
    lm_group_sync(rg);
    // row_max holds scale_log2 * (largest raw score so far); the scale is positive, so the order is the same.
    float corr[2], shift[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float m = tile_max[h];
#pragma unroll
      for (int part = 0; part < kLmParts; ++part) m = fmaxf(m, stat_s[part * kLmRows + rg * 16 + g + 8 * h]);
      const float m_new = fmaxf(row_max[h], m * scale_log2);
      corr[h] = (m_new == -INFINITY) ? 1.f : exp2f(row_max[h] - m_new);
      row_max[h] = m_new;
      row_sum[h] *= corr[h];
      shift[h] = m_new == -INFINITY ? 0.f : -m_new;
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float p = exp2f(fmaf(s[i][r], scale_log2, shift[r >> 1]));  // exp2(-inf) = 0 for hidden keys
        s[i][r] = p;
        row_sum[r >> 1] += p;
      }
      const int chunk = kh * 2 + i;
      const int r0 = rg * 16 + g, r1 = r0 + 8;
      *reinterpret_cast<uint32_t*>(p_s + lm_offset<P_CHUNKS>(r0, chunk) + 4 * c) = lm_pack(s[i][0], s[i][1]);
      *reinterpret_cast<uint32_t*>(p_s + lm_offset<P_CHUNKS>(r1, chunk) + 4 * c) = lm_pack(s[i][2], s[i][3]);
    }
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0];
      o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
    lm_group_sync(rg);

    // ---- O += P V: 16 rows x VC/4 columns a warp ----------------------------------------------------------------
#pragma unroll
    for (int kk = 0; kk < kLmKeys / 16; ++kk) {
      uint32_t a[4];
      lm_ldmatrix(a, lm_smem(p_s + lm_offset<P_CHUNKS>(a_row, 2 * kk + (lane >> 4))));
      const int value_row = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int dp = 0; dp < NT / 2; ++dp) {
        uint32_t b[4];
        lm_ldmatrix_trans(b, lm_smem(k_tile + lm_offset<CHUNKS>(value_row, kh * NT + 2 * dp + (lane >> 4))));
        lm_mma(o[2 * dp], a, b[0], b[1]);
        lm_mma(o[2 * dp + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();  // this stage, P and the maxima are overwritten in the next iteration
  }
  lm_wait<0>();

  // ---- the warps of a row group add their sums; the sink joins the denominator; store -----------------------
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float l = row_sum[h];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    row_sum[h] = l;
    if (c == 0) stat_s[kh * kLmRows + rg * 16 + g + 8 * h] = l;
  }
  lm_group_sync(rg);
  const bool leave_parts = SINGLE && gridDim.z > 1;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = rg * 16 + g + 8 * h;
    float l = 0.f;
#pragma unroll
    for (int part = 0; part < kLmParts; ++part) l += stat_s[part * kLmRows + row];
    if (row >= rows) continue;
    const int t = SINGLE ? t0 : t0 + row, head = SINGLE ? h0 + row : h0;
    if (leave_parts) {
      // (a split without keys leaves zeros, a maximum of -inf and a sum of 0: the merge gives it no weight)
      float* dst = partial + (((size_t)blockIdx.z * tokens + t) * heads + head) * (size_t)(rank + 2);
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const int col = (kh * NT + i) * 8 + 2 * c;
        if (col < rank) *reinterpret_cast<float2*>(dst + col) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
      }
      if (kh == 0 && c == 0) {
        dst[rank] = row_max[h] * 0.6931471805599453f;
        dst[rank + 1] = l;
      }
      continue;
    }
    const float sink2 = sink ? sink[head] * 1.4426950408889634f : -INFINITY;
    const float top = fmaxf(row_max[h], sink2);
    const float shrink = row_max[h] == -INFINITY ? 0.f : exp2f(row_max[h] - top);
    const float den = l * shrink + (sink ? exp2f(sink2 - top) : 0.f);
    const float inv = den > 0.f ? shrink / den : 0.f;
    __nv_bfloat16* dst = out + ((size_t)head * tokens + t) * rank;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int col = (kh * NT + i) * 8 + 2 * c;
      if (col < rank) *reinterpret_cast<uint32_t*>(dst + col) = lm_pack(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
    }
  }
}

template <int ROW, int VC, int RG, bool SINGLE>
static int launch_latent_mma(const void* folded, const void* rotated, void* out, int tokens, int heads, int rank, int rot,
                             const int* q_tiles, int num_tiles, const int* positions, const int* token_seq,
                             const int* seq_seat, const int* block_table, int table_width, const void* k_cache,
                             int page_size, int num_pages, float scale, const float* sink, float* partial, int first,
                             int count, int splits, int* error, cudaStream_t stream) {
  constexpr int kRows = 16 * RG;
  const size_t shared = (size_t)kRows * ROW * 2 + 2 * (size_t)kLmKeys * ROW * 2 + kRows * kLmKeys * 2 +
                        kLmParts * kRows * sizeof(float);
  auto kernel = latent_attention_mma_kernel<ROW, VC, RG, SINGLE>;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
  if (err != cudaSuccess) return (int)err;
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (page_shift = 0; (1 << page_shift) < page_size;) ++page_shift;
  const dim3 grid = SINGLE ? dim3((heads + kRows - 1) / kRows, count, splits) : dim3(heads, 2 * num_tiles);
  kernel<<<grid, RG * kLmParts * 32, shared, stream>>>(
      (const __nv_bfloat16*)folded, (const __nv_bfloat16*)rotated, (__nv_bfloat16*)out, tokens, heads, rank, rot, q_tiles,
      positions, token_seq, seq_seat, block_table, table_width, (const __nv_bfloat16*)k_cache, page_size, page_shift,
      num_pages, scale * 1.4426950408889634f, sink, partial, first, error);
  DISTIE_LAUNCH_CHECK();
  return 0;
}

}  // namespace distie

using namespace distie;

// Tokens per tile of `q_tiles` ([num_tiles, 2] int32: first token of the tile, number of rows <= 128).
// folded [heads, tokens, rank], rotated [tokens, heads, rot], out [heads, tokens, rank]: bfloat16, contiguous.
// -2: sizes this kernel does not take.
extern "C" int distie_latent_attention_tiles(const void* folded, const void* rotated, void* out, int tokens, int heads,
                                             int rank, int rot, const int* q_tiles, int num_tiles,
                                             const int* positions, const int* token_seq, const int* seq_seat,
                                             const int* block_table, int table_width, const void* k_cache,
                                             int page_size, int num_pages, float scale, const float* sink, int* error,
                                             cudaStream_t stream) {
  if (num_tiles <= 0 || tokens <= 0) return 0;
  if (heads < 1 || rank < 1 || rot < 0 || page_size < 1 || table_width < 1) return DISTIE_ERR_ARG;
  if (rank % 8 || rot % 8 || !(scale > 0.f) || 2 * (long long)num_tiles > 65535) return -2;
  const int row = rank + rot;
#define DISTIE_LATENT_MMA(ROW, VC)                                                                                   \
  return launch_latent_mma<ROW, VC, 4, false>(folded, rotated, out, tokens, heads, rank, rot, q_tiles, num_tiles,    \
                                              positions, token_seq, seq_seat, block_table, table_width, k_cache,    \
                                              page_size, num_pages, scale, sink, nullptr, 0, 0, 1, error, stream)
  if (row <= 128) DISTIE_LATENT_MMA(128, 128);
  if (row <= 320 && rank <= 256) DISTIE_LATENT_MMA(320, 256);
  if (row <= 576 && rank <= 512) DISTIE_LATENT_MMA(576, 512);
#undef DISTIE_LATENT_MMA
  return -2;
}

// Tokens first .. first + count - 1 of the step, each a single token of its request: their heads are the rows of a
// tile.  `splits` ranges of key blocks (at most 64); with more than one, `partial` holds
// [splits, tokens, heads, rank + 2] floats and the caller merges them (distie_latent_merge).  -2: sizes not taken.
extern "C" int distie_latent_attention_single(const void* folded, const void* rotated, void* out, float* partial,
                                              int tokens, int heads, int rank, int rot, const int* positions,
                                              const int* token_seq, const int* seq_seat, const int* block_table,
                                              int table_width, const void* k_cache, int page_size, int num_pages,
                                              float scale, const float* sink, int splits, int first, int count,
                                              int* error, cudaStream_t stream) {
  if (count <= 0 || tokens <= 0) return 0;
  if (heads < 1 || rank < 1 || rot < 0 || page_size < 1 || table_width < 1 || first < 0 || first + count > tokens ||
      splits < 1 || splits > 64 || (splits > 1 && !partial))
    return DISTIE_ERR_ARG;
  if (rank % 8 || rot % 8 || !(scale > 0.f) || count > 65535) return -2;
  const int row = rank + rot;
#define DISTIE_LATENT_ONE(ROW, VC, RG)                                                                               \
  return launch_latent_mma<ROW, VC, RG, true>(folded, rotated, out, tokens, heads, rank, rot, nullptr, 0, positions, \
                                              token_seq, seq_seat, block_table, table_width, k_cache, page_size,    \
                                              num_pages, scale, sink, partial, first, count, splits, error, stream)
#define DISTIE_LATENT_SINGLE(ROW, VC)          \
  do {                                         \
    if (heads <= 16) DISTIE_LATENT_ONE(ROW, VC, 1); \
    if (heads <= 32) DISTIE_LATENT_ONE(ROW, VC, 2); \
    DISTIE_LATENT_ONE(ROW, VC, 4);             \
  } while (0)
  if (row <= 128) DISTIE_LATENT_SINGLE(128, 128);
  if (row <= 320 && rank <= 256) DISTIE_LATENT_SINGLE(320, 256);
  if (row <= 576 && rank <= 512) DISTIE_LATENT_SINGLE(576, 512);
#undef DISTIE_LATENT_SINGLE
#undef DISTIE_LATENT_ONE
  return -2;
}
