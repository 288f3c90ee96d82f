// Prefill attention over the paged cache on the warp-level tensor cores (mma.sync m16n8k16,
// bfloat16 in, float accumulate): batches that hold portions of prompts, possibly beside single
// decoded tokens. The new keys and values are already in the cache when it runs.
//
// A CTA takes 64 consecutive rows of one entry and one query head; each of its four warps owns
// 16 rows. Keys and values come in tiles of 64 through a two-stage cp.async pipeline, fetched
// row by row through the block table (any page size), rows padded by 16 bytes in shared memory
// so that ldmatrix is free of bank conflicts for every head size. Scores are scaled and masked
// in float (causal, window, context length), softmax is online, P is rounded to bfloat16 for
// the second product, the output is normalised at the end. Key rows that no row of the tile may
// see at all are filled with zeros instead of being read.
//
// Formulas: kelpie-models/kelpie_models/kernels/ops/paged_attention.py:160-240. HEAD_DIM is a
// compile-time constant (-DHEAD_DIM=64), in steps of 16 up to 128: one library per head size.
#include <math.h>

#include <limits.h>

#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif

namespace {

constexpr int HD = HEAD_DIM;
constexpr int BM = 64, BN = 64, WARPS = 4;
constexpr int STAGES = HD <= 64 ? 3 : 2;      // key/value tiles in flight or in use
constexpr int CHUNKS = HD / 8;                // 16-byte pieces of a row
constexpr int PIECES = BN * CHUNKS / (WARPS * 32);  // pieces of a tile that one thread copies
static_assert(BN * CHUNKS % (WARPS * 32) == 0, "a tile's pieces divide among the threads");
constexpr int ROW_BYTES = HD * 2 + 16;        // padded row in shared memory
constexpr int TILE_BYTES = BN * ROW_BYTES;
constexpr int KSTEPS = HD / 16;               // k-steps of q.k
constexpr int DTILES = HD / 8;                // 8-wide output tiles of p.v
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 128, "head sizes come in steps of 16 up to 128");

struct PrefillParams {
  const bf16* q; int q_row_stride;
  bf16* out; int out_row_stride;
  const bf16* k_cache; const bf16* v_cache;
  long long page_stride; int page_size; int page_shift; int n_pages;
  const int32_t* block_tables; int table_width;
  const int32_t* q_start; const int32_t* seq_lens; int n_entries;
  int n_heads, n_kv_heads;
  float scale; int window;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  int bytes = pred ? 16 : 0;  // 0 source bytes: the 16 destination bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 2^x by the hardware's approximation (2 ulp; 2^-inf = 0).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(WARPS * 32)
prefill_kernel(const PrefillParams p) {
  pdl_launch_dependents();  // the next kernel may begin its prologue
  pdl_wait();               // the previous kernel's writes are visible from here on
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t* q_s = smem;                         // [BM] rows
  uint8_t* k_s = smem + TILE_BYTES;                  // STAGES tiles
  uint8_t* v_s = smem + (1 + STAGES) * TILE_BYTES;   // STAGES tiles
  __shared__ int tile_entry, tile_row0;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y;
  const int kvh = h / (p.n_heads / p.n_kv_heads);

  // which entry and which 64 rows of it this CTA has: tiles are numbered entry by entry
  if (tid == 0) {
    // tiles are handed out from the end: in a prompt the last rows see the most keys, and the
    // longest-running CTAs should start first
    int left = int(gridDim.x) - 1 - int(blockIdx.x), found = -1, row0 = 0;
    for (int e = 0; e < p.n_entries; ++e) {
      int rows = p.q_start[e + 1] - p.q_start[e];
      int tiles = (rows + BM - 1) / BM;
      if (left < tiles) {
        found = e;
        row0 = left * BM;
        break;
      }
      left -= tiles;
    }
    tile_entry = found;
    tile_row0 = row0;
  }
  __syncthreads();
  const int e = tile_entry;
  if (e < 0) return;
  const int r0 = tile_row0;
  const int t0 = p.q_start[e];
  const int n_rows = p.q_start[e + 1] - t0;
  const int seq_len = p.seq_lens[e];
  const int start = seq_len - n_rows;           // position of the entry's first row
  const int rows_here = min(BM, n_rows - r0);
  const int pmin = start + r0, pmax = start + r0 + rows_here - 1;
  const int lo = p.window > 0 ? max(0, pmin - p.window + 1) : 0;
  const int32_t* table = p.block_tables + size_t(e) * p.table_width;

  // ---- the query tile ----
  for (int id = tid; id < BM * (HD / 8); id += WARPS * 32) {
    int row = id / (HD / 8), c = id % (HD / 8);
    bool ok = row < rows_here;
    const bf16* src = p.q + size_t(t0 + r0 + (ok ? row : 0)) * p.q_row_stride + size_t(h) * HD + c * 8;
    cp_async16(smem_addr(q_s + row * ROW_BYTES + c * 16), src, ok);
  }

  // Key and value tiles are copied in 16-byte pieces, consecutive threads taking consecutive
  // pieces of a row, so that one warp's copy reads whole rows (rows of a page lie one after
  // another in memory). A thread has PIECES pieces per tile, each in a row of its own, so it
  // looks up PIECES pages. The lookups of a tile are made one iteration before its copies are
  // issued, and the copies STAGES - 1 iterations before the tile is used, so that neither
  // latency is waited for.
  auto pages_of = [&](int j0, int (&pages)[PIECES]) {
#pragma unroll
    for (int i = 0; i < PIECES; ++i) {
      int j = j0 + (tid + i * WARPS * 32) / CHUNKS;
      // the entry is checked where it is used, so that nothing waits for this load here; a row
      // outside the tile's keys is marked with a page below every valid one
      pages[i] = (j >= lo && j <= pmax) ? table[page_index(j, p.page_size, p.page_shift)] : INT_MIN;
    }
  };
  auto load_tile = [&](int j0, int stage, const int (&pages)[PIECES]) {
#pragma unroll
    for (int i = 0; i < PIECES; ++i) {
      int id = tid + i * WARPS * 32;
      int row = id / CHUNKS, c = id % CHUNKS;
      int j = j0 + row;
      bool ok = pages[i] != INT_MIN;
      int page = (pages[i] < 0 || pages[i] >= p.n_pages) ? 0 : pages[i];  // a bad entry reads the null page
      size_t off = ok ? size_t(page) * p.page_stride + (size_t(kvh) * p.page_size + page_offset(j, p.page_size, p.page_shift)) * HD + c * 8 : 0;
      uint32_t dst = uint32_t(stage * TILE_BYTES + row * ROW_BYTES + c * 16);
      cp_async16(smem_addr(k_s) + dst, p.k_cache + off, ok);
      cp_async16(smem_addr(v_s) + dst, p.v_cache + off, ok);
    }
  };

  const int j_first = lo / BN * BN;
  const int n_tiles = (pmax - j_first) / BN + 1;
  int pages_next[PIECES];
#pragma unroll
  for (int t = 0; t < STAGES - 1; ++t) {
    if (t < n_tiles) {
      pages_of(j_first + t * BN, pages_next);
      load_tile(j_first + t * BN, t, pages_next);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  if (STAGES - 1 < n_tiles) pages_of(j_first + (STAGES - 1) * BN, pages_next);

  float o[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  uint32_t qf[KSTEPS][4];
  const int g = lane >> 2, tq = lane & 3;
  const int row_a = warp * 16 + g, row_b = row_a + 8;  // this thread's two rows within the tile
  const int pos_a = pmin + row_a, pos_b = pmin + row_b;

  for (int it = 0; it < n_tiles; ++it) {
    const int stage = it % STAGES;
    const int j0 = j_first + it * BN;
    // tile `it` has landed (only the newest STAGES - 2 groups may still be in flight); after the
    // barrier every thread's part of it is visible and the stage of tile it - 1 is free
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();
    if (it + STAGES - 1 < n_tiles) load_tile(j0 + (STAGES - 1) * BN, (it + STAGES - 1) % STAGES, pages_next);
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (it + STAGES < n_tiles) pages_of(j0 + STAGES * BN, pages_next);
    if (it == 0) {
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        uint32_t addr = smem_addr(q_s + (warp * 16 + (lane & 15)) * ROW_BYTES + (ks * 16 + 8 * (lane >> 4)) * 2);
        ldmatrix_x4(addr, qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
      }
    }
    // a warp whose 16 rows all lie past the entry's rows, or before every key of this tile, rests
    const bool warp_active = warp * 16 < rows_here && j0 <= pmin + min(warp * 16 + 15, rows_here - 1);
    if (warp_active) {
      const uint8_t* kt = k_s + stage * TILE_BYTES;
      const uint8_t* vt = v_s + stage * TILE_BYTES;
      float s[BN / 8][4];
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int np = 0; np < BN / 16; ++np) {  // two 8-key tiles per ldmatrix
          uint32_t b0, b1, b2, b3;
          int key = np * 16 + (lane & 7) + 8 * (lane >> 4);
          int d = ks * 16 + 8 * ((lane >> 3) & 1);
          ldmatrix_x4(smem_addr(kt + key * ROW_BYTES + d * 2), b0, b1, b2, b3);
          mma_bf16(s[2 * np], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
          mma_bf16(s[2 * np + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
        }
      }
      // scale, mask, online softmax: rows row_a (c0, c1) and row_b (c2, c3). Scores are kept in
      // units of log2(e) so that one exp2 per element does the softmax's exponential.
      const float scale2 = p.scale * 1.4426950408889634f;
      float mx_a = -INFINITY, mx_b = -INFINITY;
      // every key of this tile is visible to every row of this warp: no mask to evaluate
      const int warp_pmin = pmin + warp * 16, warp_pmax = pmin + min(warp * 16 + 15, rows_here - 1);
      const bool all_visible = j0 + BN - 1 <= warp_pmin && warp * 16 + 15 < rows_here &&
                               (p.window == 0 || j0 > warp_pmax - p.window);
      // (the scale is positive, so the largest raw score is the largest scaled one; it goes into
      // the exponent's multiply-add)
      if (all_visible) {
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            mx_a = fmaxf(mx_a, s[nt][c]);
            mx_b = fmaxf(mx_b, s[nt][2 + c]);
          }
        }
      } else {
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            int j = j0 + nt * 8 + 2 * tq + c;
            bool va = j <= pos_a && (p.window == 0 || j > pos_a - p.window) && row_a < rows_here;
            bool vb = j <= pos_b && (p.window == 0 || j > pos_b - p.window) && row_b < rows_here;
            s[nt][c] = va ? s[nt][c] : -INFINITY;
            s[nt][2 + c] = vb ? s[nt][2 + c] : -INFINITY;
            mx_a = fmaxf(mx_a, s[nt][c]);
            mx_b = fmaxf(mx_b, s[nt][2 + c]);
          }
        }
      }
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
      const float m_a = fmaxf(m_run[0], mx_a * scale2), m_b = fmaxf(m_run[1], mx_b * scale2);
      // a row that has seen no key yet keeps exp(-inf - -inf) out of the way
      const float base_a = m_a == -INFINITY ? 0.f : m_a, base_b = m_b == -INFINITY ? 0.f : m_b;
      const float corr_a = fast_exp2(m_run[0] - base_a), corr_b = fast_exp2(m_run[1] - base_b);
      float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          s[nt][c] = fast_exp2(fmaf(s[nt][c], scale2, -base_a));
          s[nt][2 + c] = fast_exp2(fmaf(s[nt][2 + c], scale2, -base_b));
          sum_a += s[nt][c];
          sum_b += s[nt][2 + c];
        }
      }
      sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
      sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
      sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
      sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
      l_run[0] = l_run[0] * corr_a + sum_a;
      l_run[1] = l_run[1] * corr_b + sum_b;
      m_run[0] = m_a;
      m_run[1] = m_b;
#pragma unroll
      for (int dt = 0; dt < DTILES; ++dt) {
        o[dt][0] *= corr_a;
        o[dt][1] *= corr_a;
        o[dt][2] *= corr_b;
        o[dt][3] *= corr_b;
      }
      // o += p . v, 16 keys at a time
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {
        uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp) {  // two 8-wide output tiles per ldmatrix
          uint32_t b0, b1, b2, b3;
          int key = kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
          int d = dp * 16 + 8 * (lane >> 4);
          ldmatrix_x4_trans(smem_addr(vt + key * ROW_BYTES + d * 2), b0, b1, b2, b3);
          mma_bf16(o[2 * dp], a0, a1, a2, a3, b0, b1);
          mma_bf16(o[2 * dp + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  const float inv_a = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv_b = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
#pragma unroll
  for (int dt = 0; dt < DTILES; ++dt) {
    int d = dt * 8 + 2 * tq;
    if (row_a < rows_here) {
      __nv_bfloat162 v = __floats2bfloat162_rn(o[dt][0] * inv_a, o[dt][1] * inv_a);
      *reinterpret_cast<__nv_bfloat162*>(p.out + size_t(t0 + r0 + row_a) * p.out_row_stride + size_t(h) * HD + d) = v;
    }
    if (row_b < rows_here) {
      __nv_bfloat162 v = __floats2bfloat162_rn(o[dt][2] * inv_b, o[dt][3] * inv_b);
      *reinterpret_cast<__nv_bfloat162*>(p.out + size_t(t0 + r0 + row_b) * p.out_row_stride + size_t(h) * HD + d) = v;
    }
  }
}

}  // namespace

extern "C" int r2_attention_prefill_head_dim(void) { return HD; }

// n_tiles: the sum over entries of ceil(rows / 64), which the host knows from the batch.
extern "C" int r2_attention_prefill(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_cache,
                                    const void* v_cache, long long page_stride, int page_size, int n_pages,
                                    const int32_t* block_tables, int table_width, const int32_t* q_start,
                                    const int32_t* seq_lens, int n_entries, int n_tiles, int n_heads, int n_kv_heads,
                                    float scale, int window, cudaStream_t stream) {
  if (n_entries <= 0 || n_tiles <= 0) return R2_OK;
  if (n_heads < 1 || n_kv_heads < 1 || n_heads % n_kv_heads != 0 || page_size < 1 || window < 0) return R2_BAD_SHAPE;
  if (page_stride % 8 != 0 || q_row_stride % 8 != 0 || out_row_stride % 2 != 0 || (reinterpret_cast<uintptr_t>(k_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(v_cache) & 15) || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 3)) {
    return R2_BAD_ALIGN;
  }
  PrefillParams p;
  p.q = (const bf16*)q; p.q_row_stride = q_row_stride;
  p.out = (bf16*)out; p.out_row_stride = out_row_stride;
  p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
  p.page_stride = page_stride; p.page_size = page_size; p.page_shift = page_shift_of(page_size); p.n_pages = n_pages;
  p.block_tables = block_tables; p.table_width = table_width;
  p.q_start = q_start; p.seq_lens = seq_lens; p.n_entries = n_entries;
  p.n_heads = n_heads; p.n_kv_heads = n_kv_heads;
  p.scale = scale; p.window = window;
  if (!(scale > 0.f)) return R2_UNSUPPORTED;  // the softmax takes the largest raw score for the largest scaled one
  const size_t smem = (1 + 2 * STAGES) * size_t(TILE_BYTES);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return int(e);
    // several CTAs per SM hide each other's waits: ask for the shared memory that takes
    e = cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e != cudaSuccess) return int(e);
    configured = true;
  }
  r2_launch(prefill_kernel, dim3(dim3(n_tiles, n_heads)), dim3(WARPS * 32), size_t(smem), stream, p);
  return launch_status();
}
