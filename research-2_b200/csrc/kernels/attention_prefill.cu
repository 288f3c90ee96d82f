// Prefill attention over the paged cache on the warp-level tensor cores (mma.sync m16n8k16,
// bfloat16 in, float accumulate): batches that hold portions of prompts, possibly beside single
// decoded tokens. The new keys and values are already in the cache when it runs.
//
// A CTA takes 64 consecutive rows of one entry and one query head; each of its four warps owns
// 16 rows. Keys and values come in tiles of 64 through a ring of stages, in one of two ways:
//   * TMA (head size 64, page sizes 8, 16, 32 or a multiple of 64): one 4-D tensor copy per page
//     and matrix ([dim][offset in page][kv head][page], 128-byte swizzle), issued by the lanes of
//     warp 0, signalled through an mbarrier; shared-memory rows are 128 bytes, swizzled in
//     16-byte pieces by the row index, which keeps ldmatrix free of bank conflicts;
//   * cp.async (any head size up to 128 and any page size): 16-byte pieces fetched through the
//     block table, rows padded by 16 bytes against bank conflicts. Scores are scaled and masked
// in float (causal, window, context length), softmax is online, P is rounded to bfloat16 for
// the second product, the output is normalised at the end. Key rows that no row of the tile may
// see at all are filled with zeros instead of being read.
//
// Formulas: kelpie-models/kelpie_models/kernels/ops/paged_attention.py:160-240. HEAD_DIM is a
// compile-time constant (-DHEAD_DIM=64), in steps of 16 up to 128: one library per head size.
#include <cuda.h>
#include <limits.h>
#include <math.h>

#include <cstring>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tensor_maps.cuh"

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
  int box_rows;      // TMA form: key rows per tensor copy (the page size, or 64 for larger pages)
  int* error_flag;   // TMA form: where a bounded wait that ran out is recorded
};

bool g_prefill_tma = true;                    // r2_attention_prefill_set_tma
constexpr int TMA_TILE_BYTES = BN * 128;       // TMA form (head size 64): unpadded 128-byte rows
using namespace r2ptx;
#define R2_ERR_TIMEOUT_KV_TILE 5

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


// Threads: four warps that compute; the TMA form adds a fifth that only issues the tensor copies
// (a tile's two or more copies cost the issuing thread several hundred cycles, which would
// otherwise come out of one computing warp and hold the other three at the next barrier).
template <bool TMA>
__global__ void __launch_bounds__(WARPS * 32 + (TMA ? 32 : 0))
prefill_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const PrefillParams p) {
  pdl_launch_dependents();  // the next kernel may begin its prologue
  pdl_wait();               // the previous kernel's writes are visible from here on
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t* q_s = smem;                         // [BM] rows, padded
  // cp.async form: STAGES padded tiles of keys, then of values. TMA form: the same at 1,024-byte
  // alignment (the swizzle works on address bits), 128-byte rows.
  constexpr int KV_TILE = TMA ? TMA_TILE_BYTES : TILE_BYTES;
  uint8_t* k_s = TMA ? reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem + TILE_BYTES) + 1023) & ~uintptr_t(1023))
                     : smem + TILE_BYTES;
  uint8_t* v_s = k_s + STAGES * KV_TILE;
  __shared__ int tile_entry, tile_row0;
  __shared__ __align__(8) uint64_t full[STAGES];    // TMA form: a stage's copies have landed
  __shared__ __align__(8) uint64_t empty[STAGES];   // TMA form: the four computing warps are done with a stage

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
  for (int id = tid; id < BM * (HD / 8) && tid < WARPS * 32; id += WARPS * 32) {
    int row = id / (HD / 8), c = id % (HD / 8);
    bool ok = row < rows_here;
    const bf16* src = p.q + size_t(t0 + r0 + (ok ? row : 0)) * p.q_row_stride + size_t(h) * HD + c * 8;
    cp_async16(smem_u32(q_s + row * ROW_BYTES + c * 16), src, ok);
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
      cp_async16(smem_u32(k_s) + dst, p.k_cache + off, ok);
      cp_async16(smem_u32(v_s) + dst, p.v_cache + off, ok);
    }
  };

  const int j_first = lo / BN * BN;
  const int n_tiles = (pmax - j_first) / BN + 1;
  int pages_next[PIECES];

  // TMA form: lane b of the producer warp brings box b of a tile (box_rows key rows of one page,
  // keys and values); a box no row of which any query row may see is left out. The page of a box
  // is looked up one tile before its copies are issued.
  const uint32_t full_base = smem_u32(full), empty_base = smem_u32(empty);
  const int n_boxes = TMA ? BN / p.box_rows : 0;
  int box_page = INT_MIN;  // lane's page for the tile whose copies are issued next
  auto box_lookup = [&](int j0) {
    box_page = INT_MIN;
    if (lane < n_boxes) {
      const int jb = j0 + lane * p.box_rows;
      if (jb + p.box_rows - 1 >= lo && jb <= pmax) box_page = table[page_index(jb, p.page_size, p.page_shift)];
    }
  };
  auto box_issue = [&](int j0, int stage) {  // the whole producer warp, converged
    const bool mine = box_page != INT_MIN;
    const uint32_t n_mine = __popc(__ballot_sync(0xffffffffu, mine));
    const uint32_t bar = full_base + uint32_t(stage) * 8u;
    const uint32_t box_bytes = uint32_t(p.box_rows) * 128u;
    if (lane == 0) mbar_expect_tx(bar, 2u * n_mine * box_bytes);  // with no box at all the phase completes at once
    __syncwarp();
    if (mine) {
      const int jb = j0 + lane * p.box_rows;
      const int page = (box_page < 0 || box_page >= p.n_pages) ? 0 : box_page;  // a bad entry reads the null page
      const int off = page_offset(jb, p.page_size, p.page_shift);
      const uint32_t dst = uint32_t(stage * TMA_TILE_BYTES) + uint32_t(lane) * box_bytes;
      tma_load_4d(smem_u32(k_s) + dst, &map_k, 0, off, kvh, page, bar);
      tma_load_4d(smem_u32(v_s) + dst, &map_v, 0, off, kvh, page, bar);
    }
  };
  if (TMA) {
    if (tid == 0) {
      for (int st = 0; st < STAGES; ++st) {
        mbar_init(full_base + uint32_t(st) * 8u, 1);
        mbar_init(empty_base + uint32_t(st) * 8u, WARPS);
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == WARPS) {
      // ---- the producer warp: tile after tile into the ring, a stage as soon as the computing
      // warps have let go of it (the ring's first round finds every stage free) -----------------
      uint32_t round_parity = 0;
      box_lookup(j_first);
      for (int it = 0; it < n_tiles; ++it) {
        const int stage = it % STAGES;
        if (it >= STAGES && !mbar_wait(empty_base + uint32_t(stage) * 8u, round_parity ^ 1u)) {
          if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_KV_TILE);
          break;
        }
        box_issue(j_first + it * BN, stage);
        if (it + 1 < n_tiles) box_lookup(j_first + (it + 1) * BN);
        if (stage == STAGES - 1) round_parity ^= 1u;
      }
      return;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");  // the query tile
  } else {
#pragma unroll
    for (int t = 0; t < STAGES - 1; ++t) {
      if (t < n_tiles) {
        pages_of(j_first + t * BN, pages_next);
        load_tile(j_first + t * BN, t, pages_next);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    if (STAGES - 1 < n_tiles) pages_of(j_first + (STAGES - 1) * BN, pages_next);
  }
  uint32_t tile_parity = 0;  // TMA form: parity of the ring's current round
  bool tiles_ok = true;

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
    if (TMA) {
      if (it == 0) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");  // the query tile
        asm volatile("bar.sync 1, %0;" ::"n"(WARPS * 32) : "memory");
      }
      // tile `it` has landed when its barrier's phase completes
      if (tiles_ok && !mbar_wait(full_base + uint32_t(stage) * 8u, tile_parity)) {
        if (tid == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_KV_TILE);
        tiles_ok = false;
      }
      if (stage == STAGES - 1) tile_parity ^= 1u;
      if (j0 < lo || j0 + BN - 1 > pmax) {
        // Rows of the tile outside the keys that any query row may see were not copied, or hold
        // whatever their slots held: their scores are masked by selection, but a value row is
        // multiplied by p = 0, so it has to be finite. They are set to zero.
        for (int row = tid; row < BN; row += WARPS * 32) {
          const int j = j0 + row;
          if (j < lo || j > pmax) {
            const uint32_t dst = smem_u32(v_s) + uint32_t(stage * TMA_TILE_BYTES + row * 128);
#pragma unroll
            for (int c = 0; c < 8; ++c) asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst + c * 16), "r"(0u) : "memory");
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // later tensor copies overwrite these rows
        asm volatile("bar.sync 1, %0;" ::"n"(WARPS * 32) : "memory");     // the four computing warps
      }
    } else {
      // tile `it` has landed (only the newest STAGES - 2 groups may still be in flight); after the
      // barrier every thread's part of it is visible and the stage of tile it - 1 is free
      asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
      __syncthreads();
      if (it + STAGES - 1 < n_tiles) load_tile(j0 + (STAGES - 1) * BN, (it + STAGES - 1) % STAGES, pages_next);
      asm volatile("cp.async.commit_group;" ::: "memory");
      if (it + STAGES < n_tiles) pages_of(j0 + STAGES * BN, pages_next);
    }
    if (it == 0) {
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        uint32_t addr = smem_u32(q_s + (warp * 16 + (lane & 15)) * ROW_BYTES + (ks * 16 + 8 * (lane >> 4)) * 2);
        ldmatrix_x4(addr, qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
      }
    }
    // a warp whose 16 rows all lie past the entry's rows, or before every key of this tile, rests
    const bool warp_active = warp * 16 < rows_here && j0 <= pmin + min(warp * 16 + 15, rows_here - 1);
    if (warp_active) {
      const uint32_t kt = smem_u32(k_s) + uint32_t(stage * KV_TILE);
      const uint32_t vt = smem_u32(v_s) + uint32_t(stage * KV_TILE);
      // a row's 16-byte piece `c`: padded rows, or 128-byte rows swizzled by the row index
      auto piece = [&](uint32_t tile, int row, int c) -> uint32_t {
        return TMA ? tile + uint32_t(row * 128 + ((c ^ (row & 7)) << 4)) : tile + uint32_t(row * ROW_BYTES + c * 16);
      };
      float s[BN / 8][4];
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int np = 0; np < BN / 16; ++np) {  // two 8-key tiles per ldmatrix
          uint32_t b0, b1, b2, b3;
          int key = np * 16 + (lane & 7) + 8 * (lane >> 4);
          ldmatrix_x4(piece(kt, key, ks * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
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
        // key k of the tile is seen by a row if lo <= k <= hi (two compares against registers: the same test
        // written with && and || over the position compiles to a chain of branches per element)
        const int hi_a = row_a < rows_here ? pos_a - j0 : -1, hi_b = row_b < rows_here ? pos_b - j0 : -1;
        const int lo_a = p.window > 0 ? pos_a - p.window + 1 - j0 : 0, lo_b = p.window > 0 ? pos_b - p.window + 1 - j0 : 0;
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int k = nt * 8 + 2 * tq + c;
            const bool va = (k <= hi_a) & (k >= lo_a);
            const bool vb = (k <= hi_b) & (k >= lo_b);
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
          ldmatrix_x4_trans(piece(vt, key, dp * 2 + (lane >> 4)), b0, b1, b2, b3);
          mma_bf16(o[2 * dp], a0, a1, a2, a3, b0, b1);
          mma_bf16(o[2 * dp + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
    if (TMA) {
      // this warp is done with the stage (its ldmatrix reads have returned): the producer may refill it
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_base + uint32_t(stage) * 8u) : "memory");
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

namespace {

template <bool TMA>
int launch(const CUtensorMap& mk, const CUtensorMap& mv, const PrefillParams& p, int n_tiles, cudaStream_t stream) {
  const size_t smem = TMA ? size_t(TILE_BYTES) + 1024 + 2 * STAGES * size_t(TMA_TILE_BYTES) : (1 + 2 * STAGES) * size_t(TILE_BYTES);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_kernel<TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return int(e);
    // several CTAs per SM hide each other's waits: ask for the shared memory that takes
    e = cudaFuncSetAttribute(prefill_kernel<TMA>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e != cudaSuccess) return int(e);
    configured = true;
  }
  r2_launch(prefill_kernel<TMA>, dim3(dim3(n_tiles, p.n_heads)), dim3(WARPS * 32 + (TMA ? 32 : 0)), size_t(smem), stream, mk, mv, p);
  return launch_status();
}

}  // namespace

// n_tiles: the sum over entries of ceil(rows / 64), which the host knows from the batch (more is
// harmless: the CTAs beyond find no tile). error_flag: a device word in which a bounded wait that
// ran out is recorded (may be null; the tensor-copy form is then not used).
extern "C" int r2_attention_prefill(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_cache,
                                    const void* v_cache, long long page_stride, int page_size, int n_pages,
                                    const int32_t* block_tables, int table_width, const int32_t* q_start,
                                    const int32_t* seq_lens, int n_entries, int n_tiles, int n_heads, int n_kv_heads,
                                    float scale, int window, int* error_flag, cudaStream_t stream) {
  if (n_entries <= 0 || n_tiles <= 0) return R2_OK;
  if (n_heads < 1 || n_kv_heads < 1 || n_heads % n_kv_heads != 0 || page_size < 1 || window < 0) return R2_BAD_SHAPE;
  if (page_stride % 8 != 0 || q_row_stride % 8 != 0 || out_row_stride % 2 != 0 || (reinterpret_cast<uintptr_t>(k_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(v_cache) & 15) || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 3)) {
    return R2_BAD_ALIGN;
  }
  if (!(scale > 0.f)) return R2_UNSUPPORTED;  // the softmax takes the largest raw score for the largest scaled one
  PrefillParams p;
  p.q = (const bf16*)q; p.q_row_stride = q_row_stride;
  p.out = (bf16*)out; p.out_row_stride = out_row_stride;
  p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
  p.page_stride = page_stride; p.page_size = page_size; p.page_shift = page_shift_of(page_size); p.n_pages = n_pages;
  p.block_tables = block_tables; p.table_width = table_width;
  p.q_start = q_start; p.seq_lens = seq_lens; p.n_entries = n_entries;
  p.n_heads = n_heads; p.n_kv_heads = n_kv_heads;
  p.scale = scale; p.window = window;
  p.box_rows = 0;
  p.error_flag = error_flag;
  CUtensorMap mk, mv;
  const bool page_fits = page_size == 8 || page_size == 16 || page_size == 32 || page_size % 64 == 0;
  if (HD == 64 && page_fits && error_flag != nullptr && g_prefill_tma) {
    p.box_rows = page_size < 64 ? page_size : 64;
    if (r2::page_map(&mk, k_cache, page_stride, page_size, n_kv_heads, n_pages, p.box_rows, HD) &&
        r2::page_map(&mv, v_cache, page_stride, page_size, n_kv_heads, n_pages, p.box_rows, HD)) {
      return launch<true>(mk, mv, p, n_tiles, stream);
    }
    p.box_rows = 0;
  }
  memset(&mk, 0, sizeof(mk));
  memset(&mv, 0, sizeof(mv));
  return launch<false>(mk, mv, p, n_tiles, stream);
}

// Tests and measurements compare the two ways of bringing the tiles in.
extern "C" int r2_attention_prefill_set_tma(int on) {
  int before = g_prefill_tma ? 1 : 0;
  g_prefill_tma = on != 0;
  return before;
}
