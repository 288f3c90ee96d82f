// Prefill attention over the paged cache on the 5th-generation tensor cores (tcgen05), head size
// 64, bfloat16: portions of prompts, possibly beside single decoded tokens. The new keys and
// values are already in the cache when it runs.
//
// A CTA takes 128 consecutive rows of one entry and one query head. Roles by warp:
//   warp 0     brings the query tile (2-D tensor copy) and, through a three-stage ring, 64-key
//              tiles of keys and values (4-D tensor copies [dim][offset in page][kv head][page],
//              one per page, 128-byte swizzle); page lookups run one tile ahead;
//   warp 1     issues the products: S = Q K^T (128 x 64, four k-steps) into one of two score
//              buffers in tensor memory, and O += P V (128 x 64) into the output accumulator;
//              the scores of tile i + 1 are issued before it waits for the softmax of tile i;
//   warps 2-5  the softmax, one thread per row (a warp owns the tensor-memory lanes of quadrant
//              warp % 4): the thread reads its row of 64 scores out of tensor memory, masks
//              (causal, window, length), keeps the running maximum and sum in float, and writes
//              P as packed bfloat16 back into tensor memory over the first 32 columns of the
//              score buffer it has just read: the second product takes its A operand from there.
//              The maximum that the exponents are taken against only moves when a tile's maximum
//              exceeds it by more than 8 (in units of log2): P stays below 2^8, the row's sum
//              and O keep their scale, and O (in tensor memory) is rescaled only then.
// With few CTAs for the GPU (a prompt or two) the step waits for the CTA with the most keys, so the
// kernel then runs as clusters of two: CTA c of a cluster takes the key tiles c, c + 2, c + 4, ... of
// the same 128 rows on an SM of its own, the second writes its maximum, sum and unnormalised output
// per row into the first one's shared memory, and after a cluster barrier the first joins the two.
// A score buffer is overwritten by the scores two tiles on; warp 1 issues that product only when
// the second product of this tile has completed (products into different accumulators are not
// ordered by their issue).
// The softmax is the chain that bounds a tile: its 8,192 exponentials alone take 512 cycles of
// the SM's special-function units (16 a cycle), the two products about 256.
//
// Formulas: kelpie-models/kelpie_models/kernels/ops/paged_attention.py:160-240. Every wait on an
// mbarrier is bounded; on time-out the thread records an error code, the roles leave their
// loops, tensor memory is freed and the kernel returns.
#include <cuda.h>
#include <limits.h>
#include <math.h>

#include <cstring>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tensor_maps.cuh"

namespace {

constexpr int HD = 64;
constexpr int BM = 128, BN = 64, STAGES = 3;
constexpr int THREADS = 192;
constexpr int SOFTMAX_WARPS = 4;
constexpr int Q_BYTES = BM * 128, KV_BYTES = BN * 128;
constexpr float RESCALE_STEP = 8.f;  // log2 of how far a tile's maximum may exceed the one in use
#define R2_ERR_TIMEOUT_ATTN 6

struct Params {
  bf16* out; int out_row_stride;
  long long page_stride; int page_size; int page_shift; int n_pages;
  const int32_t* block_tables; int table_width;
  const int32_t* q_start; const int32_t* seq_lens; int n_entries;
  int n_heads, n_kv_heads;
  float scale; int window;
  int box_rows;
  int* error_flag;
};

using namespace r2ptx;

// The join buffer in the first CTA's shared memory: [HD outputs, maximum, sum][128 rows] floats, so that a warp's
// accesses are consecutive.
constexpr int JOIN_BYTES = (HD + 2) * BM * 4;

template <int SPLIT>
__global__ void __launch_bounds__(THREADS)
prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;                                  // [128 rows][64 dims], swizzled
  uint8_t* k_s = q_s + Q_BYTES;                         // STAGES x [64 keys][64 dims]
  uint8_t* v_s = k_s + STAGES * KV_BYTES;               // STAGES x [64 keys][64 dims]
  float* join_s = reinterpret_cast<float*>(v_s + STAGES * KV_BYTES);   // (SPLIT > 1 only)
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + STAGES * KV_BYTES + (SPLIT > 1 ? JOIN_BYTES : 0));
  uint64_t* q_full = bars;                 // the query tile has landed
  uint64_t* kv_full = bars + 1;            // [STAGES] a stage's keys and values have landed
  uint64_t* kv_empty = kv_full + STAGES;   // [STAGES] the second product has read the stage
  uint64_t* s_ready = kv_empty + STAGES;   // [2] a score buffer holds S of its tile
  // [2] P of the tile is in tensor memory and O is rescaled (one arrival per softmax warp). One per score buffer: a warp may
  // be a tile ahead of another (the next scores exist before this tile's P is complete), and two arrivals of one warp must
  // not count for one tile; two tiles ahead it cannot be, since those scores are issued after this wait.
  uint64_t* p_ready = s_ready + 2;
  uint64_t* pv_done = p_ready + 2;         // the second product of the tile has completed
  // The last second product has completed. A barrier of its own: a wait by parity is only right
  // for a phase that is the current one or the one before, and a softmax warp that is a tile ahead
  // of the others finishes while pv_done may still be two phases back.
  uint64_t* o_done = pv_done + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 1);
  __shared__ int tile_info[5];  // entry, first row of the tile within it, the entry's first row in the batch, its rows, its length

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chain = SPLIT > 1 ? int(blockIdx.z) : 0;   // the CTA's rank in its cluster (the cluster lies along z)
  const int h = blockIdx.x;   // heads vary fastest: CTAs start in the order of their tiles, the longest of an entry first
  const int kvh = h / (p.n_heads / p.n_kv_heads);

  const uint32_t q_full_a = smem_u32(q_full), kv_full_a = smem_u32(kv_full), kv_empty_a = smem_u32(kv_empty);
  const uint32_t s_ready_a = smem_u32(s_ready), p_ready_a = smem_u32(p_ready), pv_done_a = smem_u32(pv_done), o_done_a = smem_u32(o_done);
  // Which entry and which 128 rows of it this CTA has: tiles are handed out from the end of the
  // batch (blockIdx.y counts them). Warp 0 looks through the entries 32 at a time (these read the batch, which no kernel
  // writes), while warp 1 sets up the barriers and the tensor memory.
  if (warp == 1) {
    if (lane == 0) {
      mbar_init(q_full_a, 1);
      for (int s = 0; s < STAGES; ++s) {
        mbar_init(kv_full_a + s * 8, 1);
        mbar_init(kv_empty_a + s * 8, 1);
      }
      mbar_init(s_ready_a, 1);
      mbar_init(s_ready_a + 8, 1);
      mbar_init(p_ready_a, SOFTMAX_WARPS);
      mbar_init(p_ready_a + 8, SOFTMAX_WARPS);
      mbar_init(pv_done_a, 1);
      mbar_init(o_done_a, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
    __syncwarp();
    // two score buffers and the output accumulator, 64 columns each: 256 is the power of two that holds them
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (warp == 0) {
    const int left = int(gridDim.y) - 1 - int(blockIdx.y);
    int found = -1, row0 = 0, first = 0, rows_of = 0, len_of = 0, before = 0;
    for (int e0 = 0; e0 < p.n_entries && found < 0; e0 += 32) {
      const int e = e0 + lane;
      const int a = e < p.n_entries ? p.q_start[e] : 0;
      const int rows = e < p.n_entries ? p.q_start[e + 1] - a : 0;
      const int len = e < p.n_entries ? p.seq_lens[e] : 0;
      const int tiles = (rows + BM - 1) / BM;
      int upto = tiles;  // tiles of the entries up to and including this lane's
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int other = __shfl_up_sync(0xffffffffu, upto, d);
        if (lane >= d) upto += other;
      }
      const bool hit = left >= before + upto - tiles && left < before + upto;
      const uint32_t hits = __ballot_sync(0xffffffffu, hit);
      if (hits) {
        const int src_lane = __ffs(hits) - 1;
        found = e0 + src_lane;
        row0 = (left - before - __shfl_sync(0xffffffffu, upto - tiles, src_lane)) * BM;
        first = __shfl_sync(0xffffffffu, a, src_lane);
        rows_of = __shfl_sync(0xffffffffu, rows, src_lane);
        len_of = __shfl_sync(0xffffffffu, len, src_lane);
      }
      before += __shfl_sync(0xffffffffu, upto, 31);
    }
    if (lane == 0) {
      tile_info[0] = found;
      tile_info[1] = row0;
      tile_info[2] = first;
      tile_info[3] = rows_of;
      tile_info[4] = len_of;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 128u;  // columns [0, 64) and [64, 128): scores; [128, 192): output
  // (the next kernel's trigger comes after the tensor-memory allocation: its CTAs allocate before they wait)
  pdl_launch_dependents();
  const int e = tile_info[0];
  if (e < 0) {  // the grid is sized for the most tiles that the batch's rows could make
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
    return;
  }
  const int r0 = tile_info[1];
  const int t0 = tile_info[2];
  const int n_rows = tile_info[3];
  const int seq_len = tile_info[4];
  const int start = seq_len - n_rows;           // position of the entry's first row
  const int rows_here = min(BM, n_rows - r0);
  const int pmin = start + r0, pmax = start + r0 + rows_here - 1;
  const int lo = p.window > 0 ? max(0, pmin - p.window + 1) : 0;
  const int32_t* table = p.block_tables + size_t(e) * p.table_width;
  const int j_first = lo / BN * BN;
  const int n_tiles = (pmax - j_first) / BN + 1;
  // Rows with few keys stay with the first CTA of the two: the second would cost more than it saves.
  const bool joined = SPLIT > 1 && n_tiles >= 4;
  if (SPLIT > 1 && !joined && chain != 0) {
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
    return;
  }
  // This CTA's tiles: number i of them is tile step * i + chain of the rows, keys from j_of(i) on.
  const int step = joined ? SPLIT : 1;
  const int n_mine = (n_tiles - chain + step - 1) / step;
  auto j_of = [&](int i) { return j_first + (step * i + chain) * BN; };

  // (a softmax thread's running maximum and sum, and whether its waits all came true: they outlive the role's block)
  float m_run = -INFINITY, l_run = 0.f;
  bool ok = true;
  if (joined) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");  // "this CTA runs": waited for before its shared memory is written

  if (warp == 0) {
    // ---- producer ---------------------------------------------------------------------------
    const int n_boxes = BN / p.box_rows;
    const uint32_t box_bytes = uint32_t(p.box_rows) * 128u;
    int box_page = INT_MIN;
    auto box_lookup = [&](int j0) {
      box_page = INT_MIN;
      if (lane < n_boxes) {
        const int jb = j0 + lane * p.box_rows;
        if (jb + p.box_rows - 1 >= lo && jb <= pmax) box_page = table[page_index(jb, p.page_size, p.page_shift)];
      }
    };
    if (n_mine > 0) box_lookup(j_of(0));
    pdl_wait();  // the previous kernels wrote the queries and the cache
    if (lane == 0 && n_mine > 0) {  // (a CTA without tiles asks for nothing: no copy may land after it has gone)
      mbar_expect_tx(q_full_a, Q_BYTES);
      tma_load_2d(smem_u32(q_s), &map_q, h * HD, t0 + r0, q_full_a);
    }
    uint32_t round_parity = 0;
    for (int it = 0; it < n_mine; ++it) {
      const int stage = it % STAGES;
      if (it >= STAGES && !mbar_wait(kv_empty_a + stage * 8, round_parity ^ 1u)) {
        if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_ATTN);
        break;
      }
      const int j0 = j_of(it);
      const bool mine = box_page != INT_MIN;
      const uint32_t n_boxes_here = __popc(__ballot_sync(0xffffffffu, mine));
      const uint32_t bar = kv_full_a + stage * 8;
      if (lane == 0) mbar_expect_tx(bar, 2u * n_boxes_here * box_bytes);  // with no box at all the phase completes at once
      __syncwarp();
      if (mine) {
        const int jb = j0 + lane * p.box_rows;
        const int page = (box_page < 0 || box_page >= p.n_pages) ? 0 : box_page;  // a bad entry reads the null page
        const int off = page_offset(jb, p.page_size, p.page_shift);
        const uint32_t dst = uint32_t(stage * KV_BYTES) + uint32_t(lane) * box_bytes;
        tma_load_4d(smem_u32(k_s) + dst, &map_k, 0, off, kvh, page, bar);
        tma_load_4d(smem_u32(v_s) + dst, &map_v, 0, off, kvh, page, bar);
      }
      if (it + 1 < n_mine) box_lookup(j_of(it + 1));
      if (stage == STAGES - 1) round_parity ^= 1u;
    }
  } else if (warp == 1) {
    // ---- the products: the warp runs the loop, one elected lane issues ------------------------
    // both products: M = 128, N = 64, bfloat16 in, float out; A K-major (the queries in shared memory, P in
    // tensor memory); B K-major (keys) or MN-major (values)
    const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(BN >> 3) << 17) | (uint32_t(BM >> 4) << 24);
    const uint32_t idesc_o = idesc_s | (1u << 16);
    const uint32_t q_at = (smem_u32(q_s) >> 4) & 0x3FFFu;
    const uint32_t k_at = (smem_u32(k_s) >> 4) & 0x3FFFu, v_at = (smem_u32(v_s) >> 4) & 0x3FFFu;
    const uint64_t kmajor = smem_desc(0, 16, 1024), mnmajor = smem_desc(0, BN * 128, 1024);
    ok = n_mine == 0 || mbar_wait(q_full_a, 0);
    if (!ok && lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_ATTN);
    auto scores = [&](int it) {  // S(it) = Q K(it)^T into score buffer it & 1
      const int stage = it % STAGES;
      if (!mbar_wait(kv_full_a + stage * 8, uint32_t(it / STAGES) & 1u)) {
        if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_ATTN);
        ok = false;
        return;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (elect_one()) {
        const uint32_t kt = k_at + uint32_t(stage * KV_BYTES >> 4);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          umma_bf16(tmem_base + uint32_t(it & 1) * 64u, kmajor + uint64_t(q_at + kk * 2), kmajor + uint64_t(kt + kk * 2), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(s_ready_a + uint32_t(it & 1) * 8u);
      }
      __syncwarp();
    };
    if (ok && n_mine > 0) scores(0);
    for (int it = 0; it < n_mine && ok; ++it) {
      // The scores of tile it + 1 go where P of tile it - 1 lies: that second product must have
      // completed (products into different accumulators are not ordered among themselves). It also
      // keeps pv_done at most one phase behind any softmax warp that has these scores, which is
      // what its waits by parity need.
      if (it > 0 && !mbar_wait(pv_done_a, uint32_t(it - 1) & 1u)) {
        if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_ATTN);
        break;
      }
      if (it + 1 < n_mine) scores(it + 1);  // under the softmax of tile `it`
      if (!ok) break;
      if (!mbar_wait(p_ready_a + uint32_t(it & 1) * 8u, uint32_t(it >> 1) & 1u)) {
        if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_ATTN);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (elect_one()) {
        const int stage = it % STAGES;
        const uint32_t vt = v_at + uint32_t(stage * KV_BYTES >> 4);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          // 16 keys further: 8 columns along a row of P (two to a column), 16 rows of 128 bytes in the value tile
          umma_bf16_a_tmem(tmem_o, tmem_base + uint32_t(it & 1) * 64u + uint32_t(kk * 8), mnmajor + uint64_t(vt + kk * 128), idesc_o,
                           (it > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(kv_empty_a + uint32_t(stage) * 8u);
        umma_commit(pv_done_a);
        if (it == n_mine - 1) umma_commit(o_done_a);
      }
      __syncwarp();
    }
  } else {
    // ---- softmax and output: one thread per row ------------------------------------------------
    const int q = warp & 3;                       // tensor-memory lanes [32q, 32q + 32) belong to warps with id % 4 == q
    const int row = q * 32 + lane;
    // (a row past the entry's last, whose queries are zeros, takes the last row's mask: its result is
    // finite and never stored, and its thread goes the way of the warp's other threads)
    const int pos = min(pmin + row, pmax);
    const uint32_t lane_base = tmem_base + (uint32_t(q * 32) << 16);
    const float scale2 = p.scale * 1.4426950408889634f;  // scores in units of log2(e): one exp2 per element
    // (m_run: the maximum in use; l_run: the sum against it)
    // A tile's scores are asked for while the tile before it is still being handed over (its P on the way
    // into tensor memory, the arrival at the barrier): the wait for the scores, their way into the registers
    // and the store's completion pass under one another instead of one after the other. `fetch` always
    // issues its loads (past the last tile: of a buffer that exists), so that the registers are defined on
    // one path only and nothing the compiler adds reads them before the wait at the end of the loop's body.
    uint32_t s0[32], s1[32];
    auto fetch = [&](int it) {
      if (it < n_mine && ok && !mbar_wait(s_ready_a + uint32_t(it & 1) * 8u, uint32_t(it >> 1) & 1u)) {
        if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_ATTN);
        ok = false;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t at = lane_base + uint32_t(it & 1) * 64u;
      tmem_load32(at, s0);
      tmem_load32(at + 32u, s1);
    };
    fetch(0);
    tmem_load_wait(s0);
    tmem_tie(s1);
    for (int it = 0; it < n_mine; ++it) {
      const int j0 = j_of(it);
      const uint32_t s_at = lane_base + uint32_t(it & 1) * 64u;
      // mask in float: causal and window. Key c of the tile is seen if lo_c <= c <= hi (plain predicate
      // logic on two registers: written with && and || over the position this loop took 1,300 cycles a tile).
      const int hi = pos - j0;
      const int lo_c = p.window > 0 ? pos - p.window + 1 - j0 : 0;
      if (hi < BN - 1 || lo_c > 0) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const bool seen_a = (c <= hi) & (c >= lo_c);
          const bool seen_b = (c + 32 <= hi) & (c + 32 >= lo_c);
          s0[c] = seen_a ? s0[c] : __float_as_uint(-INFINITY);
          s1[c] = seen_b ? s1[c] : __float_as_uint(-INFINITY);
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains: the maximum's latency, not its count, is what costs
#pragma unroll
      for (int c = 0; c < 32; ++c) mx4[c & 3] = max3(mx4[c & 3], __uint_as_float(s0[c]), __uint_as_float(s1[c]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // The maximum in use moves only when this tile's exceeds it by more than the step.
      const float m_tile = mx * scale2;
      const bool grow = m_tile > m_run + RESCALE_STEP || (m_run == -INFINITY && m_tile > -INFINITY);
      const float m_new = grow ? m_tile : m_run;
      const float base = m_new == -INFINITY ? 0.f : m_new;  // a row that has seen no key yet
      const float corr = grow ? fast_exp2(m_run - base) : 1.f;
      float sum_a = 0.f, sum_b = 0.f;
      uint32_t pk[32];  // the row of P, two bfloat16 to a word: keys 2w and 2w + 1
#pragma unroll
      for (int w = 0; w < 16; ++w) {
        const float a0 = fast_exp2(fmaf(__uint_as_float(s0[2 * w]), scale2, -base));
        const float a1 = fast_exp2(fmaf(__uint_as_float(s0[2 * w + 1]), scale2, -base));
        const float b0 = fast_exp2(fmaf(__uint_as_float(s1[2 * w]), scale2, -base));
        const float b1 = fast_exp2(fmaf(__uint_as_float(s1[2 * w + 1]), scale2, -base));
        sum_a += a0 + a1;
        sum_b += b0 + b1;
        pk[w] = pack_bf16(a0, a1);
        pk[16 + w] = pack_bf16(b0, b1);
      }
      l_run = l_run * corr + (sum_a + sum_b);
      m_run = m_new;
      if (it > 0 && __any_sync(0xffffffffu, grow)) {
        // O times the correction, once the product of the previous tile has completed (the warp
        // decides together: every lane's tensor-memory access is one instruction)
        if (ok && !mbar_wait(pv_done_a, uint32_t(it - 1) & 1u)) {
          if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_ATTN);
          ok = false;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int part = 0; part < 2; ++part) {
          uint32_t o[32];
          tmem_load32(lane_base + 128u + uint32_t(part * 32), o);
          tmem_load_wait(o);
#pragma unroll
          for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * corr);
          tmem_store32(lane_base + 128u + uint32_t(part * 32), o);
        }
      }
      tmem_store32(s_at, pk);  // over the scores this thread has read
      fetch(it + 1);           // (the registers of the scores are free)
      if (j0 < lo || j0 + BN - 1 > pmax) {
        // Keys of this tile outside those that any row may see were not copied, or hold whatever
        // their slots held: their p is 0, but the product multiplies, so their value rows must
        // be finite. They are set to zero (the stage has landed: its scores exist).
        const int j = j0 + row;
        if (row < BN && (j < lo || j > pmax)) {
          const uint32_t dst = smem_u32(v_s) + uint32_t((it % STAGES) * KV_BYTES + row * 128);
#pragma unroll
          for (int c = 0; c < 8; ++c) asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst + c * 16), "r"(0u) : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the zeroed rows are read by the tensor core
      }
      tmem_store_wait();
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready_a + uint32_t(it & 1) * 8u);
      tmem_load_wait(s0);  // the next tile's scores
      tmem_tie(s1);
    }
    // this CTA's last product has completed
    if (ok && n_mine > 0 && !mbar_wait(o_done_a, 0)) {
      if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_ATTN);
      ok = false;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }

  if (joined) {
    __syncwarp();
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // the other CTA runs
    if (warp >= 2 && chain != 0) {
      // the second CTA's row: 64 unnormalised outputs, maximum and sum into the first CTA's join buffer
      const int q = warp & 3, row = q * 32 + lane;
      const uint32_t lane_base = tmem_base + (uint32_t(q * 32) << 16);
      uint32_t remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(join_s)), "r"(0));
      remote += uint32_t(row) * 4u;
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        uint32_t o[32];
        tmem_load32(lane_base + 128u + uint32_t(part * 32), o);
        tmem_load_wait(o);
#pragma unroll
        for (int c = 0; c < 32; ++c) asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(remote + uint32_t((part * 32 + c) * BM * 4)), "r"(o[c]) : "memory");
      }
      asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(remote + uint32_t(HD * BM * 4)), "r"(__float_as_uint(m_run)) : "memory");
      asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(remote + uint32_t((HD + 1) * BM * 4)), "r"(__float_as_uint(l_run)) : "memory");
    }
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }

  if (warp >= 2 && chain == 0) {
    // ---- the output rows: (O of this CTA and of the other one, each against its own maximum) / the joint sum ----
    const int q = warp & 3, row = q * 32 + lane;
    const uint32_t lane_base = tmem_base + (uint32_t(q * 32) << 16);
    float w_mine = 1.f, w_other = 0.f, l_all = l_run;
    if (joined) {
      const float m_other = join_s[HD * BM + row], l_other = join_s[(HD + 1) * BM + row];
      const float m_all = fmaxf(m_run, m_other);
      const float base = m_all == -INFINITY ? 0.f : m_all;
      w_mine = fast_exp2(m_run - base);
      w_other = fast_exp2(m_other - base);
      l_all = l_run * w_mine + l_other * w_other;
    }
    const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
    w_mine *= inv;
    w_other *= inv;
    // The row goes through the query tile's shared memory (every product that read it has
    // completed), so that the warp's stores to global memory are whole 128-byte rows.
    const uint32_t o_row = smem_u32(q_s) + uint32_t(row * 128);
#pragma unroll
    for (int part = 0; part < 2; ++part) {
      uint32_t o[32];
      tmem_load32(lane_base + 128u + uint32_t(part * 32), o);
      tmem_load_wait(o);
      float r[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        r[c] = __uint_as_float(o[c]) * w_mine;
        if (joined) r[c] = fmaf(join_s[(part * 32 + c) * BM + row], w_other, r[c]);
      }
#pragma unroll
      for (int c8 = 0; c8 < 4; ++c8) {
        const uint32_t w0 = pack_bf16(r[c8 * 8], r[c8 * 8 + 1]);
        const uint32_t w1 = pack_bf16(r[c8 * 8 + 2], r[c8 * 8 + 3]);
        const uint32_t w2 = pack_bf16(r[c8 * 8 + 4], r[c8 * 8 + 5]);
        const uint32_t w3 = pack_bf16(r[c8 * 8 + 6], r[c8 * 8 + 7]);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(o_row + uint32_t(((part * 4 + c8) ^ (row & 7)) << 4)), "r"(w0), "r"(w1),
                     "r"(w2), "r"(w3) : "memory");
      }
    }
    __syncwarp();
    if (ok) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {  // four rows of the warp's 32 at a time, eight lanes to a row
        const int r = q * 32 + i * 4 + (lane >> 3), piece = lane & 7;
        if (r < rows_here) {
          uint4 w;
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w)
                       : "r"(smem_u32(q_s) + uint32_t(r * 128 + ((piece ^ (r & 7)) << 4))));
          *reinterpret_cast<uint4*>(p.out + size_t(t0 + r0 + r) * p.out_row_stride + size_t(h) * HD + piece * 8) = w;
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
  }
}

// ---- host side ------------------------------------------------------------------------------

// The queries [rows][heads * 64] (row stride in elements), boxes of 128 rows of one head.
bool query_map(CUtensorMap* out, const void* base, long long rows, long long row_stride, int n_heads) {
  cuuint64_t dims[2] = {cuuint64_t(n_heads) * HD, cuuint64_t(rows)};
  cuuint64_t strides[1] = {cuuint64_t(row_stride) * 2};
  cuuint32_t box[2] = {cuuint32_t(HD), cuuint32_t(BM)};
  return r2::cached_bf16_map(out, r2::MapKey{base, rows, row_stride, n_heads, -1, 0, 0}, 2, dims, strides, box);
}

}  // namespace

// q [n_rows, n_heads * 64] bfloat16 (row stride in elements), out likewise; n_tiles: at least the
// sum over entries of ceil(rows / 128) (more is harmless: the CTAs beyond find no tile).
// R2_UNSUPPORTED for what this kernel does not take (page sizes other than 8, 16, 32 or multiples
// of 64; rows that are no multiple of 16 bytes): the caller then uses the mma.sync kernel.
extern "C" int r2_attention_prefill_tc(const void* q, int q_row_stride, int n_rows, void* out, int out_row_stride, const void* k_cache,
                                       const void* v_cache, long long page_stride, int page_size, int n_pages,
                                       const int32_t* block_tables, int table_width, const int32_t* q_start,
                                       const int32_t* seq_lens, int n_entries, int n_tiles, int n_heads, int n_kv_heads,
                                       float scale, int window, int* error_flag, cudaStream_t stream) {
  if (n_entries <= 0 || n_tiles <= 0 || n_rows <= 0) return R2_OK;
  if (n_heads < 1 || n_kv_heads < 1 || n_heads % n_kv_heads != 0 || page_size < 1 || window < 0) return R2_BAD_SHAPE;
  const bool page_fits = page_size == 8 || page_size == 16 || page_size == 32 || page_size % 64 == 0;
  if (!page_fits || error_flag == nullptr || !(scale > 0.f)) return R2_UNSUPPORTED;
  if (page_stride % 8 != 0 || q_row_stride % 8 != 0 || out_row_stride % 8 != 0 || (reinterpret_cast<uintptr_t>(k_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(v_cache) & 15) || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) {
    return R2_UNSUPPORTED;
  }
  Params p;
  p.out = (bf16*)out; p.out_row_stride = out_row_stride;
  p.page_stride = page_stride; p.page_size = page_size; p.page_shift = page_shift_of(page_size); p.n_pages = n_pages;
  p.block_tables = block_tables; p.table_width = table_width;
  p.q_start = q_start; p.seq_lens = seq_lens; p.n_entries = n_entries;
  p.n_heads = n_heads; p.n_kv_heads = n_kv_heads;
  p.scale = scale; p.window = window;
  p.box_rows = page_size < 64 ? page_size : 64;
  p.error_flag = error_flag;
  CUtensorMap mq, mk, mv;
  if (!query_map(&mq, q, n_rows, q_row_stride, n_heads) ||
      !r2::page_map(&mk, k_cache, page_stride, page_size, n_kv_heads, n_pages, p.box_rows, HD) ||
      !r2::page_map(&mv, v_cache, page_stride, page_size, n_kv_heads, n_pages, p.box_rows, HD)) {
    return R2_UNSUPPORTED;
  }
  if (n_tiles > 65535) return R2_UNSUPPORTED;
  static bool configured = false;
  static int n_sms = 0;
  const size_t smem_one = 1024 + Q_BYTES + 2 * STAGES * size_t(KV_BYTES) + 16 * 8 + 16, smem_two = smem_one + JOIN_BYTES;
  if (!configured) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return R2_UNSUPPORTED;
    cudaError_t e = cudaFuncSetAttribute(prefill_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 120 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(prefill_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_two));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(prefill_tc_kernel<1>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(prefill_tc_kernel<2>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e != cudaSuccess) return int(e);
    configured = true;
  }
  // How many CTAs have rows: about one per 128 rows, and at least one per entry (`n_tiles` is only an upper
  // bound). With fewer than one per SM (a single prompt or a portion of one) the step waits for the CTA with
  // the most keys while SMs stand idle: pairs of CTAs then share the keys of each 128 rows (1 x 1,024 tokens
  // x 12 heads: 11.9 us against 14.4; at 2 x 1,024, with twice the CTAs, 16.6 against 14.9, so not there).
  const long busy = long(n_rows / BM > n_entries ? n_rows / BM : n_entries) * n_heads;
  if (busy <= n_sms) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(n_heads, n_tiles, 2);
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = smem_two;
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 2;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = (g_r2_pdl && !t_r2_plain_order) ? 2 : 1;
    cudaLaunchKernelEx(&config, prefill_tc_kernel<2>, mq, mk, mv, p);  // a failure shows in launch_status()
  } else {
    // Two CTAs share an SM's special-function units and each runs slower for it. With many CTAs that is the
    // better trade (one CTA's softmax under the other's products); with fewer than two per SM the step waits
    // for the CTA with the most keys, which then should have an SM to itself: the CTA asks for more than half
    // an SM's shared memory, and the ones that do not fit at first start as the short ones end.
    const size_t smem = busy <= 2L * n_sms ? size_t(120) * 1024 : smem_one;
    r2_launch(prefill_tc_kernel<1>, dim3(n_heads, n_tiles), dim3(THREADS), smem, stream, mq, mk, mv, p);
  }
  return launch_status();
}
