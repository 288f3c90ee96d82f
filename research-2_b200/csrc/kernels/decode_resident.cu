// A decode step's layers as ONE kernel whose CTAs stay resident on all SMs.
//
// For a batch in which every row is one new token (up to 64 rows) a layer is five dependent
// products and attention over a few megabytes of weights: as kernels of their own each sits on
// a floor of several microseconds (launch, first loads, a cluster exchange) that is many times
// the time its bytes take. Here one CTA per SM runs all layers; a layer is five phases,
//
//   A  LayerNorm, q/k/v product + bias                      -> qkv (bfloat16)
//   B  attention over the paged cache, new key/value written -> mixed (bfloat16)
//   C  output product + bias + residual                      -> x (float32, in place)
//   D  LayerNorm, first feed-forward product + bias + act    -> hidden (bfloat16)
//   E  second feed-forward product + bias + residual         -> x
//
// separated by grid barriers (an arrival counter in global memory; every wait is bounded and a
// wait that runs out records R2_ERR_TIMEOUT_GRID in the error word, after which every CTA
// leaves). All CTAs are resident at once: the grid is what the occupancy query says fits.
//
// Products: the batch is small, so the weights are the 16-row side of mma.sync m16n8k16 and the
// tokens its 8 columns. Weights are stored a second time in the order in which a warp's lanes
// hold an operand tile (`pack`: [feature tile][k tile][lane][8 values]), so a tile is one
// 16-byte load per lane straight into the operand registers, 512 contiguous bytes per warp. A
// unit of work is 16 output features over all of k; a CTA's eight warps take the k tiles of a
// unit in turn and their sums are added in warp order in shared memory. Every sum has a fixed
// order: a row's result does not depend on the batch around it. What a phase needs and nothing
// in the step changes (its first weight tiles, its bias, the LayerNorm's gain and shift, the
// residual values it will add to, attention's page lookups) is requested BEFORE the barrier in
// front of it is waited on, so that after the barrier a phase is one round trip for its input
// rows, the products, and its stores. Weights travel in items of 48 k tiles (24 KB), each ONE bulk
// copy (cp.async.bulk, completion counted in bytes on an mbarrier) into a ring in shared memory;
// the LayerNorm's gain and shift and the bfloat16 input rows come the same way.
//
// Attention: a CTA takes a (row, kv head) pair at a time and its eight warps an eighth of the
// pair's keys each: 32-key tiles by 16-byte asynchronous copies straight into padded rows of
// shared memory (two tiles in flight per warp for head sizes up to 64), scores and outputs by
// mma.sync with the group's query heads as rows, online softmax in float, the warps' results
// merged in warp order in shared memory. The newest key's rows and cache slot are asked for at the
// phase's start by the warp whose keys end with them.
//
// Everything that one CTA writes and another reads inside the kernel (x, qkv, mixed, hidden,
// partial sums) is read with loads that bypass the L1.
//
// Formulas: kelpie-models/kelpie_models/models/torch/gpt2.py:80-131 (the layer),
// kernels/ops/paged_attention.py:160-240 (attention). HEAD_DIM is a compile-time constant.
#include <math.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif

#define R2_ERR_TIMEOUT_GRID 7

extern "C" {

// One layer's weights and constants (device pointers), as the launcher reads them from an
// array in device memory.
struct R2ResidentLayer {
  const void* w_qkv;   // packed [ (H + 2 Hkv) * hd / 16 ][ D / 16 ][32][8] bfloat16
  const void* w_out;   // packed [ D / 16 ][ H * hd / 16 ][32][8]
  const void* w_fc;    // packed [ F / 16 ][ D / 16 ][32][8]
  const void* w_pr;    // packed [ D / 16 ][ F / 16 ][32][8]
  const float* b_qkv; const float* b_out; const float* b_fc; const float* b_pr;
  const float* ln1_g; const float* ln1_b; const float* ln2_g; const float* ln2_b;
  void* k_cache; void* v_cache;   // the layer's member of the paged cache
  long long page_stride;          // elements between pages of that member's group
  int group;                      // the cache group whose block tables and slots the layer uses
  int page_size, n_pages, window;
  float scale, eps1, eps2;
  int act;
};

#define R2_RESIDENT_MAX_GROUPS 4

struct R2ResidentShape {
  int n_layers, width, inner, n_heads, n_kv_heads;  // width D, inner F; head size is the library's
  int n_rows;                                       // 1..64
};

struct R2ResidentBuffers {
  float* x;            // [rows, D] float32: the residual stream, in and out
  void* qkv;           // [rows, (H + 2 Hkv) * hd] bfloat16
  void* mixed;         // [rows, H * hd] bfloat16
  void* hidden;        // [rows, F] bfloat16
  unsigned* barrier;   // [2]: arrivals at the grid barrier, and CTAs that have left; zero between launches
  int* error_flag;
  const int32_t* positions; const int32_t* seq_lens;
  const int32_t* block_tables[R2_RESIDENT_MAX_GROUPS];  // per cache group [rows, table_width]
  const int32_t* slot_mapping[R2_RESIDENT_MAX_GROUPS];  // per cache group [rows]
  int table_width[R2_RESIDENT_MAX_GROUPS];
  // Profiling hook, normally null: the nanosecond clock at the kernel's start and after every phase and
  // barrier of every layer (n = 1 + 10 * layers points), as three arrays of n values: CTA 0's, the
  // earliest CTA's (to be filled with a large value beforehand) and the latest CTA's (zeros beforehand).
  long long* stamps;
};

}  // extern "C"

namespace {

constexpr int HD = HEAD_DIM;
constexpr int WARPS = 8, THREADS = WARPS * 32;
constexpr int MAX_ROWS = 64;
constexpr int VECS = HD / 8;                 // 16-byte pieces of a key row
constexpr int ROW_BYTES = HD * 2 + 16;       // a key's row in shared memory, padded against bank conflicts
constexpr int NBUF = HD <= 64 ? 2 : 1;       // key/value tiles in flight per warp
constexpr int ATTN_SMEM = WARPS * NBUF * 2 * 32 * ROW_BYTES;
constexpr uint32_t SPIN_LIMIT = 1u << 22;
constexpr int SMEM_LIMIT = 227 * 1024;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 128, "the resident kernel takes head sizes in steps of 16 up to 128");

constexpr int WKT = 48;                      // k tiles of one weight item
constexpr int WITEM = WKT * 512;             // its bytes
constexpr int LN_MAX_K = 2048;               // widest row that the LayerNorm inside holds in registers
constexpr int LNP_BYTES = 2 * LN_MAX_K * 4;  // gain and shift in shared memory
__host__ __device__ constexpr int max2(int a, int b) { return a > b ? a : b; }
// By token tiles NT (8 rows each): slots of the weight ring, and k elements of the input rows that
// shared memory holds at a time.
__host__ __device__ constexpr int w_slots(int nt) { return nt == 8 ? 2 : 4; }
__host__ __device__ constexpr int chunk_k(int nt) { return nt == 1 ? 3072 : 6144 / nt; }
__host__ __device__ constexpr int stage_bytes(int nt) { return nt * 8 * (chunk_k(nt) + 8) * 2; }
__host__ __device__ constexpr int red_bytes(int nt) { return WARPS * nt * 32 * 16; }
__host__ __device__ constexpr int merge_bytes() { return WARPS * 8 * (HD + 2) * 4; }  // the warps' attention results
// Shared memory of the product phases: [weight slot 0][input rows][warps' sums][gain, shift][weight
// slots 1 ...]. Attention's key/value tiles lie over it from 0, the warps' attention results behind them.
__host__ __device__ constexpr int hs_off(int) { return WITEM; }
__host__ __device__ constexpr int red_off(int nt) { return hs_off(nt) + stage_bytes(nt); }
__host__ __device__ constexpr int lnp_off(int nt) { return red_off(nt) + red_bytes(nt); }
__host__ __device__ constexpr int slot_off(int nt, int s) { return s == 0 ? 0 : lnp_off(nt) + LNP_BYTES + (s - 1) * WITEM; }
__host__ __device__ constexpr int merge_off(int) { return ATTN_SMEM; }
__host__ __device__ constexpr int total_smem(int nt) { return max2(slot_off(nt, w_slots(nt)), ATTN_SMEM + merge_bytes()); }
static_assert(total_smem(1) <= SMEM_LIMIT && total_smem(2) <= SMEM_LIMIT && total_smem(4) <= SMEM_LIMIT && total_smem(8) <= SMEM_LIMIT,
              "the kernel's shared memory must fit an SM's");

struct Params {
  const R2ResidentLayer* layers;
  R2ResidentShape s;
  R2ResidentBuffers b;
  int page_shift;           // log2 of the page size where all groups share a power of two; else -1
};

// One product of a phase.
struct Gemm {
  const uint4* w; const float* bias;
  int K, N, kt_total, n_tiles;
  int ln;                                   // 1: the input is LayerNorm(x); 0: bfloat16 rows
  const float* ln_g; const float* ln_b; float eps;
  const bf16* in; int in_stride;            // bfloat16 input rows
  bf16* out; int out_stride; int act;       // residual == 0: bfloat16 output with activation
  int residual;                             // 1: x += result
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// The grid barrier in two halves, so that what a CTA can do for the phase ahead without the other
// CTAs' results (requesting weights, walking index chains) runs while the others arrive. `arrive`
// releases what this CTA's threads wrote in the phase behind it.
__device__ __forceinline__ void barrier_arrive(const Params& p) {
  __syncthreads();
  if (threadIdx.x == 0) asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p.b.barrier), "r"(1u) : "memory");
}
// Waits until `target` arrivals have been counted. False if the wait ran out or a kernel has recorded
// an error: the caller leaves.
__device__ bool barrier_wait(const Params& p, unsigned target, int* ok_s) {
  if (threadIdx.x == 0) {
    int ok = 0;
    for (uint32_t spin = 0; spin < SPIN_LIMIT; ++spin) {
      if (ld_acquire(p.b.barrier) >= target) {
        ok = 1;
        break;
      }
      if (spin > 256) __nanosleep(32);
      if ((spin & 1023u) == 1023u && *reinterpret_cast<volatile int*>(p.b.error_flag) != 0) break;
    }
    if (!ok) atomicMax(p.b.error_flag, R2_ERR_TIMEOUT_GRID);
    *ok_s = ok;
  }
  __syncthreads();
  return *ok_s != 0;
}

// One contiguous piece of global memory into shared memory; its bytes are counted on `bar`.
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// The mbarriers of the product phases: one per weight slot, one for gain and shift, one for the rows.
constexpr int MAX_SLOTS = 4, BAR_LNP = MAX_SLOTS, BAR_ROWS = MAX_SLOTS + 1, N_BARS = MAX_SLOTS + 2;
struct Bars {
  uint64_t* bar;      // N_BARS mbarriers in shared memory
  uint32_t phases;    // bit b: the parity that the next wait on barrier b takes (the same in every thread)
  int* error_flag;
  __device__ __forceinline__ uint32_t at(int b) const { return r2ptx::smem_u32(bar + b); }
  // every thread of the CTA waits; false after the poll limit (recorded)
  __device__ __forceinline__ bool wait(int b) {
    const bool ok = r2ptx::mbar_wait(at(b), (phases >> b) & 1u);
    phases ^= 1u << b;
    if (!ok) atomicMax(error_flag, R2_ERR_TIMEOUT_GRID);
    return ok;
  }
};

// A warp's share of attention: of a (row, kv head) pair the keys' slice number `warp` of WARPS slices.
struct Unit {
  int kvh, t, pos, last, first, tile_begin, tile_end, tile_of_new;
};
__device__ __forceinline__ Unit unit_of(const Params& p, const R2ResidentLayer& L, int pair) {
  const int warp = threadIdx.x >> 5;
  Unit un;
  un.kvh = pair % p.s.n_kv_heads;
  un.t = pair / p.s.n_kv_heads;
  un.pos = p.b.positions[un.t];
  const int seq_len = p.b.seq_lens[un.t];
  un.last = un.pos < seq_len - 1 ? un.pos : seq_len - 1;
  un.first = L.window > 0 ? (un.pos - L.window + 1 > 0 ? un.pos - L.window + 1 : 0) : 0;
  const int tiles = (un.last - un.first + 1 + 31) / 32;
  un.tile_begin = warp * tiles / WARPS;        // the tiles in eight runs whose lengths differ by one at most
  un.tile_end = (warp + 1) * tiles / WARPS;
  un.tile_of_new = un.pos == un.last ? (un.pos - un.first) / 32 : -1;
  return un;
}
// lane r finds key r of the tile in the cache: an element offset from the cache's start that holds for
// every layer of the cache group (-1 past the last key, and for the newest key, whose row comes from this
// step's q/k/v product instead)
__device__ __forceinline__ long long key_row(const Params& p, const R2ResidentLayer& L, const Unit& un, int tile) {
  const int lane = threadIdx.x & 31;
  const int j = un.first + tile * 32 + lane;
  if (j > un.last || (tile == un.tile_of_new && j == un.pos)) return -1;
  const int32_t* table = p.b.block_tables[L.group] + size_t(un.t) * p.b.table_width[L.group];
  int page = table[page_index(j, L.page_size, p.page_shift)];
  page = (page < 0 || page >= L.n_pages) ? 0 : page;
  return (long long)(size_t(page) * L.page_stride + size_t(un.kvh) * L.page_size * HD + size_t(page_offset(j, L.page_size, p.page_shift)) * HD);
}
// piece c of row `row` of a tile in shared memory
__device__ __forceinline__ uint32_t piece(int row, int c) { return uint32_t(row * ROW_BYTES + (c << 4)); }

// rows of the tile that come from the cache: the keys up to the last one, the newest key apart (its row
// comes from this step's q/k/v product and is put in place once the tile has landed)
__device__ __forceinline__ int cache_rows(const Unit& un, int tile) {
  const int j0 = un.first + tile * 32;
  const int upto = tile == un.tile_of_new ? un.pos - 1 : un.last;
  const int n = upto - j0 + 1;
  return n < 0 ? 0 : (n > 32 ? 32 : n);
}

// Requests a tile's key and value rows from the cache into the warp's buffer `buf`, straight into the padded
// rows that ldmatrix reads without bank conflicts: 16-byte asynchronous copies, a row's pieces by neighbouring
// lanes (every instruction of the warp fetches whole 128-byte lines), zeros for the rows past the last key and
// for the newest key's. Lane r has found row r's place in the cache (`at`); one commit group per tile.
// (One bulk copy per run of keys in a page, landing densely and spread to the padded rows afterwards, cost the
// warp 1,000 cycles to issue per tile and another 1,000 to spread.)
__device__ __forceinline__ void copy_tile(const R2ResidentLayer& L, const Unit& un, uint8_t* my_smem, int tile, int buf, long long at) {
  const int lane = threadIdx.x & 31;
  constexpr int RPI = 32 / VECS;    // rows that one warp-wide 16-byte access covers
  constexpr int TURNS = 32 / RPI;
  const bf16* k_cache = reinterpret_cast<const bf16*>(L.k_cache);
  const bf16* v_cache = reinterpret_cast<const bf16*>(L.v_cache);
  const uint32_t kd = smem_u32(my_smem + (size_t(buf) * 2 + 0) * 32 * ROW_BYTES);
  const uint32_t vd = smem_u32(my_smem + (size_t(buf) * 2 + 1) * 32 * ROW_BYTES);
  const int n = cache_rows(un, tile);
#pragma unroll
  for (int i = 0; i < TURNS; ++i) {
    const int row = i * RPI + lane / VECS, c = lane % VECS;
    const long long from = __shfl_sync(0xffffffffu, at, row);
    const bool there = row < n && from >= 0;
    const int bytes = there ? 16 : 0;  // 0 source bytes: zeros
    const bf16* ks = there ? k_cache + from + c * 8 : k_cache;
    const bf16* vs = there ? v_cache + from + c * 8 : v_cache;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(kd + piece(row, c)), "l"(ks), "r"(bytes) : "memory");
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(vd + piece(row, c)), "l"(vs), "r"(bytes) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}
// After the tile has landed: the newest key's and value's rows, which this step's q/k/v product made and
// the warp's first lanes hold a 16-byte piece each of (`fresh`: the key's pieces, then the value's), go into
// their place.
__device__ __forceinline__ void place_newest(const Unit& un, uint8_t* my_smem, int tile, int buf, const uint4& fresh) {
  const int lane = threadIdx.x & 31;
  if (tile == un.tile_of_new && lane < 2 * VECS) {
    const int row = un.pos - (un.first + tile * 32), which = lane / VECS, c = lane % VECS;
    uint8_t* base = my_smem + (size_t(buf) * 2 + which) * 32 * ROW_BYTES;
    *reinterpret_cast<uint4*>(base + piece(row, c)) = fresh;
  }
  __syncwarp();
}

// What a warp does ahead of time for the CTA's first (row, kv head) pair: the chain of lookups (position,
// context length, block table). The batch's arrays do not change within a step and a cache group's pages
// are the same for all its layers, so the chain is walked once per group and window, while the CTA waits
// at the barrier in front of the first attention phase.
constexpr int AHEAD_TILES = 4;  // tiles whose rows are looked up ahead
struct AttnAhead {
  Unit un;
  long long at[AHEAD_TILES];
  int pair = -1;           // -1: the CTA has no pair
  int group = -1, window = -1;
};
__device__ __forceinline__ void attention_lookups(const Params& p, const R2ResidentLayer& L, AttnAhead& ahead) {
  if (int(blockIdx.x) >= p.s.n_rows * p.s.n_kv_heads) {
    ahead.pair = -1;
    return;
  }
  if (ahead.pair < 0 || ahead.group != L.group || ahead.window != L.window) {
    ahead.pair = blockIdx.x;
    ahead.group = L.group;
    ahead.window = L.window;
    ahead.un = unit_of(p, L, ahead.pair);
#pragma unroll
    for (int i = 0; i < AHEAD_TILES; ++i) {
      ahead.at[i] = ahead.un.tile_begin + i < ahead.un.tile_end ? key_row(p, L, ahead.un, ahead.un.tile_begin + i) : -1;
    }
  }
}
// A CTA's work in a product, item by item: its units are the feature tiles blockIdx.x, + gridDim.x,
// ...; a unit's k tiles come in runs of `act_kt` (what shared memory holds of the input rows at a
// time; all of k where that fits) and within a run in weight items of at most WKT k tiles.
struct Item {
  int tile, kt0, n_kt;       // feature tile, first k tile, k tiles
  int act0, act_n;           // the run of input k tiles it belongs to
  bool first_of_act, first_of_unit, last_of_unit;
};
struct Walk {
  int j = 0, act0 = 0, kt0 = 0;
};
__device__ __forceinline__ bool walk_next(const Gemm& g, int act_kt, Walk& w, Item& it) {
  const int tile = blockIdx.x + w.j * gridDim.x;
  if (tile >= g.n_tiles) return false;
  const int act_end = min(g.kt_total, w.act0 + act_kt);
  it.tile = tile;
  it.kt0 = w.kt0;
  it.n_kt = min(WKT, act_end - w.kt0);
  it.act0 = w.act0;
  it.act_n = act_end - w.act0;
  it.first_of_act = w.kt0 == w.act0;
  it.first_of_unit = w.kt0 == 0;
  it.last_of_unit = false;
  w.kt0 += it.n_kt;
  if (w.kt0 >= act_end) {
    w.act0 = act_end;
    if (act_end >= g.kt_total) {
      it.last_of_unit = true;
      w.j += 1;
      w.act0 = w.kt0 = 0;
    }
  }
  return true;
}

// thread 0: one bulk copy brings the item into its slot
__device__ __forceinline__ void issue_item(const Gemm& g, const Item& it, uint8_t* slot, uint32_t bar) {
  const uint4* src = g.w + (size_t(it.tile) * g.kt_total + it.kt0) * 32;
  r2ptx::mbar_expect_tx(bar, uint32_t(it.n_kt) * 512u);
  bulk_copy(r2ptx::smem_u32(slot), src, uint32_t(it.n_kt) * 512u, bar);
}

// What a phase asks for before the barrier in front of it, and carries across it.
struct Prologue {
  Walk issue;          // the next item to request
  int issued = 0;      // items requested so far
  float bias[2][2];    // of the first two units' features gq and gq + 8 (threads that write)
  float res[2][4];     // the residual values that those units' results are added to
};

template <int NT>
__device__ __forceinline__ int act_tiles(const Gemm& g) { return g.K <= chunk_k(NT) ? g.kt_total : chunk_k(NT) / 16; }

template <int NT>
__device__ void prologue(const Params& p, const Gemm& g, Prologue& pro, Bars& bars, uint8_t* smem) {
  // the phase before has finished with shared memory: what its threads wrote there is ordered before
  // the bulk copies that overwrite it
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  pro.issue = Walk();
  pro.issued = 0;
  Item it;
  for (int s = 0; s < w_slots(NT); ++s) {
    if (!walk_next(g, act_tiles<NT>(g), pro.issue, it)) break;
    if (threadIdx.x == 0) issue_item(g, it, smem + slot_off(NT, s), bars.at(s));
    pro.issued += 1;
  }
  if (g.ln && pro.issued > 0 && threadIdx.x == 0) {
    const uint32_t dst = r2ptx::smem_u32(smem + lnp_off(NT));
    r2ptx::mbar_expect_tx(bars.at(BAR_LNP), uint32_t(g.K) * 8u);
    bulk_copy(dst, g.ln_g, uint32_t(g.K) * 4u, bars.at(BAR_LNP));
    bulk_copy(dst + LN_MAX_K * 4, g.ln_b, uint32_t(g.K) * 4u, bars.at(BAR_LNP));
  }
  const int nt = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  if (nt < NT) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int tile = blockIdx.x + j * gridDim.x;
      if (tile < g.n_tiles) {
        const int n = tile * 16 + gq;
        pro.bias[j][0] = __ldg(g.bias + n);
        pro.bias[j][1] = __ldg(g.bias + n + 8);
        if (g.residual) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int tok = nt * 8 + 2 * tq + (i & 1);
            pro.res[j][i] = tok < p.s.n_rows ? __ldcg(p.b.x + size_t(tok) * g.N + n + 8 * (i >> 1)) : 0.f;
          }
        }
      }
    }
  }
}

// LayerNorm of every row of x into shared memory as bfloat16: a warp holds a row in registers (one
// round trip), mean and biased variance in float (two passes over the registers), gain and shift
// from shared memory. Rows beyond the batch's are zeros.
template <int NT>
__device__ void ln_stage(const Params& p, const Gemm& g, bf16* hs, int ks, const float* lnp) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int C = LN_MAX_K / 256;
  for (int row = warp; row < NT * 8; row += WARPS) {
    if (row < p.s.n_rows) {
      float4 v[C][2];
      const float* xr = p.b.x + size_t(row) * g.K;
#pragma unroll
      for (int c = 0; c < C; ++c) {
        const int col = c * 256 + lane * 8;
        if (col < g.K) {
          v[c][0] = __ldcg(reinterpret_cast<const float4*>(xr + col));
          v[c][1] = __ldcg(reinterpret_cast<const float4*>(xr + col + 4));
        } else {
          v[c][0] = v[c][1] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < C; ++c) sum += ((v[c][0].x + v[c][0].y) + (v[c][0].z + v[c][0].w)) + ((v[c][1].x + v[c][1].y) + (v[c][1].z + v[c][1].w));
      const float mean = warp_sum(sum) / float(g.K);
      float sq = 0.f;
#pragma unroll
      for (int c = 0; c < C; ++c) {
        if (c * 256 + lane * 8 < g.K) {
          const float4 a = v[c][0], b = v[c][1];
          sq += (((a.x - mean) * (a.x - mean) + (a.y - mean) * (a.y - mean)) + ((a.z - mean) * (a.z - mean) + (a.w - mean) * (a.w - mean))) +
                (((b.x - mean) * (b.x - mean) + (b.y - mean) * (b.y - mean)) + ((b.z - mean) * (b.z - mean) + (b.w - mean) * (b.w - mean)));
        }
      }
      const float rstd = 1.f / sqrtf(warp_sum(sq) / float(g.K) + g.eps);
#pragma unroll
      for (int c = 0; c < C; ++c) {
        const int col = c * 256 + lane * 8;
        if (col < g.K) {
          const float4 ga = *reinterpret_cast<const float4*>(lnp + col), gb = *reinterpret_cast<const float4*>(lnp + col + 4);
          const float4 ba = *reinterpret_cast<const float4*>(lnp + LN_MAX_K + col), bb = *reinterpret_cast<const float4*>(lnp + LN_MAX_K + col + 4);
          const float4 a = v[c][0], b = v[c][1];
          uint4 packed;
          packed.x = pack_bf16((a.x - mean) * rstd * ga.x + ba.x, (a.y - mean) * rstd * ga.y + ba.y);
          packed.y = pack_bf16((a.z - mean) * rstd * ga.z + ba.z, (a.w - mean) * rstd * ga.w + ba.w);
          packed.z = pack_bf16((b.x - mean) * rstd * gb.x + bb.x, (b.y - mean) * rstd * gb.y + bb.y);
          packed.w = pack_bf16((b.z - mean) * rstd * gb.z + bb.z, (b.w - mean) * rstd * gb.w + bb.w);
          *reinterpret_cast<uint4*>(hs + size_t(row) * ks + col) = packed;
        }
      }
    } else {
      for (int col = lane * 8; col < g.K; col += 256) *reinterpret_cast<uint4*>(hs + size_t(row) * ks + col) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

// bfloat16 input rows, k in [k0, k0 + len), into shared memory: one bulk copy a row (thread 0), zeros
// for the rows beyond the batch's (all threads). Every thread then waits on the rows' barrier.
template <int NT>
__device__ bool copy_stage(const Params& p, const Gemm& g, int k0, int len, bf16* hs, int ks, Bars& bars) {
  if (threadIdx.x == 0) {
    r2ptx::mbar_expect_tx(bars.at(BAR_ROWS), uint32_t(p.s.n_rows) * uint32_t(len) * 2u);
    for (int row = 0; row < p.s.n_rows; ++row) {
      bulk_copy(r2ptx::smem_u32(hs + size_t(row) * ks), g.in + size_t(row) * g.in_stride + k0, uint32_t(len) * 2u, bars.at(BAR_ROWS));
    }
  }
  const int vecs = len / 8, spare = NT * 8 - p.s.n_rows;
  for (int i = threadIdx.x; i < spare * vecs; i += THREADS) {
    const int row = p.s.n_rows + i / vecs, c = (i % vecs) * 8;
    *reinterpret_cast<uint4*>(hs + size_t(row) * ks + c) = make_uint4(0u, 0u, 0u, 0u);
  }
  const bool ok = bars.wait(BAR_ROWS);
  __syncthreads();  // (the zeros)
  return ok;
}

// One product of a phase: all units of this CTA. `pro` is what `prologue` asked for ahead of the
// barrier. False if a bounded wait ran out.
template <int NT>
__device__ bool gemm_phase(const Params& p, const Gemm& g, Prologue& pro, Bars& bars, uint8_t* smem) {
  constexpr int KS = chunk_k(NT) + 8, R = w_slots(NT);
  bf16* hs = reinterpret_cast<bf16*>(smem + hs_off(NT));
  float4* red = reinterpret_cast<float4*>(smem + red_off(NT));
  const float* lnp = reinterpret_cast<const float*>(smem + lnp_off(NT));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  if (int(blockIdx.x) >= g.n_tiles) return true;
  const int act_kt = act_tiles<NT>(g);
  const bool whole = act_kt == g.kt_total;  // the input rows fit shared memory: staged once for all units
  bool ok = true;
  if (whole) {
    if (g.ln) {
      ok = bars.wait(BAR_LNP);
      ln_stage<NT>(p, g, hs, KS, lnp);
      __syncthreads();
    } else {
      ok = copy_stage<NT>(p, g, 0, g.K, hs, KS, bars);
    }
  }
  const uint32_t* hs32 = reinterpret_cast<const uint32_t*>(hs);
  Walk take;
  Item it;
  float acc[NT][4];
  int idx = 0, unit = 0;
  while (ok && walk_next(g, act_kt, take, it)) {
    if (!whole && it.first_of_act) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncthreads();  // the rows of the run before are no longer read
      ok = copy_stage<NT>(p, g, it.act0 * 16, it.act_n * 16, hs, KS, bars);
    }
    ok = bars.wait(idx % R) && ok;  // the item has landed
    if (it.first_of_unit) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    }
    {
      const uint4* slot = reinterpret_cast<const uint4*>(smem + slot_off(NT, idx % R));
      const int k_in_act = (it.kt0 - it.act0) * 16;
      for (int kt = warp; kt < it.n_kt; kt += WARPS) {
        const uint4 a = slot[kt * 32 + lane];
        const uint32_t* col = hs32 + (k_in_act + kt * 16 + 2 * tq) / 2;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint32_t* at = col + size_t(nt * 8 + gq) * (KS / 2);
          mma_bf16(acc[nt], a.x, a.y, a.z, a.w, at[0], at[4]);
        }
      }
    }
    if (it.last_of_unit) {
      // the eight warps' sums, added in warp order
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) red[(warp * NT + nt) * 32 + lane] = make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
      __syncthreads();
      const int nt = threadIdx.x >> 5;  // of the threads that write: token tile nt, lane as in the accumulator
      if (nt < NT) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
          const float4 part = red[(w * NT + nt) * 32 + lane];
          v[0] += part.x; v[1] += part.y; v[2] += part.z; v[3] += part.w;
        }
        // What the sums are added to: the first two units' bias and residual values came before the barrier.
        // (A third unit fetches them here, in a branch of its own: as the last arm of a selection the compiler
        // makes the loads unconditional, and every unit paid a round trip for values it already had.)
        float add[4];
        if (unit < 2) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            add[i] = unit == 0 ? pro.bias[0][i >> 1] : pro.bias[1][i >> 1];
            if (g.residual) add[i] += unit == 0 ? pro.res[0][i] : pro.res[1][i];
          }
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int n = it.tile * 16 + gq + 8 * (i >> 1), tok = nt * 8 + 2 * tq + (i & 1);
            add[i] = __ldg(g.bias + n);
            if (g.residual && tok < p.s.n_rows) add[i] += __ldcg(p.b.x + size_t(tok) * g.N + n);
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int n = it.tile * 16 + gq + 8 * (i >> 1), tok = nt * 8 + 2 * tq + (i & 1);
          if (tok < p.s.n_rows) {
            const float y = v[i] + add[i];
            if (g.residual) p.b.x[size_t(tok) * g.N + n] = y;
            else g.out[size_t(tok) * g.out_stride + n] = __float2bfloat16_rn(g.act == R2_ACT_GELU_TANH ? gelu_tanh_hw(y) : activate(y, g.act));  // (bfloat16 output: the hardware's tanh, as the tcgen05 product's epilogue)
          }
        }
      }
      unit += 1;
    }
    __syncthreads();  // the item's slot (and the sums' buffer) may be written again
    Item nx;
    if (walk_next(g, act_kt, pro.issue, nx)) {
      if (threadIdx.x == 0) issue_item(g, nx, smem + slot_off(NT, idx % R), bars.at(idx % R));
      pro.issued += 1;
    }
    idx += 1;
  }
  return ok;
}

// Attention of the layer: a CTA takes (row, kv head) pairs in turn, its warps the pair's keys in eight
// slices; the slices' results are merged in warp order in shared memory.
__device__ bool attention_phase(const Params& p, const R2ResidentLayer& L, const AttnAhead& ahead, uint8_t* smem, float* merge) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.s.n_heads / p.s.n_kv_heads;
  const int q_width = p.s.n_heads * HD, kv_width = p.s.n_kv_heads * HD, qkv_stride = q_width + 2 * kv_width;
  const bf16* qkv = reinterpret_cast<const bf16*>(p.b.qkv);
  bf16* out = reinterpret_cast<bf16*>(p.b.mixed);
  uint8_t* my_smem = smem + size_t(warp) * NBUF * 2 * 32 * ROW_BYTES;
  constexpr int KS = HD / 16, DT = HD / 8;
  const int gq = lane >> 2, tq = lane & 3;
  const int n_pairs = p.s.n_rows * p.s.n_kv_heads;
  const int page_size = L.page_size, shift = p.page_shift;
  bool ok = true;

  for (int pair = blockIdx.x; pair < n_pairs; pair += gridDim.x) {
    const bool mine = pair == ahead.pair;
    const Unit un = mine ? ahead.un : unit_of(p, L, pair);
    const int kvh = un.kvh, t = un.t, last = un.last, first = un.first;
    const int tile_begin = un.tile_begin, tile_end = un.tile_end, tile_of_new = un.tile_of_new;
    const int h0 = kvh * G;
    const size_t head_off = size_t(kvh) * page_size * HD;
    const bf16* k_new = qkv + size_t(t) * qkv_stride + q_width + size_t(kvh) * HD;
    const bf16* v_new = k_new + kv_width;
    const bool has_new = tile_of_new >= tile_begin && tile_of_new < tile_end;

    auto issue = [&](int tile, int buf) {
      const int i = tile - tile_begin;
      long long at;
      if (mine && i < AHEAD_TILES) at = i == 0 ? ahead.at[0] : i == 1 ? ahead.at[1] : i == 2 ? ahead.at[2] : ahead.at[3];
      else at = key_row(p, L, un, tile);
      copy_tile(L, un, my_smem, tile, buf, at);
    };
    if (tile_begin < tile_end) issue(tile_begin, 0);
    // The warp whose keys end with the newest one asks for its rows (a 16-byte piece a lane) and its cache
    // slot now: both are needed again at the end, where a round trip for each would be nobody's but the whole
    // phase's time. (They are first used when the tile that holds them has landed.)
    int new_slot = -1;
    uint4 fresh = make_uint4(0u, 0u, 0u, 0u);
    if (has_new) {
      new_slot = p.b.slot_mapping[L.group][t];
      if (lane < 2 * VECS) fresh = __ldcg(reinterpret_cast<const uint4*>(lane < VECS ? k_new : v_new) + lane % VECS);
    }

    uint32_t qf[KS][4];
    {
      const bf16* qa = qkv + size_t(t) * qkv_stride + size_t(h0 + gq) * HD + 2 * tq;
      const bf16* qb = qa + size_t(8) * HD;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        qf[ks][0] = gq < G ? __ldcg(reinterpret_cast<const uint32_t*>(qa + ks * 16)) : 0u;
        qf[ks][1] = gq + 8 < G ? __ldcg(reinterpret_cast<const uint32_t*>(qb + ks * 16)) : 0u;
        qf[ks][2] = gq < G ? __ldcg(reinterpret_cast<const uint32_t*>(qa + ks * 16 + 8)) : 0u;
        qf[ks][3] = gq + 8 < G ? __ldcg(reinterpret_cast<const uint32_t*>(qb + ks * 16 + 8)) : 0u;
      }
    }
    float o[DT][4], m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < DT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    int it = 0;
    for (int tile = tile_begin; tile < tile_end; ++tile, ++it) {
      const int j0 = first + tile * 32;
      const int buf = NBUF == 2 ? (it & 1) : 0;
      if (NBUF == 2 && tile + 1 < tile_end) issue(tile + 1, buf ^ 1);
      if (NBUF == 2 && tile + 1 < tile_end) asm volatile("cp.async.wait_group 1;" ::: "memory");  // this tile's rows have landed
      else asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncwarp();
      place_newest(un, my_smem, tile, buf, fresh);
      const uint32_t kt = smem_u32(my_smem + (size_t(buf) * 2 + 0) * 32 * ROW_BYTES);
      const uint32_t vt = smem_u32(my_smem + (size_t(buf) * 2 + 1) * 32 * ROW_BYTES);
      float sc[4][4];  // [8-key tile][row gq: 2 keys, row gq + 8: 2 keys]
#pragma unroll
      for (int n8 = 0; n8 < 4; ++n8) sc[n8][0] = sc[n8][1] = sc[n8][2] = sc[n8][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int np = 0; np < 2; ++np) {  // two 8-key tiles per ldmatrix
          uint32_t b0, b1, b2, b3;
          const int key = np * 16 + (lane & 7) + 8 * (lane >> 4);
          ldmatrix_x4(kt + piece(key, ks * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
          mma_bf16(sc[2 * np], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
          mma_bf16(sc[2 * np + 1], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b2, b3);
        }
      }
      // scale, mask keys past the last one, online softmax over the lane's two rows (in float)
      float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
      for (int n8 = 0; n8 < 4; ++n8) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const bool seen = j0 + n8 * 8 + 2 * tq + c <= last;
          sc[n8][c] = seen ? sc[n8][c] * L.scale : -INFINITY;
          sc[n8][2 + c] = seen ? sc[n8][2 + c] * L.scale : -INFINITY;
          mx_a = fmaxf(mx_a, sc[n8][c]);
          mx_b = fmaxf(mx_b, sc[n8][2 + c]);
        }
      }
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
      const float m_a = fmaxf(m_run[0], mx_a), m_b = fmaxf(m_run[1], mx_b);  // finite: a tile has a key that is seen
      const float corr_a = __expf(m_run[0] - m_a), corr_b = __expf(m_run[1] - m_b);
      float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
      for (int n8 = 0; n8 < 4; ++n8) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          sc[n8][c] = __expf(sc[n8][c] - m_a);
          sc[n8][2 + c] = __expf(sc[n8][2 + c] - m_b);
          sum_a += sc[n8][c];
          sum_b += sc[n8][2 + c];
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
      for (int dt = 0; dt < DT; ++dt) {
        o[dt][0] *= corr_a;
        o[dt][1] *= corr_a;
        o[dt][2] *= corr_b;
        o[dt][3] *= corr_b;
      }
      // o += p . v, 16 keys at a time (rows past the last key are zeros in shared memory and p = 0)
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const uint32_t a0 = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]), a1 = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
        const uint32_t a2 = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]), a3 = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < DT / 2; ++dp) {  // two 8-wide output tiles per ldmatrix
          uint32_t b0, b1, b2, b3;
          const int key = kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
          ldmatrix_x4_trans(vt + piece(key, dp * 2 + (lane >> 4)), b0, b1, b2, b3);
          mma_bf16(o[2 * dp], a0, a1, a2, a3, b0, b1);
          mma_bf16(o[2 * dp + 1], a0, a1, a2, a3, b2, b3);
        }
      }
      __syncwarp();  // the tile's rows have been read: its buffer may be filled again
      if (NBUF == 1 && tile + 1 < tile_end) issue(tile + 1, 0);
    }
    // this slice's result for the group's heads: lanes hold rows gq (and gq + 8), columns 8 dt + 2 tq (+ 1)
    float* mine_m = merge + size_t(warp) * 8 * (HD + 2);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int g = gq + 8 * half;
      if (g < G) {
        float* at = mine_m + g * (HD + 2);
        if (tq == 0) {
          at[0] = m_run[half];
          at[1] = l_run[half];
        }
#pragma unroll
        for (int dt = 0; dt < DT; ++dt) *reinterpret_cast<float2*>(at + 2 + dt * 8 + 2 * tq) = make_float2(o[dt][2 * half], o[dt][2 * half + 1]);
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * (HD / 2); i += THREADS) {
      const int g = i / (HD / 2), d = (i % (HD / 2)) * 2;
      float mx = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) mx = fmaxf(mx, merge[(w * 8 + g) * (HD + 2)]);
      float oa = 0.f, ob = 0.f, lsum = 0.f;
      if (mx > -INFINITY) {
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
          const float* at = merge + (w * 8 + g) * (HD + 2);
          const float c = __expf(at[0] - mx);
          oa += c * at[2 + d];
          ob += c * at[3 + d];
          lsum += c * at[1];
        }
      }
      const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
      *reinterpret_cast<uint32_t*>(out + size_t(t) * q_width + size_t(h0 + g) * HD + d) = pack_bf16(oa * inv, ob * inv);
    }
    // the newest key and value go into the cache (off the path to the output): the warp whose slice holds them
    if (has_new) {
      const int slot = new_slot;
      const int page = slot < 0 ? -1 : page_index(slot, page_size, shift);
      if (page >= 0 && page < L.n_pages && lane < 2 * VECS) {
        const size_t dst = size_t(page) * L.page_stride + head_off + size_t(page_offset(slot, page_size, shift)) * HD;
        bf16* to = reinterpret_cast<bf16*>(lane < VECS ? L.k_cache : L.v_cache) + dst;
        reinterpret_cast<uint4*>(to)[lane % VECS] = fresh;
      }
    }
    __syncthreads();  // the warps' results have been read
  }
  return ok;
}

__device__ __forceinline__ Gemm product(const Params& p, const R2ResidentLayer& L, int which) {
  const int q_width = p.s.n_heads * HD, qkv_width = q_width + 2 * p.s.n_kv_heads * HD;
  Gemm g;
  g.ln = 0; g.ln_g = nullptr; g.ln_b = nullptr; g.eps = 0.f;
  g.in = nullptr; g.in_stride = 0; g.out = nullptr; g.out_stride = 0; g.act = R2_ACT_NONE; g.residual = 0;
  if (which == 0) {         // A: LayerNorm, q/k/v
    g.w = reinterpret_cast<const uint4*>(L.w_qkv); g.bias = L.b_qkv; g.K = p.s.width; g.N = qkv_width;
    g.ln = 1; g.ln_g = L.ln1_g; g.ln_b = L.ln1_b; g.eps = L.eps1;
    g.out = reinterpret_cast<bf16*>(p.b.qkv); g.out_stride = qkv_width;
  } else if (which == 1) {  // C: output product + residual
    g.w = reinterpret_cast<const uint4*>(L.w_out); g.bias = L.b_out; g.K = q_width; g.N = p.s.width;
    g.in = reinterpret_cast<const bf16*>(p.b.mixed); g.in_stride = q_width; g.residual = 1;
  } else if (which == 2) {  // D: LayerNorm, first feed-forward product
    g.w = reinterpret_cast<const uint4*>(L.w_fc); g.bias = L.b_fc; g.K = p.s.width; g.N = p.s.inner;
    g.ln = 1; g.ln_g = L.ln2_g; g.ln_b = L.ln2_b; g.eps = L.eps2;
    g.out = reinterpret_cast<bf16*>(p.b.hidden); g.out_stride = p.s.inner; g.act = L.act;
  } else {                  // E: second feed-forward product + residual
    g.w = reinterpret_cast<const uint4*>(L.w_pr); g.bias = L.b_pr; g.K = p.s.inner; g.N = p.s.width;
    g.in = reinterpret_cast<const bf16*>(p.b.hidden); g.in_stride = p.s.inner; g.residual = 1;
  }
  g.kt_total = g.K / 16;
  g.n_tiles = g.N / 16;
  return g;
}

__device__ __forceinline__ void stamp(const Params& p, int& at) {
  if (p.b.stamps != nullptr && threadIdx.x == 0) {
    long long now;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
    const int n = 1 + 10 * p.s.n_layers;
    if (blockIdx.x == 0) p.b.stamps[at] = now;
    atomicMin(reinterpret_cast<long long*>(p.b.stamps) + n + at, now);
    atomicMax(reinterpret_cast<long long*>(p.b.stamps) + 2 * n + at, now);
  }
  ++at;
}

template <int NT>
__global__ void __launch_bounds__(THREADS, 1) resident_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ int ok_s;
  __shared__ __align__(8) uint64_t bar_s[N_BARS];
  Bars bars;
  bars.bar = bar_s;
  bars.phases = 0u;
  bars.error_flag = p.b.error_flag;
  if (threadIdx.x == 0) {
    for (int i = 0; i < N_BARS; ++i) r2ptx::mbar_init(r2ptx::smem_u32(bar_s + i), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_wait();  // x comes from the kernel before
  Prologue pro;
  AttnAhead ahead;
  unsigned target = 0;
  bool ok = true;
  int n_stamps = 0;
  Gemm g = product(p, p.layers[0], 0);
  prologue<NT>(p, g, pro, bars, smem);
  stamp(p, n_stamps);
  for (int l = 0; l < p.s.n_layers && ok; ++l) {
    const R2ResidentLayer& L = p.layers[l];
    ok = gemm_phase<NT>(p, g, pro, bars, smem);
    stamp(p, n_stamps);
    barrier_arrive(p);
    attention_lookups(p, L, ahead);
    ok = barrier_wait(p, target += gridDim.x, &ok_s) && ok;
    stamp(p, n_stamps);
    if (!ok) break;
    ok = attention_phase(p, L, ahead, smem, reinterpret_cast<float*>(smem + merge_off(NT)));
    stamp(p, n_stamps);
    for (int which = 1; which < 4 && ok; ++which) {
      barrier_arrive(p);
      g = product(p, L, which);
      prologue<NT>(p, g, pro, bars, smem);
      ok = barrier_wait(p, target += gridDim.x, &ok_s);
      stamp(p, n_stamps);
      // The last phase of the last layer occupies a third of the CTAs: the others leave now, and the kernel
      // behind this one may start on their SMs (it fetches its weights before it waits for this kernel's end).
      if (which == 3 && l + 1 == p.s.n_layers) pdl_launch_dependents();
      if (ok) ok = gemm_phase<NT>(p, g, pro, bars, smem);
      stamp(p, n_stamps);
    }
    if (ok && l + 1 < p.s.n_layers) {
      barrier_arrive(p);
      g = product(p, p.layers[l + 1], 0);
      prologue<NT>(p, g, pro, bars, smem);
      ok = barrier_wait(p, target += gridDim.x, &ok_s);
    }
    stamp(p, n_stamps);
  }
  // the CTA that leaves last puts the counters back to zero for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.b.barrier + 1, 1u) == gridDim.x - 1) {
      p.b.barrier[0] = 0u;
      p.b.barrier[1] = 0u;
    }
  }
  pdl_launch_dependents();
}

template <int NT>
int grid_for(int n_sms) {
  static int cached[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  if (cached[device] == 0) {
    if (cudaFuncSetAttribute(resident_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, total_smem(NT)) != cudaSuccess) return 0;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, resident_kernel<NT>, THREADS, total_smem(NT)) != cudaSuccess || per_sm < 1) {
      cudaGetLastError();
      return 0;
    }
    cached[device] = n_sms;  // one CTA to an SM: every CTA is resident from the start
  }
  return cached[device];
}

template <int NT>
int launch(const Params& p, int n_sms, cudaStream_t stream) {
  const int grid = grid_for<NT>(n_sms);
  if (grid < 1) return R2_UNSUPPORTED;
  r2_launch(resident_kernel<NT>, dim3(grid), dim3(THREADS), size_t(total_smem(NT)), stream, p);
  return launch_status();
}

}  // namespace

extern "C" int r2_decode_resident_head_dim(void) { return HD; }
extern "C" int r2_decode_resident_max_rows(void) { return MAX_ROWS; }

// All layers of a decode-only step. `layers` is an array of R2ResidentLayer in device memory.
// Refuses (R2_UNSUPPORTED) what the kernel does not take: more than 64 rows, widths that are no
// multiple of 16 or wider than the LayerNorm inside takes for the batch's size (2,048; 1,536 above
// 16 rows; 768 above 32), groups of more than 8 query heads per kv head.
extern "C" int r2_decode_resident(const R2ResidentLayer* layers, const R2ResidentShape* shape, const R2ResidentBuffers* buffers,
                                  int page_shift, int n_sms, cudaStream_t stream) {
  if (layers == nullptr || shape == nullptr || buffers == nullptr) return R2_BAD_SHAPE;
  const R2ResidentShape& s = *shape;
  if (s.n_rows <= 0) return R2_OK;
  if (s.n_rows > MAX_ROWS || s.n_layers < 1 || s.n_heads < 1 || s.n_kv_heads < 1 || s.n_heads % s.n_kv_heads != 0) return R2_UNSUPPORTED;
  if (s.n_heads / s.n_kv_heads > 8 || s.width % 16 != 0 || s.inner % 16 != 0) return R2_UNSUPPORTED;
  if (buffers->error_flag == nullptr || buffers->barrier == nullptr) return R2_BAD_SHAPE;
  Params p;
  p.layers = layers;
  p.s = s;
  p.b = *buffers;
  p.page_shift = page_shift;
  // the LayerNorm inside holds a row in registers and its output for all of k in shared memory
  const int nt = s.n_rows <= 8 ? 1 : s.n_rows <= 16 ? 2 : s.n_rows <= 32 ? 4 : 8;
  if (s.width > LN_MAX_K || s.width > chunk_k(nt)) return R2_UNSUPPORTED;
  if (nt == 1) return launch<1>(p, n_sms, stream);
  if (nt == 2) return launch<2>(p, n_sms, stream);
  if (nt == 4) return launch<4>(p, n_sms, stream);
  return launch<8>(p, n_sms, stream);
}
