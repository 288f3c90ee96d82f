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
// unit of work is (16 output features, a range of k); a CTA's eight warps take the k tiles of
// a unit in turn and their sums are added in warp order in shared memory. Where a product has
// fewer feature tiles than there are CTAs its k range is split over several CTAs; partial sums
// go to global memory and the CTA that arrives last at the tile's counter adds them in split
// order. Every sum has a fixed order: a row's result does not depend on the batch around it.
// The first weight tiles of the next phase are requested BEFORE the barrier is waited on:
// weights depend on nothing, so their latency runs under the barrier's.
//
// Attention: a warp takes a (row, kv head, slice of the keys) at a time: 32-key tiles through
// shared memory by 16-byte asynchronous copies (two tiles in flight per warp for head sizes up
// to 64), scores and outputs by mma.sync with the group's query heads as rows, online softmax
// in float, the slices of a (row, kv head) merged in slice order by the warp that arrives last.
//
// Everything that one CTA writes and another reads inside the kernel (x, qkv, mixed, hidden,
// partial sums) is read with loads that bypass the L1.
//
// Formulas: kelpie-models/kelpie_models/models/torch/gpt2.py:80-131 (the layer),
// kernels/ops/paged_attention.py:160-240 (attention). HEAD_DIM is a compile-time constant.
#include <math.h>

#include "common.cuh"

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
  int attn_slices;                                  // slices of the keys per (row, kv head)
};

struct R2ResidentBuffers {
  float* x;            // [rows, D] float32: the residual stream, in and out
  void* qkv;           // [rows, (H + 2 Hkv) * hd] bfloat16
  void* mixed;         // [rows, H * hd] bfloat16
  void* hidden;        // [rows, F] bfloat16
  float* partial;      // split sums of the products: [max splits][64][D]
  float* attn_o;       // [rows, H, slices, hd]
  float* attn_ml;      // [rows, H, slices, 2]
  int* tile_counters;  // [D / 16], zero between launches
  int* attn_counters;  // [rows * Hkv], zero between launches
  unsigned* barrier;   // [2]: arrivals at the grid barrier, and CTAs that have left; zero between launches
  int* error_flag;
  const int32_t* positions; const int32_t* seq_lens;
  const int32_t* block_tables[R2_RESIDENT_MAX_GROUPS];  // per cache group [rows, table_width]
  const int32_t* slot_mapping[R2_RESIDENT_MAX_GROUPS];  // per cache group [rows]
  int table_width[R2_RESIDENT_MAX_GROUPS];
  // Profiling hook, normally null: CTA 0 writes the nanosecond clock at the kernel's start and after
  // every phase and barrier of every layer (1 + 10 * layers values).
  long long* stamps;
};

}  // extern "C"

namespace {

constexpr int HD = HEAD_DIM;
constexpr int WARPS = 8, THREADS = WARPS * 32;
constexpr int RT = 8;                        // weight tiles a warp keeps in flight
constexpr int MAX_ROWS = 64;
constexpr int VECS = HD / 8;                 // 16-byte pieces of a key row
constexpr int ROW_BYTES = HD * 2 + 16;       // a key's row in shared memory, padded against bank conflicts
constexpr int NBUF = HD <= 64 ? 2 : 1;       // key/value tiles in flight per warp
constexpr int ATTN_SMEM = WARPS * NBUF * 2 * 32 * ROW_BYTES;
constexpr uint32_t SPIN_LIMIT = 1u << 22;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 128, "the resident kernel takes head sizes in steps of 16 up to 128");

// k elements of a product's input that are staged in shared memory at a time, by token tiles
__host__ __device__ constexpr int chunk_k(int nt) { return 8192 / nt; }
__host__ __device__ constexpr int stage_bytes(int nt) { return nt * 8 * (chunk_k(nt) + 8) * 2; }
__host__ __device__ constexpr int red_bytes(int nt) { return WARPS * nt * 32 * 16; }
__host__ __device__ constexpr int gemm_smem(int nt) { return stage_bytes(nt) + red_bytes(nt) + MAX_ROWS * 8; }
__host__ __device__ constexpr int total_smem(int nt) { return gemm_smem(nt) > ATTN_SMEM ? gemm_smem(nt) : ATTN_SMEM; }

struct Params {
  const R2ResidentLayer* layers;
  R2ResidentShape s;
  R2ResidentBuffers b;
  int splits_c, splits_e;   // k splits of the two products that write x
  int page_shift;           // log2 of the page size where all groups share a power of two; else -1
};

// One product of a phase.
struct Gemm {
  const uint4* w; const float* bias;
  int K, N, kt_total, n_tiles, splits, kt_per_split;
  int ln;                                   // 1: the input is LayerNorm(x); 0: bfloat16 rows
  const float* ln_g; const float* ln_b; float eps;
  const bf16* in; int in_stride;            // bfloat16 input rows
  bf16* out; int out_stride; int act;       // residual == 0: bfloat16 output with activation
  int residual;                             // 1: x += result
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ uint4 ld_weight(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
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

// Every CTA arrives and waits until `target` arrivals have been counted. False if the wait ran out
// or a kernel has recorded an error: the caller leaves.
__device__ bool grid_barrier(const Params& p, unsigned target, int* ok_s) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(p.b.barrier, 1u);
    int ok = 0;
    for (uint32_t spin = 0; spin < SPIN_LIMIT; ++spin) {
      if (ld_acquire(p.b.barrier) >= target) {
        ok = 1;
        break;
      }
      if (spin > 64) __nanosleep(32);
      if ((spin & 1023u) == 1023u && *reinterpret_cast<volatile int*>(p.b.error_flag) != 0) break;
    }
    if (!ok) atomicMax(p.b.error_flag, R2_ERR_TIMEOUT_GRID);
    __threadfence();
    *ok_s = ok;
  }
  __syncthreads();
  return *ok_s != 0;
}

// The first RT weight tiles of this warp for the unit's chunk that starts at k tile `kt0` and has
// `n_kt` k tiles; batch b holds the warp's tiles b * RT ... (the warp's i-th tile is k tile warp + 8 i).
__device__ __forceinline__ void load_batch(const Gemm& g, int tile, int kt0, int n_kt, int batch, uint4 (&wv)[RT]) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint4* base = g.w + (size_t(tile) * g.kt_total + kt0) * 32 + lane;
#pragma unroll
  for (int r = 0; r < RT; ++r) {
    const int kt = warp + WARPS * (batch * RT + r);
    wv[r] = kt < n_kt ? ld_weight(base + size_t(kt) * 32) : make_uint4(0u, 0u, 0u, 0u);
  }
}

// The unit of a product that this CTA takes first, and its first chunk: what may be requested early.
template <int NT>
__device__ __forceinline__ void prefetch(const Gemm& g, uint4 (&pre)[RT]) {
  const int u = blockIdx.x;
  if (u >= g.n_tiles * g.splits) return;
  const int tile = u / g.splits, split = u - tile * g.splits;
  const int kt_begin = split * g.kt_per_split, kt_end = min(g.kt_total, kt_begin + g.kt_per_split);
  load_batch(g, tile, kt_begin, min(chunk_k(NT) / 16, kt_end - kt_begin), 0, pre);
}

// mean and 1 / sqrt(variance + eps) of every row of x (biased variance, two passes, float)
__device__ void row_stats(const Params& p, int K, float eps, float* stats) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = warp; row < p.s.n_rows; row += WARPS) {
    const float4* xr = reinterpret_cast<const float4*>(p.b.x + size_t(row) * K);
    float sum = 0.f;
    for (int i = lane; i < K / 4; i += 32) {
      const float4 v = __ldcg(xr + i);
      sum += (v.x + v.y) + (v.z + v.w);
    }
    const float mean = warp_sum(sum) / float(K);
    float sq = 0.f;
    for (int i = lane; i < K / 4; i += 32) {
      const float4 v = __ldcg(xr + i);
      const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
      sq += (a * a + b * b) + (c * c + d * d);
    }
    const float var = warp_sum(sq) / float(K);
    if (lane == 0) {
      stats[2 * row] = mean;
      stats[2 * row + 1] = 1.f / sqrtf(var + eps);
    }
  }
}

// The product's input for k in [k0, k0 + len) as bfloat16 rows of stride `ks` in shared memory;
// rows beyond the batch's are zeros.
template <int NT>
__device__ void stage(const Params& p, const Gemm& g, int k0, int len, bf16* hs, int ks, const float* stats) {
  const int vecs = len / 8;  // 8 values per thread and turn
  for (int i = threadIdx.x; i < NT * 8 * vecs; i += THREADS) {
    const int row = i / vecs, c = (i - row * vecs) * 8;
    uint4 packed = make_uint4(0u, 0u, 0u, 0u);
    if (row < p.s.n_rows) {
      if (g.ln) {
        const float mean = stats[2 * row], rstd = stats[2 * row + 1];
        const float4* xr = reinterpret_cast<const float4*>(p.b.x + size_t(row) * g.K + k0 + c);
        const float4* gr = reinterpret_cast<const float4*>(g.ln_g + k0 + c);
        const float4* br = reinterpret_cast<const float4*>(g.ln_b + k0 + c);
        const float4 a = __ldcg(xr), b = __ldcg(xr + 1);
        const float4 ga = __ldg(gr), gb = __ldg(gr + 1), ba = __ldg(br), bb = __ldg(br + 1);
        packed.x = pack_bf16((a.x - mean) * rstd * ga.x + ba.x, (a.y - mean) * rstd * ga.y + ba.y);
        packed.y = pack_bf16((a.z - mean) * rstd * ga.z + ba.z, (a.w - mean) * rstd * ga.w + ba.w);
        packed.z = pack_bf16((b.x - mean) * rstd * gb.x + bb.x, (b.y - mean) * rstd * gb.y + bb.y);
        packed.w = pack_bf16((b.z - mean) * rstd * gb.z + bb.z, (b.w - mean) * rstd * gb.w + bb.w);
      } else {
        packed = __ldcg(reinterpret_cast<const uint4*>(g.in + size_t(row) * g.in_stride + k0 + c));
      }
    }
    *reinterpret_cast<uint4*>(hs + size_t(row) * ks + c) = packed;
  }
}

// One product of a phase, all its units that fall to this CTA. `pre` holds the first weight tiles of
// the CTA's first unit if `have_pre`.
template <int NT>
__device__ void gemm_phase(const Params& p, const Gemm& g, uint4 (&pre)[RT], bool have_pre, uint8_t* smem, int* flag_s) {
  constexpr int KC = chunk_k(NT), KS = KC + 8;
  bf16* hs = reinterpret_cast<bf16*>(smem);
  float4* red = reinterpret_cast<float4*>(smem + stage_bytes(NT));
  float* stats = reinterpret_cast<float*>(smem + stage_bytes(NT) + red_bytes(NT));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  const int n_units = g.n_tiles * g.splits;
  if (int(blockIdx.x) >= n_units) return;
  if (g.ln) row_stats(p, g.K, g.eps, stats);  // made visible by the barrier ahead of the first staging
  const uint32_t* hs32 = reinterpret_cast<const uint32_t*>(hs);
  bool first = have_pre;
  for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
    const int tile = u / g.splits, split = u - tile * g.splits;
    const int kt_begin = split * g.kt_per_split, kt_end = min(g.kt_total, kt_begin + g.kt_per_split);
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    for (int c0 = kt_begin; c0 < kt_end; c0 += KC / 16) {
      const int n_kt = min(KC / 16, kt_end - c0);
      uint4 wv[RT];
      if (first) {
#pragma unroll
        for (int r = 0; r < RT; ++r) wv[r] = pre[r];
        first = false;
      } else {
        load_batch(g, tile, c0, n_kt, 0, wv);
      }
      __syncthreads();  // the staged rows of the chunk before are no longer read
      stage<NT>(p, g, c0 * 16, n_kt * 16, hs, KS, stats);
      __syncthreads();
      const int mine = n_kt > warp ? (n_kt - warp + WARPS - 1) / WARPS : 0;  // this warp's k tiles in the chunk
      for (int b0 = 0; b0 < mine; b0 += RT) {
        uint4 nx[RT];
        if (b0 + RT < mine) load_batch(g, tile, c0, n_kt, b0 / RT + 1, nx);
#pragma unroll
        for (int r = 0; r < RT; ++r) {
          if (b0 + r < mine) {
            const int kt = warp + WARPS * (b0 + r);
            const uint32_t* col = hs32 + (kt * 16 + 2 * tq) / 2;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              const uint32_t* at = col + size_t(nt * 8 + gq) * (KS / 2);
              mma_bf16(acc[nt], wv[r].x, wv[r].y, wv[r].z, wv[r].w, at[0], at[4]);
            }
          }
        }
        if (b0 + RT < mine) {
#pragma unroll
          for (int r = 0; r < RT; ++r) wv[r] = nx[r];
        }
      }
    }
    // the eight warps' sums, added in warp order
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) red[(warp * NT + nt) * 32 + lane] = make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
    __syncthreads();
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    const int nt = threadIdx.x >> 5;  // of the threads that write: token tile nt, lane as in the accumulator
    if (nt < NT) {
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float4 part = red[(w * NT + nt) * 32 + lane];
        v[0] += part.x; v[1] += part.y; v[2] += part.z; v[3] += part.w;
      }
    }
    bool writes = nt < NT;
    if (g.splits > 1) {
      // partial sums to global memory; the CTA that arrives last at the tile adds them in split order
      if (nt < NT) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int n = tile * 16 + gq + 8 * (i >> 1), tok = nt * 8 + 2 * tq + (i & 1);
          if (tok < p.s.n_rows) p.b.partial[(size_t(split) * MAX_ROWS + tok) * g.N + n] = v[i];
        }
      }
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        const int arrived = atomicAdd(p.b.tile_counters + tile, 1);
        const int last = arrived == g.splits - 1;
        if (last) p.b.tile_counters[tile] = 0;  // ready for the next product
        *flag_s = last;
      }
      __syncthreads();
      writes = writes && *flag_s != 0;
      if (writes) {
        __threadfence();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int n = tile * 16 + gq + 8 * (i >> 1), tok = nt * 8 + 2 * tq + (i & 1);
          float sum = 0.f;
          if (tok < p.s.n_rows) {
            for (int s = 0; s < g.splits; ++s) sum += __ldcg(&p.b.partial[(size_t(s) * MAX_ROWS + tok) * g.N + n]);
          }
          v[i] = sum;
        }
      }
    }
    if (writes) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int n = tile * 16 + gq + 8 * (i >> 1), tok = nt * 8 + 2 * tq + (i & 1);
        if (tok < p.s.n_rows && n < g.N) {
          const float y = v[i] + __ldg(g.bias + n);
          if (g.residual) {
            float* xp = p.b.x + size_t(tok) * g.N + n;
            *xp = __ldcg(xp) + y;
          } else {
            g.out[size_t(tok) * g.out_stride + n] = __float2bfloat16_rn(activate(y, g.act));
          }
        }
      }
    }
  }
}

// Attention of the layer: a warp takes (row, kv head, slice) units in turn.
__device__ void attention_phase(const Params& p, const R2ResidentLayer& L, uint8_t* smem) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.s.n_heads / p.s.n_kv_heads, S = p.s.attn_slices;
  const int q_width = p.s.n_heads * HD, kv_width = p.s.n_kv_heads * HD, qkv_stride = q_width + 2 * kv_width;
  const bf16* qkv = reinterpret_cast<const bf16*>(p.b.qkv);
  const bf16* k_cache = reinterpret_cast<const bf16*>(L.k_cache);
  const bf16* v_cache = reinterpret_cast<const bf16*>(L.v_cache);
  bf16* out = reinterpret_cast<bf16*>(p.b.mixed);
  uint8_t* my_smem = smem + size_t(warp) * NBUF * 2 * 32 * ROW_BYTES;
  constexpr int KS = HD / 16, DT = HD / 8;
  const int gq = lane >> 2, tq = lane & 3;
  const int n_units = p.s.n_rows * p.s.n_kv_heads * S;
  const int page_size = L.page_size, shift = p.page_shift;

  for (int u = warp * gridDim.x + blockIdx.x; u < n_units; u += WARPS * gridDim.x) {
    const int slice = u % S, kvh = (u / S) % p.s.n_kv_heads, t = u / (S * p.s.n_kv_heads);
    const int h0 = kvh * G;
    const int pos = p.b.positions[t], seq_len = p.b.seq_lens[t];
    const int last = pos < seq_len - 1 ? pos : seq_len - 1;
    const int first = L.window > 0 ? (pos - L.window + 1 > 0 ? pos - L.window + 1 : 0) : 0;
    const int n_keys = last - first + 1;
    const int tiles = (n_keys + 31) / 32;
    const int tiles_per = (tiles + S - 1) / S;
    const int tile_begin = slice * tiles_per, tile_end = min(tiles, tile_begin + tiles_per);
    const int32_t* table = p.b.block_tables[L.group] + size_t(t) * p.b.table_width[L.group];
    const size_t head_off = size_t(kvh) * page_size * HD;
    const bf16* k_new = qkv + size_t(t) * qkv_stride + q_width + size_t(kvh) * HD;
    const bf16* v_new = k_new + kv_width;
    const int tile_of_new = pos == last ? (pos - first) / 32 : -1;

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

    // lane r finds key r of the tile: element offsets from the cache's start; the newest key's row
    // comes from this step's q/k/v product, not from the cache
    auto issue = [&](int tile, int buf) {
      const int j = first + tile * 32 + lane;
      long long my_k = -1, my_v = -1;
      if (j <= last) {
        if (tile == tile_of_new && j == pos) {
          my_k = k_new - k_cache;
          my_v = v_new - v_cache;
        } else {
          int page = table[page_index(j, page_size, shift)];
          page = (page < 0 || page >= L.n_pages) ? 0 : page;
          my_k = my_v = (long long)(size_t(page) * L.page_stride + head_off + size_t(page_offset(j, page_size, shift)) * HD);
        }
      }
      const uint32_t kd = smem_u32(my_smem + (size_t(buf) * 2 + 0) * 32 * ROW_BYTES);
      const uint32_t vd = smem_u32(my_smem + (size_t(buf) * 2 + 1) * 32 * ROW_BYTES);
#pragma unroll
      for (int i = 0; i < VECS; ++i) {
        const int f = lane + 32 * i;
        const int row = f / VECS, c = f % VECS;
        const long long ko = __shfl_sync(0xffffffffu, my_k, row);
        const long long vo = __shfl_sync(0xffffffffu, my_v, row);
        const bool valid = first + tile * 32 + row <= last;
        const int bytes = valid ? 16 : 0;  // 0 source bytes: zeros
        const bf16* ksrc = valid ? k_cache + ko + c * 8 : k_cache;
        const bf16* vsrc = valid ? v_cache + vo + c * 8 : v_cache;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(kd + row * ROW_BYTES + c * 16), "l"(ksrc), "r"(bytes) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(vd + row * ROW_BYTES + c * 16), "l"(vsrc), "r"(bytes) : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };

    if (tile_begin < tile_end) issue(tile_begin, 0);
    int it = 0;
    for (int tile = tile_begin; tile < tile_end; ++tile, ++it) {
      const int j0 = first + tile * 32;
      const int buf = NBUF == 2 ? (it & 1) : 0;
      if (tile == tile_of_new) {
        // the newest key lies in this tile: this warp also puts its key and value into the cache
        const int slot = p.b.slot_mapping[L.group][t];
        const int page = slot < 0 ? -1 : page_index(slot, page_size, shift);
        if (page >= 0 && page < L.n_pages) {
          const size_t dst = size_t(page) * L.page_stride + head_off + size_t(page_offset(slot, page_size, shift)) * HD;
          const uint32_t* ks = reinterpret_cast<const uint32_t*>(k_new);
          const uint32_t* vs = reinterpret_cast<const uint32_t*>(v_new);
          uint32_t* kd = reinterpret_cast<uint32_t*>(reinterpret_cast<bf16*>(L.k_cache) + dst);
          uint32_t* vd = reinterpret_cast<uint32_t*>(reinterpret_cast<bf16*>(L.v_cache) + dst);
          for (int i = lane; i < HD / 2; i += 32) {
            kd[i] = __ldcg(ks + i);
            vd[i] = __ldcg(vs + i);
          }
        }
      }
      if (NBUF == 2) {
        if (tile + 1 < tile_end) {
          issue(tile + 1, buf ^ 1);
          asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
          asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
      } else {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
      }
      __syncwarp();
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
          ldmatrix_x4(kt + uint32_t(key * ROW_BYTES + (ks * 2 + ((lane >> 3) & 1)) * 16), b0, b1, b2, b3);
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
          ldmatrix_x4_trans(vt + uint32_t(key * ROW_BYTES + (dp * 2 + (lane >> 4)) * 16), b0, b1, b2, b3);
          mma_bf16(o[2 * dp], a0, a1, a2, a3, b0, b1);
          mma_bf16(o[2 * dp + 1], a0, a1, a2, a3, b2, b3);
        }
      }
      __syncwarp();  // the tile's rows have been read: its buffer may be filled again
      if (NBUF == 1 && tile + 1 < tile_end) issue(tile + 1, 0);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // this slice's result for the group's heads: lanes hold rows gq (and gq + 8), columns 8 dt + 2 tq (+ 1)
    if (S == 1) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int g = gq + 8 * half;
        if (g < G) {
          const float inv = l_run[half] > 0.f ? 1.f / l_run[half] : 0.f;
          uint32_t* dst = reinterpret_cast<uint32_t*>(out + size_t(t) * q_width + size_t(h0 + g) * HD);
#pragma unroll
          for (int dt = 0; dt < DT; ++dt) dst[(dt * 8 + 2 * tq) / 2] = pack_bf16(o[dt][2 * half] * inv, o[dt][2 * half + 1] * inv);
        }
      }
      continue;
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int g = gq + 8 * half;
      if (g < G) {
        const size_t at = (size_t(t) * p.s.n_heads + h0 + g) * S + slice;
        if (tq == 0) {
          p.b.attn_ml[at * 2] = m_run[half];
          p.b.attn_ml[at * 2 + 1] = l_run[half];
        }
        float2* dst = reinterpret_cast<float2*>(p.b.attn_o + at * HD);
#pragma unroll
        for (int dt = 0; dt < DT; ++dt) dst[(dt * 8 + 2 * tq) / 2] = make_float2(o[dt][2 * half], o[dt][2 * half + 1]);
      }
    }
    // the slice that arrives last merges all of them, in slice order
    __threadfence();
    __syncwarp();
    int is_last = 0;
    if (lane == 0) {
      int* counter = p.b.attn_counters + size_t(t) * p.s.n_kv_heads + kvh;
      const int arrived = atomicAdd(counter, 1);
      is_last = arrived == S - 1;
      if (is_last) *counter = 0;  // ready for the next layer
    }
    is_last = __shfl_sync(0xffffffffu, is_last, 0);
    if (is_last) {
      __threadfence();
      for (int i = lane; i < G * (HD / 2); i += 32) {
        const int g = i / (HD / 2), d = (i % (HD / 2)) * 2;
        const size_t base = (size_t(t) * p.s.n_heads + h0 + g) * S;
        float mx = -INFINITY;
        for (int s = 0; s < S; ++s) mx = fmaxf(mx, __ldcg(&p.b.attn_ml[(base + s) * 2]));
        float oa = 0.f, ob = 0.f, lsum = 0.f;
        if (mx > -INFINITY) {
          for (int s = 0; s < S; ++s) {
            const float c = __expf(__ldcg(&p.b.attn_ml[(base + s) * 2]) - mx);
            const float2 part = __ldcg(reinterpret_cast<const float2*>(&p.b.attn_o[(base + s) * HD + d]));
            oa += c * part.x;
            ob += c * part.y;
            lsum += c * __ldcg(&p.b.attn_ml[(base + s) * 2 + 1]);
          }
        }
        const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
        *reinterpret_cast<uint32_t*>(out + size_t(t) * q_width + size_t(h0 + g) * HD + d) = pack_bf16(oa * inv, ob * inv);
      }
    }
  }
}

__device__ __forceinline__ Gemm product(const Params& p, const R2ResidentLayer& L, int which) {
  const int q_width = p.s.n_heads * HD, qkv_width = q_width + 2 * p.s.n_kv_heads * HD;
  Gemm g;
  g.ln = 0; g.ln_g = nullptr; g.ln_b = nullptr; g.eps = 0.f;
  g.in = nullptr; g.in_stride = 0; g.out = nullptr; g.out_stride = 0; g.act = R2_ACT_NONE; g.residual = 0; g.splits = 1;
  if (which == 0) {         // A: LayerNorm, q/k/v
    g.w = reinterpret_cast<const uint4*>(L.w_qkv); g.bias = L.b_qkv; g.K = p.s.width; g.N = qkv_width;
    g.ln = 1; g.ln_g = L.ln1_g; g.ln_b = L.ln1_b; g.eps = L.eps1;
    g.out = reinterpret_cast<bf16*>(p.b.qkv); g.out_stride = qkv_width;
  } else if (which == 1) {  // C: output product + residual
    g.w = reinterpret_cast<const uint4*>(L.w_out); g.bias = L.b_out; g.K = q_width; g.N = p.s.width;
    g.in = reinterpret_cast<const bf16*>(p.b.mixed); g.in_stride = q_width; g.residual = 1; g.splits = p.splits_c;
  } else if (which == 2) {  // D: LayerNorm, first feed-forward product
    g.w = reinterpret_cast<const uint4*>(L.w_fc); g.bias = L.b_fc; g.K = p.s.width; g.N = p.s.inner;
    g.ln = 1; g.ln_g = L.ln2_g; g.ln_b = L.ln2_b; g.eps = L.eps2;
    g.out = reinterpret_cast<bf16*>(p.b.hidden); g.out_stride = p.s.inner; g.act = L.act;
  } else {                  // E: second feed-forward product + residual
    g.w = reinterpret_cast<const uint4*>(L.w_pr); g.bias = L.b_pr; g.K = p.s.inner; g.N = p.s.width;
    g.in = reinterpret_cast<const bf16*>(p.b.hidden); g.in_stride = p.s.inner; g.residual = 1; g.splits = p.splits_e;
  }
  g.kt_total = g.K / 16;
  g.n_tiles = g.N / 16;
  g.kt_per_split = (g.kt_total + g.splits - 1) / g.splits;
  return g;
}

__device__ __forceinline__ void stamp(const Params& p, int& at) {
  if (p.b.stamps != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
    long long now;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
    p.b.stamps[at] = now;
  }
  ++at;
}

template <int NT>
__global__ void __launch_bounds__(THREADS, 1) resident_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ int ok_s, flag_s;
  pdl_wait();  // x comes from the kernel before
  uint4 pre[RT];
  unsigned target = 0;
  bool ok = true;
  int n_stamps = 0;
  Gemm g = product(p, p.layers[0], 0);
  prefetch<NT>(g, pre);
  stamp(p, n_stamps);
  for (int l = 0; l < p.s.n_layers && ok; ++l) {
    const R2ResidentLayer& L = p.layers[l];
    gemm_phase<NT>(p, g, pre, true, smem, &flag_s);
    stamp(p, n_stamps);
    ok = grid_barrier(p, target += gridDim.x, &ok_s);
    stamp(p, n_stamps);
    if (!ok) break;
    attention_phase(p, L, smem);
    stamp(p, n_stamps);
    for (int which = 1; which < 4 && ok; ++which) {
      g = product(p, L, which);
      prefetch<NT>(g, pre);
      ok = grid_barrier(p, target += gridDim.x, &ok_s);
      stamp(p, n_stamps);
      if (ok) gemm_phase<NT>(p, g, pre, true, smem, &flag_s);
      stamp(p, n_stamps);
    }
    if (ok && l + 1 < p.s.n_layers) {
      g = product(p, p.layers[l + 1], 0);
      prefetch<NT>(g, pre);
      ok = grid_barrier(p, target += gridDim.x, &ok_s);
    }
    stamp(p, n_stamps);
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  // the CTA that leaves last puts the counters back to zero for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.b.barrier + 1, 1u) == gridDim.x - 1) {
      p.b.barrier[0] = 0u;
      p.b.barrier[1] = 0u;
      if (!ok) {  // a step that was given up may have left counters behind
        for (int i = 0; i < p.s.width / 16; ++i) p.b.tile_counters[i] = 0;
        for (int i = 0; i < p.s.n_rows * p.s.n_kv_heads; ++i) p.b.attn_counters[i] = 0;
      }
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
  Params q = p;
  // products that write x have D / 16 feature tiles: their k range is split over the CTAs that would idle
  const int tiles = p.s.width / 16;
  const int spare = grid / tiles > 0 ? grid / tiles : 1;
  auto splits_for = [&](int k) {
    int s = spare;
    const int kt = k / 16;
    while (s > 1 && (kt + s - 1) / s < WARPS) --s;  // at least one k tile per warp
    return s > 8 ? 8 : s;
  };
  q.splits_c = splits_for(p.s.n_heads * HD);
  q.splits_e = splits_for(p.s.inner);
  r2_launch(resident_kernel<NT>, dim3(grid), dim3(THREADS), size_t(total_smem(NT)), stream, q);
  return launch_status();
}

}  // namespace

extern "C" int r2_decode_resident_head_dim(void) { return HD; }
extern "C" int r2_decode_resident_max_rows(void) { return MAX_ROWS; }
extern "C" int r2_decode_resident_max_splits(void) { return 8; }

// Slices of the keys per (row, kv head): what makes the longest chain of 32-key tiles that a warp
// walks the shortest, given `n_warps` warps on the device.
extern "C" int r2_decode_resident_slices(int n_rows, int n_kv_heads, int max_context, int n_warps) {
  const int pairs = n_rows * n_kv_heads > 0 ? n_rows * n_kv_heads : 1;
  const int tiles = (max_context + 31) / 32 > 0 ? (max_context + 31) / 32 : 1;
  int best = 1, best_cost = 1 << 30;
  for (int s = 1; s <= 16 && s <= tiles; ++s) {
    const int rounds = (pairs * s + n_warps - 1) / n_warps;
    const int cost = rounds * ((tiles + s - 1) / s + 1) + (s > 1 ? 1 : 0);  // + 1: a unit's set-up; + 1: the merge
    if (cost < best_cost) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

// All layers of a decode-only step. `layers` is an array of R2ResidentLayer in device memory.
// Refuses (R2_UNSUPPORTED) what the kernel does not take: more than 64 rows, widths that are no
// multiple of 16, groups of more than 8 query heads per kv head.
extern "C" int r2_decode_resident(const R2ResidentLayer* layers, const R2ResidentShape* shape, const R2ResidentBuffers* buffers,
                                  int page_shift, int n_sms, cudaStream_t stream) {
  if (layers == nullptr || shape == nullptr || buffers == nullptr) return R2_BAD_SHAPE;
  const R2ResidentShape& s = *shape;
  if (s.n_rows <= 0) return R2_OK;
  if (s.n_rows > MAX_ROWS || s.n_layers < 1 || s.n_heads < 1 || s.n_kv_heads < 1 || s.n_heads % s.n_kv_heads != 0) return R2_UNSUPPORTED;
  if (s.n_heads / s.n_kv_heads > 8 || s.width % 16 != 0 || s.inner % 16 != 0 || s.attn_slices < 1 || s.attn_slices > 16) return R2_UNSUPPORTED;
  if (buffers->error_flag == nullptr || buffers->barrier == nullptr) return R2_BAD_SHAPE;
  Params p;
  p.layers = layers;
  p.s = s;
  p.b = *buffers;
  p.splits_c = p.splits_e = 1;
  p.page_shift = page_shift;
  if (s.n_rows <= 8) return launch<1>(p, n_sms, stream);
  if (s.n_rows <= 16) return launch<2>(p, n_sms, stream);
  if (s.n_rows <= 32) return launch<4>(p, n_sms, stream);
  return launch<8>(p, n_sms, stream);
}
