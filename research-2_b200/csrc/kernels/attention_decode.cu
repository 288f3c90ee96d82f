// Decode attention over the paged cache, bfloat16 cache and queries, float arithmetic: rows
// that are one new token each, the case whose time is the reading of the cache.
//
// A CTA takes one (row, kv head, slice of the keys). Its four warps walk the slice's 32-key
// tiles in turn: lane = key for q.k (each lane reads its key's row in 16-byte pieces), lanes
// over the head dimension for p.v; all query heads that share the kv head ride along on the
// same loads. Every warp keeps an online-softmax state; the warps' states are merged in
// shared memory. With one slice the CTA writes the output row; with several it leaves
// (max, sum, unnormalised output) per slice in a scratch buffer and `merge` combines them.
// The slicing depends on the row's own context length and on the number of slices only.
//
// Formulas: kelpie-models/kelpie_models/kernels/ops/paged_attention.py:160-240. HEAD_DIM is a
// compile-time constant (-DHEAD_DIM=64): one library per head size, built on first use.
#include <math.h>

#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif

namespace {

constexpr int HD = HEAD_DIM;
constexpr int WARPS = 4;
constexpr int VECS = HD / 8;                 // 16-byte pieces of a key row
constexpr int DPL = (HD + 63) / 64;          // pairs of head-dimension elements per lane in p.v
constexpr int ROW_BYTES = HD * 2 + 16;       // a key's row in shared memory, padded against bank conflicts
constexpr int NBUF = 1;                      // tiles in flight per warp; other warps' work hides the wait
constexpr int TILE_SMEM = WARPS * NBUF * 2 * 32 * ROW_BYTES;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head sizes come in steps of 16 up to 256");

struct DecodeParams {
  const bf16* q; int q_row_stride;
  bf16* out; int out_row_stride;
  const bf16* k_cache; const bf16* v_cache;
  long long page_stride; int page_size; int page_shift; int n_pages;
  const int32_t* block_tables; int table_width;
  const int32_t* row_entry; const int32_t* positions; const int32_t* seq_lens;
  int n_heads, n_kv_heads;
  float scale; int window;
  int n_slices;
  float* part_o;   // [rows, n_heads, n_slices, HD]
  float* part_ml;  // [rows, n_heads, n_slices, 2]
  // The fused form: the kernel itself puts the new token's key and value into the cache (the
  // warp that owns the tile of the newest key does), and the CTA that finishes last among the
  // slices of a (row, kv head) merges them (arrival counters in global memory, reset after use).
  const bf16* k_new; const bf16* v_new; int new_row_stride;  // [rows, n_kv_heads * HD], or null
  const int32_t* slot_mapping;
  bf16* k_cache_w; bf16* v_cache_w;
  int* counters;  // [rows, n_kv_heads], zero between launches; null: a separate merge kernel follows
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

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
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

constexpr bool MMA_FITS = HD <= 128;   // the tensor-core form keeps HD / 2 output floats per lane
bool g_decode_mma = true;              // r2_attention_decode_set_mma (tests compare the two forms)

// MMA: scores and outputs of a tile on the warp-level tensor cores (mma.sync m16n8k16): the G query
// heads of the kv head are rows of a 16-row operand (the rest zeros), a tile's 32 keys its columns.
// A tile then costs a warp 32 mma and 16 ldmatrix instead of some 500 scalar instructions, which
// is what bounds this kernel at large batches (at batch 64 it read the cache at 0.57 of the copy
// bandwidth with the scalar form).
template <int G, bool MMA>
__global__ void __launch_bounds__(WARPS * 32, (MMA && HD <= 64) ? 5 : 1)  // five CTAs to an SM is what the tiles' shared memory allows
decode_kernel(const DecodeParams p) {
  pdl_launch_dependents();  // the next kernel may begin its prologue
  // The wait on the previous kernel comes further down: positions, context lengths and block
  // tables belong to the batch, which no kernel writes, so the chain of lookups that leads to the
  // first tile's addresses runs while the previous kernel (the product that makes q, k and v) ends.
  __shared__ float q_s[G][HD];
  __shared__ float red_o[WARPS][G][HD];
  __shared__ float red_m[WARPS][G], red_l[WARPS][G];
  __shared__ int is_last_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slice = blockIdx.x, kvh = blockIdx.y, t = blockIdx.z;
  const int h0 = kvh * G;
  // Every row is an entry of its own, in order: row t is entry t. A pad row is an entry of no keys
  // (context length 0, position 0), which the code below turns into zeros without a branch of
  // its own; so nothing here waits for a lookup of the row's entry before the others start.
  const int e = t;
  const int pos = p.positions[t];
  const int seq_len = p.seq_lens[e];
  const int last = pos < seq_len - 1 ? pos : seq_len - 1;
  const int first = p.window > 0 ? (pos - p.window + 1 > 0 ? pos - p.window + 1 : 0) : 0;
  const int n_keys = last - first + 1;
  // this slice's keys: equal runs of whole 32-key tiles
  const int tiles = (n_keys + 31) / 32;
  const int tiles_per = (tiles + p.n_slices - 1) / p.n_slices;
  const int tile_begin = slice * tiles_per;
  const int tile_end = min(tiles, tile_begin + tiles_per);
  const int32_t* table = p.block_tables + size_t(e) * p.table_width;

  float m[G], l[G], acc[G][DPL][2];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[g][i][0] = acc[g][i][1] = 0.f;
  }
  // tensor-core form: this lane's rows are heads gq and gq + 8 of the group (those below G exist)
  constexpr int KS = MMA ? HD / 16 : 1, DT = MMA ? HD / 8 : 1;
  const int gq = lane >> 2, tq = lane & 3;
  uint32_t qf[KS][4];
  float o[DT][4], m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
#pragma unroll
  for (int i = 0; i < DT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const size_t head_off = size_t(kvh) * p.page_size * HD;

  // Tiles of 32 keys go through shared memory: every lane copies its own key's K row and V row
  // with 16-byte asynchronous copies, so a tile's 2 x 32 rows are all in flight at once, and
  // (for head sizes up to 128) the next tile is on its way while this one is used. The newest
  // key's row comes from the projection's output (k_new, v_new), not from the cache.
  extern __shared__ __align__(16) uint8_t tile_smem[];
  uint8_t* my_smem = tile_smem + size_t(warp) * NBUF * 2 * 32 * ROW_BYTES;
  const int tile_of_new = (p.k_new != nullptr && pos == last) ? (pos - first) / 32 : -1;

  // lane r finds row r's place: element offsets from k_cache / v_cache; -1 for a row past the last key
  auto lookup = [&](int tile, long long& my_k, long long& my_v) {
    const int j = first + tile * 32 + lane;
    if (j > last) {
      my_k = my_v = -1;
    } else if (tile == tile_of_new && j == pos) {
      my_k = (p.k_new + size_t(t) * p.new_row_stride + size_t(kvh) * HD) - p.k_cache;
      my_v = (p.v_new + size_t(t) * p.new_row_stride + size_t(kvh) * HD) - p.v_cache;
    } else {
      int page = table[page_index(j, p.page_size, p.page_shift)];
      page = (page < 0 || page >= p.n_pages) ? 0 : page;
      my_k = my_v = (long long)(size_t(page) * p.page_stride + head_off + size_t(page_offset(j, p.page_size, p.page_shift)) * HD);
    }
  };
  // then consecutive lanes copy consecutive 16-byte pieces of a row, then the next row: whole
  // lines per request
  auto copy = [&](int tile, int buf, long long my_k, long long my_v) {
    const int j0 = first + tile * 32;
    const uint32_t kd = smem_u32(my_smem + (size_t(buf) * 2 + 0) * 32 * ROW_BYTES);
    const uint32_t vd = smem_u32(my_smem + (size_t(buf) * 2 + 1) * 32 * ROW_BYTES);
#pragma unroll
    for (int i = 0; i < VECS; ++i) {
      const int f = lane + 32 * i;
      const int row = f / VECS, c = f % VECS;
      const long long ko = __shfl_sync(0xffffffffu, my_k, row);
      const long long vo = __shfl_sync(0xffffffffu, my_v, row);
      const bool valid = ko >= 0 || (tile == tile_of_new && j0 + row == pos);
      const int bytes = valid ? 16 : 0;  // 0 source bytes: zeros
      const bf16* ksrc = valid ? p.k_cache + ko + c * 8 : p.k_cache;
      const bf16* vsrc = valid ? p.v_cache + vo + c * 8 : p.v_cache;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(kd + row * ROW_BYTES + c * 16), "l"(ksrc), "r"(bytes) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(vd + row * ROW_BYTES + c * 16), "l"(vsrc), "r"(bytes) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto issue = [&](int tile, int buf) {
    long long my_k, my_v;
    lookup(tile, my_k, my_v);
    copy(tile, buf, my_k, my_v);
  };

  // The first tile's addresses are found before the wait; its copies (one row of which may be the
  // new key and value, which the previous kernel made) and the query's fetch come after it.
  long long first_k = -1, first_v = -1;
  if (tile_begin + warp < tile_end) lookup(tile_begin + warp, first_k, first_v);
  pdl_wait();  // the previous kernel's writes are visible from here on
  if (tile_begin + warp < tile_end) copy(tile_begin + warp, 0, first_k, first_v);
  if (MMA) {
    // the query heads straight into the lane's operand registers (unscaled: the scale goes on the scores)
    const bf16* qa = p.q + size_t(t) * p.q_row_stride + size_t(h0 + gq) * HD + 2 * tq;
    const bf16* qb = qa + size_t(8) * HD;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      qf[ks][0] = gq < G ? *reinterpret_cast<const uint32_t*>(qa + ks * 16) : 0u;
      qf[ks][1] = gq + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + ks * 16) : 0u;
      qf[ks][2] = gq < G ? *reinterpret_cast<const uint32_t*>(qa + ks * 16 + 8) : 0u;
      qf[ks][3] = gq + 8 < G ? *reinterpret_cast<const uint32_t*>(qb + ks * 16 + 8) : 0u;
    }
  } else {
    for (int i = threadIdx.x; i < G * HD; i += WARPS * 32) {
      int g = i / HD, d = i % HD;
      q_s[g][d] = __bfloat162float(p.q[size_t(t) * p.q_row_stride + size_t(h0 + g) * HD + d]) * p.scale;
    }
    __syncthreads();
  }
  int it = 0;
  for (int tile = tile_begin + warp; tile < tile_end; tile += WARPS, ++it) {
    const int j0 = first + tile * 32;
    const int buf = NBUF == 2 ? (it & 1) : 0;
    if (tile == tile_of_new) {
      // the newest key lies in this tile: this warp also puts its key and value into the cache
      const int slot = p.slot_mapping[t];
      const int page = slot < 0 ? -1 : page_index(slot, p.page_size, p.page_shift);
      if (page >= 0 && page < p.n_pages) {
        const size_t dst = size_t(page) * p.page_stride + size_t(kvh) * p.page_size * HD + size_t(page_offset(slot, p.page_size, p.page_shift)) * HD;
        const __nv_bfloat162* ks = reinterpret_cast<const __nv_bfloat162*>(p.k_new + size_t(t) * p.new_row_stride + size_t(kvh) * HD);
        const __nv_bfloat162* vs = reinterpret_cast<const __nv_bfloat162*>(p.v_new + size_t(t) * p.new_row_stride + size_t(kvh) * HD);
        __nv_bfloat162* kd = reinterpret_cast<__nv_bfloat162*>(p.k_cache_w + dst);
        __nv_bfloat162* vd = reinterpret_cast<__nv_bfloat162*>(p.v_cache_w + dst);
        for (int i = lane; i < HD / 2; i += 32) {
          kd[i] = ks[i];
          vd[i] = vs[i];
        }
      }
    }
    if (NBUF == 2) {
      if (tile + WARPS < tile_end) {
        issue(tile + WARPS, buf ^ 1);
        asm volatile("cp.async.wait_group 1;" ::: "memory");
      } else {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
      }
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncwarp();
    const uint8_t* k_tile = my_smem + (size_t(buf) * 2 + 0) * 32 * ROW_BYTES;
    const uint8_t* v_tile = my_smem + (size_t(buf) * 2 + 1) * 32 * ROW_BYTES;
    if (MMA) {
      const uint32_t kt = smem_u32(k_tile), vt = smem_u32(v_tile);
      float sc[4][4];  // [8-key tile][row gq: 2 keys, row gq + 8: 2 keys]
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
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
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const bool seen = j0 + nt * 8 + 2 * tq + c <= last;
          sc[nt][c] = seen ? sc[nt][c] * p.scale : -INFINITY;
          sc[nt][2 + c] = seen ? sc[nt][2 + c] * p.scale : -INFINITY;
          mx_a = fmaxf(mx_a, sc[nt][c]);
          mx_b = fmaxf(mx_b, sc[nt][2 + c]);
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
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          sc[nt][c] = __expf(sc[nt][c] - m_a);
          sc[nt][2 + c] = __expf(sc[nt][2 + c] - m_b);
          sum_a += sc[nt][c];
          sum_b += sc[nt][2 + c];
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
      if (NBUF == 1) {
        __syncwarp();
        if (tile + WARPS < tile_end) issue(tile + WARPS, 0);
      } else {
        __syncwarp();
      }
      continue;
    }
    const int j = j0 + lane;
    const bool valid = j <= last;
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = 0.f;
    {
      const uint4* kr = reinterpret_cast<const uint4*>(k_tile + lane * ROW_BYTES);
#pragma unroll
      for (int c = 0; c < VECS; ++c) {
        uint4 kv = kr[c];
        const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kv);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float2 kf = __bfloat1622float2(k2[u]);
#pragma unroll
          for (int g = 0; g < G; ++g) {
            s[g] = fmaf(q_s[g][c * 8 + 2 * u], kf.x, s[g]);
            s[g] = fmaf(q_s[g][c * 8 + 2 * u + 1], kf.y, s[g]);
          }
        }
      }
    }
    float pr[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float sv = valid ? s[g] : -INFINITY;
      float m_new = fmaxf(m[g], warp_max(sv));
      float corr = __expf(m[g] - m_new);
      pr[g] = valid ? __expf(sv - m_new) : 0.f;
      l[g] = l[g] * corr + warp_sum(pr[g]);
      m[g] = m_new;
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        acc[g][i][0] *= corr;
        acc[g][i][1] *= corr;
      }
    }
    // p.v from shared memory: lanes over the head dimension, keys in turn (rows past the last key are zeros)
#pragma unroll 8
    for (int jj = 0; jj < 32; ++jj) {
      const __nv_bfloat162* vr = reinterpret_cast<const __nv_bfloat162*>(v_tile + jj * ROW_BYTES);
      float2 vv[DPL];
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        int pair = lane + 32 * i;
        vv[i] = (HD % 64 == 0 || 2 * pair < HD) ? __bfloat1622float2(vr[pair]) : make_float2(0.f, 0.f);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float pj = __shfl_sync(0xffffffffu, pr[g], jj);
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
          acc[g][i][0] = fmaf(pj, vv[i].x, acc[g][i][0]);
          acc[g][i][1] = fmaf(pj, vv[i].y, acc[g][i][1]);
        }
      }
    }
    if (NBUF == 1) {
      __syncwarp();
      if (tile + WARPS < tile_end) issue(tile + WARPS, 0);
    } else {
      __syncwarp();  // the buffer may be overwritten by the copy after next
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  // merge the four warps' states
  if (MMA) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int g = gq + 8 * half;
      if (g < G) {
        if (tq == 0) {
          red_m[warp][g] = m_run[half];
          red_l[warp][g] = l_run[half];
        }
#pragma unroll
        for (int dt = 0; dt < DT; ++dt) {
          red_o[warp][g][dt * 8 + 2 * tq] = o[dt][2 * half];
          red_o[warp][g][dt * 8 + 2 * tq + 1] = o[dt][2 * half + 1];
        }
      }
    }
  }
#pragma unroll
  for (int g = 0; g < G && !MMA; ++g) {
    if (lane == 0) {
      red_m[warp][g] = m[g];
      red_l[warp][g] = l[g];
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      int d = 2 * (lane + 32 * i);
      if (HD % 64 == 0 || d < HD) {
        red_o[warp][g][d] = acc[g][i][0];
        red_o[warp][g][d + 1] = acc[g][i][1];
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * HD; i += WARPS * 32) {
    int g = i / HD, d = i % HD;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) mx = fmaxf(mx, red_m[w][g]);
    float o = 0.f, lsum = 0.f;
    if (mx > -INFINITY) {
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        float c = __expf(red_m[w][g] - mx);
        o += c * red_o[w][g][d];
        lsum += c * red_l[w][g];
      }
    }
    if (p.n_slices == 1) {
      p.out[size_t(t) * p.out_row_stride + size_t(h0 + g) * HD + d] = __float2bfloat16_rn(lsum > 0.f ? o / lsum : 0.f);
    } else {
      size_t at = (size_t(t) * p.n_heads + h0 + g) * p.n_slices + slice;
      p.part_o[at * HD + d] = o;
      if (d == 0) {
        p.part_ml[at * 2] = mx;
        p.part_ml[at * 2 + 1] = lsum;
      }
    }
  }
  if (p.n_slices > 1 && p.counters != nullptr) {
    // the slice that arrives last merges all of them, in slice order
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      int* counter = p.counters + size_t(t) * p.n_kv_heads + kvh;
      int arrived = atomicAdd(counter, 1);
      is_last_s = arrived == p.n_slices - 1;
      if (is_last_s) *counter = 0;  // ready for the next launch
    }
    __syncthreads();
    if (is_last_s) {
      __threadfence();
      for (int i = threadIdx.x; i < G * HD; i += WARPS * 32) {
        int g = i / HD, d = i % HD;
        const size_t base = (size_t(t) * p.n_heads + h0 + g) * p.n_slices;
        float mx = -INFINITY;
        for (int s = 0; s < p.n_slices; ++s) mx = fmaxf(mx, __ldcg(&p.part_ml[(base + s) * 2]));
        float o = 0.f, lsum = 0.f;
        if (mx > -INFINITY) {
          for (int s = 0; s < p.n_slices; ++s) {
            float c = __expf(__ldcg(&p.part_ml[(base + s) * 2]) - mx);
            o += c * __ldcg(&p.part_o[(base + s) * HD + d]);
            lsum += c * __ldcg(&p.part_ml[(base + s) * 2 + 1]);
          }
        }
        p.out[size_t(t) * p.out_row_stride + size_t(h0 + g) * HD + d] = __float2bfloat16_rn(lsum > 0.f ? o / lsum : 0.f);
      }
    }
  }
}

// out[t, h, :] = sum_s exp(m_s - m) o_s / sum_s exp(m_s - m) l_s, slices in order.
__global__ void merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                             int out_row_stride, int n_heads, int n_slices) {
  pdl_launch_dependents();  // the next kernel may begin its prologue
  pdl_wait();               // the previous kernel's writes are visible from here on
  const int t = blockIdx.y, h = blockIdx.x;
  const size_t base = (size_t(t) * n_heads + h) * n_slices;
  float mx = -INFINITY;
  for (int s = 0; s < n_slices; ++s) mx = fmaxf(mx, part_ml[(base + s) * 2]);
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float o = 0.f, l = 0.f;
    if (mx > -INFINITY) {
      for (int s = 0; s < n_slices; ++s) {
        float c = __expf(part_ml[(base + s) * 2] - mx);
        o += c * part_o[(base + s) * HD + d];
        l += c * part_ml[(base + s) * 2 + 1];
      }
    }
    out[size_t(t) * out_row_stride + size_t(h) * HD + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
  }
}

template <int G, bool MMA>
bool configure_smem() {
  // once per kernel instance and device (function attributes belong to a device's context): room for
  // the tiles beyond the default 48 KB
  static bool done_on[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return false;
  bool& done = done_on[device];
  if (!done) {
    if (cudaFuncSetAttribute(decode_kernel<G, MMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, TILE_SMEM) != cudaSuccess) return false;
    // the CTAs hide each other's waits: ask for the shared memory that lets as many as fit be resident
    if (cudaFuncSetAttribute(decode_kernel<G, MMA>, cudaFuncAttributePreferredSharedMemoryCarveout, 100) != cudaSuccess) return false;
    done = true;
  }
  return true;
}

template <int G, bool MMA>
int launch_form(const DecodeParams& p, int n_rows, cudaStream_t stream) {
  dim3 grid(p.n_slices, p.n_kv_heads, n_rows);
  if (!configure_smem<G, MMA>()) return R2_UNSUPPORTED;
  r2_launch(decode_kernel<G, MMA>, dim3(grid), dim3(WARPS * 32), size_t(TILE_SMEM), stream, p);
  return launch_status();
}

template <int G>
int launch(const DecodeParams& p, int n_rows, cudaStream_t stream) {
  if constexpr (MMA_FITS) {
    if (g_decode_mma) return launch_form<G, true>(p, n_rows, stream);
  }
  return launch_form<G, false>(p, n_rows, stream);
}

}  // namespace

extern "C" int r2_attention_decode_head_dim(void) { return HD; }

// Floats of scratch that n_slices > 1 needs: the unnormalised outputs, then (max, sum) pairs.
extern "C" long long r2_attention_decode_scratch_floats(int n_rows, int n_heads, int n_slices) {
  return n_slices > 1 ? (long long)n_rows * n_heads * n_slices * (HD + 2) : 0;
}

extern "C" int r2_attention_decode(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_cache,
                                   const void* v_cache, long long page_stride, int page_size, int n_pages,
                                   const int32_t* block_tables, int table_width, const int32_t* row_entry,
                                   const int32_t* positions, const int32_t* seq_lens, int n_rows, int n_heads,
                                   int n_kv_heads, float scale, int window, int n_slices, float* scratch,
                                   long long scratch_floats, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (n_heads < 1 || n_kv_heads < 1 || n_heads % n_kv_heads != 0 || page_size < 1 || window < 0 || n_slices < 1) return R2_BAD_SHAPE;
  if (page_stride % 8 != 0 || (reinterpret_cast<uintptr_t>(k_cache) & 15)) return R2_BAD_ALIGN;
  if (n_slices > 1 && (scratch == nullptr || scratch_floats < r2_attention_decode_scratch_floats(n_rows, n_heads, n_slices))) return R2_BAD_SHAPE;
  DecodeParams p;
  p.q = (const bf16*)q; p.q_row_stride = q_row_stride;
  p.out = (bf16*)out; p.out_row_stride = out_row_stride;
  p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
  p.page_stride = page_stride; p.page_size = page_size; p.page_shift = page_shift_of(page_size); p.n_pages = n_pages;
  p.block_tables = block_tables; p.table_width = table_width;
  p.row_entry = row_entry; p.positions = positions; p.seq_lens = seq_lens;
  p.n_heads = n_heads; p.n_kv_heads = n_kv_heads;
  p.scale = scale; p.window = window; p.n_slices = n_slices;
  p.part_o = scratch;
  p.part_ml = scratch != nullptr ? scratch + (long long)n_rows * n_heads * n_slices * HD : nullptr;
  p.k_new = nullptr; p.v_new = nullptr; p.new_row_stride = 0; p.slot_mapping = nullptr;
  p.k_cache_w = nullptr; p.v_cache_w = nullptr; p.counters = nullptr;
  int status;
  switch (n_heads / n_kv_heads) {
    case 1: status = launch<1>(p, n_rows, stream); break;
    case 2: status = launch<2>(p, n_rows, stream); break;
    case 4: status = launch<4>(p, n_rows, stream); break;
    case 8: status = launch<8>(p, n_rows, stream); break;
    default: return R2_UNSUPPORTED;
  }
  if (status != R2_OK || n_slices == 1) return status;
  r2_launch(merge_kernel, dim3(dim3(n_heads, n_rows)), dim3(HD >= 128 ? 128 : 64), size_t(0), stream, p.part_o, p.part_ml, (bf16*)out, out_row_stride, n_heads, n_slices);
  return launch_status();
}

namespace {

template <int G>
int launch_fused(const DecodeParams& p, int n_rows, cudaStream_t stream) { return launch<G>(p, n_rows, stream); }

}  // namespace

// One launch for a decode-only batch: the new tokens' keys and values (k_new, v_new:
// [rows, n_kv_heads * HD] with row stride new_row_stride) are written to their cache slots by
// the kernel itself, and the slices of a (row, kv head) are merged by whichever of their CTAs
// finishes last, so there is neither a separate cache-write kernel nor a merge kernel.
// `scratch` as for r2_attention_decode; `counters` holds n_rows * n_kv_heads ints that are
// zero before the call and zero again after it.
extern "C" int r2_attention_decode_fused(const void* q, int q_row_stride, void* out, int out_row_stride, void* k_cache,
                                         void* v_cache, long long page_stride, int page_size, int n_pages,
                                         const int32_t* block_tables, int table_width, const int32_t* row_entry,
                                         const int32_t* positions, const int32_t* seq_lens, int n_rows, int n_heads,
                                         int n_kv_heads, float scale, int window, int n_slices, const void* k_new,
                                         const void* v_new, int new_row_stride, const int32_t* slot_mapping,
                                         float* scratch, long long scratch_floats, int* counters, int n_counters,
                                         cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (n_heads < 1 || n_kv_heads < 1 || n_heads % n_kv_heads != 0 || page_size < 1 || window < 0 || n_slices < 1) return R2_BAD_SHAPE;
  if (n_slices > 1 && (scratch == nullptr || counters == nullptr || n_counters < n_rows * n_kv_heads ||
                       scratch_floats < r2_attention_decode_scratch_floats(n_rows, n_heads, n_slices))) return R2_BAD_SHAPE;
  if (page_stride % 8 != 0 || (reinterpret_cast<uintptr_t>(k_cache) & 15) || (reinterpret_cast<uintptr_t>(v_cache) & 15)) return R2_BAD_ALIGN;
  if (k_new != nullptr && (v_new == nullptr || slot_mapping == nullptr || new_row_stride % 8 != 0 ||
                           (reinterpret_cast<uintptr_t>(k_new) & 15) || (reinterpret_cast<uintptr_t>(v_new) & 15))) return R2_UNSUPPORTED;
  DecodeParams p;
  p.q = (const bf16*)q; p.q_row_stride = q_row_stride;
  p.out = (bf16*)out; p.out_row_stride = out_row_stride;
  p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
  p.page_stride = page_stride; p.page_size = page_size; p.page_shift = page_shift_of(page_size); p.n_pages = n_pages;
  p.block_tables = block_tables; p.table_width = table_width;
  p.row_entry = row_entry; p.positions = positions; p.seq_lens = seq_lens;
  p.n_heads = n_heads; p.n_kv_heads = n_kv_heads;
  p.scale = scale; p.window = window; p.n_slices = n_slices;
  p.part_o = scratch;
  p.part_ml = scratch != nullptr ? scratch + (long long)n_rows * n_heads * n_slices * HD : nullptr;
  p.k_new = (const bf16*)k_new; p.v_new = (const bf16*)v_new; p.new_row_stride = new_row_stride;
  p.slot_mapping = slot_mapping;
  p.k_cache_w = (bf16*)k_cache; p.v_cache_w = (bf16*)v_cache;
  p.counters = n_slices > 1 ? counters : nullptr;
  switch (n_heads / n_kv_heads) {
    case 1: return launch_fused<1>(p, n_rows, stream);
    case 2: return launch_fused<2>(p, n_rows, stream);
    case 4: return launch_fused<4>(p, n_rows, stream);
    case 8: return launch_fused<8>(p, n_rows, stream);
    default: return R2_UNSUPPORTED;
  }
}

// ---------------------------------------------------------------------------------------------
// The same computation for callers that cannot allocate device memory: the slices' partial
// results go to a file-scope device array instead of a buffer that the caller passes in.
// Declaration, limits and rules for the caller: attention_decode_static.h.
#include <stdio.h>

#include <mutex>

#include "attention_decode_static.h"

// In host code this name is only a stand-in for the device array, not its address: it must not
// be handed to a kernel. The address comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) float r2_static_scratch[R2_STATIC_SCRATCH_FLOATS];

namespace {

constexpr int MAX_DEVICES = 64;
float* g_static_scratch[MAX_DEVICES] = {};  // the array's device address, by device ordinal
std::mutex g_static_setup;
thread_local char g_static_error[320] = "";

// The device address of the static scratch array on the current device; looked up on the first
// call for that device (which is why that call should come before any stream capture).
float* static_scratch_for_current_device() {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= MAX_DEVICES) {
    snprintf(g_static_error, sizeof g_static_error, "r2_attention_decode_static: no usable current device (%s, ordinal %d)",
             cudaGetErrorString(e), device);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_static_setup);
  if (g_static_scratch[device] == nullptr) {
    float* address = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), r2_static_scratch);
    if (e != cudaSuccess || address == nullptr) {
      snprintf(g_static_error, sizeof g_static_error,
               "r2_attention_decode_static: cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(e));
      return nullptr;
    }
    g_static_scratch[device] = address;
  }
  return g_static_scratch[device];
}

}  // namespace

extern "C" const char* r2_attention_decode_static_error(void) { return g_static_error; }

extern "C" int r2_attention_decode_static(const void* q, int q_row_stride, void* out, int out_row_stride,
                                          const void* k_cache, const void* v_cache, long long page_stride, int page_size,
                                          int n_pages, const int32_t* block_tables, int table_width,
                                          const int32_t* row_entry, const int32_t* positions, const int32_t* seq_lens,
                                          int n_rows, int n_heads, int n_kv_heads, float scale, int window, int n_slices,
                                          cudaStream_t stream) {
  g_static_error[0] = 0;
  if (n_rows <= 0) return R2_OK;
  if (n_heads < 1 || n_slices < 1) return R2_BAD_SHAPE;
  const long long need = r2_attention_decode_scratch_floats(n_rows, n_heads, n_slices);
  if (need > (long long)R2_STATIC_SCRATCH_FLOATS) {
    snprintf(g_static_error, sizeof g_static_error,
             "r2_attention_decode_static: %d rows x %d heads x %d slices of head size %d need %lld floats of scratch, "
             "the built-in array holds %d; use fewer slices or rows, or r2_attention_decode with a buffer of your own",
             n_rows, n_heads, n_slices, HD, need, int(R2_STATIC_SCRATCH_FLOATS));
    return R2_STATIC_SCRATCH_TOO_SMALL;
  }
  float* scratch = nullptr;
  if (n_slices > 1) {
    scratch = static_scratch_for_current_device();
    if (scratch == nullptr) return R2_STATIC_SETUP_FAILED;
  }
  // Every (row, head, slice) word of the scratch that the merge reads is written by this call's
  // own slices first (empty slices write zeros and a -inf maximum), so nothing needs clearing.
  // The kernels of this entry point take plain stream order: the engine's own launches let a kernel
  // read its index arrays while its predecessor still runs (nothing in the engine writes them on the
  // device), which a caller who fills them with a kernel of its own must not be exposed to.
  struct PlainOrder {
    PlainOrder() { t_r2_plain_order = 1; }
    ~PlainOrder() { t_r2_plain_order = 0; }
  } plain_order;
  return r2_attention_decode(q, q_row_stride, out, out_row_stride, k_cache, v_cache, page_stride, page_size, n_pages,
                             block_tables, table_width, row_entry, positions, seq_lens, n_rows, n_heads, n_kv_heads,
                             scale, window, n_slices, scratch, (long long)R2_STATIC_SCRATCH_FLOATS, stream);
}

// Tests and measurements compare the tensor-core form of a tile's arithmetic with the scalar one.
extern "C" int r2_attention_decode_set_mma(int on) {
  int before = g_decode_mma ? 1 : 0;
  g_decode_mma = on != 0;
  return before;
}
