// bfloat16 matrix product on the 5th-generation tensor cores (tcgen05) with the accumulator in
// tensor memory, operands brought to shared memory by TMA, and a fused epilogue:
//
//   out[token, feature] = act(sum_k x[token, k] * w(k, feature) + bias[feature]) (+ residual)
//
// One CTA computes one 128 x BN tile (or one K-slice of it). Warp 0 issues the TMA loads, one
// thread of warp 1 issues the MMAs, warps 2..5 read the accumulator back and write the result.
// The 128-row side of the tile ("a side") is the tokens when there are many of them; for 64
// tokens or fewer the operands swap and the 128-row side is the weight's output features, so
// that a decode step streams the weights through full-height tiles (the tile is written back
// transposed). With few tiles the K range is split over the CTAs of a thread-block cluster: each
// streams its share of the weights, the others send their float partial sums into the leader's
// shared memory (distributed shared memory), and after a cluster barrier the leader adds them in
// rank order and runs the epilogue. The order is fixed, so the result is the same bits every run.
//
// Weights stored [K, N] (GPT-2's Conv1D layout) are the MN-major operand form, weights stored
// [N, K] (a tied embedding as the head) the K-major form; both are loaded with 128-byte swizzle.
// Every wait on an mbarrier is bounded: on time-out the thread records an error code in
// `error_flag`, all roles leave their loops, tensor memory is freed and the kernel returns.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tensor_maps.cuh"

// Where the key and value columns of a fused q/k/v product go (an argument of r2_gemm_tc): the
// rows' cache slots. `col` is the first key column, `width` the keys' (and the values') width;
// head_dim a multiple of 8.
extern "C" struct R2KvScatter {
  const int32_t* slots;
  void* k_cache;
  void* v_cache;
  long long page_stride;
  int page_size, n_pages, col, width, head_dim;
};

namespace {

constexpr int BM = 128;          // rows of the a side = UMMA M
constexpr int BK = 64;           // one 128-byte swizzle span of bfloat16
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;     // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue
constexpr int MAX_STAGES = 8;
constexpr uint32_t SPIN_LIMIT = 1u << 22;

#define R2_ERR_TIMEOUT_FULL 1
#define R2_ERR_TIMEOUT_EMPTY 2
#define R2_ERR_TIMEOUT_ACC 3
#define R2_ERR_TIMEOUT_TOKENS 4

// The current device's number of multiprocessors: the plans below spread tiles and K-splits over it.
static int n_sms() {
  static int cached[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = 1;
    }
    cached[dev] = n;
  }
  return cached[dev];
}

struct GemmParams {
  int a_total, b_total, k_total;  // extents of the a side, the b side and K
  int bn;                         // tile width on the b side = UMMA N (multiple of 16, <= 256)
  int n_kb, kb_per_split, splits, stages;
  int n_tiles, col_tiles;         // the pair form: tiles in all, and per row of tiles (tile = row * col_tiles + column)
  const float* bias;
  const float* residual;
  int ldr;
  void* out;
  int ldo;
  int out_is_bf16;
  int act;
  int* error_flag;
  // LayerNorm of the tokens fused in front of the product (swapped form only): the token operand
  // is built in shared memory from float rows instead of being loaded by TMA.
  const float* ln_x;       // [*, k] float rows, or null: no fused norm
  int ln_ldx;
  const int32_t* ln_rows;  // token i reads row ln_rows[i] (null: row i)
  const float* ln_gamma;
  const float* ln_beta;
  float ln_eps;
  // The weight of the product that runs next: asked into L2 while this one runs, a slice per CTA.
  const uint8_t* prefetch;
  long long prefetch_bytes;
  // Token-major bfloat16 output whose columns from kv_col on are keys, then values, of this step's
  // tokens: those columns go straight into the rows' cache slots instead of into `out`.
  const int32_t* kv_slots;   // [rows] slot = page * page_size + offset; null: no such columns
  bf16* kv_k;
  bf16* kv_v;
  long long kv_page_stride;
  int kv_page_size, kv_page_shift, kv_n_pages, kv_col, kv_width, kv_head_dim, kv_head_shift;
  // Profiling hook, normally null: six times of the nanosecond clock per CTA of the single-CTA forms (its start,
  // before and after the wait on the kernel before, tokens ready (the form with the norm inside), products
  // complete, end), [CTA][6], for the first `cta_stamps_cap` CTAs: shows how many CTAs an SM really holds.
  long long* cta_stamps;
  int cta_stamps_cap;
};

__device__ __forceinline__ void cta_stamp(const GemmParams& p, int which) {
  if (p.cta_stamps != nullptr && threadIdx.x == 64) {
    const int cta = int(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
    if (cta < p.cta_stamps_cap) {
      long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      p.cta_stamps[cta * 6 + which] = now;
    }
  }
}


__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

// The barrier and tile arguments below are shared-memory addresses as 32-bit numbers: the loops
// that use them are run by one thread each, at one dependent instruction every few cycles, so
// pointer conversions, multiplications and divisions inside them show in the k-block rate.
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done;
}

// Waits for the phase with the given parity to complete; false after SPIN_LIMIT polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  for (uint32_t spin = 0; spin < SPIN_LIMIT; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if (spin > 1024) __nanosleep(64);
  }
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) { return mbar_wait(smem_u32(bar), parity); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// Shared-memory matrix descriptor for a 128-byte-swizzled tile (version 1 = Blackwell).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((addr >> 4) & 0x3FFF);
  d |= uint64_t((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= uint64_t(1) << 46;   // descriptor version
  d |= uint64_t(2) << 61;   // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// gelu_new for the bfloat16 epilogue: tanh through one fast exponential (the result is rounded
// to bfloat16 anyway; the float32 path keeps tanhf).
__device__ __forceinline__ float gelu_tanh_fast(float x) {
  const float k = 0.7978845608028654f;
  float u = k * (x + 0.044715f * x * x * x);
  float e = __expf(2.f * u);
  float t = 1.f - __fdividef(2.f, e + 1.f);  // tanh(u); e = inf gives 1, e = 0 gives -1
  return 0.5f * x * (1.f + t);
}

// True in one lane of the (converged) warp. The loops that issue TMA and tensor-core
// instructions are run by the whole warp with the instruction itself under this predicate:
// their addresses and descriptors are then warp-uniform values, which is the form those
// instructions take their operands in.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"   // one statement: no use of the registers can come between the load and its wait
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// LayerNorm of the token rows, written as the K-major, 128-byte-swizzled bfloat16 tiles that the
// tensor core reads: warp `w` of the four takes rows w, w + 4, ...; a lane holds every 32nd group
// of four elements of its row (rows of at most 1,024 elements, at most 16 tokens); mean and
// variance are two passes over registers, in float
// (kelpie-models/kelpie_models/kernels/ops/layer_norm.py:21-23). Rows past the last token are not
// written: their columns of the product are never stored. The gain and shift are weights, so they
// are fetched before the wait on the previous kernel.
constexpr int LN_MAX_K = 1024;
constexpr int LN_MAX_TOKENS = 16;
constexpr int LN_CHUNKS = LN_MAX_K / 128;

// Gain and shift for the lane's elements inside this CTA's share of K.
__device__ __forceinline__ void load_norm_weights(const GemmParams& p, int kb_begin, int n_kb, int lane, float4 (&gam)[LN_CHUNKS],
                                                  float4 (&bet)[LN_CHUNKS]) {
  const int k_lo = kb_begin * BK, k_hi = min(p.k_total, (kb_begin + n_kb) * BK);
#pragma unroll
  for (int i = 0; i < LN_CHUNKS; ++i) {
    int k = (lane + 32 * i) * 4;
    bool mine = k >= k_lo && k < k_hi;
    gam[i] = mine ? __ldg(reinterpret_cast<const float4*>(p.ln_gamma + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
    bet[i] = mine ? __ldg(reinterpret_cast<const float4*>(p.ln_beta + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// Two sums over the warp at once: the shuffles of one hide the latency of the other's.
__device__ __forceinline__ void warp_sum2(float& a, float& b) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ta = __shfl_xor_sync(0xffffffffu, a, o), tb = __shfl_xor_sync(0xffffffffu, b, o);
    a += ta;
    b += tb;
  }
}

// `src_first`: the source rows of this warp's first two tokens (w and w + 4), looked up before the
// wait on the previous kernel (the index list is part of the batch, not of its output); -1: none.
__device__ __forceinline__ void build_normed_tokens(const GemmParams& p, uint8_t* b_tiles, uint32_t b_stride, int kb_begin,
                                                    int n_kb, int w, int lane, const float4 (&gam)[LN_CHUNKS],
                                                    const float4 (&bet)[LN_CHUNKS], const int (&src_first)[2]) {
  const int k_total = p.k_total;
  const int k_lo = kb_begin * BK, k_end = (kb_begin + n_kb) * BK, k_hi = min(k_total, k_end);
  const float inv_k = 1.f / float(k_total);
  // Rows past the last token are left as they are: their columns of the product are never stored.
  // Two rows at a time, in lockstep and free of per-row branches, so that the loads and the
  // reductions of one row pass under those of the other.
  for (int r0 = w; r0 < p.b_total; r0 += 8) {
    float4 v[2][LN_CHUNKS];
    bool live[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int r = r0 + 4 * u;
      live[u] = r < p.b_total;
      int src = 0;
      if (live[u]) src = r0 == w ? src_first[u] : (p.ln_rows != nullptr ? p.ln_rows[r] : r);
      const float4* row = reinterpret_cast<const float4*>(p.ln_x + size_t(src) * p.ln_ldx);
#pragma unroll
      for (int i = 0; i < LN_CHUNKS; ++i) {
        int k = (lane + 32 * i) * 4;
        v[u][i] = (live[u] && k < k_total) ? row[lane + 32 * i] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < LN_CHUNKS; ++i) {
      sum[0] += v[0][i].x + v[0][i].y + v[0][i].z + v[0][i].w;
      sum[1] += v[1][i].x + v[1][i].y + v[1][i].z + v[1][i].w;
    }
    warp_sum2(sum[0], sum[1]);
    const float mean[2] = {sum[0] * inv_k, sum[1] * inv_k};
    float sq[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < LN_CHUNKS; ++i) {
      int k = (lane + 32 * i) * 4;
      if (k < k_total) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          float a = v[u][i].x - mean[u], b = v[u][i].y - mean[u], c = v[u][i].z - mean[u], d = v[u][i].w - mean[u];
          sq[u] += a * a + b * b + c * c + d * d;
        }
      }
    }
    warp_sum2(sq[0], sq[1]);
    const float rstd[2] = {1.f / sqrtf(sq[0] * inv_k + p.ln_eps), 1.f / sqrtf(sq[1] * inv_k + p.ln_eps)};
#pragma unroll
    for (int i = 0; i < LN_CHUNKS; ++i) {
      int k = (lane + 32 * i) * 4;
      if (k < k_lo || k >= k_end) continue;  // another CTA's share of K, or past the tiles
      const int kb = k / BK - kb_begin, kin = k % BK;
      uint8_t* tile = b_tiles + size_t(kb) * b_stride;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (!live[u]) continue;
        const int r = r0 + 4 * u;
        uint32_t lo = 0u, hi = 0u;
        if (k < k_hi) {
          lo = pack2((v[u][i].x - mean[u]) * rstd[u] * gam[i].x + bet[i].x, (v[u][i].y - mean[u]) * rstd[u] * gam[i].y + bet[i].y);
          hi = pack2((v[u][i].z - mean[u]) * rstd[u] * gam[i].z + bet[i].z, (v[u][i].w - mean[u]) * rstd[u] * gam[i].w + bet[i].w);
        }
        uint32_t off = uint32_t(r / 8) * 1024u + uint32_t(r % 8) * 128u + (uint32_t((kin / 8) ^ (r % 8)) * 16u) + uint32_t(kin % 8) * 2u;
        *reinterpret_cast<uint2*>(tile + off) = make_uint2(lo, hi);
      }
    }
  }
}

__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n\t"
      "tcgen05.wait::ld.sync.aligned;"   // one statement: no use of the registers can come between the load and its wait
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void st_shared16(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ld_shared16(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}

// The same load without its wait: several may be in flight before one tmem_wait().
__device__ __forceinline__ void tmem_load32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
// The wait for them. The loaded registers are operands of the wait (`tmem_tie` for a second set): to the compiler
// a load is complete when its statement is, and without this tie it may place a use of the registers before the wait.
__device__ __forceinline__ void tmem_wait(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]) : : "memory");
}
__device__ __forceinline__ void tmem_tie(uint32_t (&r)[32]) {
  asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]) : : "memory");
}

constexpr int STAGING_ROW = 36;                       // words per staged row: 32 and four of padding (rows stay 16-byte aligned)
constexpr int STAGING_WORDS = 32 * STAGING_ROW;       // per epilogue warp
constexpr int BIAS_SLOTS = 256;                       // floats: the widest tile

// The epilogue of a 32-row slab of a token-major tile over the tile's columns [c_begin, c_end)
// (one warp; lane = accumulator row). The accumulator comes out of tensor memory one row per
// lane, which written straight to global memory is 32 scattered pieces per store and one exposed
// load latency per piece of the residual. So each group of columns takes two steps: (1) bias and
// activation on the lane's row, written to a padded shared-memory slab; (2) read back with eight
// lanes to a row, 16 bytes each, so that every global access of the warp is four whole 128-byte
// pieces of rows. The residual of a whole group is requested before step (1), so its latency
// passes under it. An epilogue warp has a scheduler almost to itself and issues about one
// instruction every six cycles, so the count of instructions per element is what is kept small.
// `bias_s` holds the tile's bias (zeros without one), 16-byte aligned. bfloat16 output without a
// residual moves 64 columns a group as packed pairs; everything else 32 columns as floats.
// `slab` is the warp's 32 x STAGING_ROW words of shared memory, as a shared-space address.
__device__ __forceinline__ void finish_tile_rows(const GemmParams& p, uint32_t lane_addr, uint32_t slab, const float* bias_s,
                                                 int row0, int col0, int c_begin, int c_end, int lane, bool have_acc) {
  const int rows = min(32, p.a_total - row0);        // rows of this slab that exist
  const int sub = lane >> 3, piece = lane & 7;       // step (2): the row within four, the 16-byte piece of it
  // 32 columns from c on, given their accumulators: + bias, activated
  auto finish_values = [&](int c, const uint32_t (&r)[32], float (&v)[32]) {
    const float4* b4 = reinterpret_cast<const float4*>(bias_s + (c & (BIAS_SLOTS - 1)));
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 b = b4[j];
      v[4 * j] = __uint_as_float(r[4 * j]) + b.x;
      v[4 * j + 1] = __uint_as_float(r[4 * j + 1]) + b.y;
      v[4 * j + 2] = __uint_as_float(r[4 * j + 2]) + b.z;
      v[4 * j + 3] = __uint_as_float(r[4 * j + 3]) + b.w;
    }
    if (p.act == R2_ACT_GELU_TANH) {
      if (p.out_is_bf16) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = gelu_tanh_hw(v[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = gelu_tanh_fast(v[j]);
      }
    } else if (p.act == R2_ACT_GELU_ERF) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
    }
  };
  auto row_values = [&](int c, float (&v)[32]) {     // the same, reading the accumulators first
    uint32_t r[32];
    if (have_acc) {
      tmem_load32(lane_addr + uint32_t(c), r);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = 0u;
    }
    finish_values(c, r, v);
  };
  const bool inside = rows == 32 && col0 + c_end <= p.b_total;  // the whole slab lies inside the output
  if (p.out_is_bf16 && p.residual == nullptr) {
    bf16* out = reinterpret_cast<bf16*>(p.out);
    const bool vec_ok = (p.ldo & 7) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (col0 & 7) == 0;
    // Where in a cache tensor this lane's row (row0 + lane) lies: elements from the tensor's start to the row's
    // slot in kv head 0, or -1 for a row that is not stored. Asked for and worked out once per slab, ahead of the
    // first group's accumulators; step (2) gets the eight rows it stores from their lanes by shuffles, so that
    // nothing more than this is held while the accumulators fill the registers.
    const bool scatters = p.kv_slots != nullptr && col0 + c_end > p.kv_col;
    long long my_at = -1;
    if (scatters && lane < rows) {
      const int slot = p.kv_slots[row0 + lane];
      const int page = slot >= 0 ? page_index(slot, p.kv_page_size, p.kv_page_shift) : p.kv_n_pages;
      if (page < p.kv_n_pages) my_at = (long long)page * p.kv_page_stride + (long long)page_offset(slot, p.kv_page_size, p.kv_page_shift) * p.kv_head_dim;
    }
    for (int c0 = c_begin; c0 < c_end; c0 += 64) {
      if (col0 + c0 >= p.b_total) break;
      {
        // both halves' accumulators are asked for before either is waited for
        const bool two = c0 + 32 < c_end;
        uint32_t r0[32], r1[32];
        if (have_acc) {
          tmem_load32_issue(lane_addr + uint32_t(c0), r0);
          if (two) tmem_load32_issue(lane_addr + uint32_t(c0 + 32), r1);
          tmem_wait(r0);
          if (two) tmem_tie(r1);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r0[j] = r1[j] = 0u;
        }
        float v[32];
        finish_values(c0, r0, v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          st_shared16(slab + uint32_t(lane * STAGING_ROW + 4 * j) * 4u, pack2(v[8 * j], v[8 * j + 1]), pack2(v[8 * j + 2], v[8 * j + 3]),
                      pack2(v[8 * j + 4], v[8 * j + 5]), pack2(v[8 * j + 6], v[8 * j + 7]));
        }
        if (two) {
          finish_values(c0 + 32, r1, v);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            st_shared16(slab + uint32_t(lane * STAGING_ROW + 16 + 4 * j) * 4u, pack2(v[8 * j], v[8 * j + 1]), pack2(v[8 * j + 2], v[8 * j + 3]),
                        pack2(v[8 * j + 4], v[8 * j + 5]), pack2(v[8 * j + 6], v[8 * j + 7]));
          }
        }
      }
      __syncwarp();
      // Step (2). Each lane decides for its own eight columns; the warp stays together.
      const int col = col0 + c0 + 8 * piece;                                   // this lane's eight columns
      const int n_cols = min(8, min(c_end - (c0 + 8 * piece), p.b_total - col));
      long long slot_at[8];
      if (scatters) {  // (the whole warp)
#pragma unroll
        for (int i = 0; i < 8; ++i) slot_at[i] = __shfl_sync(0xffffffffu, my_at, 4 * i + sub);
      }
      if (n_cols <= 0) {
        // nothing of this lane's lies inside the output
      } else if (scatters && col >= p.kv_col) {
        // keys or values of one kv head: each row's piece goes to the row's slot in the cache
        // ([page][kv head][offset][dim]); nothing of it goes to `out`
        const int rel = col - p.kv_col;
        const int which = rel >= p.kv_width ? 1 : 0, within = rel - which * p.kv_width;   // keys, then values
        const int head = p.kv_head_shift >= 0 ? within >> p.kv_head_shift : within / p.kv_head_dim;
        const int dim = within - head * p.kv_head_dim;
        bf16* base = (which == 0 ? p.kv_k : p.kv_v) + size_t(head) * p.kv_page_size * p.kv_head_dim + dim;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint4 w = ld_shared16(slab + uint32_t((4 * i + sub) * STAGING_ROW + 4 * piece) * 4u);
          if (slot_at[i] >= 0) *reinterpret_cast<uint4*>(base + slot_at[i]) = w;
        }
      } else if (inside && vec_ok && n_cols == 8) {
        // the common case, free of per-element conditions
        bf16* d = out + size_t(row0 + sub) * p.ldo + col;
        const size_t step = size_t(4) * p.ldo;
#pragma unroll
        for (int r4 = 0; r4 < 32; r4 += 4, d += step) {
          *reinterpret_cast<uint4*>(d) = ld_shared16(slab + uint32_t((r4 + sub) * STAGING_ROW + 4 * piece) * 4u);
        }
      } else {
#pragma unroll
        for (int r4 = 0; r4 < 32; r4 += 4) {
          const int r = r4 + sub;
          const uint4 w = ld_shared16(slab + uint32_t(r * STAGING_ROW + 4 * piece) * 4u);
          if (r < rows) {
            bf16* d = out + size_t(row0 + r) * p.ldo + col;
            if (n_cols == 8 && vec_ok) {
              *reinterpret_cast<uint4*>(d) = w;
            } else {
              const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if (j < n_cols) d[j] = __ushort_as_bfloat16(uint16_t(words[j >> 1] >> (16 * (j & 1))));
              }
            }
          }
        }
      }
      __syncwarp();
    }
    return;
  }
  const bool vec_ok = (p.ldo & 3) == 0 && (p.out_is_bf16 || (reinterpret_cast<uintptr_t>(p.out) & 15) == 0) && (col0 & 3) == 0 &&
                      (p.residual == nullptr || ((p.ldr & 3) == 0 && (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0));
  for (int c0 = c_begin; c0 < c_end; c0 += 32) {
    if (col0 + c0 >= p.b_total) break;
    const int col = col0 + c0 + 4 * piece;                                     // this lane's four columns
    if (inside && vec_ok && c0 + 32 <= c_end && !p.out_is_bf16) {
      // the common case, free of per-element conditions
      float4 x[8];
      if (p.residual != nullptr) {
        const float* src = p.residual + size_t(row0 + sub) * p.ldr + col;
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = *reinterpret_cast<const float4*>(src + size_t(4 * i) * p.ldr);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      {
        float v[32];
        row_values(c0, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          st_shared16(slab + uint32_t(lane * STAGING_ROW + 4 * j) * 4u, __float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]),
                      __float_as_uint(v[4 * j + 2]), __float_as_uint(v[4 * j + 3]));
        }
      }
      __syncwarp();
      float* d = reinterpret_cast<float*>(p.out) + size_t(row0 + sub) * p.ldo + col;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4 w = ld_shared16(slab + uint32_t((4 * i + sub) * STAGING_ROW + 4 * piece) * 4u);
        *reinterpret_cast<float4*>(d + size_t(4 * i) * p.ldo) =
            make_float4(__uint_as_float(w.x) + x[i].x, __uint_as_float(w.y) + x[i].y, __uint_as_float(w.z) + x[i].z, __uint_as_float(w.w) + x[i].w);
      }
      __syncwarp();
      continue;
    }
    const int n_cols = min(4, min(c_end - (c0 + 4 * piece), p.b_total - col));
    const bool whole = n_cols == 4 && vec_ok;
    float4 x[8];  // the residual of this lane's columns, its eight rows of the slab, in flight during step (1)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = 4 * i + sub;
      x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (p.residual != nullptr && r < rows && n_cols > 0) {
        const float* src = p.residual + size_t(row0 + r) * p.ldr + col;
        if (whole) {
          x[i] = *reinterpret_cast<const float4*>(src);
        } else {
          x[i].x = src[0];
          if (n_cols > 1) x[i].y = src[1];
          if (n_cols > 2) x[i].z = src[2];
          if (n_cols > 3) x[i].w = src[3];
        }
      }
    }
    {
      float v[32];
      row_values(c0, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        st_shared16(slab + uint32_t(lane * STAGING_ROW + 4 * j) * 4u, __float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]),
                    __float_as_uint(v[4 * j + 2]), __float_as_uint(v[4 * j + 3]));
      }
    }
    __syncwarp();
    if (n_cols > 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = 4 * i + sub;
        const uint4 w = ld_shared16(slab + uint32_t(r * STAGING_ROW + 4 * piece) * 4u);
        if (r < rows) {
          const float y[4] = {__uint_as_float(w.x) + x[i].x, __uint_as_float(w.y) + x[i].y, __uint_as_float(w.z) + x[i].z,
                              __uint_as_float(w.w) + x[i].w};
          if (p.out_is_bf16) {
            bf16* d = reinterpret_cast<bf16*>(p.out) + size_t(row0 + r) * p.ldo + col;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (j < n_cols) d[j] = __float2bfloat16_rn(y[j]);
            }
          } else {
            float* d = reinterpret_cast<float*>(p.out) + size_t(row0 + r) * p.ldo + col;
            if (whole) {
              *reinterpret_cast<float4*>(d) = make_float4(y[0], y[1], y[2], y[3]);
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (j < n_cols) d[j] = y[j];
              }
            }
          }
        }
      }
    }
    __syncwarp();
  }
}

// A_MN / B_MN: the operand's tile in shared memory is MN-major (rows of 64 MN-elements, one row
// per k) instead of K-major (rows of 64 k-elements, one row per MN index).
// TRANSPOSED: the a side is the features and the b side the tokens.
template <bool A_MN, bool B_MN, bool TRANSPOSED, bool FUSED_LN = false>
__global__ void __launch_bounds__(THREADS, (TRANSPOSED && !FUSED_LN) ? 1 : 2)  // token-major tiles run two CTAs to an SM, and so does the form with the norm inside (the logits' 393 CTAs)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t a_bytes = BM * BK * 2;
  const uint32_t b_bytes = uint32_t(p.bn) * BK * 2;
  const uint32_t b_stride = (b_bytes + 1023u) & ~1023u;
  constexpr bool fused_ln = TRANSPOSED && FUSED_LN;  // a variant of its own: the norm's registers stay out of the others
  const int b_slots = fused_ln ? p.kb_per_split : p.stages;  // with a fused norm every token tile stays resident
  uint8_t* a_tiles = smem;
  uint8_t* b_tiles = smem + size_t(p.stages) * a_bytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(b_tiles + size_t(b_slots) * b_stride);
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* acc_ready = empty + MAX_STAGES;
  uint64_t* tokens_ready = acc_ready + 1;
  uint64_t* partials_ready = tokens_ready + 1;  // leader: the other CTAs' partial sums have landed (counted in bytes)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(partials_ready + 1);
  // partial sums of the other CTAs of the cluster, [rank - 1][column][row], used in the leader only
  // (feature-major form); the token-major form keeps the tile's bias in the same place
  float* reduce = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(tmem_slot + 4) + 15) & ~uintptr_t(15));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  cta_stamp(p, 0);
  const int a0 = blockIdx.x * BM, b0 = blockIdx.y * p.bn;
  uint32_t rank = 0;  // this CTA's place in its cluster = its slice of K
  if (p.splits > 1) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  // feature-major split-K: columns (tokens) of this tile that exist, rounded up to 16-byte pieces
  const int live_cols = min(p.bn, ((p.b_total - b0 + 3) / 4) * 4);
  const int kb_begin = int(rank) * p.kb_per_split;
  const int kb_end = min(p.n_kb, kb_begin + p.kb_per_split);
  const int n_kb = kb_end - kb_begin;
  uint32_t tmem_cols = 32;
  while (tmem_cols < uint32_t(p.bn)) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_ready, 1);
    mbar_init(tokens_ready, 4);  // one arrival per epilogue warp
    mbar_init(partials_ready, 1);
    if (p.splits > 1 && rank == 0) {
      // every other CTA sends its whole tile of partial sums, rows padded
      mbar_expect_tx(smem_u32(partials_ready), uint32_t(p.splits - 1) * BM * (uint32_t(live_cols) + 4u) * 4u);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  // The next kernel may start (set up, prefetch its weights) from here on, and not earlier: its
  // CTAs allocate tensor memory before they wait for this kernel, so a CTA of this kernel that
  // still had to allocate could find every column taken by CTAs that wait for it.
  pdl_launch_dependents();
  // The weight is never written by a kernel, so its first tiles are requested before the wait
  // on the previous kernel; the activations, which that kernel may have written, after it.
  const uint32_t a_base = smem_u32(a_tiles), b_base = smem_u32(b_tiles);
  const uint32_t full_base = smem_u32(full), empty_base = smem_u32(empty);
  auto load_weight = [&](int k0, uint32_t a_dst, uint32_t b_dst, uint32_t bar) {
    if (TRANSPOSED) {
      if (A_MN) {  // [k rows][64 a-elements] boxes, one per 64 a-elements
        tma_load_2d(a_dst, &map_a, a0, k0, bar);
        tma_load_2d(a_dst + BK * 128, &map_a, a0 + 64, k0, bar);
      } else {     // [a rows][64 k-elements]
        tma_load_2d(a_dst, &map_a, k0, a0, bar);
      }
    } else {
      if (B_MN) {
        for (int j = 0; j < p.bn; j += 64, b_dst += BK * 128) tma_load_2d(b_dst, &map_b, b0 + j, k0, bar);
      } else {
        tma_load_2d(b_dst, &map_b, k0, b0, bar);
      }
    }
  };
  auto load_tokens = [&](int k0, uint32_t a_dst, uint32_t b_dst, uint32_t bar) {
    if (TRANSPOSED) {
      tma_load_2d(b_dst, &map_b, k0, b0, bar);  // tokens are K-major
    } else {
      tma_load_2d(a_dst, &map_a, k0, a0, bar);
    }
  };
  const int first = min(n_kb, p.stages);
  const uint32_t stage_bytes = a_bytes + (fused_ln ? 0u : b_bytes);
  // the first round of the ring: lane s of warp 0 fills stage s, all at the same time
  const bool fills = warp == 0 && lane < first;
  const int fill_k0 = (kb_begin + lane) * BK;
  const uint32_t fill_a = a_base + uint32_t(lane) * a_bytes, fill_b = b_base + uint32_t(lane) * b_stride;
  const uint32_t fill_bar = full_base + uint32_t(lane) * 8u;
  if (fills) {
    mbar_expect_tx(fill_bar, stage_bytes);
    load_weight(fill_k0, fill_a, fill_b, fill_bar);
  }
  __syncwarp();
  if (p.splits > 1) cluster_sync();  // every CTA of the cluster is running before anyone writes into another

  if (warp == 0) {
    if (fills) {
      pdl_wait();
      if (!fused_ln) load_tokens(fill_k0, fill_a, fill_b, fill_bar);
    }
    __syncwarp();
    if (first < n_kb) {
      // ---- producer: from the ring's second round on the warp runs the loop and one elected
      // lane issues ------------------------------------------------------------------------
      int stage = 0, k0 = (kb_begin + first) * BK;   // first == p.stages here
      uint32_t parity = 0, a_dst = a_base, b_dst = b_base;
      for (int i = first; i < n_kb; ++i) {
        if (!mbar_wait(empty_base + uint32_t(stage) * 8u, parity)) {
          if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_EMPTY);
          break;
        }
        if (elect_one()) {
          const uint32_t bar = full_base + uint32_t(stage) * 8u;
          mbar_expect_tx(bar, stage_bytes);
          load_weight(k0, a_dst, b_dst, bar);
          if (!fused_ln) load_tokens(k0, a_dst, b_dst, bar);
        }
        __syncwarp();
        k0 += BK;
        a_dst += a_bytes;
        b_dst += b_stride;
        if (++stage == p.stages) {
          stage = 0;
          parity ^= 1u;
          a_dst = a_base;
          b_dst = b_base;
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the warp runs the loop, one elected lane issues -------------------------
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(A_MN) << 15) | (uint32_t(B_MN) << 16) |
                           (uint32_t(p.bn >> 3) << 17) | (uint32_t(BM >> 4) << 24);
    bool ok = true;
    if (fused_ln && !mbar_wait(tokens_ready, 0)) {
      if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_TOKENS);
      ok = false;
    }
    // Descriptors without their address field, and the address (in 16-byte units) of the current
    // stage's tiles. 16 k-elements further is 32 bytes along a K-major row, or 16 rows of 128
    // bytes in an MN-major tile, whose 64-element chunks lie 8192 bytes apart.
    const uint64_t da_fixed = A_MN ? smem_desc(0, BK * 128, 1024) : smem_desc(0, 16, 1024);
    const uint64_t db_fixed = B_MN ? smem_desc(0, BK * 128, 1024) : smem_desc(0, 16, 1024);
    constexpr uint32_t a_step = (A_MN ? UMMA_K * 128 : 32) >> 4, b_step = (B_MN ? UMMA_K * 128 : 32) >> 4;
    int stage = 0;
    // (only the offset within the CTA's shared memory goes into a descriptor: in a cluster the
    // address of a CTA other than the first carries its rank in high bits)
    const uint32_t a_first = (a_base >> 4) & 0x3FFFu, b_first = (b_base >> 4) & 0x3FFFu;
    uint32_t parity = 0, a_at = a_first, b_at = b_first;
    for (int i = 0; i < n_kb && ok; ++i) {
      if (!mbar_wait(full_base + uint32_t(stage) * 8u, parity)) {
        if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_FULL);
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
          umma_bf16(tmem_base, da_fixed + uint64_t(a_at + kk * a_step), db_fixed + uint64_t(b_at + kk * b_step), idesc,
                    (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(empty_base + uint32_t(stage) * 8u);  // the stage is free once these MMAs have read it
      }
      __syncwarp();
      a_at += a_bytes >> 4;
      b_at += b_stride >> 4;  // with a fused norm the token tiles are not a ring: tile i follows tile i - 1
      if (++stage == p.stages) {
        stage = 0;
        parity ^= 1u;
        a_at = a_first;
        if (!fused_ln) b_at = b_first;
      }
    }
    if (elect_one()) umma_commit(smem_u32(acc_ready));  // arrives when every MMA above has completed (also on the error path)
    __syncwarp();
  }

  // ---- epilogue: warps 2..5, each on the 32 accumulator lanes it may read ------------------
  bool acc_ok = true;
  float bias_ahead = 0.f, res_ahead[32];  // feature-major epilogue: the lane's bias, and its residual for the first 32 tokens
#pragma unroll
  for (int j = 0; j < 32; ++j) res_ahead[j] = 0.f;
  if (threadIdx.x == 64 && p.prefetch != nullptr) {
    // weights never change: this CTA's slice of the next product's weight goes to L2 right away
    const long long n_ctas = (long long)gridDim.x * gridDim.y * gridDim.z;
    const long long cta = blockIdx.x + (long long)gridDim.x * (blockIdx.y + (long long)gridDim.y * blockIdx.z);
    const long long per = ((p.prefetch_bytes + n_ctas - 1) / n_ctas + 4095) / 4096 * 4096;
    const long long begin = cta * per, end = min(p.prefetch_bytes, begin + per);
    for (long long at = begin; at < end; at += 4096) {
      const uint32_t size = uint32_t(min(4096ll, end - at)) & ~15u;
      if (size > 0) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.prefetch + at), "r"(size) : "memory");
    }
  }
  if (warp >= 2) {
    float4 gam[fused_ln ? LN_CHUNKS : 1], bet[fused_ln ? LN_CHUNKS : 1];
    int src_first[2] = {-1, -1};
    if constexpr (fused_ln) {
      load_norm_weights(p, kb_begin, n_kb, lane, gam, bet);
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int r = (warp & 3) + 4 * u;
        if (r < p.b_total) src_first[u] = p.ln_rows != nullptr ? p.ln_rows[r] : r;
      }
    }
    cta_stamp(p, 1);
    pdl_wait();  // the epilogue reads the residual stream and writes the output
    cta_stamp(p, 2);
    if constexpr (fused_ln) {
      build_normed_tokens(p, b_tiles, b_stride, kb_begin, n_kb, warp & 3, lane, gam, bet, src_first);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes, read by the tensor core
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(tokens_ready)) : "memory");
      cta_stamp(p, 3);
    }
    const int q = warp & 3;  // tensor-memory lanes [32q, 32q + 32) belong to warps with id % 4 == q
    if constexpr (!TRANSPOSED) {
      // the tile's bias, once for the four epilogue warps, while the products run
      for (int j = int(threadIdx.x) - 64; j < p.bn; j += 128) reduce[j] = (p.bias != nullptr && b0 + j < p.b_total) ? p.bias[b0 + j] : 0.f;
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    if constexpr (TRANSPOSED) {
      // what the epilogue adds does not depend on the products: it is fetched while they run
      const int a = a0 + q * 32 + lane;
      if (rank == 0 && a < p.a_total) {
        if (p.bias != nullptr) bias_ahead = p.bias[a];
        if (p.residual != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j) res_ahead[j] = (j < p.bn && b0 + j < p.b_total) ? p.residual[size_t(b0 + j) * p.ldr + a] : 0.f;
        }
      }
    }
    bool ok = n_kb <= 0 || mbar_wait(acc_ready, 0);
    cta_stamp(p, 4);
    if (!ok) atomicMax(p.error_flag, R2_ERR_TIMEOUT_ACC);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t lane_addr = tmem_base + (uint32_t(q * 32) << 16);
    acc_ok = ok;
    if (p.splits > 1 && rank != 0) {
      // This slice's partial sums go to the leader's shared memory as [rank - 1][row][column] with
      // rows padded by 16 bytes (the leader's 16-byte reads of 32 rows then fall on different
      // banks): they are laid out in this CTA's own (otherwise unused) copy of the buffer first,
      // and one bulk copy carries the whole tile over, its bytes counted on the leader's barrier.
      // (Thousands of separate 16-byte remote stores took more than a microsecond to land.)
      // Only the columns of tokens that exist are sent.
      const uint32_t row_words = uint32_t(live_cols) + 4u;
      const uint32_t mine = smem_u32(reduce) + uint32_t(q * 32 + lane) * row_words * 4u;
      for (int c0 = 0; c0 < live_cols; c0 += 16) {
        uint32_t r[16];
        if (ok && n_kb > 0) {
          tmem_load16(lane_addr + uint32_t(c0), r);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
          if (c0 + j < live_cols) st_shared16(mine + uint32_t(c0 + j) * 4u, r[j], r[j + 1], r[j + 2], r[j + 3]);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes, read by the bulk copy
      asm volatile("bar.sync 1, 128;" ::: "memory");               // the four epilogue warps
      if (threadIdx.x == 64) {
        uint32_t remote, remote_bar;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(reduce)), "r"(0u));
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(smem_u32(partials_ready)), "r"(0u));
        const uint32_t tile_bytes = BM * row_words * 4u;
        asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(remote + uint32_t(rank - 1) * tile_bytes), "r"(smem_u32(reduce)), "r"(tile_bytes), "r"(remote_bar)
                     : "memory");
      }
    }
  }
  if (p.splits > 1 && warp >= 2 && rank == 0 && acc_ok) {
    // the other CTAs' partial sums have landed in this CTA's shared memory
    if (!mbar_wait(partials_ready, 0)) {
      atomicMax(p.error_flag, R2_ERR_TIMEOUT_ACC);
      acc_ok = false;
    }
  }
  if (warp >= 2 && rank == 0) {
    const int q = warp & 3;
    const int a = a0 + q * 32 + lane;
    const uint32_t lane_addr = tmem_base + (uint32_t(q * 32) << 16);
    const bool ok = acc_ok;
    if constexpr (!TRANSPOSED) {
      // every product has completed: the first tiles' shared memory serves as the warps' slabs
      if (ok && a0 + q * 32 < p.a_total) {
        finish_tile_rows(p, lane_addr, smem_u32(a_tiles) + uint32_t(q * STAGING_WORDS) * 4u, reduce, a0 + q * 32, b0, 0, p.bn, lane, n_kb > 0);
      }
    } else if (ok) {
      const bool a_ok = a < p.a_total;
      // In the transposed form the thread's feature is fixed: one bias value serves every column.
      const float bias_a = bias_ahead;
      const uint32_t row_words = uint32_t(live_cols) + 4u;
      const uint32_t my_row = smem_u32(reduce) + uint32_t(q * 32 + lane) * row_words * 4u;
      for (int c0 = 0; c0 < p.bn; c0 += 16) {
        float v[16];
        {
          uint32_t r[16];
          if (n_kb > 0) {
            tmem_load16(lane_addr + uint32_t(c0), r);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = 0u;
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
        }
        for (int z = 1; z < p.splits; ++z) {  // rank order: the sum is the same bits every run
          const uint32_t part = my_row + (uint32_t(z - 1) * BM * row_words + uint32_t(c0)) * 4u;
#pragma unroll
          for (int j = 0; j < 16; j += 4) {
            if (c0 + j >= live_cols) break;
            const uint4 w = ld_shared16(part + uint32_t(j) * 4u);
            v[j] += __uint_as_float(w.x);
            v[j + 1] += __uint_as_float(w.y);
            v[j + 2] += __uint_as_float(w.z);
            v[j + 3] += __uint_as_float(w.w);
          }
        }
        const int nb = min(16, p.b_total - (b0 + c0));  // columns of this chunk that exist
        if (!a_ok || nb <= 0) continue;
        {
          // lanes hold consecutive features: every column is one coalesced row segment
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] += bias_a;
          if (p.act == R2_ACT_GELU_TANH) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = gelu_tanh_fast(v[j]);
          } else if (p.act == R2_ACT_GELU_ERF) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = gelu_erf(v[j]);
          }
          if (p.residual != nullptr) {
            if (c0 == 0) {  // (asked for before the products ran: a chunk's residual read here costs it a round trip to L2)
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] += res_ahead[j];
            } else if (c0 == 16) {
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] += res_ahead[16 + j];
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (j < nb) v[j] += p.residual[size_t(b0 + c0 + j) * p.ldr + a];
              }
            }
          }
          if (p.out_is_bf16) {
            bf16* dst = reinterpret_cast<bf16*>(p.out) + size_t(b0 + c0) * p.ldo + a;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (j < nb) dst[size_t(j) * p.ldo] = __float2bfloat16_rn(v[j]);
            }
          } else {
            float* dst = reinterpret_cast<float*>(p.out) + size_t(b0 + c0) * p.ldo + a;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (j < nb) dst[size_t(j) * p.ldo] = v[j];
            }
          }
        }
      }
    }
  }

  cta_stamp(p, 5);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  // A CTA whose tile is still being copied out of its shared memory must not leave: the leader
  // comes here after it has received every tile, the others wait for it here.
  if (p.splits > 1) cluster_sync();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// ---- the pair form: two CTAs, 256 x BN tiles, one after another -----------------------------
//
// For many tokens the product is bound by what the SMs can pull from L2 and by the shared-memory
// reads of the tensor core, so the tile is doubled without doubling any CTA's loads: the two CTAs
// of a cluster each hold 128 token rows and HALF of the weight tile's columns, and the leader's
// MMA warp issues tcgen05.mma.cta_group::2, which reads both CTAs' shared memory and writes each
// CTA's 128 x BN accumulator into its own tensor memory. Per CTA and k-block that is 16 KB of
// tokens + BN/2 x 128 B of weights for 128 x BN x 64 multiply-adds: half the bytes per flop of
// the single-CTA tile of the same width.
//
// The kernel is persistent: a pair takes tiles pair, pair + n_pairs, ... and keeps TWO
// accumulators in tensor memory, so that the eight epilogue warps write tile i out while the
// products of tile i + 1 run. The ring of stages runs on across tiles.
//
// Barriers. `full[s]` (leader's): both CTAs' TMA loads signal it (the loads carry .cta_group::2,
// which lets the barrier lie in the peer CTA). `empty[s]`, `acc_full[b]` (each CTA's own): the
// leader's commits arrive on both CTAs' (multicast commit). `acc_empty[b]` (leader's): every
// epilogue warp of both CTAs arrives on it once it has read accumulator b. Both CTAs allocate
// and free tensor memory as a pair. Waits are bounded as in the single-CTA kernel.

__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrives on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs
// issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(uint16_t(3)) : "memory");
}

// One arrival on a barrier given by its address in the cluster's shared memory (possibly the
// peer's). Relaxed: it hands over tensor memory that this warp has finished reading (ordered by
// tcgen05.wait::ld and the tcgen05 fence before it), and must not wait for the warp's global
// stores, as a release would.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}

constexpr int PAIR_THREADS = 320;        // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-9: epilogue
constexpr int PAIR_EPILOGUE_WARPS = 8;
constexpr int PAIR_SLAB_BYTES = PAIR_EPILOGUE_WARPS * STAGING_WORDS * 4;

template <bool B_MN>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int half = p.bn / 2;                              // weight columns held by one CTA
  const uint32_t a_bytes = BM * BK * 2;
  const uint32_t b_bytes = uint32_t(half) * BK * 2;       // a multiple of 1024: half is a multiple of 8
  uint8_t* a_tiles = smem;
  uint8_t* b_tiles = smem + size_t(p.stages) * a_bytes;
  uint8_t* slabs = b_tiles + size_t(p.stages) * b_bytes;  // the epilogue warps' staging rows
  uint64_t* full = reinterpret_cast<uint64_t*>(slabs + PAIR_SLAB_BYTES);
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* acc_full = empty + MAX_STAGES;                // [2]
  uint64_t* acc_empty = acc_full + 2;                     // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  float* bias_s = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(tmem_slot + 4) + 15) & ~uintptr_t(15));  // the tile's bias, BIAS_SLOTS floats

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;  // the cluster lies along x
  const int n_kb = p.n_kb;
  uint32_t tmem_cols = 32;
  while (tmem_cols < 2u * uint32_t(p.bn)) tmem_cols <<= 1;      // two accumulators

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 2 * PAIR_EPILOGUE_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync();  // both CTAs' barriers exist before either's loads, commits or arrivals signal them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  // The next kernel may start (set up, prefetch its weights) from here on, and not earlier: its
  // CTAs allocate tensor memory before they wait for this kernel, so a CTA of this kernel that
  // still had to allocate could find every column taken by CTAs that wait for it.
  pdl_launch_dependents();

  const uint32_t a_base = smem_u32(a_tiles), b_base = smem_u32(b_tiles);
  const uint32_t full_base = smem_u32(full), empty_base = smem_u32(empty);
  const uint32_t acc_full_base = smem_u32(acc_full);
  uint32_t leader_full_base, leader_acc_empty_base;  // the leader's barriers as seen from this CTA
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(leader_full_base) : "r"(full_base), "r"(0u));
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(leader_acc_empty_base) : "r"(smem_u32(acc_empty)), "r"(0u));
  const uint32_t pair_bytes = 2u * (a_bytes + b_bytes);  // what both CTAs bring into one stage

  if (warp == 0) {
    // ---- producer: the warp runs the loop, one elected lane issues. A stage is waited for with
    // the opposite of the ring's parity, which a fresh barrier passes at once. -----------------
    int stage = 0;
    uint32_t parity = 0, a_dst = a_base, b_dst = b_base;
    bool waited = false, ok = true;
    for (int tile = pair; tile < p.n_tiles && ok; tile += n_pairs) {
      const int a0 = ((tile / p.col_tiles) * 2 + int(rank)) * BM;
      const int b0 = (tile % p.col_tiles) * p.bn + int(rank) * half;
      for (int kb = 0; kb < n_kb; ++kb) {
        if (!mbar_wait(empty_base + uint32_t(stage) * 8u, parity ^ 1u)) {
          if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_EMPTY);
          ok = false;
          break;
        }
        const uint32_t bar = leader_full_base + uint32_t(stage) * 8u;
        const int k0 = kb * BK;
        auto load_weights = [&]() {
          if (rank == 0) mbar_expect_tx(full_base + uint32_t(stage) * 8u, pair_bytes);
          if (B_MN) {
            uint32_t dst = b_dst;
            for (int j = 0; j < half; j += 64, dst += BK * 128) tma_load_2d_pair(dst, &map_b, b0 + j, k0, bar);
          } else {
            tma_load_2d_pair(b_dst, &map_b, k0, b0, bar);
          }
        };
        if (waited) {
          if (elect_one()) {
            load_weights();
            tma_load_2d_pair(a_dst, &map_a, k0, a0, bar);
          }
        } else {
          // the weights of the first k-block go on their way; the tokens may have been written by
          // the previous kernel, so they are asked for only once it has completed
          if (elect_one()) load_weights();
          pdl_wait();
          waited = true;
          if (elect_one()) tma_load_2d_pair(a_dst, &map_a, k0, a0, bar);
        }
        __syncwarp();
        a_dst += a_bytes;
        b_dst += b_bytes;
        if (++stage == p.stages) {
          stage = 0;
          parity ^= 1u;
          a_dst = a_base;
          b_dst = b_base;
        }
      }
    }
  } else if (warp == 1 && rank == 0) {
    // ---- MMA issuer of the pair (M = 256 over the two CTAs, N = bn): the warp runs the loop, one
    // elected lane issues ------------------------------------------------------------------------
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(B_MN) << 16) | (uint32_t(p.bn >> 3) << 17) |
                           (uint32_t((2 * BM) >> 4) << 24);
    const uint64_t da_fixed = smem_desc(0, 16, 1024);
    const uint64_t db_fixed = B_MN ? smem_desc(0, BK * 128, 1024) : smem_desc(0, 16, 1024);
    constexpr uint32_t a_step = 32 >> 4, b_step = (B_MN ? UMMA_K * 128 : 32) >> 4;
    int stage = 0;
    const uint32_t a_first = (a_base >> 4) & 0x3FFFu, b_first = (b_base >> 4) & 0x3FFFu;
    uint32_t parity = 0, a_at = a_first, b_at = b_first;
    bool ok = true;
    int local = 0;  // this pair's count of tiles: accumulator local & 1, its use number local >> 1
    for (int tile = pair; tile < p.n_tiles && ok; tile += n_pairs, ++local) {
      const uint32_t buf = uint32_t(local & 1);
      // the epilogue warps have read this accumulator's previous tile (a fresh barrier passes)
      if (!mbar_wait(smem_u32(acc_empty) + buf * 8u, (uint32_t(local >> 1) & 1u) ^ 1u)) {
        if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_ACC);
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t acc = tmem_base + buf * uint32_t(p.bn);
      for (int kb = 0; kb < n_kb; ++kb) {
        if (!mbar_wait(full_base + uint32_t(stage) * 8u, parity)) {
          if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_FULL);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            umma_bf16_pair(acc, da_fixed + uint64_t(a_at + kk * a_step), db_fixed + uint64_t(b_at + kk * b_step), idesc,
                           (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit_pair(empty_base + uint32_t(stage) * 8u);
        }
        __syncwarp();
        a_at += a_bytes >> 4;
        b_at += b_bytes >> 4;
        if (++stage == p.stages) {
          stage = 0;
          parity ^= 1u;
          a_at = a_first;
          b_at = b_first;
        }
      }
      // also on the error path: the epilogues go on and the flag tells
      if (elect_one()) umma_commit_pair(acc_full_base + buf * 8u);
      __syncwarp();
    }
  } else if (warp >= 2) {
    // ---- epilogue: each CTA writes its own 128 rows of each tile's bn columns ------------------
    pdl_wait();
    const int q = warp & 3;              // the accumulator rows (tensor-memory lanes) this warp may read
    const int side = (warp - 2) >> 2;    // warps 2..5 take the tile's first half of the columns, 6..9 the second
    const uint32_t slab = smem_u32(slabs) + uint32_t((warp - 2) * STAGING_WORDS) * 4u;
    bool ok = true;
    int local = 0;
    for (int tile = pair; tile < p.n_tiles; tile += n_pairs, ++local) {
      const uint32_t buf = uint32_t(local & 1);
      const int a0 = ((tile / p.col_tiles) * 2 + int(rank)) * BM;
      const int b_tile0 = (tile % p.col_tiles) * p.bn;
      // the tile's bias, once for the eight warps: after all have finished the previous tile
      asm volatile("bar.sync 1, %0;" ::"n"(PAIR_EPILOGUE_WARPS * 32) : "memory");
      for (int j = int(threadIdx.x) - 64; j < p.bn; j += PAIR_EPILOGUE_WARPS * 32) {
        bias_s[j] = (p.bias != nullptr && b_tile0 + j < p.b_total) ? p.bias[b_tile0 + j] : 0.f;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(PAIR_EPILOGUE_WARPS * 32) : "memory");
      if (ok && !mbar_wait(acc_full_base + buf * 8u, uint32_t(local >> 1) & 1u)) {
        if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_ACC);
        ok = false;  // this and the later tiles are not written; the flag tells
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (ok && a0 + q * 32 < p.a_total) {
        const uint32_t lane_addr = tmem_base + buf * uint32_t(p.bn) + (uint32_t(q * 32) << 16);
        finish_tile_rows(p, lane_addr, slab, bias_s, a0 + q * 32, b_tile0, side * half, (side + 1) * half, lane, true);
      }
      // this warp has read the accumulator: the leader may overwrite it with the tile after next
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_acc_empty_base + buf * 8u);
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync();  // neither CTA frees tensor memory or leaves while the other may still use it
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// ---- host side ------------------------------------------------------------------------------

// A 2-D bfloat16 tensor [outer, inner] with row stride `ld` elements; boxes of box_inner x box_outer.
bool make_map(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner, uint32_t box_outer) {
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  return r2::encode_bf16_map(map, base, 2, dims, strides, box);
}

template <bool A_MN, bool B_MN, bool TRANSPOSED, bool FUSED_LN = false>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid, size_t smem, cudaStream_t stream) {
  auto kernel = gemm_tc_kernel<A_MN, B_MN, TRANSPOSED, FUSED_LN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return int(e);
    // all of the SM's on-chip memory as shared memory: two CTAs of ~110 KB fit side by side
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    configured = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (p.splits > 1) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 1;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = unsigned(p.splits);
    ++n_attr;
  }
  if (g_r2_pdl) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  config.attrs = attr;
  config.numAttrs = n_attr;
  cudaError_t e = cudaLaunchKernelEx(&config, kernel, ma, mb, p);
  if (e != cudaSuccess) return int(e);
  return launch_status();
}

struct Plan {
  bool swapped;
  int a_total, b_total, bn, n_kb, splits, kb_per_split, stages;
  size_t smem;
};

// How many clusters of `size` CTAs (one CTA per SM at this shared-memory use) the GPU can hold at
// once: an SM group that a cluster must fit into does not always divide evenly, so it is asked, not
// computed. Queried once per size.
int max_resident_clusters(int size) {
  static int cached[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
  if (size < 1 || size > 8) return 0;
  if (cached[size] == 0) {
    auto kernel = gemm_tc_kernel<true, false, true>;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(1, 1, size);
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = 120 * 1024;  // more than half an SM's: one CTA per SM, as the plan assumes
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = unsigned(size);
    config.attrs = attr;
    config.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &config) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = n_sms() / size / 2;  // a cautious guess
    }
    cached[size] = n;
  }
  return cached[size];
}

Plan make_plan(int m, int n, int k, int w_is_nk, bool fused_ln = false) {
  Plan pl;
  pl.swapped = m <= 64;
  pl.a_total = pl.swapped ? n : m;
  pl.b_total = pl.swapped ? m : n;
  if (pl.swapped) {
    pl.bn = ((pl.b_total + 15) / 16) * 16;               // tokens, K-major: any multiple of 16
    // more than 32 tokens and few feature tiles: two token tiles double the CTAs that stream the
    // weights (the second pass over a weight tile comes from L2) and halve the leader's reduce buffer
    if (pl.b_total > 32 && ((pl.a_total + BM - 1) / BM) * 8 < n_sms()) pl.bn = 32;
  } else if (w_is_nk) {
    pl.bn = pl.b_total >= 128 ? 128 : ((pl.b_total + 15) / 16) * 16;
  } else {
    pl.bn = pl.b_total > 64 ? 128 : 64;                   // MN-major boxes are 64 features wide
  }
  const int tiles = ((pl.a_total + BM - 1) / BM) * ((pl.b_total + pl.bn - 1) / pl.bn);
  pl.n_kb = (k + BK - 1) / BK;
  // A CTA streams its K range at well under 100 GB/s, so a product with few tiles uses the CTAs
  // of a cluster (at most 8) on one tile, each with a share of K; the leader's shared memory
  // must hold the others' partial tiles.
  pl.splits = 1;
  if (pl.swapped && tiles * 2 <= n_sms()) {
    int s = n_sms() / tiles;
    if (s > 8) s = 8;
    if (s > pl.n_kb) s = pl.n_kb;
    for (; s > 1; --s) {
      if (size_t(s - 1) * (pl.bn + 4) * BM * 4 > 100 * 1024) continue;  // the leader's reduce buffer
      int per = (pl.n_kb + s - 1) / s;
      int actual = (pl.n_kb + per - 1) / per;
      if (actual != s) continue;                                  // the same split with fewer CTAs comes later
      if (tiles <= max_resident_clusters(s)) break;               // all clusters run at once
    }
    if (s < 1) s = 1;
    pl.splits = s;
  }
  pl.kb_per_split = (pl.n_kb + pl.splits - 1) / pl.splits;
  const size_t a_bytes = BM * BK * 2, b_stride = (size_t(pl.bn) * BK * 2 + 1023) & ~size_t(1023);
  const size_t fixed = 1024 + (2 * MAX_STAGES + 3) * 8 + 32 +
                       (pl.swapped ? size_t(pl.splits - 1) * (pl.bn + 4) * BM * 4 : size_t(BIAS_SLOTS) * 4);  // partial sums, or the bias
  // with more tiles than SMs, leave room for two CTAs on an SM: one's epilogue under the other's loads
  const size_t budget = (tiles * pl.splits > n_sms() ? 113 * 1024 : 227 * 1024) - fixed;
  if (fused_ln) {
    // the normalised token tiles of the CTA's whole K share stay resident; the ring holds weights only
    const size_t tokens = size_t(pl.kb_per_split) * b_stride;
    int stages = tokens + a_bytes <= budget ? int((budget - tokens) / a_bytes) : 0;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages > pl.kb_per_split) stages = pl.kb_per_split;
    pl.stages = stages;  // 0: does not fit
    pl.smem = fixed + tokens + size_t(stages) * a_bytes;
    return pl;
  }
  int stages = int(budget / (a_bytes + b_stride));
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages > pl.kb_per_split) stages = pl.kb_per_split;
  if (stages < 1) stages = 1;
  // the token-major epilogue lays its four slabs over the tiles: a short K keeps stages it does not fill
  while (!pl.swapped && size_t(stages) * (a_bytes + b_stride) < 4 * size_t(STAGING_WORDS) * 4) ++stages;
  pl.stages = stages;
  pl.smem = fixed + size_t(stages) * (a_bytes + b_stride);
  return pl;
}

// The pair form: tile width (256, or 128 when that gives too few CTAs), stages, shared memory.
struct PairPlan {
  bool use;
  int bn, n_kb, stages, n_tiles, col_tiles;
  size_t smem;
  dim3 grid;
};

// How many CTA pairs the GPU holds at once (one CTA to an SM at this kernel's shared-memory use).
int max_resident_pairs() {
  static int cached = 0;
  if (cached == 0) {
    auto kernel = gemm_tc_pair_kernel<true>;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2, 1, 1);
    config.blockDim = dim3(PAIR_THREADS);
    config.dynamicSmemBytes = 200 * 1024;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &config) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = n_sms() / 2 - 2;  // a cautious guess
    }
    cached = n;
  }
  return cached;
}

PairPlan make_pair_plan(int m, int n, int k, int w_is_nk, bool always) {
  PairPlan pl;
  pl.use = false;
  if (m < 192 || n < 128) return pl;  // the second CTA of a pair would hold (almost) no rows, or the tile no columns
  (void)w_is_nk;
  // Measured at 512 to 8,192 rows (K 768 and 3,072, N 768 to 3,072): the persistent pairs reach
  // 0.9 to 1.3 PFLOP/s once every pair has several tiles, but pay about a microsecond more of
  // set-up and an epilogue that nothing hides; with fewer than about 2.5 single-CTA tiles per SM
  // the single-CTA form (two CTAs to an SM) is the faster one.
  const int single_tiles = ((m + BM - 1) / BM) * ((n + 127) / 128);
  if (!always && 2 * single_tiles < 5 * n_sms()) return pl;
  const int row_pairs = (m + 2 * BM - 1) / (2 * BM);
  const int pairs = max_resident_pairs();
  pl.n_kb = (k + BK - 1) / BK;
  // Tile width by a small model of the pair's time, in cycles measured on a B200: a k-block takes
  // about 545 (width 256, bound by the tensor core) or 361 (width 128, bound by the issue of its
  // four MMAs), and the last tile's epilogue, which nothing hides, about 3,900 or 2,000.
  long best = -1;
  pl.bn = 128;
  for (int bn = 256; bn >= 128; bn -= 128) {
    if (n < bn) continue;
    const long tiles = long(row_pairs) * ((n + bn - 1) / bn);
    const long rounds = (tiles + pairs - 1) / pairs;
    const long cost = rounds * pl.n_kb * (bn == 256 ? 545 : 361) + (bn == 256 ? 3900 : 2000);
    if (best < 0 || cost < best) {
      best = cost;
      pl.bn = bn;
    }
  }
  pl.col_tiles = (n + pl.bn - 1) / pl.bn;
  pl.n_tiles = row_pairs * pl.col_tiles;
  const size_t stage = size_t(BM) * BK * 2 + size_t(pl.bn / 2) * BK * 2;
  const size_t fixed = 1024 + size_t(PAIR_SLAB_BYTES) + (2 * MAX_STAGES + 4) * 8 + 48 + size_t(BIAS_SLOTS) * 4;
  const size_t budget = 227 * 1024 - fixed;  // one CTA per SM: its eight epilogue warps need the registers
  int stages = int(budget / stage);
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages < 1) return pl;
  pl.stages = stages;
  pl.smem = fixed + size_t(stages) * stage;
  pl.grid = dim3(2 * unsigned(pl.n_tiles < pairs ? pl.n_tiles : pairs), 1, 1);
  pl.use = true;
  return pl;
}

template <bool B_MN>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, const PairPlan& pl, cudaStream_t stream) {
  auto kernel = gemm_tc_pair_kernel<B_MN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return int(e);
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    configured = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = pl.grid;
  config.blockDim = dim3(PAIR_THREADS);
  config.dynamicSmemBytes = pl.smem;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  attr[n_attr].id = cudaLaunchAttributeClusterDimension;
  attr[n_attr].val.clusterDim.x = 2;
  attr[n_attr].val.clusterDim.y = 1;
  attr[n_attr].val.clusterDim.z = 1;
  ++n_attr;
  if (g_r2_pdl) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  config.attrs = attr;
  config.numAttrs = n_attr;
  cudaError_t e = cudaLaunchKernelEx(&config, kernel, ma, mb, p);
  if (e != cudaSuccess) return int(e);
  return launch_status();
}

long long* g_cta_stamps = nullptr;  // (r2_gemm_tc_set_cta_stamps)
int g_cta_stamps_cap = 0, g_last_grid = 0;

int g_pair_form = 1;  // 0: never, 1: where it is the faster form, 2: wherever it can run (r2_gemm_tc_set_pair; tests compare the forms)

}  // namespace

// Profiling: launches from now on leave six times per CTA in `buffer` ([cap][6] int64 on the device; null: off).
// Returns the number of CTAs of the last launch of a single-CTA form.
extern "C" int r2_gemm_tc_set_cta_stamps(long long* buffer, int cap) {
  g_cta_stamps = buffer;
  g_cta_stamps_cap = buffer != nullptr ? cap : 0;
  return g_last_grid;
}

extern "C" int r2_gemm_tc_set_pair(int mode) {
  int before = g_pair_form;
  g_pair_form = mode < 0 ? 0 : (mode > 2 ? 2 : mode);
  return before;
}

// How r2_gemm_tc would run (m, n, k): tile width on the b side, CTAs per cluster (slices of K), stages.
extern "C" int r2_gemm_tc_plan(int m, int n, int k, int w_is_nk, int* bn_out, int* splits_out, int* stages_out) {
  Plan pl = make_plan(m, n, k, w_is_nk);
  *bn_out = pl.bn;
  *splits_out = pl.splits;
  *stages_out = pl.stages;
  return R2_OK;
}

// x [m, k] bfloat16 (row stride lda), w [k, n] or [n, k] bfloat16 (row stride ldw), bias [n] float or null,
// residual [m, n] float or null, out [m, n] bfloat16 or float. Returns R2_UNSUPPORTED for shapes
// whose rows are not 16-byte multiples; the caller then uses the CUDA-core kernel.
//
// With ln_x != null the tokens are LayerNorm(ln_x[ln_rows[i]] or ln_x[i]) computed inside the kernel
// (`x` is then ignored); this form takes at most 16 tokens and k <= 1024, else R2_UNSUPPORTED.
// `prefetch` (may be null) names memory, typically the next product's weight, that the kernel asks into L2.
extern "C" int r2_gemm_tc(const void* x, int lda, const void* w, int ldw, int w_is_nk, const float* bias,
                          const float* residual, int ldr, void* out, int ldo, int m, int n, int k, int act,
                          int out_dtype, int* error_flag, const float* ln_x, int ln_ldx, const int32_t* ln_rows,
                          const float* ln_gamma, const float* ln_beta, float ln_eps, const void* prefetch,
                          long long prefetch_bytes, const R2KvScatter* kv, cudaStream_t stream) {
  if (m <= 0 || n <= 0) return R2_OK;
  const bool fused_ln = ln_x != nullptr;
  if (fused_ln) {
    if (m > LN_MAX_TOKENS || k > LN_MAX_K || k % 8 != 0 || ln_ldx % 4 != 0 || ln_gamma == nullptr || ln_beta == nullptr) return R2_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(ln_x) & 15) || (reinterpret_cast<uintptr_t>(ln_gamma) & 15) || (reinterpret_cast<uintptr_t>(ln_beta) & 15)) return R2_UNSUPPORTED;
    x = w;  // only its alignment is looked at below
    lda = 8;
  }
  if (k < 1) return R2_BAD_SHAPE;
  if (act < R2_ACT_NONE || act > R2_ACT_GELU_ERF) return R2_UNSUPPORTED;
  if (out_dtype != R2_F32 && out_dtype != R2_BF16) return R2_BAD_DTYPE;
  if (error_flag == nullptr) return R2_BAD_SHAPE;
  if (lda % 8 != 0 || ldw % 8 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return R2_UNSUPPORTED;
  if (k % 8 != 0 || (!w_is_nk && n % 8 != 0)) return R2_UNSUPPORTED;
  const Plan pl = make_plan(m, n, k, w_is_nk, fused_ln);
  if (pl.stages < 1) return R2_UNSUPPORTED;
  GemmParams p;
  p.ln_x = ln_x;
  p.ln_ldx = ln_ldx;
  p.ln_rows = ln_rows;
  p.ln_gamma = ln_gamma;
  p.ln_beta = ln_beta;
  p.ln_eps = ln_eps;
  const bool prefetch_ok = prefetch != nullptr && prefetch_bytes >= 16 && !(reinterpret_cast<uintptr_t>(prefetch) & 15);
  p.prefetch = prefetch_ok ? static_cast<const uint8_t*>(prefetch) : nullptr;
  p.prefetch_bytes = prefetch_ok ? prefetch_bytes : 0;
  p.kv_slots = nullptr;
  if (kv != nullptr) {
    // keys and values straight into the cache: token-major bfloat16 output without activation or
    // residual only, 16-byte pieces that never straddle a head or the boundary between q, k and v
    const bool fits = m > 64 && !fused_ln && out_dtype == R2_BF16 && residual == nullptr && act == R2_ACT_NONE &&
                      kv->head_dim % 8 == 0 && kv->width % kv->head_dim == 0 && kv->col % 8 == 0 && kv->col + 2 * kv->width == n &&
                      kv->page_stride % 8 == 0 && kv->page_size >= 1 && !(reinterpret_cast<uintptr_t>(kv->k_cache) & 15) &&
                      !(reinterpret_cast<uintptr_t>(kv->v_cache) & 15);
    if (!fits) return R2_UNSUPPORTED;
    p.kv_slots = kv->slots;
    p.kv_k = static_cast<bf16*>(kv->k_cache);
    p.kv_v = static_cast<bf16*>(kv->v_cache);
    p.kv_page_stride = kv->page_stride;
    p.kv_page_size = kv->page_size;
    p.kv_page_shift = page_shift_of(kv->page_size);
    p.kv_n_pages = kv->n_pages;
    p.kv_col = kv->col;
    p.kv_width = kv->width;
    p.kv_head_dim = kv->head_dim;
    p.kv_head_shift = (kv->head_dim & (kv->head_dim - 1)) == 0 ? page_shift_of(kv->head_dim) : -1;
  }
  p.cta_stamps = g_cta_stamps;
  p.cta_stamps_cap = g_cta_stamps_cap;
  p.a_total = pl.a_total;
  p.b_total = pl.b_total;
  p.k_total = k;
  p.bn = pl.bn;
  p.n_kb = pl.n_kb;
  p.splits = pl.splits;
  p.kb_per_split = pl.kb_per_split;
  p.stages = pl.stages;
  p.bias = bias;
  p.residual = residual;
  p.ldr = ldr;
  p.out = out;
  p.ldo = ldo;
  p.out_is_bf16 = out_dtype == R2_BF16;
  p.act = act;
  p.error_flag = error_flag;
  const int bn = pl.bn;
  const size_t smem = pl.smem;
  dim3 grid((p.a_total + BM - 1) / BM, (p.b_total + bn - 1) / bn, pl.splits);

  if (!pl.swapped && !fused_ln && g_pair_form != 0) {
    const PairPlan pp = make_pair_plan(m, n, k, w_is_nk, g_pair_form == 2);
    if (pp.use) {
      p.bn = pp.bn;
      p.stages = pp.stages;
      p.splits = 1;
      p.kb_per_split = pp.n_kb;
      p.n_tiles = pp.n_tiles;
      p.col_tiles = pp.col_tiles;
      CUtensorMap pa, pb;
      bool maps = make_map(&pa, x, uint64_t(k), uint64_t(m), uint64_t(lda), BK, BM);
      if (w_is_nk) {
        maps = maps && make_map(&pb, w, uint64_t(k), uint64_t(n), uint64_t(ldw), BK, uint32_t(pp.bn / 2));
        if (maps) return launch_pair<false>(pa, pb, p, pp, stream);
      } else {
        maps = maps && make_map(&pb, w, uint64_t(n), uint64_t(k), uint64_t(ldw), 64, BK);
        if (maps) return launch_pair<true>(pa, pb, p, pp, stream);
      }
      p.bn = pl.bn;  // no tensor map: the single-CTA form decides
      p.stages = pl.stages;
      p.splits = pl.splits;
      p.kb_per_split = pl.kb_per_split;
    }
  }

  g_last_grid = int(grid.x * grid.y * grid.z);
  CUtensorMap ma, mb;
  bool ok;
  if (!pl.swapped) {
    // a side: tokens [m, k] K-major; b side: the weight
    ok = make_map(&ma, x, uint64_t(k), uint64_t(m), uint64_t(lda), BK, BM);
    if (w_is_nk) {
      ok = ok && make_map(&mb, w, uint64_t(k), uint64_t(n), uint64_t(ldw), BK, uint32_t(bn));
      if (!ok) return R2_UNSUPPORTED;
      return launch<false, false, false>(ma, mb, p, grid, smem, stream);
    }
    ok = ok && make_map(&mb, w, uint64_t(n), uint64_t(k), uint64_t(ldw), 64, BK);
    if (!ok) return R2_UNSUPPORTED;
    return launch<false, true, false>(ma, mb, p, grid, smem, stream);
  }
  // swapped: a side = the weight's features, b side = tokens [m, k] K-major
  ok = fused_ln ? make_map(&mb, w, 64, 64, 64, BK, 16)  // a placeholder map: the kernel never uses it
                : make_map(&mb, x, uint64_t(k), uint64_t(m), uint64_t(lda), BK, uint32_t(bn));
  if (w_is_nk) {
    ok = ok && make_map(&ma, w, uint64_t(k), uint64_t(n), uint64_t(ldw), BK, BM);
    if (!ok) return R2_UNSUPPORTED;
    return fused_ln ? launch<false, false, true, true>(ma, mb, p, grid, smem, stream)
                    : launch<false, false, true>(ma, mb, p, grid, smem, stream);
  }
  ok = ok && make_map(&ma, w, uint64_t(n), uint64_t(k), uint64_t(ldw), 64, BK);
  if (!ok) return R2_UNSUPPORTED;
  return fused_ln ? launch<true, false, true, true>(ma, mb, p, grid, smem, stream)
                  : launch<true, false, true>(ma, mb, p, grid, smem, stream);
}
