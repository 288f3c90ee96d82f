// A feed-forward for a few rows (a decode step) as ONE kernel, bfloat16 on tcgen05:
//     out = residual + act(LayerNorm(x) W1 + b1) W2 + b2
// Two matrix products with a dependency between them are otherwise two kernels, each on a
// floor of several microseconds, for 9 MB of weights that the memory system delivers in two.
//
// CTA c owns 64 of the hidden features. Before it waits for the previous kernel it asks for
// both of its weight slices, W1[:, 64c .. 64c+64) and W2[64c .. 64c+64, :], which then lie in
// shared memory whole (no ring): the weights of a layer are in flight under the previous
// kernel's tail. After the wait:
//   warps 2-5  normalise the rows (statistics in float, two passes over registers, as
//              kelpie-models/kelpie_models/kernels/ops/layer_norm.py:21-23) into K-major token
//              tiles in shared memory, the B operand of the first product;
//   warp 1     first product (features x tokens, 128 x 16 per instruction, operands swapped so
//              that the 64 hidden features are accumulator rows): acc1[64, tokens];
//   warps 2-3  bias, activation, bfloat16: the hidden activations become the K-major B operand
//              (tokens x 64) of the second product, in shared memory, never in global memory;
//   warp 1     second product: this CTA's share of out^T[n_out, tokens] over its 64 hidden
//              features, n_out / 128 accumulators in tensor memory;
//   warps 2-5  write that partial result to shared memory.
// The sum over the hidden dimension is a sum over CTAs. Inside a cluster of 8 it is a
// reduce-scatter through distributed shared memory: every CTA sends slice j of its partial to
// CTA j with one bulk copy counted on j's mbarrier, and adds the eight slices it received in
// rank order. Across the clusters (hidden / 512 of them) the slices go through global memory:
// a cluster's CTA j writes its slice, and the last cluster to arrive at slice j's counter adds
// all of them in cluster order with bias and residual and writes the output rows. Both sums
// have a fixed order: the result is the same bits every run.
//
// Measured (8 rows, 768 -> 3,072 -> 768, one B200): 9.7 us alone and 17.3 us per launch inside a
// CUDA graph of such launches, against 6.9 + 4.9 us for the two products as kernels of their own,
// so the engine does not use it unless it is switched on. `clock64` stamps of one CTA say why: the
// second weight slice has landed only 10,300 cycles after entry. 192 KB through one SM's tensor
// copies in 128-byte rows arrive at about 19 bytes a cycle, and 48 SMs pull the layer's 9.4 MB
// no faster than that, where the separate products spread the same bytes over 144 and 48 CTAs
// with half as much each. The second product, 24 instructions into six accumulators, takes
// 1,150 cycles to issue; the exchange and the combine take 5,000 to 6,000 more. What would make
// this form pay is twice as many CTAs with 32 hidden features each (64-byte swizzled boxes).
//
// Formulas: kelpie-models/kelpie_models/models/torch/gpt2.py:94-96. Every wait on an mbarrier
// is bounded; on time-out an error code is recorded, the roles go on without the data (the
// output is then wrong and the caller sees the code), tensor memory is freed, the kernel returns.
#include <cuda.h>
#include <math.h>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tensor_maps.cuh"

namespace {

using namespace r2ptx;

constexpr int THREADS = 192;
constexpr int HS = 64;            // hidden features per CTA
constexpr int BK = 64;            // k-block: 64 bfloat16 = one 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int CLUSTER = 8;
constexpr int MAX_TOKENS = 16;    // one 16-column accumulator per 128 output features
constexpr int MAX_K = 1024;       // a row of x is held in registers while it is normalised
constexpr int LN_CHUNKS = MAX_K / 128;
constexpr int ATOM_BYTES = 64 * 128;   // 64 rows of 128 bytes: one box of a weight slice
constexpr int TOKEN_TILE_BYTES = MAX_TOKENS * 128;
#define R2_ERR_TIMEOUT_MLP 7

struct MlpParams {
  const float* x; int ldx; const int32_t* rows; const float* gamma; const float* beta; float eps;
  int n_tokens, k, hidden, n_out;
  const float* b1; const float* b2;
  const float* residual; int ldr;
  float* out; int ldo;
  int act;
  float* scratch;        // [clusters][n_out][live] the clusters' sums
  unsigned int* counters;  // [CLUSTER], zero between launches
  int n_clusters;
  int* error_flag;
};

__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// gelu_new through one fast exponential (the value is rounded to bfloat16 next), as the
// separate product's epilogue has it.
__device__ __forceinline__ float gelu_tanh_fast(float x) {
  const float k = 0.7978845608028654f;
  float u = k * (x + 0.044715f * x * x * x);
  float e = __expf(2.f * u);
  float t = 1.f - __fdividef(2.f, e + 1.f);
  return 0.5f * x * (1.f + t);
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

// LayerNorm of the rows into K-major token tiles [k-block][token][64 k], 128-byte swizzle: warp w
// of four takes rows w, w + 4, ... two at a time. Rows past the last token are left as they are:
// their columns of the products are never read.
__device__ __forceinline__ void build_normed_tokens(const MlpParams& p, uint8_t* tiles, int w, int lane, const float4 (&gam)[LN_CHUNKS],
                                                    const float4 (&bet)[LN_CHUNKS], const int (&src_first)[2]) {
  const int k_total = p.k;
  const float inv_k = 1.f / float(k_total);
  for (int r0 = w; r0 < p.n_tokens; r0 += 8) {
    float4 v[2][LN_CHUNKS];
    bool live[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int r = r0 + 4 * u;
      live[u] = r < p.n_tokens;
      int src = 0;
      if (live[u]) src = r0 == w ? src_first[u] : (p.rows != nullptr ? p.rows[r] : r);
      const float4* row = reinterpret_cast<const float4*>(p.x + size_t(src) * p.ldx);
#pragma unroll
      for (int i = 0; i < LN_CHUNKS; ++i) {
        const int k = (lane + 32 * i) * 4;
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
      const int k = (lane + 32 * i) * 4;
      if (k < k_total) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const float a = v[u][i].x - mean[u], b = v[u][i].y - mean[u], c = v[u][i].z - mean[u], d = v[u][i].w - mean[u];
          sq[u] += a * a + b * b + c * c + d * d;
        }
      }
    }
    warp_sum2(sq[0], sq[1]);
    const float rstd[2] = {1.f / sqrtf(sq[0] * inv_k + p.eps), 1.f / sqrtf(sq[1] * inv_k + p.eps)};
#pragma unroll
    for (int i = 0; i < LN_CHUNKS; ++i) {
      const int k = (lane + 32 * i) * 4;
      if (k >= k_total) continue;
      const int kb = k / BK, kin = k % BK;
      uint8_t* tile = tiles + size_t(kb) * TOKEN_TILE_BYTES;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (!live[u]) continue;
        const int r = r0 + 4 * u;
        const uint32_t lo = pack_bf16((v[u][i].x - mean[u]) * rstd[u] * gam[i].x + bet[i].x, (v[u][i].y - mean[u]) * rstd[u] * gam[i].y + bet[i].y);
        const uint32_t hi = pack_bf16((v[u][i].z - mean[u]) * rstd[u] * gam[i].z + bet[i].z, (v[u][i].w - mean[u]) * rstd[u] * gam[i].w + bet[i].w);
        const uint32_t off = uint32_t(r / 8) * 1024u + uint32_t(r % 8) * 128u + (uint32_t((kin / 8) ^ (r % 8)) * 16u) + uint32_t(kin % 8) * 2u;
        *reinterpret_cast<uint2*>(tile + off) = make_uint2(lo, hi);
      }
    }
  }
}

__global__ void __launch_bounds__(THREADS, 1)
mlp_fused_kernel(const __grid_constant__ CUtensorMap map_w1, const __grid_constant__ CUtensorMap map_w2, const MlpParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int n_kb = p.k / BK;                 // k-blocks of the first product
  const int n_atoms = p.n_out / 64;          // 64-feature boxes of the second weight slice
  const int n_acc = p.n_out / 128;           // accumulators of the second product
  const int live = (p.n_tokens + 3) & ~3;    // token columns that are kept, a multiple of four floats
  uint8_t* w1_s = smem;                                        // [n_kb][64 k][64 features]
  uint8_t* w2_s = w1_s + size_t(n_kb) * ATOM_BYTES;            // [n_atoms][64 hidden][64 features]
  uint8_t* tok_s = w2_s + size_t(n_atoms) * ATOM_BYTES;        // [n_kb][16 tokens][64 k]
  uint8_t* act_s = tok_s + size_t(n_kb) * TOKEN_TILE_BYTES;    // [16 tokens][64 hidden]
  uint64_t* bars = reinterpret_cast<uint64_t*>(act_s + TOKEN_TILE_BYTES);
  // Once the first product has completed the first weight slice is dead: this CTA's partial
  // result [n_out][live] and the eight slices it receives [CLUSTER][n_out / 8][live] lie there.
  float* partial = reinterpret_cast<float*>(w1_s);
  float* received = partial + size_t(p.n_out) * live;
  uint64_t* w1_full = bars;
  uint64_t* w2_full = bars + 1;
  uint64_t* tokens_ready = bars + 2;   // four arrivals: the normalising warps
  uint64_t* acc1_ready = bars + 3;
  uint64_t* act_ready = bars + 4;      // four arrivals
  uint64_t* acc2_ready = bars + 5;
  uint64_t* recv_full = bars + 6;      // counts the bytes of the eight slices
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);
  volatile int* is_last = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int cluster_id = int(blockIdx.x) / CLUSTER;
  const int h0 = int(blockIdx.x) * HS;  // this CTA's hidden features

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(w1_full), 1);
    mbar_init(smem_u32(w2_full), 1);
    mbar_init(smem_u32(tokens_ready), 4);
    mbar_init(smem_u32(acc1_ready), 1);
    mbar_init(smem_u32(act_ready), 4);
    mbar_init(smem_u32(acc2_ready), 1);
    mbar_init(smem_u32(recv_full), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w1) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w2) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(uint32_t(p.n_out >= 896 ? 256 : 128)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_cols = p.n_out >= 896 ? 256u : 128u;   // 16 columns for the first product, 16 per 128 output features
  // (the next kernel's trigger comes after the tensor-memory allocation: its CTAs allocate before they wait)
  pdl_launch_dependents();

  bool ok = true;
  if (warp == 0) {
    // ---- the weights: all of this CTA's, at once, before the wait on the previous kernel -------
    if (elect_one()) {
      mbar_expect_tx(smem_u32(w1_full), uint32_t(n_kb) * ATOM_BYTES);
      for (int kb = 0; kb < n_kb; ++kb) tma_load_2d(smem_u32(w1_s) + uint32_t(kb) * ATOM_BYTES, &map_w1, h0, kb * BK, smem_u32(w1_full));
      mbar_expect_tx(smem_u32(w2_full), uint32_t(n_atoms) * ATOM_BYTES);
      for (int a = 0; a < n_atoms; ++a) tma_load_2d(smem_u32(w2_s) + uint32_t(a) * ATOM_BYTES, &map_w2, a * 64, h0, smem_u32(w2_full));
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---- the products: the warp runs the loops, one elected lane issues ------------------------
    // M = 128 (features), N = 16 (tokens), bfloat16 in, float out; A MN-major (features contiguous:
    // weights stored [in, out]), B K-major. An A tile is two 64-feature boxes 8,192 bytes apart;
    // the first product has one box of features per k-block, so its second box is the next
    // k-block's (or the start of the second slice): rows 64 to 127 of that accumulator are never read.
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (uint32_t(MAX_TOKENS >> 3) << 17) | (uint32_t(128 >> 4) << 24);
    const uint64_t da = smem_desc(0, ATOM_BYTES, 1024), db = smem_desc(0, 16, 1024);
    const uint32_t w1_at = (smem_u32(w1_s) >> 4) & 0x3FFFu, w2_at = (smem_u32(w2_s) >> 4) & 0x3FFFu;
    const uint32_t tok_at = (smem_u32(tok_s) >> 4) & 0x3FFFu, act_at = (smem_u32(act_s) >> 4) & 0x3FFFu;
    if (!mbar_wait(smem_u32(w1_full), 0) || !mbar_wait(smem_u32(tokens_ready), 0)) {
      if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_MLP);
      ok = false;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (elect_one()) {
      for (int kb = 0; kb < n_kb; ++kb) {
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
          umma_bf16(tmem_base, da + uint64_t(w1_at + uint32_t(kb * ATOM_BYTES + kk * UMMA_K * 128) / 16u),
                    db + uint64_t(tok_at + uint32_t(kb * TOKEN_TILE_BYTES + kk * 32) / 16u), idesc, (kb > 0 || kk > 0) ? 1u : 0u);
        }
      }
      umma_commit(smem_u32(acc1_ready));
    }
    __syncwarp();
    if (!mbar_wait(smem_u32(w2_full), 0) || !mbar_wait(smem_u32(act_ready), 0)) {
      if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_MLP);
      ok = false;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (elect_one()) {
      for (int t = 0; t < n_acc; ++t) {
#pragma unroll
        for (int kk = 0; kk < HS / UMMA_K; ++kk) {
          umma_bf16(tmem_base + 16u + uint32_t(t) * 16u, da + uint64_t(w2_at + uint32_t(t * 2 * ATOM_BYTES + kk * UMMA_K * 128) / 16u),
                    db + uint64_t(act_at + uint32_t(kk * 32) / 16u), idesc, kk > 0 ? 1u : 0u);
        }
      }
      umma_commit(smem_u32(acc2_ready));
    }
    __syncwarp();
  } else {
    // ---- rows in, activations across, partial result out ----------------------------------------
    const int q = warp & 3;  // tensor-memory lanes [32q, 32q + 32) belong to warps with id % 4 == q
    const uint32_t lane_addr = tmem_base + (uint32_t(q * 32) << 16);
    float4 gam[LN_CHUNKS], bet[LN_CHUNKS];
#pragma unroll
    for (int i = 0; i < LN_CHUNKS; ++i) {  // weights: fetched before the wait
      const int k = (lane + 32 * i) * 4;
      gam[i] = k < p.k ? __ldg(reinterpret_cast<const float4*>(p.gamma + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
      bet[i] = k < p.k ? __ldg(reinterpret_cast<const float4*>(p.beta + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    int src_first[2] = {-1, -1};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int r = q + 4 * u;
      if (r < p.n_tokens) src_first[u] = p.rows != nullptr ? p.rows[r] : r;
    }
    const float bias1 = q < 2 ? p.b1[h0 + q * 32 + lane] : 0.f;
    pdl_wait();  // the rows come from the previous kernel
    build_normed_tokens(p, tok_s, q, lane, gam, bet, src_first);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes, read by the tensor core
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(tokens_ready));

    if (!mbar_wait(smem_u32(acc1_ready), 0)) {
      if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_MLP);
      ok = false;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (q < 2) {
      // hidden feature f = 32q + lane of this CTA's 64, for the 16 token columns: the K-major
      // tile [token][64 hidden] of the second product
      uint32_t r[16];
      tmem_load16(lane_addr, r);
      const int f = q * 32 + lane;
#pragma unroll
      for (int t = 0; t < MAX_TOKENS; ++t) {
        float v = __uint_as_float(r[t]) + bias1;
        v = p.act == R2_ACT_GELU_TANH ? gelu_tanh_fast(v) : (p.act == R2_ACT_GELU_ERF ? gelu_erf(v) : v);
        const uint32_t off = uint32_t(t / 8) * 1024u + uint32_t(t % 8) * 128u + (uint32_t((f / 8) ^ (t % 8)) * 16u) + uint32_t(f % 8) * 2u;
        *reinterpret_cast<bf16*>(act_s + off) = __float2bfloat16_rn(v);
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(act_ready));

    if (!mbar_wait(smem_u32(acc2_ready), 0)) {
      if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_MLP);
      ok = false;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // (both products have completed: the first weight slice may be overwritten)
    for (int t = 0; t < n_acc; ++t) {
      uint32_t r[16];
      tmem_load16(lane_addr + 16u + uint32_t(t) * 16u, r);
      float* dst = partial + size_t(t * 128 + q * 32 + lane) * live;
#pragma unroll
      for (int j = 0; j < MAX_TOKENS; j += 4) {
        if (j < live) *reinterpret_cast<uint4*>(dst + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes, read by the bulk copies
  }

  // ---- the sum over the hidden features ------------------------------------------------------------
  // Every CTA of the cluster has its partial result complete (and its first weight slice dead) once
  // all have passed this barrier; then slice j of every partial goes to CTA j.
  __syncthreads();
  cluster_sync();
  const int slice_rows = p.n_out / CLUSTER;
  const uint32_t slice_bytes = uint32_t(slice_rows) * uint32_t(live) * 4u;
  if (threadIdx.x == 64) {
    mbar_expect_tx(smem_u32(recv_full), slice_bytes * CLUSTER);
    for (uint32_t j = 0; j < CLUSTER; ++j) {
      const uint32_t peer = (rank + j) % CLUSTER;  // (each CTA starts with itself: the copies spread over the peers)
      uint32_t remote, remote_bar;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(received) + rank * slice_bytes), "r"(peer));
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(smem_u32(recv_full)), "r"(peer));
      asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(remote), "r"(smem_u32(partial) + peer * slice_bytes), "r"(slice_bytes), "r"(remote_bar)
                   : "memory");
    }
  }
  if (warp >= 2) {
    if (!mbar_wait(smem_u32(recv_full), 0)) {
      if (lane == 0) atomicMax(p.error_flag, R2_ERR_TIMEOUT_MLP);
      ok = false;
    }
    // this CTA's slice of the cluster's sum: rows [rank * slice_rows, +slice_rows) x live, in rank order
    const int n_values = slice_rows * live;
    const int first_row = int(rank) * slice_rows;
    float* mine = p.scratch + (size_t(cluster_id) * p.n_out + first_row) * live;
    for (int i = int(threadIdx.x) - 64; i < n_values; i += 128) {
      float v = 0.f;
#pragma unroll
      for (int z = 0; z < CLUSTER; ++z) v += received[size_t(z) * n_values + i];
      mine[i] = v;
    }
    __threadfence();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (threadIdx.x == 64) *is_last = atomicAdd(&p.counters[rank], 1u) == unsigned(p.n_clusters - 1) ? 1 : 0;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (*is_last) {
      // every cluster's slice is in global memory: their sum in cluster order, bias, residual
      __threadfence();
      for (int i = int(threadIdx.x) - 64; i < slice_rows * p.n_tokens; i += 128) {
        const int tkn = i / slice_rows, f = first_row + i % slice_rows;  // consecutive threads, consecutive features
        float v = 0.f;
        for (int c = 0; c < p.n_clusters; ++c) v += __ldcg(p.scratch + (size_t(c) * p.n_out + f) * live + tkn);
        v += p.b2 != nullptr ? p.b2[f] : 0.f;
        if (p.residual != nullptr) v += p.residual[size_t(tkn) * p.ldr + f];
        if (ok) p.out[size_t(tkn) * p.ldo + f] = v;
      }
      if (threadIdx.x == 64) p.counters[rank] = 0u;  // for the next launch
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  // A CTA whose partial is still being copied out of its shared memory must not leave: every CTA
  // comes here after it has received its eight slices.
  cluster_sync();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// A bfloat16 matrix [rows][cols] with row stride ld, in boxes of 64 x 64 (128-byte swizzle).
bool weight_map(CUtensorMap* out, const void* base, long long rows, long long cols, long long ld) {
  cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
  cuuint64_t strides[1] = {cuuint64_t(ld) * 2};
  cuuint32_t box[2] = {64, 64};
  return r2::cached_bf16_map(out, r2::MapKey{base, rows, cols, int(ld), 64, 64, 7}, 2, dims, strides, box);
}

}  // namespace

// out [n_tokens, n_out] float32 = residual + act(LayerNorm(x[rows[i]] or x[i]) w1 + b1) w2 + b2.
// x float32 [*, k] (row stride ldx), w1 [k, hidden] and w2 [hidden, n_out] bfloat16 stored [in, out]
// (row strides in elements), scratch of at least (hidden / 512) * n_out * 16 floats, eight counters
// that are zero between launches. R2_UNSUPPORTED for what this kernel does not take: the caller
// then runs the two products as kernels of their own.
extern "C" int r2_mlp_fused(const float* x, int ldx, const int32_t* rows, const float* gamma, const float* beta, float eps, int n_tokens,
                            int k, const void* w1, int ldw1, const float* b1, int hidden, const void* w2, int ldw2, const float* b2,
                            int n_out, const float* residual, int ldr, float* out, int ldo, int act, float* scratch,
                            long long scratch_floats, unsigned int* counters, int* error_flag, cudaStream_t stream) {
  if (n_tokens <= 0) return R2_OK;
  if (k < 1 || hidden < 1 || n_out < 1) return R2_BAD_SHAPE;
  if (n_tokens > MAX_TOKENS || k > MAX_K || k % BK != 0 || hidden % (HS * CLUSTER) != 0 || n_out % 128 != 0 || n_out % (CLUSTER * 4) != 0 ||
      n_out > 1920 || ldx % 4 != 0 || ldw1 % 8 != 0 || ldw2 % 8 != 0 || gamma == nullptr || beta == nullptr || b1 == nullptr ||
      error_flag == nullptr || counters == nullptr || scratch == nullptr ||
      (reinterpret_cast<uintptr_t>(w1) & 15) || (reinterpret_cast<uintptr_t>(w2) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) {
    return R2_UNSUPPORTED;
  }
  const int live = (n_tokens + 3) & ~3;
  const int n_clusters = hidden / (HS * CLUSTER);
  const size_t w1_bytes = size_t(k / BK) * ATOM_BYTES, w2_bytes = size_t(n_out / 64) * ATOM_BYTES;
  if (2 * size_t(n_out) * live * 4 > w1_bytes) return R2_UNSUPPORTED;   // the exchange buffers lie over the first slice
  if (size_t(n_clusters) * n_out * live > size_t(scratch_floats)) return R2_UNSUPPORTED;
  const size_t smem = 1024 + w1_bytes + w2_bytes + size_t(k / BK + 1) * TOKEN_TILE_BYTES + 8 * 8 + 16;
  if (smem > 227 * 1024) return R2_UNSUPPORTED;
  CUtensorMap m1, m2;
  if (!weight_map(&m1, w1, k, hidden, ldw1) || !weight_map(&m2, w2, hidden, n_out, ldw2)) return R2_UNSUPPORTED;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(mlp_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);  // (no static shared memory)
    if (e != cudaSuccess) return int(e);
    cudaFuncSetAttribute(mlp_fused_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    configured = true;
  }
  MlpParams p;
  p.x = x; p.ldx = ldx; p.rows = rows; p.gamma = gamma; p.beta = beta; p.eps = eps;
  p.n_tokens = n_tokens; p.k = k; p.hidden = hidden; p.n_out = n_out;
  p.b1 = b1; p.b2 = b2; p.residual = residual; p.ldr = ldr; p.out = out; p.ldo = ldo; p.act = act;
  p.scratch = scratch; p.counters = counters; p.n_clusters = n_clusters; p.error_flag = error_flag;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(unsigned(hidden / HS));
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  attr[n_attr].id = cudaLaunchAttributeClusterDimension;
  attr[n_attr].val.clusterDim.x = CLUSTER;
  attr[n_attr].val.clusterDim.y = 1;
  attr[n_attr].val.clusterDim.z = 1;
  ++n_attr;
  if (g_r2_pdl) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  config.attrs = attr;
  config.numAttrs = unsigned(n_attr);
  cudaError_t e = cudaLaunchKernelEx(&config, mlp_fused_kernel, m1, m2, p);
  return e == cudaSuccess ? R2_OK : int(e);
}
