// Sampling: one token per logits row, greedy or a Gumbel-max draw with an optional top-k filter.
//
// Reference: kelpie-models/kelpie_models/kernels/ops/sample.py.
//   * top_k == 1: argmax over float logits, first index on ties (:103-108). Greedy requests are
//     stored as (T = 1, top_k = 1) by the scheduler (kelpie-core/src/request.zig:140-144).
//   * else: keep = all tokens (top_k == 0) or every token >= the k-th largest value (ties kept);
//     token = argmax(keep ? logit / T + g : -inf), g = -log(-log u),
//     u = ((c0 & 0xFFFFFF) + 0.5) * 2^-24, c0 the first word of Philox-4x32-10 (:23-52,114-137).
// The Philox counter is (position of the drawn token, 0, token id, 0) and the key is the
// request's own, so a request draws the same numbers whatever batch it is in (the reference
// keys the draw by the batch: kelpie-engine/kelpie_engine/sdk/plan.py:96-106).
#include <math.h>

#include "common.cuh"

namespace {

constexpr int THREADS = 512;

__device__ __forceinline__ uint32_t philox_c0(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    if (r > 0) {
      k0 += 0x9E3779B9u;
      k1 += 0xBB67AE85u;
    }
    uint32_t hi0 = __umulhi(c0, 0xD2511F53u), lo0 = c0 * 0xD2511F53u;
    uint32_t hi1 = __umulhi(c2, 0xCD9E8D57u), lo1 = c2 * 0xCD9E8D57u;
    uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
  }
  return c0;
}

__device__ __forceinline__ float gumbel(uint32_t position, uint32_t token, uint32_t k0, uint32_t k1) {
  uint32_t c0 = philox_c0(position, 0u, token, 0u, k0, k1);
  float u = (float(c0 & 0xFFFFFFu) + 0.5f) * (1.0f / 16777216.0f);
  return -logf(-logf(u));
}

// Floats as unsigned keys whose order is the floats' order.
__device__ __forceinline__ uint32_t order_key(float v) {
  uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct Best {
  float v;
  int i;
};

__device__ __forceinline__ Best better(Best a, Best b) {
  if (b.i < 0) return a;
  if (a.i < 0) return b;
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ Best block_best(Best mine, Best* scratch) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other;
    other.v = __shfl_xor_sync(0xffffffffu, mine.v, o);
    other.i = __shfl_xor_sync(0xffffffffu, mine.i, o);
    mine = better(mine, other);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = mine;
  __syncthreads();
  if (warp == 0) {
    Best t = lane < THREADS / 32 ? scratch[lane] : Best{0.f, -1};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best other;
      other.v = __shfl_xor_sync(0xffffffffu, t.v, o);
      other.i = __shfl_xor_sync(0xffffffffu, t.i, o);
      t = better(t, other);
    }
    if (lane == 0) scratch[0] = t;
  }
  __syncthreads();
  Best r = scratch[0];
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int vocab, const float* __restrict__ temperature,
              const int32_t* __restrict__ top_k, const uint32_t* __restrict__ key0, const uint32_t* __restrict__ key1,
              const int32_t* __restrict__ sample_pos, int32_t* __restrict__ tokens) {
  pdl_launch_dependents();  // the next kernel may begin its prologue
  pdl_wait();               // the previous kernel's writes are visible from here on
  __shared__ Best best_s[THREADS / 32];
  __shared__ uint32_t hist[256];
  __shared__ uint32_t sel_prefix, sel_remaining;
  const int row = blockIdx.x;
  const float* lg = logits + size_t(row) * ld;
  const int k = top_k[row];

  if (k == 1) {
    Best mine{0.f, -1};
    for (int i = threadIdx.x; i < vocab; i += THREADS) {
      float v = lg[i];
      if (mine.i < 0 || v > mine.v) mine = Best{v, i};
    }
    Best r = block_best(mine, best_s);
    if (threadIdx.x == 0) tokens[row] = r.i < 0 ? 0 : r.i;
    return;
  }

  // The k-th largest value by radix selection over the order keys, 8 bits at a time.
  float kth = -INFINITY;
  if (k > 1 && k < vocab) {
    if (threadIdx.x == 0) {
      sel_prefix = 0u;
      sel_remaining = uint32_t(k);
    }
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int b = threadIdx.x; b < 256; b += THREADS) hist[b] = 0u;
      __syncthreads();
      uint32_t prefix = sel_prefix;
      uint32_t mask = shift == 24 ? 0u : (0xFFFFFFFFu << (shift + 8));
      for (int i = threadIdx.x; i < vocab; i += THREADS) {
        uint32_t key = order_key(lg[i]);
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xFFu], 1u);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        uint32_t remaining = sel_remaining;
        int b = 255;
        for (; b > 0; --b) {
          if (hist[b] >= remaining) break;
          remaining -= hist[b];
        }
        sel_prefix = prefix | (uint32_t(b) << shift);
        sel_remaining = remaining;
      }
      __syncthreads();
    }
    uint32_t key = sel_prefix;
    uint32_t bits = (key & 0x80000000u) ? (key & 0x7FFFFFFFu) : ~key;
    kth = __uint_as_float(bits);
  }

  const float temp = temperature[row];
  const uint32_t k0 = key0[row], k1 = key1[row];
  const uint32_t position = uint32_t(sample_pos[row]);
  Best mine{0.f, -1};
  for (int i = threadIdx.x; i < vocab; i += THREADS) {
    float v = lg[i];
    bool keep = (v >= kth) && isfinite(v);
    if (!keep) continue;  // a filtered token is selected out, never added to
    float score = v / temp + gumbel(position, uint32_t(i), k0, k1);
    if (mine.i < 0 || score > mine.v) mine = Best{score, i};
  }
  Best r = block_best(mine, best_s);
  if (threadIdx.x == 0) tokens[row] = r.i < 0 ? 0 : r.i;
}

}  // namespace

// logits [n_rows, vocab] float with row stride ld; per row temperature (> 0), top_k (0 = all,
// 1 = greedy, k > 1), the request's Philox key and the position of the token being drawn.
extern "C" int r2_sample(const float* logits, int ld, int n_rows, int vocab, const float* temperature,
                         const int32_t* top_k, const uint32_t* key0, const uint32_t* key1, const int32_t* sample_pos,
                         int32_t* tokens, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (vocab < 1 || ld < vocab) return R2_BAD_SHAPE;
  r2_launch(sample_kernel, dim3(n_rows), dim3(THREADS), size_t(0), stream, logits, ld, vocab, temperature, top_k, key0, key1, sample_pos, tokens);
  return launch_status();
}
