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
//
// A row's vocabulary is split over up to 16 CTAs (the noise costs ten Philox rounds a token: one
// CTA for 50,257 tokens took 65 us). Without a top-k filter each CTA finds the best of its slice and
// the CTA that arrives last at the row's counter takes the best of the slices' bests (ties to the
// lower token, so the split does not show) and resets the counter.
//
// With a top-k filter only about k tokens need noise, but the k-th largest value is a fact of the
// whole row. Each CTA counts its slice into 4,096 bins (sign, exponent and three bits of the
// fraction of the value) and adds its counts to the row's bins in global memory; the CTA that
// arrives last finds the bin that holds the k-th largest value, goes over the row once (values in
// higher bins are kept at once, values in that bin are listed in shared memory), selects the exact
// k-th value inside the list, and draws among the kept. (Every CTA of a row selecting over the whole
// row for itself, four passes each, took 130 us for 64 rows of 50,257; this takes 15.) A list that
// does not fit (a row of thousands of equal values) falls back to the radix selection over the row.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int THREADS = 512;
constexpr int MAX_SPLIT = 16;
constexpr int MAX_SPLIT_ROWS = 1024;  // more rows than this run one CTA each

struct Best {
  float v;
  int i;
};
// Scratch of the split form: launches on one stream follow one another, which is what the engine does.
__device__ Best slice_best[MAX_SPLIT_ROWS * MAX_SPLIT];
__device__ unsigned int slices_arrived[MAX_SPLIT_ROWS];
constexpr int BINS = 4096;             // of the top 12 bits of a value's order key
constexpr int LIST_CAP = 2048;         // values of the k-th value's bin that shared memory lists
constexpr int MAX_BINNED_ROWS = 256;   // rows whose bins global memory holds (more rows than this: one CTA a row)
__device__ unsigned int row_bins[MAX_BINNED_ROWS * BINS];   // zero between launches

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

// The row's token from its slices' bests: the CTA that arrives last reduces them.
__device__ void finish_row(Best r, int row, int slice, int n_slices, int32_t* tokens, bool* last_of_row) {
  if (n_slices == 1) {
    if (threadIdx.x == 0) tokens[row] = r.i < 0 ? 0 : r.i;
    return;
  }
  if (threadIdx.x == 0) {
    slice_best[row * MAX_SPLIT + slice] = r;
    __threadfence();
    *last_of_row = atomicAdd(&slices_arrived[row], 1u) == unsigned(n_slices - 1);
  }
  __syncthreads();
  if (!*last_of_row) return;
  if (threadIdx.x < 32) {
    __threadfence();
    Best b{0.f, -1};
    if (int(threadIdx.x) < n_slices) {
      const volatile Best* src = &slice_best[row * MAX_SPLIT + threadIdx.x];
      b.v = src->v;
      b.i = src->i;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
      b = better(b, other);
    }
    if (threadIdx.x == 0) {
      tokens[row] = b.i < 0 ? 0 : b.i;
      slices_arrived[row] = 0u;  // for the next launch
    }
  }
}

// The k-th largest value of a row by radix selection over the order keys, 8 bits at a time: four passes
// over the row (each costs the latency of its reads: about 10 us for 50,257 tokens from the L2). Every
// thread of the CTA calls it. Logits crowd into the few bins of their common exponents, and shared-memory
// atomics on one address run one after another, so the lanes count into eight columns,
// lanes_hist[bin][lane % 8] (at most four lanes of a warp meet), and the columns are summed afterwards.
__device__ float select_kth(const float* __restrict__ src, int vocab, int k, uint32_t* lanes_hist, uint32_t* hist, uint32_t* sel) {
  if (threadIdx.x == 0) {
    sel[0] = 0u;           // the prefix chosen so far
    sel[1] = uint32_t(k);  // how many of the elements that match it are still wanted
  }
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int b = threadIdx.x; b < 256 * 8; b += THREADS) lanes_hist[b] = 0u;
    __syncthreads();
    const uint32_t prefix = sel[0];
    const uint32_t mask = shift == 24 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int base = 0; base < vocab; base += 8 * THREADS) {
      const int i0 = base + int(threadIdx.x);
      float v[8];  // eight loads in flight
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = i0 + u * THREADS < vocab ? src[i0 + u * THREADS] : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint32_t key = order_key(v[u]);
        if (i0 + u * THREADS < vocab && (key & mask) == prefix) atomicAdd(&lanes_hist[((key >> shift) & 0xFFu) * 8u + (threadIdx.x & 7u)], 1u);
      }
    }
    __syncthreads();
    if (threadIdx.x < 256) {
      uint32_t total = 0u;
#pragma unroll
      for (int l = 0; l < 8; ++l) total += lanes_hist[threadIdx.x * 8 + l];
      hist[threadIdx.x] = total;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // The highest bin at which the count from the top reaches what is still wanted: lane l
      // has bins 255 - 8l down to 248 - 8l. The elements that match the prefix are at least as
      // many as are wanted, so there is such a bin.
      const int lane = threadIdx.x;
      uint32_t c[8], sum = 0u;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        c[j] = hist[255 - 8 * lane - j];
        sum += c[j];
      }
      uint32_t upto = sum;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        uint32_t other = __shfl_up_sync(0xffffffffu, upto, d);
        if (lane >= d) upto += other;
      }
      const uint32_t remaining = sel[1];
      __syncwarp();  // every lane has read the count before the selecting lane overwrites it
      uint32_t above = upto - sum;  // in bins above this lane's
      if (above < remaining && remaining <= upto) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (above < remaining && remaining <= above + c[j]) {
            sel[0] = prefix | (uint32_t(255 - 8 * lane - j) << shift);
            sel[1] = remaining - above;
          }
          above += c[j];
        }
      }
    }
    __syncthreads();
  }
  const uint32_t key = sel[0];
  const uint32_t bits = (key & 0x80000000u) ? (key & 0x7FFFFFFFu) : ~key;
  return __uint_as_float(bits);
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int vocab, const float* __restrict__ temperature,
              const int32_t* __restrict__ top_k, const uint32_t* __restrict__ key0, const uint32_t* __restrict__ key1,
              const int32_t* __restrict__ sample_pos, int32_t* __restrict__ tokens) {
  pdl_launch_dependents();  // the next kernel may begin its prologue
  pdl_wait();               // the previous kernel's writes are visible from here on
  __shared__ Best best_s[THREADS / 32];
  __shared__ uint32_t lanes_hist[256 * 8];
  __shared__ uint32_t hist[256];
  __shared__ uint32_t sel[2];
  __shared__ bool last_of_row;
  const int row = blockIdx.x;
  const int n_slices = int(gridDim.y), slice = int(blockIdx.y);
  const int per_slice = (vocab + n_slices - 1) / n_slices;
  const int i_begin = slice * per_slice, i_end = min(vocab, i_begin + per_slice);
  const float* lg = logits + size_t(row) * ld;
  const int k = top_k[row];

  if (k == 1) {
    Best mine{0.f, -1};
    for (int i = i_begin + threadIdx.x; i < i_end; i += THREADS) {
      float v = lg[i];
      if (mine.i < 0 || v > mine.v) mine = Best{v, i};
    }
    Best r = block_best(mine, best_s);
    finish_row(r, row, slice, n_slices, tokens, &last_of_row);
    return;
  }

  const float temp = temperature[row];
  const uint32_t k0 = key0[row], k1 = key1[row];
  const uint32_t position = uint32_t(sample_pos[row]);

  if (k > 1 && k < vocab && (n_slices == 1 || row < MAX_BINNED_ROWS)) {
    // ---- top-k: counts per bin by every CTA of the row, the rest by the one that arrives last ----
    // (the list takes the bins' place once the bin is found: greedy rows run the same kernel, and what it
    // declares bounds how many of their CTAs an SM holds)
    __shared__ uint32_t bins_s[BINS];
    static_assert(2 * LIST_CAP == BINS, "the list lies over the bins");
    float* list_v = reinterpret_cast<float*>(bins_s);
    int* list_i = reinterpret_cast<int*>(bins_s + LIST_CAP);
    __shared__ uint32_t n_list, the_bin, n_above;
    __shared__ float kth_s;
    __shared__ uint32_t warp_sums[THREADS / 32];
    for (int b = threadIdx.x; b < BINS; b += THREADS) bins_s[b] = 0u;
    __syncthreads();
    for (int base = i_begin; base < i_end; base += 8 * THREADS) {
      const int i0 = base + int(threadIdx.x);
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = i0 + u * THREADS < i_end ? lg[i0 + u * THREADS] : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        // (-0 counts as +0: the filter below compares values, and the two are one value)
        if (i0 + u * THREADS < i_end) atomicAdd(&bins_s[order_key(v[u] + 0.f) >> 20], 1u);
      }
    }
    __syncthreads();
    if (n_slices > 1) {
      unsigned int* g = row_bins + size_t(row) * BINS;
      for (int b = threadIdx.x; b < BINS; b += THREADS) {
        const uint32_t c = bins_s[b];
        if (c) atomicAdd(g + b, c);
      }
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) last_of_row = atomicAdd(&slices_arrived[row], 1u) == unsigned(n_slices - 1);
      __syncthreads();
      if (!last_of_row) return;
      __threadfence();
      for (int b = threadIdx.x; b < BINS; b += THREADS) {
        bins_s[b] = __ldcg(g + b);
        g[b] = 0u;  // for the next launch
      }
      __syncthreads();
    }
    // The highest bin at which the count from the top reaches k: thread t has bins BINS - 1 - 8t down to
    // BINS - 8 - 8t. The row has more than k values, so there is such a bin.
    {
      const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
      uint32_t c[8], sum = 0u;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        c[j] = bins_s[BINS - 1 - 8 * int(threadIdx.x) - j];
        sum += c[j];
      }
      uint32_t upto = sum;  // of this warp's threads up to this one
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const uint32_t other = __shfl_up_sync(0xffffffffu, upto, d);
        if (lane >= d) upto += other;
      }
      if (lane == 31) warp_sums[warp] = upto;
      if (threadIdx.x == 0) {
        n_list = 0u;
        kth_s = -INFINITY;
      }
      __syncthreads();
      for (int w = 0; w < warp; ++w) upto += warp_sums[w];
      uint32_t above = upto - sum;  // in bins above this thread's
      if (above < uint32_t(k) && uint32_t(k) <= upto) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (above < uint32_t(k) && uint32_t(k) <= above + c[j]) {
            the_bin = uint32_t(BINS - 1 - 8 * int(threadIdx.x) - j);
            n_above = above;
          }
          above += c[j];
        }
      }
      __syncthreads();
    }
    const uint32_t bin = the_bin;
    const int wanted = k - int(n_above);  // of the values in that bin, from the largest down
    // One pass over the row: values in higher bins are kept, values in the bin are listed.
    Best mine{0.f, -1};
    for (int base = 0; base < vocab; base += 16 * THREADS) {
      const int i0 = base + int(threadIdx.x);
      float v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) v[u] = i0 + u * THREADS < vocab ? lg[i0 + u * THREADS] : 0.f;
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int i = i0 + u * THREADS;
        if (i >= vocab) continue;
        const uint32_t b = order_key(v[u] + 0.f) >> 20;
        if (b > bin) {
          if (isfinite(v[u])) mine = better(mine, Best{v[u] / temp + gumbel(position, uint32_t(i), k0, k1), i});
        } else if (b == bin) {
          const uint32_t at = atomicAdd(&n_list, 1u);
          if (at < uint32_t(LIST_CAP)) {
            list_v[at] = v[u];
            list_i[at] = i;
          }
        }
      }
    }
    __syncthreads();
    const int n = int(n_list);
    if (n <= LIST_CAP) {
      // the `wanted`-th largest of the list: the value with fewer than `wanted` values above it and at
      // least `wanted` values at or above it (equal values give the same answer)
      for (int e = threadIdx.x; e < n; e += THREADS) {
        const float ve = list_v[e];
        int gt = 0, ge = 0;
        for (int j = 0; j < n; ++j) {
          gt += list_v[j] > ve ? 1 : 0;
          ge += list_v[j] >= ve ? 1 : 0;
        }
        if (gt < wanted && wanted <= ge) kth_s = ve;
      }
      __syncthreads();
      const float kth = kth_s;
      for (int e = threadIdx.x; e < n; e += THREADS) {
        const float v = list_v[e];
        if (v >= kth && isfinite(v)) mine = better(mine, Best{v / temp + gumbel(position, uint32_t(list_i[e]), k0, k1), list_i[e]});
      }
    } else {
      // thousands of values in one bin (a row of equal logits): the radix selection over the row
      const float kth = select_kth(lg, vocab, k, lanes_hist, hist, sel);
      mine = Best{0.f, -1};
      for (int i = threadIdx.x; i < vocab; i += THREADS) {
        const float v = lg[i];
        if (v >= kth && isfinite(v)) mine = better(mine, Best{v / temp + gumbel(position, uint32_t(i), k0, k1), i});
      }
    }
    const Best r = block_best(mine, best_s);
    if (threadIdx.x == 0) {
      tokens[row] = r.i < 0 ? 0 : r.i;
      if (n_slices > 1) slices_arrived[row] = 0u;  // for the next launch
    }
    return;
  }

  // No filter (top_k 0, or k as large as the vocabulary), or a top-k row beyond those that global memory
  // holds bins for: each CTA its slice, and for the latter the k-th value by the CTA's own selection.
  float kth = -INFINITY;
  if (k > 1 && k < vocab) kth = select_kth(lg, vocab, k, lanes_hist, hist, sel);
  Best mine{0.f, -1};
  for (int i = i_begin + threadIdx.x; i < i_end; i += THREADS) {
    float v = lg[i];
    bool keep = (v >= kth) && isfinite(v);
    if (!keep) continue;  // a filtered token is selected out, never added to
    float score = v / temp + gumbel(position, uint32_t(i), k0, k1);
    if (mine.i < 0 || score > mine.v) mine = Best{score, i};
  }
  Best r = block_best(mine, best_s);
  finish_row(r, row, slice, n_slices, tokens, &last_of_row);
}

}  // namespace

// logits [n_rows, vocab] float with row stride ld; per row temperature (> 0), top_k (0 = all,
// 1 = greedy, k > 1), the request's Philox key and the position of the token being drawn.
extern "C" int r2_sample(const float* logits, int ld, int n_rows, int vocab, const float* temperature,
                         const int32_t* top_k, const uint32_t* key0, const uint32_t* key1, const int32_t* sample_pos,
                         int32_t* tokens, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (vocab < 1 || ld < vocab) return R2_BAD_SHAPE;
  int n_slices = (vocab + 8 * THREADS - 1) / (8 * THREADS);  // about eight tokens a thread
  n_slices = n_rows > MAX_SPLIT_ROWS ? 1 : (n_slices < 1 ? 1 : (n_slices > MAX_SPLIT ? MAX_SPLIT : n_slices));
  r2_launch(sample_kernel, dim3(n_rows, n_slices), dim3(THREADS), size_t(0), stream, logits, ld, vocab, temperature, top_k, key0, key1,
            sample_pos, tokens);
  return launch_status();
}
