// What a scheduler (one of an SM's four) can issue of the instructions that a softmax over a tile of
// scores is made of: measured, not assumed, because it bounds the prefill attention kernel. One CTA,
// one or two warps per scheduler, every warp the same chain-free work on registers; cycles by clock64.
//
//   mode 0  16 ex2 + N independent fma a round (does the special-function unit hold up the other pipes?)
//   mode 1  the loop of a 64-score row: scale, 64 ex2, sums, 32 packs of two floats into bfloat16 pairs
//   mode 2  32 packs (+ 32 adds)
//   mode 3  32 three-input maxima
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace {

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack(float a, float b) {
  uint32_t r;
  asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
__device__ __forceinline__ float max_of_3(float a, float b, float c) {
  float y;
  asm volatile("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}

constexpr int ROUNDS = 64;

template <int MODE, int N_FMA>
__global__ void probe_kernel(float* sink, long long* cycles, float seed) {
  float s[64];
#pragma unroll
  for (int i = 0; i < 64; ++i) s[i] = seed * float(i) + float(threadIdx.x) * 1e-3f;
  uint32_t pk[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) pk[i] = 0u;
  float acc = 0.f;
  __syncthreads();
  const long long t0 = clock64();
#pragma unroll 1
  for (int round = 0; round < ROUNDS; ++round) {
    if (MODE == 0) {
#pragma unroll
      for (int i = 0; i < 16; ++i) s[i] = ex2(s[i]);
#pragma unroll
      for (int j = 0; j < N_FMA; ++j) asm volatile("fma.rn.f32 %0, %0, %1, %1;" : "+f"(s[16 + (j & 15)]) : "f"(seed));
    }
    if (MODE == 1) {
      float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
      for (int w = 0; w < 16; ++w) {
        const float a0 = ex2(fmaf(s[2 * w], seed, -acc)), a1 = ex2(fmaf(s[2 * w + 1], seed, -acc));
        const float b0 = ex2(fmaf(s[32 + 2 * w], seed, -acc)), b1 = ex2(fmaf(s[32 + 2 * w + 1], seed, -acc));
        sum_a += a0 + a1;
        sum_b += b0 + b1;
        pk[w] ^= pack(a0, a1);
        pk[16 + w] ^= pack(b0, b1);
      }
      acc = acc * 0.5f + sum_a + sum_b;
    }
    if (MODE == 2) {
#pragma unroll
      for (int w = 0; w < 32; ++w) pk[w] ^= pack(s[2 * w] + acc, s[2 * w + 1]);
      acc += 1.f;
    }
    if (MODE == 3) {
      float mx[4] = {acc, acc, acc, acc};
#pragma unroll
      for (int c = 0; c < 32; ++c) mx[c & 3] = max_of_3(mx[c & 3], s[c], s[c + 32]);
      acc += fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * 1e-9f;
    }
  }
  const long long t1 = clock64();
#pragma unroll
  for (int i = 0; i < 32; ++i) acc += __uint_as_float(pk[i]) + s[i] + s[32 + i];
  sink[threadIdx.x] = acc;
  if (threadIdx.x == 0) *cycles = t1 - t0;
}

template <int MODE, int N_FMA>
double run(int warps_per_scheduler, float* sink, long long* cycles) {
  for (int it = 0; it < 3; ++it) probe_kernel<MODE, N_FMA><<<1, 128 * warps_per_scheduler>>>(sink, cycles, 0.001f);
  long long host = 0;
  if (cudaMemcpy(&host, cycles, sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess) return -1.0;
  return double(host) / ROUNDS;
}

}  // namespace

// Cycles a round for each (mode, warps per scheduler) pair below, in this order; returns how many were written.
extern "C" int r2_sfu_probe(double* out, int cap) {
  float* sink = nullptr;
  long long* cycles = nullptr;
  if (cudaMalloc(&sink, 256 * sizeof(float)) != cudaSuccess || cudaMalloc(&cycles, sizeof(long long)) != cudaSuccess) return -1;
  double r[16];
  int n = 0;
  r[n++] = run<0, 0>(1, sink, cycles);
  r[n++] = run<0, 48>(1, sink, cycles);
  r[n++] = run<0, 96>(1, sink, cycles);
  r[n++] = run<0, 128>(1, sink, cycles);
  r[n++] = run<0, 0>(2, sink, cycles);
  r[n++] = run<0, 96>(2, sink, cycles);
  r[n++] = run<1, 0>(1, sink, cycles);
  r[n++] = run<1, 0>(2, sink, cycles);
  r[n++] = run<2, 0>(1, sink, cycles);
  r[n++] = run<2, 0>(2, sink, cycles);
  r[n++] = run<3, 0>(1, sink, cycles);
  r[n++] = run<3, 0>(2, sink, cycles);
  cudaFree(sink);
  cudaFree(cycles);
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  for (int i = 0; i < n && i < cap; ++i) out[i] = r[i];
  return n < cap ? n : cap;
}
