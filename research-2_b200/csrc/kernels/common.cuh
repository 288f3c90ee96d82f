// Shared device helpers for the sm_100a kernels: element types, loads that widen to float,
// warp reductions, and the status codes that launchers return.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// Launcher status: 0 = launched; > 0 = a CUDA runtime error code; < 0 = refused before launch.
#define R2_OK 0
#define R2_BAD_DTYPE (-1)
#define R2_BAD_SHAPE (-2)
#define R2_BAD_ALIGN (-3)
#define R2_UNSUPPORTED (-4)

#define R2_F32 0
#define R2_BF16 1

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < n_warps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// The activations of a feed-forward's inner layer, in float.
#define R2_ACT_NONE 0
#define R2_ACT_GELU_TANH 1
#define R2_ACT_GELU_ERF 2

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k = 0.7978845608028654f;  // sqrt(2 / pi)
  float inner = k * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.f + tanhf(inner));
}

// gelu_new with the hardware's tanh (relative error about 2^-11, below bfloat16's rounding).
__device__ __forceinline__ float gelu_tanh_hw(float x) {
  const float x2 = x * x;
  const float u = x * fmaf(x2, 0.7978845608028654f * 0.044715f, 0.7978845608028654f);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  const float hx = 0.5f * x;
  return fmaf(hx, t, hx);
}

__device__ __forceinline__ float gelu_erf(float x) {
  return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
}

__device__ __forceinline__ float activate(float x, int act) {
  if (act == R2_ACT_GELU_TANH) return gelu_tanh(x);
  if (act == R2_ACT_GELU_ERF) return gelu_erf(x);
  return x;
}

// A position's page and offset within it. Page sizes are powers of two in practice: the host
// passes log2(size) as `shift` (-1 for another size), which spares the kernels' inner loops an
// integer division whose instruction sequence is long.
inline int page_shift_of(int page_size) {
  if (page_size < 1 || (page_size & (page_size - 1)) != 0) return -1;
  int s = 0;
  while ((1 << s) < page_size) ++s;
  return s;
}
__device__ __forceinline__ int page_index(int j, int page_size, int shift) { return shift >= 0 ? (j >> shift) : (j / page_size); }
__device__ __forceinline__ int page_offset(int j, int page_size, int shift) { return shift >= 0 ? (j & (page_size - 1)) : (j % page_size); }

// Programmatic dependent launch: a kernel may start while its predecessor in the stream is still
// running. Everything it does before `pdl_wait()` must neither read what the predecessor writes
// nor write anything; `pdl_wait()` returns once the predecessor has completed and its writes are
// visible. `pdl_launch_dependents()` lets the successor start its own prologue. Both are no-ops
// for a kernel launched without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static int g_r2_pdl = 1;
// Set by an entry point (on the calling thread, around its launches) whose callers may produce the
// kernel's index arrays with the kernel just before it in the stream: such launches take plain
// stream order, so that nothing is read before that predecessor has completed.
static thread_local int t_r2_plain_order = 0;
// Every kernel library exports this switch (1 = launch with programmatic stream serialization).
extern "C" void r2_set_pdl(int on) { g_r2_pdl = on ? 1 : 0; }

template <typename... KArgs, typename... Args>
static inline void r2_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = (g_r2_pdl && !t_r2_plain_order) ? 1 : 0;
  cudaLaunchKernelEx(&config, kernel, static_cast<Args&&>(args)...);  // a failure shows in launch_status()
}

static inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? R2_OK : int(e);
}
