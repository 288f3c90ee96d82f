// A kernel whose only work is a bounded wait that runs out: it waits, poll by poll as every
// mbarrier wait of the tensor-core kernels does, on an mbarrier in its own shared memory on
// which nothing ever arrives, and after `polls` polls records `code` in the device's error
// word and returns. Nothing is in flight and no tensor memory is held when it gives up, so the
// context stays usable. Tests use it to check that a kernel's recorded time-out reaches the
// caller of the engine as an exception (the reference treats a failed launch status as fatal:
// kelpie-core/src/step_loop.zig:272-273, re-raised by kelpie_engine/sdk/engine.py:534-551).
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace {

__global__ void wait_selftest_kernel(int* error_flag, uint32_t polls, int code) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    r2ptx::mbar_init(r2ptx::smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_wait();
  if (threadIdx.x == 0) {
    bool arrived = false;
    for (uint32_t spin = 0; spin < polls && !arrived; ++spin) {
      arrived = r2ptx::mbar_try_wait(r2ptx::smem_u32(&bar), 0) != 0;
      if (spin > 1024) __nanosleep(64);
    }
    if (!arrived) atomicMax(error_flag, code);
  }
}

}  // namespace

// polls is capped at the kernels' own limit (a quarter of a second of polling at most).
extern "C" int r2_wait_selftest(int* error_flag, unsigned polls, int code, cudaStream_t stream) {
  if (error_flag == nullptr || code < 1) return R2_BAD_SHAPE;
  if (polls > r2ptx::SPIN_LIMIT) polls = r2ptx::SPIN_LIMIT;
  r2_launch(wait_selftest_kernel, dim3(1), dim3(32), 0, stream, error_flag, uint32_t(polls), code);
  return launch_status();
}
