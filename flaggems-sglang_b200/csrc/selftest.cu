// Self-test of the device-side time-out path.
//
// Every wait in the grouped-GEMM kernels is bounded: when it runs out, the waiting role raises
// the CTA's abort flag, every other role notices the flag in its own next wait and leaves, the
// CTA writes a code into the caller's status word and the kernel returns with the context
// intact.  In a healthy run none of these waits ever runs out, so this kernel provokes the
// situation harmlessly: a consumer warp waits on an mbarrier on which nobody ever arrives, with a
// limit the caller chooses (a millisecond in the tests), while a second warp sits in a longer wait
// of its own and must be released by the abort flag rather than by its own clock.  Nothing here
// faults, traps or spins without a limit.
#include "common.cuh"

namespace b200moe {

namespace {

__global__ void __launch_bounds__(64)
selftest_timeout_kernel(unsigned long long limit_ns, int* status, int* observed) {
  __shared__ uint64_t bar_never;     // nobody arrives on this one
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar_never), 1);
    abort_word = 0;
    fence_mbar_init();
  }
  __syncthreads();
  if (lane == 0) {
    if (warp == 0) {
      // the wait that runs out
      const bool ok = mbar_wait_limit(smem_u32(&bar_never), 0, abort_flag, DEV_TIMEOUT_SELFTEST, limit_ns);
      observed[0] = ok ? 1 : 0;
    } else {
      // a sibling role with a much longer limit: it must leave because the flag was raised
      const unsigned long long t0 = globaltimer_ns();
      const bool ok = mbar_wait_limit(smem_u32(&bar_never), 0, abort_flag, DEV_TIMEOUT_EPILOGUE, 1000ull * limit_ns);
      observed[1] = ok ? 1 : 0;
      observed[2] = static_cast<int>((globaltimer_ns() - t0) / 1000ull);   // microseconds it sat there
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    mbar_inval(smem_u32(&bar_never));
    if (abort_word != 0) atomicCAS(status, 0, abort_word);
  }
}

}  // namespace

int launch_selftest_timeout(unsigned long long limit_ns, int* status, int* observed, cudaStream_t stream) {
  note_launch("selftest_timeout_kernel");
  selftest_timeout_kernel<<<1, 64, 0, stream>>>(limit_ns, status, observed);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ERR_CUDA;
}

}  // namespace b200moe
