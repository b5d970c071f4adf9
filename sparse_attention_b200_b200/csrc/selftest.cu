// Self-test of the bounded-wait machinery: a kernel that waits on an mbarrier nobody will ever
// arrive on, with a short cycle limit and nothing in flight, so that the give-up path (status
// word, CTA-wide abort flag, orderly exit) can be exercised without a protocol bug and without
// hanging anything. The reference's waits spin without a limit
// (attention/q_centric/common.cuh:38-52); it has no counterpart of this.
#include "ptx.cuh"
#include "internal.h"

namespace sb {
namespace {

constexpr int SELFTEST_CODE = 0x7e57;

// Warp 0 waits (all lanes, as the load warp of the attention kernel does); warp 1 polls the abort
// flag the way the other roles do between their own waits, with its own iteration limit.
__global__ void __launch_bounds__(64) bounded_wait_selftest_kernel(int* status, long long limit_cycles,
                                                                   int* observed) {
  __shared__ __align__(8) unsigned long long barrier_word;
  __shared__ int abort_flag;
  const uint32_t bar = smem_u32(&barrier_word);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  Guard guard{&abort_flag, status};
  if (threadIdx.x < 32) {
    const bool done = mbar_wait_limited(bar, 0, guard, SELFTEST_CODE, limit_cycles);
    if (threadIdx.x == 0 && observed) observed[0] = done ? 1 : 0;     // 0: the wait gave up
  } else {
    const long long t0 = clock64();
    bool saw = false;
    while (!saw && clock64() - t0 < 64 * limit_cycles + 1000000) saw = *guard.abort_flag != 0;
    if (threadIdx.x == 32 && observed) observed[1] = saw ? 1 : 0;     // 1: the other role saw the abort
  }
}

}  // namespace

int launch_bounded_wait_selftest(long long limit_cycles, int* observed, cudaStream_t stream) {
  DeviceCtx* ctx = device_ctx();
  if (!ctx) return SB_ERR_CUDA;
  bounded_wait_selftest_kernel<<<1, 64, 0, stream>>>(ctx->status, limit_cycles, observed);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SB_OK : set_error(SB_ERR_CUDA, cudaGetErrorString(e));
}

}  // namespace sb
