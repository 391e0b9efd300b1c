// Device-side self-test of the bounded waits: every mbarrier wait in the attention kernels goes through
// ptx::mbar_wait, which gives up after a cycle limit, raises the CTA's abort flag so that the other roles stop too,
// and lets the kernel report MAGI_E_TIMEOUT through the status word instead of hanging.  This kernel runs that very
// function on a barrier that nothing ever completes, with a short limit, so the give-up path is exercised on the GPU
// without any fault: the kernel returns normally and the context stays usable.
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace magi {
using namespace ptx;

__global__ void __launch_bounds__(64, 1) bounded_wait_selftest_kernel(void* plan, long long limit_cycles) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  __shared__ int gave_up[2];
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);  // one arrival expected; none will come
    abort_flag = 0;
    gave_up[0] = gave_up[1] = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // warp 0 plays a single-thread role (producer / issuer), warp 1 a whole-warp role (softmax): both must come back
  if (warp == 1 || lane == 0) {
    const bool ok = mbar_wait(&bar, 0, &abort_flag, limit_cycles);
    if (!ok && lane == 0) gave_up[warp] = 1;
  }
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag && gave_up[0] && gave_up[1]) plan_view(plan).hdr->status = MAGI_E_TIMEOUT;
}

}  // namespace magi

extern "C" int magi_selftest_bounded_wait(magi_ctx* ctx, long long limit_cycles, void* stream) {
  if (!ctx) return MAGI_E_BADARG;
  if (limit_cycles < 1000 || limit_cycles > 200000000LL)
    return magi::set_err(ctx, MAGI_E_BADARG, "selftest: limit_cycles must be within [1e3, 2e8]");
  int prev = 0;
  cudaGetDevice(&prev);
  if (prev != ctx->device) cudaSetDevice(ctx->device);
  magi::bounded_wait_selftest_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(ctx->workspace, limit_cycles);
  cudaError_t e = cudaGetLastError();
  if (prev != ctx->device) cudaSetDevice(prev);
  if (e != cudaSuccess) return magi::set_err(ctx, MAGI_E_CUDA, "selftest launch failed: %s", cudaGetErrorString(e));
  return MAGI_OK;
}
