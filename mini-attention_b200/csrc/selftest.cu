// Device-side failure-detection self-test: one CTA waits on an mbarrier that nothing
// ever arrives on.  The bounded wait must give up after `limit_ns`, raise kErrTest in
// the status word and let the kernel return normally, leaving the context usable.
#include "ptx.cuh"

namespace ma {

__global__ void wait_selftest_kernel(int32_t* status, unsigned long long limit_ns) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const WaitCtx wc{&abort_flag, status, limit_ns};
  const bool ok = mbar_wait(smem_u32(&bar), 0, wc, kErrTest);
  if (ok && threadIdx.x == 0) atomicOr(status, 1 << 29);  // must not happen
}

cudaError_t launch_wait_selftest(int32_t* status, unsigned long long limit_ns, cudaStream_t st) {
  wait_selftest_kernel<<<1, 64, 0, st>>>(status, limit_ns);
  return cudaGetLastError();
}

}  // namespace ma
