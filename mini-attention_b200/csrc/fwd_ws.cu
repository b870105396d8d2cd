#include "common.cuh"
#include "ptx.cuh"
namespace ma {
cudaError_t launch_fwd_simple(int D, bool bf16, const CUtensorMap* tm, const FwdArgs& a, cudaStream_t st);
cudaError_t launch_fwd_ws(int D, bool bf16, const CUtensorMap* tm, const FwdArgs& a, int sm_count, cudaStream_t st) {
  return launch_fwd_simple(D, bf16, tm, a, st);
}
}
