// Tensor-core (tcgen05) path of LinearCompressed.forward.  Placeholder dispatch until the
// kernel is enabled: reports every shape as unsupported so the CUDA-core kernel runs.
#include "common.cuh"

namespace tsb {
int linear_tc(const tsb200_linear_desc*, const void*, void*, int64_t, void*, size_t, cudaStream_t) {
  return TSB200_ERR_UNSUPPORTED;
}
}  // namespace tsb
