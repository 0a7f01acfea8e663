// tsb200_linear: picks the kernel for LinearCompressed.forward
// (transformersurgeon/blocks/linear_compressed.py:81-105).
#include "common.cuh"

namespace tsb {
int validate_linear(const tsb200_linear_desc* d, const void* x, void* y, int64_t M, bool& noop);
// Tensor-core path (linear_tc.cu); returns TSB200_ERR_UNSUPPORTED when the shape/dtype is
// outside what it implements, in which case the CUDA-core kernel takes the call.
int linear_tc(const tsb200_linear_desc* d, const void* x, void* y, int64_t M, void* workspace, size_t workspace_bytes,
              cudaStream_t s);
}  // namespace tsb

using namespace tsb;

extern "C" int tsb200_linear(const tsb200_linear_desc* d, const void* x, void* y, int64_t M, void* workspace,
                             size_t workspace_bytes, void* stream) {
  TSB_REQUIRE_DEVICE();
  bool noop;
  int st = validate_linear(d, x, y, M, noop);
  if (st != TSB200_OK || noop) return st;
  st = linear_tc(d, x, y, M, workspace, workspace_bytes, as_stream(stream));
  if (st != TSB200_ERR_UNSUPPORTED) return st;
  return tsb200_linear_simt(d, x, y, M, workspace, workspace_bytes, stream);
}
