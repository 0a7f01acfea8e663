// tsb200_linear: picks the kernel for LinearCompressed.forward
// (transformersurgeon/blocks/linear_compressed.py:81-105).
#include "common.cuh"

namespace tsb {
int validate_linear(const tsb200_linear_desc* d, const void* x, void* y, int64_t M, bool& noop);
// Tensor-core path (linear_tc.cu); returns TSB200_ERR_UNSUPPORTED when the shape/dtype is
// outside what it implements, in which case the CUDA-core kernel takes the call.
int linear_tc(const tsb200_linear_desc* d, const void* x, void* y, int64_t M, void* workspace, size_t workspace_bytes,
              cudaStream_t s);
int linear_argmax_tc(const tsb200_linear_desc* d, const void* x, int64_t* tokens, int64_t M, void* amax, int* status, cudaStream_t s);
int argmax_rows(const void* y, int dtype, int64_t M, int64_t N, int64_t* tokens, cudaStream_t s);
}  // namespace tsb

using namespace tsb;

// Workspace of the greedy head: the linear layer's own workspace, then either the per-tile (maximum, column) pairs of
// the fused route or the logits of the general route (whichever is larger).
extern "C" size_t tsb200_linear_argmax_workspace_bytes(const tsb200_linear_desc* d, int64_t M) {
  if (!d || M <= 0) return tsb200_linear_workspace_bytes(d, M);
  const size_t lin = (tsb200_linear_workspace_bytes(d, M) + 255) / 256 * 256;
  const size_t tiles = (size_t)((d->out_features + 127) / 128);
  const size_t pairs = (size_t)M * tiles * 8;
  const size_t logits = (size_t)M * (size_t)d->out_features * (d->act_dtype == TSB200_F32 ? 4 : 2);
  return lin + (pairs > logits ? pairs : logits) + 256;
}

extern "C" int tsb200_linear_argmax(const tsb200_linear_desc* d, const void* x, int64_t* tokens, int64_t M, void* workspace,
                                    size_t workspace_bytes, void* stream) {
  TSB_REQUIRE_DEVICE();
  if (!d || M < 0) return TSB200_ERR_ARG;
  if (M == 0) return TSB200_OK;
  if (!tokens || !x || !workspace || !aligned(workspace, 256)) return TSB200_ERR_ARG;
  if (workspace_bytes < tsb200_linear_argmax_workspace_bytes(d, M)) return TSB200_ERR_WORKSPACE;
  const size_t lin = (tsb200_linear_workspace_bytes(d, M) + 255) / 256 * 256;
  void* extra = (uint8_t*)workspace + lin;
  cudaStream_t s = as_stream(stream);
  int st = linear_argmax_tc(d, x, tokens, M, extra, (int*)workspace, s);
  if (st != TSB200_ERR_UNSUPPORTED) return st;
  st = tsb200_linear(d, x, extra, M, workspace, lin, stream);          // logits into the scratch, then their argmax
  if (st != TSB200_OK) return st;
  return argmax_rows(extra, d->act_dtype, M, d->out_features, tokens, s);
}

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
