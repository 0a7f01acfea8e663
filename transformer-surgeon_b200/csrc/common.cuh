// Shared helpers for the sm_100a kernels behind the C ABI in include/tsb200.h.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <stdint.h>
#include "../../include/tsb200.h"

namespace tsb {

extern int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = (int)e;
  return TSB200_ERR_CUDA;
}
#define TSB_CUDA(expr)                                   \
  do {                                                   \
    cudaError_t _e = (expr);                             \
    if (_e != cudaSuccess) return ::tsb::cuda_fail(_e);  \
  } while (0)
#define TSB_LAUNCH_CHECK() TSB_CUDA(cudaPeekAtLastError())

// Programmatic dependent launch (tsb200_set_pdl): kernels are launched with the programmatic
// stream-serialization attribute, so a kernel's prologue (and its loads of constant weights) may
// overlap the tail of its predecessor; every kernel calls pdl_wait() before it reads or writes
// anything a predecessor may still touch.
extern int g_pdl;

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                 Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = g_pdl ? attr : nullptr;
  cfg.numAttrs = g_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#ifdef __CUDACC__
// Wait until every prerequisite grid has completed and its memory is visible (no-op without PDL).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
// Allow the dependent grid to start launching (it still waits in pdl_wait for this grid to finish).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
#endif

int check_device_cached();   // TSB200_OK iff current device is CC 10.0
#define TSB_REQUIRE_DEVICE()                    \
  do {                                          \
    int _s = ::tsb::check_device_cached();      \
    if (_s != TSB200_OK) return _s;             \
  } while (0)

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// ---- dtype access ---------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Round an fp32 value to the precision of T and return it as fp32.
template <typename T> __device__ __forceinline__ float rnd(float v) { return to_f32<T>(from_f32<T>(v)); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sign-extend the low `bits` of v.
__device__ __forceinline__ int sext(int v, int bits) { return (v << (32 - bits)) >> (32 - bits); }

// Sub-byte containers are little-endian 32-bit words of per = 32/bits fields covering `per`
// consecutive columns in "pair-interleaved" order: field i < per/2 holds column 2i of the
// group, field i >= per/2 holds column 2(i - per/2) + 1.  Returns the field index of column
// c (0 <= c < per) inside its word.
__device__ __host__ __forceinline__ int field_of_column(int c, int per) { return (c >> 1) + (c & 1) * (per >> 1); }

// Decode code `col` of a packed row.
__device__ __forceinline__ int load_code(const uint8_t* row, int64_t col, int bits) {
  if (bits == 8) return (int)(int8_t)row[col];
  const int per = 32 / bits;
  const unsigned w = reinterpret_cast<const unsigned*>(row)[col / per];
  const unsigned f = (w >> (bits * field_of_column((int)(col % per), per))) & ((1u << bits) - 1u);
  if (bits == 1) return (int)f * 2 - 1;
  return sext((int)f, bits);
}

}  // namespace tsb
