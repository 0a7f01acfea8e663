// Tensor-parallel epilogue in one kernel: all-reduce of the row-parallel partial outputs over PEER
// MEMORY (plain NVLink loads only) fused with the residual add and RMSNorm that follow it.
//
//   delta = sum over ranks s of partial_s            (fp32, ranks in index order: every rank gets the
//                                                     same bits, so the replicated residual never drifts)
//   residual += delta ; y = RMSNorm(residual) * w    (the Hugging Face decoder-layer order; rounding
//                                                     points of add_rmsnorm_hf_bf16_kernel)
//
// replacing, on the decode step of a tensor-parallel engine, an NCCL all-reduce of [M, hidden] plus a
// separate normalisation launch (two of each per layer).  The reference has no multi-GPU path.
//
// One CTA per token row.  Every rank's partial buffer and flag block are mapped into every other
// rank's address space by the host (CUDA IPC).  Protocol per call and row, epoch e = calls so far + 1:
//   1. the partial of this rank is complete (it was written by the preceding kernel of this stream);
//      lane s (s != rank) stores e into flags_s[rank][row] with release.sys - "my row is readable";
//   2. lane s polls flags_rank[s][row] with acquire.sys until it is >= e - bounded; on expiry the
//      row is summed without that peer and a status code is recorded (the context stays usable);
//   3. the row of every rank is read (peers: L1-bypassing loads) and summed.
// A partial buffer may be rewritten once every rank has passed step 2 of the NEXT call on the group,
// so callers alternate two buffers between consecutive calls (the decoder's o_proj / down_proj).
// The epoch lives in device memory and is advanced by the last CTA of each launch, so a captured
// CUDA graph replays correctly.
#include "common.cuh"
#include <cuda.h>
#include <cstring>

namespace tsb {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kFlagRows = 1024;              // rows (tokens) a flag block covers
constexpr unsigned kPollLimit = 1u << 21;    // x ~100 ns: about a quarter of a second

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = (l < nw) ? sh[l] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  __syncthreads();
  return r;
}

__global__ void __launch_bounds__(256)
peer_allreduce_add_rmsnorm_kernel(tsb200_peer_desc pd, __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ w,
                                  __nv_bfloat16* __restrict__ y, int hidden, float eps) {
  __shared__ float sh[32];
  __shared__ unsigned s_missing;             // bit s: peer s did not show up in time
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const unsigned e = *reinterpret_cast<volatile unsigned*>(pd.epoch) + 1u;
  if (threadIdx.x == 0) s_missing = 0u;
  __syncthreads();
  if (threadIdx.x < (unsigned)pd.world && (int)threadIdx.x != pd.rank) {
    const int s = threadIdx.x;
    st_release_sys(pd.flags[s] + pd.rank * kFlagRows + row, e);
    const unsigned* mine = pd.flags[pd.rank] + s * kFlagRows + row;
    bool seen = false;
    for (unsigned i = 0; i < kPollLimit; ++i) {
      if ((int)(ld_acquire_sys(mine) - e) >= 0) { seen = true; break; }
      __nanosleep(100);
    }
    if (!seen) {
      atomicOr(&s_missing, 1u << s);
      atomicMax(pd.status, 21);
    }
  }
  __syncthreads();
  const unsigned missing = s_missing;

  const int nvec = hidden >> 3;
  uint4* r = reinterpret_cast<uint4*>(residual + (int64_t)row * hidden);
  float v[4][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int i = threadIdx.x + it * 256;
    if (i < nvec) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int s = 0; s < pd.world; ++s) {
        if (missing & (1u << s)) continue;
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(pd.partial[s]) + (int64_t)row * hidden) + i;
        const uint4 a = s == pd.rank ? *src : __ldcg(src);
        const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(ap[j]);
          acc[2 * j] += f.x; acc[2 * j + 1] += f.y;
        }
      }
      const uint4 rr = r[i];
      const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rr);
      uint4 o;
      __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // the all-reduced projection output is a bf16 tensor in the unfused path: round the sum first
        const float2 d = __bfloat1622float2(__floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]));
        const float2 fr = __bfloat1622float2(rp[j]);
        op[j] = __floats2bfloat162_rn(__fadd_rn(fr.x, d.x), __fadd_rn(fr.y, d.y));
        const float2 fo = __bfloat1622float2(op[j]);
        v[it][2 * j] = fo.x; v[it][2 * j + 1] = fo.y;
      }
      r[i] = o;
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[it][j] * v[it][j];
    }
  }
  const float var = block_sum(ss, sh) / (float)hidden;
  const float inv = 1.0f / sqrtf(var + eps);
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  uint4* yo = reinterpret_cast<uint4*>(y + (int64_t)row * hidden);
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int i = threadIdx.x + it * 256;
    if (i < nvec) {
      const uint4 ww = wv[i];
      const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&ww);
      uint4 o;
      __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 fw = __bfloat1622float2(wp[j]);
        const __nv_bfloat162 n = __floats2bfloat162_rn(__fmul_rn(v[it][2 * j], inv), __fmul_rn(v[it][2 * j + 1], inv));
        const float2 fn = __bfloat1622float2(n);
        op[j] = __floats2bfloat162_rn(__fmul_rn(fw.x, fn.x), __fmul_rn(fw.y, fn.y));
      }
      yo[i] = o;
    }
  }
  // the last CTA of the launch advances the epoch (every CTA read it at its start)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(pd.epoch + 1, 1u) == gridDim.x - 1) {
      pd.epoch[1] = 0u;
      __threadfence();
      pd.epoch[0] = e;
    }
  }
}

}  // namespace
}  // namespace tsb

using namespace tsb;

extern "C" size_t tsb200_peer_flag_bytes(void) { return (size_t)kMaxRanks * kFlagRows * sizeof(unsigned); }

extern "C" int tsb200_enable_peer_access(int peer_device) {
  TSB_REQUIRE_DEVICE();
  int dev = 0, can = 0;
  TSB_CUDA(cudaGetDevice(&dev));
  if (peer_device == dev) return TSB200_OK;
  TSB_CUDA(cudaDeviceCanAccessPeer(&can, dev, peer_device));
  if (!can) return TSB200_ERR_UNSUPPORTED;
  const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { (void)cudaGetLastError(); return TSB200_OK; }
  TSB_CUDA(e);
  return TSB200_OK;
}

// Export side: the IPC handle of the cudaMalloc allocation that contains `ptr`, and ptr's offset inside it (a
// tensor library's allocator carves many tensors out of one allocation).  Memory from a virtual-memory
// ("expandable") allocator has no such handle: the call then fails with the CUDA error.
extern "C" int tsb200_ipc_export(const void* ptr, void* handle64_out, uint64_t* offset_out) {
  TSB_REQUIRE_DEVICE();
  if (!ptr || !handle64_out || !offset_out) return TSB200_ERR_ARG;
  typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  static RangeFn range_fn = nullptr;
  if (!range_fn) {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || !f)
      return TSB200_ERR_CUDA;
    range_fn = reinterpret_cast<RangeFn>(f);
  }
  CUdeviceptr base = 0;
  size_t size = 0;
  if (range_fn(&base, &size, (CUdeviceptr)(uintptr_t)ptr) != CUDA_SUCCESS) return TSB200_ERR_CUDA;
  cudaIpcMemHandle_t h;
  TSB_CUDA(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>((uintptr_t)base)));
  memcpy(handle64_out, &h, sizeof(h));
  *offset_out = (uint64_t)((uintptr_t)ptr - (uintptr_t)base);
  return TSB200_OK;
}

// Maps an allocation exported by another process of this node (cudaIpcGetMemHandle, 64 bytes) into the CURRENT
// device's address space; peer access to the exporting device is enabled on the way (lazy flag).  Memory imported
// while another device is current is not reachable from kernels of this one, hence no detour through a tensor
// library's own import.
extern "C" int tsb200_ipc_open(const void* handle64, void** base_out) {
  TSB_REQUIRE_DEVICE();
  if (!handle64 || !base_out) return TSB200_ERR_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  TSB_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *base_out = p;
  return TSB200_OK;
}
extern "C" int tsb200_ipc_close(void* base) {
  if (!base) return TSB200_OK;
  TSB_CUDA(cudaIpcCloseMemHandle(base));
  return TSB200_OK;
}

extern "C" int tsb200_peer_allreduce_add_rmsnorm(const tsb200_peer_desc* pd, void* residual, const void* w, void* y, int dtype,
                                                 int64_t M, int64_t hidden, float eps, void* stream) {
  TSB_REQUIRE_DEVICE();
  if (!pd || pd->world < 2 || pd->world > kMaxRanks || pd->rank < 0 || pd->rank >= pd->world) return TSB200_ERR_ARG;
  if (M < 0 || hidden <= 0) return TSB200_ERR_ARG;
  if (M == 0) return TSB200_OK;
  if (dtype != TSB200_BF16 || hidden % 8 || hidden > 8192 || M > kFlagRows) return TSB200_ERR_UNSUPPORTED;
  if (!residual || !w || !y || !pd->epoch || !pd->status) return TSB200_ERR_ARG;
  if (!aligned(residual, 16) || !aligned(w, 16) || !aligned(y, 16)) return TSB200_ERR_ARG;
  for (int s = 0; s < pd->world; ++s)
    if (!pd->partial[s] || !pd->flags[s] || !aligned(pd->partial[s], 16) || !aligned(pd->flags[s], 4)) return TSB200_ERR_ARG;
  TSB_CUDA(launch_kernel(peer_allreduce_add_rmsnorm_kernel, dim3((unsigned)M), dim3(256), 0, as_stream(stream), *pd,
                         (__nv_bfloat16*)residual, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, (int)hidden, eps));
  return TSB200_OK;
}
