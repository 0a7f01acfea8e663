// Dequantizing gather of a paged KV cache into dense tensors.
//
// Attention reads of a quantized cache always see dequantized values.  The decode kernels do that
// on the fly; a prefill over T > 1 query tokens (served by a library attention kernel) needs the
// cached keys and values as dense [B, L, Hkv, d] tensors, which this kernel produces: one thread
// block per (sequence, token), one thread per (kv head, element) pair group.  Positions at or
// beyond seq_lens[b] are written as zeros.  HBM-bound and used once per prompt.
#include "decode_attn_common.cuh"

namespace tsb {
namespace {

template <typename T, int D>
__global__ void kv_gather_kernel(tsb200_kv_desc kv, T* __restrict__ k_out, T* __restrict__ v_out, int64_t L) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t b = blockIdx.y, t = blockIdx.x;
  const int len = kv.seq_lens[b];
  const int rec_bytes = kv.format == TSB200_KV_INT8 ? 16 * D + 64
                        : kv.format == TSB200_KV_FP8 ? 16 * D
                        : kv.format == TSB200_KV_NVFP4 ? 9 * D
                        : kv.format == TSB200_KV_F32 ? 64 * D : 32 * D;
  const bool valid = t < len;
  int64_t page = 0;
  if (valid) {
    page = kv.block_table[b * kv.bt_stride + (t >> 4)];
    page = page < 0 ? 0 : (page >= kv.num_pages ? kv.num_pages - 1 : page);
  }
  const int slot = (int)(t & 15);
  for (int idx = threadIdx.x; idx < kv.hkv * D; idx += blockDim.x) {
    const int hk = idx / D, e = idx % D;
    float kf = 0.f, vf = 0.f;
    if (valid) {
      const uint8_t* kr = kv.k_pool + (page * kv.hkv + hk) * (int64_t)rec_bytes;
      const uint8_t* vr = kv.v_pool + (page * kv.hkv + hk) * (int64_t)rec_bytes;
      kf = k_elem<D>(kr, kv.format, slot, e);
      vf = v_elem<D>(vr, kv.format, slot, e);
      if (kv.format == TSB200_KV_FP8) {
        kf *= kv.k_scale[b * kv.hkv + hk];
        vf *= kv.v_scale[b * kv.hkv + hk];
      }
    }
    const int64_t o = ((b * L + t) * kv.hkv + hk) * D + e;
    k_out[o] = from_f32<T>(kf);
    v_out[o] = from_f32<T>(vf);
  }
}

template <typename T>
int launch_gather(const tsb200_kv_desc& kv, void* k_out, void* v_out, int64_t B, int64_t L, cudaStream_t st) {
  const dim3 grid((unsigned)L, (unsigned)B);
  const int threads = kv.hkv * kv.head_dim >= 256 ? 256 : 128;
  if (kv.head_dim == 64) {
    TSB_CUDA(launch_kernel(kv_gather_kernel<T, 64>, grid, dim3(threads), 0, st, kv, (T*)k_out, (T*)v_out, L));
  } else {
    TSB_CUDA(launch_kernel(kv_gather_kernel<T, 128>, grid, dim3(threads), 0, st, kv, (T*)k_out, (T*)v_out, L));
  }
  return TSB200_OK;
}

}  // namespace
}  // namespace tsb

using namespace tsb;

extern "C" int tsb200_kv_gather(const tsb200_kv_desc* kv, void* k_out, void* v_out, int dtype, int64_t B, int64_t L,
                                void* stream) {
  TSB_REQUIRE_DEVICE();
  const int st = validate_kv(kv, true);
  if (st != TSB200_OK) return st;
  if (B < 0 || L < 0) return TSB200_ERR_ARG;
  if (dtype != TSB200_F32 && dtype != TSB200_BF16) return TSB200_ERR_UNSUPPORTED;
  if (kv->head_dim != 64 && kv->head_dim != 128) return TSB200_ERR_UNSUPPORTED;
  if (B == 0 || L == 0) return TSB200_OK;
  if (!k_out || !v_out) return TSB200_ERR_ARG;
  if (B > 65535 || L > 0x7fffffffLL || L > kv->bt_stride * 16) return TSB200_ERR_ARG;
  cudaStream_t s = as_stream(stream);
  return dtype == TSB200_F32 ? launch_gather<float>(*kv, k_out, v_out, B, L, s)
                             : launch_gather<__nv_bfloat16>(*kv, k_out, v_out, B, L, s);
}
