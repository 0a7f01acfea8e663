// Paged decode attention on CUDA cores (cross-check kernel) and the split reduction.
// Restates transformersurgeon/blocks/mha.py:9-103 for one query token per sequence:
// out[h] = softmax(q[h] . K[:, h/g]^T * sm_scale) @ V[:, h/g], fp32 accumulation.
#include "decode_attn_common.cuh"

namespace tsb {

// grid (B*hkv, S, ceil(g/8)); 128 threads = 4 warps; warp w takes pages w, w+4, ...
template <typename T, int D>
__global__ void decode_attn_simt_kernel(tsb200_kv_desc kv, const T* __restrict__ q, int64_t qs, int H, float sm_scale,
                                        int64_t max_seq_len, int S, int64_t rec_bytes, float* __restrict__ ws) {
  constexpr int EPL = D / 32, GC = 8;
  const int b = blockIdx.x / kv.hkv, hk = blockIdx.x % kv.hkv, s = blockIdx.y;
  const int g = H / kv.hkv;
  const int g0 = blockIdx.z * GC, gn = min(GC, g - g0);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  int len = kv.seq_lens[b];
  len = len < 0 ? 0 : (len > max_seq_len ? (int)max_seq_len : len);
  int pb, pe;
  split_range(len, s, S, pb, pe);
  float qv[GC][EPL], acc[GC][EPL], m[GC], l[GC];
  const float kscale = kv.format == TSB200_KV_FP8 ? kv.k_scale[b * kv.hkv + hk] : 1.f;
  const float vscale = kv.format == TSB200_KV_FP8 ? kv.v_scale[b * kv.hkv + hk] : 1.f;
#pragma unroll
  for (int i = 0; i < GC; ++i) {
    m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      acc[i][e] = 0.f;
      qv[i][e] = i < gn ? to_f32<T>(q[(int64_t)b * qs + (int64_t)(hk * g + g0 + i) * D + lane * EPL + e]) * sm_scale * kscale : 0.f;
    }
  }
  for (int pg = pb + w; pg < pe; pg += 4) {
    const int64_t page = kv.block_table[(int64_t)b * kv.bt_stride + pg];
    if (page < 0 || page >= kv.num_pages) continue;
    const uint8_t* kr = kv.k_pool + (page * kv.hkv + hk) * rec_bytes;
    const uint8_t* vr = kv.v_pool + (page * kv.hkv + hk) * rec_bytes;
    const int nt = min(16, len - pg * 16);
    for (int t = 0; t < nt; ++t) {
      float kx[EPL], vx[EPL];
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        kx[e] = k_elem<D>(kr, kv.format, t, lane * EPL + e);
        vx[e] = v_elem<D>(vr, kv.format, t, lane * EPL + e) * vscale;
      }
#pragma unroll
      for (int i = 0; i < GC; ++i) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) d += qv[i][e] * kx[e];
        d = warp_sum(d);
        const float mn = fmaxf(m[i], d);
        const float c = __expf(m[i] - mn), p = __expf(d - mn);
        l[i] = l[i] * c + p;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[i][e] = acc[i][e] * c + p * vx[e];
        m[i] = mn;
      }
    }
  }
  // merge the 4 warps through shared memory
  __shared__ float sm_m[4][GC], sm_l[4][GC], sm_acc[4][GC][D];
#pragma unroll
  for (int i = 0; i < GC; ++i) {
    if (lane == 0) { sm_m[w][i] = m[i]; sm_l[w][i] = l[i]; }
#pragma unroll
    for (int e = 0; e < EPL; ++e) sm_acc[w][i][lane * EPL + e] = acc[i][e];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < gn * D; idx += blockDim.x) {
    const int i = idx / D, e = idx % D;
    float mm = -INFINITY;
    for (int ww = 0; ww < 4; ++ww) mm = fmaxf(mm, sm_m[ww][i]);
    float ll = 0.f, a = 0.f;
    for (int ww = 0; ww < 4; ++ww) {
      const float c = sm_m[ww][i] == -INFINITY ? 0.f : __expf(sm_m[ww][i] - mm);
      ll += sm_l[ww][i] * c;
      a += sm_acc[ww][i][e] * c;
    }
    float* o = ws + (((int64_t)b * H + hk * g + g0 + i) * S + s) * (2 + D);
    if (e == 0) { o[0] = mm; o[1] = ll; }
    o[2 + e] = a;
  }
}

// One warp per (b, h): combine S partials -> out.
template <typename T, int D>
__global__ void decode_attn_reduce_kernel(const float* __restrict__ ws, int64_t BH, int S, T* __restrict__ out) {
  constexpr int EPL = D / 32;
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t bh = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  if (bh >= BH) return;
  const float* p = ws + bh * S * (2 + D);
  float mm = -INFINITY;
  for (int s = 0; s < S; ++s) mm = fmaxf(mm, p[s * (2 + D)]);
  float ll = 0.f, a[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) a[e] = 0.f;
  for (int s = 0; s < S; ++s) {
    const float ms = p[s * (2 + D)];
    const float c = ms == -INFINITY ? 0.f : __expf(ms - mm);
    ll += p[s * (2 + D) + 1] * c;
#pragma unroll
    for (int e = 0; e < EPL; ++e) a[e] += p[s * (2 + D) + 2 + lane * EPL + e] * c;
  }
  const float inv = ll > 0.f ? 1.0f / ll : 0.f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) out[bh * D + lane * EPL + e] = from_f32<T>(a[e] * inv);
}

template <typename T, int D>
int launch_reduce(const float* ws, int64_t BH, int S, void* out, cudaStream_t st) {
  const int64_t blocks = (BH + 3) / 4;
  TSB_CUDA(launch_kernel(decode_attn_reduce_kernel<T, D>, dim3((unsigned)blocks), dim3(128), 0, st, ws, BH, S, (T*)out));
  return TSB200_OK;
}
template int launch_reduce<float, 64>(const float*, int64_t, int, void*, cudaStream_t);
template int launch_reduce<float, 128>(const float*, int64_t, int, void*, cudaStream_t);
template int launch_reduce<__nv_bfloat16, 64>(const float*, int64_t, int, void*, cudaStream_t);
template int launch_reduce<__nv_bfloat16, 128>(const float*, int64_t, int, void*, cudaStream_t);

int validate_attn_args(const tsb200_kv_desc* kv, const void* q, void* out, int dtype, int64_t B, int H,
                       int64_t max_seq_len, void* workspace, size_t workspace_bytes, bool& noop, size_t need_bytes) {
  noop = false;
  int st = validate_kv(kv, true);
  if (st != TSB200_OK) return st;
  if (B < 0 || H <= 0 || max_seq_len < 0) return TSB200_ERR_ARG;
  if (H % kv->hkv) return TSB200_ERR_ARG;
  // the kernels walk block_table[b][0 .. ceil(min(seq_lens[b], max_seq_len) / 16)) and clamp page ids into
  // [0, num_pages): both bounds must lie inside what the caller handed over
  if (kv->num_pages <= 0 || max_seq_len > kv->bt_stride * 16) return TSB200_ERR_ARG;
  if (dtype != TSB200_F32 && dtype != TSB200_BF16) return TSB200_ERR_UNSUPPORTED;
  if (B == 0) { noop = true; return TSB200_OK; }
  if (!q || !out || !workspace || !aligned(workspace, 16)) return TSB200_ERR_ARG;
  if (need_bytes == 0) need_bytes = tsb200_paged_decode_attn_workspace_bytes(B, H, kv->head_dim, max_seq_len);
  if (workspace_bytes < need_bytes) return TSB200_ERR_WORKSPACE;
  if (B * kv->hkv > 0x7fffffffLL) return TSB200_ERR_UNSUPPORTED;
  return TSB200_OK;
}

}  // namespace tsb

using namespace tsb;

extern "C" {

size_t tsb200_paged_decode_attn_workspace_bytes(int64_t B, int H, int head_dim, int64_t max_seq_len) {
  if (B <= 0 || H <= 0 || head_dim <= 0) return 0;
  // Splits never exceed 64; size for the worst case so the bound does not depend on hkv.
  int64_t pages = (max_seq_len + 15) / 16;
  int64_t smax = pages / 4 > 0 ? pages / 4 : 1;
  if (smax > 64) smax = 64;
  return kAttnCounterBytes + (size_t)(B * H * smax * (2 + head_dim)) * sizeof(float);
}

int tsb200_paged_decode_attn_simt(const tsb200_kv_desc* kv, const void* q, void* out, int dtype, int64_t q_batch_stride, int64_t B, int H,
                                  float sm_scale, int64_t max_seq_len, void* workspace, size_t workspace_bytes,
                                  void* stream) {
  TSB_REQUIRE_DEVICE();
  bool noop;
  int st = validate_attn_args(kv, q, out, dtype, B, H, max_seq_len, workspace, workspace_bytes, noop, 0);
  if (st != TSB200_OK || noop) return st;
  const int64_t qs = q_batch_stride ? q_batch_stride : (int64_t)H * kv->head_dim;
  if (qs < (int64_t)H * kv->head_dim) return TSB200_ERR_ARG;
  cudaStream_t s = as_stream(stream);
  const int S = choose_splits(B, kv->hkv, max_seq_len);
  const int g = H / kv->hkv;
  const int64_t rec = (int64_t)tsb200_kv_record_bytes(kv->format, kv->head_dim);
  dim3 grid((unsigned)(B * kv->hkv), (unsigned)S, (unsigned)((g + 7) / 8));
  float* ws = (float*)((char*)workspace + kAttnCounterBytes);
#define TSB_GO(TT, DD)                                                                                       \
  decode_attn_simt_kernel<TT, DD><<<grid, 128, 0, s>>>(*kv, (const TT*)q, qs, H, sm_scale, max_seq_len, S, rec, ws); \
  TSB_LAUNCH_CHECK();                                                                                        \
  return launch_reduce<TT, DD>(ws, B * H, S, out, s)
  if (dtype == TSB200_F32) { if (kv->head_dim == 64) { TSB_GO(float, 64); } else { TSB_GO(float, 128); } }
  else { if (kv->head_dim == 64) { TSB_GO(__nv_bfloat16, 64); } else { TSB_GO(__nv_bfloat16, 128); } }
#undef TSB_GO
}

}  // extern "C"
