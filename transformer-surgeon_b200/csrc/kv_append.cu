// Fused (RoPE on K +) quantize-and-append into the paged KV pools, and the FP8 scale
// reduction over a prompt.  One warp owns one (token, kv head) vector of d elements:
// lane l holds elements [l*d/32, (l+1)*d/32).  HBM-bound: reads 2*d*sizeof(act) bytes
// and writes 2*d*b_elem (+ scales) per vector.
//
// Quantization arithmetic (IEEE fp32, round-to-nearest-even) per format:
//   int8  : s = amax/127, code = clamp(rint(x/(s+1e-6)), +-127)   (the reference's weight
//           rule, compression/quantization_methods/vanilla.py:16-24, applied per vector)
//   fp8   : code = e4m3_satfinite(x / S[b, h])
//   nvfp4 : per 16 elements sb = e4m3_satfinite(amax/6), code = e2m1_satfinite(x/decode(sb))
#include "common.cuh"

namespace tsb {

__device__ __forceinline__ float e4m3_to_f32(unsigned char c) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

template <int N> struct BytesN;
template <> struct BytesN<1> { using type = uint8_t; };
template <> struct BytesN<2> { using type = uint16_t; };
template <> struct BytesN<4> { using type = uint32_t; };

// Rotate (optional) and round to T; returns this lane's EPL elements as fp32.
template <typename T, int D>
__device__ __forceinline__ void load_vec(const T* __restrict__ src, int lane, float (&x)[D / 32], bool rope,
                                         const float* __restrict__ cosr, const float* __restrict__ sinr) {
  constexpr int EPL = D / 32;
#pragma unroll
  for (int i = 0; i < EPL; ++i) x[i] = to_f32<T>(src[lane * EPL + i]);
  if (rope) {
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, x[i], 16);
      const int e = (lane & 15) * EPL + i;             // index inside the half
      const float c = rnd<T>(cosr[e]), s = rnd<T>(sinr[e]);
      const float a = rnd<T>(__fmul_rn(x[i], c));       // own * cos
      const float b = rnd<T>(__fmul_rn(other, s));      // partner * sin
      x[i] = rnd<T>(lane < 16 ? __fsub_rn(a, b) : __fadd_rn(b, a));
    }
  }
}

// Unquantized pages (TSB200_KV_F32 / TSB200_KV_BF16): K and V records are both [16 tok][d] of T.
template <typename T, int D>
__device__ __forceinline__ void dense_store(const float (&x)[D / 32], int lane, uint8_t* __restrict__ rec, int slot) {
  constexpr int EPL = D / 32;
  T* dst = reinterpret_cast<T*>(rec) + slot * D + lane * EPL;
#pragma unroll
  for (int i = 0; i < EPL; ++i) dst[i] = from_f32<T>(x[i]);
}

template <int D, int FMT, bool IS_V>
__device__ __forceinline__ void quant_store(const float (&x)[D / 32], int lane, uint8_t* __restrict__ rec, int slot,
                                            float fp8_scale) {
  constexpr int EPL = D / 32;
  if (FMT == TSB200_KV_INT8 || FMT == TSB200_KV_FP8) {
    uint8_t code[EPL];
    if (FMT == TSB200_KV_INT8) {
      float m = 0.f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) m = fmaxf(m, fabsf(x[i]));
      m = warp_max(m);
      const float s = __fdiv_rn(m, 127.0f);
      const float den = __fadd_rn(s, 1e-6f);
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        float q = fminf(fmaxf(rintf(__fdiv_rn(x[i], den)), -127.f), 127.f);
        code[i] = (uint8_t)(int8_t)(int)q;
      }
      if (lane == 0) reinterpret_cast<float*>(rec + 16 * D)[slot] = s;
    } else {
#pragma unroll
      for (int i = 0; i < EPL; ++i)
        code[i] = (uint8_t)__nv_cvt_float_to_fp8(__fdiv_rn(x[i], fp8_scale), __NV_SATFINITE, __NV_E4M3);
    }
    if (!IS_V) {
      typename BytesN<EPL>::type packed = 0;
#pragma unroll
      for (int i = 0; i < EPL; ++i) packed |= (typename BytesN<EPL>::type)code[i] << (8 * i);
      *reinterpret_cast<typename BytesN<EPL>::type*>(rec + slot * D + lane * EPL) = packed;
    } else {
#pragma unroll
      for (int i = 0; i < EPL; ++i) rec[(lane * EPL + i) * 16 + slot] = code[i];
    }
  } else {  // NVFP4
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) m = fmaxf(m, fabsf(x[i]));
#pragma unroll
    for (int o = 1; o < 16 / EPL; o <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const uint8_t sb = (uint8_t)__nv_cvt_float_to_fp8(__fdiv_rn(m, 6.0f), __NV_SATFINITE, __NV_E4M3);
    const float sd = e4m3_to_f32(sb);
    uint8_t byte[EPL / 2];
#pragma unroll
    for (int i = 0; i < EPL / 2; ++i) {
      if (sd > 0.f) {
        float2 f = make_float2(__fdiv_rn(x[2 * i], sd), __fdiv_rn(x[2 * i + 1], sd));
        byte[i] = (uint8_t)__nv_cvt_float2_to_fp4x2(f, __NV_E2M1, cudaRoundNearest);
      } else {
        byte[i] = 0;
      }
    }
    const int blk = (lane * EPL) / 16;
    const bool blk_leader = ((lane * EPL) % 16) == 0;
    if (!IS_V) {
      typename BytesN<EPL / 2>::type packed = 0;
#pragma unroll
      for (int i = 0; i < EPL / 2; ++i) packed |= (typename BytesN<EPL / 2>::type)byte[i] << (8 * i);
      *reinterpret_cast<typename BytesN<EPL / 2>::type*>(rec + slot * (D / 2) + lane * (EPL / 2)) = packed;
      if (blk_leader) rec[16 * (D / 2) + slot * (D / 16) + blk] = sb;
    } else {
#pragma unroll
      for (int i = 0; i < EPL / 2; ++i) rec[(lane * (EPL / 2) + i) * 16 + slot] = byte[i];
      if (blk_leader) rec[16 * (D / 2) + blk * 16 + slot] = sb;
    }
  }
}

template <typename T, int D, int FMT>
__global__ void kv_append_kernel(tsb200_kv_desc kv, T* __restrict__ q, int64_t qs, int qheads,
                                 const T* __restrict__ k, const T* __restrict__ v, int64_t ks,
                                 int64_t vs_, int64_t B,
                                 int64_t Tn, const int32_t* __restrict__ new_lens, const float* __restrict__ rope_cos,
                                 const float* __restrict__ rope_sin, int64_t rope_rows, int64_t rec_bytes) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t total = B * Tn * kv.hkv;
  if (warp >= total) {
    // extra warps: rotate the query heads in place (same rounding points as the key path)
    const int64_t qw = warp - total;
    if (q == nullptr || qw >= B * Tn * qheads || rope_cos == nullptr) return;
    const int qh = (int)(qw % qheads);
    const int64_t qbt = qw / qheads;
    const int64_t qb = qbt / Tn, qj = qbt - qb * Tn;
    if (new_lens && qj >= new_lens[qb]) return;
    int64_t qp = (int64_t)kv.seq_lens[qb] + qj;
    qp = qp < 0 ? 0 : (qp >= rope_rows ? rope_rows - 1 : qp);
    float xq[D / 32];
    T* dst = q + qbt * qs + (int64_t)qh * D;
    load_vec<T, D>(dst, lane, xq, true, rope_cos + qp * (D / 2), rope_sin + qp * (D / 2));
#pragma unroll
    for (int i = 0; i < D / 32; ++i) dst[lane * (D / 32) + i] = from_f32<T>(xq[i]);
    return;
  }
  const int h = (int)(warp % kv.hkv);
  const int64_t bt = warp / kv.hkv;
  const int64_t b = bt / Tn, j = bt - b * Tn;
  if (new_lens && j >= new_lens[b]) return;
  const int64_t p = (int64_t)kv.seq_lens[b] + j;
  if (p < 0 || (p >> 4) >= kv.bt_stride) return;
  const int64_t page = kv.block_table[b * kv.bt_stride + (p >> 4)];
  if (page < 0 || page >= kv.num_pages) return;
  const int slot = (int)(p & 15);
  const int64_t rec = (page * kv.hkv + h) * rec_bytes;
  const bool rope = rope_cos != nullptr;
  const int64_t rp = p >= rope_rows ? rope_rows - 1 : p;
  float x[D / 32];
  float kscale = 1.f, vscale = 1.f;
  if (FMT == TSB200_KV_FP8) {
    kscale = kv.k_scale[b * kv.hkv + h];
    vscale = kv.v_scale[b * kv.hkv + h];
  }
  load_vec<T, D>(k + bt * ks + (int64_t)h * D, lane, x, rope, rope ? rope_cos + rp * (D / 2) : nullptr, rope ? rope_sin + rp * (D / 2) : nullptr);
  if (FMT >= TSB200_KV_F32) dense_store<T, D>(x, lane, kv.k_pool + rec, slot);
  else quant_store<D, FMT, false>(x, lane, kv.k_pool + rec, slot, kscale);
  load_vec<T, D>(v + bt * vs_ + (int64_t)h * D, lane, x, false, nullptr, nullptr);
  if (FMT >= TSB200_KV_F32) dense_store<T, D>(x, lane, kv.v_pool + rec, slot);
  else quant_store<D, FMT, true>(x, lane, kv.v_pool + rec, slot, vscale);
}

// One CTA per (b, h): amax over the T tokens of the prompt -> scale = amax/448 (1 if 0).
template <typename T, int D>
__global__ void kv_fp8_scales_kernel(const T* __restrict__ k, const T* __restrict__ v, int64_t Tn, int hkv,
                                     const int32_t* __restrict__ pos0, const float* __restrict__ rope_cos,
                                     const float* __restrict__ rope_sin, int64_t rope_rows, float* __restrict__ k_scale,
                                     float* __restrict__ v_scale) {
  __shared__ float shk[32], shv[32];
  const int64_t b = blockIdx.x / hkv;
  const int h = blockIdx.x % hkv;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const bool rope = rope_cos != nullptr;
  float mk = 0.f, mv = 0.f;
  for (int64_t t = w; t < Tn; t += nw) {
    const int64_t vec = (b * Tn + t) * hkv + h;
    int64_t p = (pos0 ? (int64_t)pos0[b] : 0) + t;
    p = p >= rope_rows ? rope_rows - 1 : p;
    float x[D / 32];
    load_vec<T, D>(k + vec * D, lane, x, rope, rope ? rope_cos + p * (D / 2) : nullptr, rope ? rope_sin + p * (D / 2) : nullptr);
#pragma unroll
    for (int i = 0; i < D / 32; ++i) mk = fmaxf(mk, fabsf(x[i]));
    load_vec<T, D>(v + vec * D, lane, x, false, nullptr, nullptr);
#pragma unroll
    for (int i = 0; i < D / 32; ++i) mv = fmaxf(mv, fabsf(x[i]));
  }
  mk = warp_max(mk);
  mv = warp_max(mv);
  if (lane == 0) { shk[w] = mk; shv[w] = mv; }
  __syncthreads();
  if (w == 0) {
    mk = warp_max(lane < nw ? shk[lane] : 0.f);
    mv = warp_max(lane < nw ? shv[lane] : 0.f);
    if (lane == 0) {
      k_scale[blockIdx.x] = mk > 0.f ? __fdiv_rn(mk, 448.0f) : 1.0f;
      v_scale[blockIdx.x] = mv > 0.f ? __fdiv_rn(mv, 448.0f) : 1.0f;
    }
  }
}

template <typename T, int D>
int launch_append(const tsb200_kv_desc& kv, void* q, int64_t qs, int qheads, const void* k, const void* v, int64_t ks, int64_t vs, int64_t B, int64_t Tn, const int32_t* new_lens,
                  const float* rc, const float* rs, int64_t rr, cudaStream_t s) {
  const int64_t warps = B * Tn * (kv.hkv + (q ? qheads : 0));
  const int64_t blocks = (warps + 7) / 8;
  if (blocks > 0x7fffffffLL) return TSB200_ERR_UNSUPPORTED;
  const int64_t rec = (int64_t)tsb200_kv_record_bytes(kv.format, D);
  switch (kv.format) {
    case TSB200_KV_INT8:
      TSB_CUDA(launch_kernel(kv_append_kernel<T, D, TSB200_KV_INT8>, dim3((unsigned)blocks), dim3(256), 0, s, kv, (T*)q, qs, qheads, (const T*)k, (const T*)v, ks, vs, B, Tn, new_lens, rc, rs, rr, rec));
      break;
    case TSB200_KV_FP8:
      TSB_CUDA(launch_kernel(kv_append_kernel<T, D, TSB200_KV_FP8>, dim3((unsigned)blocks), dim3(256), 0, s, kv, (T*)q, qs, qheads, (const T*)k, (const T*)v, ks, vs, B, Tn, new_lens, rc, rs, rr, rec));
      break;
    case TSB200_KV_NVFP4:
      TSB_CUDA(launch_kernel(kv_append_kernel<T, D, TSB200_KV_NVFP4>, dim3((unsigned)blocks), dim3(256), 0, s, kv, (T*)q, qs, qheads, (const T*)k, (const T*)v, ks, vs, B, Tn, new_lens, rc, rs, rr, rec));
      break;
    default:   // unquantized pages in the act dtype
      TSB_CUDA(launch_kernel(kv_append_kernel<T, D, TSB200_KV_F32>, dim3((unsigned)blocks), dim3(256), 0, s, kv, (T*)q, qs, qheads, (const T*)k, (const T*)v, ks, vs, B, Tn, new_lens, rc, rs, rr, rec));
  }
  TSB_LAUNCH_CHECK();
  return TSB200_OK;
}

int validate_kv(const tsb200_kv_desc* kv, bool need_table) {
  if (!kv) return TSB200_ERR_ARG;
  if (kv->format < 0 || kv->format > TSB200_KV_BF16) return TSB200_ERR_UNSUPPORTED;
  if (kv->head_dim != 64 && kv->head_dim != 128) return TSB200_ERR_UNSUPPORTED;
  if (kv->hkv <= 0 || kv->num_pages < 0 || kv->bt_stride < 0) return TSB200_ERR_ARG;
  if (!kv->k_pool || !kv->v_pool || !aligned(kv->k_pool, 16) || !aligned(kv->v_pool, 16)) return TSB200_ERR_ARG;
  if (need_table && (!kv->block_table || !kv->seq_lens)) return TSB200_ERR_ARG;
  if (kv->format == TSB200_KV_FP8 && (!kv->k_scale || !kv->v_scale)) return TSB200_ERR_ARG;
  return TSB200_OK;
}

}  // namespace tsb

using namespace tsb;

extern "C" {

size_t tsb200_kv_record_bytes(int format, int head_dim) {
  if (head_dim <= 0 || head_dim % 32) return 0;
  switch (format) {
    case TSB200_KV_INT8: return (size_t)16 * head_dim + 64;
    case TSB200_KV_FP8: return (size_t)16 * head_dim;
    case TSB200_KV_NVFP4: return (size_t)16 * head_dim / 2 + (size_t)head_dim;
    case TSB200_KV_F32: return (size_t)16 * head_dim * 4;
    case TSB200_KV_BF16: return (size_t)16 * head_dim * 2;
    default: return 0;
  }
}

int tsb200_kv_fp8_scales(const void* k, const void* v, int dtype, int64_t B, int64_t T, int hkv, int head_dim,
                         const int32_t* pos0, const float* rope_cos, const float* rope_sin, int64_t rope_rows,
                         float* k_scale, float* v_scale, void* stream) {
  TSB_REQUIRE_DEVICE();
  if (B < 0 || T < 0 || hkv <= 0) return TSB200_ERR_ARG;
  if (head_dim != 64 && head_dim != 128) return TSB200_ERR_UNSUPPORTED;
  if (dtype != TSB200_F32 && dtype != TSB200_BF16) return TSB200_ERR_UNSUPPORTED;
  if (B == 0) return TSB200_OK;
  if (!k_scale || !v_scale || (T > 0 && (!k || !v))) return TSB200_ERR_ARG;
  if ((rope_cos != nullptr) != (rope_sin != nullptr) || (rope_cos && rope_rows <= 0)) return TSB200_ERR_ARG;
  if (B * hkv > 0x7fffffffLL) return TSB200_ERR_UNSUPPORTED;
  cudaStream_t s = as_stream(stream);
  const unsigned g = (unsigned)(B * hkv);
#define TSB_SC(TT, DD) kv_fp8_scales_kernel<TT, DD><<<g, 256, 0, s>>>((const TT*)k, (const TT*)v, T, hkv, pos0, rope_cos, rope_sin, rope_rows, k_scale, v_scale)
  if (dtype == TSB200_F32) { if (head_dim == 64) TSB_SC(float, 64); else TSB_SC(float, 128); }
  else { if (head_dim == 64) TSB_SC(__nv_bfloat16, 64); else TSB_SC(__nv_bfloat16, 128); }
#undef TSB_SC
  TSB_LAUNCH_CHECK();
  return TSB200_OK;
}

int tsb200_rope_append(const tsb200_kv_desc* kv, void* q, int q_heads, int64_t q_token_stride, const void* k,
                       const void* v, int dtype, int64_t k_token_stride, int64_t v_token_stride, int64_t B, int64_t T,
                       const int32_t* new_lens, const float* rope_cos, const float* rope_sin, int64_t rope_rows,
                       void* stream) {
  TSB_REQUIRE_DEVICE();
  int st = validate_kv(kv, true);
  if (st != TSB200_OK) return st;
  if (B < 0 || T < 0 || q_heads < 0) return TSB200_ERR_ARG;
  if (dtype != TSB200_F32 && dtype != TSB200_BF16) return TSB200_ERR_UNSUPPORTED;
  if (B == 0 || T == 0) return TSB200_OK;
  if (!k || !v) return TSB200_ERR_ARG;
  if ((kv->format == TSB200_KV_F32 && dtype != TSB200_F32) || (kv->format == TSB200_KV_BF16 && dtype != TSB200_BF16))
    return TSB200_ERR_UNSUPPORTED;   // unquantized pages hold the act dtype
  if ((rope_cos != nullptr) != (rope_sin != nullptr) || (rope_cos && rope_rows <= 0)) return TSB200_ERR_ARG;
  if (q && (!rope_cos || q_heads <= 0)) return TSB200_ERR_ARG;
  const int64_t dense = (int64_t)kv->hkv * kv->head_dim;
  const int64_t ks = k_token_stride ? k_token_stride : dense, vs = v_token_stride ? v_token_stride : dense;
  const int64_t qs = q_token_stride ? q_token_stride : (int64_t)q_heads * kv->head_dim;
  if (ks < dense || vs < dense || (q && qs < (int64_t)q_heads * kv->head_dim)) return TSB200_ERR_ARG;
  cudaStream_t s = as_stream(stream);
  if (dtype == TSB200_F32)
    return kv->head_dim == 64 ? launch_append<float, 64>(*kv, q, qs, q_heads, k, v, ks, vs, B, T, new_lens, rope_cos, rope_sin, rope_rows, s)
                              : launch_append<float, 128>(*kv, q, qs, q_heads, k, v, ks, vs, B, T, new_lens, rope_cos, rope_sin, rope_rows, s);
  return kv->head_dim == 64 ? launch_append<__nv_bfloat16, 64>(*kv, q, qs, q_heads, k, v, ks, vs, B, T, new_lens, rope_cos, rope_sin, rope_rows, s)
                            : launch_append<__nv_bfloat16, 128>(*kv, q, qs, q_heads, k, v, ks, vs, B, T, new_lens, rope_cos, rope_sin, rope_rows, s);
}

int tsb200_kv_append(const tsb200_kv_desc* kv, const void* k, const void* v, int dtype, int64_t k_token_stride,
                     int64_t v_token_stride, int64_t B, int64_t T, const int32_t* new_lens, const float* rope_cos,
                     const float* rope_sin, int64_t rope_rows, void* stream) {
  return tsb200_rope_append(kv, nullptr, 0, 0, k, v, dtype, k_token_stride, v_token_stride, B, T, new_lens, rope_cos,
                            rope_sin, rope_rows, stream);
}

}  // extern "C"
