// Fused (RoPE on K +) quantize-and-append into the paged KV pools, and the FP8 scale
// reduction over a prompt.  One warp owns one (token, kv head) vector of d elements:
// lane l holds elements [l*d/32, (l+1)*d/32).  HBM-bound: reads 2*d*sizeof(act) bytes
// and writes 2*d*b_elem (+ scales) per vector.  Decode steps (one token per sequence) use
// kv_append_kernel; prompt chunks of 16 tokens or more use kv_append_pages_kernel, in which
// a CTA owns a whole page and writes the token-minor V record with 16-byte vectors.
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

// This lane's EPL elements of a vector, as fp32 (one 8- or 16-byte load when the vector is aligned for it).
template <typename T, int D>
__device__ __forceinline__ void load_raw(const T* __restrict__ src, int lane, float (&x)[D / 32]) {
  constexpr int EPL = D / 32;
  const T* p = src + lane * EPL;
  if (sizeof(T) * EPL == 8 && (reinterpret_cast<uintptr_t>(p) & 7) == 0) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const T* e = reinterpret_cast<const T*>(&r);
#pragma unroll
    for (int i = 0; i < EPL; ++i) x[i] = to_f32<T>(e[i]);
  } else if (sizeof(T) * EPL == 16 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&r);
#pragma unroll
    for (int i = 0; i < EPL; ++i) x[i] = to_f32<T>(e[i]);
  } else {
#pragma unroll
    for (int i = 0; i < EPL; ++i) x[i] = to_f32<T>(p[i]);
  }
}
// Rotate (optional) and round to T; returns this lane's EPL elements as fp32.
template <typename T, int D>
__device__ __forceinline__ void rope_vec(int lane, float (&x)[D / 32], bool rope, const float* __restrict__ cosr,
                                         const float* __restrict__ sinr) {
  constexpr int EPL = D / 32;
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
template <typename T, int D>
__device__ __forceinline__ void load_vec(const T* __restrict__ src, int lane, float (&x)[D / 32], bool rope,
                                         const float* __restrict__ cosr, const float* __restrict__ sinr) {
  load_raw<T, D>(src, lane, x);
  rope_vec<T, D>(lane, x, rope, cosr, sinr);
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
  // Programmatic dependent launch: the write position, the page and the scales (inputs that the launch directly before
  // this one does not produce) are looked up while that launch drains; the wait stands in front of the first access to
  // q, k and v and of every store.
  pdl_launch_dependents();
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
    pdl_wait();
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
  pdl_wait();
  load_vec<T, D>(k + bt * ks + (int64_t)h * D, lane, x, rope, rope ? rope_cos + rp * (D / 2) : nullptr, rope ? rope_sin + rp * (D / 2) : nullptr);
  if (FMT >= TSB200_KV_F32) dense_store<T, D>(x, lane, kv.k_pool + rec, slot);
  else quant_store<D, FMT, false>(x, lane, kv.k_pool + rec, slot, kscale);
  load_vec<T, D>(v + bt * vs_ + (int64_t)h * D, lane, x, false, nullptr, nullptr);
  if (FMT >= TSB200_KV_F32) dense_store<T, D>(x, lane, kv.v_pool + rec, slot);
  else quant_store<D, FMT, true>(x, lane, kv.v_pool + rec, slot, vscale);
}

// Bulk append (T >= 16 tokens per sequence, quantized formats): ONE CTA OWNS TWO consecutive PAGES of one (sequence, kv head).
// Its 16 warps quantize the page's 16 tokens; K goes out token-major as above (one contiguous vector per warp).  V is
// stored token-minor ([element][16 tokens], so that the decode kernels read consecutive tokens of one element from
// consecutive bytes): written token by token that is one byte per 16-byte row and a partial sector per element.
// Here the warps stage the page's V codes and scales in shared memory in the token-major form, and the CTA then
// writes the record transposed, 16 bytes (one element row) per thread - whole sectors, fully coalesced.  A page the
// append only partly covers (the first / last page of the range) keeps its other slots: those are written slot by slot.
// Extra CTAs along x rotate the query heads in place.
template <typename T, int D, int FMT>
__global__ void __launch_bounds__(512)
kv_append_pages_kernel(tsb200_kv_desc kv, T* __restrict__ q, int64_t qs, int qheads, const T* __restrict__ k,
                       const T* __restrict__ v, int64_t ks, int64_t vs_, int64_t Tn, const int32_t* __restrict__ new_lens,
                       const float* __restrict__ rope_cos, const float* __restrict__ rope_sin, int64_t rope_rows,
                       int64_t rec_bytes, int page_blocks) {
  constexpr int VB = FMT == TSB200_KV_NVFP4 ? D / 2 : D;                  // bytes of V codes per token
  constexpr int REC = FMT == TSB200_KV_INT8 ? 16 * D + 64 : (FMT == TSB200_KV_FP8 ? 16 * D : 9 * D);
  __shared__ __align__(16) uint8_t stage[REC];                            // the page's V record in token-major form
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t b = blockIdx.z;
  const int h = blockIdx.y;
  const int64_t n_b = new_lens ? min((int64_t)new_lens[b], Tn) : Tn;
  const int64_t start = kv.seq_lens[b];
  if ((int)blockIdx.x >= page_blocks) {
    // ---- query rotation: 16 (token, head) vectors per CTA
    if (q == nullptr || rope_cos == nullptr) return;
    const int64_t idx = (((int64_t)blockIdx.x - page_blocks) * gridDim.y + blockIdx.y) * 16 + w;
    if (idx >= Tn * qheads) return;
    const int64_t j = idx / qheads;
    const int qh = (int)(idx - j * qheads);
    if (j >= n_b) return;
    int64_t qp = start + j;
    qp = qp < 0 ? 0 : (qp >= rope_rows ? rope_rows - 1 : qp);
    float xq[D / 32];
    T* dst = q + (b * Tn + j) * qs + (int64_t)qh * D;
    load_vec<T, D>(dst, lane, xq, true, rope_cos + qp * (D / 2), rope_sin + qp * (D / 2));
#pragma unroll
    for (int i = 0; i < D / 32; ++i) dst[lane * (D / 32) + i] = from_f32<T>(xq[i]);
    return;
  }
  // ---- pages 2 * blockIdx.x and 2 * blockIdx.x + 1 of the appended range (logical page start / 16 + ...), slot w.
  // Both pages' vectors are requested before either is used (9 % faster for FP8 pages at 2048 tokens x batch 64; the
  // exact divisions of the quantization rules are what bounds the kernel).
  struct Page {
    int64_t p;
    bool valid, store, full;
    uint8_t *krec, *vrec;
  } pg[2];
  float kscale = 1.f, vscale = 1.f;
  if (FMT == TSB200_KV_FP8) {
    kscale = kv.k_scale[b * kv.hkv + h];
    vscale = kv.v_scale[b * kv.hkv + h];
  }
  const bool rope = rope_cos != nullptr;
  float x[2][D / 32], xv[2][D / 32];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int64_t lp = (start >> 4) + 2 * (int64_t)blockIdx.x + i;
    pg[i].p = lp * 16 + w;                              // position of this warp's token
    const int64_t j = pg[i].p - start;
    pg[i].valid = j >= 0 && j < n_b;
    const bool page_ok = lp < kv.bt_stride;
    int64_t page = page_ok ? kv.block_table[b * kv.bt_stride + lp] : -1;
    pg[i].store = page >= 0 && page < kv.num_pages;
    if (!pg[i].store) page = 0;
    // the page is covered completely when its first and last positions are both appended
    pg[i].full = lp * 16 >= start && lp * 16 + 15 < start + n_b;
    pg[i].krec = kv.k_pool + (page * kv.hkv + h) * rec_bytes;
    pg[i].vrec = kv.v_pool + (page * kv.hkv + h) * rec_bytes;
    if (pg[i].valid && pg[i].store) {
      const int64_t bt = b * Tn + j;
      load_raw<T, D>(k + bt * ks + (int64_t)h * D, lane, x[i]);
      load_raw<T, D>(v + bt * vs_ + (int64_t)h * D, lane, xv[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint8_t* const krec = pg[i].krec;
    uint8_t* const vrec = pg[i].vrec;
    if (pg[i].valid && pg[i].store) {
      const int64_t rp = pg[i].p >= rope_rows ? rope_rows - 1 : pg[i].p;
      rope_vec<T, D>(lane, x[i], rope, rope ? rope_cos + rp * (D / 2) : nullptr, rope ? rope_sin + rp * (D / 2) : nullptr);
      quant_store<D, FMT, false>(x[i], lane, krec, w, kscale);
      quant_store<D, FMT, false>(xv[i], lane, stage, w, vscale);        // token-major, into shared memory
    }
    __syncthreads();
    if (pg[i].store && pg[i].full) {
      // transposed record: row e (16 bytes) = the codes of element (pair) e for tokens 0..15
      for (int e = threadIdx.x; e < VB; e += blockDim.x) {
        unsigned wds[4];
#pragma unroll
        for (int c = 0; c < 4; ++c)
          wds[c] = (unsigned)stage[(4 * c) * VB + e] | ((unsigned)stage[(4 * c + 1) * VB + e] << 8) |
                   ((unsigned)stage[(4 * c + 2) * VB + e] << 16) | ((unsigned)stage[(4 * c + 3) * VB + e] << 24);
        *reinterpret_cast<uint4*>(vrec + (int64_t)e * 16) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
      }
      if constexpr (FMT == TSB200_KV_INT8) {              // fp32 scale per token: same place in both forms
        if (threadIdx.x < 16) reinterpret_cast<float*>(vrec + 16 * D)[threadIdx.x] = reinterpret_cast<const float*>(stage + 16 * D)[threadIdx.x];
      } else if constexpr (FMT == TSB200_KV_NVFP4) {      // block scales: [16 tokens][D/16] -> [D/16][16 tokens]
        if (threadIdx.x < D) {
          const int blk = threadIdx.x >> 4, t = threadIdx.x & 15;
          vrec[16 * (D / 2) + blk * 16 + t] = stage[16 * (D / 2) + t * (D / 16) + blk];
        }
      }
    } else if (pg[i].store && pg[i].valid) {
      // partly covered page: only this warp's slot is written
      for (int e = lane; e < VB; e += 32) vrec[(int64_t)e * 16 + w] = stage[w * VB + e];
      if constexpr (FMT == TSB200_KV_INT8) {
        if (lane == 0) reinterpret_cast<float*>(vrec + 16 * D)[w] = reinterpret_cast<const float*>(stage + 16 * D)[w];
      } else if constexpr (FMT == TSB200_KV_NVFP4) {
        if (lane < D / 16) vrec[16 * (D / 2) + lane * 16 + w] = stage[16 * (D / 2) + w * (D / 16) + lane];
      }
    }
    if (i == 0) __syncthreads();                           // the staging buffer is reused by the second page
  }
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
#pragma unroll 4                         // several tokens' vectors in flight per warp: the loop is latency-bound otherwise
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
  const int64_t rec = (int64_t)tsb200_kv_record_bytes(kv.format, D);
  if (Tn >= 16 && kv.format <= TSB200_KV_NVFP4 && B <= 65535 && kv.hkv <= 65535) {
    // bulk: one CTA per (sequence, kv head, page touched) + CTAs that rotate the query heads
    const int page_blocks = (int)(((Tn + 15) / 16 + 1 + 1) / 2);  // two pages per CTA; the range may straddle one more page than it fills
    const int64_t q_blocks = q ? (Tn * qheads + 16 * kv.hkv - 1) / (16 * (int64_t)kv.hkv) : 0;
    const dim3 grid((unsigned)(page_blocks + q_blocks), (unsigned)kv.hkv, (unsigned)B);
    switch (kv.format) {
      case TSB200_KV_INT8:
        TSB_CUDA(launch_kernel(kv_append_pages_kernel<T, D, TSB200_KV_INT8>, grid, dim3(512), 0, s, kv, (T*)q, qs, qheads, (const T*)k, (const T*)v, ks, vs, Tn, new_lens, rc, rs, rr, rec, page_blocks));
        break;
      case TSB200_KV_FP8:
        TSB_CUDA(launch_kernel(kv_append_pages_kernel<T, D, TSB200_KV_FP8>, grid, dim3(512), 0, s, kv, (T*)q, qs, qheads, (const T*)k, (const T*)v, ks, vs, Tn, new_lens, rc, rs, rr, rec, page_blocks));
        break;
      default:
        TSB_CUDA(launch_kernel(kv_append_pages_kernel<T, D, TSB200_KV_NVFP4>, grid, dim3(512), 0, s, kv, (T*)q, qs, qheads, (const T*)k, (const T*)v, ks, vs, Tn, new_lens, rc, rs, rr, rec, page_blocks));
    }
    TSB_LAUNCH_CHECK();
    return TSB200_OK;
  }
  const int64_t warps = B * Tn * (kv.hkv + (q ? qheads : 0));
  const int64_t blocks = (warps + 7) / 8;
  if (blocks > 0x7fffffffLL) return TSB200_ERR_UNSUPPORTED;
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
