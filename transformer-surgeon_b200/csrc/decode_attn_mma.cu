// Split-K paged decode attention on tensor cores (int8, FP8-e4m3 and NVFP4 pages).
//
// Replaces transformersurgeon/blocks/mha.py:9-103 (attention(): GQA, softmax, @V) for the
// decode step.  One CTA = one (sequence, kv head, split); its warps (4, or 6 for int8 pages) take pages
// round-robin.  Each warp streams its pages through a private ring of shared-memory
// stages with 16-byte cp.async copies (K record placed with an XOR swizzle so the
// fragment reads are bank-conflict free), and computes, per 16-token page,
//     S^T[token, head] = K_page . Q^T          (8 x mma.m16n8k16, f16 in / f32 acc)
//     online softmax over tokens per head       (warp shuffles over the token lanes)
//     O^T[dim, head]  += V^T_page . P^T         (8 x mma.m16n8k16)
// so the whole GQA group (<= 8 query heads) shares one read of the page.  Codes are
// widened to f16 in registers (exact for e4m3 and int8); scales are applied in fp32.  NVFP4 pages:
// an e2m1 code times its e4m3 block scale is exact in f16 (2 x 4 significant bits), so K goes to
// the MMA as code * scale; for V the block scale of a token is folded into that token's softmax
// weight (one product per 16-dim block and token instead of one per element).
// Partials (m, l, acc) go to the workspace; decode_attn_reduce_kernel merges splits.
#include "decode_attn_common.cuh"

namespace tsb {

template <typename T, int D> int launch_reduce(const float* ws, int64_t BH, int S, void* out, cudaStream_t st);
template <typename T>
int launch_attn_fp8(const tsb200_kv_desc& kv, const void* q, int64_t qs, int H, float sm_scale, int64_t max_seq_len, int S,
                    int64_t B, float* ws, int* counters, void* out, int* status, cudaStream_t st);
int validate_attn_args(const tsb200_kv_desc* kv, const void* q, void* out, int dtype, int64_t B, int H,
                       int64_t max_seq_len, void* workspace, size_t workspace_bytes, bool& noop, size_t need_bytes);

namespace {

// Warps per CTA and ring stages per warp, by page format (measured at batch 32-64, context 2k-4k): int8 pages
// run 8 % faster with 6 warps x 3 stages (two CTAs = 12 warps per SM); NVFP4 and FP8 keep 4 x 4 (three CTAs).
template <int FMT> struct AttnCfg {
  static constexpr int kWarps = FMT == TSB200_KV_INT8 ? 6 : 4;
  static constexpr int kStages = FMT == TSB200_KV_INT8 ? 3 : 4;
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned movmatrix_trans(unsigned a) {
  unsigned d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ unsigned pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&h);
}
// Two 8-bit codes (low 16 bits of w) -> f16x2, low byte in the low half.
template <int FMT> __device__ __forceinline__ unsigned widen2(unsigned w16) {
  if (FMT == TSB200_KV_FP8) {
    __half2_raw r = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w16 & 0xffffu), __NV_E4M3);
    return (unsigned)r.x | ((unsigned)r.y << 16);
  } else {
    // int8 -> f16: (code ^ 0x80) | 0x6400 is the f16 1024 + 128 + code; subtract 1152.
    const unsigned u = (w16 ^ 0x8080u);
    unsigned v = __byte_perm(u, 0x64646464u, 0x4140);   // {0x64, b1, 0x64, b0}
    const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6480));
    __half2 h = __hsub2(*reinterpret_cast<__half2*>(&v), bias);
    return *reinterpret_cast<unsigned*>(&h);
  }
}
// Two e4m3 codes (low 16 bits of w) -> f16x2 holding value * 2^-8, with integer instructions only:
// sign to bit 15, exponent+mantissa shifted to f16 bits 13..7 (e4m3 exponent bias 7 vs f16 bias 15,
// hence the 2^-8; e4m3 subnormals land on f16 subnormals, also exactly).  Used for the K operand so
// that only half of the widening work sits on the conversion pipe; the caller folds 2^8 into its scale.
__device__ __forceinline__ unsigned widen2_e4m3_alu(unsigned w16) {
  const unsigned t = __byte_perm(w16, 0u, 0x1404);          // {b1, 0, b0, 0}: each code in the high byte of a half
  return (t & 0x80008000u) | ((t >> 1) & 0x3f803f80u);
}
#ifndef TSB_ATTN_ALU_WIDEN
#define TSB_ATTN_ALU_WIDEN 1
#endif
template <int FMT> __device__ __forceinline__ unsigned widen2_k(unsigned w16) {
  return (FMT == TSB200_KV_FP8 && TSB_ATTN_ALU_WIDEN) ? widen2_e4m3_alu(w16) : widen2<FMT>(w16);
}

// Row swizzle of the K record (rows of 128 bytes = 8 chunks): adjacent token rows land in
// different halves of the bank space, rows two apart in different chunks.
__device__ __forceinline__ int kswz(int row) { return ((row & 1) << 2) | ((row >> 1) & 3); }

template <int D> __device__ __forceinline__ int k_phys_chunk(int row, int j) {
  return row * (D / 16) + (D == 128 ? (j ^ kswz(row)) : j);
}
// NVFP4 K rows are D/2 bytes (D/32 chunks): rows four apart would meet in the same banks, so the
// 32-byte half of the row is flipped for every other group of four rows.
template <int D> __device__ __forceinline__ int k4_phys_chunk(int row, int j) {
  return row * (D / 32) + (D == 128 ? (j ^ (((row >> 2) & 1) << 1)) : j);
}
// e2m1 codes n_A and n_{A+4} of the 8 in a 32-bit word (16 bits apart, so one shift serves both) ->
// f16x2 holding value * 2^-14, with integer instructions only: the sign goes to bit 15 and the
// three magnitude bits (2 exponent, 1 mantissa; bias 1 against f16's 15) to f16 bits 11..9; code
// 0.5 lands on an f16 subnormal, also exactly.  The conversion instructions are far slower.
template <int A> __device__ __forceinline__ unsigned e2m1_pair_alu(unsigned w) {
  const unsigned x = w << (12 - 4 * A);
  return (x & 0x80008000u) | ((x >> 3) & 0x0E000E00u);
}
// e4m3 codes in bytes 1 and 3 of t -> f16x2 of value * 2^-8 (see widen2_e4m3_alu)
__device__ __forceinline__ unsigned e4m3_hi_bytes_alu(unsigned t) { return (t & 0x80008000u) | ((t >> 1) & 0x3f803f80u); }
__device__ __forceinline__ unsigned hmul2_u(unsigned a, unsigned b) {
  __half2 h = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<unsigned*>(&h);
}
template <int FMT, int D> struct RecBytes {
  static constexpr int value = FMT == TSB200_KV_INT8 ? 16 * D + 64 : (FMT == TSB200_KV_NVFP4 ? 9 * D : 16 * D);
};

template <typename T, int D, int FMT>
__global__ void __launch_bounds__(AttnCfg<FMT>::kWarps * 32)
decode_attn_mma_kernel(tsb200_kv_desc kv, const T* __restrict__ q, int64_t qs, int H, float sm_scale, int64_t max_seq_len, int S,
                       float* __restrict__ ws, int* __restrict__ counters, T* __restrict__ out) {
  constexpr bool FP4 = FMT == TSB200_KV_NVFP4;
  constexpr int kWarps = AttnCfg<FMT>::kWarps, kStages = AttnCfg<FMT>::kStages;
  constexpr int REC = RecBytes<FMT, D>::value;
  constexpr int CODE_CHUNKS = FP4 ? D / 2 : D; // 16-byte chunks of K codes (placed with the row swizzle)
  constexpr int ROW_CHUNKS = FP4 ? D / 32 : D / 16;
  constexpr int REC_CHUNKS = REC / 16;
  constexpr int STAGE = 2 * REC;
  constexpr int NC = D / 16;                    // k-steps of QK, m-tiles of PV
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_launch_dependents();
  pdl_wait();     // q, the page just appended and seq_lens come from the preceding kernels

  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int gid = lane >> 2, tid = lane & 3;
  const int b = blockIdx.x / kv.hkv, hk = blockIdx.x % kv.hkv, s = blockIdx.y;
  const int g = H / kv.hkv;
  const int g0 = blockIdx.z * 8, gn = min(8, g - g0);
  int len = kv.seq_lens[b];
  len = len < 0 ? 0 : (len > max_seq_len ? (int)max_seq_len : len);
  const bool fuse_reduce = S > 0;      // S < 0: |S| splits, partials only (a reducer kernel follows)
  S = S < 0 ? -S : S;
  int pb, pe;
  split_range(len, s, S, pb, pe);

  // Q^T fragments (B operand): this lane holds head g0+gid at the dims of its k-slots.
  unsigned qf[NC][2];
  {
    const bool valid = gid < gn;
    const T* qp = q + (int64_t)b * qs + (int64_t)(hk * g + g0 + (valid ? gid : 0)) * D;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      // int8 / fp8: the step's k-slots are 4 consecutive dims; NVFP4: dims (x, x + 4) and (x + 1, x + 5),
      // the pairs that e2m1_pair_alu extracts from a word of 8 codes
      const int base = FMT == TSB200_KV_NVFP4 ? 16 * (tid + 4 * (c >> 2)) + 8 * ((c & 3) >> 1) + 2 * (c & 1)
                                              : 16 * (tid + 4 * (c >> 2)) + 4 * (c & 3);
      constexpr int o1 = FMT == TSB200_KV_NVFP4 ? 4 : 1, o2 = FMT == TSB200_KV_NVFP4 ? 1 : 2, o3 = FMT == TSB200_KV_NVFP4 ? 5 : 3;
      float f0 = 0.f, f1 = 0.f, f2 = 0.f, f3 = 0.f;
      if (valid) { f0 = to_f32<T>(qp[base]); f1 = to_f32<T>(qp[base + o1]); f2 = to_f32<T>(qp[base + o2]); f3 = to_f32<T>(qp[base + o3]); }
      qf[c][0] = pack_h2(f0, f1);
      qf[c][1] = pack_h2(f2, f3);
    }
  }
  float kscale = 1.f, vscale = 1.f;
  if (FMT == TSB200_KV_FP8) { kscale = kv.k_scale[b * kv.hkv + hk]; vscale = kv.v_scale[b * kv.hkv + hk]; }
  // FP8 keys are widened to value * 2^-8 (widen2_e4m3_alu): 256 restores the scale
  // NVFP4 keys reach the MMA as code * block scale * 2^-7, values as code * 2^-14 (see below)
  if (FMT == TSB200_KV_NVFP4) vscale = 16384.0f;
  const float sc = sm_scale * 1.4426950408889634f * kscale *
                   ((FMT == TSB200_KV_FP8 && TSB_ATTN_ALU_WIDEN) ? 256.0f : (FMT == TSB200_KV_NVFP4 ? 128.0f : 1.0f));

  float oacc[NC][4];
#pragma unroll
  for (int i = 0; i < NC; ++i) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // heads 2*tid, 2*tid+1 (log2 domain)

  uint8_t* ring = smem + (size_t)w * kStages * STAGE;
  const int n_my = (pe - pb - w + kWarps - 1) / kWarps > 0 ? (pe - pb - w + kWarps - 1) / kWarps : 0;
  const int64_t rec_stride = (int64_t)kv.hkv * REC;

  auto issue = [&](int it) {
    if (it < n_my) {
      const int pg = pb + w + it * kWarps;
      int64_t page = kv.block_table[(int64_t)b * kv.bt_stride + pg];
      page = page < 0 ? 0 : (page >= kv.num_pages ? kv.num_pages - 1 : page);
      const uint8_t* kr = kv.k_pool + page * rec_stride + (int64_t)hk * REC;
      const uint8_t* vr = kv.v_pool + page * rec_stride + (int64_t)hk * REC;
      uint8_t* sK = ring + (it % kStages) * STAGE;
      uint8_t* sV = sK + REC;
#pragma unroll
      for (int ci = lane; ci < REC_CHUNKS; ci += 32) {
        int phys = ci;
        if (ci < CODE_CHUNKS)
          phys = FP4 ? k4_phys_chunk<D>(ci / ROW_CHUNKS, ci % ROW_CHUNKS) : k_phys_chunk<D>(ci / ROW_CHUNKS, ci % ROW_CHUNKS);
        cp_async16(sK + phys * 16, kr + ci * 16);
        cp_async16(sV + ci * 16, vr + ci * 16);
      }
    }
    cp_async_commit();
  };

#pragma unroll
  for (int i = 0; i < kStages - 1; ++i) issue(i);

  const int r1 = 4 * (gid >> 1) + (gid & 1), r2 = r1 + 2;   // token rows of this lane in S^T
  for (int it = 0; it < n_my; ++it) {
    issue(it + kStages - 1);
    cp_async_wait<kStages - 1>();
    __syncwarp();
    const int pg = pb + w + it * kWarps;
    const int nt = min(16, len - pg * 16);
    const uint8_t* sK = ring + (it % kStages) * STAGE;
    const uint8_t* sV = sK + REC;

    // ---- S^T = K . Q^T -----------------------------------------------------------
    float sacc[4] = {0.f, 0.f, 0.f, 0.f};
    if (FP4) {
      // the lane's 16 dims of a row = 8 bytes of codes = exactly one scale block
      const uint8_t* ksc = sK + 16 * (D / 2);
#pragma unroll
      for (int hh = 0; hh < D / 64; ++hh) {
        const int j = tid + 4 * hh;
        const uint2 ka = *reinterpret_cast<const uint2*>(sK + k4_phys_chunk<D>(r1, j >> 1) * 16 + 8 * (j & 1));
        const uint2 kb = *reinterpret_cast<const uint2*>(sK + k4_phys_chunk<D>(r2, j >> 1) * 16 + 8 * (j & 1));
        // block scale * 2^-8 (integer widening) * 2^15 -> scale * 2^7 <= 57344; code * 2^-14 times that is
        // code * scale * 2^-7, exact in f16 (6 significant bits, >= 2^-17)
        const unsigned k215 = 0x78007800u;
        const unsigned sa = hmul2_u(e4m3_hi_bytes_alu((unsigned)ksc[r1 * (D / 16) + j] * 0x01000100u), k215);
        const unsigned sb = hmul2_u(e4m3_hi_bytes_alu((unsigned)ksc[r2 * (D / 16) + j] * 0x01000100u), k215);
        mma16816(sacc, hmul2_u(e2m1_pair_alu<0>(ka.x), sa), hmul2_u(e2m1_pair_alu<0>(kb.x), sb), hmul2_u(e2m1_pair_alu<1>(ka.x), sa),
                 hmul2_u(e2m1_pair_alu<1>(kb.x), sb), qf[4 * hh][0], qf[4 * hh][1]);
        mma16816(sacc, hmul2_u(e2m1_pair_alu<2>(ka.x), sa), hmul2_u(e2m1_pair_alu<2>(kb.x), sb), hmul2_u(e2m1_pair_alu<3>(ka.x), sa),
                 hmul2_u(e2m1_pair_alu<3>(kb.x), sb), qf[4 * hh + 1][0], qf[4 * hh + 1][1]);
        mma16816(sacc, hmul2_u(e2m1_pair_alu<0>(ka.y), sa), hmul2_u(e2m1_pair_alu<0>(kb.y), sb), hmul2_u(e2m1_pair_alu<1>(ka.y), sa),
                 hmul2_u(e2m1_pair_alu<1>(kb.y), sb), qf[4 * hh + 2][0], qf[4 * hh + 2][1]);
        mma16816(sacc, hmul2_u(e2m1_pair_alu<2>(ka.y), sa), hmul2_u(e2m1_pair_alu<2>(kb.y), sb), hmul2_u(e2m1_pair_alu<3>(ka.y), sa),
                 hmul2_u(e2m1_pair_alu<3>(kb.y), sb), qf[4 * hh + 3][0], qf[4 * hh + 3][1]);
      }
    }
#pragma unroll
    for (int hh = 0; hh < (FP4 ? 0 : D / 64); ++hh) {
      const int j = tid + 4 * hh;
      const uint4 ka = *reinterpret_cast<const uint4*>(sK + k_phys_chunk<D>(r1, j) * 16);
      const uint4 kb = *reinterpret_cast<const uint4*>(sK + k_phys_chunk<D>(r2, j) * 16);
      const unsigned wa[4] = {ka.x, ka.y, ka.z, ka.w};
      const unsigned wb[4] = {kb.x, kb.y, kb.z, kb.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = 4 * hh + i;
        mma16816(sacc, widen2_k<FMT>(wa[i]), widen2_k<FMT>(wb[i]), widen2_k<FMT>(wa[i] >> 16), widen2_k<FMT>(wb[i] >> 16),
                 qf[c][0], qf[c][1]);
      }
    }
    // ---- online softmax over the page's tokens (rows) per head (column) -------------
    float ks1 = 1.f, ks2 = 1.f, vs1 = 1.f, vs2 = 1.f;
    if (FMT == TSB200_KV_INT8) {
      const float* ksc = reinterpret_cast<const float*>(sK + 16 * D);
      const float* vsc = reinterpret_cast<const float*>(sV + 16 * D);
      ks1 = ksc[r1]; ks2 = ksc[r2]; vs1 = vsc[r1]; vs2 = vsc[r2];
    }
    const bool ok1 = r1 < nt, ok2 = r2 < nt;
    const float s0 = ok1 ? sacc[0] * (sc * ks1) : -INFINITY;
    const float s1 = ok1 ? sacc[1] * (sc * ks1) : -INFINITY;
    const float s2 = ok2 ? sacc[2] * (sc * ks2) : -INFINITY;
    const float s3 = ok2 ? sacc[3] * (sc * ks2) : -INFINITY;
    float mx0 = fmaxf(s0, s2), mx1 = fmaxf(s1, s3);
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
    }
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);   // finite: token 0 of a page is always valid
    const float c0 = exp2f(m0 - mn0), c1 = exp2f(m1 - mn1);
    const float p0 = exp2f(s0 - mn0), p1 = exp2f(s1 - mn1), p2 = exp2f(s2 - mn0), p3 = exp2f(s3 - mn1);
    l0 = l0 * c0 + (p0 + p2);
    l1 = l1 * c1 + (p1 + p3);
    m0 = mn0; m1 = mn1;
    if (FP4) vs1 = vs2 = 256.0f;                // NVFP4: the block scales multiply P as scale * 2^-8
    const unsigned P1 = pack_h2(ok1 ? p0 * vs1 : 0.f, ok1 ? p1 * vs1 : 0.f);
    const unsigned P2 = pack_h2(ok2 ? p2 * vs2 : 0.f, ok2 ? p3 * vs2 : 0.f);
    unsigned pb0 = movmatrix_trans(P1);         // tokens 4*tid, 4*tid+1 of head gid
    unsigned pb1 = movmatrix_trans(P2);         // tokens 4*tid+2, 4*tid+3
    if (FP4) {                                  // NVFP4 pairs tokens (4*tid, 4*tid+2) and (4*tid+1, 4*tid+3)
      const unsigned t0 = __byte_perm(pb0, pb1, 0x5410), t1 = __byte_perm(pb0, pb1, 0x7632);
      pb0 = t0; pb1 = t1;
    }
    // bytes of this lane's 4 tokens that are inside the sequence (stale slots -> +0)
    unsigned vmask = 0xffffffffu;
    if (nt < 16) {
      const int left = nt - 4 * tid;
      vmask = left >= 4 ? 0xffffffffu : (left <= 0 ? 0u : (0xffffffffu >> (8 * (4 - left))));
    }
    // ---- O^T += V^T . P^T -----------------------------------------------------------
    if (FP4) {
      const uint8_t* vsc = sV + 16 * (D / 2);
#pragma unroll
      for (int mt = 0; mt < NC; ++mt) {
        // one word = tokens 4*tid..4*tid+3 of dims 16*mt + 2*gid (low nibbles) and + 1 (high nibbles):
        // MMA rows gid / gid + 8 are those two dims
        const unsigned wv = *reinterpret_cast<const unsigned*>(sV + (8 * mt + gid) * 16 + 4 * tid);
        const unsigned sw = *reinterpret_cast<const unsigned*>(vsc + mt * 16 + 4 * tid) & vmask;   // stale slots: scale +0
        // code pairs 16 bits apart = tokens (0, 2) and (1, 3) of the lane's four; values enter as code * 2^-14
        // (2^14 is restored with the split scale), weights as p * 2^8 * (block scale * 2^-8)
        const unsigned b0 = hmul2_u(pb0, e4m3_hi_bytes_alu(__byte_perm(sw, 0u, 0x2404)));
        const unsigned b1 = hmul2_u(pb1, e4m3_hi_bytes_alu(__byte_perm(sw, 0u, 0x3414)));
        oacc[mt][0] *= c0; oacc[mt][1] *= c1; oacc[mt][2] *= c0; oacc[mt][3] *= c1;
        mma16816(oacc[mt], e2m1_pair_alu<0>(wv), e2m1_pair_alu<1>(wv), e2m1_pair_alu<2>(wv), e2m1_pair_alu<3>(wv), b0, b1);
      }
    }
#pragma unroll
    for (int mt = 0; mt < (FP4 ? 0 : NC); ++mt) {
      const unsigned w1 = *reinterpret_cast<const unsigned*>(sV + (16 * mt + gid) * 16 + 4 * tid) & vmask;
      const unsigned w2 = *reinterpret_cast<const unsigned*>(sV + (16 * mt + gid + 8) * 16 + 4 * tid) & vmask;
      oacc[mt][0] *= c0; oacc[mt][1] *= c1; oacc[mt][2] *= c0; oacc[mt][3] *= c1;
      mma16816(oacc[mt], widen2<FMT>(w1), widen2<FMT>(w2), widen2<FMT>(w1 >> 16), widen2<FMT>(w2 >> 16), pb0, pb1);
    }
    __syncwarp();
  }
  cp_async_wait<0>();
  // row sums: add the partial sums of the 8 token lanes
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, o);
    l1 += __shfl_xor_sync(0xffffffffu, l1, o);
  }
  __syncthreads();   // every warp is done with its ring; reuse shared memory for the merge
  float* sm_m = reinterpret_cast<float*>(smem);              // [warps][8]
  float* sm_l = sm_m + kWarps * 8;                           // [warps][8]
  float* sm_acc = sm_l + kWarps * 8;                         // [warps][8][D]
  if (gid == 0) {
    sm_m[w * 8 + 2 * tid] = m0; sm_m[w * 8 + 2 * tid + 1] = m1;
    sm_l[w * 8 + 2 * tid] = l0; sm_l[w * 8 + 2 * tid + 1] = l1;
  }
#pragma unroll
  for (int mt = 0; mt < NC; ++mt) {
    float* a = sm_acc + (size_t)w * 8 * D;
    const int da = FP4 ? 16 * mt + 2 * gid : 16 * mt + gid;         // dims of MMA rows gid and gid + 8
    const int db = FP4 ? da + 1 : da + 8;
    a[(2 * tid) * D + da] = oacc[mt][0];
    a[(2 * tid + 1) * D + da] = oacc[mt][1];
    a[(2 * tid) * D + db] = oacc[mt][2];
    a[(2 * tid + 1) * D + db] = oacc[mt][3];
  }
  __syncthreads();
  // merge the 4 warps; with one split the result is final, otherwise it is this split's partial
  for (int idx = threadIdx.x; idx < gn * D; idx += blockDim.x) {
    const int i = idx / D, e = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int ww = 0; ww < kWarps; ++ww) mm = fmaxf(mm, sm_m[ww * 8 + i]);
    float ll = 0.f, a = 0.f;
#pragma unroll
    for (int ww = 0; ww < kWarps; ++ww) {
      const float mw = sm_m[ww * 8 + i];
      const float c = mw == -INFINITY ? 0.f : exp2f(mw - mm);
      ll += sm_l[ww * 8 + i] * c;
      a += sm_acc[((size_t)ww * 8 + i) * D + e] * c;
    }
    const int64_t bh = (int64_t)b * H + hk * g + g0 + i;
    if (S == 1 && fuse_reduce) {
      out[bh * D + e] = from_f32<T>(ll > 0.f ? a * vscale / ll : 0.f);
    } else {
      float* o = ws + (bh * S + s) * (2 + D);
      if (e == 0) { o[0] = mm * 0.6931471805599453f; o[1] = ll; }   // natural-log domain (shared with the reducer kernel)
      o[2 + e] = a * vscale;
    }
  }
  if (S == 1 || !fuse_reduce) return;
  // The last CTA of this (sequence, kv head, head chunk) to finish merges the S partials in split
  // order and resets the counter, so no separate reduction launch is needed.
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  int* ctr = counters + ((int64_t)blockIdx.x * gridDim.z + blockIdx.z);
  if (threadIdx.x == 0) s_last = (atomicAdd(ctr, 1) == S - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < gn * D; idx += blockDim.x) {
    const int i = idx / D, e = idx % D;
    const int64_t bh = (int64_t)b * H + hk * g + g0 + i;
    const float* pr = ws + bh * S * (2 + D);
    float mm = -INFINITY;
    for (int sp = 0; sp < S; ++sp) mm = fmaxf(mm, __ldcg(pr + sp * (2 + D)));
    float ll = 0.f, a = 0.f;
    for (int sp = 0; sp < S; ++sp) {
      const float ms = __ldcg(pr + sp * (2 + D));
      const float c = ms == -INFINITY ? 0.f : __expf(ms - mm);
      ll += __ldcg(pr + sp * (2 + D) + 1) * c;
      a += __ldcg(pr + sp * (2 + D) + 2 + e) * c;
    }
    out[bh * D + e] = from_f32<T>(ll > 0.f ? a / ll : 0.f);
  }
  if (threadIdx.x == 0) *ctr = 0;
}

template <typename T, int D, int FMT>
int launch_mma(const tsb200_kv_desc& kv, const void* q, int64_t qs, int H, float sm_scale, int64_t max_seq_len, int S, int64_t B,
               float* ws, int* counters, void* out, cudaStream_t st) {
  constexpr int REC = RecBytes<FMT, D>::value;
  constexpr int kWarps = AttnCfg<FMT>::kWarps, kStages = AttnCfg<FMT>::kStages;
  constexpr size_t pipe = (size_t)kWarps * kStages * 2 * REC;
  constexpr size_t merge = (size_t)(kWarps * 16 + kWarps * 8 * D) * sizeof(float);
  constexpr size_t smem = pipe > merge ? pipe : merge;
  static bool configured[64] = {false};   // per device: the attribute lives in the device's context
  int dev = 0;
  TSB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return TSB200_ERR_DEVICE;
  if (!configured[dev]) {
    TSB_CUDA(cudaFuncSetAttribute(decode_attn_mma_kernel<T, D, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = true;
  }
  const int g = H / kv.hkv;
  dim3 grid((unsigned)(B * kv.hkv), (unsigned)S, (unsigned)((g + 7) / 8));
  TSB_CUDA(launch_kernel(decode_attn_mma_kernel<T, D, FMT>, grid, dim3(kWarps * 32), smem, st, kv, (const T*)q, qs, H, sm_scale,
                         max_seq_len, S, ws, counters, (T*)out));
  return TSB200_OK;
}

}  // namespace
}  // namespace tsb

using namespace tsb;

// Bytes the dispatch below really uses for a problem: counters + partials of the split count it will pick
// (tsb200_paged_decode_attn_workspace_bytes is the hkv-independent upper bound of this).
static size_t attn_exact_workspace_bytes(const tsb200_kv_desc* kv, int64_t B, int H, int64_t max_seq_len) {
  const int S = choose_splits(B, kv->hkv, max_seq_len);
  return kAttnCounterBytes + (size_t)(B * H * S * (2 + kv->head_dim)) * sizeof(float);
}

static int decode_attn_dispatch(const tsb200_kv_desc* kv, const void* q, void* out, int dtype, int64_t q_batch_stride, int64_t B,
                                int H, float sm_scale, int64_t max_seq_len, void* workspace, size_t workspace_bytes,
                                size_t need_bytes, void* stream) {
  TSB_REQUIRE_DEVICE();
  bool noop;
  int st = validate_attn_args(kv, q, out, dtype, B, H, max_seq_len, workspace, workspace_bytes, noop, need_bytes);
  if (st != TSB200_OK || noop) return st;
  const int64_t qs = q_batch_stride ? q_batch_stride : (int64_t)H * kv->head_dim;
  if (qs < (int64_t)H * kv->head_dim) return TSB200_ERR_ARG;
  if (kv->format > TSB200_KV_NVFP4)    // unquantized pages: CUDA-core kernel (fp32 math)
    return tsb200_paged_decode_attn_simt(kv, q, out, dtype, q_batch_stride, B, H, sm_scale, max_seq_len, workspace, workspace_bytes, stream);
  cudaStream_t s = as_stream(stream);
  const int S = choose_splits(B, kv->hkv, max_seq_len);
  int* counters = (int*)workspace;                               // zero between calls
  float* ws = (float*)((char*)workspace + kAttnCounterBytes);
  const int D = kv->head_dim;
  const int64_t n_ctr = B * kv->hkv * ((H / kv->hkv + 7) / 8);
  // the last int of the counter block is the status word of the bounded waits, so one counter fewer is usable
  const bool fused = n_ctr < (int64_t)(kAttnCounterBytes / sizeof(int));           // else: separate reduction launch
  int* status = counters + kAttnStatusIndex;
  int r;
  if (kv->format == TSB200_KV_FP8 && D == 128 && H / kv->hkv <= 4) {
    // e4m3 pages go to the tensor cores as FP8 (decode_attn_fp8.cu)
    int* ctr = fused ? counters : nullptr;
    const int S8 = choose_splits_fp8(B, kv->hkv, max_seq_len);   // never more than choose_splits(): the workspace fits
    if (dtype == TSB200_F32) r = launch_attn_fp8<float>(*kv, q, qs, H, sm_scale, max_seq_len, S8, B, ws, ctr, out, status, s);
    else r = launch_attn_fp8<__nv_bfloat16>(*kv, q, qs, H, sm_scale, max_seq_len, S8, B, ws, ctr, out, status, s);
    if (r != TSB200_OK || fused) return r;
    return dtype == TSB200_F32 ? launch_reduce<float, 128>(ws, B * H, S8, out, s) : launch_reduce<__nv_bfloat16, 128>(ws, B * H, S8, out, s);
  }
#define TSB_GO(TT, DD, FF)                                                                                              \
  if (fused) return launch_mma<TT, DD, FF>(*kv, q, qs, H, sm_scale, max_seq_len, S, B, ws, counters, out, s);        \
  r = launch_mma<TT, DD, FF>(*kv, q, qs, H, sm_scale, max_seq_len, -S, B, ws, counters, out, s);                      \
  if (r != TSB200_OK) return r;                                                                                         \
  return launch_reduce<TT, DD>(ws, B * H, S, out, s)
  if (kv->format == TSB200_KV_NVFP4) {
    if (dtype == TSB200_F32) { if (D == 64) { TSB_GO(float, 64, TSB200_KV_NVFP4); } else { TSB_GO(float, 128, TSB200_KV_NVFP4); } }
    else { if (D == 64) { TSB_GO(__nv_bfloat16, 64, TSB200_KV_NVFP4); } else { TSB_GO(__nv_bfloat16, 128, TSB200_KV_NVFP4); } }
  }
  if (dtype == TSB200_F32) {
    if (D == 64) { if (kv->format == TSB200_KV_INT8) { TSB_GO(float, 64, TSB200_KV_INT8); } else { TSB_GO(float, 64, TSB200_KV_FP8); } }
    else { if (kv->format == TSB200_KV_INT8) { TSB_GO(float, 128, TSB200_KV_INT8); } else { TSB_GO(float, 128, TSB200_KV_FP8); } }
  } else {
    if (D == 64) { if (kv->format == TSB200_KV_INT8) { TSB_GO(__nv_bfloat16, 64, TSB200_KV_INT8); } else { TSB_GO(__nv_bfloat16, 64, TSB200_KV_FP8); } }
    else { if (kv->format == TSB200_KV_INT8) { TSB_GO(__nv_bfloat16, 128, TSB200_KV_INT8); } else { TSB_GO(__nv_bfloat16, 128, TSB200_KV_FP8); } }
  }
#undef TSB_GO
}

extern "C" int tsb200_paged_decode_attn(const tsb200_kv_desc* kv, const void* q, void* out, int dtype, int64_t q_batch_stride, int64_t B, int H,
                                        float sm_scale, int64_t max_seq_len, void* workspace, size_t workspace_bytes,
                                        void* stream) {
  return decode_attn_dispatch(kv, q, out, dtype, q_batch_stride, B, H, sm_scale, max_seq_len, workspace, workspace_bytes, 0, stream);
}


// ---------------------------------------------------------------------------------------------
// Allocation-free variant.
//
// Some callers may not allocate device memory at all: code running inside a CUDA-graph capture or
// under a framework that forbids cudaMalloc on its serving path, plugins handed a fixed memory
// budget, and host runtimes whose allocator cannot be re-entered from the calling thread.  For them
// the split partials live in the fixed array below instead of a caller-provided workspace.  Every
// GPU that loads this library carries the array (kStaticScratchBytes) until the process exits.
//
// In host code `g_attn_scratch` is only a stand-in for the symbol, not a device address; the
// address the kernels need is obtained once per device with cudaGetSymbolAddress while that device
// is current, and that pointer is what is passed to the launches.
namespace tsb {
namespace {
constexpr size_t kStaticScratchBytes = 8u << 20;     // 8 MiB: e.g. batch 32 x 32 heads x 15 splits x (2 + 128) floats
static __device__ __align__(256) unsigned char g_attn_scratch[kStaticScratchBytes];

int static_scratch_ptr(void** out) {
  static void* ptrs[64] = {nullptr};                 // one resolved address per device ordinal
  int dev = 0;
  TSB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return TSB200_ERR_DEVICE;
  if (!ptrs[dev]) {
    void* p = nullptr;
    TSB_CUDA(cudaGetSymbolAddress(&p, g_attn_scratch));   // resolves the copy owned by the current device
    if (!p) return TSB200_ERR_CUDA;
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return TSB200_OK;
}
}  // namespace
}  // namespace tsb

extern "C" size_t tsb200_paged_decode_attn_static_capacity(void) { return tsb::kStaticScratchBytes; }

extern "C" int tsb200_paged_decode_attn_static(const tsb200_kv_desc* kv, const void* q, void* out, int dtype,
                                               int64_t q_batch_stride, int64_t B, int H, float sm_scale,
                                               int64_t max_seq_len, void* stream) {
  TSB_REQUIRE_DEVICE();
  if (!kv || B < 0 || H <= 0) return TSB200_ERR_ARG;
  if (B == 0) return TSB200_OK;
  if (validate_kv(kv, true) != TSB200_OK || max_seq_len < 0) return TSB200_ERR_ARG;
  // sized by the split count this problem will really use, not by the hkv-independent bound that sizes a
  // caller's workspace: more problems fit the fixed array
  const size_t need = attn_exact_workspace_bytes(kv, B, H, max_seq_len);
  if (need > kStaticScratchBytes) return TSB200_ERR_WORKSPACE;   // problem too large for the built-in scratch
  void* scratch = nullptr;
  const int st = static_scratch_ptr(&scratch);
  if (st != TSB200_OK) return st;
  // The head of the array (split counters + status word) MUST be zero when the kernels start.  A finished call
  // leaves it zero, but a call that overlapped another one on the GPU, or was cut short, can leave a counter
  // stuck, after which the fused merge of that (sequence, head) would never fire again.  The caller cannot
  // reach the array, so every call clears the head itself, on its stream, ahead of its kernels.  The partials
  // behind the head need no clearing: each record the merge reads is written by the same call.
  TSB_CUDA(cudaMemsetAsync(scratch, 0, kAttnCounterBytes, as_stream(stream)));
  return decode_attn_dispatch(kv, q, out, dtype, q_batch_stride, B, H, sm_scale, max_seq_len, scratch, kStaticScratchBytes, need,
                              stream);
}
