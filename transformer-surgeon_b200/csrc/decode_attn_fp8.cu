// Split-K paged decode attention for FP8-e4m3 pages with the codes fed to the tensor cores AS FP8
// (mma.sync m16n8k32 e4m3 x e4m3 -> f32): no per-element widening of K or V at all.
//
// Replaces transformersurgeon/blocks/mha.py:9-103 (attention()) for the decode step, head_dim 128,
// GQA groups of up to 4 query heads per kv head (Llama-3-8B: 32/8).
//
// The other operand of each product is a higher-precision quantity (q, softmax weights), so it is
// expanded into THREE e4m3 terms hi + mid + lo (12 significant bits, about f16) that occupy separate
// MMA columns: an n-tile of 8 columns = 2 heads x (hi, mid, lo, 0); two n-tiles cover 4 heads.
//   S^T[token, col] = K_page[16 x 128] . Qexp^T          4 k-steps x 2 n-tiles per page
//   O^T[dim, col]  += V^T_pagepair[128 x 32] . Pexp^T    8 m-tiles x 2 n-tiles per PAIR of pages
// The three column sums are added in fp32 afterwards.  One CTA = (sequence, kv head, split); its 6
// warps take page pairs round-robin; each warp streams its pairs through a private 2-stage ring
// filled by cp.async.bulk (one lane, four 2 KB copies per stage) completing on an mbarrier.
// Every mbarrier wait is bounded; on expiry the warp stops consuming pages and records a status.
#include "tc_common.cuh"
#include "decode_attn_common.cuh"

namespace tsb {

template <typename T, int D> int launch_reduce(const float* ws, int64_t BH, int S, void* out, cudaStream_t st);

namespace {

using tc::mbar_arrive;
using tc::mbar_expect_tx;
using tc::mbar_init;
using tc::mbar_try_wait;
using tc::smem_u32;

// 6 warps: two CTAs (12 warps, 2 x 100 KB of rings, 2 x 32k registers) fill an SM; measured 8-11 % faster than
// 4 warps (three CTAs per SM) and 25 % faster than 8 (one CTA per SM) at batch 32-64, context 2k-4k.
#ifndef TSB_FP8_WARPS
#define TSB_FP8_WARPS 6
#endif
constexpr int kWarps = TSB_FP8_WARPS;
constexpr int kStages = 2;
constexpr int kEarlyStages = 1;            // ring stages that may be filled before the dependency wait (2 measured no faster)
constexpr int D = 128;
constexpr int REC = 16 * D;                 // bytes of one K or V record
constexpr int STAGE = 4 * REC;              // K_A, V_A, K_B, V_B
constexpr int PBUF = 2 * 4 * 16 * 4;        // softmax weights of a stage: [page][head][token] words
constexpr int WARP_SMEM = kStages * STAGE + PBUF + 64;
constexpr unsigned kWaitLimit = 1u << 22;

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void mma_e4m3(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned to_e4m3(float x) { return (unsigned)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3); }
// x -> hi | mid << 8 | lo << 16 with x ~= hi + mid + lo (each an e4m3 value); byte 3 is 0.
__device__ __forceinline__ unsigned split3(float x) {
  const unsigned hi = to_e4m3(x);
  float r = x - e4m3_byte_to_f32(hi);
  const unsigned mid = to_e4m3(r);
  r -= e4m3_byte_to_f32(mid);
  const unsigned lo = to_e4m3(r);
  return hi | (mid << 8) | (lo << 16);
}
// fp32 value rounded to 4 significant bits (what an e4m3 code holds in its normal range), with
// integer instructions: add half an ulp of the 3-bit mantissa, clear the 20 low mantissa bits.
__device__ __forceinline__ float round_4bits(float x) { return __uint_as_float((__float_as_uint(x) + 0x00080000u) & 0xfff00000u); }
// Two values at once: the codes come from the packed conversion (one instruction per term for both
// values), the residuals from round_4bits on the FMA/ALU pipes.  Below 2^-6 the code is a subnormal
// and the residual is off by < 2^-10: far below the last term's resolution.
__device__ __forceinline__ void split3x2(float x0, float x1, unsigned& w0, unsigned& w1) {
  const unsigned hi = (unsigned)__nv_cvt_float2_to_fp8x2(make_float2(x0, x1), __NV_SATFINITE, __NV_E4M3);
  const float r0 = x0 - round_4bits(x0), r1 = x1 - round_4bits(x1);
  const unsigned mid = (unsigned)__nv_cvt_float2_to_fp8x2(make_float2(r0, r1), __NV_SATFINITE, __NV_E4M3);
  const float s0 = r0 - round_4bits(r0), s1 = r1 - round_4bits(r1);
  const unsigned lo = (unsigned)__nv_cvt_float2_to_fp8x2(make_float2(s0, s1), __NV_SATFINITE, __NV_E4M3);
  w0 = (hi & 0xffu) | ((mid & 0xffu) << 8) | ((lo & 0xffu) << 16);
  w1 = ((hi >> 8) & 0xffu) | (mid & 0xff00u) | ((lo & 0xff00u) << 8);
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
decode_attn_fp8_kernel(tsb200_kv_desc kv, const T* __restrict__ q, int64_t qs, int H, float sm_scale, int64_t max_seq_len, int S,
                       float* __restrict__ ws, int* __restrict__ counters, T* __restrict__ out, int* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int gid = lane >> 2, tid = lane & 3;
  const int b = blockIdx.x / kv.hkv, hk = blockIdx.x % kv.hkv, s = blockIdx.y;
  const int g = H / kv.hkv;                                  // <= 4

  uint8_t* ring = smem + (size_t)w * WARP_SMEM;
  unsigned* pbuf = reinterpret_cast<unsigned*>(ring + kStages * STAGE);
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(ring + kStages * STAGE + PBUF);
  if (lane == 0) {
    for (int i = 0; i < kStages; ++i) mbar_init(&bars[i], 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncwarp();
  const int64_t rec_stride = (int64_t)kv.hkv * REC;
  auto page_of = [&](int pg, const uint8_t*& kr, const uint8_t*& vr) {
    int64_t page = kv.block_table[(int64_t)b * kv.bt_stride + pg];
    page = page < 0 ? 0 : (page >= kv.num_pages ? kv.num_pages - 1 : page);
    kr = kv.k_pool + page * rec_stride + (int64_t)hk * REC;
    vr = kv.v_pool + page * rec_stride + (int64_t)hk * REC;
  };

  // Before the preceding kernels are known to be complete (programmatic dependent launch): with one split the warp's
  // pairs are pages w, w + kWarps, w + 2 kWarps ... whatever the length, and pages strictly older than the one that holds the
  // newest token are not written by an append that precedes this launch - neither by one that has already counted its
  // token into seq_lens nor by one that has not.  Their copies leave now and land while those kernels finish.  (A length
  // that shrank in between only makes the copied pages unused; such stages are drained before shared memory is reused.)
  int early_pairs = 0;                                       // ring stages filled ahead of the wait
  if (S == 1) {
    int len0 = kv.seq_lens[b];                                // may be one append behind
    len0 = len0 > max_seq_len ? (int)max_seq_len : len0;
    const int old_pages = (len0 - 1) >> 4;
#pragma unroll
    for (int i = 0; i < kEarlyStages; ++i) {
      if (early_pairs == i && w + (2 * i + 1) * kWarps < old_pages) {
        early_pairs = i + 1;
        if (lane == 0) {
          uint8_t* st = ring + i * STAGE;
          mbar_expect_tx(&bars[i], 4u * REC);
          const uint8_t *kr, *vr;
          page_of(w + 2 * i * kWarps, kr, vr);
          bulk_g2s(st, kr, REC, &bars[i]);
          bulk_g2s(st + REC, vr, REC, &bars[i]);
          page_of(w + (2 * i + 1) * kWarps, kr, vr);
          bulk_g2s(st + 2 * REC, kr, REC, &bars[i]);
          bulk_g2s(st + 3 * REC, vr, REC, &bars[i]);
        }
      }
    }
  }
  pdl_wait();     // q, the page just appended and seq_lens come from the preceding kernels
  int len = kv.seq_lens[b];
  len = len < 0 ? 0 : (len > max_seq_len ? (int)max_seq_len : len);
  int pb, pe;
  split_range(len, s, S, pb, pe);

  // this warp's pages: pb + w, pb + w + kWarps, ...; consecutive two form a pair (one ring stage)
  const int n_pages = (pe - pb - w + kWarps - 1) / kWarps > 0 ? (pe - pb - w + kWarps - 1) / kWarps : 0;
  const int n_pairs = (n_pages + 1) / 2;
  auto page_ptrs = [&](int idx, const uint8_t*& kr, const uint8_t*& vr) {
    const int pg = pb + w + idx * kWarps;
    int64_t page = kv.block_table[(int64_t)b * kv.bt_stride + pg];
    page = page < 0 ? 0 : (page >= kv.num_pages ? kv.num_pages - 1 : page);
    kr = kv.k_pool + page * rec_stride + (int64_t)hk * REC;
    vr = kv.v_pool + page * rec_stride + (int64_t)hk * REC;
  };
  auto issue = [&](int pair) {
    if (pair < n_pairs && lane == 0) {
      uint8_t* st = ring + (pair % kStages) * STAGE;
      unsigned long long* bar = &bars[pair % kStages];
      const bool two = 2 * pair + 1 < n_pages;
      mbar_expect_tx(bar, two ? 4u * REC : 2u * REC);
      const uint8_t *kr, *vr;
      page_ptrs(2 * pair, kr, vr);
      bulk_g2s(st, kr, REC, bar);
      bulk_g2s(st + REC, vr, REC, bar);
      if (two) {
        page_ptrs(2 * pair + 1, kr, vr);
        bulk_g2s(st + 2 * REC, kr, REC, bar);
        bulk_g2s(st + 3 * REC, vr, REC, bar);
      }
    }
  };
  // the first copies leave before the query is expanded: their latency (block-table entry, then the copy: ~2 us) runs
  // under that work instead of after it
#pragma unroll
  for (int i = 0; i < kStages - 1; ++i)
    if (i >= early_pairs) issue(i);                          // the first pairs may already be on their way


  // ---- expanded query operand -------------------------------------------------------------------
  // column n of n-tile nt: head 2*nt + (n >> 2), term n & 3 (hi, mid, lo, zero); this lane supplies
  // column n = gid.  k-slots of QK step c (c = 0..3): lane `tid` covers dims 16*(tid + 4*(c>>1)) +
  // 8*(c&1) + [0, 8): b0 = the first four, b1 = the last four.
  // The expansion is computed once per CTA (warp h handles head h: 32 lanes x 4 dims) into shared
  // memory as words hi | mid << 8 | lo << 16, then every lane gathers the bytes of its own column.
  unsigned qf[2][4][2];
  float qamax[2];                                            // of the heads this lane tracks: 2*nt + (tid >> 1)
  {
    unsigned* qexp = reinterpret_cast<unsigned*>(smem + (size_t)kWarps * WARP_SMEM);   // [4 heads][128 dims]
    float* qam = reinterpret_cast<float*>(qexp + 4 * D);                               // [4]
    {
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (w < g) {
        const T* qp = q + (int64_t)b * qs + (int64_t)(hk * g + w) * D + lane * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = to_f32<T>(qp[i]);
      }
      const float a = warp_max(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
      const float qsc = a > 0.f ? 256.0f / a : 0.f;
      uint4 e;
      e.x = split3(v[0] * qsc); e.y = split3(v[1] * qsc); e.z = split3(v[2] * qsc); e.w = split3(v[3] * qsc);
      if (w < 4) {                                           // four head slots, whatever the number of warps
        *reinterpret_cast<uint4*>(&qexp[w * D + lane * 4]) = e;
        if (lane == 0) qam[w] = a;
      }
    }
    __syncthreads();
    const unsigned part = gid & 3;
    const unsigned sel = part | ((4u + part) << 4);          // byte `part` of two words -> bytes 0, 1
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int hq = 2 * nt + (gid >> 2);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int base = 16 * (tid + 4 * (c >> 1)) + 8 * (c & 1);
        const uint4 w0 = *reinterpret_cast<const uint4*>(&qexp[hq * D + base]);
        const uint4 w1 = *reinterpret_cast<const uint4*>(&qexp[hq * D + base + 4]);
        qf[nt][c][0] = __byte_perm(__byte_perm(w0.x, w0.y, sel), __byte_perm(w0.z, w0.w, sel), 0x5410);
        qf[nt][c][1] = __byte_perm(__byte_perm(w1.x, w1.y, sel), __byte_perm(w1.z, w1.w, sel), 0x5410);
      }
      qamax[nt] = qam[2 * nt + (tid >> 1)];
    }
  }
  const float kscale = kv.k_scale[b * kv.hkv + hk], vscale = kv.v_scale[b * kv.hkv + hk];
  float scf[2];                                              // raw MMA sum -> log2-domain score, per tracked head
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) scf[nt] = qamax[nt] * (1.0f / 256.0f) * kscale * sm_scale * 1.4426950408889634f;

  float oacc[8][2][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) oacc[i][j][0] = oacc[i][j][1] = oacc[i][j][2] = oacc[i][j][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  bool ok = true;
  for (int pair = 0; pair < n_pairs && ok; ++pair) {
    if (pair + kStages - 1 >= early_pairs) issue(pair + kStages - 1);
    {
      unsigned long long* bar = &bars[pair % kStages];
      const unsigned parity = (pair / kStages) & 1;
      unsigned spins = 0;
      while (!mbar_try_wait(bar, parity)) {
        if (++spins > kWaitLimit) { ok = false; break; }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
    }
    const uint8_t* st = ring + (pair % kStages) * STAGE;
    const bool two = 2 * pair + 1 < n_pages;
    const int pgA = pb + w + (2 * pair) * kWarps;
    const int ntA = min(16, len - pgA * 16);
    const int ntB = two ? min(16, len - (pgA + kWarps) * 16) : 0;

    // ---- S^T = K . Qexp^T for the pages of the pair ---------------------------------------------
    float sv[2][2][2];                                       // [page][n-tile][token row gid / gid+8]
#pragma unroll
    for (int X = 0; X < 2; ++X) {
      float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      if (X == 0 || two) {
        const uint8_t* sK = st + X * 2 * REC;
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          const uint4 ka = *reinterpret_cast<const uint4*>(sK + gid * D + 16 * (tid + 4 * h2));
          const uint4 kb = *reinterpret_cast<const uint4*>(sK + (gid + 8) * D + 16 * (tid + 4 * h2));
#pragma unroll
          for (int nt = 0; nt < 2; ++nt) {
            mma_e4m3(sacc[nt], ka.x, kb.x, ka.y, kb.y, qf[nt][2 * h2][0], qf[nt][2 * h2][1]);
            mma_e4m3(sacc[nt], ka.z, kb.z, ka.w, kb.w, qf[nt][2 * h2 + 1][0], qf[nt][2 * h2 + 1][1]);
          }
        }
      }
      const int ntX = X == 0 ? ntA : ntB;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        // columns 2*tid, 2*tid+1 are two terms of head 2*nt + (tid>>1); the partner lane (tid ^ 1) has the rest
        float v0 = sacc[nt][0] + sacc[nt][1], v1 = sacc[nt][2] + sacc[nt][3];
        v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
        v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
        sv[X][nt][0] = gid < ntX ? v0 * scf[nt] : -INFINITY;
        sv[X][nt][1] = gid + 8 < ntX ? v1 * scf[nt] : -INFINITY;
      }
    }
    // ---- online softmax per tracked head (over the 32 tokens of the pair) -------------------------
    float corr[2];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      float mx = fmaxf(fmaxf(sv[0][nt][0], sv[0][nt][1]), fmaxf(sv[1][nt][0], sv[1][nt][1]));
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float mn = fmaxf(m_run[nt], mx);                 // finite: token 0 of page A is always valid
      corr[nt] = exp2f(m_run[nt] - mn);
      m_run[nt] = mn;
    }
    // lanes with even tid own page A's weights, odd tid page B's (the partner computed the same scores)
    const int X = tid & 1;
    float psum[2];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const float p0 = exp2f(sv[X][nt][0] - m_run[nt]), p1 = exp2f(sv[X][nt][1] - m_run[nt]);
      psum[nt] = p0 + p1;
      const int head = 2 * nt + (tid >> 1);
      unsigned w0, w1;
      split3x2(p0 * 256.0f, p1 * 256.0f, w0, w1);
      pbuf[(X * 4 + head) * 16 + gid] = w0;
      pbuf[(X * 4 + head) * 16 + gid + 8] = w1;
      l_run[nt] = l_run[nt] * corr[nt] + psum[nt];
    }
    __syncwarp();
    // ---- Pexp^T operand: column gid = (head 2*nt + (gid>>2), term gid&3); k-slots = 4 tokens of A, 4 of B
    unsigned pf[2][2];
    {
      const unsigned part = gid & 3;
      const unsigned sel = part | ((4u + part) << 4);        // byte `part` of two words -> bytes 0, 1
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int head = 2 * nt + (gid >> 2);
#pragma unroll
        for (int Y = 0; Y < 2; ++Y) {
          const uint4 wd = *reinterpret_cast<const uint4*>(&pbuf[(Y * 4 + head) * 16 + 4 * tid]);
          const unsigned lo = __byte_perm(wd.x, wd.y, sel), hi = __byte_perm(wd.z, wd.w, sel);
          pf[nt][Y] = __byte_perm(lo, hi, 0x5410);
        }
      }
    }
    // ---- O^T += V^T . Pexp^T ---------------------------------------------------------------------
    const bool rescale = __any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f);
    const uint8_t* sVA = st + REC;
    const uint8_t* sVB = st + 3 * REC;
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
      const unsigned a0 = *reinterpret_cast<const unsigned*>(sVA + (16 * mt + gid) * 16 + 4 * tid);
      const unsigned a1 = *reinterpret_cast<const unsigned*>(sVA + (16 * mt + gid + 8) * 16 + 4 * tid);
      unsigned a2 = 0u, a3 = 0u;
      if (two) {
        a2 = *reinterpret_cast<const unsigned*>(sVB + (16 * mt + gid) * 16 + 4 * tid);
        a3 = *reinterpret_cast<const unsigned*>(sVB + (16 * mt + gid + 8) * 16 + 4 * tid);
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        if (rescale) {
          oacc[mt][nt][0] *= corr[nt]; oacc[mt][nt][1] *= corr[nt]; oacc[mt][nt][2] *= corr[nt]; oacc[mt][nt][3] *= corr[nt];
        }
        mma_e4m3(oacc[mt][nt], a0, a1, a2, a3, pf[nt][0], pf[nt][1]);
      }
    }
    __syncwarp();     // all lanes are done with this stage and with pbuf before they are refilled
  }
  for (int i = n_pairs; i < early_pairs && ok; ++i) {        // copies issued for a length that no longer holds: let them land
    unsigned spins = 0;
    while (!mbar_try_wait(&bars[i], 0)) {
      if (++spins > kWaitLimit) { ok = false; break; }
    }
  }
  if (!ok) {
    // error path only: a wait ran out.  Give the copies still in flight a bounded time to land before
    // shared memory is reused, and record the event.
    if (lane == 0 && status) atomicMax(status, 8);
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }

  // ---- per-warp results -> shared memory, then the same cross-warp / cross-split merge as the f16 kernel
  // row sums: add the partner lane (other page) and the 8 token lanes
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    l_run[nt] += __shfl_xor_sync(0xffffffffu, l_run[nt], 1);
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) l_run[nt] += __shfl_xor_sync(0xffffffffu, l_run[nt], o);
  }
  __syncthreads();
  float* sm_m = reinterpret_cast<float*>(smem);              // [warps][8]
  float* sm_l = sm_m + kWarps * 8;
  float* sm_acc = sm_l + kWarps * 8;                         // [warps][8][D]
  if (gid == 0 && (tid & 1) == 0) {
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      sm_m[w * 8 + 2 * nt + (tid >> 1)] = m_run[nt];
      sm_l[w * 8 + 2 * nt + (tid >> 1)] = l_run[nt];
    }
  }
#pragma unroll
  for (int mt = 0; mt < 8; ++mt)
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      float v0 = oacc[mt][nt][0] + oacc[mt][nt][1], v1 = oacc[mt][nt][2] + oacc[mt][nt][3];
      v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
      v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
      if ((tid & 1) == 0) {
        float* a = sm_acc + ((size_t)w * 8 + 2 * nt + (tid >> 1)) * D;
        a[16 * mt + gid] = v0;
        a[16 * mt + gid + 8] = v1;
      }
    }
  __syncthreads();
  const float oscale = vscale * (1.0f / 256.0f);
  const bool fuse_reduce = counters != nullptr;
  for (int idx = threadIdx.x; idx < g * D; idx += blockDim.x) {
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
    const int64_t bh = (int64_t)b * H + hk * g + i;
    if (S == 1 && fuse_reduce) {
      out[bh * D + e] = from_f32<T>(ll > 0.f ? a * oscale / ll : 0.f);
    } else {
      float* o = ws + (bh * S + s) * (2 + D);
      if (e == 0) { o[0] = mm * 0.6931471805599453f; o[1] = ll; }
      o[2 + e] = a * oscale;
    }
  }
  if (S == 1 || !fuse_reduce) return;
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  int* ctr = counters + blockIdx.x;
  if (threadIdx.x == 0) s_last = (atomicAdd(ctr, 1) == S - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < g * D; idx += blockDim.x) {
    const int i = idx / D, e = idx % D;
    const int64_t bh = (int64_t)b * H + hk * g + i;
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

}  // namespace

// FP8 pages, head_dim 128, group <= 4: returns TSB200_ERR_UNSUPPORTED otherwise (the caller then
// uses the f16 tensor-core kernel).  `counters` may be null: partials only, a reducer launch follows.
template <typename T>
int launch_attn_fp8(const tsb200_kv_desc& kv, const void* q, int64_t qs, int H, float sm_scale, int64_t max_seq_len, int S,
                    int64_t B, float* ws, int* counters, void* out, int* status, cudaStream_t st) {
  constexpr size_t pipe = (size_t)kWarps * WARP_SMEM + 4 * D * 4 + 64;   // rings + expanded q
  constexpr size_t merge = (size_t)(kWarps * 16 + kWarps * 8 * D) * sizeof(float);
  constexpr size_t smem = pipe > merge ? pipe : merge;
  static bool configured[64] = {false};
  int dev = 0;
  TSB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return TSB200_ERR_DEVICE;
  if (!configured[dev]) {
    TSB_CUDA(cudaFuncSetAttribute(decode_attn_fp8_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = true;
  }
  dim3 grid((unsigned)(B * kv.hkv), (unsigned)S, 1);
  TSB_CUDA(launch_kernel(decode_attn_fp8_kernel<T>, grid, dim3(kWarps * 32), smem, st, kv, (const T*)q, qs, H, sm_scale, max_seq_len,
                         S, ws, counters, (T*)out, status));
  return TSB200_OK;
}
template int launch_attn_fp8<float>(const tsb200_kv_desc&, const void*, int64_t, int, float, int64_t, int, int64_t, float*, int*,
                                    void*, int*, cudaStream_t);
template int launch_attn_fp8<__nv_bfloat16>(const tsb200_kv_desc&, const void*, int64_t, int, float, int64_t, int, int64_t, float*,
                                            int*, void*, int*, cudaStream_t);

}  // namespace tsb
