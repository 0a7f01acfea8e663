// Causal attention of a PROMPT CHUNK on tcgen05: T query tokens per sequence over the L >= T tokens of the
// cache (query i sits at position L - T + i), reading the DEQUANTIZED cache - what every attention read of a
// quantized cache sees.  Replaces transformersurgeon/blocks/mha.py:9-103 (attention(): GQA, softmax(q k^T / sqrt d) v)
// for T > 1, i.e. what the reference hands to torch's scaled-dot-product attention during prefill.
//
// Inputs are produced by tsb200_kv_gather_heads (below): K as [B, hkv, L, d] and V TRANSPOSED as [B, hkv, d, Lp]
// (tokens contiguous, zero beyond L), both bf16, so that every MMA operand tile is K-major and one TMA box:
//     S[128 q, 128 keys]  = Q[128, d] . K_tile[128, d]^T          (tcgen05.mma kind::f16, fp32 in TMEM)
//     O[128 q, d]        += P[128, 128] . Vt_tile[d, 128]^T
// One CTA = one (sequence, query head, 128-query tile); tiles are issued longest first.  Warp roles (6 warps):
//   warp 0      TMA: the Q tile once, then K / Vt tiles into a 2-stage ring
//   warp 1      TMEM allocation (S double-buffered, O); one lane issues the MMAs: S(j+1) is issued before it
//               waits for P(j), so the score MMAs of the next tile overlap the softmax of this one
//   warps 2..5  softmax: one thread = one query row (its TMEM lane): tcgen05.ld the 128 scores, mask the
//               diagonal tile, running maximum with LAZY rescaling (O and the row sum are rescaled only when the
//               maximum grew by more than 2^8; the final division uses the same reference maximum, so the result is
//               exact), exp2, row sum in fp32, P rounded to bf16 into shared memory in the swizzled K-major layout
//               the MMA descriptor expects; at the end O / l, rounded, 16-byte stores
// Every mbarrier wait is bounded; on expiry the CTA records a code in the status word, frees its TMEM and returns.
#include "tc_common.cuh"
#include "decode_attn_common.cuh"

namespace tsb {
using namespace tc;
namespace {

constexpr int kPfThreads = 192;
constexpr int BQ = 128, BKEY = 128;

__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32f(unsigned taddr, const unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait_pf() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

struct PfParams {
  int64_t B, T, L;
  int H, hkv;
  float scale_log2;          // sm_scale * log2(e)
  __nv_bfloat16* out;        // [B, T, H, D]
  int* status;
};

template <int D> struct PfLayout {
  static constexpr int KB = D / 64;                    // 64-column blocks of the head dimension
  static constexpr int kQ = KB * BQ * 128;             // Q tile
  static constexpr int kK = KB * BKEY * 128;           // K tile: KB blocks of [128 keys x 128 B]
  static constexpr int kV = 2 * D * 128;               // Vt tile: 2 blocks (64 keys each) of [D rows x 128 B]
  static constexpr int kP = 2 * BQ * 128;              // P tile: 2 blocks (64 keys each) of [128 rows x 128 B]
  static constexpr int kStage = kK + kV;
  static constexpr int kBytes = kQ + 2 * kStage + kP + 1024 /*barriers*/ + 1024 /*alignment*/;
  static constexpr unsigned kSCol = 0;                 // S buffers at columns 0 and 128
  static constexpr unsigned kOCol = 256;               // O accumulator: D columns
};

template <int D>
__global__ void __launch_bounds__(kPfThreads, 1)
prefill_attn_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_vt, PfParams p) {
  using Lt = PfLayout<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + Lt::kQ;                          // 2 stages of {K, Vt}
  uint8_t* sP = sKV + 2 * Lt::kStage;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(sP + Lt::kP);
  unsigned long long* q_full = bars;                   // [1]
  unsigned long long* kv_full = bars + 1;              // [2] K and Vt tile landed
  unsigned long long* kv_empty = bars + 3;             // [2] the tile's second MMA group (P.V) is complete
  unsigned long long* s_full = bars + 5;               // [2] scores of a tile are in TMEM buffer (tile & 1)
  unsigned long long* p_full = bars + 7;               // [1] the four softmax warps wrote P (and are done with S)
  unsigned long long* o_done = bars + 8;               // [1] P.V of a tile is complete: P and O may be touched
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;            // longest tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.hkv);
  const int64_t off = p.L - p.T;                                   // position of query 0
  const int64_t q0 = (int64_t)qt * BQ;
  const int64_t max_pos = off + min(p.T - 1, q0 + BQ - 1);
  const int n_tiles = (int)(max_pos / BKEY) + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); mbar_init(&s_full[i], 1); }
    mbar_init(p_full, 4);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, (unsigned)Lt::kQ);
      for (int kb = 0; kb < Lt::KB; ++kb)
        tma_load_3d(sQ + kb * BQ * 128, &map_q, kb * 64, h, (int)(b * p.T + q0), q_full);
      const int64_t krow0 = ((int64_t)b * p.hkv + hk) * p.L;
      const int64_t vrow0 = ((int64_t)b * p.hkv + hk) * D;
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        if (j >= 2 && !mbar_wait(&kv_empty[s], ((j >> 1) - 1) & 1, abort_flag, 1)) break;
        uint8_t* st = sKV + s * Lt::kStage;
        mbar_expect_tx(&kv_full[s], (unsigned)Lt::kStage);
        for (int kb = 0; kb < Lt::KB; ++kb)
          tma_load_2d(st + kb * BKEY * 128, &map_k, kb * 64, (int)(krow0 + (int64_t)j * BKEY), &kv_full[s]);
        for (int kb = 0; kb < 2; ++kb)
          tma_load_2d(st + Lt::kK + kb * D * 128, &map_vt, j * BKEY + kb * 64, (int)vrow0, &kv_full[s]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr unsigned idesc_s = idesc_bf16(BKEY);
      constexpr unsigned idesc_o = idesc_bf16(D);
      bool ok = mbar_wait(q_full, 0, abort_flag, 2);
      auto issue_s = [&](int j) {                      // scores of tile j into S buffer j & 1
        const int s = j & 1;
        if (!mbar_wait(&kv_full[s], (j >> 1) & 1, abort_flag, 3)) return false;
        tc_fence_after();
        const unsigned d_tmem = tmem_base + Lt::kSCol + (unsigned)s * 128;
        const uint8_t* st = sKV + s * Lt::kStage;
#pragma unroll
        for (int kb = 0; kb < Lt::KB; ++kb) {
          const unsigned long long ad = smem_desc_sw128(smem_u32(sQ + kb * BQ * 128));
          const unsigned long long bd = smem_desc_sw128(smem_u32(st + kb * BKEY * 128));
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(d_tmem, ad + 2 * k, bd + 2 * k, idesc_s, (kb | k) ? 1u : 0u);
        }
        umma_commit(&s_full[s]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        // S buffer (j + 1) & 1 was read by the softmax of tile j - 1, which p_full(j - 1) reported
        if (j + 1 < n_tiles) ok = issue_s(j + 1);
        if (!ok) break;
        ok = mbar_wait(p_full, j & 1, abort_flag, 4);
        if (!ok) break;
        tc_fence_after();
        const int s = j & 1;
        const uint8_t* st = sKV + s * Lt::kStage + Lt::kK;
        const unsigned o_tmem = tmem_base + Lt::kOCol;
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          const unsigned long long ad = smem_desc_sw128(smem_u32(sP + kb * BQ * 128));
          const unsigned long long bd = smem_desc_sw128(smem_u32(st + kb * D * 128));
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(o_tmem, ad + 2 * k, bd + 2 * k, idesc_o, (j | kb | k) ? 1u : 0u);
        }
        umma_commit(&kv_empty[s]);
        umma_commit(o_done);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int quarter = warp & 3;                      // TMEM lane quarter this warp may access
    const int row = quarter * 32 + lane;               // query row of the tile
    const unsigned lane_addr = tmem_base + ((unsigned)(quarter * 32) << 16);
    const int64_t qpos = off + q0 + row;               // position of this row's query
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j & 1;
      ok = mbar_wait(&s_full[s], (j >> 1) & 1, abort_flag, 5);
      if (!ok) break;
      tc_fence_after();
      float sc[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        unsigned r[32];
        tmem_ld32(lane_addr + Lt::kSCol + (unsigned)s * 128 + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) sc[c * 32 + i] = __uint_as_float(r[i]) * p.scale_log2;
      }
      const int64_t key0 = (int64_t)j * BKEY;
      if (key0 + BKEY - 1 > off + q0) {                // a tile that reaches past the tile's first query: mask
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (key0 + i > qpos) sc[i] = -INFINITY;
      }
      float m_tile = sc[0];
#pragma unroll
      for (int i = 1; i < 128; ++i) m_tile = fmaxf(m_tile, sc[i]);
      // lazy rescaling: keep the reference maximum until the true maximum has outgrown it by 2^8
      float alpha = 1.0f;
      const bool grow = m_tile > m_ref + 8.0f || m_ref == -INFINITY;
      if (grow && m_tile > -INFINITY) {
        alpha = m_ref == -INFINITY ? 0.f : exp2f(m_ref - m_tile);
        m_ref = m_tile;
        l_sum *= alpha;
      }
      const float mr = m_ref == -INFINITY ? 0.f : m_ref;
      float psum = 0.f;
      unsigned pk[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        const float p0 = exp2f(sc[2 * i] - mr), p1 = exp2f(sc[2 * i + 1] - mr);
        psum += p0 + p1;
        __nv_bfloat162 q2 = __floats2bfloat162_rn(p0, p1);
        pk[i] = *reinterpret_cast<unsigned*>(&q2);
      }
      l_sum += psum;
      // P(j - 1) . V must be complete before P is overwritten and before O is rescaled
      if (j > 0) {
        ok = mbar_wait(o_done, (j - 1) & 1, abort_flag, 6);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            unsigned r[32];
            tmem_ld32(lane_addr + Lt::kOCol + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st32f(lane_addr + Lt::kOCol + c * 32, r);
          }
          tmem_st_wait_pf();
        }
      }
#pragma unroll
      for (int kb = 0; kb < 2; ++kb)
#pragma unroll
        for (int c = 0; c < 8; ++c)
          store_chunk(sP + kb * BQ * 128, row, c, make_uint4(pk[kb * 32 + c * 4], pk[kb * 32 + c * 4 + 1], pk[kb * 32 + c * 4 + 2], pk[kb * 32 + c * 4 + 3]));
      fence_async_proxy();                             // generic-proxy writes -> visible to the MMA (async proxy)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- epilogue: O / l
    if (ok && n_tiles > 0) ok = mbar_wait(o_done, (n_tiles - 1) & 1, abort_flag, 7);
    if (ok) {
      tc_fence_after();
      const float inv = l_sum > 0.f ? 1.0f / l_sum : 0.f;
      const int64_t tok = q0 + row;
      __nv_bfloat16* o = p.out + (((int64_t)b * p.T + tok) * p.H + h) * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        unsigned r[32];
        tmem_ld32(lane_addr + Lt::kOCol + c * 32, r);
        tmem_ld_wait();
        if (tok < p.T) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            __nv_bfloat162 q2;
            q2 = __floats2bfloat162_rn(__uint_as_float(r[8 * i]) * inv, __uint_as_float(r[8 * i + 1]) * inv); v.x = *reinterpret_cast<unsigned*>(&q2);
            q2 = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv); v.y = *reinterpret_cast<unsigned*>(&q2);
            q2 = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv); v.z = *reinterpret_cast<unsigned*>(&q2);
            q2 = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv); v.w = *reinterpret_cast<unsigned*>(&q2);
            *reinterpret_cast<uint4*>(o + c * 32 + i * 8) = v;
          }
        }
      }
    }
  }
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);   // error path only: let copies in flight land
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicMax(p.status, *abort_flag);
}

// ---- head-major gather: K [B, hkv, L, D], V transposed [B, hkv, D, Lp] (zeros beyond seq_lens[b] and in [L, Lp))
template <int D>
__global__ void kv_gather_heads_kernel(tsb200_kv_desc kv, __nv_bfloat16* __restrict__ k_out, __nv_bfloat16* __restrict__ vt_out,
                                       int64_t L, int64_t Lp) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t b = blockIdx.z, hk = blockIdx.y, pg = blockIdx.x;          // one CTA per (sequence, kv head, page)
  const int len = min((int64_t)kv.seq_lens[b], L);
  const int rec_bytes = kv.format == TSB200_KV_INT8 ? 16 * D + 64
                        : kv.format == TSB200_KV_FP8 ? 16 * D
                        : kv.format == TSB200_KV_NVFP4 ? 9 * D
                        : kv.format == TSB200_KV_F32 ? 64 * D : 32 * D;
  const int64_t t0 = pg * 16;
  const bool any = t0 < len;
  int64_t page = 0;
  if (any) {
    page = kv.block_table[b * kv.bt_stride + pg];
    page = page < 0 ? 0 : (page >= kv.num_pages ? kv.num_pages - 1 : page);
  }
  const uint8_t* kr = kv.k_pool + (page * kv.hkv + hk) * (int64_t)rec_bytes;
  const uint8_t* vr = kv.v_pool + (page * kv.hkv + hk) * (int64_t)rec_bytes;
  const float ks = kv.format == TSB200_KV_FP8 ? kv.k_scale[b * kv.hkv + hk] : 1.0f;
  const float vs = kv.format == TSB200_KV_FP8 ? kv.v_scale[b * kv.hkv + hk] : 1.0f;
  __nv_bfloat16* ko = k_out + ((b * kv.hkv + hk) * L + t0) * D;
  __nv_bfloat16* vo = vt_out + (b * kv.hkv + hk) * (int64_t)D * Lp + t0;
  for (int idx = threadIdx.x; idx < 16 * D; idx += blockDim.x) {
    {   // K: token-major output, element fastest
      const int t = idx / D, e = idx % D;
      if (t0 + t < L) ko[(int64_t)t * D + e] = __float2bfloat16_rn((any && t0 + t < len) ? k_elem<D>(kr, kv.format, t, e) * ks : 0.f);
    }
    {   // V: element-major output, token fastest (16 consecutive tokens = 32 bytes)
      const int e = idx / 16, t = idx % 16;
      if (t0 + t < Lp) vo[(int64_t)e * Lp + t] = __float2bfloat16_rn((any && t0 + t < len) ? v_elem<D>(vr, kv.format, t, e) * vs : 0.f);
    }
  }
}

template <int D>
int launch_prefill(const void* q, int64_t q_token_stride, const void* k, const void* vt, void* out, int64_t B, int64_t T, int64_t L,
                   int64_t Lp, int H, int hkv, float sm_scale, int* status, cudaStream_t s) {
  using Lt = PfLayout<D>;
  static bool configured[64] = {false};
  int dev = 0;
  TSB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return TSB200_ERR_DEVICE;
  if (!configured[dev]) {
    TSB_CUDA(cudaFuncSetAttribute(prefill_attn_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Lt::kBytes));
    configured[dev] = true;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return TSB200_ERR_CUDA;
  CUtensorMap mq, mk, mv;
  {   // q [B*T tokens][H heads][D]: box = 64 columns of one head for 128 tokens
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)(B * T)};
    cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)q_token_stride * 2};
    cuuint32_t box[3] = {64, 1, BQ};
    cuuint32_t estr[3] = {1, 1, 1};
    if (fn(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return TSB200_ERR_CUDA;
  }
  if (!make_map(&mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, k, (uint64_t)D, (uint64_t)(B * hkv * L), (uint64_t)D * 2, 64, BKEY, CU_TENSOR_MAP_SWIZZLE_128B))
    return TSB200_ERR_CUDA;
  if (!make_map(&mv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, vt, (uint64_t)Lp, (uint64_t)(B * hkv * D), (uint64_t)Lp * 2, 64, D, CU_TENSOR_MAP_SWIZZLE_128B))
    return TSB200_ERR_CUDA;
  PfParams p;
  p.B = B; p.T = T; p.L = L; p.H = H; p.hkv = hkv;
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  p.out = (__nv_bfloat16*)out;
  p.status = status;
  dim3 grid((unsigned)((T + BQ - 1) / BQ), (unsigned)H, (unsigned)B);
  TSB_CUDA(launch_kernel(prefill_attn_kernel<D>, grid, dim3(kPfThreads), (size_t)Lt::kBytes, s, mq, mk, mv, p));
  return TSB200_OK;
}

}  // namespace
}  // namespace tsb

using namespace tsb;

extern "C" int tsb200_kv_gather_heads(const tsb200_kv_desc* kv, void* k_out, void* vt_out, int64_t B, int64_t L, int64_t Lp,
                                      void* stream) {
  TSB_REQUIRE_DEVICE();
  const int st = validate_kv(kv, true);
  if (st != TSB200_OK) return st;
  if (B < 0 || L < 0 || Lp < L || (Lp & 7)) return TSB200_ERR_ARG;
  if (B == 0 || L == 0) return TSB200_OK;
  if (!k_out || !vt_out || !aligned(k_out, 16) || !aligned(vt_out, 16)) return TSB200_ERR_ARG;
  if (B > 65535 || kv->hkv > 65535 || L > kv->bt_stride * 16) return TSB200_ERR_ARG;
  const dim3 grid((unsigned)((Lp + 15) / 16), (unsigned)kv->hkv, (unsigned)B);
  cudaStream_t s = as_stream(stream);
  if (kv->head_dim == 64) {
    TSB_CUDA(launch_kernel(kv_gather_heads_kernel<64>, grid, dim3(256), 0, s, *kv, (__nv_bfloat16*)k_out, (__nv_bfloat16*)vt_out, L, Lp));
  } else {
    TSB_CUDA(launch_kernel(kv_gather_heads_kernel<128>, grid, dim3(256), 0, s, *kv, (__nv_bfloat16*)k_out, (__nv_bfloat16*)vt_out, L, Lp));
  }
  return TSB200_OK;
}

extern "C" int tsb200_prefill_attn(const void* q, int64_t q_token_stride, const void* k, const void* vt, void* out, int64_t B,
                                   int64_t T, int64_t L, int64_t Lp, int H, int hkv, int head_dim, float sm_scale, int32_t* status,
                                   void* stream) {
  TSB_REQUIRE_DEVICE();
  if (B < 0 || T < 0 || L < T || Lp < L || (Lp & 7) || H <= 0 || hkv <= 0 || H % hkv) return TSB200_ERR_ARG;
  if (head_dim != 64 && head_dim != 128) return TSB200_ERR_UNSUPPORTED;
  if (B == 0 || T == 0) return TSB200_OK;
  if (!q || !k || !vt || !out || !aligned(q, 16) || !aligned(k, 16) || !aligned(vt, 16) || !aligned(out, 16)) return TSB200_ERR_ARG;
  const int64_t qs = q_token_stride ? q_token_stride : (int64_t)H * head_dim;
  if (qs < (int64_t)H * head_dim || (qs & 7)) return TSB200_ERR_ARG;
  if (B > 65535 || H > 65535 || B * T > 0x7fffffffLL || B * hkv * L > 0x7fffffffLL) return TSB200_ERR_UNSUPPORTED;
  cudaStream_t s = as_stream(stream);
  return head_dim == 64 ? launch_prefill<64>(q, qs, k, vt, out, B, T, L, Lp, H, hkv, sm_scale, status, s)
                        : launch_prefill<128>(q, qs, k, vt, out, B, T, L, Lp, H, hkv, sm_scale, status, s);
}
