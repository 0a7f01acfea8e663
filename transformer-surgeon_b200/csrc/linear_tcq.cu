// Persistent tcgen05 kernel for LinearCompressed with QUANTIZED factors (int8 / int4 / int2):
//   Y[M, N] = (X[M, K] . Wq[N, K]^T) * scale[N] + bias[N]        (bf16 activations)
// restating transformersurgeon/blocks/linear_compressed.py:96-100 on packed codes.
//
// Decode-time GEMMs stream a few MB of packed weights per call, so the kernel is built around
// keeping many weight bytes in flight per SM and paying the set-up cost once per SM:
//   * grid = min(#work items, #SMs); a work item = (128-row weight tile, token tile, K split);
//     each CTA walks its items round-robin while one producer lane keeps issuing TMA loads
//     across item boundaries into a ring of stages {raw codes of several k-blocks, activation tiles};
//   * 8 dequant warps turn raw codes into bf16 (exact integers) inside a small ring of
//     128-byte-swizzled A tiles; one lane issues tcgen05.mma (weights = A operand, M = 128;
//     tokens = B operand, N = token tile) accumulating in TMEM;
//   * the same 8 warps run the epilogue from TMEM (one lane = one weight row): scale, bias, store;
//   * split-K: every item stores its fp32 partial tile in a private slice of the workspace (plain
//     stores, no zero-fill needed); the last CTA to finish a tile (a per-tile counter, reset by
//     that CTA) sums the slices in split order - a deterministic result - and writes the
//     output, so no memset and no second kernel are needed.
// Every mbarrier wait is bounded (see tc_common.cuh); on expiry the CTA records a code in the
// status word, drains, frees its TMEM and returns.
#include "tc_common.cuh"

namespace tsb {
using namespace tc;
namespace {

constexpr int NA = 3;                  // A-tile ring depth
constexpr int kDqWarps = 8;
constexpr int kThreadsQ = 64 + kDqWarps * 32;
constexpr int kSmemBudget = 200 * 1024;

// A ring stage holds KBS consecutive k-blocks: one weight box of 128 rows x (KBS*64 codes) - rows of
// up to 128 bytes, so every row is one full-width DRAM request - and KBS activation tiles.
template <int TN, int BITS> struct QLayout {
  static constexpr int kKbsFull = 1024 / BITS / BK;        // k-blocks in a 128-byte row of codes
  static constexpr int KBS = TN <= 32 ? kKbsFull : (kKbsFull < 2 ? kKbsFull : 2);
  static constexpr int kRawRow = BK * BITS / 8;            // bytes of one weight row per k-block
  static constexpr int kRawStageRow = KBS * kRawRow;       // bytes of one weight row per stage
  static constexpr int kRaw = BM * kRawStageRow;
  static constexpr int kXTile = TN * 128;
  static constexpr int kX = KBS * kXTile;
  static constexpr int kStage = kX + kRaw;                 // multiple of 1024
  static constexpr int kATile = BM * 128;
  static constexpr int kNRraw = (kSmemBudget - NA * kATile) / kStage;
  static constexpr int NR = kNRraw > 16 ? 16 : kNRraw;
  static constexpr int kBarBytes = 1024;
  static constexpr int kBytes = NA * kATile + NR * kStage + kBarBytes + 1024;
};

// Address of 16-byte chunk `chunk` of weight row `row` inside a raw stage whose rows are RB bytes and
// which the copy engine wrote with the RB-byte swizzle (chunk index XOR a function of the row), so
// that threads reading the same chunk of consecutive rows hit different banks.
template <int RB>
__device__ __forceinline__ const uint8_t* raw_chunk(const uint8_t* raw, int row, int chunk) {
  const int x = RB == 128 ? (row & 7) : (RB == 64 ? ((row >> 1) & 3) : ((row >> 2) & 1));
  return raw + row * RB + ((chunk ^ x) << 4);
}

// One dequant thread converts half a weight row of k-block `sub` of the stage: 32 codes -> 4 chunks of
// 8 bf16 written into the 128-byte-swizzled A tile.
template <int BITS, int RB>
__device__ __forceinline__ void dequant_half_row(const uint8_t* __restrict__ raw, uint8_t* a_tile, int r, int sub, int half) {
  if (BITS == 4) {
    const uint4 q = *reinterpret_cast<const uint4*>(raw_chunk<RB>(raw, r, sub * 2 + half));
    const unsigned w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const unsigned t = w[c] ^ 0x88888888u;
      uint4 o;
      o.x = bf16x2_sub(((t)&0x000f000fu) | 0x43004300u, 0x43084308u);
      o.y = bf16x2_sub(((t >> 4) & 0x000f000fu) | 0x43004300u, 0x43084308u);
      o.z = bf16x2_sub(((t >> 8) & 0x000f000fu) | 0x43004300u, 0x43084308u);
      o.w = bf16x2_sub(((t >> 12) & 0x000f000fu) | 0x43004300u, 0x43084308u);
      store_chunk(a_tile, r, 4 * half + c, o);
    }
  } else if (BITS == 2) {
    const uint2 q = *reinterpret_cast<const uint2*>(raw_chunk<RB>(raw, r, sub) + 8 * half);
    const unsigned w[2] = {q.x, q.y};
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      const unsigned t = w[g] ^ 0xAAAAAAAAu;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint4 o;
        o.x = bf16x2_sub(((t >> (8 * h)) & 0x00030003u) | 0x43004300u, 0x43024302u);
        o.y = bf16x2_sub(((t >> (8 * h + 2)) & 0x00030003u) | 0x43004300u, 0x43024302u);
        o.z = bf16x2_sub(((t >> (8 * h + 4)) & 0x00030003u) | 0x43004300u, 0x43024302u);
        o.w = bf16x2_sub(((t >> (8 * h + 6)) & 0x00030003u) | 0x43004300u, 0x43024302u);
        store_chunk(a_tile, r, 4 * half + 2 * g + h, o);
      }
    }
  } else {  // 8-bit
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint2 q = *reinterpret_cast<const uint2*>(raw_chunk<RB>(raw, r, sub * 4 + half * 2 + (c >> 1)) + 8 * (c & 1));
      const unsigned t0 = q.x ^ 0x80808080u, t1 = q.y ^ 0x80808080u;
      float f[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        f[i] = __uint_as_float(0x4B000000u | ((t0 >> (8 * i)) & 0xffu)) - 8388736.0f;
        f[4 + i] = __uint_as_float(0x4B000000u | ((t1 >> (8 * i)) & 0xffu)) - 8388736.0f;
      }
      uint4 o;
      __nv_bfloat162 p;
      p = __floats2bfloat162_rn(f[0], f[1]); o.x = *reinterpret_cast<unsigned*>(&p);
      p = __floats2bfloat162_rn(f[2], f[3]); o.y = *reinterpret_cast<unsigned*>(&p);
      p = __floats2bfloat162_rn(f[4], f[5]); o.z = *reinterpret_cast<unsigned*>(&p);
      p = __floats2bfloat162_rn(f[6], f[7]); o.w = *reinterpret_cast<unsigned*>(&p);
      store_chunk(a_tile, r, 4 * half + c, o);
    }
  }
}

__device__ __forceinline__ void tmem_ld8(unsigned taddr, unsigned (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
// Rendezvous of the 8 dequant/epilogue warps on an mbarrier (count 8) with a bounded wait, so a
// warp that gave up elsewhere can never leave the others blocked.
__device__ __forceinline__ bool warps_rendezvous(unsigned long long* bar, int& uses, int lane, volatile int* abort_flag) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
  const bool ok = mbar_wait(bar, (unsigned)(uses & 1), abort_flag, 7);
  ++uses;
  return ok;
}

struct QParams {
  int64_t M, N, K;
  int kb_total, kb_per_split, splits;
  int n_tiles, m_tiles, items;
  const float* scale;
  const __nv_bfloat16* bias;
  __nv_bfloat16* y;
  float* partial;      // split-K: fp32 slices [items][TN][128], written before they are read
  int* counters;       // split-K: zero-filled int32 [n_tiles * m_tiles], left zero
  int* status;
};

template <int TN, int BITS>
__global__ void __launch_bounds__(kThreadsQ, 1)
linear_tcq_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, QParams p) {
  using L = QLayout<TN, BITS>;
  constexpr int NR = L::NR;
  constexpr int KBS = L::KBS;
  constexpr unsigned TX_BYTES = (unsigned)L::kStage;
  constexpr unsigned TMEM_COLS = TN < 32 ? 32 : TN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* a_ring = smem;                                   // NA x 16 KB
  uint8_t* r_ring = smem + NA * L::kATile;                  // NR x {X tile, raw codes}
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(r_ring + NR * L::kStage);
  unsigned long long* raw_full = bars;                      // [NR] TMA landed
  unsigned long long* raw_empty = bars + NR;                // [NR] 8 dequant warps + MMA commit
  unsigned long long* a_ready = bars + 2 * NR;              // [NA] 8 dequant warps
  unsigned long long* a_empty = a_ready + NA;               // [NA] MMA commit
  unsigned long long* acc_full = a_empty + NA;              // [1]  MMA commit (accumulator complete)
  unsigned long long* ep_bar = acc_full + 1;                // [1]  epilogue rendezvous of the 8 warps
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(ep_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = abort_flag + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NR; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], kDqWarps + 1); }
    for (int i = 0; i < NA; ++i) { mbar_init(&a_ready[i], kDqWarps); mbar_init(&a_empty[i], 1); }
    mbar_init(acc_full, 1);
    mbar_init(ep_bar, kDqWarps);
    *abort_flag = 0;
    *last_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;

  // item -> (n tile, m tile, split); the same enumeration in every role
  auto decode = [&](int item, int& nt, int& mt, int& kb0, int& nkb) {
    const int sp = item % p.splits;
    const int t = item / p.splits;
    nt = t % p.n_tiles;
    mt = t / p.n_tiles;
    kb0 = sp * p.kb_per_split;
    nkb = min(p.kb_per_split, p.kb_total - kb0);
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int gs = 0;                                             // global stage counter of this CTA
      bool ok = true;
      for (int item = blockIdx.x; item < p.items && ok; item += gridDim.x) {
        int nt, mt, kb0, nkb;
        decode(item, nt, mt, kb0, nkb);
        for (int i = 0; i < nkb; i += KBS, ++gs) {
          const int s = gs % NR;
          if (gs >= NR && !mbar_wait(&raw_empty[s], ((gs / NR) - 1) & 1, abort_flag, 1)) { ok = false; break; }
          uint8_t* st = r_ring + s * L::kStage;
          mbar_expect_tx(&raw_full[s], TX_BYTES);
          const int kcol = (kb0 + i) * BK;
#pragma unroll
          for (int j = 0; j < KBS; ++j)                       // columns beyond K are zero-filled by the copy engine
            tma_load_2d(st + j * L::kXTile, &map_x, kcol + j * BK, mt * TN, &raw_full[s]);
          tma_load_2d(st + L::kX, &map_w, kcol * BITS / 8, nt * BM, &raw_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr unsigned idesc = idesc_bf16(TN);
      int g = 0, gs = 0;                                      // k-block / stage counters of this CTA
      bool ok = true;
      for (int item = blockIdx.x; item < p.items && ok; item += gridDim.x) {
        int nt, mt, kb0, nkb;
        decode(item, nt, mt, kb0, nkb);
        for (int i = 0; i < nkb; ++i, ++g) {
          const int sub = i % KBS;
          const int s = gs % NR, a = g % NA;
          ok = mbar_wait(&raw_full[s], (gs / NR) & 1, abort_flag, 2) && mbar_wait(&a_ready[a], (g / NA) & 1, abort_flag, 3);
          if (!ok) break;
          tc_fence_after();
          const unsigned long long adesc = smem_desc_sw128(smem_u32(a_ring + a * L::kATile));
          const unsigned long long bdesc = smem_desc_sw128(smem_u32(r_ring + s * L::kStage + sub * L::kXTile));
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
          umma_commit(&a_empty[a]);
          if (sub == KBS - 1 || i == nkb - 1) { umma_commit(&raw_empty[s]); ++gs; }
        }
        if (ok) umma_commit(acc_full);
      }
    }
  } else {
    // ---------------------------------------------------------------- dequant + epilogue
    const int td = threadIdx.x - 64;                         // 0..255
    const int row = td & 127, half = td >> 7;
    const int q = warp & 3;                                  // TMEM lane quarter of this warp
    const int chalf = (warp - 2) >> 2;                       // which half of the token columns
    int g = 0, gs = 0, it = 0, ep_uses = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < p.items && ok; item += gridDim.x, ++it) {
      int nt, mt, kb0, nkb;
      decode(item, nt, mt, kb0, nkb);
      for (int i = 0; i < nkb; ++i, ++g) {
        const int sub = i % KBS;
        const int s = gs % NR, a = g % NA;
        ok = mbar_wait(&raw_full[s], (gs / NR) & 1, abort_flag, 4);
        if (ok && g >= NA) ok = mbar_wait(&a_empty[a], ((g / NA) - 1) & 1, abort_flag, 5);
        if (!ok) break;
        const uint8_t* raw = r_ring + s * L::kStage + L::kX;
        dequant_half_row<BITS, L::kRawStageRow>(raw, a_ring + a * L::kATile, row, sub, half);
        fence_async_proxy();
        __syncwarp();
        const bool stage_done = (sub == KBS - 1 || i == nkb - 1);
        if (lane == 0) {
          mbar_arrive(&a_ready[a]);
          if (stage_done) mbar_arrive(&raw_empty[s]);
        }
        if (stage_done) ++gs;
      }
      if (!ok) break;
      ok = mbar_wait(acc_full, it & 1, abort_flag, 6);
      if (!ok) break;
      tc_fence_after();
      const int trow = q * 32 + lane;                        // TMEM lane = weight row within the tile
      const int64_t n = (int64_t)nt * BM + trow;
      const int64_t m0 = (int64_t)mt * TN;
      const bool split = p.splits > 1;
      const float sc = (p.scale && n < p.N) ? p.scale[n] : 1.0f;
      const float bv = (p.bias && n < p.N) ? __bfloat162float(p.bias[n]) : 0.f;
      constexpr int CH = TN / 2;                             // columns handled by this warp
      float* slice = p.partial + (size_t)item * (TN * BM);   // [TN][128] of this item
#pragma unroll 1
      for (int c0 = chalf * CH; c0 < (chalf + 1) * CH; c0 += 8) {
        unsigned r[8];
        tmem_ld8(tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)c0, r);
        tmem_ld_wait();
        if (split) {
#pragma unroll
          for (int j = 0; j < 8; ++j) __stcg(&slice[(c0 + j) * BM + trow], __uint_as_float(r[j]));
        } else if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int64_t m = m0 + c0 + j;
            if (m < p.M) p.y[m * p.N + n] = __float2bfloat16_rn(__uint_as_float(r[j]) * sc + bv);
          }
        }
      }
      tc_fence_before();
      if (split) {
        // last CTA of this (n tile, m tile) finalizes: sum of the slices -> y, then reset the counter
        __threadfence();
        if (!(ok = warps_rendezvous(ep_bar, ep_uses, lane, abort_flag))) break;
        if (td == 0) {
          const int old = atomicAdd(&p.counters[mt * p.n_tiles + nt], 1);
          *last_flag = (old == p.splits - 1);
        }
        if (!(ok = warps_rendezvous(ep_bar, ep_uses, lane, abort_flag))) break;
        const bool last = *last_flag != 0;
        if (last) {
          __threadfence();
          if (n < p.N) {
            const float* tile0 = p.partial + (size_t)(item - item % p.splits) * (TN * BM);
            for (int c = chalf * CH; c < (chalf + 1) * CH; ++c) {
              const int64_t m = m0 + c;
              if (m < p.M) {
                float v = 0.f;
                for (int sp = 0; sp < p.splits; ++sp) v += __ldcg(&tile0[(size_t)sp * (TN * BM) + c * BM + trow]);
                p.y[m * p.N + n] = __float2bfloat16_rn(v * sc + bv);
              }
            }
          }
          if (td == 0) p.counters[mt * p.n_tiles + nt] = 0;
        }
        if (!(ok = warps_rendezvous(ep_bar, ep_uses, lane, abort_flag))) break;   // last_flag is reused by the next item
      }
      tc_fence_after();
    }
  }
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);         // error path: let copies in flight land
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicMax(p.status, *abort_flag);
}

}  // namespace
}  // namespace tsb

namespace tsb {
namespace {

template <int TN, int BITS>
int launch_q(const CUtensorMap& mw, const CUtensorMap& mx, const QParams& p, int grid, cudaStream_t s) {
  using L = QLayout<TN, BITS>;
  static bool configured[64] = {false};
  int dev = 0;
  TSB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return TSB200_ERR_DEVICE;
  if (!configured[dev]) {
    TSB_CUDA(cudaFuncSetAttribute(linear_tcq_kernel<TN, BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes));
    configured[dev] = true;
  }
  linear_tcq_kernel<TN, BITS><<<grid, kThreadsQ, L::kBytes, s>>>(mw, mx, p);
  TSB_LAUNCH_CHECK();
  return TSB200_OK;
}

template <int TN>
int launch_q_bits(int bits, const CUtensorMap& mw, const CUtensorMap& mx, const QParams& p, int grid, cudaStream_t s) {
  switch (bits) {
    case 2: return launch_q<TN, 2>(mw, mx, p, grid, s);
    case 4: return launch_q<TN, 4>(mw, mx, p, grid, s);
    case 8: return launch_q<TN, 8>(mw, mx, p, grid, s);
    default: return TSB200_ERR_UNSUPPORTED;
  }
}

// Inner extent (bytes) of the weight box: must equal QLayout<TN, BITS>::kRawStageRow.
int raw_box_bytes(int tn, int bits) {
  const int full = 1024 / bits / BK;
  const int kbs = tn <= 32 ? full : (full < 2 ? full : 2);
  return kbs * BK * bits / 8;
}

int num_sms() {
  static int sms[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!sms[dev]) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    sms[dev] = v;
  }
  return sms[dev];
}

}  // namespace

// y[M, N] = x[M, K] . Wq[N, K]^T * scale + bias; Wq packed at `bits` in {2, 4, 8}; bf16 in/out.
// partial: split-K slice scratch (plan_gemm().slice_bytes); counters: zero-filled, left zero.
int gemm_tcq(const void* W, int bits, const float* scale, const void* bias, const void* x, void* y, int64_t M, int64_t K,
             int64_t N, float* partial, int* counters, int* status, cudaStream_t s) {
  const GemmPlan g = plan_gemm(M, N, K);
  const int tn = g.tn;
  CUtensorMap mw, mx;
  const uint64_t rb = tsb200_packed_row_bytes(K, bits);
  if (!make_map(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, W, rb, (uint64_t)N, rb, (uint32_t)raw_box_bytes(tn, bits), BM,
                raw_box_bytes(tn, bits) == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                               : (raw_box_bytes(tn, bits) == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B)))
    return TSB200_ERR_CUDA;
  if (!make_map(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, BK, (uint32_t)tn, CU_TENSOR_MAP_SWIZZLE_128B))
    return TSB200_ERR_CUDA;
  const int sms = num_sms();
  if ((int64_t)g.n_tiles * g.m_tiles * g.splits > 0x3fffffffLL) return TSB200_ERR_UNSUPPORTED;
  QParams p;
  p.M = M; p.N = N; p.K = K;
  p.kb_total = g.kb_total; p.kb_per_split = g.kb_per_split; p.splits = g.splits;
  p.n_tiles = g.n_tiles; p.m_tiles = g.m_tiles; p.items = g.items;
  p.scale = scale; p.bias = (const __nv_bfloat16*)bias; p.y = (__nv_bfloat16*)y;
  p.partial = partial; p.counters = counters; p.status = status;
  const int grid = p.items < sms ? p.items : sms;
  switch (tn) {
    case 16: return launch_q_bits<16>(bits, mw, mx, p, grid, s);
    case 32: return launch_q_bits<32>(bits, mw, mx, p, grid, s);
    case 64: return launch_q_bits<64>(bits, mw, mx, p, grid, s);
    default: return launch_q_bits<128>(bits, mw, mx, p, grid, s);
  }
}

}  // namespace tsb
