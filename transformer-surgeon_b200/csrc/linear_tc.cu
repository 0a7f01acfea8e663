// LinearCompressed.forward on the 5th-generation tensor cores (tcgen05 / TMEM / TMA).
//
// Replaces transformersurgeon/blocks/linear_compressed.py:96-100 for bf16 activations:
//   Y[M, N] = (X[M, K] . Wq[N, K]^T) * scale[N] + bias[N]
// called once for the V factor (N = rank, result rounded to bf16 = the rank-r intermediate)
// and once for the U factor.  The GEMM is issued "swapped": the weight tile is the MMA A
// operand (M_mma = 128 weight rows), the activations are the B operand (N_mma = token tile),
// so decode batches of 16..128 tokens still fill the 128-row datapath, and the per-row
// dequantization scale and bias are per-TMEM-lane constants in the epilogue.
//
// Warp roles (6 warps):
//   warp 0      TMA producer: activation tile (TN x 64 bf16, 128-byte swizzle) and the packed
//               weight tile (128 rows x 64 codes, raw bytes) per k-block into a 4-stage ring
//   warp 1      TMEM allocation; one lane issues tcgen05.mma (4 x K=16 per k-block) and
//               tcgen05.commit to release stages / publish the accumulator
//   warps 2..5  dequantize: raw codes -> bf16 (exact integers) written in the 128-byte-swizzled
//               K-major layout the MMA descriptor expects; afterwards the epilogue:
//               tcgen05.ld the fp32 accumulator (one TMEM lane = one weight row per thread),
//               scale, bias, store (or fp32 atomics into a split-K buffer)
// Every mbarrier wait is bounded; on expiry the kernel records a code in the status word
// (first 4 bytes of the workspace), drains and frees TMEM, and returns.
#include "tc_common.cuh"

namespace tsb {
using namespace tc;
namespace {

constexpr int NSTG = 4;
constexpr int kThreads = 192;

// ---------------------------------------------------------------- dequantization ---
// One thread converts one weight row of the k-block: 64 codes -> 64 bf16.
template <int BITS>
__device__ __forceinline__ void dequant_row(const uint8_t* __restrict__ raw_row, uint8_t* a_tile, int r) {
  if (BITS == 4) {
    // word = 8 columns, field j -> column 2j, field j+4 -> column 2j+1.  (w ^ 0x88888888) biases every
    // nibble by +8; 0x4300 | u is the bf16 128 + u; subtracting 136 leaves the signed code.
    const uint4 q0 = *reinterpret_cast<const uint4*>(raw_row);
    const uint4 q1 = *reinterpret_cast<const uint4*>(raw_row + 16);
    const unsigned w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const unsigned t = w[c] ^ 0x88888888u;
      uint4 o;
      o.x = bf16x2_sub(((t)&0x000f000fu) | 0x43004300u, 0x43084308u);
      o.y = bf16x2_sub(((t >> 4) & 0x000f000fu) | 0x43004300u, 0x43084308u);
      o.z = bf16x2_sub(((t >> 8) & 0x000f000fu) | 0x43004300u, 0x43084308u);
      o.w = bf16x2_sub(((t >> 12) & 0x000f000fu) | 0x43004300u, 0x43084308u);
      store_chunk(a_tile, r, c, o);
    }
  } else if (BITS == 2) {
    // word = 16 columns, field j -> column 2j, field j+8 -> column 2j+1; bias +2, subtract 130.
    const uint4 q0 = *reinterpret_cast<const uint4*>(raw_row);
    const unsigned w[4] = {q0.x, q0.y, q0.z, q0.w};
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const unsigned t = w[g] ^ 0xAAAAAAAAu;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint4 o;
        o.x = bf16x2_sub(((t >> (8 * h)) & 0x00030003u) | 0x43004300u, 0x43024302u);
        o.y = bf16x2_sub(((t >> (8 * h + 2)) & 0x00030003u) | 0x43004300u, 0x43024302u);
        o.z = bf16x2_sub(((t >> (8 * h + 4)) & 0x00030003u) | 0x43004300u, 0x43024302u);
        o.w = bf16x2_sub(((t >> (8 * h + 6)) & 0x00030003u) | 0x43004300u, 0x43024302u);
        store_chunk(a_tile, r, 2 * g + h, o);
      }
    }
  } else {  // BITS == 8: natural byte order; int8 -> f32 by the 2^23 trick, then pack to bf16x2
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint2 q = *reinterpret_cast<const uint2*>(raw_row + 8 * c);
      const unsigned t0 = q.x ^ 0x80808080u, t1 = q.y ^ 0x80808080u;
      float f[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        f[i] = __uint_as_float(0x4B000000u | ((t0 >> (8 * i)) & 0xffu)) - 8388736.0f;       // 2^23 + 128
        f[4 + i] = __uint_as_float(0x4B000000u | ((t1 >> (8 * i)) & 0xffu)) - 8388736.0f;
      }
      uint4 o;
      __nv_bfloat162 p;
      p = __floats2bfloat162_rn(f[0], f[1]); o.x = *reinterpret_cast<unsigned*>(&p);
      p = __floats2bfloat162_rn(f[2], f[3]); o.y = *reinterpret_cast<unsigned*>(&p);
      p = __floats2bfloat162_rn(f[4], f[5]); o.z = *reinterpret_cast<unsigned*>(&p);
      p = __floats2bfloat162_rn(f[6], f[7]); o.w = *reinterpret_cast<unsigned*>(&p);
      store_chunk(a_tile, r, c, o);
    }
  }
}

struct TcParams {
  int64_t M, N, K;
  int kb_total;            // k-blocks of 64 over the whole K
  int kb_per_split;
  const float* scale;      // [N] or null (dense)
  const __nv_bfloat16* bias;  // [N] or null
  __nv_bfloat16* y;        // [M, N]
  float* partial;          // [M, N] fp32 accumulation buffer when gridDim.z > 1
  int* status;             // device status word
};

template <int TN> struct SmemLayout {
  static constexpr int kA = BM * 128;            // 16 KB bf16 A tile
  static constexpr int kX = TN * 128;            // activation tile
  static constexpr int kRaw = BM * 64;           // raw codes (sized for 8-bit)
  static constexpr int kStage = kA + kX + kRaw;
  static constexpr int kBytes = NSTG * kStage + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <int TN, int BITS>
__global__ void __launch_bounds__(kThreads, 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TcParams p) {
  using L = SmemLayout<TN>;
  constexpr int RAW_ROW = BITS == 16 ? 0 : BK * BITS / 8;     // bytes of one weight row per k-block
  constexpr unsigned TX_BYTES = (unsigned)(TN * 128 + (BITS == 16 ? BM * 128 : BM * RAW_ROW));
  constexpr unsigned TMEM_COLS = TN < 32 ? 32 : TN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + NSTG * L::kStage);
  unsigned long long* full_bar = bars;                 // TMA landed            [NSTG]
  unsigned long long* ready_bar = bars + NSTG;         // A tile dequantized    [NSTG]
  unsigned long long* empty_bar = bars + 2 * NSTG;     // MMA done with stage   [NSTG]
  unsigned long long* acc_bar = bars + 3 * NSTG;       // accumulator complete  [1]
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 3 * NSTG + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM;                      // first weight row of this CTA
  const int m0 = blockIdx.y * TN;                      // first token
  const int kb0 = blockIdx.z * p.kb_per_split;
  const int nkb = min(p.kb_per_split, p.kb_total - kb0);

  if (threadIdx.x == 0) {
    for (int i = 0; i < NSTG; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&ready_bar[i], 4);                     // one arrival per dequant warp
      mbar_init(&empty_bar[i], 1);
    }
    mbar_init(acc_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();     // activations (and the split-K buffer) belong to the preceding kernels

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer -----
    if (lane == 0) {
      for (int i = 0; i < nkb; ++i) {
        const int s = i % NSTG;
        if (i >= NSTG && !mbar_wait(&empty_bar[s], ((i / NSTG) - 1) & 1, abort_flag, 1)) break;
        uint8_t* st = smem + s * L::kStage;
        mbar_expect_tx(&full_bar[s], TX_BYTES);
        const int kcol = (kb0 + i) * BK;
        tma_load_2d(st + L::kA, &map_x, kcol, m0, &full_bar[s]);
        if (BITS == 16) tma_load_2d(st, &map_w, kcol, n0, &full_bar[s]);
        else tma_load_2d(st + L::kA + L::kX, &map_w, kcol * BITS / 8, n0, &full_bar[s]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer -------
    if (lane == 0) {
      constexpr unsigned idesc = idesc_bf16(TN);
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % NSTG;
        const unsigned ph = (i / NSTG) & 1;
        ok = mbar_wait(&full_bar[s], ph, abort_flag, 2) && mbar_wait(&ready_bar[s], ph, abort_flag, 3);
        if (!ok) break;
        tc_fence_after();
        uint8_t* st = smem + s * L::kStage;
        const unsigned long long adesc = smem_desc_sw128(smem_u32(st));
        const unsigned long long bdesc = smem_desc_sw128(smem_u32(st + L::kA));
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)   // +32 bytes (2 x 16-byte units) along K inside the swizzle atom
          umma_bf16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(&empty_bar[s]);
      }
      if (ok) umma_commit(acc_bar);
    }
  } else {
    // ------------------------------------------------------------ dequant + epilogue
    const int t = threadIdx.x - 64;                    // 0..127 = weight row inside the tile
    bool ok = true;
    for (int i = 0; i < nkb && ok; ++i) {
      const int s = i % NSTG;
      const unsigned ph = (i / NSTG) & 1;
      ok = mbar_wait(&full_bar[s], ph, abort_flag, 4);
      if (!ok) break;
      if (BITS != 16) {
        uint8_t* st = smem + s * L::kStage;
        dequant_row<BITS == 16 ? 8 : BITS>(st + L::kA + L::kX + t * RAW_ROW, st, t);
        fence_async_proxy();                           // generic-proxy writes -> visible to the MMA (async proxy)
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ready_bar[s]);
    }
    // epilogue: TMEM lane quarter of this warp is (warp % 4)
    if (ok && nkb > 0) ok = mbar_wait(acc_bar, 0, abort_flag, 5);
    if (ok && nkb > 0) {
      tc_fence_after();
      const int q = warp & 3;
      const int row = q * 32 + lane;                   // TMEM lane = weight row in tile
      const int64_t n = (int64_t)n0 + row;
      const float sc = (p.scale && n < p.N) ? p.scale[n] : 1.0f;
      const float bv = (p.bias && n < p.N && blockIdx.z == 0) ? __bfloat162float(p.bias[n]) : 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < TN; c0 += 16) {
        unsigned r[16];
        tmem_ld16(tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)c0, r);
        tmem_ld_wait();
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int64_t m = (int64_t)m0 + c0 + j;
            if (m < p.M) {
              const float v = __uint_as_float(r[j]) * sc + bv;
              if (gridDim.z == 1) p.y[m * p.N + n] = __float2bfloat16_rn(v);
              else atomicAdd(&p.partial[m * p.N + n], v);
            }
          }
        }
      }
    }
  }
  if (*abort_flag) {
    // error path only: give copies that may still be in flight a bounded time to land
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicMax(p.status, *abort_flag);
}

// fp32 split-K buffer -> bf16 output.
__global__ void splitk_finalize_kernel(float* __restrict__ partial, __nv_bfloat16* __restrict__ y, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    y[i] = __float2bfloat16_rn(partial[i]);
    partial[i] = 0.f;     // the split-K buffer is shared with the persistent kernel, which expects zeros
  }
}

// ---------------------------------------------------------------- host side --------
template <int TN, int BITS>
int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const TcParams& p, dim3 grid, cudaStream_t s) {
  using L = SmemLayout<TN>;
  static bool configured[64] = {false};
  int dev = 0;
  TSB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return TSB200_ERR_DEVICE;
  if (!configured[dev]) {
    TSB_CUDA(cudaFuncSetAttribute(linear_tc_kernel<TN, BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes));
    configured[dev] = true;
  }
  TSB_CUDA(launch_kernel(linear_tc_kernel<TN, BITS>, grid, dim3(kThreads), (size_t)L::kBytes, s, mw, mx, p));
  return TSB200_OK;
}

template <int TN>
int launch_tc_bits(int bits, const CUtensorMap& mw, const CUtensorMap& mx, const TcParams& p, dim3 grid, cudaStream_t s) {
  switch (bits) {
    case 2: return launch_tc<TN, 2>(mw, mx, p, grid, s);
    case 4: return launch_tc<TN, 4>(mw, mx, p, grid, s);
    case 8: return launch_tc<TN, 8>(mw, mx, p, grid, s);
    case 16: return launch_tc<TN, 16>(mw, mx, p, grid, s);
    default: return TSB200_ERR_UNSUPPORTED;
  }
}

// One quantized GEMM: y[M, N] = x[M, K] . W[N, K]^T * scale + bias (bf16 in/out).
int gemm_tc(const void* W, int bits, const float* scale, const void* bias, const void* x, void* y, int64_t M, int64_t K,
            int64_t N, float* partial, int* status, cudaStream_t s) {
  const int tn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  CUtensorMap mw, mx;
  if (bits == 16) {
    if (!make_map(&mw, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, W, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, BK, BM,
                  CU_TENSOR_MAP_SWIZZLE_128B))
      return TSB200_ERR_CUDA;
  } else {
    const uint64_t rb = tsb200_packed_row_bytes(K, bits);
    if (!make_map(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, W, rb, (uint64_t)N, rb, (uint32_t)(BK * bits / 8), BM,
                  CU_TENSOR_MAP_SWIZZLE_NONE))
      return TSB200_ERR_CUDA;
  }
  if (!make_map(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, BK, (uint32_t)tn,
                CU_TENSOR_MAP_SWIZZLE_128B))
    return TSB200_ERR_CUDA;
  const int kb_total = (int)((K + BK - 1) / BK);
  const int64_t n_tiles = (N + BM - 1) / BM, m_tiles = (M + tn - 1) / tn;
  // split K until the grid covers the 148 SMs (each split keeps >= 4 k-blocks)
  int splits = 1;
  while (n_tiles * m_tiles * splits < 148 && splits * 2 <= 16 && kb_total / (splits * 2) >= 4) splits *= 2;
  const int kb_per_split = (kb_total + splits - 1) / splits;
  splits = (kb_total + kb_per_split - 1) / kb_per_split;
  if (n_tiles > 0x7fffffffLL || m_tiles > 65535) return TSB200_ERR_UNSUPPORTED;
  TcParams p;
  p.M = M; p.N = N; p.K = K; p.kb_total = kb_total; p.kb_per_split = kb_per_split;
  p.scale = scale; p.bias = (const __nv_bfloat16*)bias; p.y = (__nv_bfloat16*)y; p.partial = partial; p.status = status;
  if (splits > 1) TSB_CUDA(cudaMemsetAsync(partial, 0, (size_t)M * N * sizeof(float), s));
  dim3 grid((unsigned)n_tiles, (unsigned)m_tiles, (unsigned)splits);
  int st;
  switch (tn) {
    case 16: st = launch_tc_bits<16>(bits, mw, mx, p, grid, s); break;
    case 32: st = launch_tc_bits<32>(bits, mw, mx, p, grid, s); break;
    case 64: st = launch_tc_bits<64>(bits, mw, mx, p, grid, s); break;
    default: st = launch_tc_bits<128>(bits, mw, mx, p, grid, s); break;
  }
  if (st != TSB200_OK) return st;
  if (splits > 1) {
    const int64_t n = M * N;
    int64_t g = (n + 255) / 256;
    if (g > 148 * 8) g = 148 * 8;
    splitk_finalize_kernel<<<(unsigned)g, 256, 0, s>>>(partial, (__nv_bfloat16*)y, n);
    TSB_LAUNCH_CHECK();
  }
  return TSB200_OK;
}

// 1-bit rows are 8 bytes per 64 columns: the copy engine wants a 16-byte row pitch
bool tc_supported_factor(int bits, int64_t K) {
  if (bits == 1) return K % 128 == 0;
  return (bits == 2 || bits == 4 || bits == 8 || bits == 16) && (K % 8) == 0;
}

}  // namespace

// Persistent kernel for packed factors (linear_tcq.cu).
int gemm_tcq(const void* W, int bits, const float* scale, const void* bias, const void* x, void* y, int64_t M, int64_t K,
             int64_t N, float* partial, int* counters, int* status, cudaStream_t s);

int linear_tc(const tsb200_linear_desc* d, const void* x, void* y, int64_t M, void* workspace, size_t workspace_bytes,
              cudaStream_t s) {
  if (d->act_dtype != TSB200_BF16) return TSB200_ERR_UNSUPPORTED;
  const int64_t ku = d->rank > 0 ? d->rank : d->in_features;
  if (!tc_supported_factor(d->u_bits, ku)) return TSB200_ERR_UNSUPPORTED;
  if (d->rank > 0 && !tc_supported_factor(d->v_bits, d->in_features)) return TSB200_ERR_UNSUPPORTED;
  if (!aligned(x, 16) || !aligned(y, 2)) return TSB200_ERR_ARG;
  if (!workspace || !aligned(workspace, 256)) return TSB200_ERR_ARG;
  if (workspace_bytes < tsb200_linear_workspace_bytes(d, M)) return TSB200_ERR_WORKSPACE;
  uint8_t* ws = (uint8_t*)workspace;
  int* status = (int*)ws;
  int* counters = (int*)(ws + kWsCounters);
  void* h = ws + kWsHeader;
  const size_t hbytes = ((size_t)M * (size_t)(d->rank > 0 ? d->rank : 0) * 2 + 255) / 256 * 256;
  float* partial = (float*)(ws + kWsHeader + hbytes);
  auto gemm = [&](const void* W, int bits, const float* scale, const void* bias, const void* in, void* out, int64_t K,
                  int64_t N) {
    return bits == 16 ? gemm_tc(W, bits, scale, bias, in, out, M, K, N, partial, status, s)
                      : gemm_tcq(W, bits, scale, bias, in, out, M, K, N, partial, counters, status, s);
  };
  if (d->rank > 0 && d->u_bits == d->v_bits && d->u_bits <= 8) {
    // both factors packed alike: V then U as two phases of ONE launch (grid barrier in between);
    // the rank-r intermediate is produced and consumed through L2
    PhaseSpec ps[2];
    ps[0].nsub = 1; ps[0].gated = 0;
    ps[0].g[0] = GemmSpec{d->v, d->v_scale, nullptr, x, h, d->rank, d->in_features};
    ps[1].nsub = 1; ps[1].gated = 0;
    ps[1].g[0] = GemmSpec{d->u, d->u_scale, d->bias, h, y, d->out_features, d->rank};
    return run_program_tcq(ps, 2, d->u_bits, M, (uint8_t*)partial, counters, (int*)(ws + kWsGridBar), status, s);
  }
  const void* in = x;
  if (d->rank > 0) {
    int st = gemm(d->v, d->v_bits, d->v_scale, nullptr, x, h, d->in_features, d->rank);
    if (st != TSB200_OK) return st;
    in = h;
  }
  return gemm(d->u, d->u_bits, d->u_scale, d->bias, in, y, ku, d->out_features);
}

}  // namespace tsb
