// tcgen05 GEMM for LinearCompressed with DENSE bf16 factors (e.g. an unquantized lm_head):
//   Y[M, N] = X[M, K] . W[N, K]^T + bias[N]
// restating transformersurgeon/blocks/linear_compressed.py:96-100.  Packed (quantized) factors are served by
// the persistent kernel in linear_tcq.cu; this file also holds the dispatch between the two (linear_tc()).
//
// One CTA = one (128-row weight tile, token tile, K split).  Warp roles (6 warps):
//   warp 0      TMA producer: activation tile (TN x 64 bf16) and weight tile (128 x 64 bf16), both with the
//               128-byte swizzle, per k-block into a 4-stage ring
//   warp 1      TMEM allocation; one lane issues tcgen05.mma (4 x K=16 per k-block, both operands from shared
//               memory) and tcgen05.commit to release stages / publish the accumulator
//   warps 2..5  epilogue: tcgen05.ld the fp32 accumulator (one TMEM lane = one weight row per thread), bias,
//               store - or fp32 atomics into the split-K buffer, which a small kernel then rounds to bf16
// Every mbarrier wait is bounded; on expiry the kernel records a code in the status word
// (first 4 bytes of the workspace), drains and frees TMEM, and returns.
#include "tc_common.cuh"

namespace tsb {
using namespace tc;
namespace {

constexpr int NSTG = 4;
constexpr int kThreads = 192;

struct TcParams {
  int64_t M, N, K;
  int kb_total;            // k-blocks of 64 over the whole K
  int kb_per_split;
  const float* scale;      // [N] or null (dense)
  const __nv_bfloat16* bias;  // [N] or null
  __nv_bfloat16* y;        // [M, N]
  float* partial;          // [M, N] fp32 accumulation buffer when gridDim.z > 1
  int* status;             // device status word
  float* amax_val;         // greedy head: per (token, weight tile) maximum of the rounded logits [M][n_tiles] ...
  int* amax_idx;           // ... and the column that holds it (the first one on ties)
};

template <int TN> struct SmemLayout {
  static constexpr int kA = BM * 128;            // 16 KB bf16 weight tile (the MMA's A operand)
  static constexpr int kX = TN * 128;            // activation tile
  static constexpr int kStage = (kA + kX + 1023) / 1024 * 1024;
  static constexpr int kBytes = NSTG * kStage + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// ARGMAX: the epilogue does not store y; it reduces every token's logits of this 128-column tile to (maximum, column)
// - the greedy head: the [M, vocabulary] logits are never written.
template <int TN, bool ARGMAX>
__global__ void __launch_bounds__(kThreads, 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, TcParams p) {
  using L = SmemLayout<TN>;
  constexpr unsigned TX_BYTES = (unsigned)(TN * 128 + BM * 128);
  constexpr unsigned TMEM_COLS = TN < 32 ? 32 : TN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(smem + NSTG * L::kStage);
  unsigned long long* full_bar = bars;                 // TMA landed            [NSTG]
  unsigned long long* empty_bar = bars + NSTG;         // MMA done with stage   [NSTG]
  unsigned long long* acc_bar = bars + 2 * NSTG;       // accumulator complete  [1]
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * NSTG + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM;                      // first weight row of this CTA
  const int m0 = blockIdx.y * TN;                      // first token
  const int kb0 = blockIdx.z * p.kb_per_split;
  const int nkb = min(p.kb_per_split, p.kb_total - kb0);

  if (threadIdx.x == 0) {
    for (int i = 0; i < NSTG; ++i) {
      mbar_init(&full_bar[i], 1);
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
        tma_load_2d(st, &map_w, kcol, n0, &full_bar[s]);
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
        ok = mbar_wait(&full_bar[s], ph, abort_flag, 2);
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
    // ------------------------------------------------------------ epilogue
    bool ok = true;
    // epilogue: TMEM lane quarter of this warp is (warp % 4)
    if (ok && nkb > 0) ok = mbar_wait(acc_bar, 0, abort_flag, 5);
    if (ok && nkb > 0) {
      tc_fence_after();
      const int q = warp & 3;
      const int row = q * 32 + lane;                   // TMEM lane = weight row in tile
      const int64_t n = (int64_t)n0 + row;
      const float sc = (p.scale && n < p.N) ? p.scale[n] : 1.0f;
      const float bv = (p.bias && n < p.N && blockIdx.z == 0) ? __bfloat162float(p.bias[n]) : 0.f;
      if (ARGMAX) {
        // logits of the tile -> shared memory [token][row] (the ring is idle: every MMA has completed), rounded to
        // bf16 as the stored logits would be, so that the choice equals an argmax over them
        float* vt = reinterpret_cast<float*>(smem);                  // [TN][129]
        float* best_v = vt + TN * 129;                               // [TN][parts]
        int* best_i = reinterpret_cast<int*>(best_v + 128);
#pragma unroll 1
        for (int c0 = 0; c0 < TN; c0 += 16) {
          unsigned r[16];
          tmem_ld16(tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j)
            vt[(c0 + j) * 129 + row] = n < p.N ? __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[j]) * sc + bv)) : -INFINITY;
        }
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        constexpr int PARTS = 128 / TN;                               // threads per token; each scans TN consecutive rows
        const int tid = threadIdx.x - 64, col = tid % TN, part = tid / TN;
        float bvv = -INFINITY;
        int bii = part * TN;
        for (int rr = 0; rr < TN; ++rr) {
          const float v = vt[col * 129 + part * TN + rr];
          if (v > bvv) { bvv = v; bii = part * TN + rr; }             // ascending scan, strict: the first maximum wins
        }
        best_v[col * PARTS + part] = bvv;
        best_i[col * PARTS + part] = bii;
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        if (tid < TN && (int64_t)m0 + tid < p.M) {
          float fv = best_v[tid * PARTS];
          int fi = best_i[tid * PARTS];
          for (int pp = 1; pp < PARTS; ++pp)
            if (best_v[tid * PARTS + pp] > fv) { fv = best_v[tid * PARTS + pp]; fi = best_i[tid * PARTS + pp]; }
          const int64_t o = ((int64_t)m0 + tid) * gridDim.x + blockIdx.x;
          p.amax_val[o] = fv;
          p.amax_idx[o] = n0 + fi;
        }
      } else {
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

// Greedy head, second step: the per-tile (maximum, column) pairs of one token -> its token id.  Ties go to the
// smaller column, as in an argmax that returns the first maximum.
__global__ void argmax_finalize_kernel(const float* __restrict__ val, const int* __restrict__ idx, int n_tiles, int64_t* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sv[256];
  __shared__ int si[256];
  const int64_t m = blockIdx.x;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int t = threadIdx.x; t < n_tiles; t += blockDim.x) {
    const float v = val[m * n_tiles + t];
    const int i = idx[m * n_tiles + t];
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
  sv[threadIdx.x] = bv;
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if ((int)threadIdx.x < s) {
      const float v = sv[threadIdx.x + s];
      const int i = si[threadIdx.x + s];
      if (v > sv[threadIdx.x] || (v == sv[threadIdx.x] && i < si[threadIdx.x])) { sv[threadIdx.x] = v; si[threadIdx.x] = i; }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) out[m] = si[0] == 0x7fffffff ? 0 : si[0];
}

// Argmax over stored logits y [M, N] (the route for heads the fused epilogue does not serve).
template <typename T>
__global__ void argmax_rows_kernel(const T* __restrict__ y, int64_t N, int64_t* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sv[256];
  __shared__ int si[256];
  const int64_t m = blockIdx.x;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int64_t n = threadIdx.x; n < N; n += blockDim.x) {
    const float v = to_f32<T>(y[m * N + n]);
    if (v > bv) { bv = v; bi = (int)n; }               // ascending per thread: the first maximum is kept
  }
  sv[threadIdx.x] = bv;
  si[threadIdx.x] = bi;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if ((int)threadIdx.x < s) {
      const float v = sv[threadIdx.x + s];
      const int i = si[threadIdx.x + s];
      if (v > sv[threadIdx.x] || (v == sv[threadIdx.x] && i < si[threadIdx.x])) { sv[threadIdx.x] = v; si[threadIdx.x] = i; }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) out[m] = si[0] == 0x7fffffff ? 0 : si[0];
}

// fp32 split-K buffer -> bf16 output.
__global__ void splitk_finalize_kernel(float* __restrict__ partial, __nv_bfloat16* __restrict__ y, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    y[i] = __float2bfloat16_rn(partial[i]);
    partial[i] = 0.f;     // the split-K buffer is shared with the persistent kernel, which expects zeros
  }
}

// ---------------------------------------------------------------- host side --------
template <int TN, bool ARGMAX>
int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, const TcParams& p, dim3 grid, cudaStream_t s) {
  using L = SmemLayout<TN>;
  static bool configured[64] = {false};
  int dev = 0;
  TSB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return TSB200_ERR_DEVICE;
  if (!configured[dev]) {
    TSB_CUDA(cudaFuncSetAttribute(linear_tc_kernel<TN, ARGMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes));
    configured[dev] = true;
  }
  TSB_CUDA(launch_kernel(linear_tc_kernel<TN, ARGMAX>, grid, dim3(kThreads), (size_t)L::kBytes, s, mw, mx, p));
  return TSB200_OK;
}

// One dense GEMM: y[M, N] = x[M, K] . W[N, K]^T + bias (bf16 in/out; bits must be 16).  tokens != null: the greedy
// head instead - no y; amax scratch (float [M][n_tiles], then int [M][n_tiles]) -> tokens [M] (M <= 128).
int gemm_tc(const void* W, int bits, const float* scale, const void* bias, const void* x, void* y, int64_t M, int64_t K,
            int64_t N, float* partial, int* status, cudaStream_t s, int64_t* tokens = nullptr, void* amax = nullptr) {
  const int tn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  if (bits != 16) return TSB200_ERR_UNSUPPORTED;
  CUtensorMap mw, mx;
  if (!make_map(&mw, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, W, (uint64_t)K, (uint64_t)N, (uint64_t)K * 2, BK, BM,
                CU_TENSOR_MAP_SWIZZLE_128B))
    return TSB200_ERR_CUDA;
  if (!make_map(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, BK, (uint32_t)tn,
                CU_TENSOR_MAP_SWIZZLE_128B))
    return TSB200_ERR_CUDA;
  const int kb_total = (int)((K + BK - 1) / BK);
  const int64_t n_tiles = (N + BM - 1) / BM, m_tiles = (M + tn - 1) / tn;
  // split K until the grid covers the 148 SMs (each split keeps >= 4 k-blocks)
  int splits = 1;
  while (!tokens && n_tiles * m_tiles * splits < 148 && splits * 2 <= 16 && kb_total / (splits * 2) >= 4) splits *= 2;
  const int kb_per_split = (kb_total + splits - 1) / splits;
  splits = (kb_total + kb_per_split - 1) / kb_per_split;
  if (n_tiles > 0x7fffffffLL || m_tiles > 65535) return TSB200_ERR_UNSUPPORTED;
  TcParams p;
  p.M = M; p.N = N; p.K = K; p.kb_total = kb_total; p.kb_per_split = kb_per_split;
  p.scale = scale; p.bias = (const __nv_bfloat16*)bias; p.y = (__nv_bfloat16*)y; p.partial = partial; p.status = status;
  p.amax_val = (float*)amax;
  p.amax_idx = (int*)((float*)amax + (tokens ? M * n_tiles : 0));
  if (tokens) {
    if (m_tiles != 1) return TSB200_ERR_UNSUPPORTED;
    dim3 g((unsigned)n_tiles, 1, 1);
    int st2;
    switch (tn) {
      case 16: st2 = launch_tc<16, true>(mw, mx, p, g, s); break;
      case 32: st2 = launch_tc<32, true>(mw, mx, p, g, s); break;
      case 64: st2 = launch_tc<64, true>(mw, mx, p, g, s); break;
      default: st2 = launch_tc<128, true>(mw, mx, p, g, s); break;
    }
    if (st2 != TSB200_OK) return st2;
    TSB_CUDA(launch_kernel(argmax_finalize_kernel, dim3((unsigned)M), dim3(256), 0, s, (const float*)p.amax_val, (const int*)p.amax_idx,
                           (int)n_tiles, tokens));
    return TSB200_OK;
  }
  if (splits > 1) TSB_CUDA(cudaMemsetAsync(partial, 0, (size_t)M * N * sizeof(float), s));
  dim3 grid((unsigned)n_tiles, (unsigned)m_tiles, (unsigned)splits);
  int st;
  switch (tn) {
    case 16: st = launch_tc<16, false>(mw, mx, p, grid, s); break;
    case 32: st = launch_tc<32, false>(mw, mx, p, grid, s); break;
    case 64: st = launch_tc<64, false>(mw, mx, p, grid, s); break;
    default: st = launch_tc<128, false>(mw, mx, p, grid, s); break;
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

// Greedy head.  Fused route (dense bf16, full rank, M <= 128): no logits in memory.  Returns TSB200_ERR_UNSUPPORTED
// for every other layer (the caller then computes the logits and reduces them).
int linear_argmax_tc(const tsb200_linear_desc* d, const void* x, int64_t* tokens, int64_t M, void* amax, int* status, cudaStream_t s) {
  if (d->act_dtype != TSB200_BF16 || d->rank > 0 || d->u_bits != 16 || M > 128 || (d->in_features % 8)) return TSB200_ERR_UNSUPPORTED;
  if (!aligned(x, 16)) return TSB200_ERR_ARG;
  return gemm_tc(d->u, 16, nullptr, d->bias, x, nullptr, M, d->in_features, d->out_features, nullptr, status, s, tokens, amax);
}
int argmax_rows(const void* y, int dtype, int64_t M, int64_t N, int64_t* tokens, cudaStream_t s) {
  if (dtype == TSB200_F32) TSB_CUDA(launch_kernel(argmax_rows_kernel<float>, dim3((unsigned)M), dim3(256), 0, s, (const float*)y, N, tokens));
  else TSB_CUDA(launch_kernel(argmax_rows_kernel<__nv_bfloat16>, dim3((unsigned)M), dim3(256), 0, s, (const __nv_bfloat16*)y, N, tokens));
  return TSB200_OK;
}

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
