// tcgen05 / TMEM / TMA / mbarrier PTX wrappers and descriptor builders shared by the
// tensor-core LinearCompressed kernels.
#pragma once
#include <cuda.h>
#include "common.cuh"

namespace tsb {
namespace tc {

constexpr int BM = 128;            // weight rows per tile = MMA M
constexpr int BK = 64;             // k per k-block: one 128-byte swizzle atom of bf16
constexpr unsigned kSpinLimit = 1u << 20;   // try_wait attempts before a bounded wait gives up

// Workspace header shared by the linear kernels: status word (byte 0), grid-barrier counters of the
// multi-phase kernel (byte 64..), then split-K tile counters.
constexpr size_t kWsGridBar = 64;
constexpr size_t kWsCounters = 256;
constexpr int kMaxCounters = 4096;
constexpr size_t kWsHeader = kWsCounters + kMaxCounters * sizeof(int);

// Work decomposition of one packed-weight GEMM (host): token tile, K splits, item count.
// Planned for a fixed 148-SM part so that workspace sizing and launch agree; the launch clamps
// the grid to the SMs actually present.
constexpr int kPlanSMs = 148;
struct GemmPlan {
  int tn, kb_total, kb_per_split, splits, n_tiles, m_tiles, items;
  size_t slice_bytes;      // split-K scratch: one fp32 [tn][128] slice per item (0 when splits == 1)
};
// nsub: number of equally shaped matrices sharing the launch (their tiles add up); no_split: keep
// every tile's K range whole (needed when the epilogue combines two accumulators).
// kb_align: every split starts at a multiple of kb_align k-blocks (1-bit containers: 2, so that the byte offset
// of a weight box stays a multiple of 16); a larger alignment never needs more slices than kb_align = 1.
inline GemmPlan plan_gemm(int64_t M, int64_t N, int64_t K, int nsub = 1, bool no_split = false, int kb_align = 1) {
  GemmPlan g;
  // above 128 tokens a 256-token tile with two k-blocks per stage: every widened weight tile then meets twice as many
  // tokens, and one M128 x N256 x K16 MMA (128 cycles of the tensor pipe) outlasts the ~115 cycles its lane needs to
  // issue it (M = 2048, rank 1024, int4: 524 -> 566 TFLOP/s; with one k-block per stage it was slower than 128)
  g.tn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256)));
#ifdef TSB_FORCE_TN128
  if (g.tn == 256) g.tn = 128;
#endif
  g.kb_total = (int)((K + BK - 1) / BK);
  const int64_t n_tiles = (N + BM - 1) / BM, m_tiles = (M + g.tn - 1) / g.tn;
  const int64_t base = n_tiles * m_tiles * nsub;
  int splits = 1;
  if (!no_split && base > 0 && base < kPlanSMs * 3 / 4 && base <= kMaxCounters) {
    // fill the SMs once (prefer a single, nearly full wave); each split keeps >= 4 k-blocks
    const int lo = (int)(kPlanSMs / base), hi = (int)((kPlanSMs + base - 1) / base);
    splits = (base * lo >= kPlanSMs * 3 / 4) ? lo : hi;
    const int cap = g.kb_total / 4 > 0 ? g.kb_total / 4 : 1;
    if (splits > cap) splits = cap;
    if (splits < 1) splits = 1;
  }
  g.kb_per_split = (g.kb_total + splits - 1) / splits;
  g.kb_per_split = (g.kb_per_split + kb_align - 1) / kb_align * kb_align;
  g.splits = (g.kb_total + g.kb_per_split - 1) / g.kb_per_split;
  g.n_tiles = (int)n_tiles;
  g.m_tiles = (int)m_tiles;
  g.items = (int)(base * g.splits);       // over all nsub matrices
  g.slice_bytes = g.splits > 1 ? (size_t)g.items * g.tn * BM * sizeof(float) : 0;
  return g;
}

// ---------------------------------------------------------------- PTX wrappers -----
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and raises the CTA-wide abort flag) when it gives up.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* abort_flag, int code) {
  for (unsigned i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u && *abort_flag) return false;
  }
  *abort_flag = code;
  return false;
}
// Same, for warps that are not on the critical path: sleeps between polls, so that many waiting warps do
// not crowd the single lanes that issue copies and MMAs out of the issue slots and the memory pipeline.
__device__ __forceinline__ bool mbar_wait_relaxed(unsigned long long* bar, unsigned parity, volatile int* abort_flag, int code) {
  for (unsigned i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u && *abort_flag) return false;
    __nanosleep(64);
  }
  *abort_flag = code;
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, unsigned long long* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void tmem_alloc(unsigned* smem_dst, unsigned ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(unsigned d_tmem, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                          unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(unsigned taddr, unsigned (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand tile with 128-byte swizzle, rows of 128
// bytes, 8-row groups 1024 bytes apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ unsigned long long smem_desc_sw128(unsigned saddr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((saddr >> 4) & 0x3FFFu);
  d |= (unsigned long long)1u << 16;                 // leading byte offset (unused for swizzled K-major)
  d |= (unsigned long long)(1024u >> 4) << 32;       // stride byte offset
  d |= (unsigned long long)1u << 46;                 // version
  d |= (unsigned long long)2u << 61;                 // SWIZZLE_128B
  return d;
}
// Instruction descriptor, kind::f16: D=f32, A=B=bf16, both K-major, M=128, N=n.
__host__ __device__ constexpr unsigned idesc_bf16(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
}


// Write 8 bf16 (one 16-byte chunk `c` of row `r`) into a 128-byte-swizzled K-major tile.
__device__ __forceinline__ void store_chunk(uint8_t* a_tile, int r, int c, uint4 v) {
  *reinterpret_cast<uint4*>(a_tile + r * 128 + ((c ^ (r & 7)) << 4)) = v;
}
__device__ __forceinline__ unsigned bf16x2_sub(unsigned a, unsigned b) {
  __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
  return *reinterpret_cast<unsigned*>(&r);
}

// Host: 2-D row-major tensor map; box = [box_rows, box_inner] elements of `dt`.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}
inline bool make_map(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t rows,
                     uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {inner, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// bf16 activations x[M, K] (K a multiple of 64) viewed as [K/64 k-blocks][M rows][64 columns]: one box of
// (64, box_rows, box_kb) lands as box_kb consecutive 128-byte-swizzled tiles of box_rows x 64.
inline bool make_map_x3d(CUtensorMap* map, const void* base, uint64_t K, uint64_t M, uint32_t box_rows, uint32_t box_kb) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {64, M, K / 64};
  cuuint64_t strides[2] = {K * 2, 128};
  cuuint32_t box[3] = {64, box_rows, box_kb};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tc

// Host-side description of one matrix product y[M, N] = x[M, K] . W[N, K]^T * scale + bias.
struct GemmSpec {
  const void* W;
  const float* scale;
  const void* bias;
  const void* x;
  void* y;
  int64_t N, K;
};
// One phase of a multi-phase launch: 1 matrix, 2 independent matrices of the same shape, or
// (gated) a gate / up pair whose epilogue stores silu(gate) * up into g[0].y.
struct PhaseSpec {
  GemmSpec g[2];
  int nsub;
  int gated;
};
int run_program_tcq(const PhaseSpec* specs, int n_phases, int bits, int64_t M, uint8_t* scratch, int* counters, int* grid_bar,
                    int* status, cudaStream_t s);
size_t phase_scratch_bytes(int64_t M, int64_t N, int64_t K, int nsub, bool gated);

}  // namespace tsb
