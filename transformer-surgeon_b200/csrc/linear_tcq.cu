// Persistent tcgen05 kernel for LinearCompressed with QUANTIZED factors (int8 / int4 / int2 / 1-bit):
//   Y[M, N] = (X[M, K] . Wq[N, K]^T) * scale[N] + bias[N]        (bf16 activations)
// restating transformersurgeon/blocks/linear_compressed.py:96-100 on packed codes.
//
// Decode-time GEMMs stream a few MB of packed weights per call, so the kernel is built around
// keeping many weight bytes in flight per SM, paying the set-up cost once per SM, and
// synchronising once per 16 KB of weights rather than once per k-block.  Warp roles (12 warps):
//   * warps 0 and 11, one lane each: PRODUCERS.  grid = min(#work items, #SMs); a work item = (128-row
//     weight tile, token tile, K split); each lane walks the CTA's items and keeps issuing TMA loads across
//     item and phase boundaries into a ring of STAGES.  A stage = KBS consecutive k-blocks: one
//     weight box of 128 rows x up to 128 bytes of codes (swizzled, warp 0) + the activation tiles of those
//     k-blocks (one 3-D box, warp 11).  Issuing one copy costs its lane several hundred cycles, hence a
//     lane per operand; the weight lane runs ahead of the grid barrier that the activation lane must
//     respect (weights are constants), so a phase's first weight boxes land before its activations exist;
//   * warps 2-9: DEQUANT, two groups of 4 sharing every stage (even / odd k-blocks).  A thread owns
//     one weight row: it reads the row's codes from shared memory, widens them to bf16 pairs in
//     registers (exact integers) and stores them with tcgen05.st straight into TENSOR MEMORY, where
//     they are the A operand of the MMA (M = 128 weight rows; K-major, two bf16 per 32-bit column)
//     - no shared-memory A tile, no generic->async proxy fence;
//   * warps 1 and 10, one lane each: MMA ISSUERS (A from TMEM, B = activation tile from shared
//     memory through a 128-byte-swizzle descriptor, N = token tile), each into its own accumulator
//     chain (see QLayout); one barrier per stage tells them that both operands are in place, one
//     commit per stage frees the stage's shared memory and A buffer;
//   * the 8 dequant warps run the epilogue from TMEM (one lane = one weight row): chains added,
//     scale, bias, store;
//   * split-K: every item stores its fp32 partial tile in a private slice of the workspace (plain
//     stores, no zero-fill needed).  When each CTA holds one item of the phase, the CTAs of a tile
//     meet at the tile's counter (one device-scope fence by the signalling thread, acquire polling)
//     and each sums its share of the token columns with all its slice loads in flight at once;
//     otherwise the last CTA to finish a tile sums all of it.  Slices are added in split order: a
//     deterministic result;
//   * a launch executes a PROGRAM of up to 4 phases separated by grid-wide barriers (all CTAs are
//     co-resident: grid <= #SMs, one CTA per SM, cooperative launch): the V and U factors of a
//     low-rank layer, or the whole gated MLP (gate|up V, gate|up U with SiLU(g)*u in the epilogue,
//     down V, down U), run in ONE launch; the rank-r intermediates never leave L2, and the
//     dequant warps already fill both A buffers of the next phase while the barrier is pending.
// Every mbarrier / grid-barrier wait is bounded (see tc_common.cuh); on expiry the CTA records a
// code in the status word, drains, frees its TMEM and returns.
#include <type_traits>
#include "tc_common.cuh"

namespace tsb {
using namespace tc;
namespace {

constexpr int kDqWarps = 8;                 // two groups of four
constexpr int kThreadsQ = 64 + kDqWarps * 32 + 64;   // weight producer, MMA issuer 0, 8 dequant warps, MMA issuer 1, activation producer
constexpr int kIssuer1Warp = 2 + kDqWarps;
constexpr int kXWarp = 3 + kDqWarps;
constexpr int kSmemBudget = 216 * 1024;     // three 72 KB stages of the 256-token tile (int4), six 32 KB stages of the decode tiles
constexpr unsigned kTmemCols = 512;

template <int TN, int BITS> struct QLayout {
  static constexpr int kKbsFull = 1024 / BITS / BK;        // k-blocks in a 128-byte row of codes
  // A buffer = KBS * 32 TMEM columns <= 128; 64- and 256-token tiles keep two k-blocks per stage (16 / 64 KB of activations)
  static constexpr int kKbsCap = (TN <= 32 || TN == 128) ? 4 : 2;
  // A buffers (KBS x 32 TMEM columns each) above the accumulators.  Token tiles up to 32 need at most 4 x 32 accumulator
  // columns (two chains, gate and up), the others 256.  As many buffers as fit (up to 4, and no more than ring stages):
  // the dequant warps then run NBUF - 1 stages ahead of the MMAs, and the chain "dequantize -> MMAs issued -> MMAs
  // complete -> buffer free" (traced at 256 tokens: 920 + 310 + 970 + 520 cycles per TWO stages with two buffers, i.e.
  // 685 cycles per k-block against 512 of the tensor pipe) no longer sets the pace of the main loop.
  static constexpr unsigned kACol0 = TN <= 32 ? 128 : 256;  // TMEM column of A buffer 0; buffer b at + kABufCols b
  static constexpr int KBS = kKbsFull < kKbsCap ? kKbsFull : kKbsCap;
  static constexpr int kRawRow = BK * BITS / 8;            // bytes of one weight row per k-block
  static constexpr int kRawStageRow = KBS * kRawRow;       // bytes of one weight row per stage (32/64/128)
  static constexpr int kRaw = BM * kRawStageRow;
  static constexpr int kXTile = TN * 128;
  static constexpr int kX = KBS * kXTile;
  static constexpr int kXRows = TN >= 128 ? 128 : TN;      // tokens per activation box
  static constexpr int kXPieces = TN / kXRows;             // boxes per k-block
  static constexpr int kXLanes = KBS * kXPieces;           // lanes that issue a stage's activation boxes together
  static constexpr int kStage = kX + kRaw;                 // multiple of 1024
  static constexpr int kNRraw = kSmemBudget / kStage;
  static constexpr int NR = kNRraw > 12 ? 12 : kNRraw;
  static constexpr int kABufCols = KBS * 32;
  static constexpr int kNBufFit = (512 - (int)kACol0) / kABufCols;
  static constexpr int NBUF = kNBufFit < NR ? (kNBufFit < 4 ? kNBufFit : 4) : (NR < 4 ? NR : 4);
  static_assert(NBUF >= 2 && kACol0 + NBUF * kABufCols <= 512, "tensor memory columns");
  static constexpr int kBarBytes = 1024;
  // Token tiles of 128 and more transpose their outputs through shared memory (16 tokens x 32 rows of bf16 per warp),
  // so that they leave as 16-byte stores instead of 2-byte stores
  static constexpr int kOutStage = TN >= 128 ? kDqWarps * 16 * 32 * 2 : 0;
  static constexpr int kBytes = NR * kStage + kBarBytes + kOutStage + 1024;
  static_assert(kBytes <= 227 * 1024, "shared memory of one CTA");
  // The tensor pipe needs ~55 + N/2 cycles per tcgen05.mma (the A operand is read from tensor memory), and
  // the lane that issues them spends another ~300-400 cycles per stage between its last MMA and the next
  // stage's first (commit, wait, descriptors) during which the pipe would idle.  Two lanes of different warps
  // therefore issue ALTERNATE STAGES, so one lane's gap hides behind the other's MMAs.  MMAs of different
  // threads are not ordered, so each lane accumulates into its own CHAIN (accumulator) and the epilogue adds
  // the chains.  Accumulators own tensor-memory columns [0, 256): chain c of a plain item at c * TN; of a
  // gated item gate at (2 c) * TN and up at (2 c + 1) * TN.
  // Narrow token tiles (decode: items of one to a few stages, 4 k-blocks per stage) instead split every stage
  // between the lanes by k-block parity, which also halves the latency of a single-stage item.
  static constexpr bool kTwoChains = 2 * TN <= 256;
  static constexpr bool kTwoChainsGated = 4 * TN <= 256;
  static constexpr bool kSplitStage = TN <= 32 && KBS >= 2;
  // The 256-token tile has one accumulator of 256 columns; its two halves are independent accumulators, so each lane
  // issues every stage's MMAs for ITS 128 tokens (N = 128: the lane's ~114 cycles per MMA cover 64 cycles of the pipe,
  // two lanes keep it busy; one lane issuing N = 256 needs 141-171 cycles per 128 cycles of the pipe)
  static constexpr bool kSplitTokens = TN == 256;
};

__device__ __forceinline__ uint4 lds128(unsigned addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(unsigned addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

// Shared address of 16-byte chunk `chunk` of weight row `row` inside a raw stage whose rows are RB
// bytes, written by the copy engine with the RB-byte swizzle (chunk index XOR a function of the row),
// so threads reading the same chunk of consecutive rows hit different banks.
template <int RB>
__device__ __forceinline__ unsigned raw_chunk(unsigned raw, int row, int chunk) {
  const int x = RB == 128 ? (row & 7) : (RB == 64 ? ((row >> 1) & 3) : (RB == 32 ? ((row >> 2) & 1) : 0));   // 16-byte rows: no swizzle
  return raw + row * RB + ((chunk ^ x) << 4);
}

// Widen the 64 codes of weight row `r`, k-block `sub` of the stage, to 32 registers of bf16 pairs:
// register c holds columns (2c, 2c+1) of the k-block - the TMEM A-operand packing.
template <int BITS, int RB>
__device__ __forceinline__ void dequant_row_regs(unsigned raw, int r, int sub, unsigned (&o)[32]) {
  if (BITS == 4) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint4 q = lds128(raw_chunk<RB>(raw, r, sub * 2 + h));
      const unsigned w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const unsigned t = w[c] ^ 0x88888888u;              // nibble + 8; 0x4300 | u = bf16(128 + u)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          o[h * 16 + c * 4 + j] = bf16x2_sub(((t >> (4 * j)) & 0x000f000fu) | 0x43004300u, 0x43084308u);
      }
    }
  } else if (BITS == 1) {
    // 8 bytes per k-block: word w covers columns 32 w .. 32 w + 31, bit i = column 2 i, bit 16 + i = column 2 i + 1,
    // so one shift brings the two bits of an output pair to bits 0 and 16; bit 1 -> +1.0, bit 0 -> -1.0 (the sign
    // bit of bf16 1.0 is the inverted code bit)
    const uint2 q = lds64(raw_chunk<RB>(raw, r, sub >> 1) + 8 * (sub & 1));
    const unsigned w[2] = {~q.x, ~q.y};
#pragma unroll
    for (int g = 0; g < 2; ++g)
#pragma unroll
      for (int j = 0; j < 16; ++j) o[g * 16 + j] = (((w[g] >> j) & 0x00010001u) << 15) | 0x3F803F80u;
  } else if (BITS == 2) {
    const uint4 q = lds128(raw_chunk<RB>(raw, r, sub));
    const unsigned w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const unsigned t = w[g] ^ 0xAAAAAAAAu;                // field + 2
#pragma unroll
      for (int j = 0; j < 8; ++j)
        o[g * 8 + j] = bf16x2_sub(((t >> (2 * j)) & 0x00030003u) | 0x43004300u, 0x43024302u);
    }
  } else {  // 8-bit, natural byte order
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint2 q = lds64(raw_chunk<RB>(raw, r, sub * 4 + (c >> 1)) + 8 * (c & 1));
      const unsigned t[2] = {q.x ^ 0x80808080u, q.y ^ 0x80808080u};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const unsigned tw = t[j >> 1];
        const float f0 = __uint_as_float(0x4B000000u | ((tw >> (16 * (j & 1))) & 0xffu)) - 8388736.0f;      // 2^23 + 128
        const float f1 = __uint_as_float(0x4B000000u | ((tw >> (16 * (j & 1) + 8)) & 0xffu)) - 8388736.0f;
        __nv_bfloat162 p = __floats2bfloat162_rn(f0, f1);
        o[c * 4 + j] = *reinterpret_cast<unsigned*>(&p);
      }
    }
  }
}

__device__ __forceinline__ void tmem_st32(unsigned taddr, const unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_ld8(unsigned taddr, unsigned (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
template <int W> __device__ __forceinline__ void tmem_ldw(unsigned taddr, unsigned (&r)[W]) {
  if constexpr (W == 16) tmem_ld16(taddr, r);
  else tmem_ld8(taddr, r);
}
// D[tmem] (+)= A[tmem] . B[smem descriptor]; kind::f16, A K-major in tensor memory.
__device__ __forceinline__ void umma_bf16_ts(unsigned d_tmem, unsigned a_tmem, unsigned long long bdesc, unsigned idesc,
                                             unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
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

// CNT token columns of one warp (32 weight rows) -> y, transposed through the warp's staging tile [CNT][32] bf16: lane
// `lane` deposits its CNT values, then every lane moves 16-byte pieces (8 consecutive rows of one token), so a token's
// 32 outputs leave as four 16-byte stores of one 64-byte run instead of 32 2-byte stores.  Slot j holds token column
// c_first + j * c_stride of the tile; columns beyond the tile or beyond M and row pieces beyond N (a multiple of 8) are
// skipped.  Warp-local: no other warp is waited for.
template <int CNT, int TN>
__device__ __forceinline__ void store_transposed(const float (&v)[CNT], __nv_bfloat16* sb, int lane, __nv_bfloat16* y, int64_t N, int64_t M,
                                                 int64_t n_warp0, int64_t m0, int c_first, int c_stride) {
#pragma unroll
  for (int j = 0; j < CNT; ++j) sb[j * 32 + lane] = __float2bfloat16_rn(v[j]);
  __syncwarp();
#pragma unroll
  for (int p = lane; p < CNT * 4; p += 32) {
    const int slot = p >> 2, part = p & 3;
    const int c = c_first + slot * c_stride;
    const int64_t m = m0 + c, nn = n_warp0 + part * 8;
    if (c < TN && m < M && nn < N) *reinterpret_cast<uint4*>(y + m * N + nn) = *reinterpret_cast<const uint4*>(sb + slot * 32 + part * 8);
  }
  __syncwarp();
}

constexpr int kMaxPhases = 4;

struct SubGemm {                 // one packed weight matrix and its operands
  CUtensorMap map_w;             // uint8 [N, row_bytes], box 128 rows x stage-row bytes, swizzled
  CUtensorMap map_x;             // bf16 [M, K]: box TN rows x 64, 128-byte swizzle; or (x3d) the 3-D view
                                 //    [K/64][M][64] with box (64, TN, KBS): one copy per stage
  const float* scale;            // [N]
  const __nv_bfloat16* bias;     // [N] or null
  __nv_bfloat16* y;              // [M, N]
};
struct Phase {
  SubGemm sub[2];
  int nsub;                      // 1, or 2 matrices of identical shape sharing the plan
  int gated;                     // 1: an item computes sub[0] (gate) and sub[1] (up) tiles and stores
                                 //    silu(gate) * up to sub[0].y; requires splits == 1 and TN <= 64
  int64_t N, K;
  int kb_total, kb_per_split, splits;
  int n_tiles, m_tiles, items_per_sub, items;
  float* partial;                // split-K: fp32 slices [items][TN][128] of this phase
  int* counters;                 // split-K: zero-filled int32 [nsub * n_tiles * m_tiles], left zero
  int x3d;                       // activations loaded with one 3-D box per stage (K a multiple of 64)
  int scatter;                   // split-K: 1 = every CTA holds at most one item of the phase and all CTAs are
                                 //    co-resident, so the CTAs of a tile wait for one another and each sums its
                                 //    share of the tile's columns; 0 = the last CTA to arrive sums the whole tile
};
struct Program {
  int64_t M;
  int n_phases;
  int* status;                   // workspace header: [0] status word
  int* grid_bar;                 // kMaxPhases barrier counters + 1 exit counter, zero between launches
  Phase ph[kMaxPhases];
};

// Bounded wait for `*ctr >= target` (another CTA's release increments).  False = gave up.
__device__ __forceinline__ bool grid_wait(const int* ctr, int target, volatile int* abort_flag) {
  for (unsigned i = 0; i < (1u << 22); ++i) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(v) : "l"(ctr) : "memory");
    if (v >= target) return true;
    if ((i & 63u) == 63u && *abort_flag) return false;
  }
  *abort_flag = 9;
  return false;
}

template <int TN, int BITS>
// 128 registers (not the 168 a 384-thread CTA could have): the CTA of a launch then fits beside the CTAs of the small
// kernel before it, so its set-up and first weight copies run under programmatic dependent launch while that kernel
// still executes.  With 168 registers the decode step was 4 % slower although this kernel alone was faster.
__global__ void __maxnreg__(128)
linear_tcq_kernel(const __grid_constant__ Program prog) {
  using L = QLayout<TN, BITS>;
  constexpr int NR = L::NR;
  constexpr int KBS = L::KBS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* r_ring = smem;                                   // NR x {KBS activation tiles, raw codes}
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(r_ring + NR * L::kStage);
  unsigned long long* w_full = bars;                        // [NR] weight box landed (the dequant warps wait on it)
  unsigned long long* x_full = bars + NR;                   // [NR] stage ready for the MMA lanes: activation tiles landed
                                                            //      (one arrival + bytes) AND the 8 dequant warps stored
                                                            //      its A operand - one wait per stage for the issuers
  unsigned long long* stage_done = bars + 2 * NR;           // [NR] MMA commit: the stage's MMAs are complete, so its
                                                            //      weight box, activation tiles and A buffer are free
  unsigned long long* acc_full = bars + 3 * NR;             // [1]  MMA commit: accumulator(s) of the item complete
  unsigned long long* ep_bar = acc_full + 1;                // [1]  rendezvous of the 8 warps
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(ep_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = abort_flag + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();

  // Work enumeration, identical in every role.  Phase -> items (round-robin over CTAs) -> passes
  // (one per matrix the item touches: 2 for a gated item) -> stages of KBS k-blocks.
  struct Item { int sub, nt, mt, kb0, nkb, ns; };        // ns = stages of the item's K range
  auto decode = [&](const Phase& ph, int item) {
    Item it;
    int local = item;
    it.sub = 0;
    if (!ph.gated && ph.nsub == 2 && item >= ph.items_per_sub) { it.sub = 1; local = item - ph.items_per_sub; }
    const int sp = local % ph.splits;
    const int t = local / ph.splits;
    it.nt = t % ph.n_tiles;
    it.mt = t / ph.n_tiles;
    it.kb0 = sp * ph.kb_per_split;
    it.nkb = min(ph.kb_per_split, ph.kb_total - it.kb0);
    it.ns = (it.nkb + KBS - 1) / KBS;
    return it;
  };

  int pre_w = 0;                                            // weight boxes issued during the set-up (thread 0)
  if (threadIdx.x == 0) {
    for (int i = 0; i < NR; ++i) { mbar_init(&w_full[i], 1); mbar_init(&x_full[i], 1 + kDqWarps); mbar_init(&stage_done[i], (L::kSplitStage || L::kSplitTokens) ? 2 : 1); }
    mbar_init(acc_full, 2);                                 // both issuers commit, with or without MMAs of their own
    mbar_init(ep_bar, kDqWarps);
    *abort_flag = 0;
    *last_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    // The first weight boxes of this CTA (first item of phase 0, first pass) leave NOW, before the tensor-memory
    // allocation and the CTA-wide barrier: their latency (cold translation, tensor-map fetch, DRAM: about 2 us) is the
    // head of every launch's critical path.  This thread is the weight producer: its loop below skips them.
    const Phase& ph0 = prog.ph[0];
    if ((int)blockIdx.x < ph0.items) {
      const Item it = decode(ph0, blockIdx.x);
      const SubGemm& sg = ph0.sub[ph0.gated ? 0 : it.sub];
      for (; pre_w < it.ns && pre_w < NR; ++pre_w) {
        mbar_expect_tx(&w_full[pre_w], (unsigned)L::kRaw);
        tma_load_2d(r_ring + pre_w * L::kStage + L::kX, &sg.map_w, (it.kb0 + pre_w * KBS) * (BK * BITS / 8), it.nt * BM, &w_full[pre_w]);
      }
    }
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer: packed weights
    // The codes are constants, so this lane never waits for another kernel or phase: it keeps the ring full
    // across item and phase boundaries, limited only by free stages.  (One lane needs several hundred cycles to
    // issue one copy; weights and activations therefore have a lane each, in different warps.)
    if (lane == 0) {
      bool ok = true;
      int gs = 0;                                             // absolute stage counter
#pragma unroll 1
      for (int p = 0; p < prog.n_phases && ok; ++p) {
        const Phase& ph = prog.ph[p];
        for (int j = 0; j < ph.nsub; ++j) asm volatile("prefetch.tensormap [%0];\n" ::"l"(&ph.sub[j].map_w) : "memory");
        const int passes = ph.gated ? 2 : 1;
#pragma unroll 1
        for (int item = blockIdx.x; item < ph.items && ok; item += gridDim.x) {
          const Item it = decode(ph, item);
#pragma unroll 1
          for (int ps = 0; ps < passes && ok; ++ps) {
            const SubGemm& sg = ph.sub[ph.gated ? ps : it.sub];
#pragma unroll 1
            for (int jj = 0; jj < it.ns; ++jj, ++gs) {
              const int s = gs % NR, kb = it.kb0 + jj * KBS;
              if (gs < pre_w) continue;                        // issued during the set-up
              // the stage is free once its previous user's MMAs are complete
              if (gs >= NR && !mbar_wait(&stage_done[s], ((gs / NR) - 1) & 1, abort_flag, 1)) { ok = false; break; }
              mbar_expect_tx(&w_full[s], (unsigned)L::kRaw);
              tma_load_2d(r_ring + s * L::kStage + L::kX, &sg.map_w, kb * (BK * BITS / 8), it.nt * BM, &w_full[s]);
            }
          }
        }
      }
    }
  } else if (warp == kXWarp) {
    // ---------------------------------------------------------------- TMA producer: activations
    // Same stage sequence; a phase's activations exist once the preceding kernel (phase 0) or the previous phase
    // (grid barrier) has produced them.
    // One lane issues ~23 bytes per cycle whatever the box (measured, data resident in L2), lanes of one warp that
    // execute the copy instruction together issue side by side (4 lanes: 71 bytes per cycle).  Token tiles of 128 and
    // more therefore fetch a stage as kXLanes boxes of 128 tokens x one k-block from as many lanes; the waits stay
    // with lane 0 and their outcome is broadcast, so the warp runs the loop convergently.
    if constexpr (TN >= 128) {
        bool ok = true;
        int gs = 0;
#pragma unroll 1
        for (int p = 0; p < prog.n_phases && ok; ++p) {
          const Phase& ph = prog.ph[p];
          if (lane == 0)
            for (int j = 0; j < ph.nsub; ++j) asm volatile("prefetch.tensormap [%0];\n" ::"l"(&ph.sub[j].map_x) : "memory");
          if (p == 0) {
            pdl_wait();
          } else {
            if (lane == 0) ok = grid_wait(&prog.grid_bar[p - 1], (int)gridDim.x, abort_flag);
            ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
            asm volatile("fence.proxy.async;\n" ::: "memory");  // other CTAs' stores -> visible to the copy engine
          }
          const int passes = ph.gated ? 2 : 1;
#pragma unroll 1
          for (int item = blockIdx.x; item < ph.items && ok; item += gridDim.x) {
            const Item it = decode(ph, item);
#pragma unroll 1
            for (int ps = 0; ps < passes && ok; ++ps) {
              const SubGemm& sg = ph.sub[ph.gated ? ps : it.sub];
#pragma unroll 1
              for (int jj = 0; jj < it.ns; ++jj, ++gs) {
                const int s = gs % NR, kb = it.kb0 + jj * KBS;
                if (lane == 0) {
                  if (gs >= NR) ok = mbar_wait(&stage_done[s], ((gs / NR) - 1) & 1, abort_flag, 1);
                  if (ok) mbar_expect_tx(&x_full[s], (unsigned)L::kX);
                }
                ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;   // also orders the expected byte count before the copies
                if (!ok) break;
                uint8_t* st = r_ring + s * L::kStage;
                if constexpr (TN >= 128) {                      // rows beyond M and columns beyond K are zero-filled
                  if (lane < L::kXLanes) {
                    const int j = lane / L::kXPieces, q = lane % L::kXPieces;
                    tma_load_2d(st + j * L::kXTile + q * (L::kXRows * 128), &sg.map_x, (kb + j) * BK, it.mt * TN + q * L::kXRows, &x_full[s]);
                  }
                } else if (lane == 0) {
                  if (ph.x3d) {                                 // k-blocks beyond K are zero-filled by the copy engine
                    tma_load_3d(st, &sg.map_x, 0, it.mt * TN, kb, &x_full[s]);
                  } else {
#pragma unroll 1
                    for (int j = 0; j < KBS; ++j)               // columns beyond K are zero-filled by the copy engine
                      tma_load_2d(st + j * L::kXTile, &sg.map_x, (kb + j) * BK, it.mt * TN, &x_full[s]);
                  }
                }
              }
            }
          }
        }
    } else {
      if (lane == 0) {
        bool ok = true;
        int gs = 0;
#pragma unroll 1
        for (int p = 0; p < prog.n_phases && ok; ++p) {
          const Phase& ph = prog.ph[p];
          for (int j = 0; j < ph.nsub; ++j) asm volatile("prefetch.tensormap [%0];\n" ::"l"(&ph.sub[j].map_x) : "memory");
          if (p == 0) {
            pdl_wait();
          } else {
            ok = grid_wait(&prog.grid_bar[p - 1], (int)gridDim.x, abort_flag);
            asm volatile("fence.proxy.async;\n" ::: "memory");  // other CTAs' stores -> visible to the copy engine
          }
          const int passes = ph.gated ? 2 : 1;
#pragma unroll 1
          for (int item = blockIdx.x; item < ph.items && ok; item += gridDim.x) {
            const Item it = decode(ph, item);
#pragma unroll 1
            for (int ps = 0; ps < passes && ok; ++ps) {
              const SubGemm& sg = ph.sub[ph.gated ? ps : it.sub];
#pragma unroll 1
              for (int jj = 0; jj < it.ns; ++jj, ++gs) {
                const int s = gs % NR, kb = it.kb0 + jj * KBS;
                if (gs >= NR && !mbar_wait(&stage_done[s], ((gs / NR) - 1) & 1, abort_flag, 1)) { ok = false; break; }
                uint8_t* st = r_ring + s * L::kStage;
                mbar_expect_tx(&x_full[s], (unsigned)L::kX);
                if (ph.x3d) {                                   // k-blocks beyond K are zero-filled by the copy engine
                  tma_load_3d(st, &sg.map_x, 0, it.mt * TN, kb, &x_full[s]);
                } else {
#pragma unroll 1
                  for (int j = 0; j < KBS; ++j)                 // columns beyond K are zero-filled by the copy engine
                    tma_load_2d(st + j * L::kXTile, &sg.map_x, (kb + j) * BK, it.mt * TN, &x_full[s]);
                }
              }
            }
          }
        }
      }
    }
  } else if (warp == 1 || warp == kIssuer1Warp) {
    // ---------------------------------------------------------------- MMA issuers
    if (lane == 0) {
      const int me = warp == 1 ? 0 : 1;                       // issuer 0: even stages / chain 0; issuer 1: odd stages / chain 1
      constexpr unsigned idesc = idesc_bf16(L::kSplitTokens ? TN / 2 : TN);
      int gs = 0;
      bool ok = true;
      for (int p = 0; p < prog.n_phases && ok; ++p) {
        const Phase& ph = prog.ph[p];
        const bool two = ph.gated ? L::kTwoChainsGated : L::kTwoChains;
        for (int item = blockIdx.x; item < ph.items && ok; item += gridDim.x) {
          const Item it = decode(ph, item);
          const int passes = ph.gated ? 2 : 1;
          for (int ps = 0; ps < passes && ok; ++ps) {
            const unsigned d_tmem = L::kSplitTokens ? tmem_base + (unsigned)(me * (TN / 2))
                                                    : tmem_base + (unsigned)((ph.gated ? 2 * (two ? me : 0) + ps : (two ? me : 0)) * TN);
            bool first = true;                                // the chain's first MMA of the pass overwrites
            for (int jj = 0; jj < it.ns; ++jj, ++gs) {
              if (!L::kSplitStage && !L::kSplitTokens && (two ? (gs & 1) != me : me != 0)) {   // the other lane's stage
                // a lane without any stage in this pass (single chain) still commits the item below: it follows the
                // stages one by one (a parity wait is only meaningful in order), so that its arrival cannot fall into
                // the previous item's phase of the accumulator barrier
                if (!two) ok = mbar_wait(&x_full[gs % NR], (gs / NR) & 1, abort_flag, 2);
                continue;
              }
              const int i = jj * KBS;
              const int s = gs % NR, buf = gs % L::NBUF;
              ok = mbar_wait(&x_full[s], (gs / NR) & 1, abort_flag, 2);
              if (!ok) break;
              tc_fence_after();
              const unsigned a_tmem = tmem_base + L::kACol0 + buf * L::kABufCols;
              const unsigned x_base = smem_u32(r_ring + s * L::kStage) + (L::kSplitTokens ? me * (TN / 2) * 128 : 0);   // this lane's tokens
              const int nsub = min(KBS, it.nkb - i);
              const bool halves = L::kSplitStage && two;      // this lane takes the k-blocks of its parity
              for (int j = halves ? me : 0; j < nsub && (!L::kSplitStage || two || me == 0); j += halves ? 2 : 1) {
                const unsigned long long bdesc = smem_desc_sw128(x_base + j * L::kXTile);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k) { // A: 8 TMEM columns per K=16; B: +32 bytes inside the swizzle atom
                  umma_bf16_ts(d_tmem, a_tmem + j * 32 + k * 8, bdesc + 2 * k, idesc, first ? 0u : 1u);
                  first = false;
                }
              }
              umma_commit(&stage_done[s]);                     // arrives once the stage's MMAs are complete
            }
          }
          if (ok) umma_commit(acc_full);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- dequant + epilogue
    const int grp = (warp - 2) >> 2;                         // dequant group 0 / 1: k-blocks of that parity in every stage
    const int q = warp & 3;                                  // TMEM lane quarter this warp may access
    const int row = q * 32 + lane;                           // weight row within the tile = TMEM lane
    const unsigned lane_addr = tmem_base + ((unsigned)(q * 32) << 16);
    int gs = 0, it_count = 0, ep_uses = 0;
    __nv_bfloat16* out_stage = reinterpret_cast<__nv_bfloat16*>(r_ring + NR * L::kStage + L::kBarBytes) + (warp - 2) * (16 * 32);   // this warp's
    bool ok = true;
    bool waited = false;
    for (int p = 0; p < prog.n_phases && ok; ++p) {
      const Phase& ph = prog.ph[p];
      for (int item = blockIdx.x; item < ph.items && ok; item += gridDim.x, ++it_count) {
        const Item it = decode(ph, item);
        const int passes = ph.gated ? 2 : 1;
        // per-row epilogue constants (weights-side data): requested now, consumed after the main loop
        const int64_t n = (int64_t)it.nt * BM + row;
        const SubGemm& sg0 = ph.sub[ph.gated ? 0 : it.sub];
        const float sc0 = n < ph.N ? __ldg(&sg0.scale[n]) : 1.0f;
        const float bv0 = (sg0.bias && n < ph.N) ? __bfloat162float(sg0.bias[n]) : 0.f;
        float sc1 = 1.0f, bv1 = 0.f;
        if (ph.gated) {
          sc1 = n < ph.N ? __ldg(&ph.sub[1].scale[n]) : 1.0f;
          bv1 = (ph.sub[1].bias && n < ph.N) ? __bfloat162float(ph.sub[1].bias[n]) : 0.f;
        }
        for (int ps = 0; ps < passes && ok; ++ps) {
          for (int jj = 0; jj < it.ns; ++jj, ++gs) {
            const int i = jj * KBS;
            const int s = gs % NR, buf = gs % L::NBUF;
            ok = mbar_wait_relaxed(&w_full[s], (gs / NR) & 1, abort_flag, 4);
            // the A buffer is free once the MMAs of the stage NBUF back are complete
            if (ok && gs >= L::NBUF) ok = mbar_wait_relaxed(&stage_done[(gs - L::NBUF) % NR], ((gs - L::NBUF) / NR) & 1, abort_flag, 5);
            if (!ok) break;
            tc_fence_after();
            const unsigned raw = smem_u32(r_ring + s * L::kStage + L::kX);
            const int nsub = min(KBS, it.nkb - i);
            for (int j = grp; j < nsub; j += 2) {              // both groups work on the stage: half the latency
              unsigned regs[32];
              dequant_row_regs<BITS, L::kRawStageRow>(raw, row, j, regs);
              tmem_st32(lane_addr + L::kACol0 + buf * L::kABufCols + j * 32, regs);
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&x_full[s]);
          }
        }
        if (!ok) break;
        ok = mbar_wait_relaxed(acc_full, it_count & 1, abort_flag, 6);
        if (!ok) break;
        tc_fence_after();
        if (!waited) { pdl_wait(); waited = true; }          // outputs / scratch may still be in use upstream
        const int64_t m0 = (int64_t)it.mt * TN;
        const bool split = ph.splits > 1;
        constexpr int CH = TN / 2;                           // token columns handled by this warp
        // accumulator chains: with two issuers chain c holds the stages of parity c; a pass of a single stage
        // leaves the other chain unwritten.  g0 = first stage of the (gate) pass, g0u = of the up pass.
        const bool two = ph.gated ? L::kTwoChainsGated : L::kTwoChains;
        const int g0 = gs - passes * it.ns, g0u = gs - it.ns;
        const bool v0 = L::kSplitStage || !two || it.ns >= 2 || (g0 & 1) == 0;
        const bool v1 = two && (L::kSplitStage ? it.nkb >= 2 : (it.ns >= 2 || (g0 & 1) == 1));
        const bool u0 = L::kSplitStage || !two || it.ns >= 2 || (g0u & 1) == 0;
        const bool u1 = two && (L::kSplitStage ? it.nkb >= 2 : (it.ns >= 2 || (g0u & 1) == 1));
        const unsigned acc1 = (unsigned)((ph.gated ? 2 : 1) * TN);   // column offset of chain 1
        float* slice = ph.partial + (size_t)item * (TN * BM);
        __nv_bfloat16* y = sg0.y;
        // outputs through the staging tile: token tiles of 128 and more, rows of y 16-byte aligned
        const bool vec = TN >= 128 && ph.N % 8 == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0;
        // W columns per step, the tensor-memory loads of both chains issued before one wait (a tcgen05.ld costs its
        // warp ~115 cycles to issue whatever its width, so few wide loads, not many narrow ones); a gated item first
        // turns the gate columns into SiLU(g), then fetches the up columns into the freed registers
        constexpr int W = CH >= 16 ? 16 : 8;
#pragma unroll 1
        for (int c0 = grp * CH; c0 < (grp + 1) * CH; c0 += W) {
          unsigned r[W], t[W];
          tmem_ldw<W>(lane_addr + (v0 ? 0u : acc1) + (unsigned)c0, r);
          if (v0 && v1) tmem_ldw<W>(lane_addr + acc1 + (unsigned)c0, t);
          tmem_ld_wait();
          if (v0 && v1) {
#pragma unroll
            for (int j = 0; j < W; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(t[j]));
          }
          if (ph.gated) {
            // same rounding points as separate gate / up / SiLU*up kernels (blocks/mlp.py:181-183)
#pragma unroll
            for (int j = 0; j < W; ++j) {
              const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[j]) * sc0 + bv0));
              r[j] = __float_as_uint(__bfloat162float(__float2bfloat16_rn(__fdividef(g, 1.0f + __expf(-g)))));
            }
            tmem_ldw<W>(lane_addr + (u0 ? 0u : acc1) + (unsigned)(TN + c0), t);
            unsigned t2[W];
            if (u0 && u1) tmem_ldw<W>(lane_addr + acc1 + (unsigned)(TN + c0), t2);
            tmem_ld_wait();
            if (u0 && u1) {
#pragma unroll
              for (int j = 0; j < W; ++j) t[j] = __float_as_uint(__uint_as_float(t[j]) + __uint_as_float(t2[j]));
            }
            if (n < ph.N) {
#pragma unroll
              for (int j = 0; j < W; ++j) {
                const int64_t m = m0 + c0 + j;
                if (m < prog.M) {
                  const float u = __bfloat162float(__float2bfloat16_rn(__uint_as_float(t[j]) * sc1 + bv1));
                  y[m * ph.N + n] = __float2bfloat16_rn(__fmul_rn(__uint_as_float(r[j]), u));
                }
              }
            }
          } else if (split) {
#pragma unroll
            for (int j = 0; j < W; ++j) __stcg(&slice[(c0 + j) * BM + row], __uint_as_float(r[j]));
          } else {
            if constexpr (TN >= 128) {
              if (vec) {
                float v[W];
#pragma unroll
                for (int j = 0; j < W; ++j) v[j] = __uint_as_float(r[j]) * sc0 + bv0;
                store_transposed<W, TN>(v, out_stage, lane, y, ph.N, prog.M, (int64_t)it.nt * BM + q * 32, m0, c0, 1);
                continue;
              }
            }
            if (n < ph.N) {
#pragma unroll
              for (int j = 0; j < W; ++j) {
                const int64_t m = m0 + c0 + j;
                if (m < prog.M) y[m * ph.N + n] = __float2bfloat16_rn(__uint_as_float(r[j]) * sc0 + bv0);
              }
            }
          }
        }
        tc_fence_before();
        // every warp is done reading the accumulator before any warp stores the next item's A operand
        if (!(ok = warps_rendezvous(ep_bar, ep_uses, lane, abort_flag))) break;
        if (split && ph.scatter) {
          // The CTAs of this (matrix, n tile, m tile) meet at the tile's counter; CTA `sp` then sums token
          // columns sp, sp + splits, ... over all slices in split order (the order the single-finalizer
          // path uses), with every load of a column in flight at once.
          int* ctr = &ph.counters[(it.sub * ph.m_tiles + it.mt) * ph.n_tiles + it.nt];
          if (threadIdx.x == 64) {
            // one device-scope fence by the signalling thread: the slice stores of the other epilogue threads are
            // ordered before it by the rendezvous above, and the fence is cumulative
            __threadfence();
            atomicAdd(ctr, 1);
            grid_wait(ctr, ph.splits, abort_flag);             // acquire loads; failure raises the abort flag
            // departure: the counter counts `splits` arrivals, then `splits` departures, and the last departure wraps
            // it to 0 for the next launch (a CTA departs only after it has seen every arrival; nothing waits for the
            // departures, and the increment returns nothing, so neither does this thread)
            atomicInc(reinterpret_cast<unsigned*>(ctr), 2u * (unsigned)ph.splits - 1u);
          }
          if (!(ok = warps_rendezvous(ep_bar, ep_uses, lane, abort_flag))) break;
          if (*abort_flag) { ok = false; break; }
          // the slices are read with L2 loads (ld.global.cg) after that acquire and the rendezvous: no further fence
          const int sp = item % ph.splits;
          if constexpr (TN >= 128) {
            {
              const float* tile0 = ph.partial + (size_t)(item - sp) * (TN * BM) + row;
              // all of this thread's columns and slices in flight at once (up to 16 x 2, 8 x 4, 4 x 8 or 2 x 16 loads; a round trip to freshly written slices costs ~2200 cycles, and 64 loads
              // per thread spill under the 128-register cap): one round
              // trip to the L2 instead of one per column.  A column's slices are added in split order.  (Rows beyond N exist in
              // the slices and are summed like the others; they are never stored.)
              const int cstep = 2 * ph.splits;
              auto batch = [&](auto cb_c, auto sb_c) -> bool {
                constexpr int CB = decltype(cb_c)::value, SB = decltype(sb_c)::value;
                for (int cb = sp + grp * ph.splits; cb < TN; cb += CB * cstep) {
                  float v[CB];
#pragma unroll
                  for (int u = 0; u < CB; ++u) v[u] = 0.f;
                  for (int s0 = 0; s0 < ph.splits; s0 += SB) {
                    float a[CB][SB];
#pragma unroll
                    for (int u = 0; u < CB; ++u)
#pragma unroll
                      for (int t = 0; t < SB; ++t)
                        a[u][t] = (cb + u * cstep < TN && s0 + t < ph.splits)
                                      ? __ldcg(tile0 + (size_t)(s0 + t) * (TN * BM) + (cb + u * cstep) * BM) : 0.f;
#pragma unroll
                    for (int u = 0; u < CB; ++u)
#pragma unroll
                      for (int t = 0; t < SB; ++t)
                        if (s0 + t < ph.splits) v[u] += a[u][t];
                  }
                  if constexpr (CB >= 8) {
                    if (vec) {
#pragma unroll
                      for (int u = 0; u < CB; ++u) v[u] = v[u] * sc0 + bv0;
                      constexpr int CS = CB < 16 ? CB : 16;      // the staging tile holds 16 token columns
#pragma unroll
                      for (int h = 0; h < CB / CS; ++h)
                        store_transposed<CS, TN>(*reinterpret_cast<const float(*)[CS]>(&v[h * CS]), out_stage, lane, y, ph.N, prog.M,
                                                 (int64_t)it.nt * BM + q * 32, m0, cb + h * CS * cstep, cstep);
                      continue;
                    }
                  }
                  if (n < ph.N) {
#pragma unroll
                    for (int u = 0; u < CB; ++u) {
                      const int c = cb + u * cstep;
                      const int64_t m = m0 + c;
                      if (c < TN && m < prog.M) y[m * ph.N + n] = __float2bfloat16_rn(v[u] * sc0 + bv0);
                    }
                  }
                }
                return true;
              };
              if (ph.splits <= 2) ok = batch(std::integral_constant<int, 16>{}, std::integral_constant<int, 2>{});
              else if (ph.splits <= 4) ok = batch(std::integral_constant<int, 8>{}, std::integral_constant<int, 4>{});
              else if (ph.splits <= 8) ok = batch(std::integral_constant<int, 4>{}, std::integral_constant<int, 8>{});
              else ok = batch(std::integral_constant<int, 2>{}, std::integral_constant<int, 16>{});
              if (!ok) break;
            }
          } else {
            if (n < ph.N) {
              const float* tile0 = ph.partial + (size_t)(item - sp) * (TN * BM) + row;
              // all of this thread's columns and slices in flight at once (up to 8 x 4, 4 x 8 or 2 x 16 loads): one round trip
              // to the L2 instead of one per column.  A column's slices are added in split order.
              const int cstep = 2 * ph.splits;
              auto batch = [&](auto cb_c, auto sb_c) {
                constexpr int CB = decltype(cb_c)::value, SB = decltype(sb_c)::value;
                for (int cb = sp + grp * ph.splits; cb < TN; cb += CB * cstep) {
                  float v[CB];
#pragma unroll
                  for (int u = 0; u < CB; ++u) v[u] = 0.f;
                  for (int s0 = 0; s0 < ph.splits; s0 += SB) {
                    float a[CB][SB];
#pragma unroll
                    for (int u = 0; u < CB; ++u)
#pragma unroll
                      for (int t = 0; t < SB; ++t)
                        a[u][t] = (cb + u * cstep < TN && s0 + t < ph.splits)
                                      ? __ldcg(tile0 + (size_t)(s0 + t) * (TN * BM) + (cb + u * cstep) * BM) : 0.f;
#pragma unroll
                    for (int u = 0; u < CB; ++u)
#pragma unroll
                      for (int t = 0; t < SB; ++t)
                        if (s0 + t < ph.splits) v[u] += a[u][t];
                  }
#pragma unroll
                  for (int u = 0; u < CB; ++u) {
                    const int c = cb + u * cstep;
                    const int64_t m = m0 + c;
                    if (c < TN && m < prog.M) y[m * ph.N + n] = __float2bfloat16_rn(v[u] * sc0 + bv0);
                  }
                }
              };
              if (ph.splits <= 4) batch(std::integral_constant<int, 8>{}, std::integral_constant<int, 4>{});
              else if (ph.splits <= 8) batch(std::integral_constant<int, 4>{}, std::integral_constant<int, 8>{});
              else batch(std::integral_constant<int, 2>{}, std::integral_constant<int, 16>{});
            }
          }
        } else if (split) {
          // last CTA of this (matrix, n tile, m tile) finalizes: sum of the slices -> y, then resets the counter
          int* ctr = &ph.counters[(it.sub * ph.m_tiles + it.mt) * ph.n_tiles + it.nt];
          __threadfence();
          if (!(ok = warps_rendezvous(ep_bar, ep_uses, lane, abort_flag))) break;
          if (threadIdx.x == 64) *last_flag = (atomicAdd(ctr, 1) == ph.splits - 1);
          if (!(ok = warps_rendezvous(ep_bar, ep_uses, lane, abort_flag))) break;
          const bool last = *last_flag != 0;
          if (last) {
            __threadfence();
            if (n < ph.N) {
              const float* tile0 = ph.partial + (size_t)(item - item % ph.splits) * (TN * BM) + row;
              // 8 token columns at a time, 4 splits in flight; splits are added in index order, so the
              // result does not depend on arrival order
              for (int c0 = grp * CH; c0 < (grp + 1) * CH; c0 += 8) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = 0.f;
                int sp = 0;
                for (; sp + 4 <= ph.splits; sp += 4) {
                  float a[4][8];
#pragma unroll
                  for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int j = 0; j < 8; ++j) a[u][j] = __ldcg(tile0 + (size_t)(sp + u) * (TN * BM) + (c0 + j) * BM);
#pragma unroll
                  for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] += a[u][j];
                }
                for (; sp < ph.splits; ++sp) {
                  float a[8];
#pragma unroll
                  for (int j = 0; j < 8; ++j) a[j] = __ldcg(tile0 + (size_t)sp * (TN * BM) + (c0 + j) * BM);
#pragma unroll
                  for (int j = 0; j < 8; ++j) v[j] += a[j];
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const int64_t m = m0 + c0 + j;
                  if (m < prog.M) y[m * ph.N + n] = __float2bfloat16_rn(v[j] * sc0 + bv0);
                }
              }
            }
            if (threadIdx.x == 64) *ctr = 0;
          }
          if (!(ok = warps_rendezvous(ep_bar, ep_uses, lane, abort_flag))) break;   // last_flag is reused by the next item
        }
        tc_fence_after();
      }
      if (!ok) break;
      // ---- end of phase: publish this CTA's outputs, then signal the grid barrier ------------------
      if (p + 1 < prog.n_phases) {
        if (!waited) { pdl_wait(); waited = true; }
        asm volatile("fence.proxy.async;\n" ::: "memory");    // generic stores -> visible to other CTAs' copy engines
        if (!(ok = warps_rendezvous(ep_bar, ep_uses, lane, abort_flag))) break;
        if (threadIdx.x == 64) {
          // one device-scope fence by the signalling thread: the stores of the other epilogue threads are ordered
          // before it by the rendezvous, and the fence is cumulative
          __threadfence();
          atomicAdd(&prog.grid_bar[p], 1);
        }
      }
    }
  }
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);         // error path: let copies in flight land
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0) {
    if (*abort_flag) atomicMax(prog.status, *abort_flag);
    if (prog.n_phases > 1) {
      // the last CTA to leave resets the grid-barrier counters for the next launch
      __threadfence();
      if (atomicAdd(&prog.grid_bar[kMaxPhases], 1) == (int)gridDim.x - 1) {
        for (int i = 0; i <= kMaxPhases; ++i) prog.grid_bar[i] = 0;
      }
    }
  }
}

}  // namespace
}  // namespace tsb

namespace tsb {
namespace {

template <int TN, int BITS>
int launch_q(const Program& prog, int grid, bool coresident, cudaStream_t s) {
  using L = QLayout<TN, BITS>;
  static bool configured[64] = {false};
  int dev = 0;
  TSB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return TSB200_ERR_DEVICE;
  if (!configured[dev]) {
    TSB_CUDA(cudaFuncSetAttribute(linear_tcq_kernel<TN, BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes));
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kThreadsQ);
  cfg.dynamicSmemBytes = (size_t)L::kBytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (coresident) {            // grid barriers / tile rendezvous: every CTA must be resident at once
    attr[na].id = cudaLaunchAttributeCooperative;
    attr[na].val.cooperative = 1;
    ++na;
  }
  if (g_pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, linear_tcq_kernel<TN, BITS>, prog);
  if (e != cudaSuccess && na == 2) {   // the two attributes are not accepted together: keep co-residency
    (void)cudaGetLastError();
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, linear_tcq_kernel<TN, BITS>, prog);
  }
  TSB_CUDA(e);
  return TSB200_OK;
}

template <int TN>
int launch_q_bits(int bits, const Program& prog, int grid, bool coresident, cudaStream_t s) {
  switch (bits) {
    case 1: return launch_q<TN, 1>(prog, grid, coresident, s);
    case 2: return launch_q<TN, 2>(prog, grid, coresident, s);
    case 4: return launch_q<TN, 4>(prog, grid, coresident, s);
    case 8: return launch_q<TN, 8>(prog, grid, coresident, s);
    default: return TSB200_ERR_UNSUPPORTED;
  }
}

// Inner extent (bytes) of the weight box: must equal QLayout<TN, BITS>::kRawStageRow.
int raw_box_bytes(int tn, int bits) {
  const int full = 1024 / bits / BK;
  const int cap = (tn <= 32 || tn == 128) ? 4 : 2;
  const int kbs = full < cap ? full : cap;
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

// k-blocks per stage: must equal QLayout<TN, BITS>::KBS
int stage_kbs(int tn, int bits) { return raw_box_bytes(tn, bits) / (BK * bits / 8); }

bool fill_sub(SubGemm& sg, const GemmSpec& g, int64_t M, int tn, int bits, bool x3d) {
  const uint64_t rb = tsb200_packed_row_bytes(g.K, bits);
  const int box = raw_box_bytes(tn, bits);
  const CUtensorMapSwizzle sw = box == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                : (box == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : (box == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE));
  if (!make_map(&sg.map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, g.W, rb, (uint64_t)g.N, rb, (uint32_t)box, BM, sw)) return false;
  if (tn >= 128) {                                                     // boxes of 128 tokens x one k-block, one per lane
    if (!make_map(&sg.map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, g.x, (uint64_t)g.K, (uint64_t)M, (uint64_t)g.K * 2, BK, 128,
                  CU_TENSOR_MAP_SWIZZLE_128B))
      return false;
  } else if (x3d) {
    if (!make_map_x3d(&sg.map_x, g.x, (uint64_t)g.K, (uint64_t)M, (uint32_t)tn, (uint32_t)stage_kbs(tn, bits))) return false;
  } else if (!make_map(&sg.map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, g.x, (uint64_t)g.K, (uint64_t)M, (uint64_t)g.K * 2, BK,
                       (uint32_t)tn, CU_TENSOR_MAP_SWIZZLE_128B)) {
    return false;
  }
  sg.scale = g.scale;
  sg.bias = (const __nv_bfloat16*)g.bias;
  sg.y = (__nv_bfloat16*)g.y;
  return true;
}

}  // namespace

size_t phase_scratch_bytes(int64_t M, int64_t N, int64_t K, int nsub, bool gated) {
  return plan_gemm(M, N, K, nsub, gated).slice_bytes;
}

// Run a program of phases in one launch.  All matrices packed at `bits`; bf16 activations.
// scratch: split-K slices (sum over phases of phase_scratch_bytes); counters / grid_bar / status:
// the zero-filled workspace header.
int run_program_tcq(const PhaseSpec* specs, int n_phases, int bits, int64_t M, uint8_t* scratch, int* counters, int* grid_bar,
                    int* status, cudaStream_t s) {
  if (n_phases < 1 || n_phases > kMaxPhases) return TSB200_ERR_ARG;
  Program prog;
  prog.M = M;
  prog.n_phases = n_phases;
  prog.status = status;
  prog.grid_bar = grid_bar;
  int tn = 0, max_items = 0, ctr_off = 0;
  size_t sc_off = 0;
  for (int p = 0; p < n_phases; ++p) {
    const PhaseSpec& ps = specs[p];
    Phase& ph = prog.ph[p];
    const GemmPlan g = plan_gemm(M, ps.g[0].N, ps.g[0].K, ps.gated ? 1 : ps.nsub, ps.gated != 0, bits == 1 ? 2 : 1);
    if (p == 0) tn = g.tn;
    if (ps.gated && (g.tn > 64 || ps.nsub != 2)) return TSB200_ERR_UNSUPPORTED;
    ph.nsub = ps.nsub;
    ph.gated = ps.gated;
    ph.N = ps.g[0].N;
    ph.K = ps.g[0].K;
    ph.kb_total = g.kb_total;
    ph.kb_per_split = g.kb_per_split;
    ph.splits = g.splits;
    ph.n_tiles = g.n_tiles;
    ph.m_tiles = g.m_tiles;
    ph.items = g.items;
    ph.items_per_sub = ps.gated ? g.items : g.items / ps.nsub;
    ph.x3d = (ph.K % BK == 0) ? 1 : 0;
    for (int j = 0; j < ps.nsub; ++j) {
      if (ps.g[j].N != ph.N || ps.g[j].K != ph.K) return TSB200_ERR_ARG;
      if (!fill_sub(ph.sub[j], ps.g[j], M, g.tn, bits, ph.x3d != 0)) return TSB200_ERR_CUDA;
    }
    const int tiles = ps.nsub * g.n_tiles * g.m_tiles;
    if (g.splits > 1 && ctr_off + tiles > kMaxCounters) return TSB200_ERR_UNSUPPORTED;
    ph.counters = counters + ctr_off;
    ph.partial = (float*)(scratch + sc_off);
    if (g.splits > 1) { ctr_off += tiles; sc_off += g.slice_bytes; }
    if (g.items > max_items) max_items = g.items;
  }
  const int sms = num_sms();
  const int grid = max_items < sms ? max_items : sms;
  bool coresident = n_phases > 1;
  for (int p = 0; p < n_phases; ++p) {
    Phase& ph = prog.ph[p];
    ph.scatter = (ph.splits > 1 && ph.items <= grid) ? 1 : 0;
    coresident = coresident || ph.scatter;
  }
  switch (tn) {
    case 16: return launch_q_bits<16>(bits, prog, grid, coresident, s);
    case 32: return launch_q_bits<32>(bits, prog, grid, coresident, s);
    case 64: return launch_q_bits<64>(bits, prog, grid, coresident, s);
    case 256: return launch_q_bits<256>(bits, prog, grid, coresident, s);
    default: return launch_q_bits<128>(bits, prog, grid, coresident, s);
  }
}

// y[M, N] = x[M, K] . Wq[N, K]^T * scale + bias; Wq packed at `bits` in {2, 4, 8}; bf16 in/out.
// partial: split-K slice scratch (plan_gemm().slice_bytes); counters: zero-filled, left zero.
int gemm_tcq(const void* W, int bits, const float* scale, const void* bias, const void* x, void* y, int64_t M, int64_t K,
             int64_t N, float* partial, int* counters, int* status, cudaStream_t s) {
  PhaseSpec ps;
  ps.nsub = 1;
  ps.gated = 0;
  ps.g[0] = GemmSpec{W, scale, bias, x, y, N, K};
  return run_program_tcq(&ps, 1, bits, M, (uint8_t*)partial, counters, (int*)((uint8_t*)status + kWsGridBar), status, s);
}

}  // namespace tsb
