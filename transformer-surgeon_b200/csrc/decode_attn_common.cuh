// Shared pieces of the paged decode-attention kernels: split bookkeeping, the partial
// (m, l, acc) workspace layout and the cross-split reduction.
#pragma once
#include "common.cuh"

namespace tsb {

// Workspace: kAttnCounterBytes of int32 counters (zero between calls; one per (sequence, kv head,
// head chunk), used by the tensor-core kernel to let the last split merge the partials), then
// float [B][H][S][2 + d]  ->  m, l, acc[d] per (sequence, q head, split).
constexpr size_t kAttnCounterBytes = 16384;
// The last int32 of the counter block is a status word: a kernel that gave up on a bounded wait for its own
// copies records a non-zero code there (the result of that call is then not to be trusted).
constexpr int kAttnStatusIndex = (int)(kAttnCounterBytes / sizeof(int)) - 1;
struct AttnSplit {
  int splits;
};

inline int choose_splits(int64_t B, int hkv, int64_t max_seq_len) {
  const int64_t base = B * hkv;
  const int64_t pages = (max_seq_len + 15) / 16;
  int64_t s = (148 * 8 + base - 1) / (base > 0 ? base : 1);
  // few (sequence, kv head) pairs, long contexts: about 768 CTAs measured fastest (8 sequences x 4 kv heads x 32k
  // tokens, NVFP4 pages: 24 splits 99 us, 37 splits 115 us, 13 splits 128 us)
  if (base > 0 && base < 148) {
    s = (768 + base - 1) / base;
  } else if (s >= 3) {
    // a power of two measured fastest (int8 / NVFP4 pages, 4k-32k tokens: 32 x 8 pairs 4 splits against 5: 5 % faster at
    // 4k; 64 x 8 pairs 4 against 3: 3-6 %; 128 x 8 pairs 2 stays): the nearest one
    int64_t p2 = 1;
    while (2 * p2 <= s) p2 *= 2;
    s = (2 * s >= 3 * p2) ? 2 * p2 : p2;
  }
  const int64_t cap = pages / 4 > 0 ? pages / 4 : 1;   // at least 4 pages per split
  if (s > cap) s = cap;
  if (s < 1) s = 1;
  if (s > 64) s = 64;
  return (int)s;
}

// Split count of the fp8-MMA kernel.  Two 6-warp CTAs fit an SM (296 slots): with that many (sequence, kv head)
// pairs or more, one split each is fastest (a second wave of CTAs costs more than it saves); below that the pairs
// are split so that the grid fills the slots without spilling into a second wave, each split keeping at least
// 24 pages (two page pairs per warp) to amortise the per-CTA query expansion and merge.
inline int choose_splits_fp8(int64_t B, int hkv, int64_t max_seq_len) {
  const int64_t base = B * hkv;
  const int64_t pages = (max_seq_len + 15) / 16;
  int64_t s = base > 0 ? 296 / base : 1;
  // two splits pay from about 1.5k tokens on (128 pairs: 1k tokens 18.8 us against 17.2 us for one split, 2k 25.9 / 28.5,
  // 4k 38.9 / 50.9, 8k 64.0 / 94.2 - one split leaves every SM with a single CTA)
  if (s == 2 && pages < 96) s = 1;
  const int64_t cap = pages / 24 > 0 ? pages / 24 : 1;
  if (s > cap) s = cap;
  if (s < 1) s = 1;
  if (s > 64) s = 64;
  return (int)s;
}

// Pages [begin, end) of sequence with `len` tokens handled by split s of S.
__device__ __forceinline__ void split_range(int len, int s, int S, int& begin, int& end) {
  const int pages = (len + 15) >> 4;
  const int per = (pages + S - 1) / S;
  begin = s * per;
  end = min(pages, begin + per);
}

__device__ __forceinline__ float e4m3_byte_to_f32(unsigned int c) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
__device__ __forceinline__ float e2m1_nibble_to_f32(unsigned int c) {
  __half_raw h = __nv_cvt_fp4_to_halfraw((__nv_fp4_storage_t)(c & 15), __NV_E2M1);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// Dequantized K / V element (token slot t, element e) of one page record; slow path used
// by the CUDA-core kernel.  fp8 scale is applied by the caller.
template <int D>
__device__ __forceinline__ float dense_elem(const uint8_t* __restrict__ rec, int fmt, int t, int e) {
  if (fmt == TSB200_KV_F32) return reinterpret_cast<const float*>(rec)[t * D + e];
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(rec)[t * D + e]);
}
template <int D>
__device__ __forceinline__ float k_elem(const uint8_t* __restrict__ rec, int fmt, int t, int e) {
  if (fmt >= TSB200_KV_F32) return dense_elem<D>(rec, fmt, t, e);
  if (fmt == TSB200_KV_INT8)
    return (float)(int8_t)rec[t * D + e] * reinterpret_cast<const float*>(rec + 16 * D)[t];
  if (fmt == TSB200_KV_FP8) return e4m3_byte_to_f32(rec[t * D + e]);
  const unsigned b = rec[t * (D / 2) + (e >> 1)];
  return e2m1_nibble_to_f32(b >> ((e & 1) * 4)) * e4m3_byte_to_f32(rec[16 * (D / 2) + t * (D / 16) + (e >> 4)]);
}
template <int D>
__device__ __forceinline__ float v_elem(const uint8_t* __restrict__ rec, int fmt, int t, int e) {
  if (fmt >= TSB200_KV_F32) return dense_elem<D>(rec, fmt, t, e);
  if (fmt == TSB200_KV_INT8)
    return (float)(int8_t)rec[e * 16 + t] * reinterpret_cast<const float*>(rec + 16 * D)[t];
  if (fmt == TSB200_KV_FP8) return e4m3_byte_to_f32(rec[e * 16 + t]);
  const unsigned b = rec[(e >> 1) * 16 + t];
  return e2m1_nibble_to_f32(b >> ((e & 1) * 4)) * e4m3_byte_to_f32(rec[16 * (D / 2) + (e >> 4) * 16 + t]);
}

int validate_kv(const tsb200_kv_desc* kv, bool need_table);

}  // namespace tsb
