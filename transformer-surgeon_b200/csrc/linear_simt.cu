// LinearCompressed.forward on CUDA cores: a weight-streaming kernel for tiny M (decode
// with one or a few tokens) and the cross-check of the tensor-core kernel.
//
// Restates transformersurgeon/blocks/linear_compressed.py:96-100: h = x @ V^T (rounded
// to the act dtype, as F.linear returns it), y = h @ U^T + bias.  Quantized factors are
// dequantized on the fly: y[m,o] = scale[o] * sum_k code[o,k] * x[m,k]  (fp32 accumulate).
// One warp per output row streams that row's packed codes once (16-byte aligned vector
// loads) for up to 8 activation rows held in shared memory.
#include "tc_common.cuh"

namespace tsb {
namespace {

constexpr int MT = 8;        // activation rows per pass
constexpr int KT = 1024;     // k-tile staged in shared memory
constexpr int ROWS_PER_CTA = 8;

// Decode 8 consecutive weights starting at column k0 (k0 % 8 == 0) of a row.
template <int BITS>
__device__ __forceinline__ void load8(const uint8_t* __restrict__ row, int64_t k0, float (&wv)[8]) {
  if (BITS == 32) {
    const float4 a = *reinterpret_cast<const float4*>(row + k0 * 4);
    const float4 b = *reinterpret_cast<const float4*>(row + k0 * 4 + 16);
    wv[0] = a.x; wv[1] = a.y; wv[2] = a.z; wv[3] = a.w; wv[4] = b.x; wv[5] = b.y; wv[6] = b.z; wv[7] = b.w;
  } else if (BITS == 16) {
    const uint4 a = *reinterpret_cast<const uint4*>(row + k0 * 2);
    const unsigned u[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      wv[2 * i] = __uint_as_float(u[i] << 16);
      wv[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
  } else if (BITS == 8) {
    const uint2 a = *reinterpret_cast<const uint2*>(row + k0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      wv[i] = (float)(int8_t)(a.x >> (8 * i));
      wv[4 + i] = (float)(int8_t)(a.y >> (8 * i));
    }
  } else if (BITS == 4) {          // one word = 8 columns: field j -> column 2j, field j+4 -> column 2j+1
    const unsigned a = *reinterpret_cast<const unsigned*>(row + k0 / 2);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      wv[2 * j] = (float)sext((int)(a >> (4 * j)), 4);
      wv[2 * j + 1] = (float)sext((int)(a >> (4 * j + 16)), 4);
    }
  } else if (BITS == 2) {          // one word = 16 columns; k0 % 16 in {0, 8}
    const unsigned a = *reinterpret_cast<const unsigned*>(row + (k0 / 16) * 4);
    const int j0 = (int)(k0 % 16) / 2;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      wv[2 * j] = (float)sext((int)(a >> (2 * (j0 + j))), 2);
      wv[2 * j + 1] = (float)sext((int)(a >> (2 * (j0 + j) + 16)), 2);
    }
  } else {                         // one word = 32 columns; k0 % 32 in {0, 8, 16, 24}
    const unsigned a = *reinterpret_cast<const unsigned*>(row + (k0 / 32) * 4);
    const int j0 = (int)(k0 % 32) / 2;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      wv[2 * j] = (float)(int)(((a >> (j0 + j)) & 1u) * 2u) - 1.0f;
      wv[2 * j + 1] = (float)(int)(((a >> (j0 + j + 16)) & 1u) * 2u) - 1.0f;
    }
  }
}

// y[m, o] = scale[o] * sum_k W[o,k] x[m,k] + bias[o] for m in [m0, m0+MT).
// K is the logical reduction length; rows of W are row_bytes apart (dense: K*elt).
template <typename T, int BITS>
__global__ void __launch_bounds__(ROWS_PER_CTA * 32)
linear_simt_kernel(const uint8_t* __restrict__ W, int64_t row_bytes, const float* __restrict__ scale,
                   const T* __restrict__ bias, const T* __restrict__ x, T* __restrict__ y, int64_t M, int64_t K,
                   int64_t N, int64_t m0) {
  __shared__ __align__(16) float xs[MT][KT];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t o = (int64_t)blockIdx.x * ROWS_PER_CTA + w;
  const int mt = (int)min((int64_t)MT, M - m0);
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0.f;
  const uint8_t* wrow = W + (o < N ? o : 0) * row_bytes;
  for (int64_t kb = 0; kb < K; kb += KT) {
    const int kt = (int)min((int64_t)KT, K - kb);
    __syncthreads();
    for (int idx = threadIdx.x; idx < MT * KT; idx += blockDim.x) {
      const int m = idx / KT, k = idx % KT;
      xs[m][k] = (m < mt && k < kt) ? to_f32<T>(x[(m0 + m) * K + kb + k]) : 0.f;
    }
    __syncthreads();
    if (o < N) {
      for (int k0 = lane * 8; k0 < kt; k0 += 256) {
        float wv[8];
        load8<BITS>(wrow, kb + k0, wv);
        if (BITS >= 16) {   // dense rows are not padded: zero the tail beyond K
#pragma unroll
          for (int i = 0; i < 8; ++i) if (k0 + i >= kt) wv[i] = 0.f;
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const float4 xa = *reinterpret_cast<const float4*>(&xs[m][k0]);
          const float4 xb = *reinterpret_cast<const float4*>(&xs[m][k0 + 4]);
          acc[m] += wv[0] * xa.x + wv[1] * xa.y + wv[2] * xa.z + wv[3] * xa.w + wv[4] * xb.x + wv[5] * xb.y +
                    wv[6] * xb.z + wv[7] * xb.w;
        }
      }
    }
  }
  if (o >= N) return;
  const float sc = scale ? scale[o] : 1.0f;
  const float bv = bias ? to_f32<T>(bias[o]) : 0.f;
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    const float v = warp_sum(acc[m]);
    if (lane == 0 && m < mt) y[(m0 + m) * N + o] = from_f32<T>(v * sc + bv);
  }
}

template <typename T, int BITS>
int launch_one(const void* W, int64_t row_bytes, const float* scale, const void* bias, const void* x, void* y,
               int64_t M, int64_t K, int64_t N, cudaStream_t s) {
  const int64_t blocks = (N + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
  if (blocks > 0x7fffffffLL) return TSB200_ERR_UNSUPPORTED;
  for (int64_t m0 = 0; m0 < M; m0 += MT) {
    linear_simt_kernel<T, BITS><<<(unsigned)blocks, ROWS_PER_CTA * 32, 0, s>>>(
        (const uint8_t*)W, row_bytes, scale, (const T*)bias, (const T*)x, (T*)y, M, K, N, m0);
    TSB_LAUNCH_CHECK();
  }
  return TSB200_OK;
}

template <typename T>
int launch_bits(int bits, const void* W, const float* scale, const void* bias, const void* x, void* y, int64_t M,
                int64_t K, int64_t N, cudaStream_t s) {
  switch (bits) {
    case 1: return launch_one<T, 1>(W, (int64_t)tsb200_packed_row_bytes(K, 1), scale, bias, x, y, M, K, N, s);
    case 2: return launch_one<T, 2>(W, (int64_t)tsb200_packed_row_bytes(K, 2), scale, bias, x, y, M, K, N, s);
    case 4: return launch_one<T, 4>(W, (int64_t)tsb200_packed_row_bytes(K, 4), scale, bias, x, y, M, K, N, s);
    case 8: return launch_one<T, 8>(W, (int64_t)tsb200_packed_row_bytes(K, 8), scale, bias, x, y, M, K, N, s);
    case 16: return launch_one<T, 16>(W, K * 2, nullptr, bias, x, y, M, K, N, s);
    case 32: return launch_one<T, 32>(W, K * 4, nullptr, bias, x, y, M, K, N, s);
    default: return TSB200_ERR_UNSUPPORTED;
  }
}

}  // namespace

int validate_linear(const tsb200_linear_desc* d, const void* x, void* y, int64_t M, bool& noop) {
  noop = false;
  if (!d) return TSB200_ERR_ARG;
  if (d->in_features <= 0 || d->out_features <= 0 || d->rank < 0 || M < 0 || d->reserved != 0) return TSB200_ERR_ARG;
  if (d->act_dtype != TSB200_F32 && d->act_dtype != TSB200_BF16) return TSB200_ERR_UNSUPPORTED;
  auto ok_bits = [&](int b, const void* p, const float* sc) -> int {
    if (!(b == 1 || b == 2 || b == 4 || b == 8 || b == 16 || b == 32)) return TSB200_ERR_UNSUPPORTED;
    if (!p || !aligned(p, 16)) return TSB200_ERR_ARG;
    if (b <= 8 && !sc) return TSB200_ERR_ARG;
    // dense factors are stored in the act dtype
    if (b == 16 && d->act_dtype != TSB200_BF16) return TSB200_ERR_UNSUPPORTED;
    if (b == 32 && d->act_dtype != TSB200_F32) return TSB200_ERR_UNSUPPORTED;
    return TSB200_OK;
  };
  int st = ok_bits(d->u_bits, d->u, d->u_scale);
  if (st != TSB200_OK) return st;
  if (d->rank > 0) {
    st = ok_bits(d->v_bits, d->v, d->v_scale);
    if (st != TSB200_OK) return st;
  }
  // dense rows are read 8 elements at a time
  const int64_t ku = d->rank > 0 ? d->rank : d->in_features;
  if (d->u_bits >= 16 && (ku % 8)) return TSB200_ERR_UNSUPPORTED;
  if (d->rank > 0 && d->v_bits >= 16 && (d->in_features % 8)) return TSB200_ERR_UNSUPPORTED;
  if (M == 0) { noop = true; return TSB200_OK; }
  if (!x || !y) return TSB200_ERR_ARG;
  return TSB200_OK;
}

}  // namespace tsb

using namespace tsb;

static constexpr size_t kWsHeaderBytes = 256 + 4096 * sizeof(int);   // = tc::kWsHeader

extern "C" {

// Workspace layout shared by all linear kernels: [0, 256) status word (a kernel that gave up on
// a bounded wait stores a non-zero code there), [256, 256 + 16 KB) split-K tile counters (zero
// between calls), then the rank-r intermediate [M, rank] in the act dtype, then split-K scratch
// (fp32 [M, max(rank, out)] for the dense kernel, per-item slices for the packed kernel).
size_t tsb200_linear_workspace_bytes(const tsb200_linear_desc* d, int64_t M) {
  if (!d || M <= 0) return kWsHeaderBytes;
  const size_t elt = d->act_dtype == TSB200_F32 ? 4 : 2;
  const size_t h = ((size_t)M * (size_t)(d->rank > 0 ? d->rank : 0) * elt + 255) / 256 * 256;
  const size_t nmax = (size_t)(d->rank > d->out_features ? d->rank : d->out_features);
  size_t scratch = (size_t)M * nmax * 4;
  const int64_t ku = d->rank > 0 ? d->rank : d->in_features;
  const size_t s_u = tc::plan_gemm(M, d->out_features, ku).slice_bytes;
  const size_t s_v = d->rank > 0 ? tc::plan_gemm(M, d->rank, d->in_features).slice_bytes : 0;
  if (s_u + s_v > scratch) scratch = s_u + s_v;     // the fused V -> U launch keeps both phases' slices apart
  return kWsHeaderBytes + h + (scratch + 255) / 256 * 256;
}

int tsb200_linear_simt(const tsb200_linear_desc* d, const void* x, void* y, int64_t M, void* workspace,
                       size_t workspace_bytes, void* stream) {
  TSB_REQUIRE_DEVICE();
  bool noop;
  int st = validate_linear(d, x, y, M, noop);
  if (st != TSB200_OK || noop) return st;
  cudaStream_t s = as_stream(stream);
  const void* in = x;
  int64_t K = d->in_features;
  if (d->rank > 0) {
    if (!workspace || !aligned(workspace, 16)) return TSB200_ERR_ARG;
    if (workspace_bytes < tsb200_linear_workspace_bytes(d, M)) return TSB200_ERR_WORKSPACE;
    void* h = (uint8_t*)workspace + kWsHeaderBytes;
    st = d->act_dtype == TSB200_F32
             ? launch_bits<float>(d->v_bits, d->v, d->v_scale, nullptr, x, h, M, d->in_features, d->rank, s)
             : launch_bits<__nv_bfloat16>(d->v_bits, d->v, d->v_scale, nullptr, x, h, M, d->in_features, d->rank, s);
    if (st != TSB200_OK) return st;
    in = h;
    K = d->rank;
  }
  return d->act_dtype == TSB200_F32
             ? launch_bits<float>(d->u_bits, d->u, d->u_scale, d->bias, in, y, M, K, d->out_features, s)
             : launch_bits<__nv_bfloat16>(d->u_bits, d->u, d->u_scale, d->bias, in, y, M, K, d->out_features, s);
}

}  // extern "C"
