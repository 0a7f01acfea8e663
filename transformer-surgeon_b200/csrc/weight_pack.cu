// Weight quantization, bit packing and reconstruction.
//
// Follows transformersurgeon/compression/quantization_methods/vanilla.py:5-37 step by
// step, in the parameter dtype: for bf16 parameters every intermediate (amax/qmax,
// scale+eps, w/(scale+eps)) is rounded to bf16 before the next op, exactly as the
// chain of torch ops does; rounding of the quotient to an integer is half-to-even.
#include "common.cuh"

namespace tsb {

__device__ __forceinline__ float block_max(float v, float* sh) {
  v = warp_max(v);
  int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = (l < nw) ? sh[l] : 0.f;
  r = warp_max(r);
  __syncthreads();
  return r;
}
__device__ __forceinline__ double block_sum_d(double v, double* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) sh[w] = v;
  __syncthreads();
  double r = (l < nw) ? sh[l] : 0.0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  __syncthreads();
  return r;
}

struct TensorStats {       // lives in the caller's workspace (16 bytes)
  unsigned int amax_bits;  // max |w| as fp32 bits (non-negative floats order like uints)
  unsigned int pad;
  double abs_sum;
};

template <typename T>
__global__ void tensor_stats_kernel(const T* __restrict__ w, int64_t n, TensorStats* st) {
  __shared__ float shf[32];
  __shared__ double shd[32];
  float m = 0.f;
  double s = 0.0;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float a = fabsf(to_f32<T>(w[i]));
    m = fmaxf(m, a);
    s += (double)a;
  }
  m = block_max(m, shf);
  s = block_sum_d(s, shd);
  if (threadIdx.x == 0) {
    atomicMax(&st->amax_bits, __float_as_uint(m));
    atomicAdd(&st->abs_sum, s);
  }
}

// One CTA per row.  precision 0 = binary.
template <typename T>
__global__ void quantize_rows_kernel(const T* __restrict__ w, int64_t rows, int64_t cols, int precision,
                                     int per_channel, float eps, int8_t* __restrict__ codes,
                                     float* __restrict__ scales, const TensorStats* st) {
  __shared__ float shf[32];
  __shared__ double shd[32];
  const int64_t r = blockIdx.x;
  const T* wr = w + r * cols;
  int8_t* cr = codes + r * cols;
  if (precision == 0) {
    float scale;
    if (per_channel) {
      double s = 0.0;
      for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) s += (double)fabsf(to_f32<T>(wr[c]));
      s = block_sum_d(s, shd);
      scale = rnd<T>((float)(s / (double)cols));
    } else {
      scale = rnd<T>((float)(st->abs_sum / (double)(rows * cols)));
    }
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
      float v = to_f32<T>(wr[c]);
      cr[c] = (int8_t)((v > 0.f) - (v < 0.f));
    }
    if (threadIdx.x == 0) scales[r] = scale;
    return;
  }
  const float qmax = (float)((1 << (precision - 1)) - 1);
  float amax;
  if (per_channel) {
    float m = 0.f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, fabsf(to_f32<T>(wr[c])));
    amax = block_max(m, shf);
  } else {
    amax = __uint_as_float(st->amax_bits);
  }
  const float scale = rnd<T>(__fdiv_rn(amax, qmax));
  const float denom = rnd<T>(__fadd_rn(scale, eps));
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    float q = rnd<T>(__fdiv_rn(to_f32<T>(wr[c]), denom));
    q = fminf(fmaxf(rintf(q), -qmax), qmax);
    cr[c] = (int8_t)(int)q;   // NaN (0/0 cannot occur: denom >= eps) -> not reached
  }
  if (threadIdx.x == 0) scales[r] = scale;
}

// One thread per packed 32-bit word (bits < 8) or per byte (bits == 8).
__global__ void pack_codes_kernel(const int8_t* __restrict__ codes, int64_t rows, int64_t cols, int bits,
                                  int64_t row_bytes, uint8_t* __restrict__ packed, int32_t* zero_flag) {
  if (bits == 8) {
    const int64_t total = rows * row_bytes;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
      const int64_t r = i / row_bytes, c = i - r * row_bytes;
      packed[i] = c < cols ? (uint8_t)codes[r * cols + c] : (uint8_t)0;
    }
    return;
  }
  const int per = 32 / bits;
  const int64_t row_words = row_bytes / 4;
  const int64_t total = rows * row_words;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / row_words, g = i - r * row_words;
    const int8_t* cr = codes + r * cols;
    unsigned int out = 0;
    for (int j = 0; j < per; ++j) {
      const int64_t c = g * per + j;
      const int q = (c < cols) ? (int)cr[c] : 0;
      const int f = field_of_column(j, per);
      if (bits == 1) {
        if (c < cols && q == 0 && zero_flag) *zero_flag = 1;
        out |= (unsigned)(q > 0) << f;
      } else {
        out |= ((unsigned)q & ((1u << bits) - 1u)) << (bits * f);
      }
    }
    reinterpret_cast<unsigned*>(packed)[i] = out;
  }
}

__global__ void unpack_codes_kernel(const uint8_t* __restrict__ packed, int64_t rows, int64_t cols, int bits,
                                    int64_t row_bytes, int8_t* __restrict__ codes) {
  const int64_t total = rows * cols;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / cols, c = i - r * cols;
    codes[i] = (int8_t)load_code(packed + r * row_bytes, c, bits);
  }
}

template <typename T>
__global__ void dequantize_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales, int64_t rows,
                                  int64_t cols, int bits, int64_t row_bytes, T* __restrict__ out) {
  const int64_t total = rows * cols;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / cols, c = i - r * cols;
    const int q = load_code(packed + r * row_bytes, c, bits);
    out[i] = from_f32<T>(__fmul_rn((float)q, scales[r]));
  }
}

inline int grid_for(int64_t n, int block) {
  int64_t g = (n + block - 1) / block;
  const int64_t cap = 148 * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace tsb

using namespace tsb;

extern "C" {

size_t tsb200_packed_row_bytes(int64_t cols, int bits) {
  if (cols <= 0 || !(bits == 1 || bits == 2 || bits == 4 || bits == 8)) return 0;
  return (size_t)((cols + 63) / 64 * 64 * bits / 8);
}

int tsb200_quantize_weight(const void* w, int dtype, int64_t rows, int64_t cols, int precision,
                           int per_channel, float eps, int8_t* codes, float* scales,
                           void* workspace, size_t workspace_bytes, void* stream) {
  TSB_REQUIRE_DEVICE();
  if (rows < 0 || cols < 0) return TSB200_ERR_ARG;
  if (rows == 0 || cols == 0) return TSB200_OK;
  if (!w || !codes || !scales) return TSB200_ERR_ARG;
  if (!(precision == 0 || (precision >= 2 && precision <= 8))) return TSB200_ERR_UNSUPPORTED;
  if (dtype != TSB200_F32 && dtype != TSB200_BF16) return TSB200_ERR_UNSUPPORTED;
  if (rows > 0x7fffffffLL) return TSB200_ERR_UNSUPPORTED;
  cudaStream_t s = as_stream(stream);
  TensorStats* st = nullptr;
  if (!per_channel) {
    if (!workspace || !aligned(workspace, 8)) return TSB200_ERR_ARG;
    if (workspace_bytes < sizeof(TensorStats)) return TSB200_ERR_WORKSPACE;
    st = (TensorStats*)workspace;
    TSB_CUDA(cudaMemsetAsync(st, 0, sizeof(TensorStats), s));
    const int64_t n = rows * cols;
    if (dtype == TSB200_F32) tensor_stats_kernel<float><<<grid_for(n, 256), 256, 0, s>>>((const float*)w, n, st);
    else tensor_stats_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, s>>>((const __nv_bfloat16*)w, n, st);
    TSB_LAUNCH_CHECK();
  }
  if (dtype == TSB200_F32)
    quantize_rows_kernel<float><<<(unsigned)rows, 256, 0, s>>>((const float*)w, rows, cols, precision, per_channel, eps, codes, scales, st);
  else
    quantize_rows_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, s>>>((const __nv_bfloat16*)w, rows, cols, precision, per_channel, eps, codes, scales, st);
  TSB_LAUNCH_CHECK();
  return TSB200_OK;
}

int tsb200_pack_codes(const int8_t* codes, int64_t rows, int64_t cols, int bits, uint8_t* packed,
                      int32_t* zero_flag, void* stream) {
  TSB_REQUIRE_DEVICE();
  if (rows < 0 || cols < 0) return TSB200_ERR_ARG;
  const size_t rb = tsb200_packed_row_bytes(cols > 0 ? cols : 1, bits);
  if (rb == 0) return TSB200_ERR_UNSUPPORTED;
  if (rows == 0 || cols == 0) return TSB200_OK;
  if (!codes || !packed || !aligned(packed, 4)) return TSB200_ERR_ARG;
  pack_codes_kernel<<<grid_for(rows * (int64_t)(bits == 8 ? rb : rb / 4), 256), 256, 0, as_stream(stream)>>>(codes, rows, cols, bits, (int64_t)rb, packed, zero_flag);
  TSB_LAUNCH_CHECK();
  return TSB200_OK;
}

int tsb200_unpack_codes(const uint8_t* packed, int64_t rows, int64_t cols, int bits, int8_t* codes, void* stream) {
  TSB_REQUIRE_DEVICE();
  if (rows < 0 || cols < 0) return TSB200_ERR_ARG;
  const size_t rb = tsb200_packed_row_bytes(cols > 0 ? cols : 1, bits);
  if (rb == 0) return TSB200_ERR_UNSUPPORTED;
  if (rows == 0 || cols == 0) return TSB200_OK;
  if (!codes || !packed) return TSB200_ERR_ARG;
  unpack_codes_kernel<<<grid_for(rows * cols, 256), 256, 0, as_stream(stream)>>>(packed, rows, cols, bits, (int64_t)rb, codes);
  TSB_LAUNCH_CHECK();
  return TSB200_OK;
}

int tsb200_dequantize_weight(const uint8_t* packed, const float* scales, int64_t rows, int64_t cols, int bits,
                             int dtype, void* w_out, void* stream) {
  TSB_REQUIRE_DEVICE();
  if (rows < 0 || cols < 0) return TSB200_ERR_ARG;
  const size_t rb = tsb200_packed_row_bytes(cols > 0 ? cols : 1, bits);
  if (rb == 0) return TSB200_ERR_UNSUPPORTED;
  if (dtype != TSB200_F32 && dtype != TSB200_BF16) return TSB200_ERR_UNSUPPORTED;
  if (rows == 0 || cols == 0) return TSB200_OK;
  if (!packed || !scales || !w_out) return TSB200_ERR_ARG;
  cudaStream_t s = as_stream(stream);
  if (dtype == TSB200_F32)
    dequantize_kernel<float><<<grid_for(rows * cols, 256), 256, 0, s>>>(packed, scales, rows, cols, bits, (int64_t)rb, (float*)w_out);
  else
    dequantize_kernel<__nv_bfloat16><<<grid_for(rows * cols, 256), 256, 0, s>>>(packed, scales, rows, cols, bits, (int64_t)rb, (__nv_bfloat16*)w_out);
  TSB_LAUNCH_CHECK();
  return TSB200_OK;
}

}  // extern "C"
