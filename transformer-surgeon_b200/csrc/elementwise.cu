// Small decoder ops: RoPE (half-split), residual-add + RMSNorm (two variants), SwiGLU.
// Each op rounds to the activation dtype at the same points as the chain of torch ops
// it replaces, so bf16 results track the reference closely.
#include "common.cuh"

namespace tsb {

// x [B, T, heads, d]; one thread per (token, head, i < d/2).
template <typename T>
__global__ void rope_kernel(T* __restrict__ x, int64_t xs, int64_t B, int64_t Tn, int heads, int d, const int32_t* __restrict__ pos0,
                            const float* __restrict__ cosT, const float* __restrict__ sinT, int64_t rope_rows) {
  const int half = d / 2;
  const int64_t total = B * Tn * heads * half;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx % half);
    const int64_t th = idx / half;           // (b, t, head)
    const int64_t bt = th / heads;
    const int hd = (int)(th - bt * heads);
    const int64_t b = bt / Tn, t = bt - b * Tn;
    int64_t pos = (pos0 ? (int64_t)pos0[b] : 0) + t;
    pos = pos < 0 ? 0 : (pos >= rope_rows ? rope_rows - 1 : pos);
    const float c = rnd<T>(cosT[pos * half + i]);
    const float s = rnd<T>(sinT[pos * half + i]);
    T* p = x + bt * xs + (int64_t)hd * d;
    const float xr = to_f32<T>(p[i]), xi = to_f32<T>(p[i + half]);
    const float yr = __fsub_rn(rnd<T>(__fmul_rn(xr, c)), rnd<T>(__fmul_rn(xi, s)));
    const float yi = __fadd_rn(rnd<T>(__fmul_rn(xr, s)), rnd<T>(__fmul_rn(xi, c)));
    p[i] = from_f32<T>(yr);
    p[i + half] = from_f32<T>(yi);
  }
}

__device__ __forceinline__ float block_reduce_sum(float v, float* sh) {
  v = warp_sum(v);
  int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = (l < nw) ? sh[l] : 0.f;
  r = warp_sum(r);
  __syncthreads();
  return r;
}
__device__ __forceinline__ float block_reduce_max(float v, float* sh) {
  v = warp_max(v);
  int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = (l < nw) ? sh[l] : 0.f;
  r = warp_max(r);
  __syncthreads();
  return r;
}

// One CTA per row.
template <typename T>
__global__ void add_rmsnorm_kernel(T* __restrict__ residual, const T* __restrict__ delta, const T* __restrict__ w,
                                   T* __restrict__ y, int64_t hidden, float eps, int variant) {
  __shared__ float sh[32];
  const int64_t row = blockIdx.x;
  T* r = residual + row * hidden;
  const T* dl = delta ? delta + row * hidden : nullptr;
  T* yo = y + row * hidden;
  float ss = 0.f, mx = 0.f;
  for (int64_t c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = to_f32<T>(r[c]);
    if (dl) {
      v = rnd<T>(__fadd_rn(v, to_f32<T>(dl[c])));
      r[c] = from_f32<T>(v);
    }
    ss += v * v;
    mx = fmaxf(mx, fabsf(v));
  }
  if (variant == 0) {
    const float var = block_reduce_sum(ss, sh) / (float)hidden;
    const float inv = 1.0f / sqrtf(var + eps);
    for (int64_t c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float v = to_f32<T>(r[c]);
      yo[c] = from_f32<T>(__fmul_rn(to_f32<T>(w[c]), rnd<T>(__fmul_rn(v, inv))));
    }
  } else {
    mx = fmaxf(block_reduce_max(mx, sh), 1.0f);
    float s2 = 0.f;
    for (int64_t c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float v = rnd<T>(__fdiv_rn(to_f32<T>(r[c]), mx));
      s2 += rnd<T>(__fmul_rn(v, v));
    }
    const float var = rnd<T>(block_reduce_sum(s2, sh) / (float)hidden);
    const float inv = rnd<T>(1.0f / sqrtf(rnd<T>(__fadd_rn(var, 1e-5f))));
    for (int64_t c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float v = rnd<T>(__fdiv_rn(to_f32<T>(r[c]), mx));
      yo[c] = from_f32<T>(__fmul_rn(to_f32<T>(w[c]), rnd<T>(__fmul_rn(v, inv))));
    }
  }
}

// Hugging Face variant, bf16, hidden % 8 == 0 and hidden <= 8192: one pass over global memory with
// 16-byte loads; the row stays in registers between the statistic and the scaling.
__global__ void __launch_bounds__(256)
add_rmsnorm_hf_bf16_kernel(__nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ delta,
                           const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, int hidden, float eps) {
  __shared__ float sh[32];
  pdl_launch_dependents();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const int nvec = hidden >> 3;
  uint4* r = reinterpret_cast<uint4*>(residual + row * hidden);
  const uint4* dl = delta ? reinterpret_cast<const uint4*>(delta + row * hidden) : nullptr;
  float v[4][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int i = threadIdx.x + it * 256;
    if (i < nvec) {
      uint4 a = r[i];
      const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
      if (dl) {
        const uint4 b = dl[i];
        const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
        uint4 o;
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fa = __bfloat1622float2(ap[j]), fb = __bfloat1622float2(bp[j]);
          op[j] = __floats2bfloat162_rn(__fadd_rn(fa.x, fb.x), __fadd_rn(fa.y, fb.y));
          const float2 fo = __bfloat1622float2(op[j]);
          v[it][2 * j] = fo.x; v[it][2 * j + 1] = fo.y;
        }
        r[i] = o;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fa = __bfloat1622float2(ap[j]);
          v[it][2 * j] = fa.x; v[it][2 * j + 1] = fa.y;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[it][j] * v[it][j];
    }
  }
  const float var = block_reduce_sum(ss, sh) / (float)hidden;
  const float inv = 1.0f / sqrtf(var + eps);
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  uint4* yo = reinterpret_cast<uint4*>(y + row * hidden);
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int i = threadIdx.x + it * 256;
    if (i < nvec) {
      const uint4 ww = wv[i];
      const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&ww);
      uint4 o;
      __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 fw = __bfloat1622float2(wp[j]);
        const __nv_bfloat162 n = __floats2bfloat162_rn(__fmul_rn(v[it][2 * j], inv), __fmul_rn(v[it][2 * j + 1], inv));
        const float2 fn = __bfloat1622float2(n);
        op[j] = __floats2bfloat162_rn(__fmul_rn(fw.x, fn.x), __fmul_rn(fw.y, fn.y));
      }
      yo[i] = o;
    }
  }
}

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ y, int64_t M, int64_t n,
                              int64_t gs, int64_t us, int64_t ys) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = M * n;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / n, c = i - m * n;
    const float g = to_f32<T>(gate[m * gs + c]);
    const float u = to_f32<T>(up[m * us + c]);
    const float a = rnd<T>(g / (1.0f + expf(-g)));
    y[m * ys + c] = from_f32<T>(__fmul_rn(a, u));
  }
}

// Same arithmetic, eight bf16 elements (16 bytes) per thread and step: rows of n % 8 == 0 elements whose starts are
// 16-byte aligned (a prompt-sized [65536, 14336] call moves 5.6 GB: the element-wise form ran at half the copy rate).
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                                     __nv_bfloat16* __restrict__ y, int64_t M, int64_t n8, int64_t gs, int64_t us, int64_t ys) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = M * n8;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / n8, c = (i - m * n8) * 8;
    const uint4 gv = *reinterpret_cast<const uint4*>(gate + m * gs + c);
    const uint4 uv = *reinterpret_cast<const uint4*>(up + m * us + c);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* upp = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = __bfloat1622float2(gp[j]), u = __bfloat1622float2(upp[j]);
      const float a0 = rnd<__nv_bfloat16>(g.x / (1.0f + expf(-g.x))), a1 = rnd<__nv_bfloat16>(g.y / (1.0f + expf(-g.y)));
      op[j] = __halves2bfloat162(from_f32<__nv_bfloat16>(__fmul_rn(a0, u.x)), from_f32<__nv_bfloat16>(__fmul_rn(a1, u.y)));
    }
    *reinterpret_cast<uint4*>(y + m * ys + c) = o;
  }
}

inline int egrid(int64_t n) {
  int64_t g = (n + 255) / 256;
  return (int)(g < 1 ? 1 : (g > 148 * 8 ? 148 * 8 : g));
}
}  // namespace tsb

using namespace tsb;

extern "C" {

int tsb200_rope(void* x, int dtype, int64_t token_stride, int64_t B, int64_t T, int heads, int head_dim, const int32_t* pos0,
                const float* rope_cos, const float* rope_sin, int64_t rope_rows, void* stream) {
  TSB_REQUIRE_DEVICE();
  if (B < 0 || T < 0 || heads <= 0 || head_dim <= 0 || (head_dim & 1)) return TSB200_ERR_ARG;
  if (B == 0 || T == 0) return TSB200_OK;
  if (!x || !rope_cos || !rope_sin || rope_rows <= 0) return TSB200_ERR_ARG;
  const int64_t n = B * T * heads * (head_dim / 2);
  const int64_t xs = token_stride ? token_stride : (int64_t)heads * head_dim;
  if (xs < (int64_t)heads * head_dim) return TSB200_ERR_ARG;
  if (dtype == TSB200_F32)
    rope_kernel<float><<<egrid(n), 256, 0, as_stream(stream)>>>((float*)x, xs, B, T, heads, head_dim, pos0, rope_cos, rope_sin, rope_rows);
  else if (dtype == TSB200_BF16)
    rope_kernel<__nv_bfloat16><<<egrid(n), 256, 0, as_stream(stream)>>>((__nv_bfloat16*)x, xs, B, T, heads, head_dim, pos0, rope_cos, rope_sin, rope_rows);
  else
    return TSB200_ERR_UNSUPPORTED;
  TSB_LAUNCH_CHECK();
  return TSB200_OK;
}

int tsb200_add_rmsnorm(void* residual, const void* delta, const void* w, void* y, int dtype, int64_t M,
                       int64_t hidden, float eps, int variant, void* stream) {
  TSB_REQUIRE_DEVICE();
  if (M < 0 || hidden <= 0) return TSB200_ERR_ARG;
  if (variant != 0 && variant != 1) return TSB200_ERR_UNSUPPORTED;
  if (M == 0) return TSB200_OK;
  if (!residual || !w || !y) return TSB200_ERR_ARG;
  if (M > 0x7fffffffLL) return TSB200_ERR_UNSUPPORTED;
  if (dtype == TSB200_BF16 && variant == 0 && hidden % 8 == 0 && hidden <= 8192 && aligned(residual, 16) &&
      aligned(y, 16) && aligned(w, 16) && (!delta || aligned(delta, 16))) {
    TSB_CUDA(launch_kernel(add_rmsnorm_hf_bf16_kernel, dim3((unsigned)M), dim3(256), 0, as_stream(stream),
                           (__nv_bfloat16*)residual, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)w, (__nv_bfloat16*)y,
                           (int)hidden, eps));
    return TSB200_OK;
  }
  if (dtype == TSB200_F32)
    add_rmsnorm_kernel<float><<<(unsigned)M, 256, 0, as_stream(stream)>>>((float*)residual, (const float*)delta, (const float*)w, (float*)y, hidden, eps, variant);
  else if (dtype == TSB200_BF16)
    add_rmsnorm_kernel<__nv_bfloat16><<<(unsigned)M, 256, 0, as_stream(stream)>>>((__nv_bfloat16*)residual, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, hidden, eps, variant);
  else
    return TSB200_ERR_UNSUPPORTED;
  TSB_LAUNCH_CHECK();
  return TSB200_OK;
}

int tsb200_swiglu(const void* gate, const void* up, void* y, int dtype, int64_t M, int64_t n, int64_t gate_stride,
                  int64_t up_stride, int64_t y_stride, void* stream) {
  TSB_REQUIRE_DEVICE();
  if (M < 0 || n < 0) return TSB200_ERR_ARG;
  if (M == 0 || n == 0) return TSB200_OK;
  if (!gate || !up || !y || gate_stride < n || up_stride < n || y_stride < n) return TSB200_ERR_ARG;
  if (dtype == TSB200_F32)
    swiglu_kernel<float><<<egrid(M * n), 256, 0, as_stream(stream)>>>((const float*)gate, (const float*)up, (float*)y, M, n, gate_stride, up_stride, y_stride);
  else if (dtype == TSB200_BF16) {
    const bool vec = n % 8 == 0 && gate_stride % 8 == 0 && up_stride % 8 == 0 && y_stride % 8 == 0 && aligned(gate, 16) &&
                     aligned(up, 16) && aligned(y, 16) && M * n >= 8 * 256 * 148;
    if (vec)
      TSB_CUDA(launch_kernel(swiglu_bf16x8_kernel, dim3(egrid(M * n / 8)), dim3(256), 0, as_stream(stream), (const __nv_bfloat16*)gate,
                             (const __nv_bfloat16*)up, (__nv_bfloat16*)y, M, n / 8, gate_stride, up_stride, y_stride));
    else
      TSB_CUDA(launch_kernel(swiglu_kernel<__nv_bfloat16>, dim3(egrid(M * n)), dim3(256), 0, as_stream(stream),
                             (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, (__nv_bfloat16*)y, M, n, gate_stride, up_stride, y_stride));
  }
  else
    return TSB200_ERR_UNSUPPORTED;
  TSB_LAUNCH_CHECK();
  return TSB200_OK;
}

}  // extern "C"
