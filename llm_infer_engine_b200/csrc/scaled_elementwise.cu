// Row kernels of blocks that scale a branch's output on its way into the residual stream, and of a feed-forward whose
// activation is a sum of normalised powers:
//
//   scaled_add_rmsnorm   h += s (.) (c1 d1 + c2 d2);  y = h / sqrt(mean(h^2) + eps) * w
//                        s a vector over the width (a learned scale per channel, or none), c1 and c2 constants, d1 and
//                        d2 branch outputs (the second optional: two mixers side by side); either half may be left out:
//                        no w and y = only the add, no d1 = only the norm
//   poly_norm            y = a N(z) + b N(z^2) + c N(z^3) + e, N(t) = t / sqrt(mean(t^2) + eps) over the row, powers
//                        element by element; a, b, c, e learned numbers in device memory
//
// The stream h and all arithmetic are float32 in both precisions; d1, d2, z and y have the activation type or float32.
// A block per row; the row is staged in shared memory between the sum of squares and the store.
#include "common.cuh"

namespace llmie {

__device__ __forceinline__ float load_any(const void* p, int dtype, size_t i) {
  return dtype == LLMIE_F32 ? reinterpret_cast<const float*>(p)[i] : to_f32(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ float4 load4_any(const void* p, int dtype, size_t i) {
  if (dtype == LLMIE_F32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
  const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&lo);
  raw.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

// The same kernel four channels a thread (d a multiple of 4, every row 16-byte aligned): the element's arithmetic is
// the scalar kernel's, only who sums which squares differs.
template <typename TY>
__global__ void scaled_add_rmsnorm4_kernel(float* __restrict__ h, const void* __restrict__ d1, int d1_dtype, float c1,
                                           const void* __restrict__ d2, int d2_dtype, float c2,
                                           const float* __restrict__ s, const float* __restrict__ w, float eps,
                                           TY* __restrict__ y, const int* __restrict__ rows, int d) {
  extern __shared__ float row_smem[];
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const size_t r_out = blockIdx.x;
  const size_t src = (rows ? (size_t)rows[r_out] : r_out) * d;
  float ss = 0.f;
  for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
    float4 x = *reinterpret_cast<const float4*>(h + src + c);
    if (d1) {
      const float4 a = load4_any(d1, d1_dtype, src + c);
      float4 b = make_float4(c1 * a.x, c1 * a.y, c1 * a.z, c1 * a.w);
      if (d2) {
        const float4 e = load4_any(d2, d2_dtype, src + c);
        b = make_float4(fmaf(c2, e.x, b.x), fmaf(c2, e.y, b.y), fmaf(c2, e.z, b.z), fmaf(c2, e.w, b.w));
      }
      if (s) {
        const float4 sv = *reinterpret_cast<const float4*>(s + c);
        x = make_float4(fmaf(sv.x, b.x, x.x), fmaf(sv.y, b.y, x.y), fmaf(sv.z, b.z, x.z), fmaf(sv.w, b.w, x.w));
      } else {
        x = make_float4(x.x + b.x, x.y + b.y, x.z + b.z, x.w + b.w);
      }
      if (!rows) *reinterpret_cast<float4*>(h + src + c) = x;
    }
    *reinterpret_cast<float4*>(row_smem + c) = x;
    ss = fmaf(x.x, x.x, ss);
    ss = fmaf(x.y, x.y, ss);
    ss = fmaf(x.z, x.z, ss);
    ss = fmaf(x.w, x.w, ss);
  }
  if (!y) return;
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)d + eps);
  for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
    const float4 x = *reinterpret_cast<const float4*>(row_smem + c);
    const float4 wv = *reinterpret_cast<const float4*>(w + c);
    store4(y + r_out * d + c, make_float4(x.x * rstd * wv.x, x.y * rstd * wv.y, x.z * rstd * wv.z, x.w * rstd * wv.w));
  }
}

template <typename TY>
__global__ void scaled_add_rmsnorm_kernel(float* __restrict__ h, const void* __restrict__ d1, int d1_dtype, float c1,
                                          const void* __restrict__ d2, int d2_dtype, float c2,
                                          const float* __restrict__ s, const float* __restrict__ w, float eps,
                                          TY* __restrict__ y, const int* __restrict__ rows, int d) {
  extern __shared__ float row_smem[];
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const size_t r_out = blockIdx.x;
  const size_t src = (rows ? (size_t)rows[r_out] : r_out) * d;
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float x = h[src + c];
    if (d1) {
      float b = c1 * load_any(d1, d1_dtype, src + c);
      if (d2) b = fmaf(c2, load_any(d2, d2_dtype, src + c), b);
      x = s ? fmaf(s[c], b, x) : x + b;
      if (!rows) h[src + c] = x;
    }
    row_smem[c] = x;
    ss = fmaf(x, x, ss);
  }
  if (!y) return;
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)d + eps);
  for (int c = threadIdx.x; c < d; c += blockDim.x) y[r_out * d + c] = from_f32<TY>(row_smem[c] * rstd * w[c]);
}

template <typename T>
__global__ void poly_norm_kernel(const T* __restrict__ z, const float* __restrict__ coef, float eps, T* __restrict__ y,
                                 int n) {
  extern __shared__ float row_smem[];
  __shared__ float red[32];
  pdl_launch_dependents();
  const float a = coef[0], b = coef[1], c3 = coef[2], e = coef[3];      // weights: no kernel writes them
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * n;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float x = to_f32(z[base + i]);
    const float x2 = x * x, x3 = x2 * x;
    row_smem[i] = x;
    s2 += x2;
    s4 = fmaf(x2, x2, s4);
    s6 = fmaf(x3, x3, s6);
  }
  s2 = block_sum(s2, red);
  s4 = block_sum(s4, red);
  s6 = block_sum(s6, red);
  const float r1 = a / sqrtf(s2 / (float)n + eps), r2 = b / sqrtf(s4 / (float)n + eps),
              r3 = c3 / sqrtf(s6 / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float x = row_smem[i];
    const float x2 = x * x;
    y[base + i] = from_f32<T>(fmaf(r1, x, fmaf(r2, x2, fmaf(r3, x2 * x, e))));
  }
}

// Eight values a thread (n a multiple of 8, rows 16-byte aligned); the element's arithmetic is the scalar kernel's.
template <typename T>
__global__ void poly_norm8_kernel(const T* __restrict__ z, const float* __restrict__ coef, float eps, T* __restrict__ y,
                                  int n) {
  extern __shared__ float row_smem[];
  __shared__ float red[32];
  pdl_launch_dependents();
  const float a = coef[0], b = coef[1], c3 = coef[2], e = coef[3];
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * n;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = threadIdx.x * 8; i < n; i += blockDim.x * 8) {
    float x[8];
    load8(z + base + i, x);
    store8(row_smem + i, x);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float x2 = x[k] * x[k], x3 = x2 * x[k];
      s2 += x2;
      s4 = fmaf(x2, x2, s4);
      s6 = fmaf(x3, x3, s6);
    }
  }
  s2 = block_sum(s2, red);
  s4 = block_sum(s4, red);
  s6 = block_sum(s6, red);
  const float r1 = a / sqrtf(s2 / (float)n + eps), r2 = b / sqrtf(s4 / (float)n + eps),
              r3 = c3 / sqrtf(s6 / (float)n + eps);
  for (int i = threadIdx.x * 8; i < n; i += blockDim.x * 8) {
    float xs[8], v[8];
    load8(row_smem + i, xs);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float x = xs[k];
      const float x2 = x * x;
      v[k] = fmaf(r1, x, fmaf(r2, x2, fmaf(r3, x2 * x, e)));
    }
    store8(y + base + i, v);
  }
}

static inline int row_block(int d) {
  int t = ((d / 4 + 31) / 32) * 32;
  return t < 64 ? 64 : (t > 512 ? 512 : t);
}

}  // namespace llmie

using namespace llmie;

// h float32 [T, d]; d1, d2 (d2 only with d1) [T, d] of their own dtypes, or null; s float32 [d] or null; w float32 [d]
// with y [n_out, d] of y_dtype, or both null (the add alone); rows int32 [n_out] or null (then n_out == T and h is
// updated in place). A row must fit shared memory (d <= 12,288).
extern "C" int llmie_scaled_add_rmsnorm(float* h, const void* d1, int d1_dtype, float c1, const void* d2, int d2_dtype,
                                        float c2, const float* s, const float* w, float eps, void* y, int y_dtype,
                                        const int* rows, int n_out, int d, cudaStream_t stream) {
  if (n_out < 0 || d <= 0 || !h || (d2 && !d1) || (!y) != (!w) || (!y && (rows || !d1))) return LLMIE_ERR_BAD_ARG;
  if ((y && y_dtype != LLMIE_F32 && y_dtype != LLMIE_BF16) || (d1 && d1_dtype != LLMIE_F32 && d1_dtype != LLMIE_BF16) ||
      (d2 && d2_dtype != LLMIE_F32 && d2_dtype != LLMIE_BF16))
    return LLMIE_ERR_DTYPE;
  if ((size_t)d * sizeof(float) > 48 * 1024) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (n_out == 0) return LLMIE_OK;
  const dim3 grid(n_out), block(row_block(d));
  const size_t smem = (size_t)d * sizeof(float);
  const bool by4 = d % 4 == 0 && aligned16(h) && (!s || aligned16(s)) && (!w || aligned16(w)) &&
                   (!d1 || aligned16(d1)) && (!d2 || aligned16(d2)) && (!y || aligned16(y));
  if (by4) {
    if (y && y_dtype == LLMIE_BF16)
      launch_k(scaled_add_rmsnorm4_kernel<__nv_bfloat16>, grid, block, smem, stream, h, d1, d1_dtype, c1, d2, d2_dtype,
               c2, s, w, eps, (__nv_bfloat16*)y, rows, d);
    else
      launch_k(scaled_add_rmsnorm4_kernel<float>, grid, block, smem, stream, h, d1, d1_dtype, c1, d2, d2_dtype, c2, s, w,
               eps, (float*)y, rows, d);
    LLMIE_LAUNCH_CHECK();
    return LLMIE_OK;
  }
  if (y && y_dtype == LLMIE_BF16)
    launch_k(scaled_add_rmsnorm_kernel<__nv_bfloat16>, grid, block, smem, stream, h, d1, d1_dtype, c1, d2, d2_dtype, c2, s,
             w, eps, (__nv_bfloat16*)y, rows, d);
  else
    launch_k(scaled_add_rmsnorm_kernel<float>, grid, block, smem, stream, h, d1, d1_dtype, c1, d2, d2_dtype, c2, s, w,
             eps, (float*)y, rows, d);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// z, y [T, n] of `dtype`; coef float32 [4] = (a, b, c, e) on the device. n <= 51,200 (a row in shared memory).
extern "C" int llmie_poly_norm(const void* z, const float* coef, float eps, void* y, int n_tokens, int n, int dtype,
                               cudaStream_t stream) {
  if (n_tokens < 0 || n <= 0 || !coef) return LLMIE_ERR_BAD_ARG;
  if ((size_t)n * sizeof(float) > 200 * 1024) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (n_tokens == 0) return LLMIE_OK;
  const dim3 grid(n_tokens), block(row_block(n));
  const size_t smem = (size_t)n * sizeof(float);
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(poly_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(poly_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  if (n % 8 == 0 && aligned16(z) && aligned16(y)) {
    const dim3 block8(row_block(n / 2));
    if (smem > 48 * 1024) {
      cudaFuncSetAttribute(poly_norm8_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      cudaFuncSetAttribute(poly_norm8_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    if (dtype == LLMIE_F32)
      launch_k(poly_norm8_kernel<float>, grid, block8, smem, stream, (const float*)z, coef, eps, (float*)y, n);
    else if (dtype == LLMIE_BF16)
      launch_k(poly_norm8_kernel<__nv_bfloat16>, grid, block8, smem, stream, (const __nv_bfloat16*)z, coef, eps,
               (__nv_bfloat16*)y, n);
    else
      return LLMIE_ERR_DTYPE;
    LLMIE_LAUNCH_CHECK();
    return LLMIE_OK;
  }
  if (dtype == LLMIE_F32)
    launch_k(poly_norm_kernel<float>, grid, block, smem, stream, (const float*)z, coef, eps, (float*)y, n);
  else if (dtype == LLMIE_BF16)
    launch_k(poly_norm_kernel<__nv_bfloat16>, grid, block, smem, stream, (const __nv_bfloat16*)z, coef, eps,
             (__nv_bfloat16*)y, n);
  else
    return LLMIE_ERR_DTYPE;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}
