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
