// Pointwise kernels of blocks whose two branches read ONE norm and are added to the stream together, and of
// gated feed-forwards with a choice of activation:
//
//   add_dyt      h += d1 + d2;  y = tanh(alpha * h) * w + b      Dynamic Tanh: a norm without mean or variance,
//                                                                so no row is reduced and the kernel is a plain
//                                                                element-wise sweep; alpha is a scalar on the device
//   gated_act    out = act(gate) * up over [gate | up] rows      act by code (common.cuh: apply_act)
//   scale_rows   x *= s                                          the logits of designs that scale them
//   cap_rows     x = c tanh(x / c)                                   the logits of designs that cap them
//
// The stream h and all arithmetic are float32 in both precisions; d1, d2 and y have the activation type or float32.
#include "common.cuh"

namespace llmie {

__device__ __forceinline__ float load_as_f32(const void* p, int dtype, size_t i) {
  return dtype == LLMIE_F32 ? reinterpret_cast<const float*>(p)[i] : to_f32(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// One thread per element of the produced rows. rows == nullptr: every row of h, and h is updated in place;
// otherwise only the listed rows are produced and h stays as it is.
template <typename TY>
__global__ void add_dyt_kernel(float* __restrict__ h, const void* __restrict__ d1, int d1_dtype,
                               const void* __restrict__ d2, int d2_dtype, const float* __restrict__ alpha,
                               const float* __restrict__ w, const float* __restrict__ b, TY* __restrict__ y,
                               const int* __restrict__ rows, int d, size_t total) {
  pdl_launch_dependents();
  const float a = alpha[0];          // a weight: no kernel writes it
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t r_out = i / d;
    const int c = (int)(i - r_out * d);
    const size_t src = rows ? (size_t)rows[r_out] * d + c : i;
    float x = h[src];
    if (d1) x += load_as_f32(d1, d1_dtype, src);
    if (d2) x += load_as_f32(d2, d2_dtype, src);
    if (!rows && (d1 || d2)) h[src] = x;
    y[i] = from_f32<TY>(tanhf(a * x) * w[c] + b[c]);
  }
}

// The same, eight elements a thread with 16-byte accesses: d % 8 == 0 and all pointers 16-byte aligned.
template <typename TY, typename TD>
__global__ void add_dyt_vec_kernel(float* __restrict__ h, const TD* __restrict__ d1, const TD* __restrict__ d2,
                                   const float* __restrict__ alpha, const float* __restrict__ w,
                                   const float* __restrict__ b, TY* __restrict__ y, const int* __restrict__ rows,
                                   int d, size_t total8) {
  pdl_launch_dependents();
  const float a = alpha[0];
  pdl_wait();
  const int per_row = d / 8;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total8; i += stride) {
    const size_t r_out = i / per_row;
    const int c = (int)(i - r_out * per_row) * 8;
    const size_t src = (rows ? (size_t)rows[r_out] : r_out) * d + c;
    float x[8], t[8];
    load8(h + src, x);
    if (d1) {
      load8(d1 + src, t);
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] += t[e];
    }
    if (d2) {
      load8(d2 + src, t);
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] += t[e];
    }
    if (!rows && (d1 || d2)) store8(h + src, x);
    float wv[8], bv[8], o[8];
    load8(w + c, wv);
    load8(b + c, bv);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = tanhf(a * x[e]) * wv[e] + bv[e];
    store8(y + r_out * d + c, o);
  }
}

template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int ff, int act, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t t = i / ff;
    const int j = (int)(i - t * ff);
    const float g = to_f32(gate_up[t * 2 * ff + j]);
    const float u = to_f32(gate_up[t * 2 * ff + ff + j]);
    out[i] = from_f32<T>(apply_act(g, act) * u);
  }
}

// ff % 8 == 0, 16-byte aligned: eight outputs a thread, a row of blocks per token (no index is divided)
template <typename T>
__global__ void gated_act_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int ff, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.y;
  const T* row = gate_up + t * 2 * (size_t)ff;
  for (int j = (blockIdx.x * blockDim.x + threadIdx.x) * 8; j < ff; j += gridDim.x * blockDim.x * 8) {
    float g[8], u[8], o[8];
    load8(row + j, g);
    load8(row + ff + j, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = apply_act(g[e], act) * u[e];
    store8(out + t * ff + j, o);
  }
}

__global__ void scale_rows_kernel(float* __restrict__ x, float s, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) x[i] *= s;
}

__global__ void cap_rows_kernel(float* __restrict__ x, float c, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) x[i] = c * tanhf(x[i] / c);
}

static inline int sweep_blocks(size_t items, int threads) {
  size_t b = (items + threads - 1) / threads;
  return (int)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace llmie

using namespace llmie;

// h float32 [T, d]; d1, d2 (each may be null) [T, d] of their own dtypes; alpha float32 [1]; w, b float32 [d];
// y [n_out, d] of y_dtype; rows int32 [n_out] or null (then n_out == T and h is updated in place).
extern "C" int llmie_add_dyt(float* h, const void* d1, int d1_dtype, const void* d2, int d2_dtype, const float* alpha,
                             const float* w, const float* b, void* y, int y_dtype, const int* rows, int n_out, int d,
                             cudaStream_t stream) {
  if (n_out == 0) return LLMIE_OK;
  if (n_out < 0 || d <= 0 || !h || !alpha || !w || !b || !y) return LLMIE_ERR_BAD_ARG;
  if ((y_dtype != LLMIE_F32 && y_dtype != LLMIE_BF16) || (d1 && d1_dtype != LLMIE_F32 && d1_dtype != LLMIE_BF16) ||
      (d2 && d2_dtype != LLMIE_F32 && d2_dtype != LLMIE_BF16))
    return LLMIE_ERR_DTYPE;
  if (n_out == 0) return LLMIE_OK;
  if (!d1 && d2) { d1 = d2; d1_dtype = d2_dtype; d2 = nullptr; }
  const size_t total = (size_t)n_out * d;
  const bool same = !d2 || d1_dtype == d2_dtype;
  const bool vec = d % 8 == 0 && same && aligned16(h) && aligned16(w) && aligned16(b) && aligned16(y) &&
                   (!d1 || aligned16(d1)) && (!d2 || aligned16(d2));
  if (vec) {
    const size_t total8 = total / 8;
    const int blocks = sweep_blocks(total8, 256);
    const bool df32 = !d1 || d1_dtype == LLMIE_F32;
    if (y_dtype == LLMIE_F32) {
      if (df32) launch_k(add_dyt_vec_kernel<float, float>, dim3(blocks), dim3(256), 0, stream, h, (const float*)d1, (const float*)d2, alpha, w, b, (float*)y, rows, d, total8);
      else launch_k(add_dyt_vec_kernel<float, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, h, (const __nv_bfloat16*)d1, (const __nv_bfloat16*)d2, alpha, w, b, (float*)y, rows, d, total8);
    } else {
      if (df32) launch_k(add_dyt_vec_kernel<__nv_bfloat16, float>, dim3(blocks), dim3(256), 0, stream, h, (const float*)d1, (const float*)d2, alpha, w, b, (__nv_bfloat16*)y, rows, d, total8);
      else launch_k(add_dyt_vec_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, h, (const __nv_bfloat16*)d1, (const __nv_bfloat16*)d2, alpha, w, b, (__nv_bfloat16*)y, rows, d, total8);
    }
  } else {
    const int blocks = sweep_blocks(total, 256);
    if (y_dtype == LLMIE_F32)
      launch_k(add_dyt_kernel<float>, dim3(blocks), dim3(256), 0, stream, h, d1, d1_dtype, d2, d2_dtype, alpha, w, b, (float*)y, rows, d, total);
    else
      launch_k(add_dyt_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, h, d1, d1_dtype, d2, d2_dtype, alpha, w, b, (__nv_bfloat16*)y, rows, d, total);
  }
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// gate_up [T, 2 ff] = [gate | up] per row; out [T, ff]; both of `dtype`; act one of the activation codes.
extern "C" int llmie_gated_act(const void* gate_up, void* out, int n_tokens, int ff, int act, int dtype,
                               cudaStream_t stream) {
  if (n_tokens < 0 || ff <= 0 || act < 0 || act > 4) return LLMIE_ERR_BAD_ARG;
  if (dtype != LLMIE_F32 && dtype != LLMIE_BF16) return LLMIE_ERR_DTYPE;
  if (n_tokens == 0) return LLMIE_OK;
  const size_t total = (size_t)n_tokens * ff;
  const bool vec = ff % 8 == 0 && aligned16(gate_up) && aligned16(out) && n_tokens <= 65535;
  if (vec) {
    const int bx = (ff / 8 + 127) / 128;
    dim3 grid(bx, n_tokens);
    if (dtype == LLMIE_F32) launch_k(gated_act_vec_kernel<float>, grid, dim3(128), 0, stream, (const float*)gate_up, (float*)out, ff, act);
    else launch_k(gated_act_vec_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, ff, act);
  } else {
    const int blocks = sweep_blocks(total, 256);
    if (dtype == LLMIE_F32) launch_k(gated_act_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gate_up, (float*)out, ff, act, total);
    else launch_k(gated_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, ff, act, total);
  }
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

extern "C" int llmie_scale_rows(float* x, float s, long long n, cudaStream_t stream) {
  if (n == 0) return LLMIE_OK;
  if (n < 0 || !x) return LLMIE_ERR_BAD_ARG;
  launch_k(scale_rows_kernel, dim3(sweep_blocks((size_t)n, 256)), dim3(256), 0, stream, x, s, (size_t)n);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// x float32 [n] = c tanh(x / c), c > 0.
extern "C" int llmie_cap_rows(float* x, float c, long long n, cudaStream_t stream) {
  if (n == 0) return LLMIE_OK;
  if (n < 0 || !x || !(c > 0.f)) return LLMIE_ERR_BAD_ARG;
  launch_k(cap_rows_kernel, dim3(sweep_blocks((size_t)n, 256)), dim3(256), 0, stream, x, c, (size_t)n);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}
