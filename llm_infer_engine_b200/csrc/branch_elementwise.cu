// Memory-bound kernels of layers whose norm sits on the OUTPUT of a branch (h += norm(f(h))), of an embedding stage
// with learned positions, of feed-forwards with biases, and of attention layers that normalise the whole query
// and key projections and may blend their values with those of an earlier layer.
//
// Everything that is summed, normalised or blended here is float32: the residual stream, the sums of squares,
// the norm's scale, the blend. Activations between products are T (float or bfloat16), rounded once at the store.
#include "common.cuh"
#include <math.h>

namespace llmie {

static inline int row_threads(int d) {
  int t = ((d + 31) / 32) * 32;
  return t < 32 ? 32 : (t > 512 ? 512 : t);
}

// ------------------------------------------------------------------------------------------
// Embedding stage: x = h[t] * scale + pos_table[tok_pos[t]];  h[t] = norm_w ? x * rsqrt(mean(x^2) + eps) * norm_w : x;
// act[t] = h[t] rounded to A (optional). pos_table and norm_w are optional. One block per token.
template <typename P, typename A>
__global__ void scale_pos_norm_kernel(float* __restrict__ h, float scale, const P* __restrict__ pos_table,
                                      int table_len, const int* __restrict__ tok_pos,
                                      const float* __restrict__ norm_w, float eps, A* __restrict__ act, int d) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row_buf[];
  __shared__ float red[32];
  const int t = blockIdx.x;
  float* hr = h + (size_t)t * d;
  const P* pr = nullptr;
  if (pos_table) {
    int p = tok_pos[t];
    p = p < 0 ? 0 : (p >= table_len ? table_len - 1 : p);     // the host refuses longer sequences
    pr = pos_table + (size_t)p * d;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float x = hr[i] * scale;
    if (pr) x += to_f32(pr[i]);
    row_buf[i] = x;
    ss += x * x;
  }
  float rstd = 1.f;
  if (norm_w) {
    ss = block_sum(ss, red);
    rstd = 1.f / sqrtf(ss / (float)d + eps);
  }
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float y = norm_w ? row_buf[i] * rstd * norm_w[i] : row_buf[i];
    hr[i] = y;
    if (act) act[(size_t)t * d + i] = from_f32<A>(y);
  }
}

// ------------------------------------------------------------------------------------------
// Norm on a branch's output, then the residual add:
//   x = y[t] (+ bias);  h[t] += x * rsqrt(mean(x^2) + eps) * w;  act[t] = h[t] rounded to A (optional)
// One block per row.
template <typename Y, typename A>
__global__ void branch_norm_add_kernel(float* __restrict__ h, const Y* __restrict__ y, const float* __restrict__ bias,
                                       const float* __restrict__ w, float eps, A* __restrict__ act, int d) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row_buf[];
  __shared__ float red[32];
  const int t = blockIdx.x;
  const Y* yr = y + (size_t)t * d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float x = to_f32(yr[i]);
    if (bias) x += bias[i];
    row_buf[i] = x;
    ss += x * x;
  }
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)d + eps);
  float* hr = h + (size_t)t * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float s = hr[i] + row_buf[i] * rstd * w[i];
    hr[i] = s;
    if (act) act[(size_t)t * d + i] = from_f32<A>(s);
  }
}

// The same for rows of at most 8 * 1024 elements with d % 8 == 0: a thread owns one run of 8 elements, kept in
// registers between the two passes, with 16-byte loads and stores.
template <typename Y, typename A>
__global__ void branch_norm_add_vec_kernel(float* __restrict__ h, const Y* __restrict__ y,
                                           const float* __restrict__ bias, const float* __restrict__ w, float eps,
                                           A* __restrict__ act, int d) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const int t = blockIdx.x;
  const int i = threadIdx.x * 8;
  const bool active = i < d;
  float x[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) x[e] = 0.f;
  if (active) {
    load8(y + (size_t)t * d + i, x);
    if (bias) {
      float b[8];
      load8(bias + i, b);
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] += b[e];
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)d + eps);
  if (active) {
    float wv[8], hv[8];
    load8(w + i, wv);
    float* hr = h + (size_t)t * d + i;
    load8(hr, hv);
#pragma unroll
    for (int e = 0; e < 8; ++e) hv[e] += x[e] * rstd * wv[e];
    store8(hr, hv);
    if (act) store8(act + (size_t)t * d + i, hv);
  }
}

// ------------------------------------------------------------------------------------------
// Norm AFTER the residual sum (post-norm), with a learned scale per channel on the branch:
//   x = alpha * h[t] + s (.) y[t];  h[t] = x * rsqrt(mean(x^2) + eps) * w;  act[t] = h[t] rounded to A (optional)
// s is optional (null = ones). The stream stays float32. One block per row.
template <typename Y, typename A>
__global__ void scaled_sum_norm_kernel(float* __restrict__ h, const Y* __restrict__ y, const float* __restrict__ s,
                                       float alpha, const float* __restrict__ w, float eps, A* __restrict__ act,
                                       int d) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row_buf[];
  __shared__ float red[32];
  const int t = blockIdx.x;
  const Y* yr = y + (size_t)t * d;
  float* hr = h + (size_t)t * d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float b = to_f32(yr[i]) * (s ? s[i] : 1.f);
    const float x = fmaf(alpha, hr[i], b);
    row_buf[i] = x;
    ss += x * x;
  }
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = row_buf[i] * rstd * w[i];
    hr[i] = v;
    if (act) act[(size_t)t * d + i] = from_f32<A>(v);
  }
}

// The same for rows of at most 8 * 1024 elements with d % 8 == 0: a thread owns one run of 8 elements, kept in
// registers between the two passes, with 16-byte loads and stores.
template <typename Y, typename A>
__global__ void scaled_sum_norm_vec_kernel(float* __restrict__ h, const Y* __restrict__ y,
                                           const float* __restrict__ s, float alpha, const float* __restrict__ w,
                                           float eps, A* __restrict__ act, int d) {
  pdl_launch_dependents();
  __shared__ float red[32];
  const int t = blockIdx.x;
  const int i = threadIdx.x * 8;
  const bool active = i < d;
  float x[8], sv[8], wv[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { x[e] = 0.f; sv[e] = 1.f; wv[e] = 0.f; }
  if (active) {                      // weights: no kernel writes them
    if (s) load8(s + i, sv);
    load8(w + i, wv);
  }
  pdl_wait();
  float* hr = h + (size_t)t * d + i;
  if (active) {
    float hv[8];
    load8(y + (size_t)t * d + i, x);
    load8(hr, hv);
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] = fmaf(alpha, hv[e], x[e] * sv[e]);
  }
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)d + eps);
  if (active) {
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] = x[e] * rstd * wv[e];
    store8(hr, x);
    if (act) store8(act + (size_t)t * d + i, x);
  }
}

// RMS norm of a run of columns of wider rows: out[t, i] = x * rsqrt(mean(x^2) + eps) * w[i], x = src[t * ld + off + i],
// i < n (the latent that queries pass through). float32 arithmetic, one rounding at the store. One block per row.
template <typename T>
__global__ void rmsnorm_cols_kernel(const T* __restrict__ src, int ld, int off, const float* __restrict__ w, float eps,
                                    T* __restrict__ out, int n) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const int t = blockIdx.x;
  const T* xr = src + (size_t)t * ld + off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) { const float x = to_f32(xr[i]); ss += x * x; }
  ss = block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    out[(size_t)t * n + i] = from_f32<T>(to_f32(xr[i]) * rstd * w[i]);
}

// ------------------------------------------------------------------------------------------
// out[t, j] = act(u[t, j] + bias[j]); bias optional. Activations: 0 none, 1 relu, 2 relu squared, 3 gelu (tanh
// form), 4 silu.
template <typename T, typename O>
__global__ void bias_act_kernel(const T* __restrict__ u, const float* __restrict__ bias, O* __restrict__ out, int n,
                                size_t total, int act) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    float z = to_f32(u[i]);
    if (bias) z += bias[i % n];
    out[i] = from_f32<O>(apply_act(z, act));
  }
}

// The same, eight outputs a thread with 16-byte loads (n % 8 == 0): grid (column blocks, rows), no index division.
template <typename T, typename O>
__global__ void bias_act_vec_kernel(const T* __restrict__ u, const float* __restrict__ bias, O* __restrict__ out, int n8,
                                    int n_tokens, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const int j8 = blockIdx.x * blockDim.x + threadIdx.x;
  if (j8 >= n8) return;
  float b[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) b[e] = 0.f;
  if (bias) load8(bias + (size_t)j8 * 8, b);
  // two rows at a time: both loads are on their way before either is used
  int t = blockIdx.y;
  for (; t + (int)gridDim.y < n_tokens; t += 2 * gridDim.y) {
    const size_t o0 = ((size_t)t * n8 + j8) * 8, o1 = ((size_t)(t + gridDim.y) * n8 + j8) * 8;
    float z0[8], z1[8];
    load8(u + o0, z0);
    load8(u + o1, z1);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      z0[e] = apply_act(z0[e] + b[e], act);
      z1[e] = apply_act(z1[e] + b[e], act);
    }
    store8(out + o0, z0);
    store8(out + o1, z1);
  }
  if (t < n_tokens) {
    float z[8];
    load8(u + ((size_t)t * n8 + j8) * 8, z);
#pragma unroll
    for (int e = 0; e < 8; ++e) z[e] = apply_act(z[e] + b[e], act);
    store8(out + ((size_t)t * n8 + j8) * 8, z);
  }
}

// out = float32 -> A, element by element
template <typename A>
__global__ void cast_rows_kernel(const float* __restrict__ x, A* __restrict__ out, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) out[i] = from_f32<A>(x[i]);
}

// out[t, j] *= sigmoid(gate[t * ld + j / group]): group 1 = a gate per element, group = a head's value size = one
// gate per head
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ out, const T* __restrict__ gate, int ld, int n, int group,
                                    size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t t = i / n;
    const int j = (int)(i - t * n);
    const float g = to_f32(gate[t * ld + (group > 1 ? j / group : j)]);
    out[i] = from_f32<T>(to_f32(out[i]) / (1.f + expf(-g)));
  }
}

// A temperature on the queries that grows with the position p: 1 + coef * ln(floor((p + 1) / every) + 1), float32.
__device__ __forceinline__ float query_temperature(int pos, float coef, int every) {
  return 1.f + coef * logf((float)((pos + 1) / every) + 1.f);
}

// ------------------------------------------------------------------------------------------
// Whole-projection query/key norm, value blending and the cache write of one attention layer.
// With temp_every > 0 the queries are also multiplied by query_temperature(position).
//   proj[t] (row stride ld) = [ q : n_q*hd | k : n_kv*hd | v : n_kv*hdv | ... ]
//   q_out[t]  = q * rsqrt(mean over ALL n_q*hd elements of q^2 + eps) * q_w      (q_w null: q unchanged)
//   k' likewise over all n_kv*hd elements with k_w;  v' = v_first ? (1 - lam) v + lam v_first[t] : v
//   k_cache[page(t), hk, pos % P, :] = k'   v_cache[...] = v'   (only with write_kv)
// lam is read from device memory (a checkpoint scalar). One block per token.
template <typename T>
__global__ void qk_norm_store_kernel(const T* __restrict__ proj, int ld, T* __restrict__ q_out, T* __restrict__ k_cache,
                                     T* __restrict__ v_cache, const float* __restrict__ q_w,
                                     const float* __restrict__ k_w, float eps, const float* __restrict__ lam_ptr,
                                     const T* __restrict__ v_first, int v_first_ld, const int* __restrict__ tok_pos,
                                     const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                                     const int* __restrict__ block_table, int max_pages, int page_size, int n_q,
                                     int n_kv, int hd, int hdv, int write_kv, float temp_coef, int temp_every) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const int t = blockIdx.x;
  const int nq = n_q * hd, nk = n_kv * hd, nv = n_kv * hdv;
  const T* qs = proj + (size_t)t * ld;
  const T* ks = qs + nq;
  const T* vs = ks + nk;
  float rq = 1.f, rk = 1.f;
  if (q_w) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float x = to_f32(qs[i]); ss += x * x; }
    ss = block_sum(ss, red);
    rq = 1.f / sqrtf(ss / (float)nq + eps);
  }
  if (k_w && write_kv) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float x = to_f32(ks[i]); ss += x * x; }
    ss = block_sum(ss, red);
    rk = 1.f / sqrtf(ss / (float)nk + eps);
  }
  const int pos = tok_pos[t];
  const bool temp = temp_every > 0;
  if (temp) rq *= query_temperature(pos, temp_coef, temp_every);
  T* qo = q_out + (size_t)t * nq;
  for (int i = threadIdx.x; i < nq; i += blockDim.x)
    qo[i] = (q_w || temp) ? from_f32<T>(to_f32(qs[i]) * rq * (q_w ? q_w[i] : 1.f)) : qs[i];
  if (!write_kv) return;
  const int slot = seq_slot[tok_seq[t]];
  const int page = block_table[(size_t)slot * max_pages + pos / page_size];
  const int in_page = pos % page_size;
  for (int i = threadIdx.x; i < nk; i += blockDim.x) {
    const int hk = i / hd, e = i - hk * hd;
    const size_t dst = (((size_t)page * n_kv + hk) * page_size + in_page) * hd + e;
    k_cache[dst] = k_w ? from_f32<T>(to_f32(ks[i]) * rk * k_w[i]) : ks[i];
  }
  const float lam = v_first ? *lam_ptr : 0.f;
  const T* vf = v_first ? v_first + (size_t)t * v_first_ld : nullptr;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const int hk = i / hdv, e = i - hk * hdv;
    const size_t dst = (((size_t)page * n_kv + hk) * page_size + in_page) * hdv + e;
    T v = vs[i];
    if (vf) v = from_f32<T>((1.f - lam) * to_f32(v) + lam * to_f32(vf[i]));
    v_cache[dst] = v;
  }
}

// The same with 16-byte loads and stores, for head sizes and a row pitch that are multiples of 8 (and 16-byte
// aligned tensors). A token is one block's work and a short chain (loads, one block reduction, stores), so what
// counts is how many tokens an SM has in flight: blocks are small (128 threads where that covers the query
// projection with R <= 4 runs of 8 elements a thread) and a thread's runs of q stay in registers between the sum
// and the store. Keys are read again for the store (from L1), values once. The lookups of the token's cache page,
// a chain of three dependent loads, are placed so that no data load waits behind them.
template <typename T, int R>
__global__ void qk_norm_store_vec_kernel(const T* __restrict__ proj, int ld, T* __restrict__ q_out,
                                         T* __restrict__ k_cache, T* __restrict__ v_cache,
                                         const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                         const float* __restrict__ lam_ptr, const T* __restrict__ v_first,
                                         int v_first_ld, const int* __restrict__ tok_pos,
                                         const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                                         const int* __restrict__ block_table, int max_pages, int page_size, int n_q,
                                         int n_kv, int hd, int hdv, int write_kv, float temp_coef, int temp_every) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[2][32];
  const int t = blockIdx.x;
  const int nq = n_q * hd, nk = n_kv * hd, nv = n_kv * hdv;
  const T* qs = proj + (size_t)t * ld;
  const T* ks = qs + nq;
  const T* vs = ks + nk;
  const int i0 = threadIdx.x * 8, step = blockDim.x * 8;
  const bool temp = temp_every > 0;
  const int pos = (write_kv || temp) ? tok_pos[t] : 0;
  const int sq_idx = write_kv ? tok_seq[t] : 0;
  float q[R][8];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = i0 + r * step;
    if (i < nq) {
      load8(qs + i, q[r]);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) q[r][e] = 0.f;
    }
  }
  // the second link of the page lookup waits for the first here, with every load of q already on its way
  const int slot = write_kv ? seq_slot[sq_idx] : 0;
  float sq = 0.f, sk = 0.f;
  if (k_w && write_kv) {
    for (int i = i0; i < nk; i += step) {
      float x[8];
      load8(ks + i, x);
#pragma unroll
      for (int e = 0; e < 8; ++e) sk += x[e] * x[e];
    }
  }
  if (q_w) {
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int e = 0; e < 8; ++e) sq += q[r][e] * q[r][e];
  }
  // the third link is requested before the block reduction and has arrived when the stores need it
  const int page = write_kv ? block_table[(size_t)slot * max_pages + pos / page_size] : 0;
  {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = (blockDim.x + 31) >> 5;
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    if (lane == 0) {
      red[0][warp] = sq;
      red[1][warp] = sk;
    }
    __syncthreads();
    sq = warp_sum(lane < n_warps ? red[0][lane] : 0.f);
    sk = warp_sum(lane < n_warps ? red[1][lane] : 0.f);
  }
  float rq = q_w ? 1.f / sqrtf(sq / (float)nq + eps) : 1.f;
  if (temp) rq *= query_temperature(pos, temp_coef, temp_every);
  const float rk = (k_w && write_kv) ? 1.f / sqrtf(sk / (float)nk + eps) : 1.f;
  T* qo = q_out + (size_t)t * nq;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = i0 + r * step;
    if (i < nq) {
      if (q_w) {
        float w8[8];
        load8(q_w + i, w8);
#pragma unroll
        for (int e = 0; e < 8; ++e) q[r][e] = q[r][e] * rq * w8[e];
      } else if (temp) {
#pragma unroll
        for (int e = 0; e < 8; ++e) q[r][e] *= rq;
      }
      store8(qo + i, q[r]);
    }
  }
  if (!write_kv) return;
  const int in_page = pos % page_size;
  for (int i = i0; i < nk; i += step) {
    const int hk = i / hd, e0 = i - hk * hd;
    float x[8];
    load8(ks + i, x);
    if (k_w) {
      float w8[8];
      load8(k_w + i, w8);
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] = x[e] * rk * w8[e];
    }
    store8(k_cache + (((size_t)page * n_kv + hk) * page_size + in_page) * hd + e0, x);
  }
  const float lam = v_first ? *lam_ptr : 0.f;
  const T* vf = v_first ? v_first + (size_t)t * v_first_ld : nullptr;
  for (int i = i0; i < nv; i += step) {
    const int hk = i / hdv, e0 = i - hk * hdv;
    float x[8];
    load8(vs + i, x);
    if (vf) {
      float f[8];
      load8(vf + i, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] = (1.f - lam) * x[e] + lam * f[e];
    }
    store8(v_cache + (((size_t)page * n_kv + hk) * page_size + in_page) * hdv + e0, x);
  }
}

template <typename A> struct DT { };
template <> struct DT<float> { static constexpr int code = LLMIE_F32; };
template <> struct DT<__nv_bfloat16> { static constexpr int code = LLMIE_BF16; };

static inline int flat_blocks(size_t total) {
  size_t b = (total + 255) / 256;
  return (int)(b > 148 * 16 ? 148 * 16 : (b == 0 ? 1 : b));
}

}  // namespace llmie

using namespace llmie;

// h float32 [T, d] in place; pos_table [table_len, d] of pos_dtype or null; norm_w float32 [d] or null;
// act [T, d] of act_dtype or null.
extern "C" int llmie_scale_pos_norm(float* h, float scale, const void* pos_table, int pos_dtype, int table_len,
                                    const int* tok_pos, const float* norm_w, float eps, void* act, int act_dtype,
                                    int n_tokens, int d, cudaStream_t stream) {
  if (n_tokens < 0 || d <= 0 || (pos_table && (table_len <= 0 || !tok_pos))) return LLMIE_ERR_BAD_ARG;
  if (n_tokens == 0) return LLMIE_OK;
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 48 * 1024) return LLMIE_ERR_UNSUPPORTED_SIZE;
  const dim3 grid(n_tokens), block(row_threads(d));
#define LLMIE_SPN(P, A)                                                                                          \
  launch_k(scale_pos_norm_kernel<P, A>, grid, block, smem, stream, h, scale, (const P*)pos_table, table_len,     \
           tok_pos, norm_w, eps, (A*)act, d)
  const bool pos_bf16 = pos_table && pos_dtype == LLMIE_BF16;
  if (pos_table && pos_dtype != LLMIE_BF16 && pos_dtype != LLMIE_F32) return LLMIE_ERR_DTYPE;
  if (act && act_dtype != LLMIE_BF16 && act_dtype != LLMIE_F32) return LLMIE_ERR_DTYPE;
  const bool act_bf16 = act && act_dtype == LLMIE_BF16;
  if (pos_bf16 && act_bf16) LLMIE_SPN(__nv_bfloat16, __nv_bfloat16);
  else if (pos_bf16) LLMIE_SPN(__nv_bfloat16, float);
  else if (act_bf16) LLMIE_SPN(float, __nv_bfloat16);
  else LLMIE_SPN(float, float);
#undef LLMIE_SPN
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// h float32 [T, d] += norm(y (+ bias)) * w; y [T, d] of y_dtype; bias float32 [d] or null; act of act_dtype or null.
extern "C" int llmie_branch_norm_add(float* h, const void* y, int y_dtype, const float* bias, const float* w, float eps,
                                     void* act, int act_dtype, int n_tokens, int d, cudaStream_t stream) {
  if (n_tokens < 0 || d <= 0 || !w || !y) return LLMIE_ERR_BAD_ARG;
  if (n_tokens == 0) return LLMIE_OK;
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 48 * 1024) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (y_dtype != LLMIE_BF16 && y_dtype != LLMIE_F32) return LLMIE_ERR_DTYPE;
  if (act && act_dtype != LLMIE_BF16 && act_dtype != LLMIE_F32) return LLMIE_ERR_DTYPE;
  const bool vec = d % 8 == 0 && d <= 8 * 1024 && aligned16(h) && aligned16(y) && aligned16(w) &&
                   (!bias || aligned16(bias)) && (!act || aligned16(act));
  const dim3 grid(n_tokens), block(vec ? ((d / 8 + 31) / 32) * 32 : row_threads(d));
#define LLMIE_BNA(Y, A)                                                                                          \
  if (vec) launch_k(branch_norm_add_vec_kernel<Y, A>, grid, block, 0, stream, h, (const Y*)y, bias, w, eps, (A*)act, d); \
  else launch_k(branch_norm_add_kernel<Y, A>, grid, block, smem, stream, h, (const Y*)y, bias, w, eps, (A*)act, d)
  const bool y_bf16 = y_dtype == LLMIE_BF16, act_bf16 = act && act_dtype == LLMIE_BF16;
  if (y_bf16 && act_bf16) { LLMIE_BNA(__nv_bfloat16, __nv_bfloat16); }
  else if (y_bf16) { LLMIE_BNA(__nv_bfloat16, float); }
  else if (act_bf16) { LLMIE_BNA(float, __nv_bfloat16); }
  else { LLMIE_BNA(float, float); }
#undef LLMIE_BNA
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// out[T, n] (out_dtype) = act(u[T, n] (u_dtype) + bias[n]); bias float32 or null.
extern "C" int llmie_bias_act(const void* u, int u_dtype, const float* bias, void* out, int out_dtype, int n_tokens,
                              int n, int act, cudaStream_t stream) {
  if (n_tokens < 0 || n <= 0 || act < 0 || act > 4) return LLMIE_ERR_BAD_ARG;
  if (n_tokens == 0) return LLMIE_OK;
  const size_t total = (size_t)n_tokens * n;
  const bool vec = n % 8 == 0 && aligned16(u) && aligned16(out) && (!bias || aligned16(bias));
  const int vthreads = n / 8 >= 256 ? 256 : ((n / 8 + 31) / 32) * 32;
  const int col_blocks = vec ? (n / 8 + vthreads - 1) / vthreads : 1;
  int row_blocks = (148 * 16 + col_blocks - 1) / col_blocks;        // a few thousand blocks, several rows a thread
  row_blocks = row_blocks < n_tokens ? row_blocks : n_tokens;
  const dim3 grid(vec ? col_blocks : flat_blocks(total), vec ? row_blocks : 1);
  const dim3 block(vec ? vthreads : 256);
#define LLMIE_BA(T, O)                                                                                             \
  if (vec) launch_k(bias_act_vec_kernel<T, O>, grid, block, 0, stream, (const T*)u, bias, (O*)out, n / 8, n_tokens, act); \
  else launch_k(bias_act_kernel<T, O>, grid, block, 0, stream, (const T*)u, bias, (O*)out, n, total, act)
  if (u_dtype == LLMIE_F32 && out_dtype == LLMIE_F32) { LLMIE_BA(float, float); }
  else if (u_dtype == LLMIE_F32 && out_dtype == LLMIE_BF16) { LLMIE_BA(float, __nv_bfloat16); }
  else if (u_dtype == LLMIE_BF16 && out_dtype == LLMIE_BF16) { LLMIE_BA(__nv_bfloat16, __nv_bfloat16); }
  else if (u_dtype == LLMIE_BF16 && out_dtype == LLMIE_F32) { LLMIE_BA(__nv_bfloat16, float); }
  else return LLMIE_ERR_DTYPE;
#undef LLMIE_BA
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

extern "C" int llmie_cast_rows(const float* x, void* out, int out_dtype, long long total, cudaStream_t stream) {
  if (total < 0) return LLMIE_ERR_BAD_ARG;
  if (total == 0) return LLMIE_OK;
  const dim3 grid(flat_blocks((size_t)total)), block(256);
  if (out_dtype == LLMIE_BF16) launch_k(cast_rows_kernel<__nv_bfloat16>, grid, block, 0, stream, x, (__nv_bfloat16*)out, (size_t)total);
  else if (out_dtype == LLMIE_F32) launch_k(cast_rows_kernel<float>, grid, block, 0, stream, x, (float*)out, (size_t)total);
  else return LLMIE_ERR_DTYPE;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// out[T, n] *= sigmoid(gate[t * ld + j]); both of `dtype`.
// `group` > 1: gate rows hold n / group numbers, each for a run of `group` output columns (one gate per head).
extern "C" int llmie_sigmoid_gate_grouped(void* out, const void* gate, int ld, int n_tokens, int n, int group, int dtype,
                                          cudaStream_t stream) {
  if (n_tokens < 0 || n <= 0 || group <= 0 || n % group || ld < n / group) return LLMIE_ERR_BAD_ARG;
  if (n_tokens == 0) return LLMIE_OK;
  const size_t total = (size_t)n_tokens * n;
  const dim3 grid(flat_blocks(total)), block(256);
  if (dtype == LLMIE_F32) launch_k(sigmoid_gate_kernel<float>, grid, block, 0, stream, (float*)out, (const float*)gate, ld, n, group, total);
  else if (dtype == LLMIE_BF16) launch_k(sigmoid_gate_kernel<__nv_bfloat16>, grid, block, 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate, ld, n, group, total);
  else return LLMIE_ERR_DTYPE;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

extern "C" int llmie_sigmoid_gate(void* out, const void* gate, int ld, int n_tokens, int n, int dtype,
                                  cudaStream_t stream) {
  return llmie_sigmoid_gate_grouped(out, gate, ld, n_tokens, n, 1, dtype, stream);
}

// h float32 [T, d] = norm(alpha * h + s (.) y) * w; y [T, d] of y_dtype; s float32 [d] or null; act of act_dtype or null.
extern "C" int llmie_scaled_sum_norm(float* h, const void* y, int y_dtype, const float* s, float alpha, const float* w,
                                     float eps, void* act, int act_dtype, int n_tokens, int d, cudaStream_t stream) {
  if (n_tokens < 0 || d <= 0 || !w || !y || !h) return LLMIE_ERR_BAD_ARG;
  if (n_tokens == 0) return LLMIE_OK;
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 48 * 1024) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (y_dtype != LLMIE_BF16 && y_dtype != LLMIE_F32) return LLMIE_ERR_DTYPE;
  if (act && act_dtype != LLMIE_BF16 && act_dtype != LLMIE_F32) return LLMIE_ERR_DTYPE;
  const bool vec = d % 8 == 0 && d <= 8 * 1024 && aligned16(h) && aligned16(y) && aligned16(w) &&
                   (!s || aligned16(s)) && (!act || aligned16(act));
  const dim3 grid(n_tokens), block(vec ? ((d / 8 + 31) / 32) * 32 : row_threads(d));
#define LLMIE_SSN(Y, A)                                                                                                \
  if (vec) launch_k(scaled_sum_norm_vec_kernel<Y, A>, grid, block, 0, stream, h, (const Y*)y, s, alpha, w, eps, (A*)act, d); \
  else launch_k(scaled_sum_norm_kernel<Y, A>, grid, block, smem, stream, h, (const Y*)y, s, alpha, w, eps, (A*)act, d)
  const bool y_bf16 = y_dtype == LLMIE_BF16, act_bf16 = act && act_dtype == LLMIE_BF16;
  if (y_bf16 && act_bf16) { LLMIE_SSN(__nv_bfloat16, __nv_bfloat16); }
  else if (y_bf16) { LLMIE_SSN(__nv_bfloat16, float); }
  else if (act_bf16) { LLMIE_SSN(float, __nv_bfloat16); }
  else { LLMIE_SSN(float, float); }
#undef LLMIE_SSN
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// out [T, n] = RMS norm of columns off .. off + n - 1 of src [T, ld], times w float32 [n]; both of `dtype`.
extern "C" int llmie_rmsnorm_cols(const void* src, int ld, int off, const float* w, float eps, void* out, int n_tokens,
                                  int n, int dtype, cudaStream_t stream) {
  if (n_tokens < 0 || n <= 0 || off < 0 || ld < off + n || !w || !src || !out) return LLMIE_ERR_BAD_ARG;
  if (n_tokens == 0) return LLMIE_OK;
  const dim3 grid(n_tokens), block(row_threads(n));
  if (dtype == LLMIE_F32) launch_k(rmsnorm_cols_kernel<float>, grid, block, 0, stream, (const float*)src, ld, off, w, eps, (float*)out, n);
  else if (dtype == LLMIE_BF16) launch_k(rmsnorm_cols_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)src, ld, off, w, eps, (__nv_bfloat16*)out, n);
  else return LLMIE_ERR_DTYPE;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// proj [T, ld]; q_out [T, n_q hd]; k_cache [pages, n_kv, page_size, hd]; v_cache [pages, n_kv, page_size, hdv]; all
// of `dtype`. q_w, k_w float32 or null; lam_ptr float32 scalar on the device (needed with v_first); v_first rows of
// n_kv*hdv elements, v_first_ld apart, or null.
// temp_every > 0: the queries are multiplied by 1 + temp_coef * ln(floor((position + 1) / temp_every) + 1).
extern "C" int llmie_qk_norm_store_temp(const void* proj, int ld, void* q_out, void* k_cache, void* v_cache,
                                        const float* q_w, const float* k_w, float eps, const float* lam_ptr,
                                        const void* v_first, int v_first_ld, const int* tok_pos, const int* tok_seq,
                                        const int* seq_slot, const int* block_table, int max_pages, int page_size,
                                        int n_tokens, int n_q, int n_kv, int hd, int hdv, int write_kv, int dtype,
                                        float temp_coef, int temp_every, cudaStream_t stream) {
  if (n_tokens < 0 || n_q <= 0 || n_kv <= 0 || hd <= 0 || hdv <= 0 || page_size <= 0 || max_pages <= 0)
    return LLMIE_ERR_BAD_ARG;
  if (ld < n_q * hd + n_kv * hd + n_kv * hdv) return LLMIE_ERR_BAD_ARG;
  if (v_first && (!lam_ptr || v_first_ld < n_kv * hdv)) return LLMIE_ERR_BAD_ARG;
  if (write_kv && (!k_cache || !v_cache)) return LLMIE_ERR_BAD_ARG;
  if (n_tokens == 0) return LLMIE_OK;
  const dim3 grid(n_tokens), block(row_threads(n_q * hd));
  // 16-byte accesses: every run of 8 elements (32 bytes of float32, two accesses of 16) starts on 16 bytes
  const bool vec = hd % 8 == 0 && hdv % 8 == 0 && ld % 8 == 0 && (!v_first || v_first_ld % 8 == 0) &&
                   n_q * hd <= 8 * 4 * 1024 && aligned16(proj) &&
                   aligned16(q_out) && aligned16(k_cache) && aligned16(v_cache) && aligned16(v_first) &&
                   aligned16(q_w) && aligned16(k_w);
  if (vec) {
      // runs of 8 query elements a thread: 128 threads where four runs a thread cover the projection, more threads beyond
    const int runs = (n_q * hd + 7) / 8;
    int threads = runs <= 128 ? ((runs + 31) / 32) * 32 : 128;
    if (runs > 4 * threads) threads = (((runs + 3) / 4 + 31) / 32) * 32;
    // few tokens (one-token steps): nothing to keep in flight but the token itself, so one run a thread
    if (n_tokens <= 148 && runs > threads) threads = runs <= 512 ? ((runs + 31) / 32) * 32 : 512;
    const int per_thread = (runs + threads - 1) / threads;
    const dim3 vblock(threads);
#define LLMIE_QKV(T, R)                                                                                              \
  launch_k(qk_norm_store_vec_kernel<T, R>, grid, vblock, 0, stream, (const T*)proj, ld, (T*)q_out, (T*)k_cache,       \
           (T*)v_cache, q_w, k_w, eps, lam_ptr, (const T*)v_first, v_first_ld, tok_pos, tok_seq, seq_slot, block_table, \
           max_pages, page_size, n_q, n_kv, hd, hdv, write_kv, temp_coef, temp_every)
    if (dtype == LLMIE_F32) {
      if (per_thread <= 1) LLMIE_QKV(float, 1); else if (per_thread == 2) LLMIE_QKV(float, 2); else LLMIE_QKV(float, 4);
    } else if (dtype == LLMIE_BF16) {
      if (per_thread <= 1) LLMIE_QKV(__nv_bfloat16, 1);
      else if (per_thread == 2) LLMIE_QKV(__nv_bfloat16, 2);
      else LLMIE_QKV(__nv_bfloat16, 4);
    } else {
      return LLMIE_ERR_DTYPE;
    }
#undef LLMIE_QKV
    LLMIE_LAUNCH_CHECK();
    return LLMIE_OK;
  }
  if (dtype == LLMIE_F32)
    launch_k(qk_norm_store_kernel<float>, grid, block, 0, stream, (const float*)proj, ld, (float*)q_out,
             (float*)k_cache, (float*)v_cache, q_w, k_w, eps, lam_ptr, (const float*)v_first, v_first_ld, tok_pos,
             tok_seq, seq_slot, block_table, max_pages, page_size, n_q, n_kv, hd, hdv, write_kv, temp_coef, temp_every);
  else if (dtype == LLMIE_BF16)
    launch_k(qk_norm_store_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)proj, ld,
             (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, q_w, k_w, eps, lam_ptr,
             (const __nv_bfloat16*)v_first, v_first_ld, tok_pos, tok_seq, seq_slot, block_table, max_pages, page_size,
             n_q, n_kv, hd, hdv, write_kv, temp_coef, temp_every);
  else
    return LLMIE_ERR_DTYPE;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

extern "C" int llmie_qk_norm_store(const void* proj, int ld, void* q_out, void* k_cache, void* v_cache, const float* q_w,
                                   const float* k_w, float eps, const float* lam_ptr, const void* v_first,
                                   int v_first_ld, const int* tok_pos, const int* tok_seq, const int* seq_slot,
                                   const int* block_table, int max_pages, int page_size, int n_tokens, int n_q,
                                   int n_kv, int hd, int hdv, int write_kv, int dtype, cudaStream_t stream) {
  return llmie_qk_norm_store_temp(proj, ld, q_out, k_cache, v_cache, q_w, k_w, eps, lam_ptr, v_first, v_first_ld, tok_pos,
                                  tok_seq, seq_slot, block_table, max_pages, page_size, n_tokens, n_q, n_kv, hd, hdv,
                                  write_kv, dtype, 0.f, 0, stream);
}
