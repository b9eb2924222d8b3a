// The bookkeeping of a routed feed-forward (a mixture of experts); the experts' products themselves are the routed
// form of grouped_gemm.cu.
//
//   route     z = W_r x + b in float32 (a block per token, each lane a fixed share of the columns, so a token's logits do
//             not depend on the batch); the `top` largest logits are chosen (ties: the lower index), their weights are
//             the softmax over the chosen logits alone
//             second rule (`mode` 1): scores = softmax over ALL logits; the `top` largest of score + correction are chosen
//             (the correction steers the choice only); weights = the chosen scores / (their sum + 1e-20) * a constant
//             third rule (`mode` 2): scores = sigmoid(z) one by one; the `top` largest are chosen and the weights are the
//             chosen scores themselves (times a constant), not normalised
//   gather    out[p] = weights[pair at p] * x[token at p] for the sorted positions p: for designs whose weight
//             multiplies what the expert READS (the combine then adds the experts' outputs with weight one)
//   sort      the (token, choice) pairs grouped by expert into tiles of `tile` positions, padded per expert; one block,
//             no host involvement, so the step can be captured: sizes are upper bounds, unused tiles say -1
//   combine   out[t] = sum_k weight[t, k] * y[t * top + k] (+ shared[t]) in float32, in the order of k; a choice whose
//             id is not below the number of real experts stands for an expert that returns its input: weight * x[t]
#include "common.cuh"
#include <math.h>

namespace llmie {

constexpr int kRouteWarps = 8;

template <typename T>
__global__ void __launch_bounds__(kRouteWarps * 32)
moe_route_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                 int* __restrict__ ids, float* __restrict__ weights, int n_tokens, int d, int n_experts, int top,
                 int mode, const float* __restrict__ correction, float out_scale) {
  // A block per token: the token's row is staged once as float32, its warps share out the experts, and a warp's lanes
  // take fixed columns of a dot product (four running sums each, added in a fixed order).
  extern __shared__ __align__(16) float route_smem[];            // [d] the row | [n_experts] the logits | scores
  float* xs = route_smem;
  float* z = route_smem + d;
  float* sc = z + n_experts;                                     // mode 1: the scores the weights are made of
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const T* xr = x + (size_t)t * d;
  const bool vec4 = d % 4 == 0 && (reinterpret_cast<uintptr_t>(w) & 15u) == 0;
  for (int i = threadIdx.x; i < d; i += blockDim.x) xs[i] = to_f32(xr[i]);
  __syncthreads();
  for (int e = warp; e < n_experts; e += kRouteWarps) {
    const float* wr = w + (size_t)e * d;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    int i = lane;
    if (vec4) {
      // 16 bytes a lane and four such loads in flight: a one-token step has nothing else to hide the latency behind
      const float4* w4 = reinterpret_cast<const float4*>(wr);
      const int n4 = d >> 2;
#pragma unroll 4
      for (int j = lane; j < n4; j += 32) {
        const float4 wv = w4[j];
        const float4 xv = reinterpret_cast<const float4*>(xs)[j];
        a0 = fmaf(xv.x, wv.x, a0);
        a1 = fmaf(xv.y, wv.y, a1);
        a2 = fmaf(xv.z, wv.z, a2);
        a3 = fmaf(xv.w, wv.w, a3);
      }
      i = d;
    }
    for (; i + 96 < d; i += 128) {
      a0 = fmaf(xs[i], wr[i], a0);
      a1 = fmaf(xs[i + 32], wr[i + 32], a1);
      a2 = fmaf(xs[i + 64], wr[i + 64], a2);
      a3 = fmaf(xs[i + 96], wr[i + 96], a3);
    }
    for (; i < d; i += 32) a0 = fmaf(xs[i], wr[i], a0);
    const float sum = warp_sum((a0 + a1) + (a2 + a3));
    if (lane == 0) z[e] = sum + (bias ? bias[e] : 0.f);
  }
  __syncthreads();
  if (warp != 0) return;
  __syncwarp();
  if (mode == 1) {
    // scores over all experts; z becomes what the choice is made by
    float mx = -INFINITY;
    for (int e = lane; e < n_experts; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < n_experts; e += 32) { const float p = expf(z[e] - mx); sc[e] = p; sum += p; }
    sum = warp_sum(sum);
    const float inv_sum = 1.f / sum;
    for (int e = lane; e < n_experts; e += 32) {
      const float p = sc[e] * inv_sum;
      sc[e] = p;
      z[e] = p + (correction ? correction[e] : 0.f);
    }
    __syncwarp();
  }
  float first = 0.f, denom = 0.f, mine = 0.f;      // lane k keeps the k-th chosen logit
  int mine_id = 0;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane; e < n_experts; e += 32) {
      const float v = z[e];
      if (v > best || (v == best && e < best_e)) { best = v; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
    }
    if (k == 0) first = best;
    const float p = mode == 1 ? (best_e < n_experts ? sc[best_e] : 0.f)
                    : mode == 2 ? 1.f / (1.f + expf(-best)) : expf(best - first);
    denom += p;
    if ((k & 31) == lane) { mine = p; mine_id = best_e; }
    if (lane == 0 && best_e < n_experts) z[best_e] = -INFINITY;
    __syncwarp();
    if ((k & 31) == 31 || k == top - 1) {
      // flush this run of up to 32 choices; the weights are normalised below, once the sum is complete
      const int base = k & ~31;
      if (base + lane <= k) {
        ids[(size_t)t * top + base + lane] = mine_id < n_experts ? mine_id : 0;
        weights[(size_t)t * top + base + lane] = mine;
      }
    }
  }
  __syncwarp();
  const float inv = mode == 1 ? out_scale / (denom + 1e-20f) : mode == 2 ? out_scale : 1.f / denom;
  for (int k = lane; k < top; k += 32) weights[(size_t)t * top + k] *= inv;
}

__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ ids, int n_pairs, int top, int n_experts, int tile, int max_tiles,
                int* __restrict__ sorted_token, int* __restrict__ sorted_pair, int* __restrict__ tile_group,
                int* __restrict__ group_end, int* __restrict__ pair_pos) {
  extern __shared__ int sm[];                      // counts | offsets | cursor, n_experts each
  int* counts = sm;
  int* offsets = sm + n_experts;
  int* cursor = sm + 2 * n_experts;
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, nt = blockDim.x;
  for (int e = tid; e < n_experts; e += nt) counts[e] = cursor[e] = 0;
  const int cap = max_tiles * tile;
  for (int i = tid; i < cap; i += nt) { sorted_token[i] = -1; sorted_pair[i] = -1; }
  for (int i = tid; i < max_tiles; i += nt) tile_group[i] = -1;
  __syncthreads();
  for (int i = tid; i < n_pairs; i += nt) {
    const int e = ids[i];
    if (e >= 0 && e < n_experts) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int off = 0;
    for (int e = 0; e < n_experts; ++e) {
      offsets[e] = off;
      off += (counts[e] + tile - 1) / tile * tile;
    }
  }
  __syncthreads();
  for (int e = tid; e < n_experts; e += nt) {
    const int t0 = offsets[e] / tile, n = (counts[e] + tile - 1) / tile;
    for (int j = 0; j < n && t0 + j < max_tiles; ++j) tile_group[t0 + j] = e;
    if (group_end) group_end[e] = offsets[e] + n * tile;      // where the expert's positions end, padding included
  }
  for (int i = tid; i < n_pairs; i += nt) {
    const int e = ids[i];
    if (e < 0 || e >= n_experts) continue;
    const int pos = offsets[e] + atomicAdd(&cursor[e], 1);
    if (pos < cap) { sorted_pair[pos] = i; sorted_token[pos] = i / top; }
    if (pair_pos) pair_pos[i] = pos < cap ? pos : 0;
  }
}

// out[p] = x[rows[p]] (zeros where rows[p] < 0): the tokens in the order of their experts, for a library product that
// wants each expert's rows side by side. d % 8 == 0, 16-byte aligned.
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ rows,
                                       __nv_bfloat16* __restrict__ out, int d8, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t pos = i / d8;
    const int c = (int)(i - pos * d8);
    const int r = rows[pos];
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r >= 0) v = reinterpret_cast<const uint4*>(x)[(size_t)r * d8 + c];
    reinterpret_cast<uint4*>(out)[i] = v;
  }
}

// out[p, :] = weights[sorted_pair[p]] * x[sorted_token[p], :] (zeros where sorted_token[p] < 0); the product is formed
// in float32 and rounded once to the output type.
template <typename TI, typename TO>
__global__ void moe_gather_scaled_kernel(const TI* __restrict__ x, const int* __restrict__ sorted_token,
                                         const int* __restrict__ sorted_pair, const float* __restrict__ weights,
                                         TO* __restrict__ out, int d, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t pos = i / d;
    const int c = (int)(i - pos * d);
    const int r = sorted_token[pos];
    float v = 0.f;
    if (r >= 0) v = weights[sorted_pair[pos]] * to_f32(x[(size_t)r * d + c]);
    out[i] = from_f32<TO>(v);
  }
}

// 8 elements a thread (16-byte loads and stores), bfloat16 in and out, d % 8 == 0.
__global__ void moe_gather_scaled_vec_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ sorted_token,
                                             const int* __restrict__ sorted_pair, const float* __restrict__ weights,
                                             __nv_bfloat16* __restrict__ out, int d8, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t pos = i / d8;
    const int c = (int)(i - pos * d8);
    const int r = sorted_token[pos];
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = 0.f;
    if (r >= 0) {
      const float w = weights[sorted_pair[pos]];
      load8(x + ((size_t)r * d8 + c) * 8, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] *= w;
    }
    store8(out + i * 8, v);
  }
}

template <typename TS, typename TY>
__global__ void moe_combine_kernel(const TY* __restrict__ y, const int* __restrict__ pair_pos,
                                   const float* __restrict__ weights, const TS* __restrict__ shared_out,
                                   float* __restrict__ out, int d, int top, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t t = i / d;
    const int c = (int)(i - t * d);
    float s = 0.f;
    for (int k = 0; k < top; ++k) {
      const size_t row = pair_pos ? (size_t)pair_pos[t * top + k] : t * top + k;
      s = fmaf(weights ? weights[t * top + k] : 1.f, to_f32(y[row * d + c]), s);
    }
    if (shared_out) s += to_f32(shared_out[i]);
    out[i] = s;
  }
}

__device__ __forceinline__ float load_any(const void* p, int dtype, size_t i) {
  return dtype == LLMIE_F32 ? reinterpret_cast<const float*>(p)[i] : to_f32(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// The combine with experts that return their input: a choice whose id is n_real or more adds weight * x[t].
__global__ void moe_combine_identity_kernel(const void* __restrict__ y, int y_dtype, const int* __restrict__ pair_pos,
                                            const float* __restrict__ weights, const int* __restrict__ ids, int n_real,
                                            const void* __restrict__ x, int x_dtype, float* __restrict__ out, int d,
                                            int top, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t t = i / d;
    const int c = (int)(i - t * d);
    float s = 0.f;
    for (int k = 0; k < top; ++k) {
      const float w = weights[t * top + k];
      if (ids[t * top + k] >= n_real) {
        s = fmaf(w, load_any(x, x_dtype, i), s);
      } else {
        const size_t row = pair_pos ? (size_t)pair_pos[t * top + k] : t * top + k;
        s = fmaf(w, load_any(y, y_dtype, row * d + c), s);
      }
    }
    out[i] = s;
  }
}

}  // namespace llmie

using namespace llmie;

// x [T, d] of x_dtype; w float32 [E, d]; bias float32 [E] or null; ids int32 [T, top]; weights float32 [T, top].
// mode 0: the rule above (bias added to the logits, softmax over the chosen logits). mode 1: softmax over all logits,
// choice by score + correction (float32 [E] or null), weights = chosen scores / (their sum + 1e-20) * out_scale.
// mode 2: weights = sigmoid of the chosen logits * out_scale, not normalised.
extern "C" int llmie_moe_route_ex(const void* x, int x_dtype, const float* w, const float* bias, int* ids,
                                  float* weights, int n_tokens, int d, int n_experts, int top, int mode,
                                  const float* correction, float out_scale, cudaStream_t stream) {
  if (n_tokens < 0 || d <= 0 || n_experts <= 0 || top <= 0 || top > n_experts) return LLMIE_ERR_BAD_ARG;
  if (mode < 0 || mode > 2) return LLMIE_ERR_BAD_ARG;
  if (x_dtype != LLMIE_F32 && x_dtype != LLMIE_BF16) return LLMIE_ERR_DTYPE;
  const size_t smem = ((size_t)d + 2 * (size_t)n_experts) * sizeof(float);
  if (smem > 48 * 1024) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (n_tokens == 0) return LLMIE_OK;
  const int blocks = n_tokens;
  if (x_dtype == LLMIE_F32)
    launch_k(moe_route_kernel<float>, dim3(blocks), dim3(kRouteWarps * 32), smem, stream, (const float*)x, w, bias, ids, weights, n_tokens, d, n_experts, top, mode, correction, out_scale);
  else
    launch_k(moe_route_kernel<__nv_bfloat16>, dim3(blocks), dim3(kRouteWarps * 32), smem, stream, (const __nv_bfloat16*)x, w, bias, ids, weights, n_tokens, d, n_experts, top, mode, correction, out_scale);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

extern "C" int llmie_moe_route(const void* x, int x_dtype, const float* w, const float* bias, int* ids, float* weights,
                               int n_tokens, int d, int n_experts, int top, cudaStream_t stream) {
  return llmie_moe_route_ex(x, x_dtype, w, bias, ids, weights, n_tokens, d, n_experts, top, 0, nullptr, 1.f, stream);
}

// ids int32 [n_pairs] (pair = token * top + choice); sorted_token, sorted_pair int32 [max_tiles * tile];
// tile_group int32 [max_tiles]. max_tiles must be at least n_pairs / tile + min(n_pairs, n_experts).
extern "C" int llmie_moe_sort(const int* ids, int n_pairs, int top, int n_experts, int tile, int max_tiles,
                              int* sorted_token, int* sorted_pair, int* tile_group, int* group_end, int* pair_pos,
                              cudaStream_t stream) {
  if (n_pairs < 0 || top <= 0 || n_experts <= 0 || tile <= 0 || max_tiles <= 0) return LLMIE_ERR_BAD_ARG;
  const int need = n_pairs / tile + (n_pairs < n_experts ? n_pairs : n_experts);
  if (max_tiles < need) return LLMIE_ERR_BAD_ARG;
  const size_t smem = (size_t)3 * n_experts * sizeof(int);
  if (smem > 48 * 1024) return LLMIE_ERR_UNSUPPORTED_SIZE;
  launch_k(moe_sort_kernel, dim3(1), dim3(1024), smem, stream, ids, n_pairs, top, n_experts, tile, max_tiles, sorted_token, sorted_pair, tile_group, group_end, pair_pos);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// y [rows, d] float32 or bfloat16; row of pair i = pair_pos[i] (int32 [T * top]) or i itself when pair_pos is null;
// weights float32 [T, top]; shared_out [T, d] of shared_dtype or null; out float32 [T, d].
extern "C" int llmie_moe_combine(const void* y, int y_dtype, const int* pair_pos, const float* weights,
                                 const void* shared_out, int shared_dtype, float* out, int n_tokens, int d, int top,
                                 cudaStream_t stream) {
  if (n_tokens < 0 || d <= 0 || top <= 0) return LLMIE_ERR_BAD_ARG;
  if ((shared_out && shared_dtype != LLMIE_F32 && shared_dtype != LLMIE_BF16) || (y_dtype != LLMIE_F32 && y_dtype != LLMIE_BF16))
    return LLMIE_ERR_DTYPE;
  if (n_tokens == 0) return LLMIE_OK;
  const size_t total = (size_t)n_tokens * d;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  const bool sb = shared_out && shared_dtype == LLMIE_BF16;
  const dim3 grid((unsigned)blocks), block(256);
  if (y_dtype == LLMIE_F32) {
    if (sb) launch_k(moe_combine_kernel<__nv_bfloat16, float>, grid, block, 0, stream, (const float*)y, pair_pos, weights, (const __nv_bfloat16*)shared_out, out, d, top, total);
    else launch_k(moe_combine_kernel<float, float>, grid, block, 0, stream, (const float*)y, pair_pos, weights, (const float*)shared_out, out, d, top, total);
  } else {
    if (sb) launch_k(moe_combine_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)y, pair_pos, weights, (const __nv_bfloat16*)shared_out, out, d, top, total);
    else launch_k(moe_combine_kernel<float, __nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)y, pair_pos, weights, (const float*)shared_out, out, d, top, total);
  }
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// The same with experts that return their input: ids int32 [T, top]; a choice with an id of n_real or more adds
// weight * x[t] (x [T, d] of x_dtype) and has no row in y.
extern "C" int llmie_moe_combine_identity(const void* y, int y_dtype, const int* pair_pos, const float* weights,
                                          const int* ids, int n_real, const void* x, int x_dtype, float* out,
                                          int n_tokens, int d, int top, cudaStream_t stream) {
  if (n_tokens < 0 || d <= 0 || top <= 0 || !ids || !x || n_real < 0) return LLMIE_ERR_BAD_ARG;
  if ((y_dtype != LLMIE_F32 && y_dtype != LLMIE_BF16) || (x_dtype != LLMIE_F32 && x_dtype != LLMIE_BF16))
    return LLMIE_ERR_DTYPE;
  if (n_tokens == 0) return LLMIE_OK;
  const size_t total = (size_t)n_tokens * d;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  launch_k(moe_combine_identity_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, y, y_dtype, pair_pos, weights, ids,
           n_real, x, x_dtype, out, d, top, total);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// out [n_positions, d] = x[rows[p]] (zero rows where rows[p] < 0); bfloat16, d % 8 == 0, both 16-byte aligned.
extern "C" int llmie_moe_gather_rows(const void* x, const int* rows, void* out, int n_positions, int d,
                                     cudaStream_t stream) {
  if (n_positions < 0 || d <= 0 || d % 8) return LLMIE_ERR_BAD_ARG;
  if (!aligned16(x) || !aligned16(out)) return LLMIE_ERR_ALIGNMENT;
  if (n_positions == 0) return LLMIE_OK;
  const size_t total = (size_t)n_positions * (d / 8);
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  launch_k(moe_gather_rows_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, (const __nv_bfloat16*)x, rows, (__nv_bfloat16*)out, d / 8, total);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// out [n_positions, d] of out_dtype = weights[sorted_pair[p]] * x[sorted_token[p]] (zero rows where sorted_token[p] < 0);
// x [T, d] of x_dtype; weights float32 [T * top] by pair.
extern "C" int llmie_moe_gather_scaled(const void* x, int x_dtype, const int* sorted_token, const int* sorted_pair,
                                       const float* weights, void* out, int out_dtype, int n_positions, int d,
                                       cudaStream_t stream) {
  if (n_positions < 0 || d <= 0 || !x || !sorted_token || !sorted_pair || !weights || !out) return LLMIE_ERR_BAD_ARG;
  if ((x_dtype != LLMIE_F32 && x_dtype != LLMIE_BF16) || (out_dtype != LLMIE_F32 && out_dtype != LLMIE_BF16))
    return LLMIE_ERR_DTYPE;
  if (n_positions == 0) return LLMIE_OK;
  if (x_dtype == LLMIE_BF16 && out_dtype == LLMIE_BF16 && d % 8 == 0 && aligned16(x) && aligned16(out)) {
    const size_t total = (size_t)n_positions * (d / 8);
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    launch_k(moe_gather_scaled_vec_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, (const __nv_bfloat16*)x,
             sorted_token, sorted_pair, weights, (__nv_bfloat16*)out, d / 8, total);
    LLMIE_LAUNCH_CHECK();
    return LLMIE_OK;
  }
  const size_t total = (size_t)n_positions * d;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  const dim3 grid((unsigned)blocks), block(256);
  const bool xb = x_dtype == LLMIE_BF16, ob = out_dtype == LLMIE_BF16;
  if (xb && ob) launch_k(moe_gather_scaled_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)x, sorted_token, sorted_pair, weights, (__nv_bfloat16*)out, d, total);
  else if (xb) launch_k(moe_gather_scaled_kernel<__nv_bfloat16, float>, grid, block, 0, stream, (const __nv_bfloat16*)x, sorted_token, sorted_pair, weights, (float*)out, d, total);
  else if (ob) launch_k(moe_gather_scaled_kernel<float, __nv_bfloat16>, grid, block, 0, stream, (const float*)x, sorted_token, sorted_pair, weights, (__nv_bfloat16*)out, d, total);
  else launch_k(moe_gather_scaled_kernel<float, float>, grid, block, 0, stream, (const float*)x, sorted_token, sorted_pair, weights, (float*)out, d, total);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}
