// Plain attention over the paged KV cache, for any number of new tokens per sequence.
//
// One warp per (token, query head). It is the float32 path's attention for prefill and
// decode alike, and the plain twin that the tensor-core and split-KV kernels are checked
// against. The math is that of the reference's prefill and decode kernels
// (src/flash_attn.py:42-82, src/flash_decode.py:73-113): scores q.k / sqrt(hd) over the keys
// a token may see, online softmax with float32 running max / sum / accumulator, query head
// h reading key/value head h / (Hq / Hkv).
//
// A token at absolute position p of its sequence sees keys lo..p of that sequence's slot,
// lo = max(0, p - window + 1) when window > 0, else 0, and besides them the first `keep_first` keys of the
// sequence (keys 0..keep_first-1 stay visible when the window has moved past them). Keys of this very step were
// written to the cache before this kernel runs, so prefill at any start position, decode, and mixtures need
// no separate code.
//
// Options beyond the reference's math, each off by default: a value head size `hdv` that differs from the
// query/key head size; `sink`: the softmax denominator gets one more term exp(0), a key whose score is 0 and
// whose value is nothing (p_j = exp(s_j) / (1 + sum exp(s_j))); `gate`: the output row is multiplied element
// by element with sigmoid(gate[t * gate_ld + ...]). `sink_vals`: the score of the sink is a number per query head instead
// of 0. `softcap` c > 0: a score s becomes c * tanh(s / c) (after the scale). `dist_bias` [n_q, bias_len]: a number per
// query head and distance (query position minus key position, distances of bias_len - 1 and more share the last entry) is
// added to the score after the cap, unscaled. `v_ld`: elements between the starts of two value rows of a page, for values
// that are a column range of wider rows (a latent that serves as key and value at once: v_cache then points into k_cache).
// `sig_bias` [n_q]: no softmax at all; a visible key's weight is sigmoid(score + sig_bias[head]) and the weights are not
// normalised over the keys (out_i = sum_j sigmoid(s_ij + b) v_j); excludes the sink.
#include "common.cuh"
#include <math.h>

namespace llmie {

constexpr int kAttnWarps = 4;
constexpr int kMaxHeadDim = 256;       // the common instantiation; kWideHeadDim serves single-head latents
constexpr int kWideHeadDim = 1024;

template <typename T, bool VEC, int MAXHD>
__global__ void __launch_bounds__(kAttnWarps * 32)
attention_paged_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                       T* __restrict__ out, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                       const int* __restrict__ seq_slot, const int* __restrict__ block_table, int max_pages,
                       int page_size, int n_items, int n_q, int n_kv, int hd, int hdv, float scale, int window,
                       int keep_first, int sink, const T* __restrict__ gate, int gate_ld, int v_ld, float softcap,
                       const float* __restrict__ dist_bias, int bias_len, const float* __restrict__ sink_vals,
                       const float* __restrict__ sig_bias) {
  extern __shared__ float q_smem[];  // [kAttnWarps][hd]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x * kAttnWarps + warp;
  if (item >= n_items) return;  // whole warp leaves together; no block-wide barrier below
  const int t = item / n_q, h = item - t * n_q;
  const int hk = h / (n_q / n_kv);
  const int pos = tok_pos[t];
  const int slot = seq_slot[tok_seq[t]];
  const int* pages = block_table + (size_t)slot * max_pages;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int kept = keep_first < lo ? keep_first : lo;     // keys [0, kept) are seen besides [lo, pos]

  float* qs = q_smem + warp * hd;
  const T* qrow = q + ((size_t)t * n_q + h) * hd;
  for (int i = lane; i < hd; i += 32) qs[i] = to_f32(qrow[i]) * scale;
  __syncwarp();

  constexpr int kAcc = MAXHD / 32;
  float acc[kAcc];
#pragma unroll
  for (int i = 0; i < kAcc; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  const float* bias_row = dist_bias ? dist_bias + (size_t)h * bias_len : nullptr;
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;
  const float sig_b = sig_bias ? sig_bias[h] : 0.f;

  for (int seg = 0; seg < 2; ++seg) {
    const int first = seg == 0 ? 0 : lo;
    const int last = seg == 0 ? kept - 1 : pos;          // inclusive
    for (int base = first; base <= last; base += 32) {
      const int j = base + lane;
      const bool valid = j <= last;
      int page_row = 0;                                   // (page * n_kv + hk) * page_size + offset in the page
      float s = -INFINITY;
      if (valid) {
        const int page = pages[j / page_size];
        page_row = (page * n_kv + hk) * page_size + (j % page_size);
        const T* kr = k_cache + (size_t)page_row * hd;
        float dot = 0.f;
        if (VEC) {
          for (int d0 = 0; d0 < hd; d0 += 8) {
            float kv[8];
            load8(kr + d0, kv);
#pragma unroll
            for (int e = 0; e < 8; ++e) dot = fmaf(qs[d0 + e], kv[e], dot);
          }
        } else {
          for (int d0 = 0; d0 < hd; ++d0) dot = fmaf(qs[d0], to_f32(kr[d0]), dot);
        }
        s = dot;
        if (softcap > 0.f) s = softcap * tanhf(s * inv_cap);
        if (bias_row) s += bias_row[min(pos - j, bias_len - 1)];
      }
      float p;
      if (sig_bias) {
        p = valid ? 1.f / (1.f + expf(-(s + sig_b))) : 0.f;
      } else {
        const float m_new = fmaxf(m, warp_max(s));
        p = valid ? expf(s - m_new) : 0.f;
        const float alpha = expf(m - m_new);  // m == -inf on the first chunk gives 0
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < kAcc; ++i) acc[i] *= alpha;
        m = m_new;
      }
      const int n_here = min(32, last - base + 1);
      for (int jj = 0; jj < n_here; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, p, jj);
        const int rj = __shfl_sync(0xffffffffu, page_row, jj);
        const T* vr = v_cache + (size_t)rj * v_ld;
#pragma unroll
        for (int i = 0; i < kAcc; ++i) {
          const int d = lane + 32 * i;
          if (d < hdv) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
        }
      }
    }
  }
  if (sink) {
    // one more term of score s0 (0 unless given per head): the running maximum becomes max(m, s0) and the
    // denominator gains exp(s0 - m')
    const float s0 = sink_vals ? sink_vals[h] : 0.f;
    const float m_new = fmaxf(m, s0);
    const float alpha = expf(m - m_new);
    l = l * alpha + expf(s0 - m_new);
#pragma unroll
    for (int i = 0; i < kAcc; ++i) acc[i] *= alpha;
  }
  const float inv_l = sig_bias ? 1.f : 1.f / l;
  T* orow = out + ((size_t)t * n_q + h) * hdv;
  const T* grow = gate ? gate + (size_t)t * gate_ld + (size_t)h * hdv : nullptr;
#pragma unroll
  for (int i = 0; i < kAcc; ++i) {
    const int d = lane + 32 * i;
    if (d < hdv) {
      float o = acc[i] * inv_l;
      if (grow) o = o / (1.f + expf(-to_f32(grow[d])));
      orow[d] = from_f32<T>(o);
    }
  }
}

}  // namespace llmie

using namespace llmie;

template <typename T, int MAXHD>
static void attention_paged_launch(bool vec, int blocks, size_t smem, cudaStream_t stream, const void* q,
                                   const void* k_cache, const void* v_cache, void* out, const int* tok_pos,
                                   const int* tok_seq, const int* seq_slot, const int* block_table, int max_pages,
                                   int page_size, int n_items, int n_q, int n_kv, int hd, int hdv, float scale,
                                   int window, int keep_first, int sink, const void* gate, int gate_ld, int v_ld,
                                   float softcap, const float* dist_bias, int bias_len, const float* sink_vals,
                                   const float* sig_bias) {
  if (vec)
    attention_paged_kernel<T, true, MAXHD><<<blocks, kAttnWarps * 32, smem, stream>>>(
        (const T*)q, (const T*)k_cache, (const T*)v_cache, (T*)out, tok_pos, tok_seq, seq_slot, block_table, max_pages,
        page_size, n_items, n_q, n_kv, hd, hdv, scale, window, keep_first, sink, (const T*)gate, gate_ld, v_ld, softcap,
        dist_bias, bias_len, sink_vals, sig_bias);
  else
    attention_paged_kernel<T, false, MAXHD><<<blocks, kAttnWarps * 32, smem, stream>>>(
        (const T*)q, (const T*)k_cache, (const T*)v_cache, (T*)out, tok_pos, tok_seq, seq_slot, block_table, max_pages,
        page_size, n_items, n_q, n_kv, hd, hdv, scale, window, keep_first, sink, (const T*)gate, gate_ld, v_ld, softcap,
        dist_bias, bias_len, sink_vals, sig_bias);
}

// q [n_tokens, n_q * hd]; out [n_tokens, n_q * hdv]; k_cache [n_pages, n_kv, page_size, hd]; v_cache rows of hdv
// elements, v_ld apart (v_ld == hdv: a tensor [n_pages, n_kv, page_size, hdv] of its own); gate (or null) rows of
// n_q * hdv elements, gate_ld apart; all of `dtype`. dist_bias float32 [n_q, bias_len] or null; sink_vals float32 [n_q]
// or null (with sink != 0: the sink's score is 0); sig_bias float32 [n_q] or null. Any hd, hdv up to 1024.
extern "C" int llmie_attention_paged_sig(const void* q, const void* k_cache, const void* v_cache, void* out,
                                        const int* tok_pos, const int* tok_seq, const int* seq_slot,
                                        const int* block_table, int max_pages, int page_size, int n_tokens, int n_q,
                                        int n_kv, int hd, int hdv, float scale, int window, int keep_first, int sink,
                                        const void* gate, int gate_ld, int v_ld, float softcap, const float* dist_bias,
                                        int bias_len, const float* sink_vals, const float* sig_bias, int dtype,
                                        cudaStream_t stream) {
  if (sig_bias && sink) return LLMIE_ERR_BAD_ARG;
  if (n_tokens < 0 || n_q <= 0 || n_kv <= 0 || hd <= 0 || hdv <= 0 || page_size <= 0 || max_pages <= 0)
    return LLMIE_ERR_BAD_ARG;
  if (n_q % n_kv || keep_first < 0 || window < 0 || (gate && gate_ld < n_q * hdv)) return LLMIE_ERR_BAD_ARG;
  if (v_ld < hdv || softcap < 0.f || (dist_bias && bias_len <= 0) || (sink_vals && !sink)) return LLMIE_ERR_BAD_ARG;
  if (hd > kWideHeadDim || hdv > kWideHeadDim) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (dtype != LLMIE_F32 && dtype != LLMIE_BF16) return LLMIE_ERR_DTYPE;
  if (n_tokens == 0) return LLMIE_OK;
  const long long n_items = (long long)n_tokens * n_q;
  if (n_items > 0x7fffffffLL) return LLMIE_ERR_UNSUPPORTED_SIZE;
  const int blocks = (int)((n_items + kAttnWarps - 1) / kAttnWarps);
  const size_t smem = (size_t)kAttnWarps * hd * sizeof(float);
  // 16-byte loads of the keys need rows that start on 16 bytes (32 for float32, two loads of 16)
  const bool vec = hd % 8 == 0 && aligned16(k_cache);
  const bool wide = hd > kMaxHeadDim || hdv > kMaxHeadDim;
#define LLMIE_ATTN_ARGS                                                                                              \
  vec, blocks, smem, stream, q, k_cache, v_cache, out, tok_pos, tok_seq, seq_slot, block_table, max_pages, page_size, \
      (int)n_items, n_q, n_kv, hd, hdv, scale, window, keep_first, sink, gate, gate_ld, v_ld, softcap, dist_bias,    \
      bias_len, sink_vals, sig_bias
  if (dtype == LLMIE_F32) {
    if (wide) attention_paged_launch<float, kWideHeadDim>(LLMIE_ATTN_ARGS);
    else attention_paged_launch<float, kMaxHeadDim>(LLMIE_ATTN_ARGS);
  } else {
    if (wide) attention_paged_launch<__nv_bfloat16, kWideHeadDim>(LLMIE_ATTN_ARGS);
    else attention_paged_launch<__nv_bfloat16, kMaxHeadDim>(LLMIE_ATTN_ARGS);
  }
#undef LLMIE_ATTN_ARGS
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

extern "C" int llmie_attention_paged_ex(const void* q, const void* k_cache, const void* v_cache, void* out,
                                        const int* tok_pos, const int* tok_seq, const int* seq_slot,
                                        const int* block_table, int max_pages, int page_size, int n_tokens, int n_q,
                                        int n_kv, int hd, int hdv, float scale, int window, int keep_first, int sink,
                                        const void* gate, int gate_ld, int v_ld, float softcap, const float* dist_bias,
                                        int bias_len, const float* sink_vals, int dtype, cudaStream_t stream) {
  return llmie_attention_paged_sig(q, k_cache, v_cache, out, tok_pos, tok_seq, seq_slot, block_table, max_pages,
                                   page_size, n_tokens, n_q, n_kv, hd, hdv, scale, window, keep_first, sink, gate,
                                   gate_ld, v_ld, softcap, dist_bias, bias_len, sink_vals, nullptr, dtype, stream);
}
