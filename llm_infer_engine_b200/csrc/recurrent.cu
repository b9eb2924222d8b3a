// Mixers that carry a fixed-size state from token to token instead of reading a cache of keys: a gated linear
// recurrence over a matrix state per head, and a gated linear recurrent unit over a vector state behind a short causal
// convolution. Everything that enters a recurrence (gates, decays, the state, the norms of what is read) is float32 in
// both precisions; the projections that feed the kernels have the activation type.
//
// Packed tokens: sequence s of the step owns rows cu_q[s] .. cu_q[s+1]-1, its state lives in row seq_slot[s] of a
// [slots, ...] float32 tensor and is read at the start and written at the end, so a sequence fed in pieces, or token
// by token, goes through exactly the same arithmetic as one fed whole.
//
//   matrix_gates       q = silu(q_raw), f = l + (1 - l) sigmoid(f_raw + b)           element-wise, float32 out
//   matrix_scan        S <- diag(f_t) S + (1 - f_t) v_t^T ; o_t = S^T q_t            S [dim, vdim] per head
//                      keyed form (a decay per head given): S <- a_h S + k_t v_t^T   linear attention with a constant decay
//   act_columns        float32 copies of up to three runs of columns of the projections, through an activation
//   matrix_scan_chunked  the same for long pieces, cut into chunks that run side by side (below)
//   head_rmsnorm       o / sqrt(mean(o^2) + eps) * w over each head's vdim (or over the whole row, with a weight per
//                      column), optionally times sigmoid(gate)
//   causal_conv        u_t = b + sum_j taps[:, K-1-j] x_(t-j), x before the step from the state's last K-1 inputs
//   unit_gate_values   a = exp(-c r softplus(lam)), drive = sqrt(1 - a^2) i u, r and i sigmoids of given pre-activations
//   unit_scan          S <- a_t S + drive_t ; out_t = S act(y_raw + b) ; the new conv state
//   unit_scan_chunked  the same for long pieces, 32 chunks of a sequence side by side in one block
//
// Long pieces. Both recurrences are linear in the state, S_end = A S_start + B with A the product of the chunk's gates
// and B what the chunk makes from a zero state. So a piece is cut into chunks; every chunk is run from zero (A and B),
// the chunks' true starting states follow from a short chain over the chunks, and every chunk is run again from its
// start, now with outputs. Twice the arithmetic, all of it float32 and in token order within a chunk; what differs
// from the token-by-token order is the rounding of the chain's steps only.
#include "common.cuh"
#include <math.h>

namespace llmie {

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// ------------------------------------------------------------------------------------------ matrix state
template <typename T>
__global__ void matrix_gates_kernel(const T* __restrict__ proj, int ld, int q_off, int f_off,
                                    const float* __restrict__ f_bias, const float* __restrict__ lower,
                                    float* __restrict__ q_out, float* __restrict__ f_out, int n, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t t = i / n;
    const int c = (int)(i - t * n);
    const T* row = proj + t * ld;
    const float q = to_f32(row[q_off + c]);
    const float z = to_f32(row[f_off + c]) + f_bias[c];
    const float l = lower[c];
    q_out[i] = q * sigmoidf_(q);
    f_out[i] = l + (1.f - l) * sigmoidf_(z);
  }
}

constexpr int kScanThreads = 128;
constexpr int kScanR = 16;          // state rows a thread keeps at most (one column a thread)
constexpr int kScanRWide = 8;       // ... when it owns four columns

// grid (column tiles, heads, sequences). A thread owns C adjacent columns (C = 1, or 4 when the value size allows) of its
// head's state and the rows [s R, (s+1) R) of them, S = slices (a power of two up to 32, lanes that differ in their low
// bits), R = ceil(dim / S) <= RMAX. With four columns a thread every gate, key and query entry that is loaded serves
// four state entries: the kernel is bound by what the first-level cache delivers otherwise. The next token's gate, query
// and values are requested before the current token's products.
// With `head_decay` (float32 [H]) the update is S <- head_decay[h] S + k_t v_t^T with the keys k_t in the place of fg.
// MODE 0: a sequence's whole piece, from the slot's state to the slot's state. MODE 1 and 2 work on chunk c =
// blockIdx.z % NC of sequence blockIdx.z / NC, L tokens each, with ws float32 [n_seqs, NC, H, D, Dv] and decay float32
// [n_seqs, NC, H, D]: MODE 1 runs a chunk that is not the sequence's last from a zero state, without outputs, and leaves
// its end state in ws[c + 1] and the product of its gates in decay[c + 1]; MODE 2 runs a chunk from ws[c] with outputs,
// and the last one writes the slot's state.
template <typename T, int MODE, int C, int RMAX, bool KEYED>
__global__ void __launch_bounds__(kScanThreads)
matrix_scan_kernel(const float* __restrict__ qa, const float* __restrict__ fg, const T* __restrict__ v, int v_ld,
                   float* __restrict__ state, const int* __restrict__ cu_q, const int* __restrict__ seq_slot,
                   float* __restrict__ o, int H, int D, int Dv, int S, int R, int write_state,
                   float* __restrict__ ws, float* __restrict__ decay, int L, int NC,
                   const float* __restrict__ head_decay) {
  pdl_launch_dependents();
  // keyed form: fg holds keys k_t instead of gates, and the gate of every row of head h is the constant head_decay[h]
  constexpr bool keyed = KEYED;
  const float dh = keyed ? head_decay[blockIdx.y] : 0.f;       // a constant of the model: no kernel writes it
  pdl_wait();
  const int s = threadIdx.x & (S - 1);
  const int col = threadIdx.x / S;
  const int j = (blockIdx.x * (kScanThreads / S) + col) * C;   // Dv is a multiple of C
  const int h = blockIdx.y;
  const int seq = MODE == 0 ? blockIdx.z : blockIdx.z / NC;
  const int chunk = MODE == 0 ? 0 : blockIdx.z - seq * NC;
  const bool live = j < Dv;
  const int jj = live ? j : Dv - C;
  const int i0 = s * R;
  const int seq_end = cu_q[seq + 1];
  const int t0 = MODE == 0 ? cu_q[seq] : cu_q[seq] + chunk * L;
  const int t1 = MODE == 0 ? seq_end : min(t0 + L, seq_end);
  if (MODE == 1 && t1 >= seq_end) return;          // the last chunk (or none at all): nobody needs its end state
  if (MODE == 2 && t0 >= seq_end) return;
  const int slot = seq_slot[seq];
  float* st = state + (((size_t)slot * H + h) * D) * Dv + jj;
  const size_t HDDv = (size_t)H * D * Dv;
  const float* start = MODE == 2 ? ws + ((size_t)seq * NC + chunk) * HDDv + ((size_t)h * D) * Dv + jj : st;
  float St[RMAX][C];
#pragma unroll
  for (int r = 0; r < RMAX; ++r)
#pragma unroll
    for (int c = 0; c < C; ++c)
      St[r][c] = (MODE != 1 && r < R && i0 + r < D) ? start[(size_t)(i0 + r) * Dv + c] : 0.f;
  float f[RMAX], q[RMAX], vj[C];
  const size_t HD = (size_t)H * D;
  auto fetch = [&](int t) {
    const float* fr = fg + (size_t)t * HD + (size_t)h * D + i0;
    const float* qr = qa + (size_t)t * HD + (size_t)h * D + i0;
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      const bool ok = r < R && i0 + r < D;
      f[r] = ok ? fr[r] : 0.f;
      if (MODE != 1) q[r] = ok ? qr[r] : 0.f;
    }
#pragma unroll
    for (int c = 0; c < C; ++c) vj[c] = to_f32(v[(size_t)t * v_ld + (size_t)h * Dv + jj + c]);
  };
  float prod[RMAX];                                 // MODE 1: the product of the chunk's gates
#pragma unroll
  for (int r = 0; r < RMAX; ++r) prod[r] = 1.f;
  if (t0 < t1) fetch(t0);
  for (int t = t0; t < t1; ++t) {
    float cf[RMAX], cq[RMAX], cv[C], acc[C];
#pragma unroll
    for (int c = 0; c < C; ++c) { cv[c] = vj[c]; acc[c] = 0.f; }
#pragma unroll
    for (int r = 0; r < RMAX; ++r) { cf[r] = f[r]; cq[r] = MODE != 1 ? q[r] : 0.f; }
    if (t + 1 < t1) fetch(t + 1);
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      const float gate = keyed ? dh : cf[r];
      const float write = keyed ? cf[r] : 1.f - cf[r];
#pragma unroll
      for (int c = 0; c < C; ++c) {
        St[r][c] = fmaf(gate, St[r][c], write * cv[c]);
        if (MODE != 1) acc[c] = fmaf(St[r][c], cq[r], acc[c]);
      }
      if (MODE == 1) prod[r] *= gate;
    }
    if (MODE != 1) {
#pragma unroll
      for (int c = 0; c < C; ++c) {
        for (int off = 1; off < S; off <<= 1) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], off);
        if (s == 0 && live) o[(size_t)t * H * Dv + (size_t)h * Dv + j + c] = acc[c];
      }
    }
  }
  if (MODE == 1) {
    float* end = ws + ((size_t)seq * NC + chunk + 1) * HDDv + ((size_t)h * D) * Dv + jj;
    float* dec = decay + (((size_t)seq * NC + chunk + 1) * H + h) * D;
#pragma unroll
    for (int r = 0; r < RMAX; ++r)
      if (r < R && i0 + r < D) {
        if (live) {
#pragma unroll
          for (int c = 0; c < C; ++c) end[(size_t)(i0 + r) * Dv + c] = St[r][c];
        }
        if (blockIdx.x == 0 && col == 0) dec[i0 + r] = prod[r];
      }
    return;
  }
  if (write_state && live && t1 >= seq_end) {
#pragma unroll
    for (int r = 0; r < RMAX; ++r)
      if (r < R && i0 + r < D) {
#pragma unroll
        for (int c = 0; c < C; ++c) st[(size_t)(i0 + r) * Dv + c] = St[r][c];
      }
  }
}

// How a head's state is cut among threads: C columns a thread, S slices of R rows.
struct ScanShape { int C, S, R; };
static inline ScanShape scan_shape(int D, int Dv) {
  ScanShape g;
  // four columns a thread where the value size is a multiple of four and fills a block's threads that way (a narrow
  // state would leave threads without columns); one column a thread otherwise
  int s4 = 1;
  while (s4 * kScanRWide < D) s4 <<= 1;
  g.C = (Dv % 4 == 0 && s4 <= 32 && (kScanThreads / s4) * 4 <= Dv) ? 4 : 1;
  const int rmax = g.C == 4 ? kScanRWide : kScanR;
  g.S = 1;
  while (g.S * rmax < D) g.S <<= 1;
  g.R = (D + g.S - 1) / g.S;
  return g;
}

// The chain over a sequence's chunks, a thread per element of the state: ws[0] = the slot's state and
// ws[c] = decay[c] (.) ws[c - 1] + ws[c] for the chunks the sequence has, so that ws[c] is where chunk c starts.
__global__ void matrix_scan_chain_kernel(const float* __restrict__ state, const int* __restrict__ cu_q,
                                         const int* __restrict__ seq_slot, float* __restrict__ ws,
                                         const float* __restrict__ decay, int H, int D, int Dv, int L, int NC) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.y;
  const size_t HDDv = (size_t)H * D * Dv;
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= HDDv) return;
  const int n = cu_q[seq + 1] - cu_q[seq];
  const int nc = (n + L - 1) / L;
  if (nc <= 0) return;
  const size_t hi = e / Dv;                         // (head, row) of the element
  float S = state[(size_t)seq_slot[seq] * HDDv + e];
  float* w = ws + (size_t)seq * NC * HDDv + e;
  const float* d = decay + (size_t)seq * NC * H * D + hi;
  w[0] = S;
  for (int c = 1; c < nc; ++c) {
    S = fmaf(d[(size_t)c * H * D], S, w[(size_t)c * HDDv]);
    w[(size_t)c * HDDv] = S;
  }
}

// a warp per (token, head): o float32 [T, H * Dv] -> y of the activation type. `gate` (rows gate_ld apart, null = none):
// the result is multiplied by sigmoid(gate) of the same place. An item may also be a token's whole row (Dv = the row).
template <typename T>
__global__ void head_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps,
                                    T* __restrict__ y, int Dv, size_t n_items, const T* __restrict__ gate, int gate_ld,
                                    int items_per_row) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t item = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= n_items) return;
  const float* row = o + item * Dv;
  float ss = 0.f;
  for (int i = lane; i < Dv; i += 32) { const float x = row[i]; ss = fmaf(x, x, ss); }
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)Dv + eps);
  if (!gate) {
    for (int i = lane; i < Dv; i += 32) y[item * Dv + i] = from_f32<T>(row[i] * r * w[i]);
    return;
  }
  const size_t t = item / items_per_row;
  const T* gr = gate + t * gate_ld + (item - t * items_per_row) * Dv;
  for (int i = lane; i < Dv; i += 32)
    y[item * Dv + i] = from_f32<T>(row[i] * r * w[i] / (1.f + expf(-to_f32(gr[i]))));
}

// The same for wide items (a token's whole row of concatenated heads): a block per item, so that a one-token step's few
// rows are not each one warp's work. Dv % 4 == 0 and 16-byte aligned rows: four elements a thread and access.
template <typename T>
__global__ void __launch_bounds__(256)
row_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps, T* __restrict__ y, int Dv,
                   const T* __restrict__ gate, int gate_ld, int items_per_row) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const size_t item = blockIdx.x;
  const float4* row = reinterpret_cast<const float4*>(o + item * Dv);
  const int n4 = Dv >> 2;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {
    const float4 x = row[i];
    ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / (float)Dv + eps);
  const size_t t = item / items_per_row;
  const T* gr = gate ? gate + t * gate_ld + (item - t * items_per_row) * Dv : nullptr;
  T* yr = y + item * Dv;
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {
    const float4 x = row[i];
    const float4 wv = reinterpret_cast<const float4*>(w)[i];
    float v[4] = {x.x * r * wv.x, x.y * r * wv.y, x.z * r * wv.z, x.w * r * wv.w};
    if (gr) {
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = v[e] / (1.f + expf(-to_f32(gr[4 * i + e])));
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) yr[4 * i + e] = from_f32<T>(v[e]);
  }
}

// Float32 copies of up to three runs of columns of proj [T, ld], each through the activation `act`:
// out_k[t, c] = act(proj[t, off_k + c]), c < n_k. (What a linear-attention layer reads of its projections.)
template <typename T>
__global__ void act_columns_kernel(const T* __restrict__ proj, int ld, int off0, int n0, float* __restrict__ out0,
                                   int off1, int n1, float* __restrict__ out1, int off2, int n2,
                                   float* __restrict__ out2, int act, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const int n = n0 + n1 + n2;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t t = i / n;
    int c = (int)(i - t * n);
    const T* row = proj + t * ld;
    if (c < n0) { out0[t * n0 + c] = apply_act(to_f32(row[off0 + c]), act); continue; }
    c -= n0;
    if (c < n1) { out1[t * n1 + c] = apply_act(to_f32(row[off1 + c]), act); continue; }
    c -= n1;
    out2[t * n2 + c] = apply_act(to_f32(row[off2 + c]), act);
  }
}

// ------------------------------------------------------------------------------------------ vector state
constexpr int kMaxTaps = 16;

// A thread is a channel over a run of `tile` consecutive packed tokens. x = proj[:, x_off + c] + x_bias; inputs before
// the step come from conv_state [slots, K-1, C] (the last K-1 inputs of the sequence so far, zeros at its start). The
// thread keeps the last K inputs in registers: a token that follows its predecessor in the same sequence loads ONE new
// input, the first token of a run or of a sequence's piece loads all K. Oldest input first: a fixed order of summation.
template <typename T>
__global__ void causal_conv_kernel(const T* __restrict__ proj, int ld, int x_off, const float* __restrict__ x_bias,
                                   const float* __restrict__ taps, const float* __restrict__ conv_bias,
                                   const float* __restrict__ conv_state, const int* __restrict__ cu_q,
                                   const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                                   float* __restrict__ u, int C, int K, int n_tokens, int tile) {
  pdl_launch_dependents();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float tp[kMaxTaps], w[kMaxTaps];
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k) tp[k] = k < K ? taps[(size_t)c * K + k] : 0.f;       // weights: no kernel writes them
  const float xb = x_bias ? x_bias[c] : 0.f;
  const float cb = conv_bias ? conv_bias[c] : 0.f;
  pdl_wait();
  const int ta = blockIdx.y * tile, tb = min(ta + tile, n_tokens);
  int prev_seq = -1;
  for (int t = ta; t < tb; ++t) {
    const int seq = tok_seq[t];
    const int p = t - cu_q[seq];                      // place within this step's piece of the sequence
    if (seq != prev_seq || p == 0) {
      const float* old = conv_state + (size_t)seq_slot[seq] * (K - 1) * C + c;
#pragma unroll
      for (int k = 0; k < kMaxTaps; ++k) {
        if (k < K) {
          const int m = p - (K - 1 - k);              // w[k] is the input K-1-k tokens back
          w[k] = m >= 0 ? to_f32(proj[(size_t)(t - (K - 1 - k)) * ld + x_off + c]) + xb
                        : old[(size_t)(K - 1 + m) * C];
        }
      }
      prev_seq = seq;
    } else {
#pragma unroll
      for (int k = 0; k + 1 < kMaxTaps; ++k)
        if (k + 1 < K) w[k] = w[k + 1];
      const float x = to_f32(proj[(size_t)t * ld + x_off + c]) + xb;
#pragma unroll
      for (int k = 0; k < kMaxTaps; ++k)
        if (k == K - 1) w[k] = x;
    }
    float acc = cb;
#pragma unroll
    for (int k = 0; k < kMaxTaps; ++k)
      if (k < K) acc = fmaf(tp[k], w[k], acc);
    u[(size_t)t * C + c] = acc;
  }
}

// gates [T, groups * 2 * bw]: per group the pre-activations of r (bw) and then of i (bw). In place: r's place receives
// a = exp(-c r softplus(lam)), i's place the drive sqrt(1 - a^2) * i * u.
__global__ void unit_gate_values_kernel(float* __restrict__ gates, const float* __restrict__ u,
                                        const float* __restrict__ r_bias, const float* __restrict__ i_bias,
                                        const float* __restrict__ lam, float c_decay, int C, int bw, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t t = i / C;
    const int c = (int)(i - t * C);
    const int g = c / bw, e = c - g * bw;
    float* gr = gates + t * 2 * C + (size_t)g * 2 * bw + e;
    const float r = sigmoidf_(gr[0] + r_bias[c]);
    const float in = sigmoidf_(gr[bw] + i_bias[c]);
    const float log_a = -c_decay * r * softplusf_(lam[c]);
    const float a = expf(log_a);
    gr[0] = a;
    gr[bw] = sqrtf(-expm1f(2.f * log_a)) * (in * u[i]);     // 1 - a^2 without cancellation near a = 1
  }
}

// a thread per (sequence, channel): the recurrence over the step's tokens, the output gate act(y_raw + y_bias), and
// the new state of the recurrence and of the convolution.
template <typename T>
__global__ void unit_scan_kernel(const float* __restrict__ gates, const T* __restrict__ proj, int ld, int y_off,
                                 int x_off, const float* __restrict__ y_bias, const float* __restrict__ x_bias,
                                 int act, float* __restrict__ state, float* __restrict__ conv_state,
                                 const int* __restrict__ cu_q, const int* __restrict__ seq_slot, T* __restrict__ out,
                                 int C, int bw, int K, int write_state) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int seq = blockIdx.y;
  if (c >= C) return;
  const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
  const int slot = seq_slot[seq];
  const int g = c / bw, e = c - g * bw;
  const float yb = y_bias ? y_bias[c] : 0.f;
  float S = state[(size_t)slot * C + c];
  const float* gr = gates + (size_t)g * 2 * bw + e;
  constexpr int U = 4;
  int t = t0;
  for (; t + U <= t1; t += U) {
    float a[U], d[U], y[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      a[k] = gr[(size_t)(t + k) * 2 * C];
      d[k] = gr[(size_t)(t + k) * 2 * C + bw];
      y[k] = apply_act(to_f32(proj[(size_t)(t + k) * ld + y_off + c]) + yb, act);
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
      S = fmaf(a[k], S, d[k]);
      out[(size_t)(t + k) * C + c] = from_f32<T>(S * y[k]);
    }
  }
  for (; t < t1; ++t) {
    S = fmaf(gr[(size_t)t * 2 * C], S, gr[(size_t)t * 2 * C + bw]);
    out[(size_t)t * C + c] = from_f32<T>(S * apply_act(to_f32(proj[(size_t)t * ld + y_off + c]) + yb, act));
  }
  if (!write_state) return;
  state[(size_t)slot * C + c] = S;
  // the last K-1 inputs of the sequence: this step's, and before them what the state held
  float* cs = conv_state + (size_t)slot * (K - 1) * C + c;
  const int n = t1 - t0;
  const float xb = x_bias ? x_bias[c] : 0.f;
  float keep[kMaxTaps];
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k) {
    if (k < K - 1) {
      const int m = n - (K - 1) + k;                  // place within the step, negative = before it
      keep[k] = m >= 0 ? to_f32(proj[(size_t)(t0 + m) * ld + x_off + c]) + xb : cs[(size_t)(K - 1 + m) * C];
    }
  }
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k)
    if (k < K - 1) cs[(size_t)k * C] = keep[k];
}

// The same recurrence for long pieces: a block is 32 channels by kUnitChunks chunks of one sequence. Every thread runs
// its chunk from zero (the product of its a's and what it makes), the first warp chains the chunks' starting states in
// shared memory, and every thread runs its chunk again from its start, now with outputs.
constexpr int kUnitChunks = 32;

template <typename T>
__global__ void __launch_bounds__(32 * kUnitChunks)
unit_scan_chunked_kernel(const float* __restrict__ gates, const T* __restrict__ proj, int ld, int y_off, int x_off,
                         const float* __restrict__ y_bias, const float* __restrict__ x_bias, int act,
                         float* __restrict__ state, float* __restrict__ conv_state, const int* __restrict__ cu_q,
                         const int* __restrict__ seq_slot, T* __restrict__ out, int C, int bw, int K, int write_state) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sA[kUnitChunks][33], sB[kUnitChunks][33];
  const int cx = threadIdx.x, ky = threadIdx.y;
  const int c = blockIdx.x * 32 + cx;
  const int seq = blockIdx.y;
  const bool live = c < C;
  const int cc = live ? c : C - 1;
  const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
  const int n = t1 - t0;
  const int L = (n + kUnitChunks - 1) / kUnitChunks;
  const int a0 = min(t0 + ky * L, t1), a1 = min(a0 + L, t1);
  const int slot = seq_slot[seq];
  const int g = cc / bw, e = cc - g * bw;
  const float* gr = gates + (size_t)g * 2 * bw + e;
  constexpr int U = 4;
  {
    float A = 1.f, B = 0.f;
    int t = a0;
    for (; t + U <= a1; t += U) {
      float a[U], d[U];
#pragma unroll
      for (int k = 0; k < U; ++k) {
        a[k] = gr[(size_t)(t + k) * 2 * C];
        d[k] = gr[(size_t)(t + k) * 2 * C + bw];
      }
#pragma unroll
      for (int k = 0; k < U; ++k) {
        A *= a[k];
        B = fmaf(a[k], B, d[k]);
      }
    }
    for (; t < a1; ++t) {
      const float a = gr[(size_t)t * 2 * C];
      A *= a;
      B = fmaf(a, B, gr[(size_t)t * 2 * C + bw]);
    }
    sA[ky][cx] = A;
    sB[ky][cx] = B;
  }
  __syncthreads();
  if (ky == 0) {                                       // sB[k] becomes where chunk k starts
    float S = state[(size_t)slot * C + cc];
    for (int k = 0; k < kUnitChunks; ++k) {
      const float next = fmaf(sA[k][cx], S, sB[k][cx]);
      sB[k][cx] = S;
      S = next;
    }
    if (write_state && live) state[(size_t)slot * C + c] = S;
  }
  __syncthreads();
  if (live) {
    const float yb = y_bias ? y_bias[c] : 0.f;
    float S = sB[ky][cx];
    int t = a0;
    for (; t + U <= a1; t += U) {
      float a[U], d[U], y[U];
#pragma unroll
      for (int k = 0; k < U; ++k) {
        a[k] = gr[(size_t)(t + k) * 2 * C];
        d[k] = gr[(size_t)(t + k) * 2 * C + bw];
        y[k] = apply_act(to_f32(proj[(size_t)(t + k) * ld + y_off + c]) + yb, act);
      }
#pragma unroll
      for (int k = 0; k < U; ++k) {
        S = fmaf(a[k], S, d[k]);
        out[(size_t)(t + k) * C + c] = from_f32<T>(S * y[k]);
      }
    }
    for (; t < a1; ++t) {
      S = fmaf(gr[(size_t)t * 2 * C], S, gr[(size_t)t * 2 * C + bw]);
      out[(size_t)t * C + c] = from_f32<T>(S * apply_act(to_f32(proj[(size_t)t * ld + y_off + c]) + yb, act));
    }
  }
  if (!write_state || !live || ky != 0) return;
  // the last K-1 inputs of the sequence: this step's, and before them what the state held
  float* cs = conv_state + (size_t)slot * (K - 1) * C + c;
  const float xb = x_bias ? x_bias[c] : 0.f;
  float keep[kMaxTaps];
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k) {
    if (k < K - 1) {
      const int m = n - (K - 1) + k;                  // place within the step, negative = before it
      keep[k] = m >= 0 ? to_f32(proj[(size_t)(t0 + m) * ld + x_off + c]) + xb : cs[(size_t)(K - 1 + m) * C];
    }
  }
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k)
    if (k < K - 1) cs[(size_t)k * C] = keep[k];
}

}  // namespace llmie

using namespace llmie;

static inline unsigned sweep_blocks(size_t total, int threads) {
  size_t b = (total + threads - 1) / threads;
  return (unsigned)(b > 148 * 16 ? 148 * 16 : (b ? b : 1));
}

// proj [T, ld] of `dtype` holds the raw query projection at column q_off and the raw gate projection at f_off, n
// columns each; f_bias, lower float32 [n]; q_out, f_out float32 [T, n].
extern "C" int llmie_matrix_gates(const void* proj, int ld, int q_off, int f_off, const float* f_bias, const float* lower,
                                  float* q_out, float* f_out, int n_tokens, int n, int dtype, cudaStream_t stream) {
  if (n_tokens < 0 || n <= 0 || q_off < 0 || f_off < 0 || ld < q_off + n || ld < f_off + n) return LLMIE_ERR_BAD_ARG;
  if (!f_bias || !lower) return LLMIE_ERR_BAD_ARG;
  if (n_tokens == 0) return LLMIE_OK;
  const size_t total = (size_t)n_tokens * n;
  const dim3 grid(sweep_blocks(total, 256)), block(256);
  if (dtype == LLMIE_F32)
    launch_k(matrix_gates_kernel<float>, grid, block, 0, stream, (const float*)proj, ld, q_off, f_off, f_bias, lower,
             q_out, f_out, n, total);
  else if (dtype == LLMIE_BF16)
    launch_k(matrix_gates_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)proj, ld, q_off, f_off,
             f_bias, lower, q_out, f_out, n, total);
  else
    return LLMIE_ERR_DTYPE;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// qa, fg float32 [T, H * D]; v rows of H * Dv elements of `dtype`, v_ld apart; state float32 [slots, H, D, Dv];
// o float32 [T, H * Dv]. D up to 512.
// head_decay float32 [H] or null: with it, fg holds keys and S <- head_decay[h] S + k_t v_t^T.
extern "C" int llmie_matrix_scan_ex(const float* qa, const float* fg, const void* v, int v_ld, float* state,
                                    const int* cu_q, const int* seq_slot, float* o, int n_seqs, int H, int D, int Dv,
                                    int write_state, int dtype, const float* head_decay, cudaStream_t stream) {
  if (n_seqs < 0 || H <= 0 || D <= 0 || Dv <= 0 || v_ld < H * Dv) return LLMIE_ERR_BAD_ARG;
  if (D > 32 * kScanR) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (n_seqs == 0) return LLMIE_OK;
  const ScanShape g = scan_shape(D, Dv);
  const int S = g.S, R = g.R;
  const int cols = (kScanThreads / S) * g.C;
  const dim3 grid((Dv + cols - 1) / cols, H, n_seqs), block(kScanThreads);
  if (grid.y > 65535 || grid.z > 65535) return LLMIE_ERR_UNSUPPORTED_SIZE;
#define LLMIE_SCAN0_(T, C, RM, K)                                                                                           \
  launch_k(matrix_scan_kernel<T, 0, C, RM, K>, grid, block, 0, stream, qa, fg, (const T*)v, v_ld, state, cu_q, seq_slot, o, \
           H, D, Dv, S, R, write_state, (float*)nullptr, (float*)nullptr, 0, 1, head_decay)
#define LLMIE_SCAN0(T, C, RM)                                      \
  do {                                                             \
    if (head_decay) LLMIE_SCAN0_(T, C, RM, true);                  \
    else LLMIE_SCAN0_(T, C, RM, false);                            \
  } while (0)
  if (dtype == LLMIE_F32) {
    if (g.C == 4) LLMIE_SCAN0(float, 4, kScanRWide); else LLMIE_SCAN0(float, 1, kScanR);
  } else if (dtype == LLMIE_BF16) {
    if (g.C == 4) LLMIE_SCAN0(__nv_bfloat16, 4, kScanRWide); else LLMIE_SCAN0(__nv_bfloat16, 1, kScanR);
  } else {
    return LLMIE_ERR_DTYPE;
  }
#undef LLMIE_SCAN0
#undef LLMIE_SCAN0_
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

extern "C" int llmie_matrix_scan(const float* qa, const float* fg, const void* v, int v_ld, float* state,
                                 const int* cu_q, const int* seq_slot, float* o, int n_seqs, int H, int D, int Dv,
                                 int write_state, int dtype, cudaStream_t stream) {
  return llmie_matrix_scan_ex(qa, fg, v, v_ld, state, cu_q, seq_slot, o, n_seqs, H, D, Dv, write_state, dtype, nullptr,
                              stream);
}

template <typename T, int C, int RM, bool K>
static void matrix_scan_chunked_launch(const float* qa, const float* fg, const T* v, int v_ld, float* state,
                                       const int* cu_q, const int* seq_slot, float* o, float* ws, float* decay,
                                       int n_seqs, int H, int D, int Dv, int S, int R, int L, int NC, int write_state,
                                       const float* head_decay, cudaStream_t stream) {
  const int cols = (kScanThreads / S) * C;
  const dim3 grid((Dv + cols - 1) / cols, H, n_seqs * NC), block(kScanThreads);
  launch_k(matrix_scan_kernel<T, 1, C, RM, K>, grid, block, 0, stream, qa, fg, v, v_ld, state, cu_q, seq_slot, o, H, D, Dv, S, R,
           write_state, ws, decay, L, NC, head_decay);
  const size_t HDDv = (size_t)H * D * Dv;
  launch_k(matrix_scan_chain_kernel, dim3((unsigned)((HDDv + 255) / 256), n_seqs), dim3(256), 0, stream,
           (const float*)state, cu_q, seq_slot, ws, (const float*)decay, H, D, Dv, L, NC);
  launch_k(matrix_scan_kernel<T, 2, C, RM, K>, grid, block, 0, stream, qa, fg, v, v_ld, state, cu_q, seq_slot, o, H, D, Dv, S, R,
           write_state, ws, decay, L, NC, head_decay);
}

// llmie_matrix_scan for long pieces: chunks of `chunk` tokens run side by side. n_chunks >= ceil(longest piece / chunk);
// ws float32 [n_seqs, n_chunks, H, D, Dv] and decay float32 [n_seqs, n_chunks, H, D] are scratch.
extern "C" int llmie_matrix_scan_chunked_ex(const float* qa, const float* fg, const void* v, int v_ld, float* state,
                                            const int* cu_q, const int* seq_slot, float* o, float* ws, float* decay,
                                            int n_seqs, int H, int D, int Dv, int chunk, int n_chunks, int write_state,
                                            int dtype, const float* head_decay, cudaStream_t stream) {
  if (n_seqs < 0 || H <= 0 || D <= 0 || Dv <= 0 || v_ld < H * Dv || chunk <= 0 || n_chunks <= 0 || !ws || !decay)
    return LLMIE_ERR_BAD_ARG;
  if (D > 32 * kScanR) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (n_seqs == 0) return LLMIE_OK;
  const ScanShape g = scan_shape(D, Dv);
  const int S = g.S, R = g.R;
  if (H > 65535 || (long long)n_seqs * n_chunks > 65535 || n_seqs > 65535) return LLMIE_ERR_UNSUPPORTED_SIZE;
#define LLMIE_SCANC_(T, C, RM, K)                                                                                            \
  matrix_scan_chunked_launch<T, C, RM, K>(qa, fg, (const T*)v, v_ld, state, cu_q, seq_slot, o, ws, decay, n_seqs, H, D, Dv, \
                                          S, R, chunk, n_chunks, write_state, head_decay, stream)
#define LLMIE_SCANC(T, C, RM)                                      \
  do {                                                             \
    if (head_decay) LLMIE_SCANC_(T, C, RM, true);                  \
    else LLMIE_SCANC_(T, C, RM, false);                            \
  } while (0)
  if (dtype == LLMIE_F32) {
    if (g.C == 4) LLMIE_SCANC(float, 4, kScanRWide); else LLMIE_SCANC(float, 1, kScanR);
  } else if (dtype == LLMIE_BF16) {
    if (g.C == 4) LLMIE_SCANC(__nv_bfloat16, 4, kScanRWide); else LLMIE_SCANC(__nv_bfloat16, 1, kScanR);
  } else {
    return LLMIE_ERR_DTYPE;
  }
#undef LLMIE_SCANC
#undef LLMIE_SCANC_
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

extern "C" int llmie_matrix_scan_chunked(const float* qa, const float* fg, const void* v, int v_ld, float* state,
                                         const int* cu_q, const int* seq_slot, float* o, float* ws, float* decay,
                                         int n_seqs, int H, int D, int Dv, int chunk, int n_chunks, int write_state,
                                         int dtype, cudaStream_t stream) {
  return llmie_matrix_scan_chunked_ex(qa, fg, v, v_ld, state, cu_q, seq_slot, o, ws, decay, n_seqs, H, D, Dv, chunk,
                                      n_chunks, write_state, dtype, nullptr, stream);
}

// proj [T, ld] of `dtype`; out_k float32 [T, n_k] = act(proj[:, off_k : off_k + n_k]) for up to three runs (n_k = 0: unused).
extern "C" int llmie_act_columns(const void* proj, int ld, int off0, int n0, float* out0, int off1, int n1, float* out1,
                                 int off2, int n2, float* out2, int act, int n_tokens, int dtype, cudaStream_t stream) {
  if (n_tokens < 0 || n0 <= 0 || n1 < 0 || n2 < 0 || off0 < 0 || off1 < 0 || off2 < 0) return LLMIE_ERR_BAD_ARG;
  if (ld < off0 + n0 || (n1 && ld < off1 + n1) || (n2 && ld < off2 + n2)) return LLMIE_ERR_BAD_ARG;
  if (!out0 || (n1 && !out1) || (n2 && !out2)) return LLMIE_ERR_BAD_ARG;
  if (n_tokens == 0) return LLMIE_OK;
  const size_t total = (size_t)n_tokens * (n0 + n1 + n2);
  const dim3 grid(sweep_blocks(total, 256)), block(256);
  if (dtype == LLMIE_F32)
    launch_k(act_columns_kernel<float>, grid, block, 0, stream, (const float*)proj, ld, off0, n0, out0, off1, n1, out1,
             off2, n2, out2, act, total);
  else if (dtype == LLMIE_BF16)
    launch_k(act_columns_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)proj, ld, off0, n0, out0,
             off1, n1, out1, off2, n2, out2, act, total);
  else
    return LLMIE_ERR_DTYPE;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// o float32 [n_items, Dv] (an item = a token's head); w float32 [Dv]; y [n_items, Dv] of `dtype`.
// gate (of `dtype`, rows gate_ld apart, items_per_row items a row) or null: y is also multiplied by sigmoid(gate).
extern "C" int llmie_head_rmsnorm_gated(const float* o, const float* w, float eps, void* y, long long n_items, int Dv,
                                        int dtype, const void* gate, int gate_ld, int items_per_row,
                                        cudaStream_t stream) {
  if (n_items < 0 || Dv <= 0 || (gate && (items_per_row <= 0 || gate_ld < items_per_row * Dv))) return LLMIE_ERR_BAD_ARG;
  if (n_items == 0) return LLMIE_OK;
  if (Dv >= 512 && Dv % 4 == 0 && aligned16(o) && aligned16(w) && n_items <= 0x7fffffffLL) {
    // wide items: a block each
    const dim3 grid((unsigned)n_items), block(Dv >= 1024 ? 256 : 128);
    if (dtype == LLMIE_F32)
      launch_k(row_rmsnorm_kernel<float>, grid, block, 0, stream, o, w, eps, (float*)y, Dv, (const float*)gate, gate_ld,
               items_per_row);
    else if (dtype == LLMIE_BF16)
      launch_k(row_rmsnorm_kernel<__nv_bfloat16>, grid, block, 0, stream, o, w, eps, (__nv_bfloat16*)y, Dv,
               (const __nv_bfloat16*)gate, gate_ld, items_per_row);
    else
      return LLMIE_ERR_DTYPE;
    LLMIE_LAUNCH_CHECK();
    return LLMIE_OK;
  }
  const int warps = 4;
  const long long blocks = (n_items + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return LLMIE_ERR_UNSUPPORTED_SIZE;
  const dim3 grid((unsigned)blocks), block(warps * 32);
  if (dtype == LLMIE_F32)
    launch_k(head_rmsnorm_kernel<float>, grid, block, 0, stream, o, w, eps, (float*)y, Dv, (size_t)n_items,
             (const float*)gate, gate_ld, items_per_row);
  else if (dtype == LLMIE_BF16)
    launch_k(head_rmsnorm_kernel<__nv_bfloat16>, grid, block, 0, stream, o, w, eps, (__nv_bfloat16*)y, Dv,
             (size_t)n_items, (const __nv_bfloat16*)gate, gate_ld, items_per_row);
  else
    return LLMIE_ERR_DTYPE;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

extern "C" int llmie_head_rmsnorm(const float* o, const float* w, float eps, void* y, long long n_items, int Dv,
                                  int dtype, cudaStream_t stream) {
  return llmie_head_rmsnorm_gated(o, w, eps, y, n_items, Dv, dtype, nullptr, 0, 1, stream);
}

// proj [T, ld] of `dtype` with the convolution's input at column x_off (C columns); x_bias, conv_bias float32 [C] or
// null; taps float32 [C, K] (the last column multiplies the current token); conv_state float32 [slots, K-1, C];
// u float32 [T, C].
extern "C" int llmie_causal_conv(const void* proj, int ld, int x_off, const float* x_bias, const float* taps,
                                 const float* conv_bias, const float* conv_state, const int* cu_q, const int* tok_seq,
                                 const int* seq_slot, float* u, int n_tokens, int C, int K, int dtype,
                                 cudaStream_t stream) {
  if (n_tokens < 0 || C <= 0 || K <= 0 || x_off < 0 || ld < x_off + C) return LLMIE_ERR_BAD_ARG;
  if (K > kMaxTaps) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (n_tokens == 0) return LLMIE_OK;
  const int tile = n_tokens >= 1024 ? 16 : (n_tokens >= 64 ? 4 : 1);
  const int threads = C >= 128 ? 128 : ((C + 31) / 32) * 32;
  const dim3 grid((C + threads - 1) / threads, (n_tokens + tile - 1) / tile), block(threads);
  if (grid.y > 65535) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (dtype == LLMIE_F32)
    launch_k(causal_conv_kernel<float>, grid, block, 0, stream, (const float*)proj, ld, x_off, x_bias, taps, conv_bias,
             conv_state, cu_q, tok_seq, seq_slot, u, C, K, n_tokens, tile);
  else if (dtype == LLMIE_BF16)
    launch_k(causal_conv_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)proj, ld, x_off, x_bias,
             taps, conv_bias, conv_state, cu_q, tok_seq, seq_slot, u, C, K, n_tokens, tile);
  else
    return LLMIE_ERR_DTYPE;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// gates float32 [T, 2 C] (per group of bw channels: r's pre-activations, then i's), changed in place into (a, drive);
// u float32 [T, C]; r_bias, i_bias, lam float32 [C].
extern "C" int llmie_unit_gate_values(float* gates, const float* u, const float* r_bias, const float* i_bias,
                                      const float* lam, float c_decay, int n_tokens, int C, int bw,
                                      cudaStream_t stream) {
  if (n_tokens < 0 || C <= 0 || bw <= 0 || C % bw) return LLMIE_ERR_BAD_ARG;
  if (n_tokens == 0) return LLMIE_OK;
  const size_t total = (size_t)n_tokens * C;
  launch_k(unit_gate_values_kernel, dim3(sweep_blocks(total, 256)), dim3(256), 0, stream, gates, u, r_bias, i_bias, lam,
           c_decay, C, bw, total);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// gates as left by llmie_unit_gate_values; proj [T, ld] of `dtype` with the output gate's raw projection at y_off and
// the convolution's input at x_off; state float32 [slots, C]; conv_state float32 [slots, K-1, C]; out [T, C] of `dtype`.
// chunked != 0: the form for long pieces (every sequence's piece in 32 chunks side by side).
extern "C" int llmie_unit_scan(const float* gates, const void* proj, int ld, int y_off, int x_off, const float* y_bias,
                               const float* x_bias, int act, float* state, float* conv_state, const int* cu_q,
                               const int* seq_slot, void* out, int n_seqs, int C, int bw, int K, int write_state,
                               int chunked, int dtype, cudaStream_t stream) {
  if (n_seqs < 0 || C <= 0 || bw <= 0 || C % bw || K <= 0 || y_off < 0 || x_off < 0 || ld < y_off + C || ld < x_off + C)
    return LLMIE_ERR_BAD_ARG;
  if (act < 0 || act > 4) return LLMIE_ERR_BAD_ARG;
  if (K > kMaxTaps) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (n_seqs == 0) return LLMIE_OK;
  if (n_seqs > 65535) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (chunked) {
    const dim3 grid((C + 31) / 32, n_seqs), block(32, kUnitChunks);
    if (dtype == LLMIE_F32)
      launch_k(unit_scan_chunked_kernel<float>, grid, block, 0, stream, gates, (const float*)proj, ld, y_off, x_off,
               y_bias, x_bias, act, state, conv_state, cu_q, seq_slot, (float*)out, C, bw, K, write_state);
    else if (dtype == LLMIE_BF16)
      launch_k(unit_scan_chunked_kernel<__nv_bfloat16>, grid, block, 0, stream, gates, (const __nv_bfloat16*)proj, ld,
               y_off, x_off, y_bias, x_bias, act, state, conv_state, cu_q, seq_slot, (__nv_bfloat16*)out, C, bw, K,
               write_state);
    else
      return LLMIE_ERR_DTYPE;
    LLMIE_LAUNCH_CHECK();
    return LLMIE_OK;
  }
  const int threads = C >= 128 ? 128 : ((C + 31) / 32) * 32;
  const dim3 grid((C + threads - 1) / threads, n_seqs), block(threads);
  if (dtype == LLMIE_F32)
    launch_k(unit_scan_kernel<float>, grid, block, 0, stream, gates, (const float*)proj, ld, y_off, x_off, y_bias,
             x_bias, act, state, conv_state, cu_q, seq_slot, (float*)out, C, bw, K, write_state);
  else if (dtype == LLMIE_BF16)
    launch_k(unit_scan_kernel<__nv_bfloat16>, grid, block, 0, stream, gates, (const __nv_bfloat16*)proj, ld, y_off,
             x_off, y_bias, x_bias, act, state, conv_state, cu_q, seq_slot, (__nv_bfloat16*)out, C, bw, K, write_state);
  else
    return LLMIE_ERR_DTYPE;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}
