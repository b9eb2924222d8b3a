// Attention over the paged cache on the tensor cores for the shapes the other fast kernels do not take: any head size
// that is a multiple of 16 up to 1024, a value size of its own up to 512 (a multiple of 8), values that are a column
// range of the key rows (a latent that is key and value at once), prompts and one-token steps alike, and the options
// that change single scores (a cap c tanh(s / c), a bias by distance from a per-head table, a sink whose score is a
// number per head) besides scale and window. bfloat16 in and out, float32 scores, softmax and accumulators.
// With `sig_bias` (a number per query head) there is no softmax: a visible key's weight is sigmoid(score + that number),
// nothing is normalised over the keys, and the running maximum, the rescaling and the final division fall away.
//
// All query heads that share a key/value head work on the same keys, so the rows of the problem are the (token, head)
// pairs of one key/value head of one sequence: row r = token * G + head-in-group. A block of eight warps takes 32
// consecutive rows and walks over the keys its rows may see in tiles of 32 (half a cache page, fetched with cp.async
// into a two-stage ring):
//   S = Q K^T      mma.sync m16n8k16: a warp takes 16 rows, all 32 keys and a quarter of the head size (partial tiles
//                  into shared memory, added in the softmax)
//   softmax        a warp per four rows, eight lanes a row, four keys a lane: scale, cap, bias, mask, running maximum
//                  and sum; P in bfloat16
//   O = aO + P V   every warp owns a share of the value columns for all 32 rows (V fragments by ldmatrix.trans)
// The denominator stays with the warp that owns the row; the final 1 / l (with the sink's term) goes through shared memory.
#include "common.cuh"
#include <math.h>

namespace llmie {

constexpr int kRmRows = 32;      // rows (token, head) per block
constexpr int kRmKeys = 32;      // keys per tile
constexpr int kRmWarps = 8;

struct RowsArgs {
  const __nv_bfloat16* q;        // [T, n_q * hd]
  const __nv_bfloat16* k_cache;  // [pages, n_kv, page, hd]
  const __nv_bfloat16* v_cache;  // rows of hdv elements, v_ld apart; may point into k_cache
  __nv_bfloat16* out;            // [T, n_q * hdv]
  const int* cu_q;               // [n_seqs + 1]
  const int* seq_slot;
  const int* seq_start;
  const int* block_table;
  int max_pages, page_size, n_q, n_kv, hd, hdv, v_ld;
  float scale;
  int window;
  float softcap;
  const float* dist_bias;        // [n_q, bias_len] or null
  int bias_len;
  const float* sink_vals;        // [n_q] or null
  int sink;
  const float* sig_bias;         // [n_q] or null: sigmoid weights instead of a softmax
  int shared_rows;               // 1: the values are columns of the staged key rows (no second fetch)
};

__device__ __forceinline__ void rm_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float rm_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// NTW: tiles of 8 value columns a warp owns (columns w * 8, (w + 8) * 8, ...), so hdv <= 64 * NTW.
template <int NTW>
__global__ void __launch_bounds__(kRmWarps * 32)
attention_rows_mma_kernel(const RowsArgs p) {
  extern __shared__ __align__(16) unsigned char rm_smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.z, hk = blockIdx.y;
  const int G = p.n_q / p.n_kv;
  const int q_begin = p.cu_q[seq], q_len = p.cu_q[seq + 1] - q_begin;
  const int n_rows = q_len * G;
  const int r0 = blockIdx.x * kRmRows;
  if (r0 >= n_rows) return;
  const int start = p.seq_start[seq];
  const int kpitch = p.hd + 8;                            // elements; 16 bytes more than a row, against bank conflicts
  const int vpitch = p.shared_rows ? kpitch : p.hdv + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(rm_smem);                    // [32][kpitch]
  __nv_bfloat16* Ks = Qs + kRmRows * kpitch;                                         // [2][32][kpitch]
  __nv_bfloat16* Vs = p.shared_rows ? Ks : Ks + 2 * kRmKeys * kpitch;                // [2][32][vpitch]
  unsigned char* tail = reinterpret_cast<unsigned char*>(Ks + 2 * kRmKeys * kpitch + (p.shared_rows ? 0 : 2 * kRmKeys * vpitch));
  float* S = reinterpret_cast<float*>(tail);                                         // [4][32][33] partial score tiles
  __nv_bfloat16* P = reinterpret_cast<__nv_bfloat16*>(S + 4 * kRmRows * 33);         // [32][40]
  float* alpha_s = reinterpret_cast<float*>(P + kRmRows * 40);                       // [32]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int* pages = p.block_table + (size_t)p.seq_slot[seq] * p.max_pages;

  // positions of the block's rows: the first and last token decide which keys the block walks over
  const int tok_first = r0 / G;
  const int tok_last = min(r0 + kRmRows - 1, n_rows - 1) / G;
  const int pos_last = start + tok_last;
  const int key_lo = p.window > 0 ? max(start + tok_first - p.window + 1, 0) : 0;
  const int tile_lo = key_lo / kRmKeys, tile_hi = pos_last / kRmKeys;

  // ---- the queries of the block's rows
  const int q_chunks = p.hd / 8;
  for (int c = tid; c < kRmRows * q_chunks; c += kRmWarps * 32) {
    const int r = c / q_chunks, ch = c % q_chunks;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r0 + r < n_rows) {
      const int tok = (r0 + r) / G, head = hk * G + (r0 + r) % G;
      v = *reinterpret_cast<const uint4*>(p.q + ((size_t)(q_begin + tok) * p.n_q + head) * p.hd + ch * 8);
    }
    *reinterpret_cast<uint4*>(Qs + r * kpitch + ch * 8) = v;
  }
  auto issue = [&](int tile, int stage) {
    const int key0 = tile * kRmKeys;
    const int page = pages[key0 / p.page_size];
    const size_t row0 = ((size_t)page * p.n_kv + hk) * p.page_size + key0 % p.page_size;
    const unsigned kdst = (unsigned)__cvta_generic_to_shared(Ks + stage * kRmKeys * kpitch);
    for (int c = tid; c < kRmKeys * q_chunks; c += kRmWarps * 32) {
      const int r = c / q_chunks, ch = c % q_chunks;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(kdst + (unsigned)(r * kpitch + ch * 8) * 2u),
                   "l"(p.k_cache + (row0 + r) * p.hd + ch * 8) : "memory");
    }
    if (!p.shared_rows) {
      const int v_chunks = p.hdv / 8;
      const unsigned vdst = (unsigned)__cvta_generic_to_shared(Vs + stage * kRmKeys * vpitch);
      for (int c = tid; c < kRmKeys * v_chunks; c += kRmWarps * 32) {
        const int r = c / v_chunks, ch = c % v_chunks;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(vdst + (unsigned)(r * vpitch + ch * 8) * 2u),
                     "l"(p.v_cache + (row0 + r) * p.v_ld + ch * 8) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  issue(tile_lo, 0);

  // softmax: a warp owns four rows, eight lanes a row, four keys a lane; the row's state is the same in its eight lanes
  const int sm_row = warp * 4 + (lane >> 3), sm_key0 = (lane & 7) * 4;
  float m_run = -INFINITY, l_run = 0.f;
  const int pos_row = r0 + sm_row < n_rows ? start + (r0 + sm_row) / G : -1;
  const float* bias_row = (p.dist_bias && r0 + sm_row < n_rows)
                              ? p.dist_bias + (size_t)(hk * G + (r0 + sm_row) % G) * p.bias_len : nullptr;
  float acc[2][NTW][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int i = 0; i < NTW; ++i) acc[mt][i][0] = acc[mt][i][1] = acc[mt][i][2] = acc[mt][i][3] = 0.f;
  const float inv_cap = p.softcap > 0.f ? 1.f / p.softcap : 0.f;
  const float sig_b = (p.sig_bias && r0 + sm_row < n_rows) ? p.sig_bias[hk * G + (r0 + sm_row) % G] : 0.f;
  const int s_mt = warp >> 2, s_nt = warp & 3;            // the score tile of this warp
  const int n_vt = p.hdv / 8;                             // tiles of value columns there are

  for (int tile = tile_lo; tile <= tile_hi; ++tile) {
    const int stage = (tile - tile_lo) & 1;
    if (tile < tile_hi) {
      issue(tile + 1, stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();                                      // the tile (and, the first time, Q) is in shared memory
    const __nv_bfloat16* Kt = Ks + stage * kRmKeys * kpitch;
    const __nv_bfloat16* Vt = p.shared_rows ? Kt : Vs + stage * kRmKeys * vpitch;
    // ---- S = Q K^T. A warp takes 16 rows, all 32 keys and every fourth step of 16 over the head size, so that a
    // query fragment it has fetched serves four products; the four partial tiles of a row half meet in the softmax.
    {
      float c[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.f;
      const __nv_bfloat16* qa = Qs + (s_mt * 16 + g) * kpitch + 2 * t;
      const __nv_bfloat16* kb = Kt + g * kpitch + 2 * t;
      for (int ks = s_nt * 16; ks < p.hd; ks += 64) {
        const unsigned a0 = *reinterpret_cast<const unsigned*>(qa + ks);
        const unsigned a1 = *reinterpret_cast<const unsigned*>(qa + 8 * kpitch + ks);
        const unsigned a2 = *reinterpret_cast<const unsigned*>(qa + ks + 8);
        const unsigned a3 = *reinterpret_cast<const unsigned*>(qa + 8 * kpitch + ks + 8);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const unsigned b0 = *reinterpret_cast<const unsigned*>(kb + nt * 8 * kpitch + ks);
          const unsigned b1 = *reinterpret_cast<const unsigned*>(kb + nt * 8 * kpitch + ks + 8);
          rm_mma(c[nt], a0, a1, a2, a3, b0, b1);
        }
      }
      float* s0 = S + s_nt * (kRmRows * 33) + (s_mt * 16 + g) * 33 + 2 * t;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        s0[nt * 8] = c[nt][0];
        s0[nt * 8 + 1] = c[nt][1];
        s0[8 * 33 + nt * 8] = c[nt][2];
        s0[8 * 33 + nt * 8 + 1] = c[nt][3];
      }
    }
    __syncthreads();
    // ---- softmax of this lane's row over its four keys: scale, cap, bias, mask, running maximum and sum
    {
      float sc[4];
      bool vis[4];
      float mx = -INFINITY;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = sm_row * 33 + sm_key0 + e;
        float x = ((S[col] + S[kRmRows * 33 + col]) + (S[2 * kRmRows * 33 + col] + S[3 * kRmRows * 33 + col])) * p.scale;
        if (p.softcap > 0.f) x = p.softcap * rm_tanh(x * inv_cap);
        const int dist = pos_row - (tile * kRmKeys + sm_key0 + e);
        if (bias_row) x += bias_row[min(max(dist, 0), p.bias_len - 1)];
        vis[e] = dist >= 0 && (p.window == 0 || dist < p.window);
        sc[e] = vis[e] ? x : -INFINITY;
        mx = fmaxf(mx, sc[e]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      float pr[4], al = 1.f;
      if (p.sig_bias) {
#pragma unroll
        for (int e = 0; e < 4; ++e) pr[e] = vis[e] ? 1.f / (1.f + __expf(-(sc[e] + sig_b))) : 0.f;
      } else {
        const float m_new = fmaxf(m_run, mx);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        float sum = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          pr[e] = vis[e] ? __expf(sc[e] - m_use) : 0.f;
          sum += pr[e];
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        al = __expf(m_run - m_use);                       // 0 while the row has seen no key
        l_run = l_run * al + sum;
        m_run = m_new;
      }
      __nv_bfloat162* pw = reinterpret_cast<__nv_bfloat162*>(P + sm_row * 40 + sm_key0);
      pw[0] = __floats2bfloat162_rn(pr[0], pr[1]);
      pw[1] = __floats2bfloat162_rn(pr[2], pr[3]);
      if ((lane & 7) == 0) alpha_s[sm_row] = al;
    }
    __syncthreads();
    // ---- O = alpha O + P V for this warp's value columns, both 16-row halves
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
      const float al_lo = alpha_s[mt * 16 + g], al_hi = alpha_s[mt * 16 + g + 8];
#pragma unroll
      for (int i = 0; i < NTW; ++i) {
        acc[mt][i][0] *= al_lo;
        acc[mt][i][1] *= al_lo;
        acc[mt][i][2] *= al_hi;
        acc[mt][i][3] *= al_hi;
      }
    }
#pragma unroll
    for (int ks = 0; ks < kRmKeys; ks += 16) {
      unsigned a[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const __nv_bfloat16* pa = P + (mt * 16 + g) * 40 + ks + 2 * t;
        a[mt][0] = *reinterpret_cast<const unsigned*>(pa);
        a[mt][1] = *reinterpret_cast<const unsigned*>(pa + 8 * 40);
        a[mt][2] = *reinterpret_cast<const unsigned*>(pa + 8);
        a[mt][3] = *reinterpret_cast<const unsigned*>(pa + 8 * 40 + 8);
      }
#pragma unroll
      for (int i = 0; i < NTW; ++i) {
        const int vt = warp + i * kRmWarps;
        if (vt < n_vt) {
          unsigned b0, b1;
          const unsigned addr = (unsigned)__cvta_generic_to_shared(Vt + (ks + (lane & 15)) * vpitch + vt * 8);
          asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
          rm_mma(acc[0][i], a[0][0], a[0][1], a[0][2], a[0][3], b0, b1);
          rm_mma(acc[1][i], a[1][0], a[1][1], a[1][2], a[1][3], b0, b1);
        }
      }
    }
    __syncthreads();                                      // S, P and this stage may be written again
  }
  // ---- the rows' final factors: 1 / l, with the sink's term in the denominator
  if ((lane & 7) == 0) {
    const int r = r0 + sm_row;
    float f = 0.f;
    if (r < n_rows && p.sig_bias) {
      f = 1.f;
    } else if (r < n_rows) {
      float l = l_run, num = 1.f;
      if (p.sink) {
        const float sv = p.sink_vals ? p.sink_vals[hk * G + r % G] : 0.f;
        const float mx = fmaxf(m_run, sv);
        num = m_run == -INFINITY ? 0.f : __expf(m_run - mx);
        l = l * num + __expf(sv - mx);
      }
      f = l > 0.f ? num / l : 0.f;
    }
    alpha_s[sm_row] = f;
  }
  __syncthreads();
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int rl = mt * 16 + g + 8 * half;
      const int r = r0 + rl;
      if (r >= n_rows) continue;
      const float f = alpha_s[rl];
      __nv_bfloat16* orow = p.out + ((size_t)(q_begin + r / G) * p.n_q + hk * G + r % G) * p.hdv;
#pragma unroll
      for (int i = 0; i < NTW; ++i) {
        const int vt = warp + i * kRmWarps;
        if (vt < n_vt)
          *reinterpret_cast<__nv_bfloat162*>(orow + vt * 8 + 2 * t) =
              __floats2bfloat162_rn(acc[mt][i][2 * half] * f, acc[mt][i][2 * half + 1] * f);
      }
    }
}

static size_t rows_smem_bytes(int hd, int hdv, bool shared_rows) {
  const size_t kp = hd + 8, vp = hdv + 8;
  size_t b = (size_t)kRmRows * kp * 2 + 2 * (size_t)kRmKeys * kp * 2;
  if (!shared_rows) b += 2 * (size_t)kRmKeys * vp * 2;
  return b + 4 * kRmRows * 33 * 4 + kRmRows * 40 * 2 + kRmRows * 4;
}

}  // namespace llmie

using namespace llmie;

// Whether the kernel takes these sizes (no launch).
extern "C" int llmie_attention_rows_mma_supported(int hd, int hdv, int page_size, int shared_rows) {
  if (hd <= 0 || hd % 16 || hd > 1024 || hdv <= 0 || hdv % 8 || hdv > 512 || page_size % kRmKeys) return 0;
  if (shared_rows && hdv > hd) return 0;
  return rows_smem_bytes(hd, hdv, shared_rows != 0) <= 200 * 1024 ? 1 : 0;
}

// q [T, n_q hd], out [T, n_q hdv], caches as in llmie_attention_paged_ex (v_cache rows v_ld apart; shared_rows != 0: the
// values are the first hdv columns of the key rows themselves), all bfloat16. cu_q int32 [n_seqs + 1]: where each
// sequence's tokens start; seq_start int32 [n_seqs]: tokens held before this step; max_q_len: upper bound of a
// sequence's tokens in this step (sizes the grid). sig_bias float32 [n_q] or null.
extern "C" int llmie_attention_rows_mma(const void* q, const void* k_cache, const void* v_cache, void* out,
                                        const int* cu_q, const int* seq_slot, const int* seq_start,
                                        const int* block_table, int max_pages, int page_size, int n_seqs, int max_q_len,
                                        int n_q, int n_kv, int hd, int hdv, int v_ld, int shared_rows, float scale,
                                        int window, float softcap, const float* dist_bias, int bias_len,
                                        const float* sink_vals, int sink, const float* sig_bias,
                                        cudaStream_t stream) {
  if (sig_bias && (sink || softcap > 0.f || dist_bias)) return LLMIE_ERR_BAD_ARG;
  if (n_seqs < 0 || max_q_len < 0 || n_q <= 0 || n_kv <= 0 || n_q % n_kv || max_pages <= 0 || window < 0 || softcap < 0.f)
    return LLMIE_ERR_BAD_ARG;
  if ((dist_bias && bias_len <= 0) || (sink_vals && !sink) || v_ld < hdv) return LLMIE_ERR_BAD_ARG;
  if (!llmie_attention_rows_mma_supported(hd, hdv, page_size, shared_rows)) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache) || v_ld % 8) return LLMIE_ERR_ALIGNMENT;
  if (n_seqs == 0 || max_q_len == 0) return LLMIE_OK;
  const int G = n_q / n_kv;
  const long long row_blocks = ((long long)max_q_len * G + kRmRows - 1) / kRmRows;
  if (row_blocks > 0x7fffffffLL || n_kv > 65535 || n_seqs > 65535) return LLMIE_ERR_UNSUPPORTED_SIZE;
  RowsArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out,
             cu_q, seq_slot, seq_start, block_table, max_pages, page_size, n_q, n_kv, hd, hdv, v_ld, scale, window,
             softcap, dist_bias, bias_len, sink_vals, sink ? 1 : 0, sig_bias, shared_rows ? 1 : 0};
  const size_t smem = rows_smem_bytes(hd, hdv, shared_rows != 0);
  dim3 grid((unsigned)row_blocks, n_kv, n_seqs);
  const int ntw = (hdv / 8 + kRmWarps - 1) / kRmWarps;
#define LLMIE_ROWS_LAUNCH(N)                                                                                     \
  do {                                                                                                           \
    cudaFuncSetAttribute(attention_rows_mma_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    launch_k(attention_rows_mma_kernel<N>, grid, dim3(kRmWarps * 32), smem, stream, a);                          \
  } while (0)
  if (ntw <= 1) LLMIE_ROWS_LAUNCH(1);
  else if (ntw <= 2) LLMIE_ROWS_LAUNCH(2);
  else if (ntw <= 4) LLMIE_ROWS_LAUNCH(4);
  else LLMIE_ROWS_LAUNCH(8);
#undef LLMIE_ROWS_LAUNCH
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}
