// Latent attention: what happens between the projections and the attention itself.
//
// A layer projects each token to a latent of `rank` numbers plus `rot` numbers that become ONE rotated key part shared
// by all heads. The cache keeps per token the row [c | k_rot]: c the latent after its RMS norm, k_rot after rotation.
// With per-head matrices U_k [dim, rank] (keys) and U_v [vdim, rank] (values) the scores are
//   q_plain . (U_k c) + q_rot . k_rot  =  (U_k^T q_plain) . c + q_rot . k_rot,
// so attention runs over the cached rows directly with ONE key head of size rank + rot, queries [U_k^T q_plain | q_rot],
// and the latent itself as the value (the first `rank` columns of the same rows); U_v is applied to the result. The
// two per-head products are the batched form of grouped_gemm.cu. This file holds the kernel around them:
//
//   latent_prepare   per token: RMS norm of the latent (float32, eps inside the root, plain weight), rotation of the
//                    shared key part and of every head's rotated query part (pairs (2i, 2i+1), angle from a float32
//                    (cos, sin) table by position; entries beyond the rotated ones pass unchanged), the cache write,
//                    and the rotated query parts into their columns of the query rows the attention kernel reads.
#include "common.cuh"

namespace llmie {

template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ proj, int ld, const T* __restrict__ q_src, int q_ld, int q_off, int dkv_off,
                      T* __restrict__ q_out,
                      T* __restrict__ cache, const float* __restrict__ norm_w, float eps,
                      const float* __restrict__ table, int table_len, int rot_dims, const int* __restrict__ tok_pos,
                      const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                      const int* __restrict__ block_table, int max_pages, int page_size, int n_heads, int dim, int rot,
                      int rank, int write) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int tp = pos < table_len ? pos : table_len - 1;      // the host refuses longer sequences
  const float* cs = table + (size_t)tp * (rot_dims / 2) * 2;
  const T* row = proj + (size_t)t * ld;
  if (write) {
    const T* craw = row + dkv_off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
      const float x = to_f32(craw[i]);
      ss += x * x;
    }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / (float)rank + eps);
    const int slot = seq_slot[tok_seq[t]];
    const int page = block_table[(size_t)slot * max_pages + pos / page_size];
    T* dst = cache + ((size_t)page * page_size + pos % page_size) * (rank + rot);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f32<T>(to_f32(craw[i]) * rstd * norm_w[i]);
    const T* kr = craw + rank;
    for (int i = threadIdx.x; i < rot; i += blockDim.x) {
      float v = to_f32(kr[i]);
      if (i < rot_dims) {
        const float c = cs[(i >> 1) * 2], s = cs[(i >> 1) * 2 + 1];
        const float other = to_f32(kr[i ^ 1]);
        v = (i & 1) ? v * c + other * s : v * c - other * s;
      }
      dst[rank + i] = from_f32<T>(v);
    }
  }
  const int qw = dim + rot, ow = rank + rot;
  for (int idx = threadIdx.x; idx < n_heads * rot; idx += blockDim.x) {
    const int h = idx / rot, i = idx - h * rot;
    const T* qr = q_src + (size_t)t * q_ld + q_off + (size_t)h * qw + dim;
    float v = to_f32(qr[i]);
    if (i < rot_dims) {
      const float c = cs[(i >> 1) * 2], s = cs[(i >> 1) * 2 + 1];
      const float other = to_f32(qr[i ^ 1]);
      v = (i & 1) ? v * c + other * s : v * c - other * s;
    }
    q_out[(size_t)t * n_heads * ow + (size_t)h * ow + rank + i] = from_f32<T>(v);
  }
}

}  // namespace llmie

using namespace llmie;

// proj [T, ld] rows holding the queries at column q_off (n_heads * (dim + rot)) and, when write != 0, the latent
// projection at column dkv_off (rank + rot); q_out [T, n_heads * (rank + rot)]: only the last `rot` columns of each head
// are written here; cache [n_pages, 1, page_size, rank + rot]; all three of `dtype`. norm_w float32 [rank];
// table float32 [table_len, rot_dims / 2, 2] of (cos, sin).
// The queries are read from q_src (rows q_ld apart, column q_off on), which may be another tensor than proj: designs
// whose queries pass through a latent of their own make them with a second product.
extern "C" int llmie_latent_prepare_from(const void* proj, int ld, const void* q_src, int q_ld, int q_off, int dkv_off,
                                         void* q_out, void* cache, const float* norm_w, float eps, const float* table,
                                         int table_len, int rot_dims, const int* tok_pos, const int* tok_seq,
                                         const int* seq_slot, const int* block_table, int max_pages, int page_size,
                                         int n_tokens, int n_heads, int dim, int rot, int rank, int write, int dtype,
                                         cudaStream_t stream) {
  if (!q_src || q_ld < q_off + n_heads * (dim + rot)) return LLMIE_ERR_BAD_ARG;
  if (n_tokens < 0 || n_heads <= 0 || dim <= 0 || rot < 0 || rank <= 0 || ld <= 0 || q_off < 0 || page_size <= 0 ||
      max_pages <= 0 || rot_dims < 0 || rot_dims > rot || rot_dims % 2 || table_len <= 0)
    return LLMIE_ERR_BAD_ARG;
  if (write && (!cache || !norm_w || dkv_off < 0)) return LLMIE_ERR_BAD_ARG;
  if (dtype != LLMIE_F32 && dtype != LLMIE_BF16) return LLMIE_ERR_DTYPE;
  if (n_tokens == 0) return LLMIE_OK;
  if (dtype == LLMIE_F32)
    launch_k(latent_prepare_kernel<float>, dim3(n_tokens), dim3(128), 0, stream, (const float*)proj, ld, (const float*)q_src, q_ld, q_off, dkv_off, (float*)q_out, (float*)cache, norm_w, eps, table, table_len, rot_dims, tok_pos, tok_seq, seq_slot, block_table, max_pages, page_size, n_heads, dim, rot, rank, write);
  else
    launch_k(latent_prepare_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(128), 0, stream, (const __nv_bfloat16*)proj, ld, (const __nv_bfloat16*)q_src, q_ld, q_off, dkv_off, (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache, norm_w, eps, table, table_len, rot_dims, tok_pos, tok_seq, seq_slot, block_table, max_pages, page_size, n_heads, dim, rot, rank, write);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

extern "C" int llmie_latent_prepare(const void* proj, int ld, int q_off, int dkv_off, void* q_out, void* cache,
                                    const float* norm_w, float eps, const float* table, int table_len, int rot_dims,
                                    const int* tok_pos, const int* tok_seq, const int* seq_slot, const int* block_table,
                                    int max_pages, int page_size, int n_tokens, int n_heads, int dim, int rot, int rank,
                                    int write, int dtype, cudaStream_t stream) {
  return llmie_latent_prepare_from(proj, ld, proj, ld, q_off, dkv_off, q_out, cache, norm_w, eps, table, table_len,
                                   rot_dims, tok_pos, tok_seq, seq_slot, block_table, max_pages, page_size, n_tokens,
                                   n_heads, dim, rot, rank, write, dtype, stream);
}
