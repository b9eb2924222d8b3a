// Many small matrix products in one launch: C_g = A_g W_g^T for groups g that share a shape but not their
// weights. Two ways to say which rows belong to which group:
//
//   batched   every group has the same M rows; group g reads columns [g * a_gcs, g * a_gcs + K) of A's rows and
//             writes columns [g * c_gcs, g * c_gcs + N) of C's rows (the heads of an attention layer, each with a
//             matrix of its own); grid.z = groups.
//   routed    rows were sorted by group into tiles of BM positions (`tile_group[tile]` = the group of a tile, -1 =
//             unused tile; `a_rows[pos]` = the row of A at a sorted position, -1 = padding; `c_rows[pos]` = the row of
//             C it writes): the experts of a routed feed-forward. Positions without an indirection are their own row.
//
// W is [groups][N (or 2 N), K], K contiguous. With DUAL the weight of a group is [gate rows | up rows] and the result
// is act(A gate^T) * (A up^T). float32 inputs: one FMA per k in the order k = 0..K-1 whatever the tile or the batch (no
// tensor cores, no reduced precision), so a row's result does not depend on what else is in the launch. bfloat16 inputs:
// the tensor-core kernel further down, float32 accumulators.
#include "common.cuh"

namespace llmie {

struct GroupedArgs {
  const void* A; long long lda; long long a_gcs;
  const int* a_rows;
  const void* W; long long w_gs; long long ldw;
  void* C; long long ldc; long long c_gcs;
  const int* c_rows;
  const int* tile_group;
  int M, N, K, act;
};

constexpr int kGK = 16;

template <typename TA, typename TC, int BM, int BN, int TM, int TN, bool DUAL>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
grouped_gemm_kernel(const GroupedArgs p) {
  constexpr int kThreads = (BM / TM) * (BN / TN);
  __shared__ float As[kGK][BM + 4];
  __shared__ float Ws[DUAL ? 2 : 1][kGK][BN + 4];
  __shared__ int rowA[BM], rowC[BM];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int tile = blockIdx.y;
  int group = blockIdx.z;
  if (p.tile_group) {
    group = p.tile_group[tile];
    if (group < 0) return;
  }
  const int m0 = tile * BM, n0 = blockIdx.x * BN;
  for (int r = tid; r < BM; r += kThreads) {
    const int pos = m0 + r;
    int ra = -1, rc = -1;
    if (pos < p.M) {
      ra = p.a_rows ? p.a_rows[pos] : pos;
      rc = p.c_rows ? p.c_rows[pos] : pos;
      if (ra < 0 || rc < 0) ra = rc = -1;
    }
    rowA[r] = ra;
    rowC[r] = rc;
  }
  __syncthreads();
  const TA* A = reinterpret_cast<const TA*>(p.A) + (size_t)group * p.a_gcs;
  const TA* W = reinterpret_cast<const TA*>(p.W) + (size_t)group * p.w_gs;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  float acc[DUAL ? 2 : 1][TM][TN];
#pragma unroll
  for (int s = 0; s < (DUAL ? 2 : 1); ++s)
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[s][i][j] = 0.f;

  for (int k0 = 0; k0 < p.K; k0 += kGK) {
    for (int idx = tid; idx < BM * kGK; idx += kThreads) {
      const int r = idx / kGK, c = idx % kGK;
      const int ra = rowA[r], gk = k0 + c;
      As[c][r] = (ra >= 0 && gk < p.K) ? to_f32(A[(size_t)ra * p.lda + gk]) : 0.f;
    }
    for (int idx = tid; idx < BN * kGK; idx += kThreads) {
      const int r = idx / kGK, c = idx % kGK;
      const int gn = n0 + r, gk = k0 + c;
      const bool ok = gn < p.N && gk < p.K;
      Ws[0][c][r] = ok ? to_f32(W[(size_t)gn * p.ldw + gk]) : 0.f;
      if (DUAL) Ws[DUAL ? 1 : 0][c][r] = ok ? to_f32(W[(size_t)(gn + p.N) * p.ldw + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kGK; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int s = 0; s < (DUAL ? 2 : 1); ++s) {
#pragma unroll
        for (int j = 0; j < TN; ++j) w[j] = Ws[s][kk][tx * TN + j];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) acc[s][i][j] = fmaf(a[i], w[j], acc[s][i][j]);
      }
    }
    __syncthreads();
  }
  TC* C = reinterpret_cast<TC*>(p.C) + (size_t)group * p.c_gcs;
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int rc = rowC[ty * TM + i];
    if (rc < 0) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= p.N) continue;
      float v = acc[0][i][j];
      if (DUAL) {
        // the gate is rounded to the activation type before the activation, as a separate product would leave it
        const float g = to_f32(from_f32<TC>(v)), u = to_f32(from_f32<TC>(acc[DUAL ? 1 : 0][i][j]));
        v = apply_act(g, p.act) * u;
      } else if (p.act) {
        v = apply_act(to_f32(from_f32<TC>(v)), p.act);      // a single product with its activation
      }
      C[(size_t)rc * p.ldc + gn] = from_f32<TC>(v);
    }
  }
}

// ------------------------------------------------------------------------------------------
// The same products for bfloat16 inputs on the tensor cores (mma.sync m16n8k16, float32 accumulators): tiles of
// BM x 64 outputs, four warps. With BM = 64 a warp owns 16 rows and all 64 columns; with BM = 16 (few rows a group:
// one-token steps, where the weights are what is streamed) the warps share out the columns and the K step is longer.
// A row's sums depend on that row and the weights alone (the rows of an mma are independent), so here too a result
// does not depend on what else is in the launch. `vec`: K, the leading dimensions and the group strides are multiples
// of 8 elements and the bases 16-byte aligned, so tiles are fetched 16 bytes at a time; otherwise element by element.
__device__ __forceinline__ void gg_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename TC, int BM, int BK, bool DUAL>
__global__ void __launch_bounds__(128)
grouped_gemm_mma_kernel(const GroupedArgs p, const int vec) {
  constexpr int BN = 64, PITCH = BK + 8, NW = DUAL ? 2 : 1, CH = BK / 8;
  constexpr int NT = BM == 64 ? 8 : 2;                 // n-tiles of 8 columns a warp owns
  __shared__ __align__(16) __nv_bfloat16 As[BM][PITCH];
  __shared__ __align__(16) __nv_bfloat16 Ws[NW][BN][PITCH];
  __shared__ int rowA[BM], rowC[BM];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int tile = blockIdx.y;
  int group = blockIdx.z;
  if (p.tile_group) {
    group = p.tile_group[tile];
    if (group < 0) return;
  }
  const int m0 = tile * BM, n0 = blockIdx.x * BN;
  for (int r = tid; r < BM; r += 128) {
    const int pos = m0 + r;
    int ra = -1, rc = -1;
    if (pos < p.M) {
      ra = p.a_rows ? p.a_rows[pos] : pos;
      rc = p.c_rows ? p.c_rows[pos] : pos;
      if (ra < 0 || rc < 0) ra = rc = -1;
    }
    rowA[r] = ra;
    rowC[r] = rc;
  }
  __syncthreads();
  const __nv_bfloat16* A = reinterpret_cast<const __nv_bfloat16*>(p.A) + (size_t)group * p.a_gcs;
  const __nv_bfloat16* W = reinterpret_cast<const __nv_bfloat16*>(p.W) + (size_t)group * p.w_gs;
  const int row0 = BM == 64 ? warp * 16 : 0;
  const int nt0 = BM == 64 ? 0 : warp * 2;
  float acc[NW][NT][4];
#pragma unroll
  for (int s = 0; s < NW; ++s)
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[s][i][0] = acc[s][i][1] = acc[s][i][2] = acc[s][i][3] = 0.f;

  // eight consecutive elements of a row from column gk on (zeros beyond K or for a row that is not there)
  auto fetch = [&](const __nv_bfloat16* row, bool there, int gk) -> uint4 {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (!there || gk >= p.K) return v;
    if (vec) return *reinterpret_cast<const uint4*>(row + gk);
    __nv_bfloat16 e[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = gk + i < p.K ? row[gk + i] : __float2bfloat16_rn(0.f);
    return *reinterpret_cast<const uint4*>(e);
  };

  // The next K step's pieces are requested into registers before this step's products, so that the loads are in flight
  // while the tensor cores work: with few rows a group the weights' stream is all there is to wait for.
  constexpr int A_PER = BM * CH / 128 > 0 ? BM * CH / 128 : 1, W_PER = BN * CH / 128;
  static_assert((BM * CH) % 128 == 0 || BM * CH < 128, "whole rounds of the block's threads");
  uint4 ra[A_PER], rw[NW][W_PER];
  auto request = [&](int k0) {
#pragma unroll
    for (int j = 0; j < A_PER; ++j) {
      const int c = tid + j * 128;
      if (c < BM * CH) {
        const int r = c / CH, kc = (c % CH) * 8;
        const int row = rowA[r];
        ra[j] = fetch(A + (size_t)(row < 0 ? 0 : row) * p.lda, row >= 0, k0 + kc);
      }
    }
#pragma unroll
    for (int j = 0; j < W_PER; ++j) {
      const int c = tid + j * 128;
      const int r = c / CH, kc = (c % CH) * 8;
      const int gn = n0 + r;
      rw[0][j] = fetch(W + (size_t)gn * p.ldw, gn < p.N, k0 + kc);
      if (DUAL) rw[NW - 1][j] = fetch(W + (size_t)(gn + p.N) * p.ldw, gn < p.N, k0 + kc);
    }
  };
  request(0);
  for (int k0 = 0; k0 < p.K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < A_PER; ++j) {
      const int c = tid + j * 128;
      if (c < BM * CH) *reinterpret_cast<uint4*>(&As[c / CH][(c % CH) * 8]) = ra[j];
    }
#pragma unroll
    for (int j = 0; j < W_PER; ++j) {
      const int c = tid + j * 128;
      *reinterpret_cast<uint4*>(&Ws[0][c / CH][(c % CH) * 8]) = rw[0][j];
      if (DUAL) *reinterpret_cast<uint4*>(&Ws[NW - 1][c / CH][(c % CH) * 8]) = rw[NW - 1][j];
    }
    __syncthreads();
    if (k0 + BK < p.K) request(k0 + BK);
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      const unsigned a0 = *reinterpret_cast<const unsigned*>(&As[row0 + g][kk + 2 * t]);
      const unsigned a1 = *reinterpret_cast<const unsigned*>(&As[row0 + g + 8][kk + 2 * t]);
      const unsigned a2 = *reinterpret_cast<const unsigned*>(&As[row0 + g][kk + 2 * t + 8]);
      const unsigned a3 = *reinterpret_cast<const unsigned*>(&As[row0 + g + 8][kk + 2 * t + 8]);
#pragma unroll
      for (int s = 0; s < NW; ++s)
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          const unsigned b0 = *reinterpret_cast<const unsigned*>(&Ws[s][(nt0 + i) * 8 + g][kk + 2 * t]);
          const unsigned b1 = *reinterpret_cast<const unsigned*>(&Ws[s][(nt0 + i) * 8 + g][kk + 2 * t + 8]);
          gg_mma(acc[s][i], a0, a1, a2, a3, b0, b1);
        }
    }
    __syncthreads();
  }
  TC* C = reinterpret_cast<TC*>(p.C) + (size_t)group * p.c_gcs;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int rc = rowC[row0 + g + 8 * half];
    if (rc < 0) continue;
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int gn = n0 + (nt0 + i) * 8 + 2 * t + e;
        if (gn >= p.N) continue;
        float v = acc[0][i][2 * half + e];
        if (DUAL) {
          const float gt = to_f32(from_f32<TC>(v)), up = to_f32(from_f32<TC>(acc[NW - 1][i][2 * half + e]));
          v = apply_act(gt, p.act) * up;
        } else if (p.act) {
          v = apply_act(to_f32(from_f32<TC>(v)), p.act);
        }
        C[(size_t)rc * p.ldc + gn] = from_f32<TC>(v);
      }
  }
}

template <typename TC, bool DUAL>
static int launch_grouped_mma(const GroupedArgs& p, int n_tiles, int groups_z, bool small, int vec, cudaStream_t stream) {
  dim3 grid((p.N + 63) / 64, n_tiles, groups_z);
  if (grid.y > 65535 || grid.z > 65535) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (small) launch_k(grouped_gemm_mma_kernel<TC, 16, 64, DUAL>, grid, dim3(128), 0, stream, p, vec);
  else launch_k(grouped_gemm_mma_kernel<TC, 64, 32, DUAL>, grid, dim3(128), 0, stream, p, vec);
  return LLMIE_OK;
}

template <typename TA, typename TC, bool DUAL>
static int launch_grouped(const GroupedArgs& p, int n_tiles_small, int n_tiles_big, int groups_z, bool small,
                          cudaStream_t stream) {
  if (small) {
    dim3 grid((p.N + 31) / 32, n_tiles_small, groups_z);
    if (grid.y > 65535 || grid.z > 65535) return LLMIE_ERR_UNSUPPORTED_SIZE;
    launch_k(grouped_gemm_kernel<TA, TC, 16, 32, 2, 2, DUAL>, grid, dim3(128), 0, stream, p);
  } else {
    dim3 grid((p.N + 63) / 64, n_tiles_big, groups_z);
    if (grid.y > 65535 || grid.z > 65535) return LLMIE_ERR_UNSUPPORTED_SIZE;
    launch_k(grouped_gemm_kernel<TA, TC, 64, 64, 4, 4, DUAL>, grid, dim3(256), 0, stream, p);
  }
  return LLMIE_OK;
}

}  // namespace llmie

using namespace llmie;

// Rows per tile of the two forms; the sort that prepares a routed call must use the same number.
extern "C" int llmie_grouped_gemm_tile_rows(int small) { return small ? 16 : 64; }

// A, W of in_dtype; C of out_dtype. `groups` > 0 with tile_group == null: the batched form over M rows. tile_group !=
// null: the routed form over `n_tiles` tiles of sorted positions (M = number of positions, padding included).
// `small` picks tiles of 16 rows (few rows per group) instead of 64. dual: W holds [gate | up], act is applied to the
// gate; without dual a non-zero act is applied to the product itself.
extern "C" int llmie_grouped_gemm_nt(const void* A, long long lda, long long a_gcs, const int* a_rows, const void* W,
                                     long long w_gs, long long ldw, void* C, long long ldc, long long c_gcs,
                                     const int* c_rows, const int* tile_group, int n_tiles, int groups, int M, int N,
                                     int K, int dual, int act, int small, int in_dtype, int out_dtype,
                                     cudaStream_t stream) {
  if (!A || !W || !C || M < 0 || N <= 0 || K <= 0 || lda < 0 || ldw < K || ldc < 0 || act < 0 || act > 4)
    return LLMIE_ERR_BAD_ARG;
  if (!tile_group && groups <= 0) return LLMIE_ERR_BAD_ARG;
  if (tile_group && n_tiles < 0) return LLMIE_ERR_BAD_ARG;
  if ((in_dtype != LLMIE_F32 && in_dtype != LLMIE_BF16) || (out_dtype != LLMIE_F32 && out_dtype != LLMIE_BF16))
    return LLMIE_ERR_DTYPE;
  if (in_dtype == LLMIE_F32 && out_dtype != LLMIE_F32) return LLMIE_ERR_DTYPE;
  if (M == 0 || (tile_group && n_tiles == 0)) return LLMIE_OK;
  GroupedArgs p{A, lda, a_gcs, a_rows, W, w_gs, ldw, C, ldc, c_gcs, c_rows, tile_group, M, N, K, act};
  const int bm = small ? 16 : 64;
  const int tiles = tile_group ? n_tiles : (M + bm - 1) / bm;
  const int gz = tile_group ? 1 : groups;
  int rc;
  if (in_dtype == LLMIE_F32)
    rc = dual ? launch_grouped<float, float, true>(p, tiles, tiles, gz, small, stream)
              : launch_grouped<float, float, false>(p, tiles, tiles, gz, small, stream);
  else {
    const int vec = K % 8 == 0 && lda % 8 == 0 && a_gcs % 8 == 0 && ldw % 8 == 0 && w_gs % 8 == 0 && aligned16(A) &&
                    aligned16(W);
    if (out_dtype == LLMIE_F32)
      rc = dual ? launch_grouped_mma<float, true>(p, tiles, gz, small, vec, stream)
                : launch_grouped_mma<float, false>(p, tiles, gz, small, vec, stream);
    else
      rc = dual ? launch_grouped_mma<__nv_bfloat16, true>(p, tiles, gz, small, vec, stream)
                : launch_grouped_mma<__nv_bfloat16, false>(p, tiles, gz, small, vec, stream);
  }
  if (rc != LLMIE_OK) return rc;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}
