// Building blocks of the fp32 CUDA-core kernels: a register-tiled [64 x D] x [D x D]
// product against a matrix held in shared memory, and the SM count.
#pragma once
#include "tq_common.cuh"

namespace tq {

// Column permutation of the shared-memory copy of a transposed matrix: the thread that
// owns coordinates tx*8..tx*8+7 reads two float4 at [tx*4] and [D/2 + tx*4], which is
// bank-conflict free across tx.
template <int D>
__device__ __forceinline__ int perm_col(int j) {
  const int tx = j >> 3, e = j & 7;
  return (e >> 2) * (D / 2) + tx * 4 + (e & 3);
}

// Copy a row-major [D, D] fp32 matrix into shared memory as the right-hand side of
// tile_gemm.  TRANSPOSE: MT[i][perm(j)] = M[j][i] (for x @ M^T); else MT[i][perm(j)] = M[i][j].
template <int D, bool TRANSPOSE>
__device__ void load_matrix(const float* __restrict__ M, float* __restrict__ MT, int tid, int nthreads) {
  for (int e = tid; e < D * D; e += nthreads) {
    const int a = e / D, b = e % D;
    if (TRANSPOSE) MT[b * D + perm_col<D>(a)] = __ldg(M + e);
    else MT[a * D + perm_col<D>(b)] = __ldg(M + e);
  }
}

// acc[r][c] = sum_i X[row0+r][i] * MT[i][cols of this thread]
template <int D, int XS>
__device__ __forceinline__ void tile_gemm(const float* __restrict__ X, const float* __restrict__ MT,
                                          int row0, int tx, float (&acc)[4][8]) {
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[r][c] = 0.f;
#pragma unroll 2
  for (int i4 = 0; i4 < D; i4 += 4) {
    float4 xv[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) xv[r] = *reinterpret_cast<const float4*>(X + (row0 + r) * XS + i4);
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
      const float4 m0 = *reinterpret_cast<const float4*>(MT + (i4 + ii) * D + tx * 4);
      const float4 m1 = *reinterpret_cast<const float4*>(MT + (i4 + ii) * D + D / 2 + tx * 4);
      const float m[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float xs = ii == 0 ? xv[r].x : ii == 1 ? xv[r].y : ii == 2 ? xv[r].z : xv[r].w;
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[r][c] = fmaf(xs, m[c], acc[r][c]);
      }
    }
  }
}


inline int sm_count() {
  static int cached = 0;
  if (!cached) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev);
    if (cached <= 0) cached = 148;
  }
  return cached;
}

}  // namespace tq
