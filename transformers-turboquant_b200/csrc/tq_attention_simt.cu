// fp32 CUDA-core kernels of the attention side (TQ_MODE_FP32, the parity mode):
//   * query preparation  q_cat = [ q Pi^T | coeff * (q Pi^T) S_eff^T ]   (fp32 scratch)
//   * estimator scores from packed keys (full fp32 matrix, small shapes)
//   * fused causal attention from packed keys and values (flash-style online softmax,
//     P V accumulated in the values' rotated coordinates, one back-rotation per tile)
//   * value decompression
// Follows compressors.py:163-224, :296-317, kernels/attention.py:380-461 and the adapter
// core families/llama.py:100-114 of the reference.
#include <math.h>

#include "tq_common.cuh"
#include "tq_simt.cuh"
#include "tq_attention.cuh"

namespace tq {

constexpr int kRows = 64;  // query rows and keys per tile

__device__ __forceinline__ void store8(void* base, int dtype, int64_t off, const float (&v)[8]) {
  if (dtype == TQ_F32) {
    float4* p = reinterpret_cast<float4*>(static_cast<float*>(base) + off);
    p[0] = make_float4(v[0], v[1], v[2], v[3]);
    p[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else if (dtype == TQ_BF16) {
    __nv_bfloat162 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(base) + off) = *reinterpret_cast<uint4*>(h);
  } else {
    __half2 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(static_cast<__half*>(base) + off) = *reinterpret_cast<uint4*>(h);
  }
}

// ---- query preparation ---------------------------------------------------------------

struct QPrepArgs {
  const void* q;
  int64_t n_q, Hq, Sq;
  int64_t stride_b, stride_h, stride_s;
  const float* Pi;
  const float* S_eff;
  float coeff;
  float* q_cat;  // [n_q, 2D]
  int num_tiles;
};

template <typename T, int D>
__global__ void __launch_bounds__(16 * (D / 8)) qprep_simt_kernel(const QPrepArgs a) {
  constexpr int TX = D / 8, NT = 16 * TX, XS = D + 4;
  extern __shared__ __align__(16) float smem[];
  float* PiT = smem;
  float* SeT = PiT + D * D;
  float* X = SeT + D * D;
  const int tid = threadIdx.x, tx = tid % TX, ty = tid / TX, row0 = ty * 4;
  load_matrix<D, true>(a.Pi, PiT, tid, NT);
  load_matrix<D, true>(a.S_eff, SeT, tid, NT);
  const T* src = static_cast<const T*>(a.q);
  const int64_t HS = a.Hq * a.Sq;
  for (int tile = blockIdx.x; tile < a.num_tiles; tile += gridDim.x) {
    const int64_t base = static_cast<int64_t>(tile) * kRows;
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int64_t n = base + row0 + r;
      float v[8];
      if (n < a.n_q) {
        const int64_t b = n / HS, rem = n % HS;
        load8<T>(src + b * a.stride_b + (rem / a.Sq) * a.stride_h + (rem % a.Sq) * a.stride_s + tx * 8, v);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = 0.f;
      }
      float* xr = X + (row0 + r) * XS + tx * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) xr[e] = v[e];
    }
    __syncthreads();
    float y[4][8];
    tile_gemm<D, XS>(X, PiT, row0, tx, y);
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int64_t n = base + row0 + r;
      float* xr = X + (row0 + r) * XS + tx * 8;
#pragma unroll
      for (int c = 0; c < 8; ++c) xr[c] = y[r][c];
      if (n < a.n_q) store8(a.q_cat, TQ_F32, n * 2 * D + tx * 8, y[r]);
    }
    __syncthreads();
    tile_gemm<D, XS>(X, SeT, row0, tx, y);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int64_t n = base + row0 + r;
#pragma unroll
      for (int c = 0; c < 8; ++c) y[r][c] *= a.coeff;
      if (n < a.n_q) store8(a.q_cat, TQ_F32, n * 2 * D + D + tx * 8, y[r]);
    }
  }
}

// ---- tile decode helpers -------------------------------------------------------------

// Decode keys [k0, k0+64) of one head into Ks[j][0:D] = C[idx], Ks[j][D:2D] = +-1, and
// their norms into kn[j] (vector norm) and krn[j] (residual norm).  Keys past `Sk` decode
// to zeros.
template <int D, int IB>
__device__ __forceinline__ void decode_key_tile(const uint8_t* __restrict__ idx, const uint8_t* __restrict__ sgn,
                                                const uint16_t* __restrict__ vn, const uint16_t* __restrict__ rn,
                                                int64_t head_base, int k0, int Sk, const float* __restrict__ cen,
                                                float* Ks, float* kn, float* krn, int tid, int nthreads) {
  constexpr int KS = 2 * D + 4, G = D / 8;
  for (int e = tid; e < kRows * G; e += nthreads) {
    const int j = e / G, g = e % G;
    float* dst = Ks + j * KS + g * 8;
    if (k0 + j < Sk) {
      const int64_t n = head_base + k0 + j;
      const uint64_t w = load_fields8<IB>(idx + n * (D * IB / 8) + g * IB);
      const unsigned sb = sgn[n * G + g];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        dst[c] = cen[(w >> (c * IB)) & ((1u << IB) - 1)];
        dst[D + c] = ((sb >> c) & 1u) ? 1.f : -1.f;
      }
    } else {
#pragma unroll
      for (int c = 0; c < 8; ++c) { dst[c] = 0.f; dst[D + c] = 0.f; }
    }
  }
  for (int j = tid; j < kRows; j += nthreads) {
    const bool ok = k0 + j < Sk;
    kn[j] = ok ? fp16_value(vn[head_base + k0 + j]) : 0.f;
    krn[j] = ok ? fp16_value(rn[head_base + k0 + j]) : 0.f;
  }
}

// s[r][c] = kn * <q_rot, C[idx]> + krn * <q_s, +-1> for rows row0+r, keys tx + 16c.
template <int D>
__device__ __forceinline__ void score_tile(const float* __restrict__ Qs, const float* __restrict__ Ks,
                                           const float* __restrict__ kn, const float* __restrict__ krn,
                                           int row0, int tx, float (&s)[4][4]) {
  constexpr int KS = 2 * D + 4;
  float a1[4][4], a2[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) a1[r][c] = a2[r][c] = 0.f;
#pragma unroll 2
  for (int i = 0; i < D; i += 4) {
    float4 q1[4], q2[4], k1[4], k2[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      q1[r] = *reinterpret_cast<const float4*>(Qs + (row0 + r) * KS + i);
      q2[r] = *reinterpret_cast<const float4*>(Qs + (row0 + r) * KS + D + i);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      k1[c] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * c) * KS + i);
      k2[c] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * c) * KS + D + i);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        a1[r][c] = fmaf(q1[r].x, k1[c].x, a1[r][c]);
        a1[r][c] = fmaf(q1[r].y, k1[c].y, a1[r][c]);
        a1[r][c] = fmaf(q1[r].z, k1[c].z, a1[r][c]);
        a1[r][c] = fmaf(q1[r].w, k1[c].w, a1[r][c]);
        a2[r][c] = fmaf(q2[r].x, k2[c].x, a2[r][c]);
        a2[r][c] = fmaf(q2[r].y, k2[c].y, a2[r][c]);
        a2[r][c] = fmaf(q2[r].z, k2[c].z, a2[r][c]);
        a2[r][c] = fmaf(q2[r].w, k2[c].w, a2[r][c]);
      }
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const float n1 = kn[tx + 16 * c], n2 = krn[tx + 16 * c];
#pragma unroll
    for (int r = 0; r < 4; ++r) s[r][c] = fmaf(n1, a1[r][c], n2 * a2[r][c]);
  }
}

template <int D>
__device__ __forceinline__ void load_q_tile(const float* __restrict__ q_cat, int64_t q_base, int q0, int Sq,
                                            float* Qs, int tid, int nthreads) {
  constexpr int KS = 2 * D + 4, C4 = 2 * D / 4;
  for (int e = tid; e < kRows * C4; e += nthreads) {
    const int i = e / C4, c = e % C4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (q0 + i < Sq) v = *reinterpret_cast<const float4*>(q_cat + (q_base + q0 + i) * 2 * D + c * 4);
    *reinterpret_cast<float4*>(Qs + i * KS + c * 4) = v;
  }
}

// ---- scores ------------------------------------------------------------------------------

struct ScoreArgs {
  const float* q_cat;
  int64_t Hq, Sq, Hkv, Sk;
  const uint8_t* key_idx;
  const uint8_t* key_sgn;
  const uint16_t* key_vn;
  const uint16_t* key_rn;
  const float* cen_k;
  float* scores;
};

template <int D, int IB>
__global__ void __launch_bounds__(256) scores_simt_kernel(const ScoreArgs a) {
  constexpr int KS = 2 * D + 4;
  extern __shared__ __align__(16) float smem[];
  float* Qs = smem;
  float* Ks = Qs + kRows * KS;
  float* kn = Ks + kRows * KS;
  float* krn = kn + kRows;
  __shared__ float cen[1 << IB];
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16, row0 = ty * 4;
  if (tid < (1 << IB)) cen[tid] = a.cen_k[tid];
  const int64_t bh = blockIdx.z;
  const int64_t b = bh / a.Hq, h = bh % a.Hq;
  const int64_t hk = h / (a.Hq / a.Hkv);
  const int q0 = blockIdx.y * kRows, k0 = blockIdx.x * kRows;
  __syncthreads();
  load_q_tile<D>(a.q_cat, bh * a.Sq, q0, (int)a.Sq, Qs, tid, 256);
  decode_key_tile<D, IB>(a.key_idx, a.key_sgn, a.key_vn, a.key_rn, (b * a.Hkv + hk) * a.Sk, k0, (int)a.Sk,
                         cen, Ks, kn, krn, tid, 256);
  __syncthreads();
  float s[4][4];
  score_tile<D>(Qs, Ks, kn, krn, row0, tx, s);
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int i = q0 + row0 + r, k = k0 + tx + 16 * c;
      if (i < a.Sq && k < a.Sk) a.scores[(bh * a.Sq + i) * a.Sk + k] = s[r][c];
    }
}

// ---- fused attention -----------------------------------------------------------------


template <int D, int KB, int VB>
__global__ void __launch_bounds__(256) attention_simt_kernel(const AttnArgs a) {
  constexpr int KS = 2 * D + 4, VS = D + 4, PS = kRows + 4, G = D / 8;
  constexpr int NC = D / 16;  // output coordinates per thread in the P V product
  extern __shared__ __align__(16) float smem[];
  float* Qs = smem;                    // [64][KS]; reused for Pi_v in the epilogue
  float* Ks = Qs + kRows * KS;         // [64][KS]; reused for the O tile in the epilogue
  float* Vs = Ks + kRows * KS;         // [64][VS]  n_v * C_v[idx]
  float* Ps = Vs + kRows * VS;         // [64][PS]
  float* kn = Ps + kRows * PS;
  float* krn = kn + kRows;
  __shared__ float cen_k[1 << KB];
  __shared__ float cen_v[1 << VB];
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16, row0 = ty * 4;
  if (tid < (1 << KB)) cen_k[tid] = a.cen_k[tid];
  if (tid < (1 << VB)) cen_v[tid] = a.cen_v[tid];
  const int64_t b = blockIdx.z, h = blockIdx.y;
  const int64_t bh = b * a.Hq + h;
  const int64_t kv_base = (b * a.Hkv + h / (a.Hq / a.Hkv)) * a.Sk;
  const int q0 = blockIdx.x * kRows;
  const int shift = (int)(a.Sk - a.Sq);  // query i sees keys <= i + shift when causal
  __syncthreads();
  load_q_tile<D>(static_cast<const float*>(a.q_cat), bh * a.Sq, q0, (int)a.Sq, Qs, tid, 256);

  float m_run[4], l_run[4], o[4][NC];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    m_run[r] = -INFINITY;
    l_run[r] = 0.f;
#pragma unroll
    for (int c = 0; c < NC; ++c) o[r][c] = 0.f;
  }
  int k_end = (int)a.Sk;
  if (a.causal) {
    const int last = min(q0 + kRows - 1, (int)a.Sq - 1) + shift;
    k_end = min(k_end, last + 1);
  }
  for (int k0 = 0; k0 < k_end; k0 += kRows) {
    __syncthreads();  // previous tile fully consumed
    decode_key_tile<D, KB>(a.key_idx, a.key_sgn, a.key_vn, a.key_rn, kv_base, k0, (int)a.Sk, cen_k, Ks, kn,
                           krn, tid, 256);
    for (int e = tid; e < kRows * G; e += 256) {
      const int j = e / G, g = e % G;
      float* dst = Vs + j * VS + g * 8;
      if (k0 + j < a.Sk) {
        const int64_t n = kv_base + k0 + j;
        const uint64_t w = load_fields8<VB>(a.val_idx + n * (D * VB / 8) + g * VB);
        const float nv = fp16_value(a.val_vn[n]);
#pragma unroll
        for (int c = 0; c < 8; ++c) dst[c] = nv * cen_v[(w >> (c * VB)) & ((1u << VB) - 1)];
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) dst[c] = 0.f;
      }
    }
    __syncthreads();
    float s[4][4];
    score_tile<D>(Qs, Ks, kn, krn, row0, tx, s);
    // ---- online softmax --------------------------------------------------------------
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = q0 + row0 + r;
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int k = k0 + tx + 16 * c;
        float t = s[r][c] * a.sm_scale;
        if (a.mask != nullptr && i < a.Sq && k < a.Sk)
          t += a.mask[b * a.mask_stride_b + (int64_t)i * a.mask_stride_q + k];
        if (k >= a.Sk || (a.causal && k > i + shift)) t = -INFINITY;
        s[r][c] = t;
        mx = fmaxf(mx, t);
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float m_new = fmaxf(m_run[r], mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = (m_run[r] == -INFINITY) ? 0.f : __expf(m_run[r] - m_use);
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float p = __expf(s[r][c] - m_use);
        Ps[(row0 + r) * PS + tx + 16 * c] = p;
        sum += p;
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      l_run[r] = l_run[r] * alpha + sum;
      m_run[r] = m_new;
#pragma unroll
      for (int c = 0; c < NC; ++c) o[r][c] *= alpha;
    }
    __syncthreads();
    // ---- O += P V_hat (rotated coordinates) ----------------------------------------------
#pragma unroll 2
    for (int j = 0; j < kRows; j += 4) {
      float4 p4[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) p4[r] = *reinterpret_cast<const float4*>(Ps + (row0 + r) * PS + j);
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        float v[NC];
        const float4 v0 = *reinterpret_cast<const float4*>(Vs + (j + jj) * VS + tx * 4);
        v[0] = v0.x; v[1] = v0.y; v[2] = v0.z; v[3] = v0.w;
        if (NC == 8) {
          const float4 v1 = *reinterpret_cast<const float4*>(Vs + (j + jj) * VS + D / 2 + tx * 4);
          v[NC - 4] = v1.x; v[NC - 3] = v1.y; v[NC - 2] = v1.z; v[NC - 1] = v1.w;
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float pv = jj == 0 ? p4[r].x : jj == 1 ? p4[r].y : jj == 2 ? p4[r].z : p4[r].w;
#pragma unroll
          for (int c = 0; c < NC; ++c) o[r][c] = fmaf(pv, v[c], o[r][c]);
        }
      }
    }
  }
  // ---- epilogue: normalise, rotate back by Pi_v, store ----------------------------------
  __syncthreads();
  float* Os = Ks;  // [64][VS]
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) Os[(row0 + r) * VS + tx * 4 + c] = o[r][c] * inv;
    if (NC == 8) {
#pragma unroll
      for (int c = 0; c < 4; ++c) Os[(row0 + r) * VS + D / 2 + tx * 4 + c] = o[r][NC - 4 + c] * inv;
    }
  }
  load_matrix<D, false>(a.Pi_v, Qs, tid, 256);
  __syncthreads();
  if (D == 128 || tx < 8) {  // tile_gemm maps 8 consecutive outputs to tx < D/8
    float y[4][8];
    tile_gemm<D, VS>(Os, Qs, row0, tx, y);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = q0 + row0 + r;
      if (i < a.Sq)
        store8(a.out, a.out_dtype, b * a.o_stride_b + h * a.o_stride_h + (int64_t)i * a.o_stride_s + tx * 8, y[r]);
    }
  }
}

// ---- value decompression ---------------------------------------------------------------

template <int D, int VB>
__global__ void __launch_bounds__(16 * (D / 8)) decompress_simt_kernel(const uint8_t* __restrict__ idx,
                                                                      const uint16_t* __restrict__ vn, int64_t n_vec,
                                                                      const float* __restrict__ Pi,
                                                                      const float* __restrict__ cen_g,
                                                                      float* __restrict__ out, int num_tiles) {
  constexpr int TX = D / 8, NT = 16 * TX, XS = D + 4;
  extern __shared__ __align__(16) float smem[];
  float* M = smem;
  float* X = M + D * D;
  __shared__ float cen[1 << VB];
  const int tid = threadIdx.x, tx = tid % TX, ty = tid / TX, row0 = ty * 4;
  if (tid < (1 << VB)) cen[tid] = cen_g[tid];
  load_matrix<D, false>(Pi, M, tid, NT);
  for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
    const int64_t base = static_cast<int64_t>(tile) * kRows;
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int64_t n = base + row0 + r;
      float* xr = X + (row0 + r) * XS + tx * 8;
      uint64_t w = 0;
      if (n < n_vec) w = load_fields8<VB>(idx + n * (D * VB / 8) + tx * VB);
#pragma unroll
      for (int c = 0; c < 8; ++c) xr[c] = (n < n_vec) ? cen[(w >> (c * VB)) & ((1u << VB) - 1)] : 0.f;
    }
    __syncthreads();
    float y[4][8];
    tile_gemm<D, XS>(X, M, row0, tx, y);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int64_t n = base + row0 + r;
      if (n < n_vec) {
        const float nv = fp16_value(vn[n]);
#pragma unroll
        for (int c = 0; c < 8; ++c) y[r][c] *= nv;
        store8(out, TQ_F32, n * D + tx * 8, y[r]);
      }
    }
  }
}

// ---- host side ---------------------------------------------------------------------------

template <typename T, int D>
static int launch_qprep(const QPrepArgs& a, cudaStream_t stream) {
  constexpr size_t smem = sizeof(float) * (2 * D * D + kRows * (D + 4));
  auto kern = qprep_simt_kernel<T, D>;
  TQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int grid = sm_count() * (smem > 110 * 1024 ? 1 : 2);
  if (grid > a.num_tiles) grid = a.num_tiles;
  ProfScope prof(kProfPrepareQueries, stream);
  kern<<<grid, 16 * (D / 8), smem, stream>>>(a);
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
}

int qprep_fp32(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d, int64_t sb, int64_t sh,
               int64_t ss, const float* Pi, const float* S_eff, float* q_cat, cudaStream_t stream) {
  const int64_t n = B * Hq * Sq;
  QPrepArgs a{q, n, Hq, Sq, sb, sh, ss, Pi, S_eff, sqrtf(1.5707963267948966f) / (float)d, q_cat,
              (int)((n + kRows - 1) / kRows)};
#define TQ_CASE(TYPE) return d == 128 ? launch_qprep<TYPE, 128>(a, stream) : launch_qprep<TYPE, 64>(a, stream);
  if (dtype == TQ_F32) { TQ_CASE(float) }
  if (dtype == TQ_BF16) { TQ_CASE(__nv_bfloat16) }
  TQ_CASE(__half)
#undef TQ_CASE
}

template <int D, int IB>
static int launch_scores(const ScoreArgs& a, int64_t B, cudaStream_t stream) {
  constexpr size_t smem = sizeof(float) * (2 * kRows * (2 * D + 4) + 2 * kRows);
  auto kern = scores_simt_kernel<D, IB>;
  TQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)((a.Sk + kRows - 1) / kRows), (unsigned)((a.Sq + kRows - 1) / kRows), (unsigned)(B * a.Hq));
  kern<<<grid, 256, smem, stream>>>(a);
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
}

int scores_fp32(const ScoreArgs& a, int64_t B, int d, int bits, cudaStream_t stream) {
  const int ib = bits - 1;
  if (d == 128) {
    if (ib == 1) return launch_scores<128, 1>(a, B, stream);
    if (ib == 2) return launch_scores<128, 2>(a, B, stream);
    return launch_scores<128, 3>(a, B, stream);
  }
  if (ib == 1) return launch_scores<64, 1>(a, B, stream);
  if (ib == 2) return launch_scores<64, 2>(a, B, stream);
  return launch_scores<64, 3>(a, B, stream);
}

template <int D, int BITS>
static int launch_attention(const AttnArgs& a, int64_t B, cudaStream_t stream) {
  constexpr size_t smem =
      sizeof(float) * (2 * kRows * (2 * D + 4) + kRows * (D + 4) + kRows * (kRows + 4) + 2 * kRows);
  auto kern = attention_simt_kernel<D, BITS - 1, BITS>;
  TQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)((a.Sq + kRows - 1) / kRows), (unsigned)a.Hq, (unsigned)B);
  ProfScope prof(kProfAttention, stream);
  kern<<<grid, 256, smem, stream>>>(a);
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
}

int attention_fp32(const AttnArgs& a, int64_t B, int d, int bits, cudaStream_t stream) {
  if (d == 128) {
    if (bits == 2) return launch_attention<128, 2>(a, B, stream);
    if (bits == 3) return launch_attention<128, 3>(a, B, stream);
    return launch_attention<128, 4>(a, B, stream);
  }
  if (bits == 2) return launch_attention<64, 2>(a, B, stream);
  if (bits == 3) return launch_attention<64, 3>(a, B, stream);
  return launch_attention<64, 4>(a, B, stream);
}

template <int D, int VB>
static int launch_decompress(const uint8_t* idx, const uint16_t* vn, int64_t n, const float* Pi, const float* cen,
                             float* out, cudaStream_t stream) {
  constexpr size_t smem = sizeof(float) * (D * D + kRows * (D + 4));
  auto kern = decompress_simt_kernel<D, VB>;
  TQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int tiles = (int)((n + kRows - 1) / kRows);
  int grid = sm_count() * 2;
  if (grid > tiles) grid = tiles;
  kern<<<grid, 16 * (D / 8), smem, stream>>>(idx, vn, n, Pi, cen, out, tiles);
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
}

}  // namespace tq

using namespace tq;


static int check_attention_common(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d, int64_t sb,
                                  int64_t sh, int64_t ss, int64_t Hkv, int64_t Sk, int bits, int mode) {
  TQ_REQUIRE(dtype == TQ_F32 || dtype == TQ_BF16 || dtype == TQ_F16, "unknown dtype %d", dtype);
  TQ_REQUIRE(mode == TQ_MODE_FP32 || mode == TQ_MODE_BF16, "unknown mode %d", mode);
  TQ_REQUIRE(valid_head_dim(d), "head_dim %d unsupported (64 or 128)", d);
  TQ_REQUIRE(valid_bits(bits), "bits %d unsupported (2, 3 or 4)", bits);
  TQ_REQUIRE(B >= 0 && Hq >= 0 && Sq >= 0 && Hkv >= 0 && Sk >= 0, "negative size");
  TQ_REQUIRE(Hkv > 0 ? (Hq % Hkv == 0) : Hq == 0, "query heads %lld not a multiple of key heads %lld",
             (long long)Hq, (long long)Hkv);
  TQ_REQUIRE(Sq < (1 << 30) && Sk < (1 << 30) && B * Hq < (1 << 30), "sequence or batch too large");
  if (B * Hq * Sq == 0) return TQ_OK;
  TQ_REQUIRE(q != nullptr && aligned16(q), "q must be a 16-byte aligned device pointer");
  const int64_t al = 16 / elem_size(dtype);
  TQ_REQUIRE(sb % al == 0 && sh % al == 0 && ss % al == 0, "q strides must keep every row 16-byte aligned");
  return TQ_OK;
}

extern "C" {

size_t tq_attention_workspace_bytes(int64_t B, int64_t Hq, int64_t Sq, int d, int mode) {
  if (B <= 0 || Hq <= 0 || Sq <= 0 || d <= 0) return 0;
  const size_t n = (size_t)B * Hq * Sq;
  // fp32 mode: q_cat fp32 [n, 2d].  The score matrix always uses the fp32 layout, so the
  // bf16 figure is the larger of the two.
  const size_t f32 = (n * 2 * d * 4 + 255) & ~(size_t)255;
  if (mode == TQ_MODE_FP32) return f32;
  const size_t b16 = workspace_bytes_bf16(B * Hq, Sq, d);
  return b16 > f32 ? b16 : f32;
}

int tq_decompress_values(const uint8_t* packed_idx, const uint16_t* vec_norms, int64_t n, int d, const float* Pi,
                         const float* centroids, int bits, float* out, void* stream) {
  TQ_REQUIRE(valid_head_dim(d), "head_dim %d unsupported (64 or 128)", d);
  TQ_REQUIRE(valid_bits(bits), "bits %d unsupported (2, 3 or 4)", bits);
  TQ_REQUIRE(n >= 0 && n < ((int64_t)1 << 36), "bad vector count");
  if (n == 0) return TQ_OK;
  TQ_REQUIRE(packed_idx && vec_norms && Pi && centroids && out, "NULL pointer");
  TQ_REQUIRE(aligned16(out), "out must be 16-byte aligned");
  CallScope scope(packed_idx, "packed_idx", static_cast<cudaStream_t>(stream));
  if (scope.status()) return scope.status();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (d == 128) {
    if (bits == 2) return launch_decompress<128, 2>(packed_idx, vec_norms, n, Pi, centroids, out, s);
    if (bits == 3) return launch_decompress<128, 3>(packed_idx, vec_norms, n, Pi, centroids, out, s);
    return launch_decompress<128, 4>(packed_idx, vec_norms, n, Pi, centroids, out, s);
  }
  if (bits == 2) return launch_decompress<64, 2>(packed_idx, vec_norms, n, Pi, centroids, out, s);
  if (bits == 3) return launch_decompress<64, 3>(packed_idx, vec_norms, n, Pi, centroids, out, s);
  return launch_decompress<64, 4>(packed_idx, vec_norms, n, Pi, centroids, out, s);
}

int tq_attention_scores(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d, int64_t q_stride_b,
                        int64_t q_stride_h, int64_t q_stride_s, int64_t Hkv, int64_t Sk, const uint8_t* key_idx,
                        const uint8_t* key_signs, const uint16_t* key_vec_norms,
                        const uint16_t* key_residual_norms, const float* Pi_k, const float* S_eff,
                        const float* centroids_k, int bits, float* scores, void* workspace, size_t workspace_bytes,
                        int mode, void* stream) {
  if (int st = check_attention_common(q, dtype, B, Hq, Sq, d, q_stride_b, q_stride_h, q_stride_s, Hkv, Sk, bits,
                                      mode))
    return st;
  if (B * Hq * Sq == 0 || Sk == 0) return TQ_OK;
  TQ_REQUIRE(key_idx && key_signs && key_vec_norms && key_residual_norms, "NULL key pointer");
  TQ_REQUIRE(Pi_k && S_eff && centroids_k && scores, "NULL pointer");
  const size_t need = tq_attention_workspace_bytes(B, Hq, Sq, d, TQ_MODE_FP32);
  if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u))
    return fail(TQ_ERR_WORKSPACE, "workspace of %zu bytes needed (256-byte aligned), got %zu", need, workspace_bytes);
  // The score matrix is a parity/inspection product: always evaluated in fp32.
  CallScope scope(q, "q", static_cast<cudaStream_t>(stream));
  if (scope.status()) return scope.status();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* q_cat = static_cast<float*>(workspace);
  if (int st = qprep_fp32(q, dtype, B, Hq, Sq, d, q_stride_b, q_stride_h, q_stride_s, Pi_k, S_eff, q_cat, s))
    return st;
  ScoreArgs a{q_cat, Hq, Sq, Hkv, Sk, key_idx, key_signs, key_vec_norms, key_residual_norms, centroids_k, scores};
  return scores_fp32(a, B, d, bits, s);
}

}  // extern "C"

namespace tq {

// Entry used by tq_attention_fwd (tq_api.cu) for TQ_MODE_FP32.
int attention_fwd_fp32(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d, int64_t sb, int64_t sh,
                       int64_t ss, const float* Pi_k, const float* S_eff, AttnArgs a, int bits, void* workspace,
                       cudaStream_t stream) {
  float* q_cat = static_cast<float*>(workspace);
  if (int st = qprep_fp32(q, dtype, B, Hq, Sq, d, sb, sh, ss, Pi_k, S_eff, q_cat, stream)) return st;
  a.q_cat = q_cat;
  return attention_fp32(a, B, d, bits, stream);
}

int check_attention_args(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d, int64_t sb, int64_t sh,
                         int64_t ss, int64_t Hkv, int64_t Sk, int bits, int mode) {
  return check_attention_common(q, dtype, B, Hq, Sq, d, sb, sh, ss, Hkv, Sk, bits, mode);
}

}  // namespace tq

extern "C" int tq_prepare_queries(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d,
                                  int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s, const float* Pi_k,
                                  const float* S_eff, void* q_cat, void* workspace, size_t workspace_bytes, int mode,
                                  void* stream) {
  if (int st = check_attention_common(q, dtype, B, Hq, Sq, d, q_stride_b, q_stride_h, q_stride_s, 1, 0, 2, mode))
    return st;
  if (B * Hq * Sq == 0) return TQ_OK;
  TQ_REQUIRE(Pi_k && S_eff && q_cat && aligned16(q_cat), "NULL or misaligned pointer");
  CallScope scope(q, "q", static_cast<cudaStream_t>(stream));
  if (scope.status()) return scope.status();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (mode == TQ_MODE_FP32)
    return qprep_fp32(q, dtype, B, Hq, Sq, d, q_stride_b, q_stride_h, q_stride_s, Pi_k, S_eff,
                      static_cast<float*>(q_cat), s);
  const size_t need = (size_t)2 * d * d * 2;
  if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u))
    return fail(TQ_ERR_WORKSPACE, "workspace of %zu bytes needed (256-byte aligned), got %zu", need,
                workspace_bytes);
  return prepare_queries_bf16(q, dtype, B, Hq, Sq, d, q_stride_b, q_stride_h, q_stride_s, Pi_k, S_eff, workspace,
                              q_cat, s);
}

static int attention_entry(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d, int64_t q_stride_b,
                                int64_t q_stride_h, int64_t q_stride_s, int64_t Hkv, int64_t Sk, int64_t kv_stride,
                                const uint8_t* key_idx, const uint8_t* key_signs, const uint16_t* key_vec_norms,
                                const uint16_t* key_residual_norms, const uint8_t* val_idx,
                                const uint16_t* val_vec_norms, const float* Pi_k, const float* S_eff,
                                const float* centroids_k, const float* Pi_v, const float* centroids_v, int bits,
                                float sm_scale, int causal, const float* mask, int64_t mask_stride_b,
                                int64_t mask_stride_q, void* out, int64_t o_stride_b, int64_t o_stride_h,
                                int64_t o_stride_s, void* workspace, size_t workspace_bytes, int mode, void* stream,
                                const uint8_t* prepared = nullptr) {
  if (int st = check_attention_common(q, dtype, B, Hq, Sq, d, q_stride_b, q_stride_h, q_stride_s, Hkv, Sk, bits,
                                      mode))
    return st;
  if (B * Hq * Sq == 0) return TQ_OK;
  if (prepared != nullptr) {  // the matrices and codebooks are the fp32 copies inside the constants buffer
    const ConstLayout L = const_layout(d);
    Pi_k = reinterpret_cast<const float*>(prepared + L.pi_k);
    S_eff = reinterpret_cast<const float*>(prepared + L.s_eff);
    centroids_k = reinterpret_cast<const float*>(prepared + L.cen_k);
    Pi_v = reinterpret_cast<const float*>(prepared + L.pi_v);
    centroids_v = reinterpret_cast<const float*>(prepared + L.cen_v);
  }
  TQ_REQUIRE(Sk > 0, "attention over zero keys is undefined");
  TQ_REQUIRE(!causal || Sk >= Sq, "causal attention needs Sk >= Sq (got Sq=%lld, Sk=%lld)", (long long)Sq,
             (long long)Sk);
  TQ_REQUIRE(key_idx && key_signs && key_vec_norms && key_residual_norms && val_idx && val_vec_norms,
             "NULL packed K/V pointer");
  TQ_REQUIRE(Pi_k && S_eff && centroids_k && Pi_v && centroids_v, "NULL constant pointer");
  TQ_REQUIRE(out != nullptr && aligned16(out), "out must be a 16-byte aligned device pointer");
  const int64_t al = 16 / elem_size(dtype);
  TQ_REQUIRE(o_stride_b % al == 0 && o_stride_h % al == 0 && o_stride_s % al == 0,
             "out strides must keep every row 16-byte aligned");
  TQ_REQUIRE(sm_scale == sm_scale, "sm_scale is NaN");
  const size_t need = prepared != nullptr
                          ? tq_attention_prepared_workspace_bytes(B, Hq, Sq, Hkv, Sk, kv_stride, d, mode)
                          : tq_attention_workspace_bytes(B, Hq, Sq, d, mode);
  if (need > 0 && (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u)))
    return fail(TQ_ERR_WORKSPACE, "workspace of %zu bytes needed (256-byte aligned), got %zu", need,
                workspace_bytes);
  CallScope scope(q, "q", static_cast<cudaStream_t>(stream));
  if (scope.status()) return scope.status();
  AttnArgs a{nullptr, Hq, Sq, Hkv, Sk, key_idx, key_signs, key_vec_norms, key_residual_norms, val_idx,
             val_vec_norms, centroids_k, centroids_v, Pi_v, sm_scale, causal, mask, mask_stride_b, mask_stride_q,
             out, dtype, o_stride_b, o_stride_h, o_stride_s, kv_stride};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (mode == TQ_MODE_FP32) {
    TQ_REQUIRE(kv_stride == Sk, "a cache with capacity > Sk needs TQ_MODE_BF16");
    return attention_fwd_fp32(q, dtype, B, Hq, Sq, d, q_stride_b, q_stride_h, q_stride_s, Pi_k, S_eff, a, bits,
                              workspace, s);
  }
  return attention_fwd_bf16(q, dtype, B, Hq, Sq, d, q_stride_b, q_stride_h, q_stride_s, Pi_k, S_eff, a, bits,
                            workspace, s, prepared);
}

extern "C" size_t tq_constants_bytes(int d, int bits) {
  if (!valid_head_dim(d) || !valid_bits(bits)) return 0;
  return const_layout(d).total;
}

extern "C" int tq_prepare_constants(const float* Pi_k, const float* S_eff, const float* centroids_k,
                                    const float* boundaries_k, const float* Pi_v, const float* centroids_v,
                                    const float* boundaries_v, int bits, int d, void* constants,
                                    size_t constants_bytes, void* stream) {
  TQ_REQUIRE(valid_head_dim(d), "head_dim %d unsupported (64 or 128)", d);
  TQ_REQUIRE(valid_bits(bits), "bits %d unsupported (2, 3 or 4)", bits);
  TQ_REQUIRE(Pi_k && S_eff && centroids_k && boundaries_k && Pi_v && centroids_v && boundaries_v,
             "NULL constant pointer");
  const size_t need = const_layout(d).total;
  if (constants == nullptr || constants_bytes < need || (reinterpret_cast<uintptr_t>(constants) & 255u))
    return fail(TQ_ERR_WORKSPACE, "constants buffer of %zu bytes needed (256-byte aligned), got %zu", need,
                constants_bytes);
  CallScope scope(constants, "constants", static_cast<cudaStream_t>(stream));
  if (scope.status()) return scope.status();
  return prepare_constants(Pi_k, S_eff, centroids_k, boundaries_k, Pi_v, centroids_v, boundaries_v, bits, d, constants,
                           static_cast<cudaStream_t>(stream));
}

extern "C" size_t tq_attention_prepared_workspace_bytes(int64_t B, int64_t Hq, int64_t Sq, int64_t Hkv, int64_t Sk,
                                                        int64_t kv_capacity, int d, int mode) {
  if (B <= 0 || Hq <= 0 || Sq <= 0 || d <= 0 || Hkv <= 0) return 0;
  if (mode == TQ_MODE_FP32) return ((size_t)B * Hq * Sq * 2 * d * 4 + 255) & ~(size_t)255;
  return workspace_bytes_bf16_prepared(B, Hq, Sq, Hkv, Sk, kv_capacity, d);
}

extern "C" int tq_attention_fwd_prepared(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d,
                                         int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s, int64_t Hkv,
                                         int64_t Sk, int64_t kv_capacity, const uint8_t* key_idx,
                                         const uint8_t* key_signs, const uint16_t* key_vec_norms,
                                         const uint16_t* key_residual_norms, const uint8_t* val_idx,
                                         const uint16_t* val_vec_norms, const void* constants, int bits,
                                         float sm_scale, int causal, const float* mask, int64_t mask_stride_b,
                                         int64_t mask_stride_q, void* out, int64_t o_stride_b, int64_t o_stride_h,
                                         int64_t o_stride_s, void* workspace, size_t workspace_bytes, int mode,
                                         void* stream) {
  TQ_REQUIRE(constants != nullptr && (reinterpret_cast<uintptr_t>(constants) & 255u) == 0,
             "constants must be a 256-byte aligned buffer filled by tq_prepare_constants");
  TQ_REQUIRE(kv_capacity >= Sk, "cache capacity %lld is smaller than the %lld keys in use", (long long)kv_capacity,
             (long long)Sk);
  const float* dummy = reinterpret_cast<const float*>(constants);  // replaced from the buffer inside
  return attention_entry(q, dtype, B, Hq, Sq, d, q_stride_b, q_stride_h, q_stride_s, Hkv, Sk, kv_capacity, key_idx,
                         key_signs, key_vec_norms, key_residual_norms, val_idx, val_vec_norms, dummy, dummy, dummy,
                         dummy, dummy, bits, sm_scale, causal, mask, mask_stride_b, mask_stride_q, out, o_stride_b,
                         o_stride_h, o_stride_s, workspace, workspace_bytes, mode, stream,
                         static_cast<const uint8_t*>(constants));
}

extern "C" int tq_attention_fwd(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d, int64_t q_stride_b,
                                int64_t q_stride_h, int64_t q_stride_s, int64_t Hkv, int64_t Sk,
                                const uint8_t* key_idx, const uint8_t* key_signs, const uint16_t* key_vec_norms,
                                const uint16_t* key_residual_norms, const uint8_t* val_idx,
                                const uint16_t* val_vec_norms, const float* Pi_k, const float* S_eff,
                                const float* centroids_k, const float* Pi_v, const float* centroids_v, int bits,
                                float sm_scale, int causal, const float* mask, int64_t mask_stride_b,
                                int64_t mask_stride_q, void* out, int64_t o_stride_b, int64_t o_stride_h,
                                int64_t o_stride_s, void* workspace, size_t workspace_bytes, int mode, void* stream) {
  return attention_entry(q, dtype, B, Hq, Sq, d, q_stride_b, q_stride_h, q_stride_s, Hkv, Sk, Sk, key_idx, key_signs,
                         key_vec_norms, key_residual_norms, val_idx, val_vec_norms, Pi_k, S_eff, centroids_k, Pi_v,
                         centroids_v, bits, sm_scale, causal, mask, mask_stride_b, mask_stride_q, out, o_stride_b,
                         o_stride_h, o_stride_s, workspace, workspace_bytes, mode, stream);
}

extern "C" int tq_attention_fwd_cached(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d,
                                       int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s, int64_t Hkv,
                                       int64_t Sk, int64_t kv_capacity, const uint8_t* key_idx,
                                       const uint8_t* key_signs, const uint16_t* key_vec_norms,
                                       const uint16_t* key_residual_norms, const uint8_t* val_idx,
                                       const uint16_t* val_vec_norms, const float* Pi_k, const float* S_eff,
                                       const float* centroids_k, const float* Pi_v, const float* centroids_v, int bits,
                                       float sm_scale, int causal, const float* mask, int64_t mask_stride_b,
                                       int64_t mask_stride_q, void* out, int64_t o_stride_b, int64_t o_stride_h,
                                       int64_t o_stride_s, void* workspace, size_t workspace_bytes, void* stream) {
  TQ_REQUIRE(kv_capacity >= Sk, "cache capacity %lld is smaller than the %lld keys in use", (long long)kv_capacity,
             (long long)Sk);
  // (a full cache, capacity == Sk, is the contiguous layout and may be served by any of the kernels)
  TQ_REQUIRE(d == 128 && Hkv > 0 && Hq % Hkv == 0 && (Hq / Hkv) * Sq <= 16,
             "tq_attention_fwd_cached serves head_dim 128 and (Hq / Hkv) * Sq <= 16 query rows per KV head");
  return attention_entry(q, dtype, B, Hq, Sq, d, q_stride_b, q_stride_h, q_stride_s, Hkv, Sk,
                         kv_capacity, key_idx, key_signs, key_vec_norms, key_residual_norms,
                         val_idx, val_vec_norms, Pi_k, S_eff, centroids_k, Pi_v, centroids_v, bits, sm_scale, causal,
                         mask, mask_stride_b, mask_stride_q, out, o_stride_b, o_stride_h, o_stride_s, workspace,
                         workspace_bytes, TQ_MODE_BF16, stream);
}

// ---- attention without caller-supplied scratch ---------------------------------------------
//
// Some hosts of this library may not allocate device memory themselves: a plugin running inside a
// serving process whose memory pool is owned by another component, a caller that holds only
// borrowed input and output buffers, or code on a path where cudaMalloc is forbidden (it
// synchronises the device and can fail late under memory pressure).  For them the scratch that
// tq_attention_fwd needs lives in this fixed array, which every GPU that loads the library carries
// until the process exits.
namespace {
constexpr size_t kStaticScratchBytes = 32u << 20;  // 32 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
void* g_static_scratch_addr[kMaxDevices] = {nullptr};  // device address of the array, per device
}  // namespace

extern "C" size_t tq_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int tq_attention_fwd_static(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d,
                                       int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s, int64_t Hkv,
                                       int64_t Sk, const uint8_t* key_idx, const uint8_t* key_signs,
                                       const uint16_t* key_vec_norms, const uint16_t* key_residual_norms,
                                       const uint8_t* val_idx, const uint16_t* val_vec_norms, const float* Pi_k,
                                       const float* S_eff, const float* centroids_k, const float* Pi_v,
                                       const float* centroids_v, int bits, float sm_scale, int causal,
                                       const float* mask, int64_t mask_stride_b, int64_t mask_stride_q, void* out,
                                       int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, int mode,
                                       void* stream) {
  if (int st = check_attention_common(q, dtype, B, Hq, Sq, d, q_stride_b, q_stride_h, q_stride_s, Hkv, Sk, bits,
                                      mode))
    return st;
  const size_t need = tq_attention_workspace_bytes(B, Hq, Sq, d, mode);
  if (need > kStaticScratchBytes)
    return fail(TQ_ERR_WORKSPACE,
                "problem needs %zu bytes of scratch but the built-in array holds %zu; use tq_attention_fwd with "
                "a caller-supplied workspace",
                need, kStaticScratchBytes);
  if (B * Hq * Sq == 0) return TQ_OK;
  // the array of the device that owns the queries, whatever the thread's current device is
  CallScope scope(q, "q", static_cast<cudaStream_t>(stream));
  if (scope.status()) return scope.status();
  const int dev = scope.device();
  if (g_static_scratch_addr[dev] == nullptr) {
    // In host code the array's name is only a handle; the address kernels may use comes from the
    // runtime, once per device, with that device current.
    void* p = nullptr;
    TQ_CUDA_OK(cudaGetSymbolAddress(&p, g_static_scratch));
    TQ_REQUIRE(p != nullptr, "could not resolve the built-in scratch array");
    g_static_scratch_addr[dev] = p;
  }
  return tq_attention_fwd(q, dtype, B, Hq, Sq, d, q_stride_b, q_stride_h, q_stride_s, Hkv, Sk, key_idx, key_signs,
                          key_vec_norms, key_residual_norms, val_idx, val_vec_norms, Pi_k, S_eff, centroids_k, Pi_v,
                          centroids_v, bits, sm_scale, causal, mask, mask_stride_b, mask_stride_q, out, o_stride_b,
                          o_stride_h, o_stride_s, g_static_scratch_addr[dev], kStaticScratchBytes, mode, stream);
}
