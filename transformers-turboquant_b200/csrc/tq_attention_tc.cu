// Tensor-core (tcgen05 / tensor-memory) kernels of TQ_MODE_BF16:
//   * rows_gemm_tc   out[n, NOUT] = x[n, D] * W^T   (query preparation and output back-rotation)
//   * attention_tc   flash-style fused compressed attention: packed keys / signs / values are
//                    decoded to bf16 operand tiles in shared memory, S = [q_rot | q_s] * K_hat^T and
//                    O += P * V_hat run as tcgen05 MMAs with fp32 accumulators in tensor memory,
//                    causal online softmax on the CUDA cores in between.
// Nothing of size Sq x Sk and no decompressed K/V ever reaches HBM.
//
// Estimator algebra (reference compressors.py:201-224, kernels/attention.py:380-461):
//   score(q,k) = n_k <q_rot, C[idx_k]> + coeff rn_k <q_s, sgn_k>
//              = n_k * ( <q_rot, C[idx_k]> + <coeff q_s, (rn_k/n_k) sgn_k> )
// so one MMA over the concatenated contraction dimension [C[idx] ; (rn/n) sgn] of length 2d
// followed by a per-key column scale n_k * sm_scale * log2(e) gives the softmax argument.
//
// Every device-side wait is bounded; when one expires the kernel bumps a fault counter,
// frees its tensor memory and returns, and later launches return immediately.
#include <math.h>

#include "tq_attention.cuh"
#include "tq_common.cuh"
#include "tq_simt.cuh"
#include "tq_tcgen05.cuh"

namespace tq {

__device__ unsigned long long g_wait_faults = 0ull;

int read_wait_faults(unsigned long long* out) {
  TQ_CUDA_OK(cudaMemcpyFromSymbol(out, g_wait_faults, sizeof(*out)));
  return TQ_OK;
}

__device__ __forceinline__ bool poisoned() {
  return *reinterpret_cast<volatile unsigned long long*>(&g_wait_faults) != 0ull;
}
__device__ __forceinline__ void record_fault() { atomicAdd(&g_wait_faults, 1ull); }

// ---- constant operand builder ------------------------------------------------------------
// w_cat [2d, d] bf16 = [ Pi ; coeff * S ] with S = S_eff * Pi, so that q * w_cat^T = [q_rot | coeff q_s];
// w_unrot [d, d] bf16 = Pi_v^T, so that o_rot * w_unrot^T = o_rot * Pi_v.
__global__ void build_wcat_kernel(const float* __restrict__ Pi, const float* __restrict__ S_eff, int d, float coeff,
                                  __nv_bfloat16* __restrict__ w_cat) {
  const int j = blockIdx.x, i = threadIdx.x;  // one block per row, d threads
  w_cat[j * d + i] = __float2bfloat16_rn(Pi[j * d + i]);
  float acc = 0.f;
  for (int c = 0; c < d; ++c) acc = fmaf(S_eff[j * d + c], Pi[c * d + i], acc);
  w_cat[(d + j) * d + i] = __float2bfloat16_rn(coeff * acc);
}
__global__ void build_wunrot_kernel(const float* __restrict__ Pi_v, int d, __nv_bfloat16* __restrict__ w_unrot) {
  const int j = blockIdx.x, i = threadIdx.x;
  w_unrot[j * d + i] = __float2bfloat16_rn(Pi_v[i * d + j]);
}

// ---- row GEMM ----------------------------------------------------------------------------

struct RowsGemmArgs {
  const void* x;
  int x_dtype;
  int64_t n_rows, H, S;            // row n = (b*H + h)*S + s
  int64_t xs_b, xs_h, xs_s;        // element strides of x
  const __nv_bfloat16* W;          // [NOUT, D] row-major
  void* out;
  int out_dtype;
  int64_t os_b, os_h, os_s;        // element strides of out (rows of NOUT contiguous elements)
  int num_tiles;
};

__device__ __forceinline__ uint4 load_row_chunk_bf16(const void* base, int dtype, int64_t off) {
  if (dtype == TQ_BF16) return *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + off);
  float v[8];
  if (dtype == TQ_F32) load8<float>(static_cast<const float*>(base) + off, v);
  else load8<__half>(static_cast<const __half*>(base) + off, v);
  uint4 r;
  r.x = tc::pack_bf16x2(v[0], v[1]);
  r.y = tc::pack_bf16x2(v[2], v[3]);
  r.z = tc::pack_bf16x2(v[4], v[5]);
  r.w = tc::pack_bf16x2(v[6], v[7]);
  return r;
}

__device__ __forceinline__ void store_row_chunk(void* base, int dtype, int64_t off, const uint32_t (&acc)[32]) {
  // 32 fp32 accumulator values -> 32 consecutive output elements
  if (dtype == TQ_F32) {
    float4* p = reinterpret_cast<float4*>(static_cast<float*>(base) + off);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      p[i] = make_float4(__uint_as_float(acc[4 * i]), __uint_as_float(acc[4 * i + 1]),
                         __uint_as_float(acc[4 * i + 2]), __uint_as_float(acc[4 * i + 3]));
  } else if (dtype == TQ_BF16) {
    uint4* p = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(base) + off);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 w;
      w.x = tc::pack_bf16x2(__uint_as_float(acc[8 * i]), __uint_as_float(acc[8 * i + 1]));
      w.y = tc::pack_bf16x2(__uint_as_float(acc[8 * i + 2]), __uint_as_float(acc[8 * i + 3]));
      w.z = tc::pack_bf16x2(__uint_as_float(acc[8 * i + 4]), __uint_as_float(acc[8 * i + 5]));
      w.w = tc::pack_bf16x2(__uint_as_float(acc[8 * i + 6]), __uint_as_float(acc[8 * i + 7]));
      p[i] = w;
    }
  } else {
    uint4* p = reinterpret_cast<uint4*>(static_cast<__half*>(base) + off);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        h[e] = __floats2half2_rn(__uint_as_float(acc[8 * i + 2 * e]), __uint_as_float(acc[8 * i + 2 * e + 1]));
      p[i] = *reinterpret_cast<uint4*>(h);
    }
  }
}

// 128 threads; thread t owns row t of the 128-row tile (tensor-memory lane t).
template <int D, int NOUT>
__global__ void __launch_bounds__(128) rows_gemm_tc_kernel(const RowsGemmArgs a) {
  constexpr int G = D / 8;                 // 16-byte chunks per row
  constexpr uint32_t SBO = G * 128;        // stride between 8-row groups
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* As = smem_raw;                  // [128, D] K-major
  uint8_t* Ws = As + 128 * D * 2;          // [NOUT, D] K-major
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  const int tid = threadIdx.x, warp = tid / 32;
  if (tid == 0) s_abort = poisoned() ? 1 : 0;
  __syncthreads();
  if (s_abort) return;  // an earlier bounded wait expired: do nothing rather than risk another
  if (tid == 0) {
    tc::mbar_init(tc::smem_u32(&bar), 1);
    tc::fence_mbar_init();
  }
  if (warp == 0) tc::tmem_alloc(tc::smem_u32(&tmem_slot), NOUT < 32 ? 32 : NOUT);
  // W -> shared, canonical layout: row j, chunk c at (j/8)*SBO + c*128 + (j%8)*16
  for (int e = tid; e < NOUT * G; e += 128) {
    const int j = e % 8 + 8 * (e / (8 * G)), c = (e / 8) % G;
    const uint4 v = *reinterpret_cast<const uint4*>(a.W + j * D + c * 8);
    *reinterpret_cast<uint4*>(Ws + (j / 8) * SBO + c * 128 + (j % 8) * 16) = v;
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t bar_addr = tc::smem_u32(&bar);
  constexpr uint32_t idesc = tc::idesc_bf16(128, NOUT, false, false);
  const uint64_t adesc0 = tc::smem_desc(tc::smem_u32(As), 128, SBO);
  const uint64_t bdesc0 = tc::smem_desc(tc::smem_u32(Ws), 128, SBO);
  const int64_t HS = a.H * a.S;
  uint32_t phase = 0;
  for (int tile = blockIdx.x; tile < a.num_tiles; tile += gridDim.x) {
    const int64_t n = static_cast<int64_t>(tile) * 128 + tid;
    const bool live = n < a.n_rows;
    int64_t b = 0, h = 0, s = 0;
    if (live) { b = n / HS; h = (n % HS) / a.S; s = n % a.S; }
    {
      const int64_t xoff = b * a.xs_b + h * a.xs_h + s * a.xs_s;
      uint8_t* dst = As + (tid / 8) * SBO + (tid % 8) * 16;
#pragma unroll 4
      for (int c = 0; c < G; ++c) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (live) v = load_row_chunk_bf16(a.x, a.x_dtype, xoff + c * 8);
        *reinterpret_cast<uint4*>(dst + c * 128) = v;
      }
    }
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      tc::fence_after_sync();
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks)
        tc::mma_bf16(tmem, adesc0 + (uint64_t)(ks * 256 >> 4), bdesc0 + (uint64_t)(ks * 256 >> 4), idesc, ks > 0);
      tc::mma_commit(bar_addr);
    }
    if (!tc::mbar_wait_bounded(bar_addr, phase)) { record_fault(); s_abort = 1; }
    phase ^= 1;
    tc::fence_after_sync();
    __syncthreads();
    if (s_abort) break;
    const int64_t ooff = b * a.os_b + h * a.os_h + s * a.os_s;
#pragma unroll 1
    for (int c0 = 0; c0 < NOUT; c0 += 32) {
      uint32_t acc[32];
      tc::tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + c0, acc);
      tc::wait_ld();
      if (live) store_row_chunk(a.out, a.out_dtype, ooff + c0, acc);
    }
    tc::fence_before_sync();  // the next tile's MMA overwrites the accumulator
  }
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, NOUT < 32 ? 32 : NOUT);
}

// ---- fused attention ---------------------------------------------------------------------

constexpr int kBM = 128;  // query rows per CTA
constexpr int kBN = 128;  // keys per tile

template <int D>
struct AttnSmem {
  static constexpr int G = D / 8;
  static constexpr uint32_t kQBytes = kBM * 2 * D * 2;
  static constexpr uint32_t kKBytes = kBN * 2 * D * 2;
  static constexpr uint32_t kVBytes = kBN * D * 2;
  static constexpr uint32_t kPBytes = kBM * kBN * 2;
  static constexpr uint32_t kQOff = 0;
  static constexpr uint32_t kKOff = kQOff + kQBytes;
  static constexpr uint32_t kVOff = kKOff + kKBytes;
  static constexpr uint32_t kPOff = kVOff + kVBytes;
  static constexpr uint32_t kTotal = kPOff + kPBytes;
  static constexpr uint32_t kSboQK = 2 * G * 128;   // K-major [rows, 2D]
  static constexpr uint32_t kSboP = (kBN / 8) * 128;  // K-major [rows, kBN]
  static constexpr uint32_t kSboV = 128;              // MN-major [D, kBN]: 8-coordinate chunks adjacent
  static constexpr uint32_t kLboV = G * 128;          // ... 8-key groups G core matrices apart
};

template <int D, int BITS>
__global__ void __launch_bounds__(256, 1) attention_tc_kernel(const AttnArgs a, __nv_bfloat16* __restrict__ o_rot) {
  using L = AttnSmem<D>;
  constexpr int G = L::G, KB = BITS - 1, VB = BITS;
  constexpr int kTmemCols = 256;  // S: columns [0,128), O: columns [128, 128+D)
  constexpr float kLog2e = 1.4426950408889634f;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* Qs = smem_raw + L::kQOff;
  uint8_t* Ks = smem_raw + L::kKOff;
  uint8_t* Vs = smem_raw + L::kVOff;
  uint8_t* Ps = smem_raw + L::kPOff;
  __shared__ float cscale[kBN];
  __shared__ float xmax[2][kBM];
  __shared__ uint32_t lutK[1 << (2 * KB)];
  __shared__ uint32_t lutV[1 << (2 * VB)];
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  if (tid == 0) s_abort = poisoned() ? 1 : 0;
  __syncthreads();
  if (s_abort) return;  // an earlier bounded wait expired: do nothing rather than risk another
  const int64_t b = blockIdx.z, h = blockIdx.y;
  const int64_t bh = b * a.Hq + h;
  const int64_t kv_base = (b * a.Hkv + h / (a.Hq / a.Hkv)) * a.Sk;
  // heaviest (latest) query tiles first: they have the most key tiles under the causal mask
  const int q0 = (int)(gridDim.x - 1 - blockIdx.x) * kBM;
  const int shift = (int)(a.Sk - a.Sq);

  if (tid == 0) {
    tc::mbar_init(tc::smem_u32(&bars[0]), 1);
    tc::mbar_init(tc::smem_u32(&bars[1]), 1);
    tc::fence_mbar_init();
  }
  if (warp == 0) tc::tmem_alloc(tc::smem_u32(&tmem_slot), kTmemCols);
  for (int e = tid; e < (1 << (2 * KB)); e += 256) {
    const float c0 = a.cen_k[e & ((1 << KB) - 1)], c1 = a.cen_k[e >> KB];
    lutK[e] = tc::pack_bf16x2(c0, c1);
  }
  for (int e = tid; e < (1 << (2 * VB)); e += 256) {
    const float c0 = a.cen_v[e & ((1 << VB) - 1)], c1 = a.cen_v[e >> VB];
    lutV[e] = tc::pack_bf16x2(c0, c1);
  }
  {  // Q tile: thread t loads half of row t%128 (2G chunks per row)
    const int r = tid % kBM, half = tid / kBM;
    const bool live = q0 + r < a.Sq;
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.q_cat) +
                                                      (bh * a.Sq + q0 + r) * 2 * D);
    uint8_t* dst = Qs + (r / 8) * L::kSboQK + (r % 8) * 16;
#pragma unroll 4
    for (int c = half * G; c < (half + 1) * G; ++c) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (live) v = src[c];
      *reinterpret_cast<uint4*>(dst + c * 128) = v;
    }
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_s = tmem_slot;
  const uint32_t tmem_o = tmem_s + kBN;
  const uint32_t bar_s = tc::smem_u32(&bars[0]), bar_o = tc::smem_u32(&bars[1]);
  constexpr uint32_t idesc_s = tc::idesc_bf16(kBM, kBN, false, false);
  constexpr uint32_t idesc_o = tc::idesc_bf16(kBM, D, false, true);
  const uint64_t qdesc = tc::smem_desc(tc::smem_u32(Qs), 128, L::kSboQK);
  const uint64_t kdesc = tc::smem_desc(tc::smem_u32(Ks), 128, L::kSboQK);
  const uint64_t pdesc = tc::smem_desc(tc::smem_u32(Ps), 128, L::kSboP);
  const uint64_t vdesc = tc::smem_desc(tc::smem_u32(Vs), L::kLboV, L::kSboV);

  // softmax ownership: row = tensor-memory lane; the two warp groups split the columns
  const int row = (warp % 4) * 32 + lane;
  const int chalf = warp / 4;
  const uint32_t lane_base = (uint32_t)((warp % 4) * 32) << 16;
  const int qi = q0 + row;
  float m_run = -INFINITY, l_run = 0.f;
  uint32_t phase_s = 0, phase_o = 0;

  int k_end = (int)a.Sk;
  if (a.causal) k_end = min(k_end, min(q0 + kBM - 1, (int)a.Sq - 1) + shift + 1);
  const int n_tiles = (k_end + kBN - 1) / kBN;

  for (int kt = 0; kt < n_tiles; ++kt) {
    const int k0 = kt * kBN;
    // ---- (A) decode K_hat, V_hat tiles ---------------------------------------------------
#pragma unroll 2
    for (int e = tid; e < kBN * G; e += 256) {
      const int j = (e % 8) + 8 * (e / (8 * G)), g = (e / 8) % G;
      uint4 kw = make_uint4(0, 0, 0, 0), sw = kw, vw = kw;
      if (k0 + j < a.Sk) {
        const int64_t n = kv_base + k0 + j;
        const uint64_t wk = load_fields8<KB>(a.key_idx + n * (D * KB / 8) + g * KB);
        const uint32_t sb = ~static_cast<uint32_t>(a.key_sgn[n * G + g]);
        const uint64_t wv = load_fields8<VB>(a.val_idx + n * (D * VB / 8) + g * VB);
        const float nk = fp16_value(a.key_vn[n]);
        const float rho = nk > 0.f ? fp16_value(a.key_rn[n]) / nk : 0.f;
        const uint32_t rr = tc::pack_bf16x2(rho, rho);
        const float nvf = fp16_value(a.val_vn[n]);
        const __nv_bfloat162 nv2 = __floats2bfloat162_rn(nvf, nvf);
        uint32_t kq[4], sq[4], vq[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          kq[p] = lutK[(wk >> (2 * p * KB)) & ((1u << (2 * KB)) - 1)];
          sq[p] = rr ^ (((sb >> (2 * p)) & 1u) << 15) ^ (((sb >> (2 * p + 1)) & 1u) << 31);
          const uint32_t vv = lutV[(wv >> (2 * p * VB)) & ((1u << (2 * VB)) - 1)];
          const __nv_bfloat162 prod = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&vv), nv2);
          vq[p] = *reinterpret_cast<const uint32_t*>(&prod);
        }
        kw = make_uint4(kq[0], kq[1], kq[2], kq[3]);
        sw = make_uint4(sq[0], sq[1], sq[2], sq[3]);
        vw = make_uint4(vq[0], vq[1], vq[2], vq[3]);
      }
      uint8_t* kd = Ks + (j / 8) * L::kSboQK + (j % 8) * 16;
      *reinterpret_cast<uint4*>(kd + g * 128) = kw;
      *reinterpret_cast<uint4*>(kd + (G + g) * 128) = sw;
      *reinterpret_cast<uint4*>(Vs + g * L::kSboV + (j / 8) * L::kLboV + (j % 8) * 16) = vw;
    }
    if (tid < kBN) {
      const int k = k0 + tid;
      cscale[tid] = k < a.Sk ? fp16_value(a.key_vn[kv_base + k]) * a.sm_scale * kLog2e : 0.f;
    }
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    // ---- (B) S = Q_cat * K_hat^T ---------------------------------------------------------
    if (tid == 0) {
      tc::fence_after_sync();
#pragma unroll
      for (int ks = 0; ks < 2 * D / 16; ++ks)
        tc::mma_bf16(tmem_s, qdesc + (uint64_t)(ks * 256 >> 4), kdesc + (uint64_t)(ks * 256 >> 4), idesc_s, ks > 0);
      tc::mma_commit(bar_s);
    }
    // ---- (C) online softmax ---------------------------------------------------------------
    if (!tc::mbar_wait_bounded(bar_s, phase_s)) { record_fault(); s_abort = 1; }
    phase_s ^= 1;
    tc::fence_after_sync();
    float t[64];
    {
      uint32_t raw[32];
      tc::tmem_ld32(tmem_s + lane_base + chalf * 64, raw);
      tc::wait_ld();
#pragma unroll
      for (int c = 0; c < 32; ++c) t[c] = __uint_as_float(raw[c]);
      tc::tmem_ld32(tmem_s + lane_base + chalf * 64 + 32, raw);
      tc::wait_ld();
#pragma unroll
      for (int c = 0; c < 32; ++c) t[32 + c] = __uint_as_float(raw[c]);
    }
    float mx = -INFINITY;
    const float* mrow = (a.mask != nullptr && qi < a.Sq)
                            ? a.mask + b * a.mask_stride_b + (int64_t)qi * a.mask_stride_q + k0 + chalf * 64
                            : nullptr;
#pragma unroll
    for (int c = 0; c < 64; ++c) {
      const int kc = chalf * 64 + c, k = k0 + kc;
      float v = t[c] * cscale[kc];
      if (mrow != nullptr && k < a.Sk) v = fmaf(mrow[c], kLog2e, v);
      if (k >= a.Sk || (a.causal && k > qi + shift)) v = -INFINITY;
      t[c] = v;
      mx = fmaxf(mx, v);
    }
    xmax[chalf][row] = mx;
    __syncthreads();
    if (s_abort) break;
    const float m_new = fmaxf(m_run, fmaxf(mx, xmax[1 - chalf][row]));
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
    const float alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_use);
    m_run = m_new;
    float psum = 0.f;
    {
      uint8_t* pd = Ps + (row / 8) * L::kSboP + (row % 8) * 16 + (chalf * 8) * 128;
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {
        uint32_t w[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const float p0 = exp2f(t[c8 * 8 + 2 * p] - m_use), p1 = exp2f(t[c8 * 8 + 2 * p + 1] - m_use);
          psum += p0 + p1;
          w[p] = tc::pack_bf16x2(p0, p1);
        }
        *reinterpret_cast<uint4*>(pd + c8 * 128) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    l_run = l_run * alpha + psum;
    if (kt > 0) {  // rescale this warp group's half of the output accumulator
#pragma unroll 1
      for (int c0 = 0; c0 < D / 2; c0 += 32) {
        uint32_t raw[32];
        const uint32_t addr = tmem_o + lane_base + chalf * (D / 2) + c0;
        tc::tmem_ld32(addr, raw);
        tc::wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) raw[c] = __float_as_uint(__uint_as_float(raw[c]) * alpha);
        tc::tmem_st32(addr, raw);
      }
      tc::wait_st();
    }
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    // ---- (D) O += P * V_hat -----------------------------------------------------------------
    if (tid == 0) {
      tc::fence_after_sync();
#pragma unroll
      for (int ks = 0; ks < kBN / 16; ++ks)
        tc::mma_bf16(tmem_o, pdesc + (uint64_t)(ks * 256 >> 4), vdesc + (uint64_t)(ks * 2 * L::kLboV >> 4), idesc_o,
                     (kt > 0 || ks > 0) ? 1u : 0u);
      tc::mma_commit(bar_o);
    }
    // ---- (E) operands and accumulator are free again once the MMA has drained -----------------
    if (!tc::mbar_wait_bounded(bar_o, phase_o)) { record_fault(); s_abort = 1; }
    phase_o ^= 1;
    tc::fence_after_sync();
    __syncthreads();
    if (s_abort) break;
  }

  // ---- epilogue: normalise and store the rotated output tile ------------------------------------
  if (!s_abort) {
    xmax[chalf][row] = l_run;
    __syncthreads();
    const float l_tot = l_run + xmax[1 - chalf][row];
    const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
    __nv_bfloat16* dst = o_rot + (bh * a.Sq + qi) * D + chalf * (D / 2);
#pragma unroll 1
    for (int c0 = 0; c0 < D / 2; c0 += 32) {
      uint32_t raw[32];
      tc::tmem_ld32(tmem_o + lane_base + chalf * (D / 2) + c0, raw);
      tc::wait_ld();
      if (qi < a.Sq) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 w;
          w.x = tc::pack_bf16x2(__uint_as_float(raw[8 * i]) * inv, __uint_as_float(raw[8 * i + 1]) * inv);
          w.y = tc::pack_bf16x2(__uint_as_float(raw[8 * i + 2]) * inv, __uint_as_float(raw[8 * i + 3]) * inv);
          w.z = tc::pack_bf16x2(__uint_as_float(raw[8 * i + 4]) * inv, __uint_as_float(raw[8 * i + 5]) * inv);
          w.w = tc::pack_bf16x2(__uint_as_float(raw[8 * i + 6]) * inv, __uint_as_float(raw[8 * i + 7]) * inv);
          *reinterpret_cast<uint4*>(dst + c0 + 8 * i) = w;
        }
      }
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_s, kTmemCols);
}

// ---- host side ---------------------------------------------------------------------------

template <int D, int NOUT>
static int launch_rows_gemm(const RowsGemmArgs& a, cudaStream_t stream) {
  constexpr size_t smem = (size_t)(128 + NOUT) * D * 2;
  auto kern = rows_gemm_tc_kernel<D, NOUT>;
  TQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int grid = sm_count() * 2;
  if (grid > a.num_tiles) grid = a.num_tiles;
  kern<<<grid, 128, smem, stream>>>(a);
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
}

template <int D, int BITS>
static int launch_attention_tc(const AttnArgs& a, int64_t B, __nv_bfloat16* o_rot, cudaStream_t stream) {
  constexpr size_t smem = AttnSmem<D>::kTotal;
  auto kern = attention_tc_kernel<D, BITS>;
  TQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)((a.Sq + kBM - 1) / kBM), (unsigned)a.Hq, (unsigned)B);
  {
    ProfScope prof(kProfAttention, stream);
    kern<<<grid, 256, smem, stream>>>(a, o_rot);
  }
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
}

static inline size_t round256(size_t v) { return (v + 255) & ~(size_t)255; }

// workspace layout (bf16 mode): [ w_cat | w_unrot | q_cat | o_rot ]
size_t workspace_bytes_bf16(int64_t n_q, int d) {
  return round256((size_t)2 * d * d * 2) + round256((size_t)d * d * 2) + round256((size_t)n_q * 2 * d * 2) +
         round256((size_t)n_q * d * 2);
}

// q_cat bf16 [n, 2d] = [ q Pi^T | coeff * q S^T ] on the tensor cores; `w_cat` is 2*d*d bf16 of scratch.
int prepare_queries_bf16(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d, int64_t sb, int64_t sh,
                         int64_t ss, const float* Pi_k, const float* S_eff, void* w_cat_scratch, void* q_cat,
                         cudaStream_t stream) {
  const int64_t n_q = B * Hq * Sq;
  ProfScope prof(kProfPrepareQueries, stream);
  __nv_bfloat16* w_cat = static_cast<__nv_bfloat16*>(w_cat_scratch);
  build_wcat_kernel<<<d, d, 0, stream>>>(Pi_k, S_eff, d, sqrtf(1.5707963267948966f) / (float)d, w_cat);
  TQ_CUDA_OK(cudaGetLastError());
  const int tiles = (int)((n_q + 127) / 128);
  RowsGemmArgs prep{q, dtype, n_q, Hq, Sq, sb, sh, ss, w_cat, q_cat, TQ_BF16,
                    Hq * Sq * 2 * d, Sq * 2 * d, (int64_t)2 * d, tiles};
  return d == 128 ? launch_rows_gemm<128, 256>(prep, stream) : launch_rows_gemm<64, 128>(prep, stream);
}

int attention_fwd_bf16(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d, int64_t sb, int64_t sh,
                       int64_t ss, const float* Pi_k, const float* S_eff, AttnArgs a, int bits, void* workspace,
                       cudaStream_t stream) {
  const int64_t n_q = B * Hq * Sq;
  TQ_REQUIRE(B <= 65535 && Hq <= 65535, "batch and head counts are limited to 65535 in bf16 mode");
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  __nv_bfloat16* w_cat = reinterpret_cast<__nv_bfloat16*>(ws);
  ws += round256((size_t)2 * d * d * 2);
  __nv_bfloat16* w_unrot = reinterpret_cast<__nv_bfloat16*>(ws);
  ws += round256((size_t)d * d * 2);
  __nv_bfloat16* q_cat = reinterpret_cast<__nv_bfloat16*>(ws);
  ws += round256((size_t)n_q * 2 * d * 2);
  __nv_bfloat16* o_rot = reinterpret_cast<__nv_bfloat16*>(ws);

  build_wunrot_kernel<<<d, d, 0, stream>>>(a.Pi_v, d, w_unrot);
  TQ_CUDA_OK(cudaGetLastError());
  if (int st = prepare_queries_bf16(q, dtype, B, Hq, Sq, d, sb, sh, ss, Pi_k, S_eff, w_cat, q_cat, stream)) return st;
  const int tiles = (int)((n_q + 127) / 128);

  a.q_cat = q_cat;
  int st;
  if (d == 128)
    st = bits == 2   ? launch_attention_tc<128, 2>(a, B, o_rot, stream)
         : bits == 3 ? launch_attention_tc<128, 3>(a, B, o_rot, stream)
                     : launch_attention_tc<128, 4>(a, B, o_rot, stream);
  else
    st = bits == 2   ? launch_attention_tc<64, 2>(a, B, o_rot, stream)
         : bits == 3 ? launch_attention_tc<64, 3>(a, B, o_rot, stream)
                     : launch_attention_tc<64, 4>(a, B, o_rot, stream);
  if (st) return st;

  ProfScope prof(kProfBackRotation, stream);
  RowsGemmArgs unrot{o_rot, TQ_BF16, n_q, Hq, Sq, Hq * Sq * d, Sq * d, (int64_t)d, w_unrot, a.out, a.out_dtype,
                     a.o_stride_b, a.o_stride_h, a.o_stride_s, tiles};
  return d == 128 ? launch_rows_gemm<128, 128>(unrot, stream) : launch_rows_gemm<64, 64>(unrot, stream);
}

}  // namespace tq
