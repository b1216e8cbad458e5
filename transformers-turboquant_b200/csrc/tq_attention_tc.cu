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

// Diagnostics: stage timestamps (SM clock) of one CTA of the attention kernel, see tq_trace_read.
constexpr int kTraceCap = 4096;
__device__ int g_trace_on = 0;
__device__ long long g_trace[2 * kTraceCap];
// One tracer per traced thread: role r appends to its own third of the buffer, no atomics.
struct Tracer {
  bool on;
  int role, n;
  __device__ Tracer(bool on_, int role_) : on(on_), role(role_), n(0) {}
  __device__ __forceinline__ void mark(int ev, int tile) {
    if (!on || n >= kTraceCap / 3) return;
    const int i = role * (kTraceCap / 3) + n++;
    g_trace[2 * i] = ((long long)role << 32) | ((long long)ev << 16) | (long long)tile;
    g_trace[2 * i + 1] = clock64();
  }
};

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

// ---- fused attention (warp-specialised) ------------------------------------------------------
//
// One CTA = 128 query rows of one head.  Seventeen warps in three roles, coupled only by mbarriers:
//   warps 0-7   softmax    two threads per query row (= tensor-memory lane): warp w and w+4 share the
//                          rows of lane quadrant w%4 and split each 64-key tile into two 32-column
//                          halves.  Load the scores, scale, mask, exchange the half-row maxima, keep
//                          the running max / sum, write P (bf16) into tensor memory, rescale the output
//                          accumulator when the max grew, run the epilogue.
//   warps 8-15  producers  prefetch the next tile's packed bytes into registers, stage them in shared
//                          memory, decode indices / sign bits / norms into the K_hat and V_hat
//                          operand tiles (canonical core-matrix layout), up to kStages tiles ahead
//   warp 16     MMA        one thread issues S = Q_cat K_hat^T for tile j+1, then O += P V_hat for tile j
// Both A operands (the query tile and P) live in TENSOR MEMORY: shared-memory bandwidth, the scarcest
// resource of this kernel, is spent only on the decoded K_hat / V_hat tiles.
// Keys advance in tiles of 64.  S and P are double-buffered (index = tile parity), K_hat / V_hat /
// staged bytes form a ring of kStages slots (index = tile % kStages).
//
// Barriers ("use" = how often the slot has been used before selects the mbarrier phase):
//   pk_full[s]  256 producer arrivals : the packed bytes of tile j are staged in shared memory
//   k_full[s]   256 producer arrivals : K_hat and the column scales of tile j are ready
//   v_full[s]   256 producer arrivals : V_hat of tile j is ready
//   k_empty[s]  tcgen05.commit        : the score MMA of tile j has consumed K_hat[s]
//   v_empty[s]  tcgen05.commit        : the P V_hat MMA of tile j has consumed V_hat[s]
//   s_full[b]   tcgen05.commit        : S[b] holds the scores of tile j
//   s_empty[b]  256 softmax arrivals  : S[b] has been read into registers
//   p_full[b]   256 softmax arrivals  : P[b] written (and O rescaled if needed)
//   pv_done[b]  tcgen05.commit        : O += P V_hat of tile j finished (P[b] free, O at rest)
//   q_full      256 softmax arrivals  : the query tile is in tensor memory
//   xch[q]      64 arrivals           : the two warps of lane quadrant q exchanged their half-row maxima

constexpr int kBM = 128;          // query rows per CTA
constexpr int kBN = 64;           // keys per tile
constexpr int kStages = 3;        // K_hat / V_hat ring depth
constexpr int kSoftmaxThreads = 256;
constexpr int kProducers = 256;
constexpr int kWsThreads = kSoftmaxThreads + kProducers + 32;
constexpr int kMmaWarp = kWsThreads / 32 - 1;

// Pair table: entry (i1 << B | i0) holds the bf16x2 word (C[i0], C[i1]).  Small tables of 4-byte
// entries keep random look-ups (nearly) free of bank conflicts; byte-indexed tables of 8- and
// 16-byte entries were measured slower.
template <int B>
__device__ __forceinline__ void fill_index_lut(uint32_t* lut, const float* __restrict__ cen, int tid, int nthreads) {
  for (int e = tid; e < (1 << (2 * B)); e += nthreads)
    lut[e] = tc::pack_bf16x2(cen[e & ((1 << B) - 1)], cen[e >> B]);
}
// Decode the B-bit indices of 8 consecutive coordinates (the low 8*B bits of `bits`) into 4 bf16x2 words.
template <int B>
__device__ __forceinline__ void decode_group(const uint32_t* lut, uint32_t bits, uint32_t (&out)[4]) {
#pragma unroll
  for (int q = 0; q < 4; ++q) out[q] = lut[(bits >> (2 * q * B)) & ((1u << (2 * B)) - 1)];
}

template <int D, int BITS>
struct WsSmem {
  static constexpr int G = D / 8, KB = BITS - 1, VB = BITS;
  static constexpr uint32_t kKStage = kBN * 2 * D * 2;
  static constexpr int DV = D + 16;                   // value coordinates + a 16-wide block whose first
                                                      // row is all ones: P V_hat then also yields the row sums
  static constexpr uint32_t kVStage = kBN * DV * 2;
  static constexpr uint32_t kIdxK = kBN * G * KB;     // packed key-index bytes per tile
  static constexpr uint32_t kSgn = kBN * G;
  static constexpr uint32_t kIdxV = kBN * G * VB;
  static constexpr uint32_t kPkStage = kIdxK + kSgn + kIdxV;
  static constexpr uint32_t kKOff = 0;
  static constexpr uint32_t kVOff = kKOff + kStages * kKStage;
  static constexpr uint32_t kPkOff = kVOff + kStages * kVStage;
  static constexpr uint32_t kTotal = kPkOff + kStages * kPkStage;
  static constexpr uint32_t kSboK = 2 * G * 128;        // K-major [keys, 2D]
  static constexpr uint32_t kSboV = 128;                // MN-major [D, kBN]: 8-coordinate chunks adjacent
  static constexpr uint32_t kLboV = (G + 2) * 128;      // ... 8-key groups G+2 core matrices apart
  // tensor-memory columns
  static constexpr uint32_t kColS = 0;                  // S[2]: 2 x 64
  static constexpr uint32_t kColO = 128;                // O: D value columns, then the row sum in column D
  static constexpr uint32_t kColQ = 128 + DV;           // Q_cat: 2D bf16 = D columns
  static constexpr uint32_t kColP = kColQ + D;          // P[2]: 2 x 32 (64 bf16 each)
  static constexpr uint32_t kCols = 512;
  static_assert(kColP + kBN <= kCols, "tensor memory over-subscribed");
};

template <int D, int BITS>
__global__ void __launch_bounds__(kWsThreads, 1) attention_ws_kernel(const AttnArgs a, __nv_bfloat16* __restrict__ o_rot) {
  using L = WsSmem<D, BITS>;
  constexpr int G = L::G, KB = L::KB, VB = L::VB, GP = G / 2;
  constexpr int HC = kBN / 2;     // score columns per softmax thread
  constexpr float kLog2e = 1.4426950408889634f;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // n_k * sm_scale * log2(e) per key column.  Written by the producers up to kStages tiles ahead of the score
  // MMA and read by the softmax warps up to two tiles behind it: 8 slots (tile & 7) can never collide.
  __shared__ float cscale[8][kBN];
  __shared__ float rho_s[kStages][kBN];   // rn_k / n_k
  __shared__ float nv_s[kStages][kBN];    // value norms
  __shared__ float xmax[2][2][kBM];       // [tile parity][column half][row]: half-row maxima exchanged
  __shared__ uint32_t lutK[1 << (2 * KB)];  // index pair -> bf16x2 centroids
  __shared__ uint32_t lutV[1 << (2 * VB)];
  __shared__ __align__(8) uint64_t bars[5 * kStages + 8 + 4 + 1];
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  volatile int* abort_flag = &s_abort;

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
  int k_end = (int)a.Sk;
  if (a.causal) k_end = min(k_end, min(q0 + kBM - 1, (int)a.Sq - 1) + shift + 1);
  const int n_tiles = (k_end + kBN - 1) / kBN;

  const uint32_t bar0 = tc::smem_u32(&bars[0]);
  auto k_full = [&](int i) { return bar0 + 8u * i; };
  auto v_full = [&](int i) { return bar0 + 8u * (kStages + i); };
  auto k_empty = [&](int i) { return bar0 + 8u * (2 * kStages + i); };
  auto v_empty = [&](int i) { return bar0 + 8u * (3 * kStages + i); };
  auto pk_full = [&](int i) { return bar0 + 8u * (4 * kStages + i); };
  auto s_full = [&](int i) { return bar0 + 8u * (5 * kStages + i); };
  auto s_empty = [&](int i) { return bar0 + 8u * (5 * kStages + 2 + i); };
  auto p_full = [&](int i) { return bar0 + 8u * (5 * kStages + 4 + i); };
  auto pv_done = [&](int i) { return bar0 + 8u * (5 * kStages + 6 + i); };
  auto xch = [&](int i) { return bar0 + 8u * (5 * kStages + 8 + i); };
  const uint32_t q_full = bar0 + 8u * (5 * kStages + 12);

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) {
      tc::mbar_init(k_full(i), kProducers);
      tc::mbar_init(v_full(i), kProducers);
      tc::mbar_init(k_empty(i), 1);
      tc::mbar_init(v_empty(i), 1);
      tc::mbar_init(pk_full(i), kProducers);
    }
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(s_full(i), 1);
      tc::mbar_init(s_empty(i), kSoftmaxThreads);
      tc::mbar_init(p_full(i), kSoftmaxThreads);
      tc::mbar_init(pv_done(i), 1);
    }
    for (int i = 0; i < 4; ++i) tc::mbar_init(xch(i), 64);
    tc::mbar_init(q_full, kSoftmaxThreads);
    tc::fence_mbar_init();
  }
  if (warp == kMmaWarp) tc::tmem_alloc(tc::smem_u32(&tmem_slot), L::kCols);
  fill_index_lut<KB>(lutK, a.cen_k, tid, kWsThreads);
  fill_index_lut<VB>(lutV, a.cen_v, tid, kWsThreads);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  const uint32_t tmem_o = tmem_base + L::kColO;
  bool ok = true;
  Tracer tr(g_trace_on != 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 &&
                (warp == 0 || warp == 8 || warp == kMmaWarp),
            warp == 0 ? 0 : warp == 8 ? 1 : 2);

  if (warp < 8) {
    // =============================== softmax warps ===============================
    const int quad = warp % 4, chalf = warp / 4;
    const int row = quad * 32 + lane;
    const int qi = q0 + row;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    {  // query row -> tensor memory: 2D bf16 = D columns, each of the row's two threads stores D/2
      const bool live = qi < a.Sq;
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.q_cat) +
                                                        (bh * a.Sq + qi) * 2 * D) + chalf * (D / 8);
#pragma unroll 1
      for (int c0 = 0; c0 < D / 2; c0 += 32) {
        uint32_t w[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint4 v = make_uint4(0, 0, 0, 0);
          if (live) v = src[c0 / 4 + i];
          w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
        }
        tc::tmem_st32(tmem_base + L::kColQ + lane_base + chalf * (D / 2) + c0, w);
      }
      tc::wait_st();
      tc::fence_before_sync();
      tc::mbar_arrive(q_full);
    }
    float m_run = -INFINITY;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int bb = j & 1, u = j >> 1, k0 = j * kBN;
      const int kc0 = k0 + chalf * HC;  // first key column of this thread
      tr.mark(0, j);
      if (!(ok = tc::mbar_wait_or_abort(s_full(bb), u & 1, abort_flag))) break;
      tc::fence_after_sync();
      tr.mark(1, j);
      float t[HC];
      {
        uint32_t raw[32];
        tc::tmem_ld32(tmem_base + L::kColS + lane_base + bb * kBN + chalf * HC, raw);
        tc::wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) t[c] = __uint_as_float(raw[c]);
      }
      tc::fence_before_sync();
      tc::mbar_arrive(s_empty(bb));
      tr.mark(2, j);
      float mx = -INFINITY;
      const bool edge = (k0 + kBN > a.Sk) || (a.causal && k0 + kBN - 1 > q0 + shift) || a.mask != nullptr;
      if (!edge) {
#pragma unroll
        for (int c4 = 0; c4 < HC; c4 += 4) {
          const float4 cs = *reinterpret_cast<const float4*>(&cscale[j & 7][chalf * HC + c4]);
          t[c4] *= cs.x; t[c4 + 1] *= cs.y; t[c4 + 2] *= cs.z; t[c4 + 3] *= cs.w;
          mx = fmaxf(mx, fmaxf(fmaxf(t[c4], t[c4 + 1]), fmaxf(t[c4 + 2], t[c4 + 3])));
        }
      } else {
        const float* mrow = (a.mask != nullptr && qi < a.Sq)
                                ? a.mask + b * a.mask_stride_b + (int64_t)qi * a.mask_stride_q + kc0
                                : nullptr;
#pragma unroll
        for (int c = 0; c < HC; ++c) {
          const int k = kc0 + c;
          float v = t[c] * cscale[j & 7][chalf * HC + c];
          if (mrow != nullptr && k < a.Sk) v = fmaf(mrow[c], kLog2e, v);
          if (k >= a.Sk || (a.causal && k > qi + shift)) v = -INFINITY;
          t[c] = v;
          mx = fmaxf(mx, v);
        }
      }
      // the other half of the row lives in the partner warp: swap maxima through shared memory
      // (slots alternate with the tile parity: a slot is rewritten two exchanges later, after the
      // partner has arrived at the exchange in between, i.e. after it has read this one)
      xmax[bb][chalf][row] = mx;
      tc::mbar_arrive(xch(quad));
      if (!(ok = tc::mbar_wait_or_abort(xch(quad), j & 1, abort_flag))) break;
      mx = fmaxf(mx, xmax[bb][1 - chalf][row]);
      // running max, raised lazily: rescaling O costs a tensor-memory round trip, so the max only
      // moves when some row of the quadrant outgrew it by more than 2^8 (P stays below 256)
      const float m_cand = fmaxf(m_run, mx);
      const bool grow = __any_sync(0xffffffffu, m_cand > m_run + 8.f);  // identical in both warps of the quadrant
      float alpha = 1.f;
      if (grow) {
        alpha = (m_run == -INFINITY) ? 0.f : tc::fast_exp2(m_run - m_cand);
        m_run = m_cand;
      }
      const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
      uint32_t pw[HC / 2];
#pragma unroll
      for (int c = 0; c < HC / 2; ++c)
        pw[c] = tc::pack_bf16x2(tc::fast_exp2(t[2 * c] - m_use), tc::fast_exp2(t[2 * c + 1] - m_use));
      tr.mark(3, j);
      if (u >= 1 && !(ok = tc::mbar_wait_or_abort(pv_done(bb), (u - 1) & 1, abort_flag))) break;  // P[bb] free
      tc::fence_after_sync();
      tr.mark(4, j);
      tc::tmem_st16(tmem_base + L::kColP + lane_base + bb * (kBN / 2) + chalf * (HC / 2), pw);
      if (grow && j >= 1) {
        // O must be at rest: wait for the previous tile's P V_hat; each half rescales D/2 columns
        if (!(ok = tc::mbar_wait_or_abort(pv_done((j - 1) & 1), ((j - 1) >> 1) & 1, abort_flag))) break;
        tc::fence_after_sync();
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
        if (chalf == 1) {  // the row-sum block rides along with the second half
          uint32_t raw[16];
          tc::tmem_ld16(tmem_o + lane_base + D, raw);
          tc::wait_ld();
#pragma unroll
          for (int c = 0; c < 16; ++c) raw[c] = __float_as_uint(__uint_as_float(raw[c]) * alpha);
          tc::tmem_st16(tmem_o + lane_base + D, raw);
        }
      }
      tc::wait_st();
      tc::fence_before_sync();
      tc::mbar_arrive(p_full(bb));
      tr.mark(5, j);
    }
    // ---- epilogue: normalise and store the rotated output row ----
    if (ok && n_tiles > 0)
      ok = tc::mbar_wait_or_abort(pv_done((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, abort_flag);
    if (ok) {
      tc::fence_after_sync();
      float l_tot;
      {  // column D of the accumulator is sum_k P[row][k] (the ones row of V_hat)
        uint32_t raw[16];
        tc::tmem_ld16(tmem_o + lane_base + D, raw);
        tc::wait_ld();
        l_tot = __uint_as_float(raw[0]);
      }
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
  } else if (warp < kMmaWarp) {
    // =============================== producer warps ===============================
    const int p = tid - kSoftmaxThreads;
    constexpr int UK = L::kIdxK / 8, US = L::kSgn / 8, UV = L::kIdxV / 8;  // 8-byte units per tile
    constexpr int NK = (UK + kProducers - 1) / kProducers, NV = (UV + kProducers - 1) / kProducers;
    constexpr int NI = (kBN * GP + kProducers - 1) / kProducers;  // (key, 16-coordinate) items per thread
    uint2 rk[NK], rv[NV], rs;
    uint32_t rn[3];
    const uint8_t* gk = a.key_idx + kv_base * (G * KB);
    const uint8_t* gs = a.key_sgn + kv_base * G;
    const uint8_t* gv = a.val_idx + kv_base * (G * VB);
    auto prefetch = [&](int k0) {
      const uint2 zero = make_uint2(0, 0);
#pragma unroll
      for (int i = 0; i < NK; ++i) {
        const int un = i * kProducers + p;
        rk[i] = (un < UK && k0 + (un * 8) / (G * KB) < a.Sk)
                    ? *reinterpret_cast<const uint2*>(gk + (int64_t)k0 * (G * KB) + un * 8) : zero;
      }
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int un = i * kProducers + p;
        rv[i] = (un < UV && k0 + (un * 8) / (G * VB) < a.Sk)
                    ? *reinterpret_cast<const uint2*>(gv + (int64_t)k0 * (G * VB) + un * 8) : zero;
      }
      rs = (p < US && k0 + (p * 8) / G < a.Sk) ? *reinterpret_cast<const uint2*>(gs + (int64_t)k0 * G + p * 8) : zero;
      if (p < kBN) {
        const bool live = k0 + p < a.Sk;
        rn[0] = live ? a.key_vn[kv_base + k0 + p] : 0;
        rn[1] = live ? a.key_rn[kv_base + k0 + p] : 0;
        rn[2] = live ? a.val_vn[kv_base + k0 + p] : 0;
      }
    };
    // item i of this thread: key and coordinate-pair group, fixed for the whole kernel
    int ikey[NI], igp[NI];
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int e = i * kProducers + p;
      ikey[i] = (e % 8) + 8 * (e / (8 * GP));
      igp[i] = (e / 8) % GP;
    }
    // constant part of every V_hat stage: coordinate row D is all ones (row sums), rows D+1..D+15 zero
    for (int e = p; e < kStages * kBN * 2; e += kProducers) {
      const int st = e / (kBN * 2), key = (e / 2) % kBN, blk = e % 2;
      *reinterpret_cast<uint4*>(smem_raw + L::kVOff + st * L::kVStage + (key / 8) * L::kLboV + (key % 8) * 16 +
                                (G + blk) * L::kSboV) = make_uint4(blk == 0 ? 0x00003F80u : 0u, 0u, 0u, 0u);
    }
    if (n_tiles > 0) prefetch(0);
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j % kStages, u = j / kStages;
      uint8_t* pk = smem_raw + L::kPkOff + st * L::kPkStage;
      // slot st (staged bytes, column scales, K_hat) is free once tile j-kStages' score MMA has drained;
      // its V_hat decode by this same thread is long finished
      tr.mark(0, j);
      if (u >= 1 && !(ok = tc::mbar_wait_or_abort(k_empty(st), (u - 1) & 1, abort_flag))) break;
      tr.mark(1, j);
#pragma unroll
      for (int i = 0; i < NK; ++i)
        if (i * kProducers + p < UK) *reinterpret_cast<uint2*>(pk + (i * kProducers + p) * 8) = rk[i];
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (i * kProducers + p < UV)
          *reinterpret_cast<uint2*>(pk + L::kIdxK + L::kSgn + (i * kProducers + p) * 8) = rv[i];
      if (p < US) *reinterpret_cast<uint2*>(pk + L::kIdxK + p * 8) = rs;
      if (p < kBN) {
        const float nk = fp16_value((uint16_t)rn[0]);
        cscale[j & 7][p] = nk * a.sm_scale * kLog2e;
        rho_s[st][p] = nk > 0.f ? fp16_value((uint16_t)rn[1]) / nk : 0.f;
        nv_s[st][p] = fp16_value((uint16_t)rn[2]);
      }
      // every producer's staged bytes must be visible before anyone decodes (a bounded wait
      // instead of bar.sync, so that a fault elsewhere cannot strand part of the group)
      tc::mbar_arrive(pk_full(st));
      if (!(ok = tc::mbar_wait_or_abort(pk_full(st), u & 1, abort_flag))) break;
      tr.mark(2, j);
      if (j + 1 < n_tiles) prefetch((j + 1) * kBN);  // in flight while this tile is decoded
      // ---- keys: centroid values and +-rho sign tile ----
      uint8_t* Kd = smem_raw + L::kKOff + st * L::kKStage;
      {
        uint32_t gw[NI][2], sb[NI], rr[NI];
#pragma unroll
        for (int i = 0; i < NI; ++i) {
          if (i * kProducers + p < kBN * GP) {
            const uint16_t* sk = reinterpret_cast<const uint16_t*>(pk + ikey[i] * (G * KB) + igp[i] * 2 * KB);
            uint64_t w = 0;
#pragma unroll
            for (int x = 0; x < KB; ++x) w |= (uint64_t)sk[x] << (16 * x);
            gw[i][0] = (uint32_t)w & ((1u << (8 * KB)) - 1);
            gw[i][1] = (uint32_t)(w >> (8 * KB));
            sb[i] = ~(uint32_t)*reinterpret_cast<const uint16_t*>(pk + L::kIdxK + ikey[i] * G + igp[i] * 2);
            const float rho = rho_s[st][ikey[i]];
            rr[i] = tc::pack_bf16x2(rho, rho);
          }
        }
#pragma unroll
        for (int i = 0; i < NI; ++i) {
          if (i * kProducers + p < kBN * GP) {
            uint8_t* kd = Kd + (ikey[i] / 8) * L::kSboK + (ikey[i] % 8) * 16;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              uint32_t kq[4];
              decode_group<KB>(lutK, gw[i][half], kq);
              uint32_t sq[4];
#pragma unroll
              for (int q = 0; q < 4; ++q)  // sign bit 0 -> bit 15, bit 1 -> bit 31 of the bf16x2 word
                sq[q] = rr[i] ^ ((((sb[i] >> (8 * half + 2 * q)) & 3u) * 0x40008000u) & 0x80008000u);
              const int g = 2 * igp[i] + half;
              *reinterpret_cast<uint4*>(kd + g * 128) = make_uint4(kq[0], kq[1], kq[2], kq[3]);
              *reinterpret_cast<uint4*>(kd + (G + g) * 128) = make_uint4(sq[0], sq[1], sq[2], sq[3]);
            }
          }
        }
      }
      tc::fence_async_smem();
      tc::mbar_arrive(k_full(st));
      tr.mark(3, j);
      // ---- values: V_hat[st] is free once tile j-kStages' P V_hat has drained ----
      if (u >= 1 && !(ok = tc::mbar_wait_or_abort(v_empty(st), (u - 1) & 1, abort_flag))) break;
      tr.mark(4, j);
      uint8_t* Vd = smem_raw + L::kVOff + st * L::kVStage;
      {
        uint32_t gw[NI][2];
        __nv_bfloat162 nv2[NI];
#pragma unroll
        for (int i = 0; i < NI; ++i) {
          if (i * kProducers + p < kBN * GP) {
            const uint16_t* sv =
                reinterpret_cast<const uint16_t*>(pk + L::kIdxK + L::kSgn + ikey[i] * (G * VB) + igp[i] * 2 * VB);
            uint64_t w = 0;
#pragma unroll
            for (int x = 0; x < VB; ++x) w |= (uint64_t)sv[x] << (16 * x);
            gw[i][0] = (uint32_t)w & (VB == 4 ? 0xffffffffu : ((1u << (8 * (VB & 3))) - 1));
            gw[i][1] = (uint32_t)(w >> (8 * VB));
            const float nvf = nv_s[st][ikey[i]];
            nv2[i] = __floats2bfloat162_rn(nvf, nvf);
          }
        }
#pragma unroll
        for (int i = 0; i < NI; ++i) {
          if (i * kProducers + p < kBN * GP) {
            uint8_t* vd = Vd + (ikey[i] / 8) * L::kLboV + (ikey[i] % 8) * 16;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              uint32_t vq[4];
              decode_group<VB>(lutV, gw[i][half], vq);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const __nv_bfloat162 prod = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&vq[q]), nv2[i]);
                vq[q] = *reinterpret_cast<const uint32_t*>(&prod);
              }
              *reinterpret_cast<uint4*>(vd + (2 * igp[i] + half) * L::kSboV) = make_uint4(vq[0], vq[1], vq[2], vq[3]);
            }
          }
        }
      }
      tc::fence_async_smem();
      tc::mbar_arrive(v_full(st));
      tr.mark(5, j);
    }
  } else if (lane == 0) {
    // =============================== MMA issuer ===============================
    constexpr uint32_t idesc_s = tc::idesc_bf16(kBM, kBN, false, false);
    constexpr uint32_t idesc_o = tc::idesc_bf16(kBM, L::DV, false, true);
    auto issue_scores = [&](int j) -> bool {
      const int bb = j & 1, u = j >> 1, st = j % kStages;
      tr.mark(0, j);
      if (!tc::mbar_wait_or_abort(k_full(st), (j / kStages) & 1, abort_flag)) return false;
      tr.mark(1, j);
      if (u >= 1 && !tc::mbar_wait_or_abort(s_empty(bb), (u - 1) & 1, abort_flag)) return false;
      tc::fence_after_sync();
      tr.mark(2, j);
      const uint64_t kdesc = tc::smem_desc(tc::smem_u32(smem_raw + L::kKOff + st * L::kKStage), 128, L::kSboK);
#pragma unroll
      for (int ks = 0; ks < 2 * D / 16; ++ks)
        tc::mma_bf16_ts(tmem_base + L::kColS + bb * kBN, tmem_base + L::kColQ + ks * 8,
                        kdesc + (uint64_t)(ks * 256 >> 4), idesc_s, ks > 0);
      tc::mma_commit(s_full(bb));
      tc::mma_commit(k_empty(st));
      tr.mark(3, j);
      return true;
    };
    ok = tc::mbar_wait_or_abort(q_full, 0, abort_flag);
    if (ok && n_tiles > 0) ok = issue_scores(0);
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int bb = j & 1, u = j >> 1, st = j % kStages;
      if (j + 1 < n_tiles && !(ok = issue_scores(j + 1))) break;
      tr.mark(4, j);
      if (!(ok = tc::mbar_wait_or_abort(v_full(st), (j / kStages) & 1, abort_flag))) break;
      if (!(ok = tc::mbar_wait_or_abort(p_full(bb), u & 1, abort_flag))) break;
      tc::fence_after_sync();
      tr.mark(5, j);
      const uint64_t vdesc = tc::smem_desc(tc::smem_u32(smem_raw + L::kVOff + st * L::kVStage), L::kLboV, L::kSboV);
#pragma unroll
      for (int ks = 0; ks < kBN / 16; ++ks)
        tc::mma_bf16_ts(tmem_o, tmem_base + L::kColP + bb * (kBN / 2) + ks * 8,
                        vdesc + (uint64_t)(ks * 2 * L::kLboV >> 4), idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
      tc::mma_commit(pv_done(bb));
      tc::mma_commit(v_empty(st));
      tr.mark(6, j);
    }
  }
  if (!ok && atomicExch(&s_abort, 2) != 2) record_fault();  // one fault per CTA
  tc::fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) tc::tmem_dealloc(tmem_base, L::kCols);
}

int trace_enable(int on) {
  const int v = on ? 1 : 0;
  static long long fill[2 * kTraceCap];
  for (int i = 0; i < 2 * kTraceCap; ++i) fill[i] = -1;
  TQ_CUDA_OK(cudaMemcpyToSymbol(g_trace, fill, sizeof(fill)));
  TQ_CUDA_OK(cudaMemcpyToSymbol(g_trace_on, &v, sizeof(v)));
  return TQ_OK;
}
int trace_read(long long* host_buf, int max_records, int* n_out) {
  // the buffer is copied whole; unused slots hold tag -1
  int n = kTraceCap < max_records ? kTraceCap : max_records;
  TQ_CUDA_OK(cudaDeviceSynchronize());
  TQ_CUDA_OK(cudaMemcpyFromSymbol(host_buf, g_trace, sizeof(long long) * 2 * n));
  *n_out = n;
  return TQ_OK;
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
  // every CTA takes all 512 tensor-memory columns, so keep it alone on its SM: ask for more than
  // half of the shared memory even when the tiles (d = 64) would need less
  constexpr size_t smem = WsSmem<D, BITS>::kTotal > 120 * 1024 ? WsSmem<D, BITS>::kTotal : 120 * 1024;
  auto kern = attention_ws_kernel<D, BITS>;
  TQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)((a.Sq + kBM - 1) / kBM), (unsigned)a.Hq, (unsigned)B);
  {
    ProfScope prof(kProfAttention, stream);
    kern<<<grid, kWsThreads, smem, stream>>>(a, o_rot);
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
