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
//              = < [q_rot | coeff q_s] , [ n_k C[idx_k] ; rn_k sgn_k ] >
// so one MMA over the concatenated contraction dimension of length 2d, with the norms folded into the
// decoded key operand, gives the raw score; the softmax only applies the constant sm_scale * log2(e).
//
// Every device-side wait is bounded; when one expires the kernel bumps a fault counter,
// frees its tensor memory and returns, and later launches return immediately.
#include <math.h>
#include <stdlib.h>

#include "tq_attention.cuh"
#include "tq_common.cuh"
#include "tq_rows.cuh"
#include "tq_simt.cuh"
#include "tq_tcgen05.cuh"

namespace tq {

__device__ unsigned long long g_wait_faults = 0ull;
// this device's slot of the host-visible status page (NULL until the first call on the device installs it)
__device__ unsigned long long* g_fault_mailbox_tc = nullptr;
int set_fault_mailbox_tc(unsigned long long* slot) {
  TQ_CUDA_OK(cudaMemcpyToSymbol(g_fault_mailbox_tc, &slot, sizeof(slot)));
  return TQ_OK;
}

int read_wait_faults(unsigned long long* out) {
  TQ_CUDA_OK(cudaMemcpyFromSymbol(out, g_wait_faults, sizeof(*out)));
  return TQ_OK;
}

// Diagnostics: stage timestamps (SM clock) of one CTA of the attention kernel, see tq_trace_read.
constexpr int kTraceCap = 4096;
static int g_trace_host_on = 0;  // selects the tracing build of the attention kernel at launch
__device__ long long g_trace[2 * kTraceCap];
// One tracer per traced thread: role r appends to its own third of the buffer, no atomics.  The tracing
// build of the kernel (TRACE = true) is launched only while tracing is enabled; in the production build
// every mark compiles to nothing.
template <bool TRACE>
struct Tracer {
  bool on;
  int role, n;
  __device__ Tracer(bool on_, int role_) : on(TRACE && on_), role(role_), n(0) {}
  __device__ __forceinline__ void mark(int ev, int tile) {
    if (!TRACE) return;
    if (!on || n >= kTraceCap / 3) return;
    const int i = role * (kTraceCap / 3) + n++;
    g_trace[2 * i] = ((long long)role << 32) | ((long long)ev << 16) | (long long)tile;
    g_trace[2 * i + 1] = clock64();
  }
};

__device__ __forceinline__ bool poisoned() {
  return *reinterpret_cast<volatile unsigned long long*>(&g_wait_faults) != 0ull;
}
__device__ __forceinline__ void record_fault() {
  atomicAdd(&g_wait_faults, 1ull);
  notify_host_of_fault(g_fault_mailbox_tc);
}

// ---- constant operand builder ------------------------------------------------------------
// w_cat [2d, d] bf16 = [ Pi ; coeff * S ] with S = S_eff * Pi, so that q * w_cat^T = [q_rot | coeff q_s];
// w_unrot [d, d] bf16 = Pi_v^T, so that o_rot * w_unrot^T = o_rot * Pi_v.
// `tile_rows` = 0 stores them row-major.  Otherwise every block of `tile_rows` rows is stored as the
// K-major operand image a CTA wants in shared memory (8-row groups d*16 bytes apart, 16-byte chunks of a
// group 128 bytes apart), so that one contiguous bulk copy brings a block in.
__device__ __forceinline__ int operand_index(int row, int col, int d, int tile_rows) {
  if (tile_rows == 0) return row * d + col;
  const int r = row % tile_rows;
  return (row / tile_rows) * tile_rows * d + (r / 8) * (d * 8) + (col / 8) * 64 + (r % 8) * 8 + col % 8;
}
__global__ void build_wcat_kernel(const float* __restrict__ Pi, const float* __restrict__ S_eff, int d, float coeff,
                                  __nv_bfloat16* __restrict__ w_cat, int tile_rows) {
  const int j = blockIdx.x, i = threadIdx.x;  // one block per row, d threads
  w_cat[operand_index(j, i, d, tile_rows)] = __float2bfloat16_rn(Pi[j * d + i]);
  float acc = 0.f;
  for (int c = 0; c < d; ++c) acc = fmaf(S_eff[j * d + c], Pi[c * d + i], acc);
  w_cat[operand_index(d + j, i, d, tile_rows)] = __float2bfloat16_rn(coeff * acc);
}
__global__ void build_wunrot_kernel(const float* __restrict__ Pi_v, int d, __nv_bfloat16* __restrict__ w_unrot,
                                    int tile_rows) {
  const int j = blockIdx.x, i = threadIdx.x;
  w_unrot[operand_index(j, i, d, tile_rows)] = __float2bfloat16_rn(Pi_v[i * d + j]);
}

// Pair tables of the SM-pair kernel: entry (i1 << B | i0) = bf16x2 (C[i0], C[i1]); 4^(bits-1) key entries
// followed by 4^bits value entries, so that the kernel can bulk-copy them into shared memory.
__global__ void build_luts_kernel(const float* __restrict__ cen_k, const float* __restrict__ cen_v, int kb, int vb,
                                  uint32_t* __restrict__ luts) {
  const int nk = 1 << (2 * kb), nv = 1 << (2 * vb);
  for (int e = threadIdx.x; e < nk + nv; e += blockDim.x) {
    const float* cen = e < nk ? cen_k : cen_v;
    const int b = e < nk ? kb : vb, i = e < nk ? e : e - nk;
    luts[e] = tc::pack_f16x2(cen[i & ((1 << b) - 1)], cen[i >> b]);
  }
}

// Canonical K-major operand image of a row-major fp32 [d, d] matrix, split into bf16 hi = bf16(m) and
// lo = bf16(m - hi): what the compression kernel's MMAs take as B operands (x (hi + lo)^T carries ~16 mantissa bits).
__global__ void build_split_image_kernel(const float* __restrict__ M, int d, __nv_bfloat16* __restrict__ hi,
                                         __nv_bfloat16* __restrict__ lo) {
  const int j = blockIdx.x, i = threadIdx.x;
  const float v = M[j * d + i];
  const __nv_bfloat16 h = __float2bfloat16_rn(v);
  const int at = operand_index(j, i, d, d);
  hi[at] = h;
  lo[at] = __float2bfloat16_rn(v - __bfloat162float(h));
}
__global__ void copy_floats_kernel(const float* __restrict__ src, float* __restrict__ dst, int n) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) dst[i] = src[i];
}
__global__ void write_header_kernel(uint32_t* hdr, int d, int bits) {
  hdr[0] = kConstMagic;
  hdr[1] = (uint32_t)d;
  hdr[2] = (uint32_t)bits;
}

int prepare_constants(const float* Pi_k, const float* S_eff, const float* cen_k, const float* bnd_k, const float* Pi_v,
                      const float* cen_v, const float* bnd_v, int bits, int d, void* constants, cudaStream_t stream) {
  const ConstLayout L = const_layout(d);
  uint8_t* c = static_cast<uint8_t*>(constants);
  auto f32 = [&](size_t off) { return reinterpret_cast<float*>(c + off); };
  auto b16 = [&](size_t off) { return reinterpret_cast<__nv_bfloat16*>(c + off); };
  const int kb = bits - 1, vb = bits;
  const struct { const float* src; size_t off; int n; } copies[] = {
      {Pi_k, L.pi_k, d * d}, {S_eff, L.s_eff, d * d}, {Pi_v, L.pi_v, d * d}, {cen_k, L.cen_k, 1 << kb},
      {bnd_k, L.bnd_k, (1 << kb) - 1}, {cen_v, L.cen_v, 1 << vb}, {bnd_v, L.bnd_v, (1 << vb) - 1}};
  for (const auto& cp : copies) {
    copy_floats_kernel<<<cp.n >= 4096 ? 16 : 1, 256, 0, stream>>>(cp.src, f32(cp.off), cp.n);
    TQ_CUDA_OK(cudaGetLastError());
  }
  const float coeff = sqrtf(1.5707963267948966f) / (float)d;
  build_wcat_kernel<<<d, d, 0, stream>>>(Pi_k, S_eff, d, coeff, b16(L.w_cat_pair), d);
  build_wcat_kernel<<<d, d, 0, stream>>>(Pi_k, S_eff, d, coeff, b16(L.w_cat_plain), 0);
  build_wunrot_kernel<<<d, d, 0, stream>>>(Pi_v, d, b16(L.w_unrot_pair), d / 2);
  build_wunrot_kernel<<<d, d, 0, stream>>>(Pi_v, d, b16(L.w_unrot_plain), 0);
  build_luts_kernel<<<1, 128, 0, stream>>>(cen_k, cen_v, kb, vb, reinterpret_cast<uint32_t*>(c + L.luts));
  build_split_image_kernel<<<d, d, 0, stream>>>(Pi_k, d, b16(L.pik_hi), b16(L.pik_lo));
  build_split_image_kernel<<<d, d, 0, stream>>>(S_eff, d, b16(L.se_hi), b16(L.se_lo));
  build_split_image_kernel<<<d, d, 0, stream>>>(Pi_v, d, b16(L.piv_hi), b16(L.piv_lo));
  write_header_kernel<<<1, 1, 0, stream>>>(reinterpret_cast<uint32_t*>(c + L.header), d, bits);
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
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

// ---- fused attention (warp-specialised, two query tiles per CTA) --------------------------------
//
// One CTA owns TWO query tiles of 128 rows that read the same KV head -- two query heads of one GQA
// group at the same positions, or (when the group size is odd) two consecutive position blocks of
// one head -- so that every decoded K_hat / V_hat tile feeds 256 query rows.  Decoding is CUDA-core
// work and the scarcest resource here; sharing it halves its cost per MMA.
//
// Seventeen warps in three roles, coupled only by mbarriers with bounded waits:
//   warps 0-3 / 4-7  softmax of tile A / B: thread r owns query row r (= tensor-memory lane r).  Load
//                    the 64 scores of the key tile, scale, mask, running max (raised lazily) and sum,
//                    write P (bf16) over the score columns, rescale O when the max grew, epilogue.
//   warps 8-15       producers: prefetch the next key tile's packed bytes into registers, stage them
//                    in shared memory, decode indices / sign bits / norms into the K_hat and V_hat
//                    operand tiles (canonical core-matrix layout), up to kStages tiles ahead.
//   warp 16          MMA: one thread issues, per key tile, S_t = Q_t K_hat^T and O_t += P_t V_hat for
//                    both tiles, interleaved so that the tensor pipe works for one tile while the
//                    other tile's softmax runs (ping-pong).
// Tensor memory (512 columns at d = 128, all of it): rotated queries of A and B (2 x d/2 columns of
// bf16 pairs, A operand of the first half of the score contraction), scores S_A, S_B (2 x 64 fp32
// columns; P_t overwrites the first 32 columns of S_t as packed bf16 and is the A operand of P V_hat),
// outputs O_A, O_B (2 x d fp32 columns).  The sketch half of the queries (q S^T) does not fit in tensor
// memory any more and is an A operand in shared memory.
//
// Barriers (phase = key tile index, or use count of the ring slot):
//   pk_full[2]  256 producer arrivals : packed bytes of tile j staged          (slot j & 1)
//   k_full[s]   256 producer arrivals : K_hat and column scales of tile j ready (slot j % kStages)
//   v_full[s]   256 producer arrivals : V_hat of tile j ready
//   k_empty[s]  tcgen05.commit        : both score MMAs of tile j have consumed K_hat[s]
//   v_empty[s]  tcgen05.commit        : both P V_hat MMAs of tile j have consumed V_hat[s]
//   s_full[t]   tcgen05.commit        : S_t holds the scores of key tile j
//   p_full[t]   128 softmax arrivals  : P_t written (and O_t rescaled if needed)
//   pv_done[t]  tcgen05.commit        : O_t += P_t V_hat of key tile j finished
//   q_full      256 softmax arrivals  : both query tiles are in tensor / shared memory

constexpr int kBM = 128;          // query rows per tile (two tiles per CTA)
constexpr int kBN = 64;           // keys per tile
constexpr int kProducers = 256;
constexpr int kWsThreads = 256 + kProducers + 32;
constexpr int kMmaWarp = kWsThreads / 32 - 1;

// Pair table: entry (i1 << B | i0) holds the bf16x2 word (C[i0], C[i1]).  Small tables of 4-byte
// entries keep random look-ups (nearly) free of bank conflicts; byte-indexed tables of 8- and
// 16-byte entries were measured slower.
template <int B>
__device__ __forceinline__ void fill_index_lut(uint32_t* lut, const float* __restrict__ cen, int tid, int nthreads) {
  for (int e = tid; e < (1 << (2 * B)); e += nthreads)
    lut[e] = tc::pack_f16x2(cen[e & ((1 << B) - 1)], cen[e >> B]);
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
  static constexpr int kStages = BITS == 4 ? 2 : 3;    // K_hat / V_hat ring depth (shared memory permitting)
  static constexpr uint32_t kQsBytes = kBM * D * 2;    // sketch half of one query tile, K-major
  static constexpr uint32_t kKStage = kBN * 2 * D * 2;
  static constexpr uint32_t kVStage = kBN * D * 2;
  static constexpr uint32_t kIdxK = kBN * G * KB;      // packed key-index bytes per tile
  static constexpr uint32_t kSgn = kBN * G;
  static constexpr uint32_t kIdxV = kBN * G * VB;
  static constexpr uint32_t kPkStage = kIdxK + kSgn + kIdxV;
  static constexpr uint32_t kQsOff = 0;
  static constexpr uint32_t kKOff = kQsOff + 2 * kQsBytes;
  static constexpr uint32_t kVOff = kKOff + kStages * kKStage;
  static constexpr uint32_t kPkOff = kVOff + kStages * kVStage;
  static constexpr uint32_t kTotal = kPkOff + 2 * kPkStage;
  static constexpr uint32_t kSboQs = G * 128;           // K-major [rows, D]
  static constexpr uint32_t kSboK = 2 * G * 128;        // K-major [keys, 2D]
  static constexpr uint32_t kSboV = 128;                // MN-major [D, kBN]: 8-coordinate chunks adjacent
  static constexpr uint32_t kLboV = G * 128;            // ... 8-key groups G core matrices apart
  // tensor-memory columns
  static constexpr uint32_t kColQ = 0;                  // rotated queries: 2 x D/2
  static constexpr uint32_t kColS = D;                  // S_A, S_B: 2 x 64 (P_t aliases the first 32 of S_t)
  static constexpr uint32_t kColO = D + 2 * kBN;        // O_A, O_B: 2 x D
  static constexpr uint32_t kCols = 512;
  static_assert(kColO + 2 * D <= kCols, "tensor memory over-subscribed");
};

template <int D, int BITS, bool TRACE>
__global__ void __launch_bounds__(kWsThreads, 1)
attention_ws_kernel(const AttnArgs a, __nv_bfloat16* __restrict__ o_rot, const int pair_heads) {
  using L = WsSmem<D, BITS>;
  constexpr int G = L::G, KB = L::KB, VB = L::VB, GP = G / 2, kStages = L::kStages;
  constexpr float kLog2e = 1.4426950408889634f;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // norms as stored (fp16 bit patterns), duplicated into both halves of a word: the multiplier of a packed pair
  __shared__ uint32_t nk_s[2][kBN];       // key norms            (producer-internal, slot j & 1)
  __shared__ uint32_t rho_s[2][kBN];      // key residual norms
  __shared__ uint32_t nv_s[2][kBN];       // value norms
  __shared__ uint32_t lutK[1 << (2 * KB)];  // index pair -> bf16x2 centroids
  __shared__ uint32_t lutV[1 << (2 * VB)];
  __shared__ __align__(8) uint64_t bars[4 * kStages + 2 + 6 + 1];
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  volatile int* abort_flag = &s_abort;

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  if (tid == 0) s_abort = poisoned() ? 1 : 0;
  __syncthreads();
  if (s_abort) return;  // an earlier bounded wait expired: do nothing rather than risk another

  // ---- which two query tiles -------------------------------------------------------------
  const int64_t b = blockIdx.z;
  const int xblk = (int)(gridDim.x - 1 - blockIdx.x);  // heaviest (latest) position blocks first
  int64_t head[2];
  int q0[2];
  if (pair_heads) {
    head[0] = 2 * (int64_t)blockIdx.y; head[1] = head[0] + 1;
    q0[0] = q0[1] = xblk * kBM;
  } else {
    head[0] = head[1] = blockIdx.y;
    q0[0] = 2 * xblk * kBM; q0[1] = q0[0] + kBM;
  }
  const int64_t kv_base = (b * a.Hkv + head[0] / (a.Hq / a.Hkv)) * a.Sk;
  const int shift = (int)(a.Sk - a.Sq);
  int k_end = (int)a.Sk;
  if (a.causal) k_end = min(k_end, min(q0[1] + kBM - 1, (int)a.Sq - 1) + shift + 1);
  const int n_tiles = (k_end + kBN - 1) / kBN;

  const uint32_t bar0 = tc::smem_u32(&bars[0]);
  auto k_full = [&](int i) { return bar0 + 8u * i; };
  auto v_full = [&](int i) { return bar0 + 8u * (kStages + i); };
  auto k_empty = [&](int i) { return bar0 + 8u * (2 * kStages + i); };
  auto v_empty = [&](int i) { return bar0 + 8u * (3 * kStages + i); };
  auto pk_full = [&](int i) { return bar0 + 8u * (4 * kStages + i); };
  auto s_full = [&](int i) { return bar0 + 8u * (4 * kStages + 2 + i); };
  auto p_full = [&](int i) { return bar0 + 8u * (4 * kStages + 4 + i); };
  auto pv_done = [&](int i) { return bar0 + 8u * (4 * kStages + 6 + i); };
  const uint32_t q_full = bar0 + 8u * (4 * kStages + 8);

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) {
      tc::mbar_init(k_full(i), kProducers);
      tc::mbar_init(v_full(i), kProducers);
      tc::mbar_init(k_empty(i), 1);
      tc::mbar_init(v_empty(i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(pk_full(i), kProducers);
      tc::mbar_init(s_full(i), 1);
      tc::mbar_init(p_full(i), kBM);
      tc::mbar_init(pv_done(i), 1);
    }
    tc::mbar_init(q_full, 2 * kBM);
    tc::fence_mbar_init();
  }
  if (warp == kMmaWarp) tc::tmem_alloc(tc::smem_u32(&tmem_slot), L::kCols);
  fill_index_lut<KB>(lutK, a.cen_k, tid, kWsThreads);
  fill_index_lut<VB>(lutV, a.cen_v, tid, kWsThreads);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  bool ok = true;
  Tracer<TRACE> tr(blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 &&
                (warp == 0 || warp == 8 || warp == kMmaWarp),
            warp == 0 ? 0 : warp == 8 ? 1 : 2);

  if (warp < 8) {
    // =============================== softmax warps ===============================
    const int tl = warp / 4;                    // query tile of this warp
    const int row = (warp % 4) * 32 + lane;
    const int qi = q0[tl] + row;
    const int64_t qrow = (b * a.Hq + head[tl]) * a.Sq + qi;
    const uint32_t lane_base = (uint32_t)((warp % 4) * 32) << 16;
    const uint32_t tmem_s = tmem_base + L::kColS + tl * kBN;
    const uint32_t tmem_o = tmem_base + L::kColO + tl * D;
    {  // query row: rotated half (D bf16 = D/2 columns) -> tensor memory, sketch half -> shared memory
      const bool live = qi < a.Sq;
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.q_cat) + qrow * 2 * D);
#pragma unroll 1
      for (int c0 = 0; c0 < D / 2; c0 += 32) {
        uint32_t w[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint4 v = make_uint4(0, 0, 0, 0);
          if (live) v = src[c0 / 4 + i];
          w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
        }
        tc::tmem_st32(tmem_base + L::kColQ + tl * (D / 2) + lane_base + c0, w);
      }
      uint8_t* dst = smem_raw + L::kQsOff + tl * L::kQsBytes + (row / 8) * L::kSboQs + (row % 8) * 16;
#pragma unroll 8
      for (int c = 0; c < G; ++c) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (live) v = src[G + c];
        *reinterpret_cast<uint4*>(dst + c * 128) = v;
      }
      tc::wait_st();
      tc::fence_async_smem();
      tc::fence_before_sync();
      tc::mbar_arrive(q_full);
    }
    float m_run = -INFINITY, l_run = 0.f;
    const float cexp = a.sm_scale * kLog2e, rcexp = 1.f / cexp;  // K_hat carries the key norms: S is the raw score
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int k0 = j * kBN;
      tr.mark(0, j);
      if (!(ok = tc::mbar_wait_or_abort(s_full(tl), j & 1, abort_flag))) break;
      tc::fence_after_sync();
      tr.mark(1, j);
      float t[kBN];
      {
        uint32_t raw[32];
        tc::tmem_ld32(tmem_s + lane_base, raw);
        tc::wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) t[c] = __uint_as_float(raw[c]);
        tc::tmem_ld32(tmem_s + lane_base + 32, raw);
        tc::wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) t[32 + c] = __uint_as_float(raw[c]);
      }
      tr.mark(2, j);
      float mx = -INFINITY;
      const bool edge = (k0 + kBN > a.Sk) || (a.causal && k0 + kBN - 1 > q0[tl] + shift) || a.mask != nullptr;
      if (!edge) {
        // raw scores: the positive constant sm_scale*log2(e) is applied to the maximum and inside the exp2
#pragma unroll
        for (int c4 = 0; c4 < kBN; c4 += 4)
          mx = fmaxf(mx, fmaxf(fmaxf(t[c4], t[c4 + 1]), fmaxf(t[c4 + 2], t[c4 + 3])));
        mx *= cexp;
      } else {
        const float* mrow = (a.mask != nullptr && qi < a.Sq)
                                ? a.mask + b * a.mask_stride_b + (int64_t)qi * a.mask_stride_q + k0
                                : nullptr;
#pragma unroll
        for (int c = 0; c < kBN; ++c) {
          const int k = k0 + c;
          float v = t[c] * cexp;
          // The large negative value HF masks with is clamped to -60000 (log2 units: exp2 of it is still exactly 0
          // beside any real score) so that it stays finite and small enough for the raw-unit round trip below to be
          // accurate: a row whose visible keys are all masked then averages them uniformly, as a softmax over equal
          // finite scores does in the reference, instead of coming out as zeros.
          if (mrow != nullptr && k < a.Sk) v = fmaxf(fmaf(mrow[c], kLog2e, v), -60000.f);
          if (k >= a.Sk || (a.causal && k > qi + shift)) v = -INFINITY;
          t[c] = v * rcexp;  // back to raw units: the exp2 below rescales (-inf stays -inf)
          mx = fmaxf(mx, v);
        }
      }
      // running max, raised lazily: rescaling O costs a tensor-memory round trip, so the max only
      // moves when some row of the warp outgrew it by more than 2^8 (P stays below 256)
      const float m_cand = fmaxf(m_run, mx);
      const bool grow = __any_sync(0xffffffffu, m_cand > m_run + 8.f);
      float alpha = 1.f;
      if (grow) {
        alpha = (m_run == -INFINITY) ? 0.f : tc::fast_exp2(m_run - m_cand);
        m_run = m_cand;
      }
      const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
      // P (packed bf16) goes over the first 32 score columns; this row's scores are all in registers
      float psum = 0.f;
#pragma unroll
      for (int hblk = 0; hblk < 2; ++hblk) {
        uint32_t pw[16];
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const float p0 = tc::fast_exp2(fmaf(t[32 * hblk + 2 * c], cexp, -m_use));
          const float p1 = tc::fast_exp2(fmaf(t[32 * hblk + 2 * c + 1], cexp, -m_use));
          psum += p0 + p1;
          pw[c] = tc::pack_f16x2(p0, p1);
        }
        tc::tmem_st16(tmem_s + lane_base + 16 * hblk, pw);
      }
      l_run = l_run * alpha + psum;
      tr.mark(3, j);
      if (grow && j >= 1) {
        // O_t must be at rest: wait for the previous key tile's P V_hat
        if (!(ok = tc::mbar_wait_or_abort(pv_done(tl), (j - 1) & 1, abort_flag))) break;
        tc::fence_after_sync();
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t raw[32];
          tc::tmem_ld32(tmem_o + lane_base + c0, raw);
          tc::wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) raw[c] = __float_as_uint(__uint_as_float(raw[c]) * alpha);
          tc::tmem_st32(tmem_o + lane_base + c0, raw);
        }
      }
      tc::wait_st();
      tc::fence_before_sync();
      tc::mbar_arrive(p_full(tl));
      tr.mark(4, j);
    }
    // ---- epilogue: normalise and store the rotated output row ----
    if (ok && n_tiles > 0) ok = tc::mbar_wait_or_abort(pv_done(tl), (n_tiles - 1) & 1, abort_flag);
    if (ok) {
      tc::fence_after_sync();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* dst = o_rot + qrow * D;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t raw[32];
        tc::tmem_ld32(tmem_o + lane_base + c0, raw);
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
    const int p = tid - 256;
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
    if (n_tiles > 0) prefetch(0);
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j % kStages, u = j / kStages, ps = j & 1;
      uint8_t* pk = smem_raw + L::kPkOff + ps * L::kPkStage;
      tr.mark(0, j);
      // staging slot ps was last read by this group's decode of tile j-2 (ordered by pk_full of tile j-1)
#pragma unroll
      for (int i = 0; i < NK; ++i)
        if (i * kProducers + p < UK) *reinterpret_cast<uint2*>(pk + (i * kProducers + p) * 8) = rk[i];
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (i * kProducers + p < UV)
          *reinterpret_cast<uint2*>(pk + L::kIdxK + L::kSgn + (i * kProducers + p) * 8) = rv[i];
      if (p < US) *reinterpret_cast<uint2*>(pk + L::kIdxK + p * 8) = rs;
      if (p < kBN) {
        nk_s[ps][p] = (rn[0] & 0xffffu) * 0x10001u;
        rho_s[ps][p] = (rn[1] & 0xffffu) * 0x10001u;
        nv_s[ps][p] = (rn[2] & 0xffffu) * 0x10001u;
      }
      // every producer's staged bytes must be visible before anyone decodes (a bounded wait
      // instead of bar.sync, so that a fault elsewhere cannot strand part of the group)
      tc::mbar_arrive(pk_full(ps));
      if (!(ok = tc::mbar_wait_or_abort(pk_full(ps), (j >> 1) & 1, abort_flag))) break;
      tr.mark(1, j);
      if (j + 1 < n_tiles) prefetch((j + 1) * kBN);  // in flight while this tile is decoded
      // K_hat[st] is free once both score MMAs of tile j-kStages have drained
      if (u >= 1 && !(ok = tc::mbar_wait_or_abort(k_empty(st), (u - 1) & 1, abort_flag))) break;
      tr.mark(2, j);
      // ---- keys: centroid values and +-rho sign tile ----
      uint8_t* Kd = smem_raw + L::kKOff + st * L::kKStage;
      {
        uint32_t gw[NI][2], sb[NI], rr[NI], nk2[NI];
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
            rr[i] = rho_s[ps][ikey[i]];
            nk2[i] = nk_s[ps][ikey[i]];
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
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                kq[q] = tc::mul_f16x2(kq[q], nk2[i]);
              }
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
      // ---- values: V_hat[st] is free once both P V_hat MMAs of tile j-kStages have drained ----
      if (u >= 1 && !(ok = tc::mbar_wait_or_abort(v_empty(st), (u - 1) & 1, abort_flag))) break;
      tr.mark(4, j);
      uint8_t* Vd = smem_raw + L::kVOff + st * L::kVStage;
      {
        uint32_t gw[NI][2], nv2[NI];
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
            nv2[i] = nv_s[ps][ikey[i]];
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
                vq[q] = tc::mul_f16x2(vq[q], nv2[i]);
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
    // fp16 operands for the score and P V_hat contractions: the stored fp16 norms enter the decoded operands
    // exactly and the products round a factor 8 finer than bf16
    constexpr uint32_t idesc_s = tc::idesc_f16(kBM, kBN, false, false);
    constexpr uint32_t idesc_o = tc::idesc_f16(kBM, D, false, true);
    // S_t = q_rot_t K_hat[:, :D]^T (A in tensor memory) + q_s_t K_hat[:, D:]^T (A in shared memory)
    auto issue_scores = [&](int tl, int j) {
      const int st = j % kStages;
      const uint32_t d_s = tmem_base + L::kColS + tl * kBN;
      const uint64_t kdesc = tc::smem_desc(tc::smem_u32(smem_raw + L::kKOff + st * L::kKStage), 128, L::kSboK);
      const uint64_t qsdesc = tc::smem_desc(tc::smem_u32(smem_raw + L::kQsOff + tl * L::kQsBytes), 128, L::kSboQs);
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks)
        tc::mma_bf16_ts(d_s, tmem_base + L::kColQ + tl * (D / 2) + ks * 8, kdesc + (uint64_t)(ks * 256 >> 4), idesc_s,
                        ks > 0);
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks)
        tc::mma_bf16(d_s, qsdesc + (uint64_t)(ks * 256 >> 4), kdesc + (uint64_t)((D / 16 + ks) * 256 >> 4), idesc_s,
                     1u);
      tc::mma_commit(s_full(tl));
    };
    auto issue_pv = [&](int tl, int j) {
      const int st = j % kStages;
      const uint64_t vdesc = tc::smem_desc(tc::smem_u32(smem_raw + L::kVOff + st * L::kVStage), L::kLboV, L::kSboV);
#pragma unroll
      for (int ks = 0; ks < kBN / 16; ++ks)
        tc::mma_bf16_ts(tmem_base + L::kColO + tl * D, tmem_base + L::kColS + tl * kBN + ks * 8,
                        vdesc + (uint64_t)(ks * 2 * L::kLboV >> 4), idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
      tc::mma_commit(pv_done(tl));
    };
    ok = tc::mbar_wait_or_abort(q_full, 0, abort_flag);
    if (ok && n_tiles > 0) {
      tr.mark(0, 0);
      ok = tc::mbar_wait_or_abort(k_full(0), 0, abort_flag);
      if (ok) {
        tc::fence_after_sync();
        issue_scores(0, 0);
        issue_scores(1, 0);
        tc::mma_commit(k_empty(0));
      }
    }
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j % kStages, u = j / kStages;
      const bool more = j + 1 < n_tiles;
      const int st1 = (j + 1) % kStages;
      tr.mark(1, j);
      if (!(ok = tc::mbar_wait_or_abort(v_full(st), u & 1, abort_flag))) break;
      if (!(ok = tc::mbar_wait_or_abort(p_full(0), j & 1, abort_flag))) break;
      tc::fence_after_sync();
      tr.mark(2, j);
      issue_pv(0, j);
      if (more) {
        if (!(ok = tc::mbar_wait_or_abort(k_full(st1), ((j + 1) / kStages) & 1, abort_flag))) break;
        tc::fence_after_sync();
        issue_scores(0, j + 1);  // overwrites S_A / P_A: ordered after issue_pv(0, j) on the tensor pipe
      }
      tr.mark(3, j);
      if (!(ok = tc::mbar_wait_or_abort(p_full(1), j & 1, abort_flag))) break;
      tc::fence_after_sync();
      tr.mark(4, j);
      issue_pv(1, j);
      tc::mma_commit(v_empty(st));
      if (more) {
        issue_scores(1, j + 1);
        tc::mma_commit(k_empty(st1));
      }
      tr.mark(5, j);
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
  g_trace_host_on = v;
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
#ifdef TQ_B200_TRACE  // diagnostics build only: the product library carries one instantiation per (d, bits)
  auto kern = g_trace_host_on ? attention_ws_kernel<D, BITS, true> : attention_ws_kernel<D, BITS, false>;
#else
  auto kern = attention_ws_kernel<D, BITS, false>;
#endif
  TQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  // two query tiles per CTA: two heads of one GQA group when the group size is even, otherwise
  // two consecutive position blocks of one head
  const int pair_heads = ((a.Hq / a.Hkv) % 2 == 0) ? 1 : 0;
  const int64_t blocks = (a.Sq + kBM - 1) / kBM;
  dim3 grid((unsigned)(pair_heads ? blocks : (blocks + 1) / 2), (unsigned)(pair_heads ? a.Hq / 2 : a.Hq), (unsigned)B);
  {
    ProfScope prof(kProfAttention, stream);
    kern<<<grid, kWsThreads, smem, stream>>>(a, o_rot, pair_heads);
  }
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
}

static inline size_t round256(size_t v) { return (v + 255) & ~(size_t)255; }

// workspace layout (bf16 mode): [ w_cat | w_unrot | decode tables | q_cat | o_rot | partial results of the
// split-KV kernel ]
constexpr size_t kLutBytes = 2048;  // (4^3 + 4^4) words at most
size_t workspace_bytes_bf16(int64_t BHq, int64_t Sq, int d) {
  const int64_t n_q = BHq * Sq;
  return round256((size_t)2 * d * d * 2) + round256((size_t)d * d * 2) + kLutBytes + round256((size_t)n_q * 2 * d * 2) +
         round256((size_t)n_q * d * 2) + (Sq <= 16 ? decode_workspace_bytes(BHq) : 0);
}

// q_cat bf16 [n, 2d] = [ q Pi^T | coeff * q S^T ] on the tensor cores; `w_cat` is 2*d*d bf16 of scratch.
int prepare_queries_bf16(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d, int64_t sb, int64_t sh,
                         int64_t ss, const float* Pi_k, const float* S_eff, void* w_cat_scratch, void* q_cat,
                         cudaStream_t stream, int q_cat_dtype) {
  const int64_t n_q = B * Hq * Sq;
  ProfScope prof(kProfPrepareQueries, stream);
  __nv_bfloat16* w_cat = static_cast<__nv_bfloat16*>(w_cat_scratch);
  if (Pi_k != nullptr) {  // NULL: `w_cat_scratch` already holds the row-major operand (a prepared constants buffer)
    build_wcat_kernel<<<d, d, 0, stream>>>(Pi_k, S_eff, d, sqrtf(1.5707963267948966f) / (float)d, w_cat, 0);
    TQ_CUDA_OK(cudaGetLastError());
  }
  const int tiles = (int)((n_q + 127) / 128);
  RowsGemmArgs prep{q, dtype, n_q, Hq, Sq, sb, sh, ss, w_cat, q_cat, q_cat_dtype,
                    Hq * Sq * 2 * d, Sq * 2 * d, (int64_t)2 * d, tiles};
  return d == 128 ? launch_rows_gemm<128, 256>(prep, stream) : launch_rows_gemm<64, 128>(prep, stream);
}

// The SM-pair kernel (tq_attention_c2.cu) serves head_dim 64 and 128; TQ_B200_ATTN=ws selects the single-SM
// kernel instead (diagnostics).
static bool use_sm_pairs() {
  static int cached = -1;
  if (cached < 0) {
    const char* e = getenv("TQ_B200_ATTN");
    cached = (e != nullptr && e[0] == 'w') ? 0 : 1;
  }
  return cached == 1;
}

// Which kernel serves a bf16-mode call.
enum class Bf16Path { kDecode, kPairs, kSingle };
static Bf16Path bf16_path(const AttnArgs& a, int64_t Sq, int d) {
  if (decode_applies(a, d) && Sq <= 16) return Bf16Path::kDecode;
  return ((d == 128 || d == 64) && use_sm_pairs()) ? Bf16Path::kPairs : Bf16Path::kSingle;
}

size_t workspace_bytes_bf16_prepared(int64_t B, int64_t Hq, int64_t Sq, int64_t Hkv, int64_t Sk, int64_t kv_stride,
                                     int d) {
  AttnArgs a{};
  a.Hq = Hq; a.Sq = Sq; a.Hkv = Hkv; a.Sk = Sk; a.kv_stride = kv_stride;
  const int64_t n_q = B * Hq * Sq;
  switch (bf16_path(a, Sq, d)) {
    case Bf16Path::kPairs: return 0;  // everything it needs is in the constants buffer and on the chip
    case Bf16Path::kDecode: return round256((size_t)n_q * 2 * d * 2) + decode_workspace_bytes(B * Hq);
    default: return round256((size_t)n_q * 2 * d * 2) + round256((size_t)n_q * d * 2);
  }
}

int attention_fwd_bf16(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d, int64_t sb, int64_t sh,
                       int64_t ss, const float* Pi_k, const float* S_eff, AttnArgs a, int bits, void* workspace,
                       cudaStream_t stream, const uint8_t* prepared) {
  const int64_t n_q = B * Hq * Sq;
  TQ_REQUIRE(B <= 65535 && Hq <= 65535, "batch and head counts are limited to 65535 in bf16 mode");
  TQ_REQUIRE(a.sm_scale > 0.f && a.sm_scale < 1e30f, "sm_scale must be positive and finite in bf16 mode");
  const Bf16Path path = bf16_path(a, Sq, d);
  TQ_REQUIRE(path == Bf16Path::kDecode || a.kv_stride == a.Sk,
             "a cache with capacity %lld > Sk is served by the split-KV kernel only: head_dim 128, "
             "(Hq / Hkv) * Sq <= 16", (long long)a.kv_stride);
  const bool pairs = path == Bf16Path::kPairs;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  const __nv_bfloat16 *w_cat, *w_unrot;
  const uint32_t* luts;
  if (prepared != nullptr) {
    // operand images built once per compressor pair; the scratch holds per-call data only
    const ConstLayout L = const_layout(d);
    w_cat = reinterpret_cast<const __nv_bfloat16*>(prepared + (pairs ? L.w_cat_pair : L.w_cat_plain));
    w_unrot = reinterpret_cast<const __nv_bfloat16*>(prepared + (pairs ? L.w_unrot_pair : L.w_unrot_plain));
    luts = reinterpret_cast<const uint32_t*>(prepared + L.luts);
  } else {
    w_cat = reinterpret_cast<__nv_bfloat16*>(ws);
    ws += round256((size_t)2 * d * d * 2);
    w_unrot = reinterpret_cast<__nv_bfloat16*>(ws);
    ws += round256((size_t)d * d * 2);
    luts = reinterpret_cast<uint32_t*>(ws);
    ws += kLutBytes;
  }
  __nv_bfloat16* q_cat = reinterpret_cast<__nv_bfloat16*>(ws);
  ws += round256((size_t)n_q * 2 * d * 2);
  __nv_bfloat16* o_rot = reinterpret_cast<__nv_bfloat16*>(ws);

  if (path == Bf16Path::kDecode)  // its own small kernels on both sides of the split-KV kernel; none of the operand images
    return attention_decode(a, B, bits, q, dtype, sb, sh, ss, Pi_k, S_eff, q_cat,
                            prepared != nullptr ? reinterpret_cast<uint8_t*>(o_rot)
                                                : reinterpret_cast<uint8_t*>(o_rot) + round256((size_t)n_q * d * 2),
                            stream);
  if (prepared == nullptr) {
    build_wunrot_kernel<<<d, d, 0, stream>>>(a.Pi_v, d, const_cast<__nv_bfloat16*>(w_unrot), pairs ? d / 2 : 0);
    TQ_CUDA_OK(cudaGetLastError());
  }
  if (pairs) {
    // the SM-pair kernel prepares its query tiles and back-rotates its outputs itself; each CTA of a pair
    // bulk-copies its half of either constant operand (d rows of w_cat, d/2 rows of w_unrot)
    if (prepared == nullptr) {
      build_wcat_kernel<<<d, d, 0, stream>>>(Pi_k, S_eff, d, sqrtf(1.5707963267948966f) / (float)d,
                                             const_cast<__nv_bfloat16*>(w_cat), d);
      TQ_CUDA_OK(cudaGetLastError());
      build_luts_kernel<<<1, 128, 0, stream>>>(a.cen_k, a.cen_v, bits - 1, bits, const_cast<uint32_t*>(luts));
      TQ_CUDA_OK(cudaGetLastError());
    }
    const PairArgs x{q, dtype, sb, sh, ss, w_cat, w_unrot, luts};
    return attention_c2(a, x, B, d, bits, stream);
  }
  // the attention kernel's score contraction runs on fp16 operands: its prepared queries are fp16
  if (int st = prepare_queries_bf16(q, dtype, B, Hq, Sq, d, sb, sh, ss, prepared != nullptr ? nullptr : Pi_k, S_eff,
                                    const_cast<__nv_bfloat16*>(w_cat), q_cat, stream, TQ_F16))
    return st;
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
