// Fused compressed attention on SM PAIRS (thread-block cluster of 2, tcgen05 cta_group::2).
//
// Each CTA of the pair owns one query tile of 128 rows that reads the same KV head -- two query heads
// of one GQA group at the same positions, or two consecutive position blocks of one head -- and keeps
// it WHOLE in its own tensor memory (both contraction halves), together with a double-buffered score
// tile and its output accumulator: 128 + 2*128 + 128 = 512 columns.  Keys advance in tiles of 128.
// One MMA over the pair (M = 256) reads its B operand half from each CTA's shared memory, so each CTA
// decodes only HALF of every tile: the keys [64r, 64r+64) of K_hat and the value coordinates
// [d/2*r, d/2*(r+1)) of V_hat (r = rank in the pair).  Per SM this halves the decode work and the
// operand traffic, and N = 128 runs the tensor pipe at its full rate.
//
// The kernel is self-contained: its prologue turns the raw query tile into Q_cat = q [Pi ; coeff S]^T
// with one MMA group (A = raw tile, B = this CTA's half of the constant operand, both staged in the
// still idle K_hat ring) and its epilogue multiplies the normalised output tile by Pi_v the same way
// (A = bf16 output tile in tensor memory over the retired score columns), so neither the prepared
// queries nor the rotated outputs ever reach HBM.
//
// Roles per CTA (18 warps): warps 0-7 softmax (two threads per row, 64 score columns each), warps
// 8-15 producers (prefetch packed bytes, stage, decode), warp 16 tensor-memory allocation; in the
// leader CTA (rank 0) one thread of warp 16 issues the score MMAs of the pair and one thread of warp
// 17 the P V_hat MMAs.
//
// Barriers.  "leader" ones live in rank 0's shared memory and collect one arrival per WARP of both
// CTAs (lane 0 after __syncwarp; the peer arrives through its cluster address); "both" ones exist in
// each CTA and are completed by tcgen05.commit multicast to the pair.
//   leader k_full[s], v_full[s] (16): both halves of K_hat / V_hat of tile j decoded
//   leader p_full[b] (16)            : P[b] written over S[b] (so S[b] has been read) by all softmax warps
//   both   k_empty[s], v_empty[s]    : the score / PV MMA of tile j has drained
//   both   s_full[b], pv_done[b]     : S[b] holds tile j's scores / O += P V_hat of tile j finished
//   local  pk_full[2] (8), xch[4] (64)
//   leader qp_full (32): raw query tile and constant operand staged;  both qp_done: Q_cat accumulated
//   leader q_full (16) : 1st phase Q_cat packed into tensor memory, 2nd phase output tile + Pi_v staged
//   both   e_done      : back-rotated output tile accumulated
// Every wait is bounded; an expired wait raises the CTA's abort flag, the CTA unwinds to the final
// cluster barrier, a device counter is bumped and later launches return at once.
#include <math.h>

#include "tq_attention.cuh"
#include "tq_common.cuh"
#include "tq_rows.cuh"
#include "tq_simt.cuh"
#include "tq_tcgen05.cuh"

namespace tq {

__device__ unsigned long long g_c2_faults = 0ull;
// this device's slot of the host-visible status page (NULL until the first call on the device installs it)
__device__ unsigned long long* g_fault_mailbox_c2 = nullptr;
int set_fault_mailbox_c2(unsigned long long* slot) {
  TQ_CUDA_OK(cudaMemcpyToSymbol(g_fault_mailbox_c2, &slot, sizeof(slot)));
  return TQ_OK;
}

int read_c2_faults(unsigned long long* out) {
  TQ_CUDA_OK(cudaMemcpyFromSymbol(out, g_c2_faults, sizeof(*out)));
  return TQ_OK;
}

// Diagnostics: stage timestamps of the first cluster's leader CTA, see tq_trace_read.
constexpr int kTraceCap2 = 4096;
static int g_trace2_host_on = 0;  // selects the tracing build of the kernel at launch
__device__ long long g_trace2[2 * kTraceCap2];

int trace_enable_c2(int on) {
  const int v = on ? 1 : 0;
  static long long fill[2 * kTraceCap2];
  for (int i = 0; i < 2 * kTraceCap2; ++i) fill[i] = -1;
  TQ_CUDA_OK(cudaMemcpyToSymbol(g_trace2, fill, sizeof(fill)));
  g_trace2_host_on = v;
  return TQ_OK;
}
int trace_read_c2(long long* host_buf, int max_records, int* n_out) {
  int n = kTraceCap2 < max_records ? kTraceCap2 : max_records;
  TQ_CUDA_OK(cudaDeviceSynchronize());
  TQ_CUDA_OK(cudaMemcpyFromSymbol(host_buf, g_trace2, sizeof(long long) * 2 * n));
  *n_out = n;
  return TQ_OK;
}

namespace {

// The tracing build of the kernel (TRACE = true) is launched only while tracing is enabled; in the
// production build every mark compiles to nothing.
template <bool TRACE>
struct Tracer2 {
  bool on;
  int role, n;
  __device__ Tracer2(bool on_, int role_) : on(TRACE && on_), role(role_), n(0) {}
  __device__ __forceinline__ void mark(int ev, int tile) {
    if (!TRACE) return;
    if (!on || n >= kTraceCap2 / 4) return;
    const int i = role * (kTraceCap2 / 4) + n++;
    g_trace2[2 * i] = ((long long)role << 32) | ((long long)ev << 16) | (long long)tile;
    g_trace2[2 * i + 1] = clock64();
  }
  // wall-clock nanoseconds next to the SM clock: their ratio over a CTA's life is the SM frequency under load
  __device__ __forceinline__ void mark_ns(int ev, int tile) {
    if (!TRACE) return;
    if (!on || n >= kTraceCap2 / 4) return;
    const int i = role * (kTraceCap2 / 4) + n++;
    long long ns;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
    g_trace2[2 * i] = ((long long)role << 32) | ((long long)ev << 16) | (long long)tile;
    g_trace2[2 * i + 1] = ns;
  }
};

constexpr int kBM = 128;       // query rows per CTA
constexpr int kBN = 128;       // keys per tile (64 decoded by each CTA)
constexpr int kHalfN = 64;
constexpr int kSoftmax = 256;      // 8 softmax warps: two threads per query row, 64 score columns each
                                   // (16 warps were measured slower: the exp2 throughput, not the thread count, bounds the phase)
constexpr int kProducers = 256;    // 8 producer warps
constexpr int kThreads = kSoftmax + kProducers + 64;
constexpr int kCtlWarp = kThreads / 32 - 2;   // tensor-memory allocation; issues the score MMAs in the leader CTA
constexpr int kPvWarp = kThreads / 32 - 1;    // issues the P V_hat MMAs in the leader CTA
constexpr int kSoftmaxArrivals = 2 * kSoftmax / 32;     // softmax warps of both CTAs
constexpr int kProducerArrivals = 2 * kProducers / 32;  // producer warps of both CTAs

// `bits` holds exactly 8 B-bit indices (nothing above bit 8 B), so the last pair needs no mask
template <int B>
__device__ __forceinline__ void decode_group(const uint32_t* lut, uint32_t bits, uint32_t (&out)[4]) {
#pragma unroll
  for (int q = 0; q < 3; ++q) out[q] = lut[(bits >> (2 * q * B)) & ((1u << (2 * B)) - 1)];
  out[3] = lut[bits >> (6 * B)];
}

template <int D, int BITS>
struct C2Smem {
  static constexpr int G = D / 8, KB = BITS - 1, VB = BITS;
  static constexpr int kStages = 3;
  static constexpr uint32_t kKStage = kHalfN * 2 * D * 2;       // 64 keys x 2D
  static constexpr uint32_t kVStage = (D / 2) * kBN * 2;        // d/2 coordinates x 128 keys
  static constexpr uint32_t kIdxK = kHalfN * G * KB;            // packed bytes this CTA stages per tile
  static constexpr uint32_t kSgn = kHalfN * G;
  static constexpr uint32_t kIdxV = kBN * (G / 2) * VB;
  static constexpr uint32_t kPkStage = kIdxK + kSgn + kIdxV;
  static constexpr uint32_t kKOff = 0;
  static constexpr uint32_t kVOff = kKOff + kStages * kKStage;
  static constexpr uint32_t kPkOff = kVOff + kStages * kVStage;
  static constexpr uint32_t kUOff = kPkOff + 2 * kPkStage;      // this CTA's half of Pi_v^T, [D/2, D] K-major
  static constexpr uint32_t kUBytes = (D / 2) * D * 2;
  static constexpr uint32_t kWBytes = D * D * 2;                // this CTA's half of [Pi ; coeff S]
  static constexpr uint32_t kTotal = kUOff + kUBytes;
  static constexpr uint32_t kSboK = 2 * G * 128;                // K-major [keys, 2D]
  static constexpr uint32_t kSboV = 128;                        // MN-major [d/2, 128 keys]: coordinate chunks adjacent
  static constexpr uint32_t kLboV = (G / 2) * 128;              // ... 8-key groups G/2 core matrices apart
  static constexpr uint32_t kColQ = 0;                          // Q_cat: 2D bf16 = D columns
  static constexpr uint32_t kColS = D;                          // S[2]: 2 x 128 (P[b] = first 64 columns of S[b])
  static constexpr uint32_t kColO = D + 2 * kBN;                // O: D
  static constexpr uint32_t kCols = 512;
  static_assert(kColO + D <= kCols, "tensor memory over-subscribed");
  // Prologue operands borrow the far end of the rings, so that the first two K_hat tiles can be decoded
  // meanwhile: raw query tile [128, D] in V_hat stages 0-1, half of [Pi ; coeff S] ([D, D]) in K_hat
  // stage 2.  Epilogue: the output tile is staged over the K_hat ring for coalesced stores.  All operands
  // K-major with 8-row groups kSboW apart; the two constant ones arrive by bulk copy (their global image
  // has this layout already).
  static constexpr uint32_t kSboW = G * 128;
  static constexpr uint32_t kQOff = kVOff;
  static constexpr uint32_t kWOff = kKOff + 2 * kKStage;
  static constexpr uint32_t kOutOff = kKOff;
  static_assert(kStages == 3 && kBM * D * 2 <= 2 * kVStage && D * D * 2 <= kKStage, "prologue operands must fit");
  static_assert(kBM * (D * 4 + 16) <= kPkOff - kOutOff, "the output tile must fit");
  static_assert(2 * D <= 2 * kBN, "the Q_cat accumulator borrows both score tiles");
};

template <int D, int BITS, bool TRACE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
attention_c2_kernel(const AttnArgs a, const PairArgs x, const int pair_heads) {
  using L = C2Smem<D, BITS>;
  constexpr int G = L::G, KB = L::KB, VB = L::VB, kStages = L::kStages;
  constexpr int NQ = kSoftmax / kBM;  // threads per query row
  constexpr int HC = kBN / NQ;       // score columns per softmax thread
  constexpr float kLog2e = 1.4426950408889634f;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // norms as stored (fp16 bit patterns), duplicated into both halves of a word: the multiplier of a packed pair
  __shared__ uint32_t nk_s[2][kHalfN];    // key norms, residual norms of this CTA's keys (slot j & 1)
  __shared__ uint32_t rho_s[2][kHalfN];
  __shared__ uint32_t nv_s[2][kBN];       // value norms of all keys of the tile
  __shared__ float xmax[2][kSoftmax / kBM][kBM];  // [tile parity][column part][row]
  __shared__ __align__(16) uint32_t lutK[1 << (2 * KB)];  // pair tables, bulk-copied from their global image
  __shared__ __align__(16) uint32_t lutV[1 << (2 * VB)];
  __shared__ __align__(8) uint64_t bars[4 * kStages + 22];
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  volatile int* abort_flag = &s_abort;

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const uint32_t rank = tc::cluster_ctarank();
  // Whether an earlier launch ran into an expired wait is read by one thread of the (otherwise idle)
  // P V_hat issuer warp and published with the set-up barrier below; nothing before that depends on it.
  // ---- which query tile ------------------------------------------------------------------
  const int64_t b = blockIdx.z;
  const int xpair = (int)((gridDim.x >> 1) - 1 - (blockIdx.x >> 1));  // heaviest (latest) position blocks first
  int64_t head;
  int q0, q0_last;
  if (pair_heads) {
    head = 2 * (int64_t)blockIdx.y + rank;
    q0 = q0_last = xpair * kBM;
  } else {
    head = blockIdx.y;
    q0 = (2 * xpair + (int)rank) * kBM;
    q0_last = (2 * xpair + 1) * kBM;
  }
  // 32-bit division (head counts are below 65536): the 64-bit form is a subroutine of ~100 instructions, twice,
  // on every thread's way to its first load
  const int64_t kv_base = (b * a.Hkv + (int)head / ((int)a.Hq / (int)a.Hkv)) * a.Sk;
  const int shift = (int)(a.Sk - a.Sq);
  int k_end = (int)a.Sk;
  if (a.causal) k_end = min(k_end, min(q0_last + kBM - 1, (int)a.Sq - 1) + shift + 1);
  const int n_tiles_live = (k_end + kBN - 1) / kBN;  // identical in both CTAs of the pair

  const uint32_t bar0 = tc::smem_u32(&bars[0]);
  auto k_full = [&](int i) { return bar0 + 8u * i; };                       // leader
  auto v_full = [&](int i) { return bar0 + 8u * (kStages + i); };           // leader
  auto k_empty = [&](int i) { return bar0 + 8u * (2 * kStages + i); };      // both
  auto v_empty = [&](int i) { return bar0 + 8u * (3 * kStages + i); };      // both
  auto s_full = [&](int i) { return bar0 + 8u * (4 * kStages + i); };       // both
  auto pv_done = [&](int i) { return bar0 + 8u * (4 * kStages + 2 + i); };  // both
  auto p_full = [&](int i) { return bar0 + 8u * (4 * kStages + 6 + i); };   // leader
  auto pk_full = [&](int i) { return bar0 + 8u * (4 * kStages + 8 + i); };  // local
  auto xch = [&](int i) { return bar0 + 8u * (4 * kStages + 10 + i); };     // local
  const uint32_t q_full = bar0 + 8u * (4 * kStages + 14);                   // leader
  const uint32_t qp_full = bar0 + 8u * (4 * kStages + 15);                  // leader
  const uint32_t qp_done = bar0 + 8u * (4 * kStages + 16);                  // both
  const uint32_t e_done = bar0 + 8u * (4 * kStages + 17);                   // both
  const uint32_t w_full = bar0 + 8u * (4 * kStages + 18);                   // local, bulk-copy bytes
  const uint32_t u_full = bar0 + 8u * (4 * kStages + 19);                   // local, bulk-copy bytes
  const uint32_t u_peer = bar0 + 8u * (4 * kStages + 20);                   // leader: the peer's Pi_v^T half is in
  const uint32_t lut_full = bar0 + 8u * (4 * kStages + 21);                 // local, bulk-copy bytes
  // one arrival on a barrier that lives in rank 0: local form there, cluster address from the peer
  auto arrive_leader = [&](uint32_t bar) {
    if (rank == 0) tc::mbar_arrive(bar);
    else tc::mbar_arrive_cluster(tc::map_to_cta(bar, 0));
  };

  // The softmax warps fetch the raw query tile first of all (8 threads per 128-byte core matrix of the A
  // operand), so that the DRAM latency overlaps the barrier / tensor-memory set-up below.
  const long long t_entry = TRACE ? clock64() : 0;
  constexpr int NA = kBM * (D / 8) / kSoftmax;
  uint4 qv[NA];
  if (tid < kSoftmax) {
    // chunk c of row r0 + i * rstep: the offset advances by a constant per load
    constexpr int rstep = kSoftmax / (D / 8);
    static_assert(rstep % 8 == 0, "a thread keeps its row within the 8-row group and its chunk");
    const int r0 = tid % 8 + 8 * (tid / (8 * (D / 8))), c = (tid / 8) % (D / 8);
    int64_t off = b * x.q_stride_b + head * x.q_stride_h + (int64_t)(q0 + r0) * x.q_stride_s + c * 8;
    const int64_t ostep = (int64_t)rstep * x.q_stride_s;
#pragma unroll
    for (int i = 0; i < NA; ++i, off += ostep) {
      const int r = r0 + i * rstep;
      qv[i] = make_uint4(0, 0, 0, 0);
      if (q0 + r < a.Sq) {
        if (x.q_dtype == TQ_BF16) qv[i] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(x.q) + off);
        else qv[i] = load_row_chunk_bf16(x.q, x.q_dtype, off);
      }
    }
  }
  const long long t_q = TRACE ? clock64() : 0;
  if (warp == kPvWarp) {
    // barrier initialisation, one barrier per lane and round; then lane 0 starts the bulk copies of the
    // constant operands of the prologue and epilogue MMAs (no register staging)
    constexpr int kBars = 4 * kStages + 22;
    for (int i = lane; i < kBars; i += 32) {
      const int r = i - 4 * kStages;
      uint32_t count = 1;                                     // commit / bulk-copy / single-thread barriers
      if (i < 2 * kStages) count = kProducerArrivals;         // k_full, v_full
      else if (r == 6 || r == 7 || r == 14) count = kSoftmaxArrivals;  // p_full, q_full
      else if (r == 8 || r == 9) count = kProducers / 32;     // pk_full: one arrival per producer warp
      else if (r >= 10 && r <= 13) count = 32 * (kSoftmax / kBM);      // xch
      else if (r == 15) count = kSoftmaxArrivals + 1;         // qp_full: + the peer's constant operand
      tc::mbar_init(bar0 + 8u * i, count);
    }
    tc::fence_mbar_init();
    tc::fence_async_smem();  // the copy engine completes on barriers initialised just above
    __syncwarp();
    if (lane == 0) {
      const bool poisoned = *reinterpret_cast<volatile unsigned long long*>(&g_c2_faults) != 0ull;
      s_abort = poisoned ? 1 : 0;
      if (!poisoned) {
        tc::mbar_arrive_expect_tx(w_full, L::kWBytes);
        tc::bulk_load(tc::smem_u32(smem_raw + L::kWOff), x.w_cat + (int64_t)rank * D * D, L::kWBytes, w_full);
        tc::mbar_arrive_expect_tx(u_full, L::kUBytes);
        tc::bulk_load(tc::smem_u32(smem_raw + L::kUOff), x.w_unrot + (int64_t)rank * (D / 2) * D, L::kUBytes, u_full);
        // the decode tables too: nobody waits for them here, the producers do before their first tile
        tc::mbar_arrive_expect_tx(lut_full, (uint32_t)(sizeof(lutK) + sizeof(lutV)));
        tc::bulk_load(tc::smem_u32(lutK), x.luts, (uint32_t)sizeof(lutK), lut_full);
        tc::bulk_load(tc::smem_u32(lutV), x.luts + (1 << (2 * KB)), (uint32_t)sizeof(lutV), lut_full);
      }
    }
  }
  if (warp == kCtlWarp) tc::tmem_alloc2(tc::smem_u32(&tmem_slot), L::kCols);
  const long long t_i = TRACE ? clock64() : 0;
  tc::fence_before_sync();
  __syncthreads();
  const long long t_s = TRACE ? clock64() : 0;
  tc::cluster_sync_relaxed();  // the peer's barriers and tensor memory exist before anyone signals or issues
  tc::fence_after_sync();
  const bool dead = s_abort != 0;  // an earlier bounded wait expired: do nothing but keep the cluster barriers paired
  const int n_tiles = dead ? 0 : n_tiles_live;
  const uint32_t tmem_base = tmem_slot;
  const uint32_t tmem_o = tmem_base + L::kColO;
  bool ok = true;
  // traced: the heaviest cluster of the last (head pair, batch), which runs late in the launch
  Tracer2<TRACE> tr(blockIdx.x == 0 && blockIdx.y == gridDim.y - 1 && blockIdx.z == gridDim.z - 1 && lane == 0 &&
                 (warp == 0 || warp == kSoftmax / 32 || warp >= kCtlWarp),
             warp == 0 ? 0 : warp == kSoftmax / 32 ? 1 : warp == kCtlWarp ? 2 : 3);

  if (warp < kSoftmax / 32) {
    // =============================== softmax warps ===============================
    const int quad = warp % 4, chalf = warp / 4;
    const int row = quad * 32 + lane;
    const int qi = q0 + row;
    const int64_t qrow = (b * a.Hq + head) * a.Sq + qi;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    if (TRACE && tr.on) {  // kernel entry, measured before the set-up
      const int i = tr.role * (kTraceCap2 / 4) + tr.n++;
      g_trace2[2 * i] = ((long long)tr.role << 32) | (25ll << 16) | 999ll;
      g_trace2[2 * i + 1] = t_entry;
      const long long ts[3] = {t_q, t_i, t_s};
      for (int e = 0; e < 3; ++e) {
        const int i2 = tr.role * (kTraceCap2 / 4) + tr.n++;
        g_trace2[2 * i2] = ((long long)tr.role << 32) | ((long long)(26 + e) << 16) | 999ll;
        g_trace2[2 * i2 + 1] = ts[e];
      }
    }
    tr.mark(10, 999);
    tr.mark_ns(18, 999);
    if (n_tiles > 0) {
      // raw query tile [128, D] -> A operand of the prologue MMA
      uint8_t* Aq = smem_raw + L::kQOff;
#pragma unroll
      for (int i = 0; i < NA; ++i) {
        const int e = i * kSoftmax + tid, r = e % 8 + 8 * (e / (8 * G)), c = (e / 8) % G;
        *reinterpret_cast<uint4*>(Aq + (r / 8) * L::kSboW + c * 128 + (r % 8) * 16) = qv[i];
      }
      tr.mark(21, 999);
      tc::fence_async_smem();
      tr.mark(22, 999);
      __syncwarp();
      if (lane == 0) arrive_leader(qp_full);
      tr.mark(11, 999);
      // Q_cat row (fp32, 2D columns over both score tiles) -> packed fp16 in the query columns; each of
      // the row's threads converts 2D/NQ accumulator columns
      if ((ok = tc::mbar_wait_or_abort(qp_done, 0, abort_flag))) {
        tc::fence_after_sync();
        tr.mark(12, 999);
#pragma unroll 1
        for (int c0 = 0; c0 < 2 * D / NQ; c0 += 32) {
          uint32_t raw[32], pw[16];
          tc::tmem_ld32(tmem_base + L::kColS + lane_base + chalf * (2 * D / NQ) + c0, raw);
          tc::wait_ld();
#pragma unroll
          for (int c = 0; c < 16; ++c)
            pw[c] = tc::pack_f16x2_sat(__uint_as_float(raw[2 * c]), __uint_as_float(raw[2 * c + 1]));
          tc::tmem_st16(tmem_base + L::kColQ + lane_base + chalf * (D / NQ) + c0 / 2, pw);
        }
        tc::wait_st();
        tc::fence_before_sync();
        __syncwarp();
        if (lane == 0) arrive_leader(q_full);
        tr.mark(13, 999);
      }
    }
    float m_run = -INFINITY, l_run = 0.f;
    const float cexp = a.sm_scale * kLog2e, rcexp = 1.f / cexp;  // K_hat carries the key norms: S is the raw score
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int bb = j & 1, u = j >> 1, k0 = j * kBN;
      const int kc0 = k0 + chalf * HC;
      const uint32_t tmem_s = tmem_base + L::kColS + bb * kBN;
      tr.mark(0, j);
      if (!(ok = tc::mbar_wait_or_abort(s_full(bb), u & 1, abort_flag))) break;
      tc::fence_after_sync();
      tr.mark(1, j);
      float t[HC];
      {
        static_assert(HC == 64, "two 32-column loads per thread");
        uint32_t raw0[32], raw1[32];
        tc::tmem_ld32(tmem_s + lane_base + chalf * HC, raw0);
        tc::tmem_ld32(tmem_s + lane_base + chalf * HC + 32, raw1);
        tc::wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          t[c] = __uint_as_float(raw0[c]);
          t[32 + c] = __uint_as_float(raw1[c]);
        }
      }
      const bool edge = (k0 + kBN > a.Sk) || (a.causal && k0 + kBN - 1 > q0 + shift) || a.mask != nullptr;
      if (edge) {
        // Tiles that cross the end of the keys or the causal diagonal, and every tile under an additive mask.  A
        // thread's 64 columns are the keys kc0 .. kc0 + 63: `vsk` is the last column that exists, `vis` the last one
        // this row may see.  Everything stays in raw score units (the mask is divided by sm_scale instead of the
        // scores being multiplied by it), so that the common path below takes the maximum: one compare and one
        // select per score here, where a branchy per-element form cost more than two whole tile periods.
        const int vsk = (int)a.Sk - 1 - kc0;
        const int vis = a.causal ? min(vsk, qi + shift - kc0) : vsk;
        if (a.mask != nullptr && qi < a.Sq) {
          const float* mrow = a.mask + b * a.mask_stride_b + (int64_t)qi * a.mask_stride_q + kc0;
          // The large negative value HF masks with is clamped to -60000 in log2 units (exp2 of it is still exactly
          // 0 beside any real score) so that it stays finite: a row whose visible keys are all masked then averages
          // them uniformly, as a softmax over equal finite scores does in the reference, instead of coming out as
          // zeros.
          const float m_unit = kLog2e * rcexp, floor_raw = -60000.f * rcexp;
#pragma unroll
          for (int c = 0; c < HC; ++c)
            if (c <= vsk) t[c] = fmaxf(fmaf(mrow[c], m_unit, t[c]), floor_raw);
        }
#pragma unroll
        for (int c = 0; c < HC; ++c) t[c] = c <= vis ? t[c] : -INFINITY;
      }
      float mx;
      {
        float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;  // three-input maxima, four chains
#pragma unroll
        for (int c8 = 0; c8 < HC; c8 += 8) {
          m0 = tc::fmax3(m0, t[c8], t[c8 + 1]);
          m1 = tc::fmax3(m1, t[c8 + 2], t[c8 + 3]);
          m2 = tc::fmax3(m2, t[c8 + 4], t[c8 + 5]);
          m3 = tc::fmax3(m3, t[c8 + 6], t[c8 + 7]);
        }
        mx = fmaxf(tc::fmax3(m0, m1, m2), m3) * cexp;
      }
      // exchange half-row maxima with the partner warp (slots alternate with the tile parity)
      tr.mark(2, j);
      xmax[bb][chalf][row] = mx;
      tc::mbar_arrive(xch(quad));
      if (!(ok = tc::mbar_wait_or_abort(xch(quad), j & 1, abort_flag))) break;
#pragma unroll
      for (int o = 1; o < NQ; ++o) mx = fmaxf(mx, xmax[bb][(chalf + o) % NQ][row]);
      tr.mark(3, j);
      // P[bb] overwrites the first 64 columns of S[bb]: both halves of the row must have been loaded
      // (the exchange above orders the partner's loads before this thread's store below)
      const float m_cand = fmaxf(m_run, mx);
      const bool grow = __any_sync(0xffffffffu, m_cand > m_run + 8.f);  // identical in both warps of the quadrant
      float alpha = 1.f;
      if (grow) {
        alpha = (m_run == -INFINITY) ? 0.f : tc::fast_exp2(m_run - m_cand);
        m_run = m_cand;
      }
      const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
      float psum = 0.f;
#pragma unroll
      for (int hblk = 0; hblk < HC / 32; ++hblk) {
        uint32_t pw[16];
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const float p0 = tc::fast_exp2(fmaf(t[32 * hblk + 2 * c], cexp, -m_use));
          const float p1 = tc::fast_exp2(fmaf(t[32 * hblk + 2 * c + 1], cexp, -m_use));
          psum += p0 + p1;
          pw[c] = tc::pack_f16x2(p0, p1);  // p <= 2^8: the running maximum trails a row's scores by at most 8
        }
        tc::tmem_st16(tmem_s + lane_base + chalf * (HC / 2) + 16 * hblk, pw);
      }
      l_run = l_run * alpha + psum;
      tr.mark(4, j);
      if (grow && j >= 1) {
        // O must be at rest: wait for the previous tile's P V_hat; each thread rescales D/NQ columns of its row
        if (!(ok = tc::mbar_wait_or_abort(pv_done((j - 1) & 1), ((j - 1) >> 1) & 1, abort_flag))) break;
        tc::fence_after_sync();
#pragma unroll 1
        for (int c0 = 0; c0 < D / NQ; c0 += 32) {
          uint32_t raw[32];
          const uint32_t addr = tmem_o + lane_base + chalf * (D / NQ) + c0;
          tc::tmem_ld32(addr, raw);
          tc::wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) raw[c] = __float_as_uint(__uint_as_float(raw[c]) * alpha);
          tc::tmem_st32(addr, raw);
        }
      }
      tc::wait_st();
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) arrive_leader(p_full(bb));
      tr.mark(5, j);
    }
    // ---- epilogue: out = (O / l) Pi_v on the tensor pipe ----
    if (ok && n_tiles > 0) {
      ok = tc::mbar_wait_or_abort(pv_done((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, abort_flag);
      tr.mark(14, 999);
    }
    if (ok && n_tiles > 0) {
      xmax[n_tiles & 1][chalf][row] = l_run;
      tc::mbar_arrive(xch(quad));
      ok = tc::mbar_wait_or_abort(xch(quad), n_tiles & 1, abort_flag);
    }
    if (ok && n_tiles > 0) {
      tc::fence_after_sync();
      float l_tot = l_run;
#pragma unroll
      for (int o = 1; o < NQ; ++o) l_tot += xmax[n_tiles & 1][(chalf + o) % NQ][row];
      const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
      // normalised output row as packed bf16 over the (retired) first score tile: A operand
#pragma unroll 1
      for (int c0 = 0; c0 < D / NQ; c0 += 32) {
        uint32_t raw[32], pw[16];
        tc::tmem_ld32(tmem_o + lane_base + chalf * (D / NQ) + c0, raw);
        tc::wait_ld();
#pragma unroll
        for (int c = 0; c < 16; ++c)
          pw[c] = tc::pack_bf16x2(__uint_as_float(raw[2 * c]) * inv, __uint_as_float(raw[2 * c + 1]) * inv);
        tc::tmem_st16(tmem_base + L::kColS + lane_base + chalf * (D / (2 * NQ)) + c0 / 2, pw);
      }
      tc::wait_st();
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) arrive_leader(q_full);  // second phase of this barrier
      tr.mark(15, 999);
      ok = tc::mbar_wait_or_abort(e_done, 0, abort_flag);
      tr.mark(16, 999);
    }
    if (ok && n_tiles > 0) {
      // accumulator row -> output dtype -> shared memory (padded rows), so that whole rows leave coalesced
      tc::fence_after_sync();
      const int esz = a.out_dtype == TQ_F32 ? 4 : 2;
      const int pitch = D * esz + 16;
      uint8_t* Ot = smem_raw + L::kOutOff;
#pragma unroll 1
      for (int c0 = 0; c0 < D / NQ; c0 += 32) {
        uint32_t acc[32];
        tc::tmem_ld32(tmem_base + L::kColS + kBN + lane_base + chalf * (D / NQ) + c0, acc);
        tc::wait_ld();
        store_row_chunk(Ot + row * pitch, a.out_dtype, chalf * (D / NQ) + c0, acc);
      }
      tr.mark(23, 999);
      tc::mbar_arrive(xch(quad));
      ok = tc::mbar_wait_or_abort(xch(quad), (n_tiles + 1) & 1, abort_flag);
      tr.mark(24, 999);
    }
    if (ok && n_tiles > 0) {
      // the two warps of the quadrant store 16 of its 32 rows each
      const int esz = a.out_dtype == TQ_F32 ? 4 : 2;
      static_assert(D == 128 || D == 64, "chunks per row are derived for head_dim 64 and 128");
      const int lcpr = (a.out_dtype == TQ_F32 ? 5 : 4) - (D == 64 ? 1 : 0);  // log2 of the 16-byte chunks per row
      const int pitch = D * esz + 16, cpr = 1 << lcpr;
      // lane -> (row within the iteration, 16-byte chunk); every iteration moves on by 32 / cpr rows: pointers advance
      // by constant steps (no 64-bit multiplies inside the loop)
      const int rpi = 32 >> lcpr;
      int r = quad * 32 + chalf * 16 + (lane >> lcpr);
      const int c = lane & (cpr - 1);
      const uint8_t* src = smem_raw + L::kOutOff + r * pitch + c * 16;
      uint8_t* dst = static_cast<uint8_t*>(a.out) +
                     (b * a.o_stride_b + head * a.o_stride_h + (int64_t)(q0 + r) * a.o_stride_s) * esz + c * 16;
      const int64_t dstep = (int64_t)rpi * a.o_stride_s * esz;
      const int sstep = rpi * pitch;
#pragma unroll 4
      for (int i = 0; i < 16 / rpi; ++i) {
        if (q0 + r < a.Sq) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
        r += rpi;
        src += sstep;
        dst += dstep;
      }
      tr.mark(17, 999);
      tr.mark_ns(19, 999);
    }
  } else if (warp < kCtlWarp) {
    // =============================== producer warps ===============================
    // This CTA decodes keys [k0 + 64 rank, +64) of K_hat (all 2D contraction columns) and value
    // coordinates [D/2 rank, +D/2) of all 128 keys of V_hat.
    const int p = tid - kSoftmax;
    __builtin_assume(p >= 0 && p < kProducers);      // lets the compiler drop the always-true unit guards below
    constexpr int GPK = G / 2;                       // 16-coordinate items per key row
    constexpr int GPV = G / 4;                       // ... per half value row
    constexpr int VROW = (G / 2) * VB;               // packed bytes of half a value row
    constexpr int VU = VROW % 8 == 0 ? 8 : 4;        // bytes per staged unit of the value rows (12-byte half rows: 4)
    static_assert(VROW % VU == 0 && (G * KB) % 8 == 0, "staged units must not straddle rows");
    constexpr int UK = L::kIdxK / 8, US = L::kSgn / 8, UV = L::kIdxV / VU;  // units staged per tile (keys, signs: 8 bytes)
    constexpr int NK = (UK + kProducers - 1) / kProducers, NV = (UV + kProducers - 1) / kProducers;
    constexpr int NIK = (kHalfN * GPK + kProducers - 1) / kProducers;
    constexpr int NIV = (kBN * GPV + kProducers - 1) / kProducers;
    uint2 rk[NK], rv[NV], rs;
    uint32_t rn[3];
    const uint8_t* gk = a.key_idx + kv_base * (G * KB);
    const uint8_t* gs = a.key_sgn + kv_base * G;
    const uint8_t* gv = a.val_idx + kv_base * (G * VB) + rank * VROW;
    const int koff = (int)rank * kHalfN;
    // per-thread constants of the staging copy: byte offset of each 8-byte unit inside the tile's packed
    // arrays and the key (row) it belongs to
    int k_off[NK], k_row[NK], v_off[NV], v_row[NV];
#pragma unroll
    for (int i = 0; i < NK; ++i) {
      const int un = i * kProducers + p;
      k_off[i] = un * 8;
      k_row[i] = un < UK ? koff + (un * 8) / (G * KB) : (1 << 30);
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int un = i * kProducers + p;
      const int key = (un * VU) / VROW;
      v_off[i] = key * (G * VB) + (un * VU) % VROW;
      v_row[i] = un < UV ? key : (1 << 30);
    }
    const int s_row = p < US ? koff + (p * 8) / G : (1 << 30);
    auto prefetch = [&](int k0) {
      const uint2 zero = make_uint2(0, 0);
      const int left = (int)a.Sk - k0;  // keys of this tile that exist
      const uint8_t* tk = gk + (int64_t)(k0 + koff) * (G * KB);
      const uint8_t* tv = gv + (int64_t)k0 * (G * VB);
#pragma unroll
      for (int i = 0; i < NK; ++i) rk[i] = k_row[i] < left ? *reinterpret_cast<const uint2*>(tk + k_off[i]) : zero;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        if constexpr (VU == 8) rv[i] = v_row[i] < left ? *reinterpret_cast<const uint2*>(tv + v_off[i]) : zero;
        else rv[i] = v_row[i] < left ? make_uint2(*reinterpret_cast<const uint32_t*>(tv + v_off[i]), 0u) : zero;
      }
      rs = s_row < left ? *reinterpret_cast<const uint2*>(gs + (int64_t)(k0 + koff) * G + p * 8) : zero;
      if (p < kHalfN) {
        const bool live = koff + p < left;
        rn[0] = live ? a.key_vn[kv_base + k0 + koff + p] : 0;
        rn[1] = live ? a.key_rn[kv_base + k0 + koff + p] : 0;
      }
      if (p < kBN) rn[2] = (p < left) ? a.val_vn[kv_base + k0 + p] : 0;
    };
    // Per-thread constants of the decode, as byte offsets ready for use: where an item's packed indices and sign
    // bits sit in the staging slot, where its decoded chunks go in the operand stage, which norm row it scales by
    int kkey[NIK], ksrc[NIK], ksgn[NIK], kdst[NIK], vkey[NIV], vsrc[NIV], vdst[NIV];
#pragma unroll
    for (int i = 0; i < NIK; ++i) {
      const int e = i * kProducers + p, key = (e % 8) + 8 * (e / (8 * GPK)), gp = (e / 8) % GPK;
      kkey[i] = key;
      ksrc[i] = key * (G * KB) + gp * 2 * KB;
      ksgn[i] = (int)L::kIdxK + key * G + gp * 2;
      kdst[i] = (key / 8) * (int)L::kSboK + (key % 8) * 16 + 2 * gp * 128;
    }
#pragma unroll
    for (int i = 0; i < NIV; ++i) {
      const int e = i * kProducers + p, key = (e % 8) + 8 * (e / (8 * GPV)), gp = (e / 8) % GPV;
      vkey[i] = key;
      vsrc[i] = (int)(L::kIdxK + L::kSgn) + key * VROW + gp * 2 * VB;
      vdst[i] = (key / 8) * (int)L::kLboV + (key % 8) * 16 + 2 * gp * (int)L::kSboV;
    }
    if (n_tiles > 0) {
      prefetch(0);
      ok = tc::mbar_wait_or_abort(lut_full, 0, abort_flag);  // the decode tables have landed
    }
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j % kStages, u = j / kStages, ps = j & 1;
      uint8_t* pk = smem_raw + L::kPkOff + ps * L::kPkStage;
      tr.mark(0, j);
#pragma unroll
      for (int i = 0; i < NK; ++i)
        if (i * kProducers + p < UK) *reinterpret_cast<uint2*>(pk + (i * kProducers + p) * 8) = rk[i];
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (i * kProducers + p < UV) {
          if constexpr (VU == 8) *reinterpret_cast<uint2*>(pk + L::kIdxK + L::kSgn + (i * kProducers + p) * 8) = rv[i];
          else *reinterpret_cast<uint32_t*>(pk + L::kIdxK + L::kSgn + (i * kProducers + p) * 4) = rv[i].x;
        }
      if (p < US) *reinterpret_cast<uint2*>(pk + L::kIdxK + p * 8) = rs;
      if (p < kHalfN) {
        nk_s[ps][p] = (rn[0] & 0xffffu) * 0x10001u;
        rho_s[ps][p] = (rn[1] & 0xffffu) * 0x10001u;
      }
      if (p < kBN) nv_s[ps][p] = (rn[2] & 0xffffu) * 0x10001u;
      __syncwarp();  // the warp's staged bytes are ordered before lane 0's arrival (one barrier update per warp, not 32)
      if (lane == 0) tc::mbar_arrive(pk_full(ps));
      if (!(ok = tc::mbar_wait_or_abort(pk_full(ps), (j >> 1) & 1, abort_flag))) break;
      tr.mark(1, j);
      if (j + 1 < n_tiles) prefetch((j + 1) * kBN);
      tr.mark(6, j);
      if (u >= 1 && !(ok = tc::mbar_wait_or_abort(k_empty(st), (u - 1) & 1, abort_flag))) break;
      if (j == 2 && !(ok = tc::mbar_wait_or_abort(qp_done, 0, abort_flag))) break;  // stage 2 held a prologue operand
      tr.mark(2, j);
      // ---- keys ----
      uint8_t* Kd = smem_raw + L::kKOff + st * L::kKStage;
      {
        uint32_t gw[NIK][2], sb[NIK], rr[NIK], nk2[NIK];
#pragma unroll
        for (int i = 0; i < NIK; ++i) {
          if (i * kProducers + p < kHalfN * GPK) {
            const uint16_t* sk = reinterpret_cast<const uint16_t*>(pk + ksrc[i]);
            uint64_t w = 0;
            if constexpr (KB == 2) {
              w = *reinterpret_cast<const uint32_t*>(sk);  // 4-byte aligned: rows are 32 bytes, items 4
            } else {
#pragma unroll
              for (int x = 0; x < KB; ++x) w |= (uint64_t)sk[x] << (16 * x);
            }
            gw[i][0] = (uint32_t)w & ((1u << (8 * KB)) - 1);
            gw[i][1] = (uint32_t)(w >> (8 * KB));
            sb[i] = 0xffffu ^ (uint32_t)*reinterpret_cast<const uint16_t*>(pk + ksgn[i]);
            rr[i] = rho_s[ps][kkey[i]];
            nk2[i] = nk_s[ps][kkey[i]];
          }
        }
#pragma unroll
        for (int i = 0; i < NIK; ++i) {
          if (i * kProducers + p < kHalfN * GPK) {
            uint8_t* kd = Kd + kdst[i];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              uint32_t kq[4], sq[4];
              decode_group<KB>(lutK, gw[i][half], kq);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                kq[q] = tc::mul_f16x2(kq[q], nk2[i]);
                // sign bits 2q, 2q+1 of this half -> bits 15 and 31: x * (2^15 + 2^30) puts bit i of x at i + 15 and
                // i + 30; with x < 2^15 (upper half of sb is zero, shift >= 1) no two terms meet, so only the
                // unshifted case needs the two bits isolated first
                const uint32_t x = (half == 0 && q == 0) ? (sb[i] & 3u) : (sb[i] >> (8 * half + 2 * q));
                sq[q] = rr[i] ^ ((x * 0x40008000u) & 0x80008000u);
              }
              *reinterpret_cast<uint4*>(kd + half * 128) = make_uint4(kq[0], kq[1], kq[2], kq[3]);
              *reinterpret_cast<uint4*>(kd + (G + half) * 128) = make_uint4(sq[0], sq[1], sq[2], sq[3]);
            }
          }
        }
      }
      tc::fence_async_smem();
      __syncwarp();
      if (lane == 0) arrive_leader(k_full(st));
      tr.mark(3, j);
      // ---- values ----
      if (u >= 1 && !(ok = tc::mbar_wait_or_abort(v_empty(st), (u - 1) & 1, abort_flag))) break;
      if (j < 2 && !(ok = tc::mbar_wait_or_abort(qp_done, 0, abort_flag))) break;  // stages 0, 1 held the raw query tile
      tr.mark(4, j);
      uint8_t* Vd = smem_raw + L::kVOff + st * L::kVStage;
      {
        uint32_t gw[NIV][2], nv2[NIV];
#pragma unroll
        for (int i = 0; i < NIV; ++i) {
          if (i * kProducers + p < kBN * GPV) {
            const uint16_t* sv = reinterpret_cast<const uint16_t*>(pk + vsrc[i]);
            uint64_t w = 0;
            if constexpr (VB == 2) {
              w = *reinterpret_cast<const uint32_t*>(sv);
            } else if constexpr (VB == 4) {
              w = *reinterpret_cast<const uint64_t*>(sv);
            } else {
#pragma unroll
              for (int x = 0; x < VB; ++x) w |= (uint64_t)sv[x] << (16 * x);
            }
            gw[i][0] = (uint32_t)w & (VB == 4 ? 0xffffffffu : ((1u << (8 * (VB & 3))) - 1));
            gw[i][1] = (uint32_t)(w >> (8 * VB));
            nv2[i] = nv_s[ps][vkey[i]];
          }
        }
#pragma unroll
        for (int i = 0; i < NIV; ++i) {
          if (i * kProducers + p < kBN * GPV) {
            uint8_t* vd = Vd + vdst[i];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              uint32_t vq[4];
              decode_group<VB>(lutV, gw[i][half], vq);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                vq[q] = tc::mul_f16x2(vq[q], nv2[i]);
              }
              *reinterpret_cast<uint4*>(vd + half * L::kSboV) = make_uint4(vq[0], vq[1], vq[2], vq[3]);
            }
          }
        }
      }
      tc::fence_async_smem();
      __syncwarp();
      if (lane == 0) arrive_leader(v_full(st));
      tr.mark(5, j);
    }
  } else if (warp == kCtlWarp && rank == 0 && lane == 0) {
    // =============================== score MMA issuer (leader CTA) ===============================
    // Two issuing threads, because issuing one tile's 24 MMAs and their commits from a single thread took
    // longer than the softmax of a tile; every dependency between the two streams goes through an mbarrier.
    // The score and P V_hat contractions run on fp16 operands: the norms are stored as fp16, so they enter the
    // decoded key and value operands exactly, and an 11-bit significand keeps the products' rounding a factor 8
    // below bf16 (against the oracle on keys with outlier channels: 4e-3 instead of 1.3e-2)
    constexpr uint32_t idesc_s = tc::idesc_f16(2 * kBM, kBN, false, false);
    constexpr uint32_t idesc_q = tc::idesc_bf16(2 * kBM, 2 * D, false, false);
    if (n_tiles > 0) ok = tc::mbar_wait_or_abort(w_full, 0, abort_flag);
    if (ok && n_tiles > 0 && (ok = tc::mbar_wait_or_abort(qp_full, 0, abort_flag))) {
      // Q_cat (fp32, over both score tiles) = raw tile [128, D] x half of [Pi ; coeff S] from each CTA
      tc::fence_after_sync();
      const uint64_t adesc = tc::smem_desc(tc::smem_u32(smem_raw + L::kQOff), 128, L::kSboW);
      const uint64_t bdesc = tc::smem_desc(tc::smem_u32(smem_raw + L::kWOff), 128, L::kSboW);
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks)
        tc::mma_bf16_ss2(tmem_base + L::kColS, adesc + (uint64_t)(ks * 256 >> 4), bdesc + (uint64_t)(ks * 256 >> 4),
                         idesc_q, ks > 0);
      tc::mma_commit2(qp_done, 3);
    }
    if (ok && n_tiles > 0) ok = tc::mbar_wait_or_abort(q_full, 0, abort_flag);
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int bb = j & 1, st = j % kStages;
      tr.mark(0, j);
      if (!(ok = tc::mbar_wait_or_abort(k_full(st), (j / kStages) & 1, abort_flag))) break;
      // S[bb] is free once P[bb] of tile j-2, which lives in the same columns, has been consumed
      if (j >= 2 && !(ok = tc::mbar_wait_or_abort(pv_done(bb), ((j - 2) >> 1) & 1, abort_flag))) break;
      tr.mark(1, j);
      tc::fence_after_sync();
      const uint64_t kdesc = tc::smem_desc(tc::smem_u32(smem_raw + L::kKOff + st * L::kKStage), 128, L::kSboK);
#pragma unroll
      for (int ks = 0; ks < 2 * D / 16; ++ks)
        tc::mma_bf16_ts2(tmem_base + L::kColS + bb * kBN, tmem_base + L::kColQ + ks * 8,
                         kdesc + (uint64_t)(ks * 256 >> 4), idesc_s, ks > 0);
      tc::mma_commit2(s_full(bb), 3);
      tc::mma_commit2(k_empty(st), 3);
      tr.mark(2, j);
    }
  } else if (warp == kCtlWarp && lane == 0) {
    // peer CTA: tell the leader when this half of [Pi ; coeff S] has landed
    if (n_tiles > 0 && (ok = tc::mbar_wait_or_abort(w_full, 0, abort_flag))) arrive_leader(qp_full);
  } else if (warp == kPvWarp && rank != 0 && lane == 0) {
    // peer CTA: ... and this half of Pi_v^T
    if (n_tiles > 0 && (ok = tc::mbar_wait_or_abort(u_full, 0, abort_flag))) arrive_leader(u_peer);
  } else if (warp == kPvWarp && rank == 0 && lane == 0) {
    // =============================== P V_hat MMA issuer (leader CTA) ===============================
    constexpr uint32_t idesc_o = tc::idesc_f16(2 * kBM, D, false, true);
    constexpr uint32_t idesc_e = tc::idesc_bf16(2 * kBM, D, false, false);
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int bb = j & 1, u = j >> 1, st = j % kStages;
      tr.mark(3, j);
      if (!(ok = tc::mbar_wait_or_abort(v_full(st), (j / kStages) & 1, abort_flag))) break;
      tr.mark(4, j);
      if (!(ok = tc::mbar_wait_or_abort(p_full(bb), u & 1, abort_flag))) break;
      tc::fence_after_sync();
      tr.mark(5, j);
      const uint64_t vdesc = tc::smem_desc(tc::smem_u32(smem_raw + L::kVOff + st * L::kVStage), L::kLboV, L::kSboV);
#pragma unroll
      for (int ks = 0; ks < kBN / 16; ++ks)
        tc::mma_bf16_ts2(tmem_o, tmem_base + L::kColS + bb * kBN + ks * 8, vdesc + (uint64_t)(ks * 2 * L::kLboV >> 4),
                         idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
      tc::mma_commit2(pv_done(bb), 3);
      tc::mma_commit2(v_empty(st), 3);
      tr.mark(6, j);
    }
    if (ok && n_tiles > 0) ok = tc::mbar_wait_or_abort(u_full, 0, abort_flag) && tc::mbar_wait_or_abort(u_peer, 0, abort_flag);
    if (ok && n_tiles > 0 && (ok = tc::mbar_wait_or_abort(q_full, 1, abort_flag))) {
      // out tile (fp32, second score tile) = normalised bf16 output tile x Pi_v
      tc::fence_after_sync();
      const uint64_t bdesc = tc::smem_desc(tc::smem_u32(smem_raw + L::kUOff), 128, L::kSboW);
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks)
        tc::mma_bf16_ts2(tmem_base + L::kColS + kBN, tmem_base + L::kColS + ks * 8, bdesc + (uint64_t)(ks * 256 >> 4),
                         idesc_e, ks > 0);
      tc::mma_commit2(e_done, 3);
    }
  }
  if (!ok && atomicExch(&s_abort, 2) != 2) {  // one fault per CTA
    atomicAdd(&g_c2_faults, 1ull);
    notify_host_of_fault(g_fault_mailbox_c2);
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::cluster_sync_relaxed();  // neither CTA leaves (or frees tensor memory) while the pair's MMAs or signals may touch it
  if (warp == kCtlWarp) tc::tmem_dealloc2(tmem_base, L::kCols);
}

template <int D, int BITS>
int launch_c2(const AttnArgs& a, const PairArgs& x, int64_t B, cudaStream_t stream) {
  constexpr size_t smem = C2Smem<D, BITS>::kTotal > 120 * 1024 ? C2Smem<D, BITS>::kTotal : 120 * 1024;
#ifdef TQ_B200_TRACE  // diagnostics build only: the product library carries one instantiation per (d, bits)
  auto kern = g_trace2_host_on ? attention_c2_kernel<D, BITS, true> : attention_c2_kernel<D, BITS, false>;
#else
  auto kern = attention_c2_kernel<D, BITS, false>;
#endif
  TQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int pair_heads = ((a.Hq / a.Hkv) % 2 == 0) ? 1 : 0;
  const int64_t blocks = (a.Sq + kBM - 1) / kBM;
  // x: 2 CTAs (one cluster) per pair of query tiles
  dim3 grid((unsigned)(2 * (pair_heads ? blocks : (blocks + 1) / 2)), (unsigned)(pair_heads ? a.Hq / 2 : a.Hq),
            (unsigned)B);
  {
    ProfScope prof(kProfAttention, stream);
    kern<<<grid, kThreads, smem, stream>>>(a, x, pair_heads);
  }
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
}

}  // namespace

int attention_c2(const AttnArgs& a, const PairArgs& x, int64_t B, int d, int bits, cudaStream_t stream) {
  if (d == 128)
    return bits == 2 ? launch_c2<128, 2>(a, x, B, stream) : bits == 3 ? launch_c2<128, 3>(a, x, B, stream)
                                                                      : launch_c2<128, 4>(a, x, B, stream);
  if (d == 64)
    return bits == 2 ? launch_c2<64, 2>(a, x, B, stream) : bits == 3 ? launch_c2<64, 3>(a, x, B, stream)
                                                                    : launch_c2<64, 4>(a, x, B, stream);
  return fail(TQ_ERR_UNSUPPORTED, "the SM-pair attention kernel is built for head_dim 64 and 128 only");
}

}  // namespace tq
