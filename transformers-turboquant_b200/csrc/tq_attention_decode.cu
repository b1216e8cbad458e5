// Split-KV compressed attention for decode-sized calls: few query rows per KV head (G * Sq <= 16), long
// keys.  There is no counterpart in the reference, which disables the KV cache and recomputes full
// attention per generated token (patch.py:80-81); this serves a cache kept in the library's wire format.
//
// Three launches per call: `decode_prepare_kernel` (q_cat = [q Pi^T | coeff q Pi^T S^T], fp32), `decode_kernel`
// (below) and `decode_finish_kernel` (merge of the splits + back-rotation by Pi_v, fp32).
//
// The work is bound by the packed bytes (about 100 B per key at 3 bits) and by the instructions that turn them
// into tensor-core operands, not by the contractions, so the keys of one (batch, KV head) are split over
// `nsplit` CTAs and every CTA streams its range once (packed rows and fp16 norms copied three blocks ahead
// with cp.async):
//   * everything is computed TRANSPOSED, so that the few query rows are the N = 8 dimension of
//     mma.sync.m16n8k16 (bf16, fp32 accumulation) and the long dimensions fill M = 16:
//     S^T (16 keys x 8 query rows) = K_hat Q^T and O^T (16 coordinates x 8 query rows) += V_hat^T P^T.
//     One tile of eight query rows (NT = 1) keeps its Q^T fragments in registers; 9..16 rows take two tiles;
//   * a warp takes 16 keys at a time and decodes K_hat = [C[idx] ; sign] STRAIGHT INTO the A fragments -- no
//     shared-memory operand tile, each element is decoded exactly once by the lane that feeds it to the tensor
//     core.  The contraction index of an MMA may be permuted freely as long as both operands agree, so lane t of
//     a quad owns coordinates 32 t .. 32 t + 31 of its two keys (contiguous bits of a packed row, one or two
//     words) and its four k-slots of k-step j are coordinates 32 t + 4 j .. + 3: two adjacent indices are one
//     look-up in a per-lane copy of a bf16-pair table (no bank conflicts), four adjacent sign bits one 64-bit
//     look-up.  The centroid half and the sign half accumulate separately and meet in fp32 as
//     n <q Pi^T, C[idx]> + rn <q S^T, sign>, so the sign operand is exactly +-1;
//   * online softmax on the C fragments (maxima over the keys by three shuffles across the lane groups,
//     running maximum raised lazily);
//   * P^T (bf16, with the value norms folded in) becomes the B fragment of the second MMA by one 8x8
//     transpose across the warp (movmatrix) per eight keys;
//   * the row index of the second MMA may be permuted too: lane group g owns coordinates 16 g .. 16 g + 15,
//     contiguous bits of a packed value row; two adjacent indices are one look-up (a bf16 pair along the
//     coordinate) and a byte permute per A register turns two keys' pairs into the pairs along the key that
//     the fragment wants;
//   * the four warps of a CTA merge through shared memory, the splits through a small fp32 workspace.
// The legacy tensor-core path is deliberate here: eight or sixteen query rows do not fill a tcgen05 tile, and
// what has to be fast is the decode around the MMA, not the MMA.
#include <math.h>
#include <stdlib.h>

#include <type_traits>

#include "tq_attention.cuh"
#include "tq_common.cuh"
#include "tq_simt.cuh"

namespace tq {
namespace {

constexpr int kRows = 16;        // most query rows per KV head (two N tiles of the MMA)
constexpr int kWarps = 4;
constexpr int kBlockKeys = 16;   // keys per warp iteration
constexpr int kMaxExtraUnits = 640;  // bound on the CTAs the splits are sized for (resident CTAs of the device)
constexpr int kDecodeStages = 3; // packed-row buffers per warp: the block in use and the copies in flight
constexpr int kQPitch = 2 * 128 + 16;  // bf16 elements per staged query row: rows 8 banks apart, so the
                                        // 64-bit loads of a half warp (4 rows x 4 lanes) hit 32 different banks

struct DecodeArgs {
  const __nv_bfloat16* q_cat;  // [B*Hq*Sq, 2d]
  int64_t Hq, Hkv, Sq, Sk, kv_stride;
  const uint8_t* key_idx;
  const uint8_t* key_sgn;
  const uint16_t* key_vn;
  const uint16_t* key_rn;
  const uint8_t* val_idx;
  const uint16_t* val_vn;
  const float* cen_k;
  const float* cen_v;
  float sm_scale;
  int causal;
  const float* mask;  // optional additive mask, element (b, s, k) at mask[b * mask_stride_b + s * mask_stride_q + k]
  int64_t mask_stride_b, mask_stride_q;
  float* part_o;   // [B*Hkv, nsplit, 16, d]
  float* part_ml;  // [B*Hkv, nsplit, 16, 2]  (running maximum, row sum)
  int nsplit, keys_per_split;
};

__device__ __forceinline__ uint32_t bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Programmatic dependent launch: `wait` returns when the grid this one depends on has completed and its writes
// are visible (at once when the kernel was launched without the attribute); `launch_dependents` lets the next
// kernel of the stream start early, up to its own `wait`.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// 8x8 transpose of 16-bit elements across the warp: lane (g, t) gives row g, columns 2 t, 2 t + 1 and receives
// column g, rows 2 t, 2 t + 1
__device__ __forceinline__ uint32_t transpose8x8(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}
// D (16x8, fp32) += A (16x16, bf16, row) * B (16x8, bf16, col)
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// f(integral_constant<int, I>) for I = FROM .. TO-1: a loop whose index is usable as a template argument
template <int FROM, int TO, class F>
__device__ __forceinline__ void static_for(F&& f) {
  if constexpr (FROM < TO) {
    f(std::integral_constant<int, FROM>{});
    static_for<FROM + 1, TO>(f);
  }
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_all_but() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// (field << SH) for the NBITS-bit field at compile-time bit BIT of a little-endian word array: the byte offset of
// entry `field` in a table whose entries are 2^SH bytes apart.  One shift and one mask; a funnel shift first
// when the field straddles two words.
template <int BIT, int NBITS, int SH, int NW>
__device__ __forceinline__ uint32_t scaled_field(const uint32_t (&w)[NW]) {
  constexpr int word = BIT / 32, bo = BIT % 32;
  constexpr uint32_t mask = ((1u << NBITS) - 1) << SH;
  static_assert(SH + NBITS <= 32 && word < NW, "field out of range");
  if constexpr (bo + NBITS <= 32) {
    if constexpr (bo > SH) return (w[word] >> (bo - SH)) & mask;
    else if constexpr (bo < SH) return (w[word] << (SH - bo)) & mask;
    else return w[word] & mask;
  } else {
    static_assert(bo + NBITS <= 32 || (bo >= SH && word + 1 < NW), "straddling field");
    return __funnelshift_r(w[word], w[word + 1 < NW ? word + 1 : word], bo - SH) & mask;
  }
}

// Shared-memory tables of the decode.  Every table is replicated so that the lanes of a warp read different
// banks whatever their indices are (entry e, copy k at byte (e * COPIES + k) * ENTRY); the byte offset of a
// look-up is `lane's copy | scaled_field`.
template <int BITS>
struct Tables {
  static constexpr int KB = BITS - 1, VB = BITS;
  // keys: two adjacent indices -> one operand register (a bf16 pair along the coordinate), one copy per lane.
  // A wider entry, four indices -> two registers by one 64-bit load, saves instructions but needs a copy per
  // lane of a half warp to stay free of bank conflicts: that fits for 1-bit indices (16 entries) and is used
  // there; for 2-bit indices (256 entries) only 8 copies fit, its loads collide and it measured slower.
  static constexpr bool kQuad = KB == 1;
  static constexpr int kIdxBitsK = kQuad ? 4 * KB : 2 * KB;
  static constexpr int kEntryK = kQuad ? 8 : 4;
  static constexpr int kCopiesK = kQuad ? 16 : 32;
  static constexpr int kShiftK = 7;  // log2(kEntryK * kCopiesK)
  static constexpr int kBytesK = (1 << kIdxBitsK) * kEntryK * kCopiesK;
  // signs: four adjacent sign bits -> two registers of +-1 pairs by one 64-bit load; the 16 entries cover the
  // 32 banks exactly once, so no copies are needed
  static constexpr int kBytesS = 16 * 8;
  // values: two adjacent indices -> a bf16 pair along the coordinate
  static constexpr int kCopiesV = VB == 4 ? 8 : 32;
  static constexpr int kShiftV = VB == 4 ? 5 : 7;  // log2(4 * kCopiesV)
  static constexpr int kBytesV = (1 << (2 * VB)) * 4 * kCopiesV;
  static_assert((1 << kShiftK) == kEntryK * kCopiesK && (1 << kShiftV) == 4 * kCopiesV, "table strides");
};

template <int BITS, int NT, bool MASK>
__global__ void __launch_bounds__(kWarps * 32, 4) decode_kernel(const DecodeArgs a) {
  using T = Tables<BITS>;
  constexpr bool kQInRegs = NT == 1;
  constexpr int D = 128, KB = BITS - 1, VB = BITS;
  constexpr float kLog2e = 1.4426950408889634f;
  // packed bytes of the block a warp works on and of the ones after it (copied ahead with cp.async):
  // 16 key-index rows, 16 sign rows, 16 value-index rows
  // + the fp16 norms of the 16 keys: key vector norms, residual norms, value vector norms (32 bytes each)
  constexpr int kRowBytes = kBlockKeys * 16 * (KB + 1 + VB);
  constexpr int kStageBytes = kRowBytes + 128;
  constexpr int kStages = BITS == 4 ? 2 : kDecodeStages;
  constexpr int kQBytes = kRows * kQPitch * 2;
  constexpr int kMergeBytes = kWarps * 8 * (D + 4) * 4;  // eight rows at a time
  constexpr int kLoopBytes = kQBytes + kWarps * kStages * kStageBytes;
  // One shared array: the tables, the merge bookkeeping, then a pool: staged queries + packed-row stages while the keys stream, the warps'
  // partial outputs afterwards.
  constexpr int kOffK = 0, kOffV = T::kBytesK;
  constexpr int kOffS = T::kBytesK + T::kBytesV;
  constexpr int kOffMl = kOffS + T::kBytesS;       // [kWarps][kRows][2] floats
  constexpr int kOffPool = kOffMl + kWarps * kRows * 2 * 4;
  constexpr int kPoolBytes = kLoopBytes > kMergeBytes ? kLoopBytes : kMergeBytes;
  static_assert(kOffPool % 16 == 0 && kOffPool + kPoolBytes <= 48 * 1024, "static shared memory");
  __shared__ __align__(128) uint8_t smem[kOffPool + kPoolBytes];
  uint8_t* lutK = smem + kOffK;
  uint8_t* lutV = smem + kOffV;
  uint8_t* lutS = smem + kOffS;
  float (*mrg_ml)[kRows][2] = reinterpret_cast<float (*)[kRows][2]>(smem + kOffMl);
  uint8_t* pool = smem + kOffPool;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(pool);
  auto stage_ptr = [&](int w, int st) { return pool + kQBytes + (w * kStages + st) * kStageBytes; };
  float (*mrg_o)[8][D + 4] = reinterpret_cast<float (*)[8][D + 4]>(pool);

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int gq = lane / 4, tq = lane % 4;
  const int split = blockIdx.x;
  const int64_t kvh = blockIdx.y, b = blockIdx.z;
  const int G = (int)(a.Hq / a.Hkv), R = G * (int)a.Sq;
  const int64_t kv_base = (b * a.Hkv + kvh) * a.kv_stride;
  const int shift = (int)(a.Sk - a.Sq);

  // ---- build the tables (nothing here depends on the kernel launched before this one) ----
  {
    constexpr uint32_t km = (1u << KB) - 1, vm = (1u << VB) - 1;
    for (int e = tid; e < (1 << T::kIdxBitsK) * T::kCopiesK; e += kWarps * 32) {
      const uint32_t i = e / T::kCopiesK;
      uint32_t* dst = reinterpret_cast<uint32_t*>(lutK + e * T::kEntryK);
      dst[0] = bf16x2(__ldg(a.cen_k + (i & km)), __ldg(a.cen_k + ((i >> KB) & km)));
      if constexpr (T::kQuad) dst[1] = bf16x2(__ldg(a.cen_k + ((i >> (2 * KB)) & km)), __ldg(a.cen_k + ((i >> (3 * KB)) & km)));
    }
    for (int e = tid; e < (1 << (2 * VB)) * T::kCopiesV; e += kWarps * 32) {
      const uint32_t i = e / T::kCopiesV;
      reinterpret_cast<uint32_t*>(lutV)[e] = bf16x2(__ldg(a.cen_v + (i & vm)), __ldg(a.cen_v + (i >> VB)));
    }
    if (tid < 16) {  // a set bit is a positive sign
      const uint32_t pos = 0x3f80u, neg = 0xbf80u;
      reinterpret_cast<uint2*>(lutS)[tid] = make_uint2(((tid & 1) ? pos : neg) | (((tid & 2) ? pos : neg) << 16),
                                                       ((tid & 4) ? pos : neg) | (((tid & 8) ? pos : neg) << 16));
    }
  }
  // a look-up address is (table address) + (lane's copy | entry): the tables are indexed as plain static shared
  // arrays, so the first term is the load's immediate; the second is one three-input logic operation on the
  // shifted packed word.  (Loads through an explicit 32-bit shared address cost one more add per look-up.)
  const uint32_t lane4 = (uint32_t)(lane * 4), laneV = (uint32_t)((lane % T::kCopiesV) * 4);
  const uint32_t laneK = (uint32_t)((lane % T::kCopiesK) * T::kEntryK);

  // Query rows are the N dimension of every MMA (tiles of 8): NT = 1 serves up to 8 rows, NT = 2 up to 16.  Rows
  // past R hold zero queries; their results are never read, so they are not masked.  Masking is needed only in
  // blocks that reach past the first visible limit, which is the same for the whole warp.
  // This lane's columns of the score / output fragments are query rows 8 t + 2 tq + e, e = 0, 1.
  int row_lim[NT][2];  // last visible key of the row (causal), or Sk - 1
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int r = 8 * t + 2 * tq + e;
      row_lim[t][e] = (r < R && a.causal) ? (r % (int)a.Sq) + shift : (int)a.Sk - 1;
    }
  const int lim_min = a.causal ? shift : (int)a.Sk - 1;
  const float cexp = a.sm_scale * kLog2e;
  // O^T fragments: o[t][ct][i] is coordinate 16 gq + 2 ct + (i >> 1) of query row 8 t + 2 tq + (i & 1)
  float o[NT][D / 16][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int ct = 0; ct < D / 16; ++ct)
#pragma unroll
      for (int i = 0; i < 4; ++i) o[t][ct][i] = 0.f;
  float m_run[NT][2], l_run[NT][2];  // l_run: this lane's keys only until the end
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      m_run[t][e] = -INFINITY;
      l_run[t][e] = 0.f;
    }
  const int k_lo = split * a.keys_per_split;
  const int k_hi = min((int)a.Sk, k_lo + a.keys_per_split);
  const uint8_t* kidx_base = a.key_idx + kv_base * (16 * KB);
  const uint8_t* ksgn_base = a.key_sgn + kv_base * 16;
  const uint8_t* vidx_base = a.val_idx + kv_base * (16 * VB);
  // two adjacent fp16 norms are one 4-byte copy when that copy is aligned
  const bool pair_ok = (kv_base & 1) == 0 && ((reinterpret_cast<uintptr_t>(a.key_vn) | reinterpret_cast<uintptr_t>(a.key_rn) |
                                               reinterpret_cast<uintptr_t>(a.val_vn)) & 3) == 0;
  const uint16_t* norm_src = (lane < 8 ? a.key_vn : lane < 16 ? a.key_rn : a.val_vn) + kv_base + 2 * (lane % 8);
  // copy the packed rows of keys [blk, blk + 16) into stage `st` (rows of consecutive keys are contiguous in
  // each array, 16 (KB + 1 + VB) = 32 BITS units of 16 bytes); rows past the end of the sequence become zeros
  // unit u = lane + 32 it of a stage (it < BITS) is 16 bytes of one array: where it starts for block 0, how far
  // it moves per key, and which key of the block it belongs to
  const uint8_t* unit_src[BITS];
  int unit_step[BITS], unit_key[BITS];
#pragma unroll
  for (int it = 0; it < BITS; ++it) {
    constexpr int UK = kBlockKeys * KB, US = kBlockKeys;  // 16-byte units of index and sign rows; value rows follow
    const int u = lane + 32 * it;
    if (u < UK) { unit_src[it] = kidx_base + 16 * u; unit_step[it] = 16 * KB; unit_key[it] = u / KB; }
    else if (u < UK + US) { unit_src[it] = ksgn_base + 16 * (u - UK); unit_step[it] = 16; unit_key[it] = u - UK; }
    else { unit_src[it] = vidx_base + 16 * (u - UK - US); unit_step[it] = 16 * VB; unit_key[it] = (u - UK - US) / VB; }
  }
  auto stage = [&](int blk, int st) {
    uint8_t* dst = stage_ptr(warp, st);
    const bool whole = blk + kBlockKeys <= (int)a.Sk;
#pragma unroll
    for (int it = 0; it < BITS; ++it) {
      uint8_t* d = dst + 16 * (lane + 32 * it);
      if (whole || blk + unit_key[it] < a.Sk) cp_async16(d, unit_src[it] + (int64_t)blk * unit_step[it]);
      else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
    }
    // norms: lanes 0..23 copy one aligned pair of fp16 each; ragged or unaligned blocks go element by element
    // (the block is used a later iteration, after a __syncwarp)
    uint8_t* nd = dst + kRowBytes;
    if (pair_ok && whole) {
      if (lane < 24) cp_async4(nd + 4 * lane, norm_src + blk);
    } else {
      for (int u = lane; u < 3 * kBlockKeys; u += 32) {
        const int arr = u / kBlockKeys, key = blk + u % kBlockKeys;
        const uint16_t* src = arr == 0 ? a.key_vn : arr == 1 ? a.key_rn : a.val_vn;
        reinterpret_cast<uint16_t*>(nd)[u] = key < a.Sk ? src[kv_base + key] : (uint16_t)0;
      }
    }
  };
  // blocks of this warp: blk0, blk0 + 64, ...; their packed rows are copied kStages - 1 blocks ahead
  const int blk0 = k_lo + kBlockKeys * warp;
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    const int pb = blk0 + s * kBlockKeys * kWarps;
    if (pb < k_hi) stage(pb, s);
    cp_async_commit();
  }
  // The query rows come from the kernel launched just before this one.  With programmatic dependent launch this
  // kernel may have started while that one was still running: everything above (tables, the first copies of
  // packed rows) overlapped with it, and this is where its results are waited for.
  grid_dependency_wait();
  // ---- stage the query rows (row r = g * Sq + s of query head kvh * G + g) ----
  // Within each half of a row (rotated coordinates, sketch coordinates) coordinate 32 t + 4 j + e is stored at
  // 16 j + 4 t + e: lane t of a quad owns coordinates 32 t .. 32 t + 31 (contiguous bits of a packed row), and
  // its four coordinates of k-step j are one 64-bit load.
  for (int e = tid; e < kRows * (2 * D / 8); e += kWarps * 32) {
    const int r = e / (2 * D / 8), m = e % (2 * D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < R) {
      const int64_t h = kvh * G + r / a.Sq, s = r % a.Sq;
      v = reinterpret_cast<const uint4*>(a.q_cat + ((b * a.Hq + h) * a.Sq + s) * (2 * D))[m];
    }
    const int half = m / 16, mm = m % 16;  // coordinates 8 mm .. 8 mm + 7 of the half: t = mm / 4, j = 2 (mm % 4), + 1
    __nv_bfloat16* dst = &q_s[r * kQPitch + 128 * half + 32 * (mm % 4) + 4 * (mm / 4)];
    *reinterpret_cast<uint2*>(dst) = make_uint2(v.x, v.y);
    *reinterpret_cast<uint2*>(dst + 16) = make_uint2(v.z, v.w);
  }
  __syncthreads();  // tables and query rows are complete
  // B fragments of Q^T (k-slots of k-step ks x query row gq of tile t): kept in registers when one tile is all
  uint2 qr[kQInRegs ? 16 : 1];
  if constexpr (kQInRegs) {
#pragma unroll
    for (int ks = 0; ks < 16; ++ks) qr[ks] = *reinterpret_cast<const uint2*>(&q_s[gq * kQPitch + 16 * ks + 4 * tq]);
  }
  int st = 0;
  for (int blk = blk0; blk < k_hi; blk += kBlockKeys * kWarps, st = (st + 1 == kStages ? 0 : st + 1)) {
    {
      const int pb = blk + (kStages - 1) * kBlockKeys * kWarps;
      if (pb < k_hi) stage(pb, st == 0 ? kStages - 1 : st - 1);  // the stage the previous iteration read
      cp_async_commit();
      cp_async_wait_all_but<kStages - 1>();  // this block's rows have landed; later blocks' may still be in flight
      __syncwarp();
    }
    const uint8_t* stg = stage_ptr(warp, st);
    // additive mask of this lane's score elements (query row 8 t + 2 tq + e, keys blk + gq, + 8), loaded ahead of
    // the decode work that hides its latency
    float mk[MASK ? NT : 1][4];
    if constexpr (MASK) {
#pragma unroll
      for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = 8 * t + 2 * tq + (i & 1), key = blk + gq + 8 * (i >> 1);
          // kept finite, as the large negative value HF masks with is: a row whose keys are all masked then
          // averages them uniformly, as it does in the prefill kernels and in the reference's softmax
          mk[t][i] = (r < R && key < (int)a.Sk)
                         ? fmaxf(__ldg(a.mask + b * a.mask_stride_b + (r % (int)a.Sq) * a.mask_stride_q + key) * kLog2e,
                                 -3.0e38f)
                         : 0.f;
        }
    }
    // ============ scores, transposed: S^T (16 keys x 8 query rows per tile); centroid half s1, sign half s2 ============
    float s1[NT][4], s2[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s1[t][i] = 0.f;
        s2[t][i] = 0.f;
      }
    {
      // this lane's share of keys blk + gq and blk + 8 + gq (rows gq, gq + 8 of the A operand): the packed indices
      // of coordinates 32 tq .. 32 tq + 31 (4 KB bytes at byte 4 KB tq of the row) and the sign bits of the same
      // sketch coordinates (word tq)
      uint32_t kw[2][KB], sg[2][1];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint8_t* row = stg + (8 * h + gq) * (16 * KB) + 4 * KB * tq;
        if constexpr (KB == 2) {
          const uint2 v = *reinterpret_cast<const uint2*>(row);
          kw[h][0] = v.x; kw[h][1] = v.y;
        } else {
#pragma unroll
          for (int i = 0; i < KB; ++i) kw[h][i] = reinterpret_cast<const uint32_t*>(row)[i];
        }
        sg[h][0] = reinterpret_cast<const uint32_t*>(stg + kBlockKeys * 16 * KB + (8 * h + gq) * 16)[tq];
      }
      static_for<0, 16>([&](auto ks_c) {
        constexpr int ks = decltype(ks_c)::value, j = ks % 8;
        // k-slots (2 tq, 2 tq + 1, 2 tq + 8, 2 tq + 9) of this k-step = coordinates 32 tq + 4 j .. + 3 of the half;
        // A registers: a0 / a2 = row gq, first / second slot pair; a1 / a3 = row gq + 8
        uint32_t ka[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if constexpr (ks >= 8) {
            const uint2 e = *reinterpret_cast<const uint2*>(lutS + scaled_field<4 * j, 4, 3>(sg[h]));
            ka[h] = e.x; ka[2 + h] = e.y;
          } else if constexpr (T::kQuad) {
            const uint2 e = *reinterpret_cast<const uint2*>(lutK + (laneK | scaled_field<4 * KB * j, 4 * KB, T::kShiftK>(kw[h])));
            ka[h] = e.x; ka[2 + h] = e.y;
          } else {
            ka[h] = *reinterpret_cast<const uint32_t*>(lutK + (lane4 | scaled_field<4 * KB * j, 2 * KB, T::kShiftK>(kw[h])));
            ka[2 + h] = *reinterpret_cast<const uint32_t*>(lutK + (lane4 | scaled_field<4 * KB * j + 2 * KB, 2 * KB, T::kShiftK>(kw[h])));
          }
        }
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          uint2 qb;
          if constexpr (kQInRegs) qb = qr[ks];
          else qb = *reinterpret_cast<const uint2*>(&q_s[(8 * t + gq) * kQPitch + 16 * ks + 4 * tq]);
          if constexpr (ks >= 8) mma16816(s2[t], ka, qb.x, qb.y);
          else mma16816(s1[t], ka, qb.x, qb.y);
        }
      });
    }
    // ================= online softmax on the fragments =================
    // s[t][i]: key blk + gq + 8 (i >> 1), query row 8 t + 2 tq + (i & 1)
    // score * sm_scale * log2(e) = cexp (n <q Pi^T, C[idx]> + rn <q S^T, sign>), all in fp32
    const uint16_t* nrm = reinterpret_cast<const uint16_t*>(stg + kRowBytes);  // [3][16] fp16: n, rn, value n
    float mx[NT][2];
    {
      float kn[2], rn[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        kn[h] = fp16_value(nrm[gq + 8 * h]) * cexp;
        rn[h] = fp16_value(nrm[16 + gq + 8 * h]) * cexp;
      }
      const bool need_mask = blk + kBlockKeys - 1 > lim_min;
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        mx[t][0] = -INFINITY;
        mx[t][1] = -INFINITY;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int h = i >> 1, e = i & 1;
          float x = fmaf(s2[t][i], rn[h], s1[t][i] * kn[h]);
          if constexpr (MASK) x += mk[t][i];
          if (need_mask && blk + gq + 8 * h > row_lim[t][e]) x = -INFINITY;
          s1[t][i] = x;
          mx[t][e] = fmaxf(mx[t][e], x);
        }
      }
    }
    bool grow_lane = false;
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int e = 0; e < 2; ++e) {  // the 16 keys of a query row sit in the 8 lane groups
        mx[t][e] = fmaxf(mx[t][e], __shfl_xor_sync(0xffffffffu, mx[t][e], 4));
        mx[t][e] = fmaxf(mx[t][e], __shfl_xor_sync(0xffffffffu, mx[t][e], 8));
        mx[t][e] = fmaxf(mx[t][e], __shfl_xor_sync(0xffffffffu, mx[t][e], 16));
        grow_lane |= mx[t][e] > m_run[t][e] + 8.f;
      }
    // running maximum raised lazily (only when some row of the warp outgrew it by 2^8)
    if (__any_sync(0xffffffffu, grow_lane)) {
#pragma unroll
      for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float m_new = fmaxf(m_run[t][e], mx[t][e]);
          const float alpha = (m_run[t][e] == -INFINITY) ? 0.f : ex2(m_run[t][e] - m_new);
          m_run[t][e] = m_new;
          l_run[t][e] *= alpha;
#pragma unroll
          for (int ct = 0; ct < D / 16; ++ct) {
            o[t][ct][e] *= alpha;
            o[t][ct][2 + e] *= alpha;
          }
        }
    }
    // P^T, with the value norms folded in for the MMA (the row sum uses the plain probabilities).  The C fragment
    // of S^T (key rows, query columns) becomes the B fragment of the next MMA (key k-slots, query column gq) by
    // one 8x8 transpose across the warp per eight keys.
    uint32_t pb[NT][2];
    {
      const float nv[2] = {fp16_value(nrm[32 + gq]), fp16_value(nrm[32 + gq + 8])};
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        float p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int h = i >> 1, e = i & 1;
          const float pv = ex2(s1[t][i] - (m_run[t][e] == -INFINITY ? 0.f : m_run[t][e]));
          l_run[t][e] += pv;
          p[i] = pv * nv[h];
        }
        pb[t][0] = transpose8x8(bf16x2(p[0], p[1]));  // keys blk + 2 tq, + 1       of query row 8 t + gq
        pb[t][1] = transpose8x8(bf16x2(p[2], p[3]));  // keys blk + 8 + 2 tq, + 1   of query row 8 t + gq
      }
    }
    // ================= O^T += V_hat^T P^T =================
    // Row m of MMA tile ct is any coordinate we like: lane group gq owns coordinates 16 gq .. 16 gq + 15
    // (16 VB contiguous bits of a packed row), tile ct takes 16 gq + 2 ct (row gq) and 16 gq + 2 ct + 1 (row gq + 8).
    // The k-slots are this lane's four keys blk + 2 tq, + 1, + 8 + 2 tq, + 9 + 2 tq.
    {
      uint32_t vw[4][2];
#pragma unroll
      for (int kq = 0; kq < 4; ++kq) {
        const uint8_t* row = stg + kBlockKeys * 16 * (KB + 1) + (8 * (kq >> 1) + 2 * tq + (kq & 1)) * (16 * VB);
        if constexpr (VB == 2) {
          vw[kq][0] = reinterpret_cast<const uint32_t*>(row)[gq];
          vw[kq][1] = 0;
        } else if constexpr (VB == 4) {
          const uint2 v = reinterpret_cast<const uint2*>(row)[gq];
          vw[kq][0] = v.x;
          vw[kq][1] = v.y;
        } else {  // 6 bytes at byte 6 gq: two words, then 0 or 16 bits down
          const uint32_t* w = reinterpret_cast<const uint32_t*>(row) + ((6 * gq) >> 2);
          const uint32_t w0 = w[0], w1 = w[1], sh = 16 * (gq & 1);
          vw[kq][0] = __funnelshift_r(w0, w1, sh);
          vw[kq][1] = w1 >> sh;
        }
      }
      static_for<0, D / 16>([&](auto ct_c) {
        constexpr int ct = decltype(ct_c)::value;
        // indices 2 ct, 2 ct + 1 of the lane's 16: one look-up per key gives the bf16 pair along the coordinate; the
        // fragment wants pairs along the key
        uint32_t e[4];
#pragma unroll
        for (int kq = 0; kq < 4; ++kq)
          e[kq] = *reinterpret_cast<const uint32_t*>(lutV + (laneV | scaled_field<2 * VB * ct, 2 * VB, T::kShiftV>(vw[kq])));
        const uint32_t va[4] = {__byte_perm(e[0], e[1], 0x5410), __byte_perm(e[0], e[1], 0x7632),
                                __byte_perm(e[2], e[3], 0x5410), __byte_perm(e[2], e[3], 0x7632)};
#pragma unroll
        for (int t = 0; t < NT; ++t) mma16816(o[t][ct], va, pb[t][0], pb[t][1]);
      });
    }
    __syncwarp();  // every lane is done with this stage before a later iteration refills it
  }

  // ---- merge: lane groups (row sums), the four warps, then this split's partial result ----
  grid_launch_dependents();  // the finishing kernel may start its own set-up; it waits for this grid to end
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      l_run[t][e] += __shfl_xor_sync(0xffffffffu, l_run[t][e], 4);
      l_run[t][e] += __shfl_xor_sync(0xffffffffu, l_run[t][e], 8);
      l_run[t][e] += __shfl_xor_sync(0xffffffffu, l_run[t][e], 16);
    }
  const int64_t unit = (b * a.Hkv + kvh) * a.nsplit + split;
  // eight query rows (one tile) at a time: the pool changes hands at each barrier
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    __syncthreads();  // every warp is done with the queries and its stages / with the previous eight rows
#pragma unroll
    for (int ct = 0; ct < D / 16; ++ct)
#pragma unroll
      for (int i = 0; i < 4; ++i) mrg_o[warp][2 * tq + (i & 1)][16 * gq + 2 * ct + (i >> 1)] = o[t][ct][i];
    if (gq == 0) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        mrg_ml[warp][8 * t + 2 * tq + e][0] = m_run[t][e];
        mrg_ml[warp][8 * t + 2 * tq + e][1] = l_run[t][e];
      }
    }
    __syncthreads();
    for (int e = tid; e < 8 * D; e += kWarps * 32) {
      const int r8 = e / D, c = e % D, r = r8 + 8 * t;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) m = fmaxf(m, mrg_ml[w][r][0]);
      float acc = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const float mw = mrg_ml[w][r][0];
        const float f = (mw == -INFINITY) ? 0.f : ex2(mw - m);
        acc = fmaf(mrg_o[w][r8][c], f, acc);
        l = fmaf(mrg_ml[w][r][1], f, l);
      }
      a.part_o[(unit * kRows + r) * D + c] = acc;
      if (c == 0) {
        a.part_ml[(unit * kRows + r) * 2] = m;
        a.part_ml[(unit * kRows + r) * 2 + 1] = l;
      }
    }
  }
}

__device__ __forceinline__ float load_elem(const void* base, int dtype, int64_t off) {
  if (dtype == TQ_F32) return static_cast<const float*>(base)[off];
  if (dtype == TQ_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[off]);
  return __half2float(static_cast<const __half*>(base)[off]);
}
__device__ __forceinline__ void store_elem(void* base, int dtype, int64_t off, float v) {
  if (dtype == TQ_F32) static_cast<float*>(base)[off] = v;
  else if (dtype == TQ_BF16) static_cast<__nv_bfloat16*>(base)[off] = __float2bfloat16_rn(v);
  else static_cast<__half*>(base)[off] = __float2half_rn(v);
}

// q_cat rows of one (batch, KV head): [q_rot | coeff q_rot S_eff^T] with q_rot = q Pi_k^T (the residual sketch
// lives in rotated coordinates), fp32 arithmetic on the fp32 matrices, rounded to bf16 once.  A decode-sized
// call has a few hundred query rows at most, which is no work for a tensor-core tile pipeline: one CTA per
// (batch, KV head); a warp takes four matrix rows (coalesced 512-byte loads, all in flight at once) and reduces
// each dot product across its lanes.
__global__ void __launch_bounds__(1024) decode_prepare_kernel(const void* __restrict__ q, int dtype, int64_t sb, int64_t sh,
                                                              int64_t ss, int64_t Hq, int64_t Hkv, int64_t Sq,
                                                              const float* __restrict__ Pi_k, const float* __restrict__ S_eff,
                                                              float coeff, __nv_bfloat16* __restrict__ q_cat) {
  constexpr int D = 128;
  __shared__ __align__(16) float buf[3][kRows][D];  // raw queries, rotated queries, sketch projections
  grid_launch_dependents();  // the split-KV kernel builds its tables and starts copying packed rows meanwhile
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int64_t b = blockIdx.x / Hkv, kvh = blockIdx.x % Hkv;
  const int G = (int)(Hq / Hkv), R = G * (int)Sq;
  for (int e = tid; e < R * D; e += 1024) {
    const int r = e / D, c = e % D;
    buf[0][r][c] = load_elem(q, dtype, b * sb + (kvh * G + r / Sq) * sh + (r % Sq) * ss + c);
  }
#pragma unroll
  for (int stage = 0; stage < 2; ++stage) {
    const float* W = stage == 0 ? Pi_k : S_eff;
    float4 w[4];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) w[jj] = __ldg(reinterpret_cast<const float4*>(W + (int64_t)(4 * warp + jj) * D) + lane);
    __syncthreads();  // the stage's input rows are complete
    for (int r = 0; r < R; ++r) {
      const float4 x = *reinterpret_cast<const float4*>(&buf[stage][r][4 * lane]);
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        float p = fmaf(w[jj].x, x.x, fmaf(w[jj].y, x.y, fmaf(w[jj].z, x.z, w[jj].w * x.w)));
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) p += __shfl_xor_sync(0xffffffffu, p, d);
        if (lane == jj) buf[stage + 1][r][4 * warp + jj] = p;
      }
    }
  }
  __syncthreads();
  for (int e = tid; e < R * 2 * D; e += 1024) {
    const int r = e / (2 * D), c = e % (2 * D);
    const int64_t row = (b * Hq + kvh * G + r / Sq) * Sq + r % Sq;
    const float v = c < D ? buf[1][r][c] : coeff * buf[2][r][c - D];
    q_cat[row * (2 * D) + c] = __float2bfloat16_rn(v);
  }
}

// One query row per CTA: merge the splits (O = sum_s O_s 2^(m_s - m) / sum_s l_s 2^(m_s - m)), rotate back
// (out = O Pi_v) and store in the caller's dtype and strides; fp32 throughout.  512 threads = 128 output
// columns x 4 parts of each sum, so that every thread has all its loads in flight at once.
__global__ void __launch_bounds__(512) decode_finish_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                            int nsplit, int64_t Hq, int64_t Hkv, int64_t Sq,
                                                            const float* __restrict__ Pi_v, void* __restrict__ out,
                                                            int out_dtype, int64_t osb, int64_t osh, int64_t oss) {
  constexpr int D = 128;
  __shared__ float f_s[kMaxExtraUnits + 1];
  __shared__ float part[4][D];
  __shared__ float o_s[D];
  const int tid = threadIdx.x, lane = tid % 32, j = tid % D, p = tid / D;
  const int r = blockIdx.x;
  const int64_t unit = blockIdx.y, b = unit / Hkv, kvh = unit % Hkv;
  const int G = (int)(Hq / Hkv);
  float pv[D / 4];  // this thread's part of column j of Pi_v: independent of the kernel before, loaded while it ends
#pragma unroll
  for (int c = 0; c < D / 4; ++c) pv[c] = __ldg(Pi_v + (32 * p + c) * D + j);
  grid_dependency_wait();
  const float* ml = part_ml + (unit * nsplit * kRows + r) * 2;  // split s: ml[s * kRows * 2], + 1
  // every warp finds the maximum and the total weight by itself; warp 0 also publishes the factors
  float m = -INFINITY;
  for (int s = lane; s < nsplit; s += 32) m = fmaxf(m, ml[(int64_t)s * kRows * 2]);
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
  float l = 0.f;
  for (int s = lane; s < nsplit; s += 32) {
    const float ms = ml[(int64_t)s * kRows * 2];
    const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
    if (tid < 32) f_s[s] = f;
    l = fmaf(ml[(int64_t)s * kRows * 2 + 1], f, l);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) l += __shfl_xor_sync(0xffffffffu, l, d);
  __syncthreads();
  float acc = 0.f;
#pragma unroll 4
  for (int s = p; s < nsplit; s += 4) acc = fmaf(part_o[((unit * nsplit + s) * kRows + r) * D + j], f_s[s], acc);
  part[p][j] = acc;
  __syncthreads();
  if (tid < D) o_s[tid] = l > 0.f ? (part[0][tid] + part[1][tid] + part[2][tid] + part[3][tid]) / l : 0.f;
  __syncthreads();
  float y = 0.f;
#pragma unroll
  for (int c = 0; c < D / 4; ++c) y = fmaf(o_s[32 * p + c], pv[c], y);
  part[p][j] = y;
  __syncthreads();
  if (tid < D) {
    const int64_t h = kvh * G + r / Sq, sq = r % Sq;
    store_elem(out, out_dtype, b * osb + h * osh + sq * oss + tid, part[0][tid] + part[1][tid] + part[2][tid] + part[3][tid]);
  }
}

}  // namespace

// TQ_B200_DECODE=0 routes decode-sized calls through the prefill kernels instead (diagnostics).
static bool decode_enabled() {
  static int cached = -1;
  if (cached < 0) {
    const char* e = getenv("TQ_B200_DECODE");
    cached = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return cached == 1;
}

bool decode_applies(const AttnArgs& a, int d) {
  const bool shape_ok = d == 128 && a.Hkv > 0 && (a.Hq / a.Hkv) * a.Sq <= kRows;
  if (a.kv_stride != a.Sk) return shape_ok;  // a persistent cache: the only kernel that reads strided rows
  return decode_enabled() && shape_ok && a.Sk >= 4 * kBlockKeys * kWarps;
}


size_t decode_workspace_bytes(int64_t BHq) {
  // at most (kMaxExtraUnits + B * Hkv) <= (kMaxExtraUnits + B * Hq) partial results of 16 rows x (128 + 2) floats
  return ((size_t)(kMaxExtraUnits + BHq) * kRows * (128 + 2) * sizeof(float) + 255) & ~(size_t)255;
}

// CTAs of decode_kernel<bits, nt> that one SM holds (registers and shared memory decide)
template <int BITS, int NT>
static int occupancy_of() {
  int n = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode_kernel<BITS, NT, false>, kWarps * 32, 0);
  return n > 0 ? n : 1;
}
static int resident_ctas(int bits, int nt) {
  static int cached[5][3] = {};
  if (cached[bits][nt] == 0) {
    if (nt == 1) cached[bits][nt] = bits == 2 ? occupancy_of<2, 1>() : bits == 3 ? occupancy_of<3, 1>() : occupancy_of<4, 1>();
    else cached[bits][nt] = bits == 2 ? occupancy_of<2, 2>() : bits == 3 ? occupancy_of<3, 2>() : occupancy_of<4, 2>();
  }
  return cached[bits][nt];
}

// Launch a kernel that may start before the previous kernel of the stream has finished (programmatic dependent
// launch); the kernel itself waits (grid_dependency_wait) before it touches that kernel's results.
template <typename... KArgs, typename... Args>
static cudaError_t launch_dependent(void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

int attention_decode(const AttnArgs& a, int64_t B, int bits, const void* q, int q_dtype, int64_t sb, int64_t sh,
                     int64_t ss, const float* Pi_k, const float* S_eff, void* q_cat, void* part_ws, cudaStream_t stream) {
  const int64_t units = B * a.Hkv;
  const int R = (int)((a.Hq / a.Hkv) * a.Sq);
  {
    ProfScope prof(kProfPrepareQueries, stream);
    decode_prepare_kernel<<<(unsigned)units, 1024, 0, stream>>>(q, q_dtype, sb, sh, ss, a.Hq, a.Hkv, a.Sq, Pi_k, S_eff,
                                                               sqrtf(1.5707963267948966f) / 128.f,
                                                               static_cast<__nv_bfloat16*>(q_cat));
    TQ_CUDA_OK(cudaGetLastError());
  }
  // One wave of CTAs, each with at least 64 keys (one 16-key block per warp).  The SMs run their resident
  // CTAs side by side and finish with the fullest one, so among the split counts that fit, take the one that
  // fills the SMs most evenly (the largest such count: more warps per SM hide more latency).
  const int64_t sms = sm_count();
  const int nt = R > 8 ? 2 : 1;  // tiles of eight query rows
  int64_t slots = sms * resident_ctas(bits, nt);
  if (slots > kMaxExtraUnits) slots = kMaxExtraUnits;
  int64_t n_max = slots / units;
  const int64_t max_split = (a.Sk + kBlockKeys * kWarps - 1) / (kBlockKeys * kWarps);
  if (n_max > max_split) n_max = max_split;
  int nsplit = 1;
  double best = 0.0;
  for (int64_t n = 1; n <= n_max; ++n) {
    const int64_t ctas = units * n, per_sm = (ctas + sms - 1) / sms;
    const double fill = (double)ctas / (double)(per_sm * sms);
    if (fill >= best - 1e-9) {
      best = fill;
      nsplit = (int)n;
    }
  }
  TQ_REQUIRE(units * nsplit <= kMaxExtraUnits + B * a.Hq, "partial-result workspace too small for %d splits", nsplit);
  int per = (int)((a.Sk + nsplit - 1) / nsplit);
  per = (per + kBlockKeys * kWarps - 1) / (kBlockKeys * kWarps) * (kBlockKeys * kWarps);
  nsplit = (int)((a.Sk + per - 1) / per);
  float* part_o = static_cast<float*>(part_ws);
  float* part_ml = part_o + (size_t)units * nsplit * kRows * 128;
  DecodeArgs da{static_cast<const __nv_bfloat16*>(q_cat), a.Hq, a.Hkv, a.Sq, a.Sk, a.kv_stride, a.key_idx, a.key_sgn, a.key_vn,
                a.key_rn, a.val_idx, a.val_vn, a.cen_k, a.cen_v, a.sm_scale, a.causal, a.mask, a.mask_stride_b,
                a.mask_stride_q, part_o, part_ml, nsplit, per};
  dim3 grid((unsigned)nsplit, (unsigned)a.Hkv, (unsigned)B);
  {
    ProfScope prof(kProfAttention, stream);
    void (*kern)(DecodeArgs);
    if (a.mask == nullptr)
      kern = nt == 1 ? (bits == 2 ? decode_kernel<2, 1, false> : bits == 3 ? decode_kernel<3, 1, false> : decode_kernel<4, 1, false>)
                     : (bits == 2 ? decode_kernel<2, 2, false> : bits == 3 ? decode_kernel<3, 2, false> : decode_kernel<4, 2, false>);
    else
      kern = nt == 1 ? (bits == 2 ? decode_kernel<2, 1, true> : bits == 3 ? decode_kernel<3, 1, true> : decode_kernel<4, 1, true>)
                     : (bits == 2 ? decode_kernel<2, 2, true> : bits == 3 ? decode_kernel<3, 2, true> : decode_kernel<4, 2, true>);
    TQ_CUDA_OK(launch_dependent(kern, grid, dim3(kWarps * 32), stream, da));
  }
  ProfScope prof(kProfBackRotation, stream);
  TQ_CUDA_OK(launch_dependent(decode_finish_kernel, dim3((unsigned)R, (unsigned)units), dim3(512), stream, part_o,
                              part_ml, nsplit, a.Hq, a.Hkv, a.Sq, a.Pi_v, a.out, a.out_dtype, a.o_stride_b,
                              a.o_stride_h, a.o_stride_s));
  return TQ_OK;
}

}  // namespace tq
