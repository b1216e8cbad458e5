// Fused key + value compression, one launch (TQ_MODE_BF16, bf16 inputs, head_dim 128).
//
// Replaces TurboQuantCompressorV2.compress and TurboQuantCompressorMSE.compress of the reference
// (src/turboquant_pytorch/compressors.py:98-161, :270-294) with the packed result layout of compressors.py:132-138,
// :281-285.  The arithmetic is that of tq_compress_tc.cu (rotation and sketch projection on tcgen05 from split-bf16
// operands, index by boundary counting, residual in rotated coordinates); what differs is how a CTA is organised:
//
//   * work units are 128-vector tiles of one (batch, head): all key tiles, then all value tiles, dealt round-robin
//     to a persistent grid of one CTA per SM, so every CTA handles its key tiles first and then its value tiles
//     (one switch of the constant operands in between);
//   * a control warp stages tiles with TMA (cp.async.bulk.tensor, 128-byte swizzle, three slots; a tensor map
//     over the caller's [B, H, S, d] view, so any 16-byte-aligned strides work and rows past S arrive as zeros)
//     and issues the MMAs; the raw bf16 tile is the A operand as it lands;
//   * 16 epilogue warps (row = tensor-memory lane, 32 coordinates per thread) turn accumulators into packed bytes;
//   * three accumulator slots in tensor memory: the rotation of tile i+1 runs under the epilogue of tile i.  The
//     key residual (fp32, split into bf16 hi + lo) goes back to TENSOR MEMORY and is the A operand of the sketch
//     MMA there, so it costs no shared memory and no proxy fence; its projection overwrites the rotated
//     coordinates it came from.  The sign pass of tile i runs after the index pass of tile i+1, under which the
//     sketch MMA of tile i has finished;
//   * the constant operands (Pi hi/lo, S_eff hi/lo for keys; Pi_v hi/lo for values) are bulk-copied from images
//     built once per compressor pair (tq_prepare_constants).
//
// Every wait is bounded; on expiry the CTA raises its abort flag, all roles leave their loops at their next wait,
// outstanding copies are waited for (bounded), tensor memory is freed and the fault is counted and reported.
#include <cuda.h>

#include <type_traits>

#include "tq_attention.cuh"
#include "tq_compress.cuh"
#include "tq_simt.cuh"
#include "tq_tcgen05.cuh"

namespace tq {

__device__ unsigned long long g_compress_kv_faults = 0ull;
__device__ unsigned long long* g_fault_mailbox_compress_kv = nullptr;
int set_fault_mailbox_compress_kv(unsigned long long* slot) {
  TQ_CUDA_OK(cudaMemcpyToSymbol(g_fault_mailbox_compress_kv, &slot, sizeof(slot)));
  return TQ_OK;
}
int read_compress_kv_faults(unsigned long long* out) {
  TQ_CUDA_OK(cudaMemcpyFromSymbol(out, g_compress_kv_faults, sizeof(*out)));
  return TQ_OK;
}

namespace {

constexpr int kD = 128;
constexpr int kEpiWarps = 16;
constexpr int kKvThreads = (kEpiWarps + 1) * 32;
constexpr int kSlots = 3;
constexpr uint32_t kTileBytes = 128 * kD * 2;      // one bf16 tile, two 64-column halves of 16 KB
constexpr uint32_t kMatBytes = kD * kD * 2;        // one bf16 operand image
constexpr uint32_t kOffX = 0;
constexpr uint32_t kOffConst = kSlots * kTileBytes;
constexpr uint32_t kOffExch = kOffConst + 4 * kMatBytes;
constexpr uint32_t kOffMisc = kOffExch + 4 * 128 * 4;   // barriers, tensor-memory slot, abort flag, centroids
constexpr uint32_t kSmemBytes = kOffMisc + 256;
static_assert(kSmemBytes <= 227 * 1024, "shared memory over-subscribed");
// tensor memory: three accumulator slots (rotated coordinates, later the sketch projection), residual hi, lo
constexpr uint32_t kColYP = 0, kColRH = 3 * kD, kColRL = 3 * kD + kD / 2;

struct KvArgs {
  uint32_t units_k, units_v;  // 128-vector tiles on either side (32-bit: unit arithmetic runs per thread and tile)
  uint32_t tiles_per_head;    // ceil(S / 128)
  uint32_t S, H;
  const uint8_t* consts;      // constants buffer of tq_prepare_constants
  uint8_t* key_idx;
  uint8_t* key_sgn;
  uint16_t* key_vn;
  uint16_t* key_rn;
  uint8_t* val_idx;
  uint16_t* val_vn;
  int64_t out_stride, out_offset;  // vector (bh, s) -> output row bh * out_stride + out_offset + s
  ConstLayout L;
};

__device__ __forceinline__ uint32_t bf16_bits(float v) {
  return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(v)));
}
__device__ __forceinline__ float bf16_value(uint32_t b) { return __uint_as_float(b << 16); }

// Number of ascending boundaries strictly below y (the Lloyd-Max index), without compares or selects: the sign
// bit of (b - y) is set exactly when y > b (b - y == 0 gives +0), and mad.hi by 2 adds that bit to the count.  Both
// instructions run on the FMA pipe, which issues at twice the rate of the integer/compare pipe this epilogue would
// otherwise saturate.
// Codebooks of 8 and more levels use the symmetry of the boundaries (b[NB-1-j] = -b[j], b[(NB-1)/2] = 0): the sign
// of y and the count m of positive boundaries below |y| give idx = h + m for y > 0 and h - 1 - m otherwise
// (h = (NB+1)/2), with half the subtractions.  The one difference: a NEGATIVE y that equals a boundary exactly
// lands one level higher than the strict count would put it (part of the documented tie budget).
template <int NB>
__device__ __forceinline__ uint32_t index_of(float y, const float (&bd)[NB]) {
  if constexpr (NB < 7) {
    uint32_t idx = 0;
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      const uint32_t d = __float_as_uint(bd[j] - y);
      asm("mad.hi.u32 %0, %1, 2, %2;" : "=r"(idx) : "r"(d), "r"(idx));
    }
    return idx;
  } else {
    constexpr int h = (NB + 1) / 2;
    uint32_t m = 0, pos = 0;
    const uint32_t dz = __float_as_uint(0.f - y);  // sign set iff y > 0
    asm("mad.hi.u32 %0, %1, 2, %2;" : "=r"(pos) : "r"(dz), "r"(pos));
    const float ay = fabsf(y);
#pragma unroll
    for (int j = 0; j < h - 1; ++j) {
      const uint32_t d = __float_as_uint(bd[h + j] - ay);
      asm("mad.hi.u32 %0, %1, 2, %2;" : "=r"(m) : "r"(d), "r"(m));
    }
    return (uint32_t)(h - 1) - m + pos * (2u * m + 1u);
  }
}
// OR the B-bit field of coordinate E (of this thread's 32) into the thread's B packed words (LSB-first bit stream)
template <int B, int E>
__device__ __forceinline__ void put_field(uint32_t (&w)[B], uint32_t idx) {
  constexpr int pos = E * B, k = pos / 32, sh = pos % 32;
  w[k] = idx * (1u << sh) + w[k];  // the field's bits are still zero there: + is |
  if constexpr (sh + B > 32) w[k + 1] = (idx >> (32 - sh)) + w[k + 1];
}
template <int FROM, int TO, class F>
__device__ __forceinline__ void static_for(F&& f) {
  if constexpr (FROM < TO) {
    f(std::integral_constant<int, FROM>{});
    static_for<FROM + 1, TO>(f);
  }
}

// One box of a rank-4 tiled tensor map (64 columns x 128 rows of one (batch, head)) -> shared memory, completion
// counted in bytes on `bar` of this CTA.  No multicast.
__device__ __forceinline__ void tma_load_tile(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                              uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Shared-memory descriptor of a K-major operand in the 128-byte-swizzled layout TMA writes (rows of 128 bytes,
// 8-row groups 1024 bytes apart); `saddr` is the tile base (1024-byte aligned) plus 32 bytes per K step of 16.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  return static_cast<uint64_t>((saddr >> 4) & 0x3FFFu) | (1ull << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}

template <int BITS>
__global__ void __launch_bounds__(kKvThreads, 1)
compress_kv_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const KvArgs a) {
  constexpr int KB = BITS - 1, VB = BITS;
  constexpr uint32_t SBO = (kD / 8) * 128;  // canonical (unswizzled) K-major images of the constant operands
  extern __shared__ __align__(1024) uint8_t smem[];
  float (*exch)[128] = reinterpret_cast<float (*)[128]>(smem + kOffExch);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffMisc);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffMisc + 208);
  int* s_abort_p = reinterpret_cast<int*>(smem + kOffMisc + 212);
  float* cen_s = reinterpret_cast<float*>(smem + kOffMisc + 216);  // 2^KB <= 8 key centroids
  volatile int* abort_flag = s_abort_p;
  const uint32_t bar0 = tc::smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };
  // 0: constants landed; 1-3: tile landed; 4-6: rotation done; 7-9: sketch done; 10-12: accumulator slot read out;
  // 13: residual operand written; 14-17: row-part exchange per lane quarter; 18-21: exchange buffer read out;
  // 22-24: tile read out of shared memory by the epilogue (its slot may be refilled once the rotation is done too)
  const uint32_t const_full = bar(0), r_full = bar(13);
  auto x_full = [&](int s) { return bar(1 + s); };
  auto y_done = [&](int s) { return bar(4 + s); };
  auto p_done = [&](int s) { return bar(7 + s); };
  auto yp_free = [&](int s) { return bar(10 + s); };
  auto xch = [&](int q) { return bar(14 + q); };
  auto xfree = [&](int q) { return bar(18 + q); };
  auto x_read = [&](int s) { return bar(22 + s); };

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const uint32_t total = a.units_k + a.units_v;
  const uint32_t G = gridDim.x, c = blockIdx.x;
  const int n = (int)((total - c + G - 1) / G);                                  // units of this CTA
  const int nk = c < a.units_k ? (int)((a.units_k - c + G - 1) / G) : 0;         // ... of which key tiles (first)

  if (tid == 0) {
    *s_abort_p = 0;
    tc::mbar_init(const_full, 1);
    for (int s = 0; s < kSlots; ++s) {
      tc::mbar_init(x_full(s), 1);
      tc::mbar_init(y_done(s), 1);
      tc::mbar_init(p_done(s), 1);
      tc::mbar_init(yp_free(s), kEpiWarps);
      tc::mbar_init(x_read(s), kEpiWarps);
    }
    tc::mbar_init(r_full, kEpiWarps);
    for (int q = 0; q < 4; ++q) {
      tc::mbar_init(xch(q), 4);
      tc::mbar_init(xfree(q), 4);
    }
    tc::fence_mbar_init();
  }
  if (tid < (1 << KB)) cen_s[tid] = __ldg(reinterpret_cast<const float*>(a.consts + a.L.cen_k) + tid);
  if (warp == kEpiWarps) tc::tmem_alloc(tc::smem_u32(tmem_slot), 512);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  bool ok = true;

  // global unit of this CTA's i-th unit -> side, (batch * head), first row
  auto unit_of = [&](int i, bool& is_key, int64_t& bh, int& s0) {
    const uint32_t g = c + (uint32_t)i * G;
    is_key = g < a.units_k;
    const uint32_t t = is_key ? g : g - a.units_k;
    const uint32_t h = t / a.tiles_per_head;
    bh = h;
    s0 = (int)(t - h * a.tiles_per_head) * 128;
  };

  if (warp == kEpiWarps) {
    // ======================================= control warp =======================================
    if (lane == 0 && n > 0) {
      int issued = 0;  // tiles whose copies have been issued
      auto issue_tile = [&](int i) {
        bool is_key;
        int64_t bh;
        int s0;
        unit_of(i, is_key, bh, s0);
        const int s = i % kSlots;
        const CUtensorMap* map = is_key ? &map_k : &map_v;
        const uint32_t dst = tc::smem_u32(smem + kOffX + s * kTileBytes);
        tc::mbar_arrive_expect_tx(x_full(s), kTileBytes);
        const uint32_t bi = (uint32_t)bh / a.H, hi = (uint32_t)bh - bi * a.H;
        tma_load_tile(dst, map, 0, s0, (int)hi, (int)bi, x_full(s));
        tma_load_tile(dst + kTileBytes / 2, map, 64, s0, (int)hi, (int)bi, x_full(s));
        issued = i + 1;
      };
      auto load_consts = [&](bool keys) {
        const uint32_t dst = tc::smem_u32(smem + kOffConst);
        if (keys) {
          tc::mbar_arrive_expect_tx(const_full, 4 * kMatBytes);
          tc::bulk_load(dst, a.consts + a.L.pik_hi, kMatBytes, const_full);
          tc::bulk_load(dst + kMatBytes, a.consts + a.L.pik_lo, kMatBytes, const_full);
          tc::bulk_load(dst + 2 * kMatBytes, a.consts + a.L.se_hi, kMatBytes, const_full);
          tc::bulk_load(dst + 3 * kMatBytes, a.consts + a.L.se_lo, kMatBytes, const_full);
        } else {
          tc::mbar_arrive_expect_tx(const_full, 2 * kMatBytes);
          tc::bulk_load(dst, a.consts + a.L.piv_hi, kMatBytes, const_full);
          tc::bulk_load(dst + kMatBytes, a.consts + a.L.piv_lo, kMatBytes, const_full);
        }
      };
      constexpr uint32_t idesc = tc::idesc_bf16(128, kD, false, false);
      const uint32_t cbase = tc::smem_u32(smem + kOffConst);
      const uint64_t b_hi = tc::smem_desc(cbase, 128, SBO), b_lo = tc::smem_desc(cbase + kMatBytes, 128, SBO);
      const uint64_t se_hi = tc::smem_desc(cbase + 2 * kMatBytes, 128, SBO);
      const uint64_t se_lo = tc::smem_desc(cbase + 3 * kMatBytes, 128, SBO);
      // sketch of key tile i: P = r_hi Se_hi^T + r_hi Se_lo^T + r_lo Se_hi^T, A from tensor memory, into the slot
      // whose rotated coordinates the residual was computed from
      auto issue_sketch = [&](int i) {
        if (!(ok = tc::mbar_wait_or_abort(r_full, i & 1, abort_flag))) return;
        tc::fence_after_sync();
        const uint32_t d_p = tmem + kColYP + (i % kSlots) * kD;
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks)
          tc::mma_bf16_ts(d_p, tmem + kColRH + ks * 8, se_hi + (uint64_t)(ks * 256 >> 4), idesc, ks > 0);
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks)
          tc::mma_bf16_ts(d_p, tmem + kColRH + ks * 8, se_lo + (uint64_t)(ks * 256 >> 4), idesc, 1u);
#pragma unroll
        for (int ks = 0; ks < kD / 16; ++ks)
          tc::mma_bf16_ts(d_p, tmem + kColRL + ks * 8, se_hi + (uint64_t)(ks * 256 >> 4), idesc, 1u);
        tc::mma_commit(p_done(i % kSlots));
      };
      bool keys_loaded = nk > 0;
      int const_phase = 0;
      load_consts(keys_loaded);
      for (int t = 0; t < kSlots && t < n; ++t) issue_tile(t);
      ok = tc::mbar_wait_or_abort(const_full, const_phase, abort_flag);
      bool sketch_pending = false;  // the sketch of tile i-1 has not been issued yet
      for (int i = 0; i < n && ok; ++i) {
        const int s = i % kSlots, u = i / kSlots;
        const bool is_key = i < nk;
        if (!is_key && keys_loaded) {
          // last key tile behind us: finish its sketch, wait until no MMA reads the key operands, swap them
          if (sketch_pending) {
            issue_sketch(i - 1);
            sketch_pending = false;
            if (!ok) break;
          }
          if (nk > 0 && !(ok = tc::mbar_wait_or_abort(p_done((nk - 1) % kSlots), ((nk - 1) / kSlots) & 1, abort_flag))) break;
          keys_loaded = false;
          const_phase ^= 1;
          load_consts(false);
          if (!(ok = tc::mbar_wait_or_abort(const_full, const_phase, abort_flag))) break;
        }
        if (!(ok = tc::mbar_wait_or_abort(x_full(s), u & 1, abort_flag))) break;
        if (i >= kSlots && !(ok = tc::mbar_wait_or_abort(yp_free(s), (u - 1) & 1, abort_flag))) break;
        tc::fence_after_sync();
        {
          // rotation: Y_raw = X Pi_hi^T + X Pi_lo^T; K step ks reads 32 bytes of each 128-byte row of half ks / 4
          const uint32_t xb = tc::smem_u32(smem + kOffX + s * kTileBytes);
          const uint32_t d_y = tmem + kColYP + s * kD;
#pragma unroll
          for (int ks = 0; ks < kD / 16; ++ks)
            tc::mma_bf16(d_y, smem_desc_sw128(xb + (ks / 4) * (kTileBytes / 2) + (ks % 4) * 32),
                         b_hi + (uint64_t)(ks * 256 >> 4), idesc, ks > 0);
#pragma unroll
          for (int ks = 0; ks < kD / 16; ++ks)
            tc::mma_bf16(d_y, smem_desc_sw128(xb + (ks / 4) * (kTileBytes / 2) + (ks % 4) * 32),
                         b_lo + (uint64_t)(ks * 256 >> 4), idesc, 1u);
          tc::mma_commit(y_done(s));
        }
        if (sketch_pending) {
          issue_sketch(i - 1);
          sketch_pending = false;
          if (!ok) break;
        }
        sketch_pending = is_key;
        // the slot tile i-1 came from is free once its rotation has completed AND the epilogue has read its rows
        // for the norms (the control warp runs ahead of the epilogue; a refill before that read would also let
        // the slot's barrier run two phases ahead of a waiter): refill it with tile i+2
        if (i >= 1 && i + 2 < n) {
          if (!(ok = tc::mbar_wait_or_abort(y_done((i - 1) % kSlots), ((i - 1) / kSlots) & 1, abort_flag))) break;
          if (!(ok = tc::mbar_wait_or_abort(x_read((i - 1) % kSlots), ((i - 1) / kSlots) & 1, abort_flag))) break;
          issue_tile(i + 2);
        }
      }
      if (ok && sketch_pending) issue_sketch(n - 1);
      if (!ok) {
        // give the copies in flight a bounded time to land before the CTA's shared memory goes away
        for (int i = 0; i < issued; ++i) tc::mbar_wait_bounded(x_full(i % kSlots), (i / kSlots) & 1, 20000000ll);
      }
    }
  } else {
    // ======================================= epilogue warps =======================================
    const int q = warp % 4, part = warp / 4;  // lane quarter of tensor memory; coordinates [32 part, 32 part + 32)
    const int row = q * 32 + lane;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    float bnd_k[(1 << KB) - 1], bnd_v[(1 << VB) - 1];
#pragma unroll
    for (int j = 0; j < (1 << KB) - 1; ++j) bnd_k[j] = __ldg(reinterpret_cast<const float*>(a.consts + a.L.bnd_k) + j);
#pragma unroll
    for (int j = 0; j < (1 << VB) - 1; ++j) bnd_v[j] = __ldg(reinterpret_cast<const float*>(a.consts + a.L.bnd_v) + j);
    int n_xch = 0;    // exchanges through `exch` so far in this quarter (phase of xch / xfree)
    // sum of the four parts' values of this row, in a fixed order; every part gets the same total
    auto exchange = [&](float mine, float& total_out) -> bool {
      // the buffer must have been read out by everyone since the previous exchange
      if (n_xch >= 1 && !tc::mbar_wait_or_abort(xfree(q), (n_xch - 1) & 1, abort_flag)) return false;
      exch[part][row] = mine;
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(xch(q));
      if (!tc::mbar_wait_or_abort(xch(q), n_xch & 1, abort_flag)) return false;
      total_out = ((exch[0][row] + exch[1][row]) + exch[2][row]) + exch[3][row];
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(xfree(q));
      ++n_xch;
      return true;
    };
    for (int i = 0; i <= n && ok; ++i) {
      if (i < n) {
        const int s = i % kSlots, u = i / kSlots;
        bool is_key;
        int64_t bh;
        int s0;
        unit_of(i, is_key, bh, s0);
        const bool live = (uint32_t)(s0 + row) < a.S;
        const int64_t no = bh * a.out_stride + a.out_offset + s0 + row;
        // ---- norm of the row: this thread's 64 bytes of the tile as it landed (128-byte swizzle) ----
        if (!(ok = tc::mbar_wait_or_abort(x_full(s), u & 1, abort_flag))) break;
        float ss = 0.f;
        {
          const uint8_t* xrow = smem + kOffX + s * kTileBytes + (part / 2) * (kTileBytes / 2) + row * 128;
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            const int chunk = 4 * (part % 2) + cc;  // 16-byte chunk of the row's half
            const uint4 v = *reinterpret_cast<const uint4*>(xrow + ((chunk ^ (row & 7)) << 4));
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float lo = __uint_as_float(w[e] << 16), hi = __uint_as_float(w[e] & 0xffff0000u);
              ss = fmaf(lo, lo, ss);
              ss = fmaf(hi, hi, ss);
            }
          }
        }
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(x_read(s));
        float ss_tot;
        if (!(ok = exchange(ss, ss_tot))) break;
        const float nv = sqrtf(ss_tot), den = nv + 1e-8f;
        if (!(ok = tc::mbar_wait_or_abort(y_done(s), u & 1, abort_flag))) break;
        tc::fence_after_sync();
        uint32_t raw[32];
        tc::tmem_ld32(tmem + kColYP + s * kD + lane_base + 32 * part, raw);
        tc::wait_ld();
        if (is_key) {
          // y = y_raw / den is compared with the boundaries as y_raw > b * den (den > 0)
          float bden[(1 << KB) - 1];
#pragma unroll
          for (int j = 0; j < (1 << KB) - 1; ++j) bden[j] = bnd_k[j] * den;
          float rr = 0.f;
          uint32_t packed[KB], rh[16], rl[16];
#pragma unroll
          for (int j = 0; j < KB; ++j) packed[j] = 0;
          const float neg_nv = -nv;
          static_for<0, 16>([&](auto pc) {
            constexpr int pr = decltype(pc)::value;  // coordinates 2 pr, 2 pr + 1 of this thread's 32
            float res[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const float yr = __uint_as_float(raw[2 * pr + h]);
              const uint32_t idx = index_of<(1 << KB) - 1>(yr, bden);
              if (h == 0) put_field<KB, 2 * pr>(packed, idx);
              else put_field<KB, 2 * pr + 1>(packed, idx);
              res[h] = fmaf(neg_nv, cen_s[idx], yr);   // residual in rotated coordinates
              rr = fmaf(res[h], res[h], rr);
            }
            // split into bf16 hi (truncated: the upper halves of the two words, one byte permute) and lo = the
            // exact remainder, rounded; hi + lo carries ~16 mantissa bits
            const uint32_t b0 = __float_as_uint(res[0]), b1 = __float_as_uint(res[1]);
            rh[pr] = __byte_perm(b0, b1, 0x7632);
            rl[pr] = tc::pack_bf16x2(res[0] - __uint_as_float(b0 & 0xffff0000u), res[1] - __uint_as_float(b1 & 0xffff0000u));
          });
          if (live) {
            uint32_t* dst = reinterpret_cast<uint32_t*>(a.key_idx + no * (kD * KB / 8) + 4 * KB * part);
            if constexpr (KB == 2) *reinterpret_cast<uint2*>(dst) = make_uint2(packed[0], packed[1]);
            else {
#pragma unroll
              for (int j = 0; j < KB; ++j) dst[j] = packed[j];
            }
            if (part == 0) a.key_vn[no] = fp16_bits(nv);
          }
          float rr_tot;
          if (!(ok = exchange(rr, rr_tot))) break;
          if (live && part == 0) a.key_rn[no] = fp16_bits(sqrtf(rr_tot));
          // the residual operand of the previous key tile must have been consumed by its sketch MMAs
          if (i >= 1 && !(ok = tc::mbar_wait_or_abort(p_done((i - 1) % kSlots), ((i - 1) / kSlots) & 1, abort_flag))) break;
          tc::tmem_st16(tmem + kColRH + lane_base + 16 * part, rh);
          tc::tmem_st16(tmem + kColRL + lane_base + 16 * part, rl);
          tc::wait_st();
          tc::fence_before_sync();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(r_full);
        } else {
          tc::fence_before_sync();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(yp_free(s));  // the accumulator slot is in registers now
          float bden[(1 << VB) - 1];
#pragma unroll
          for (int j = 0; j < (1 << VB) - 1; ++j) bden[j] = bnd_v[j] * den;
          uint32_t packed[VB];
#pragma unroll
          for (int j = 0; j < VB; ++j) packed[j] = 0;
          static_for<0, 32>([&](auto ec) {
            constexpr int e = decltype(ec)::value;
            put_field<VB, e>(packed, index_of<(1 << VB) - 1>(__uint_as_float(raw[e]), bden));
          });
          if (live) {
            uint32_t* dst = reinterpret_cast<uint32_t*>(a.val_idx + no * (kD * VB / 8) + 4 * VB * part);
            if constexpr (VB == 4) *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            else if constexpr (VB == 2) *reinterpret_cast<uint2*>(dst) = make_uint2(packed[0], packed[1]);
            else {
#pragma unroll
              for (int j = 0; j < VB; ++j) dst[j] = packed[j];
            }
            if (part == 0) a.val_vn[no] = fp16_bits(nv);
          }
        }
      }
      // ---- sign pass of the key tile before: its sketch MMA ran under the index pass above ----
      if (i >= 1 && i - 1 < nk) {
        const int s1 = (i - 1) % kSlots;
        bool is_key;
        int64_t bh;
        int s0;
        unit_of(i - 1, is_key, bh, s0);
        if (!(ok = tc::mbar_wait_or_abort(p_done(s1), ((i - 1) / kSlots) & 1, abort_flag))) break;
        tc::fence_after_sync();
        uint32_t raw[32];
        tc::tmem_ld32(tmem + kColYP + s1 * kD + lane_base + 32 * part, raw);
        tc::wait_ld();
        tc::fence_before_sync();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(yp_free(s1));
        // bit e = (projection >= 0) = complement of its sign bit (a projection is never -0: sums of products that
        // start from +0); the sign bits are gathered with one mask and one mad.hi each
        uint32_t neg = 0;
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const uint32_t sb = raw[e] & 0x80000000u;
          neg = (e == 31 ? sb : __umulhi(sb, 2u << e)) + neg;
        }
        if ((uint32_t)(s0 + row) < a.S)
          *reinterpret_cast<uint32_t*>(a.key_sgn + (bh * a.out_stride + a.out_offset + s0 + row) * (kD / 8) + 4 * part) = ~neg;
      }
    }
  }
  if (!ok && atomicExch(s_abort_p, 2) != 2) {  // one fault per CTA
    atomicAdd(&g_compress_kv_faults, 1ull);
    notify_host_of_fault(g_fault_mailbox_compress_kv);
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == kEpiWarps) tc::tmem_dealloc(tmem, 512);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime (the library does not link against libcuda).
EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      cudaGetLastError();
  }
  return fn;
}

// Tensor map over a bf16 [B, H, S, 128] view with element strides (sb, sh, ss): box = 64 columns x 128 rows of one
// (batch, head), 128-byte swizzle, zero fill past the end of S.
int make_map(CUtensorMap* map, const void* base, int64_t B, int64_t H, int64_t S, int64_t sb, int64_t sh, int64_t ss) {
  EncodeTiledFn enc = encode_tiled();
  if (enc == nullptr) return fail(TQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[4] = {(cuuint64_t)kD, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  // a dimension of extent 1 may carry any stride; the encoder still wants a multiple of 16 bytes
  const cuuint64_t strides[3] = {(cuuint64_t)(S > 1 ? ss : kD) * 2, (cuuint64_t)(H > 1 ? sh : kD) * 2,
                                 (cuuint64_t)(B > 1 ? sb : kD) * 2};
  const cuuint32_t box[4] = {64, 128, 1, 1}, estr[4] = {1, 1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TQ_ERR_UNSUPPORTED, "tensor map for strides (%lld, %lld, %lld) refused (CUresult %d)",
                                     (long long)sb, (long long)sh, (long long)ss, (int)r);
  return TQ_OK;
}

}  // namespace

bool compress_kv_applies(int dtype, int d, int mode) { return dtype == TQ_BF16 && d == kD && mode == TQ_MODE_BF16; }

int compress_kv(const void* k, const void* v, int64_t B, int64_t H, int64_t S, const int64_t* k_strides,
                const int64_t* v_strides, const uint8_t* consts, int bits, uint8_t* key_idx, uint8_t* key_sgn,
                uint16_t* key_vn, uint16_t* key_rn, uint8_t* val_idx, uint16_t* val_vn, int64_t out_stride,
                int64_t out_offset, cudaStream_t stream) {
  const int64_t tiles_per_head = (S + 127) / 128, units = B * H * tiles_per_head;
  TQ_REQUIRE(units < ((int64_t)1 << 31) && S < ((int64_t)1 << 31) && H < ((int64_t)1 << 31) && B < ((int64_t)1 << 31),
             "problem too large");
  CUtensorMap map_k, map_v;
  const void* any = k != nullptr ? k : v;
  const int64_t* any_strides = k != nullptr ? k_strides : v_strides;
  if (int st = make_map(&map_k, k != nullptr ? k : any, B, H, S, (k ? k_strides : any_strides)[0],
                        (k ? k_strides : any_strides)[1], (k ? k_strides : any_strides)[2]))
    return st;
  if (int st = make_map(&map_v, v != nullptr ? v : any, B, H, S, (v ? v_strides : any_strides)[0],
                        (v ? v_strides : any_strides)[1], (v ? v_strides : any_strides)[2]))
    return st;
  TQ_REQUIRE(2 * units < ((int64_t)1 << 31), "problem too large");
  KvArgs a{(uint32_t)(k != nullptr ? units : 0), (uint32_t)(v != nullptr ? units : 0), (uint32_t)tiles_per_head,
           (uint32_t)S, (uint32_t)H, consts, key_idx, key_sgn, key_vn, key_rn, val_idx, val_vn, out_stride, out_offset,
           const_layout(kD)};
  const int64_t total = (int64_t)a.units_k + a.units_v;
  int grid = sm_count();
  if (grid > total) grid = (int)total;
  auto kern = bits == 2 ? compress_kv_kernel<2> : bits == 3 ? compress_kv_kernel<3> : compress_kv_kernel<4>;
  TQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
  {
    ProfScope prof(k != nullptr ? kProfCompressKeys : kProfCompressValues, stream);
    kern<<<grid, kKvThreads, kSmemBytes, stream>>>(map_k, map_v, a);
  }
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
}

}  // namespace tq
