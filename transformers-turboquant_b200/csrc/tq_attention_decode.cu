// Split-KV compressed attention for decode-sized calls: few query rows per KV head (G * Sq <= 16), long
// keys.  There is no counterpart in the reference, which disables the KV cache and recomputes full
// attention per generated token (patch.py:80-81); this serves a cache kept in the library's wire format.
//
// The work is bound by the packed bytes (about 100 B per key at 3 bits), not by the contractions, so the
// keys of one (batch, KV head) are split over `nsplit` CTAs and every CTA streams its range once:
//   * a warp takes 16 keys at a time and decodes K_hat = [C[idx] ; (rn / n) sign] (the key norm n multiplies
//     the finished score in fp32) STRAIGHT INTO the B
//     fragments of mma.sync.m16n8k16 (bf16, fp32 accumulation) -- no shared-memory operand tile, each
//     element is decoded exactly once by the lane that feeds it to the tensor core; the 16 query rows of
//     the KV head (all its query heads x positions, zero-padded) are the A operand;
//   * online softmax on the C fragments (row maxima by two quad shuffles, running maximum raised lazily);
//   * P (bf16, with the value norms folded in) is re-used as the A fragment of O += P V_hat, whose B
//     fragments are decoded from the packed value indices the same way;
//   * the four warps of a CTA merge through shared memory, the splits through a small fp32 workspace
//     (`combine_kernel`), in the rotated output space; the caller rotates back.
// The legacy tensor-core path is deliberate here: M = 16 rows do not fill a tcgen05 tile, and what has to
// be fast is the decode around the MMA, not the MMA.
#include <math.h>
#include <stdlib.h>

#include <type_traits>

#include "tq_attention.cuh"
#include "tq_common.cuh"
#include "tq_simt.cuh"

namespace tq {
namespace {

constexpr int kRows = 16;        // query rows per KV head (M of the MMA)
constexpr int kWarps = 4;
constexpr int kBlockKeys = 16;   // keys per warp iteration
constexpr int kQPitch = 2 * 128 + 8;  // bf16 elements per staged query row (padded against bank conflicts)

struct DecodeArgs {
  const __nv_bfloat16* q_cat;  // [B*Hq*Sq, 2d]
  int64_t Hq, Hkv, Sq, Sk;
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
// D (16x8, fp32) += A (16x16, bf16, row) * B (16x8, bf16, col)
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// NBITS bits of a little-endian word array at bit offset 8 * BYTE + r, with BYTE known at compile time and
// the run-time part r <= MAXR.  Stays inside one word when it can (one shift, one mask); otherwise takes the
// four bytes starting at BYTE out of two neighbouring words with one byte permute first.
template <int NW, int BYTE, int MAXR, int NBITS>
__device__ __forceinline__ uint32_t field(const uint32_t (&w)[NW], int r) {
  constexpr int word = BYTE / 4, bo = BYTE % 4;
  constexpr uint32_t mask = (1u << NBITS) - 1;
  static_assert(MAXR + NBITS <= 32, "field wider than a window");
  if constexpr (8 * bo + MAXR + NBITS <= 32) {
    return (w[word] >> (8 * bo + r)) & mask;
  } else {
    constexpr uint32_t sel = bo == 1 ? 0x4321u : bo == 2 ? 0x5432u : 0x6543u;
    const uint32_t win = __byte_perm(w[word], w[word + 1 < NW ? word + 1 : word], sel);
    return (win >> r) & mask;
  }
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
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

template <int BITS>
__global__ void __launch_bounds__(kWarps * 32) decode_kernel(const DecodeArgs a) {
  constexpr int D = 128, KB = BITS - 1, VB = BITS;
  constexpr int KW = 4 * KB, VW = 4 * VB;  // 32-bit words of one packed key / value index row
  constexpr float kLog2e = 1.4426950408889634f;
  // packed bytes of the block a warp works on and of its next one (copied ahead with cp.async):
  // 16 key-index rows, 16 sign rows, 16 value-index rows
  constexpr int kStageBytes = kBlockKeys * 16 * (KB + 1 + VB);
  constexpr int kQBytes = kRows * kQPitch * 2;
  constexpr int kMergeBytes = kWarps * kRows * (D + 4) * 4;
  constexpr int kLoopBytes = kQBytes + kWarps * 2 * kStageBytes;
  // one pool: staged queries + packed-row stages while the keys stream, the warps' partial outputs afterwards
  __shared__ __align__(16) uint8_t pool[kLoopBytes > kMergeBytes ? kLoopBytes : kMergeBytes];
  __shared__ uint32_t lutK[1 << (2 * KB)];  // two key indices -> bf16x2 (C[i0], C[i1])
  __shared__ uint32_t lutV[1 << VB];        // one value index -> bf16 in the low half
  __shared__ float mrg_ml[kWarps][kRows][2];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(pool);
  auto stage_ptr = [&](int w, int st) { return pool + kQBytes + (w * 2 + st) * kStageBytes; };
  float (*mrg_o)[kRows][D + 4] = reinterpret_cast<float (*)[kRows][D + 4]>(pool);

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int gq = lane / 4, tq = lane % 4;
  const int split = blockIdx.x;
  const int64_t kvh = blockIdx.y, b = blockIdx.z;
  const int G = (int)(a.Hq / a.Hkv), R = G * (int)a.Sq;
  const int64_t kv_base = (b * a.Hkv + kvh) * a.Sk;
  const int shift = (int)(a.Sk - a.Sq);

  // ---- stage the query rows (row r = g * Sq + s of query head kvh * G + g), centroid tables ----
  for (int e = tid; e < kRows * (2 * D / 8); e += kWarps * 32) {
    const int r = e / (2 * D / 8), c = e % (2 * D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < R) {
      const int64_t h = kvh * G + r / a.Sq, s = r % a.Sq;
      v = reinterpret_cast<const uint4*>(a.q_cat + ((b * a.Hq + h) * a.Sq + s) * (2 * D))[c];
    }
    *reinterpret_cast<uint4*>(&q_s[r * kQPitch + c * 8]) = v;
  }
  for (int e = tid; e < (1 << (2 * KB)); e += kWarps * 32)
    lutK[e] = bf16x2(a.cen_k[e & ((1 << KB) - 1)], a.cen_k[e >> KB]);
  for (int e = tid; e < (1 << VB); e += kWarps * 32) lutV[e] = bf16x2(a.cen_v[e], 0.f);
  __syncthreads();

  // per-lane row facts: this lane's C-fragment rows are gq and gq + 8
  int row_lim[2];  // last visible key of the row (causal), or Sk - 1
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = gq + 8 * h;
    row_lim[h] = (r < R) ? (a.causal ? (r % (int)a.Sq) + shift : (int)a.Sk - 1) : -1;
  }
  const float cexp = a.sm_scale * kLog2e;
  float o[D / 8][4];
#pragma unroll
  for (int ct = 0; ct < D / 8; ++ct)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[ct][i] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  const int k_lo = split * a.keys_per_split;
  const int k_hi = min((int)a.Sk, k_lo + a.keys_per_split);
  // copy the packed rows of keys [blk, blk + 16) into stage `st` (rows of consecutive keys are contiguous in
  // each array); rows past the end of the sequence become zeros
  auto stage = [&](int blk, int st) {
    uint8_t* dst = stage_ptr(warp, st);
    constexpr int UK = kBlockKeys * KB, US = kBlockKeys, UV = kBlockKeys * VB;  // 16-byte units
    for (int u = lane; u < UK + US + UV; u += 32) {
      const uint8_t* src;
      int key;
      if (u < UK) { key = blk + u / KB; src = a.key_idx + (kv_base + blk) * (16 * KB) + 16 * u; }
      else if (u < UK + US) { key = blk + (u - UK); src = a.key_sgn + (kv_base + blk) * 16 + 16 * (u - UK); }
      else { key = blk + (u - UK - US) / VB; src = a.val_idx + (kv_base + blk) * (16 * VB) + 16 * (u - UK - US); }
      if (key < a.Sk) cp_async16(dst + 16 * u, src);
      else *reinterpret_cast<uint4*>(dst + 16 * u) = make_uint4(0, 0, 0, 0);
    }
  };
  // fp16 norms this lane needs for a block: of the two keys it decodes (vector and residual norm) and of the
  // four keys of its score / probability columns (key and value vector norms)
  struct Norms { float nk[2], rn[2], kn[4], nv[4]; };
  auto load_norms = [&](int blk, Norms& n) {
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int key = blk + 8 * nt + gq;
      n.nk[nt] = key < a.Sk ? fp16_value(a.key_vn[kv_base + key]) : 0.f;
      n.rn[nt] = key < a.Sk ? fp16_value(a.key_rn[kv_base + key]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int key = blk + 8 * (i >> 1) + 2 * tq + (i & 1);
      n.kn[i] = key < a.Sk ? fp16_value(a.key_vn[kv_base + key]) : 0.f;
      n.nv[i] = key < a.Sk ? fp16_value(a.val_vn[kv_base + key]) : 0.f;
    }
  };
  Norms cur, nxt;
  const int blk0 = k_lo + kBlockKeys * warp;
  if (blk0 < k_hi) {
    stage(blk0, 0);
    load_norms(blk0, cur);
  }
  cp_async_commit();
  int st = 0;
  for (int blk = blk0; blk < k_hi; blk += kBlockKeys * kWarps, st ^= 1) {
    {
      const int nb = blk + kBlockKeys * kWarps;
      if (nb < k_hi) {
        stage(nb, st ^ 1);
        load_norms(nb, nxt);
      }
      cp_async_commit();
      cp_async_wait_all_but_one();  // this block's rows have landed; the next block's may still be in flight
      __syncwarp();
    }
    const uint8_t* stg = stage_ptr(warp, st);
    // ================= scores: S[nt] (16 rows x 8 keys), nt = 0, 1 =================
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      uint32_t kw[2][KW], sg[2][4], rr[2];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const uint4* pi = reinterpret_cast<const uint4*>(stg + (8 * nt + gq) * (16 * KB));
#pragma unroll
        for (int i = 0; i < KB; ++i) {
          const uint4 v = pi[i];
          kw[nt][4 * i] = v.x; kw[nt][4 * i + 1] = v.y; kw[nt][4 * i + 2] = v.z; kw[nt][4 * i + 3] = v.w;
        }
        const uint4 sv = *reinterpret_cast<const uint4*>(stg + kBlockKeys * 16 * KB + (8 * nt + gq) * 16);
        sg[nt][0] = ~sv.x; sg[nt][1] = ~sv.y; sg[nt][2] = ~sv.z; sg[nt][3] = ~sv.w;  // set bit = negative
        // the key norm multiplies the finished score in fp32 (below); the sketch half carries rn / n
        const float rho = cur.nk[nt] > 0.f ? __fdividef(cur.rn[nt], cur.nk[nt]) : 0.f;
        rr[nt] = bf16x2(rho, rho);
      }
      static_for<0, 16>([&](auto ks_c) {
        constexpr int ks = decltype(ks_c)::value;
        uint32_t qa[4];
        qa[0] = *reinterpret_cast<const uint32_t*>(&q_s[gq * kQPitch + 16 * ks + 2 * tq]);
        qa[1] = *reinterpret_cast<const uint32_t*>(&q_s[(gq + 8) * kQPitch + 16 * ks + 2 * tq]);
        qa[2] = *reinterpret_cast<const uint32_t*>(&q_s[gq * kQPitch + 16 * ks + 8 + 2 * tq]);
        qa[3] = *reinterpret_cast<const uint32_t*>(&q_s[(gq + 8) * kQPitch + 16 * ks + 8 + 2 * tq]);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          uint32_t b0, b1;
          if constexpr (ks < 8) {
            // coordinates 16 ks + 2 tq, +1 (b0) and + 8, + 9 (b1): two adjacent indices = one table entry
            // (the 16 indices of this k-step start at byte 2 KB ks; a pair is 2 KB bits wide)
            const uint32_t p0 = field<KW, 2 * KB * ks, 6 * KB, 2 * KB>(kw[nt], 2 * KB * tq);
            const uint32_t p1 = field<KW, 2 * KB * ks + KB, 6 * KB, 2 * KB>(kw[nt], 2 * KB * tq);
            b0 = lutK[p0];
            b1 = lutK[p1];
          } else {
            // sign bits of sketch coordinates 16 (ks - 8) + 2 tq, +1 and + 8, + 9
            const uint32_t hw = sg[nt][(ks - 8) / 2] >> (16 * ((ks - 8) & 1));
            b0 = rr[nt] ^ ((((hw >> (2 * tq)) & 3u) * 0x40008000u) & 0x80008000u);
            b1 = rr[nt] ^ ((((hw >> (2 * tq + 8)) & 3u) * 0x40008000u) & 0x80008000u);
          }
          mma16816(s[nt], qa, b0, b1);
        }
      });
    }
    // ================= online softmax on the fragments =================
    // s[nt][0..1]: row gq, keys blk + 8 nt + 2 tq, +1;  s[nt][2..3]: row gq + 8, same keys
    float mx[2] = {-INFINITY, -INFINITY};
    float kn[4];  // key norms (times the softmax scale) of this lane's score columns
#pragma unroll
    for (int i = 0; i < 4; ++i) kn[i] = cur.kn[i] * cexp;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int key = blk + 8 * nt + 2 * tq + (i & 1), h = i >> 1;
        const float x = (key <= row_lim[h] && key < k_hi) ? s[nt][i] * kn[2 * nt + (i & 1)] : -INFINITY;
        s[nt][i] = x;
        mx[h] = fmaxf(mx[h], x);
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    }
    // running maximum raised lazily (only when some row of the warp outgrew it by 2^8)
    const bool grow = __any_sync(0xffffffffu, mx[0] > m_run[0] + 8.f || mx[1] > m_run[1] + 8.f);
    if (grow) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float m_new = fmaxf(m_run[h], mx[h]);
        const float alpha = (m_run[h] == -INFINITY) ? 0.f : ex2(m_run[h] - m_new);
        m_run[h] = m_new;
        l_run[h] *= alpha;
#pragma unroll
        for (int ct = 0; ct < D / 8; ++ct) {
          o[ct][2 * h] *= alpha;
          o[ct][2 * h + 1] *= alpha;
        }
      }
    }
    // P, with the value norms folded in for the MMA (the row sum uses the plain probabilities)
    uint32_t pa[4];
    {
      float p[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int h = i >> 1;
          const float pv = ex2(s[nt][i] - (m_run[h] == -INFINITY ? 0.f : m_run[h]));
          l_run[h] += pv;
          p[nt][i] = pv * cur.nv[2 * nt + (i & 1)];
        }
      pa[0] = bf16x2(p[0][0], p[0][1]);  // row gq,     keys 2 tq, +1
      pa[1] = bf16x2(p[0][2], p[0][3]);  // row gq + 8, keys 2 tq, +1
      pa[2] = bf16x2(p[1][0], p[1][1]);  // row gq,     keys 8 + 2 tq, +1
      pa[3] = bf16x2(p[1][2], p[1][3]);  // row gq + 8, keys 8 + 2 tq, +1
    }
    // ================= O += P V_hat =================
    {
      uint32_t vw[4][VW];  // packed value indices of keys blk + 2 tq, +1, + 8 + 2 tq, + 9 + 2 tq
#pragma unroll
      for (int kq = 0; kq < 4; ++kq) {
        const uint4* pv = reinterpret_cast<const uint4*>(stg + kBlockKeys * 16 * (KB + 1) +
                                                         (8 * (kq >> 1) + 2 * tq + (kq & 1)) * (16 * VB));
#pragma unroll
        for (int i = 0; i < VB; ++i) {
          const uint4 v = pv[i];
          vw[kq][4 * i] = v.x; vw[kq][4 * i + 1] = v.y; vw[kq][4 * i + 2] = v.z; vw[kq][4 * i + 3] = v.w;
        }
      }
      static_for<0, D / 8>([&](auto ct_c) {
        constexpr int ct = decltype(ct_c)::value;
        // coordinate 8 ct + gq of the four keys
        // (the 8 indices of this coordinate tile start at byte VB ct of the row)
        uint32_t e[4];
#pragma unroll
        for (int kq = 0; kq < 4; ++kq) e[kq] = lutV[field<VW, VB * ct, 7 * VB, VB>(vw[kq], VB * gq)];
        const uint32_t b0 = __byte_perm(e[0], e[1], 0x5410), b1 = __byte_perm(e[2], e[3], 0x5410);
        mma16816(o[ct], pa, b0, b1);
      });
    }
    cur = nxt;
    __syncwarp();  // every lane is done with this stage before the next iteration refills it
  }

  // ---- merge: lanes of a quad (row sums), the four warps, then this split's partial result ----
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();  // the pool changes hands: every warp is done with the queries and its stages
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = gq + 8 * h;
#pragma unroll
    for (int ct = 0; ct < D / 8; ++ct) {
      mrg_o[warp][r][8 * ct + 2 * tq] = o[ct][2 * h];
      mrg_o[warp][r][8 * ct + 2 * tq + 1] = o[ct][2 * h + 1];
    }
    if (tq == 0) {
      mrg_ml[warp][r][0] = m_run[h];
      mrg_ml[warp][r][1] = l_run[h];
    }
  }
  __syncthreads();
  const int64_t unit = (b * a.Hkv + kvh) * a.nsplit + split;
  for (int e = tid; e < kRows * D; e += kWarps * 32) {
    const int r = e / D, c = e % D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) m = fmaxf(m, mrg_ml[w][r][0]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float mw = mrg_ml[w][r][0];
      const float f = (mw == -INFINITY) ? 0.f : ex2(mw - m);
      acc = fmaf(mrg_o[w][r][c], f, acc);
      l = fmaf(mrg_ml[w][r][1], f, l);
    }
    a.part_o[(unit * kRows + r) * D + c] = acc;
    if (c == 0) {
      a.part_ml[(unit * kRows + r) * 2] = m;
      a.part_ml[(unit * kRows + r) * 2 + 1] = l;
    }
  }
}

// out_rot[row of (b, h, s)][c] = sum_splits O_s 2^(m_s - m) / sum_splits l_s 2^(m_s - m), bf16
__global__ void __launch_bounds__(128) combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                      int nsplit, int64_t Hq, int64_t Hkv, int64_t Sq,
                                                      __nv_bfloat16* __restrict__ o_rot) {
  constexpr int D = 128;
  const int64_t unit = blockIdx.x;  // b * Hkv + kvh
  const int64_t b = unit / Hkv, kvh = unit % Hkv;
  const int G = (int)(Hq / Hkv), R = G * (int)Sq;
  const int c = threadIdx.x;
  for (int r = 0; r < R; ++r) {
    float m = -INFINITY;
    for (int s = 0; s < nsplit; ++s) m = fmaxf(m, part_ml[((unit * nsplit + s) * kRows + r) * 2]);
    float acc = 0.f, l = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const int64_t u = (unit * nsplit + s) * kRows + r;
      const float ms = part_ml[u * 2];
      const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - m);
      acc = fmaf(part_o[u * D + c], f, acc);
      l = fmaf(part_ml[u * 2 + 1], f, l);
    }
    const int64_t h = kvh * G + r / Sq, s = r % Sq;
    o_rot[((b * Hq + h) * Sq + s) * D + c] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
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
  return decode_enabled() && d == 128 && a.mask == nullptr && a.Hkv > 0 && (a.Hq / a.Hkv) * a.Sq <= kRows && a.Sk >= 4 * kBlockKeys * kWarps;
}

constexpr int64_t kMaxExtraUnits = 512;  // bound on (resident CTAs the splits are sized for): 3 per SM

size_t decode_workspace_bytes(int64_t BHq) {
  // at most (3 SM counts + B * Hkv) <= (512 + B * Hq) partial results of 16 rows x (128 + 2) floats
  return ((size_t)(kMaxExtraUnits + BHq) * kRows * (128 + 2) * sizeof(float) + 255) & ~(size_t)255;
}

int attention_decode(const AttnArgs& a, int64_t B, int bits, const void* q_cat, void* o_rot, void* part_ws,
                     cudaStream_t stream) {
  const int64_t units = B * a.Hkv;
  // enough CTAs for three per SM (what registers allow to be resident), each with at least 64 keys (one
  // 16-key block per warp)
  int64_t want = 3 * (int64_t)sm_count();
  if (want > kMaxExtraUnits) want = kMaxExtraUnits;
  int nsplit = (int)(want / units);  // rounded down: one CTA too many would wait for a whole extra wave
  const int max_split = (int)((a.Sk + kBlockKeys * kWarps - 1) / (kBlockKeys * kWarps));
  if (nsplit > max_split) nsplit = max_split;
  if (nsplit < 1) nsplit = 1;
  TQ_REQUIRE(units * nsplit <= kMaxExtraUnits + B * a.Hq, "partial-result workspace too small for %d splits", nsplit);
  int per = (int)((a.Sk + nsplit - 1) / nsplit);
  per = (per + kBlockKeys * kWarps - 1) / (kBlockKeys * kWarps) * (kBlockKeys * kWarps);
  nsplit = (int)((a.Sk + per - 1) / per);
  float* part_o = static_cast<float*>(part_ws);
  float* part_ml = part_o + (size_t)units * nsplit * kRows * 128;
  DecodeArgs da{static_cast<const __nv_bfloat16*>(q_cat), a.Hq, a.Hkv, a.Sq, a.Sk, a.key_idx, a.key_sgn, a.key_vn,
                a.key_rn, a.val_idx, a.val_vn, a.cen_k, a.cen_v, a.sm_scale, a.causal, part_o, part_ml, nsplit, per};
  dim3 grid((unsigned)nsplit, (unsigned)a.Hkv, (unsigned)B);
  {
    ProfScope prof(kProfAttention, stream);
    if (bits == 2) decode_kernel<2><<<grid, kWarps * 32, 0, stream>>>(da);
    else if (bits == 3) decode_kernel<3><<<grid, kWarps * 32, 0, stream>>>(da);
    else decode_kernel<4><<<grid, kWarps * 32, 0, stream>>>(da);
    TQ_CUDA_OK(cudaGetLastError());
    combine_kernel<<<(unsigned)units, 128, 0, stream>>>(part_o, part_ml, nsplit, a.Hq, a.Hkv, a.Sq,
                                                        static_cast<__nv_bfloat16*>(o_rot));
  }
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
}

}  // namespace tq
