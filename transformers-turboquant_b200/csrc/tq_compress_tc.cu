// Key / value compression with the rotation and the QJL projection on the tensor cores
// (TQ_MODE_BF16, bf16 inputs).
//
// A persistent CTA walks tiles of 128 vectors with D/32 threads per vector (row r = tensor-memory lane
// r; a thread owns 32 consecutive coordinates of its row, so the per-coordinate work of the epilogues
// runs on 16 warps at head_dim 128).  Per tile:
//   1. each thread loads its 64 bytes of the row (the next tile's are prefetched into registers while the
//      current one is processed), accumulates its part of the squared norm in fp32 (parts are summed
//      through shared memory in a fixed order) and writes the raw bf16 values into the A operand tile.  bf16 inputs are EXACT operands; the fp32 rotation matrix is split
//      into bf16 hi + lo parts, so y_raw = x (Pi_hi + Pi_lo)^T carries ~16 mantissa bits;
//   2. tcgen05.mma: Y_raw = X Pi_hi^T + X Pi_lo^T (fp32 accumulation in tensor memory);
//   3. epilogue: y = y_raw / (n + 1e-8), Lloyd-Max index by boundary counting, the row's packed
//      bytes assembled in registers and stored with 16-byte stores;
//   4. keys only: residual in rotated coordinates r = y_raw - n C[idx] (fp32), its squared norm,
//      r split into bf16 hi + lo and written over the A tile; tcgen05.mma
//      proj = r_hi Se_hi^T + r_hi Se_lo^T + r_lo Se_hi^T; sign bits of proj -> 16 bytes per row.
// Follows compressors.py:98-161, :270-294 of the reference; the arithmetic differs from the fp32
// kernel only in the ~2^-17 relative rounding of the split operands.
#include "tq_compress.cuh"
#include "tq_simt.cuh"
#include "tq_tcgen05.cuh"

namespace tq {

__device__ unsigned long long g_compress_faults = 0ull;  // expired bounded waits in this file's kernels
// this device's slot of the host-visible status page (NULL until the first call on the device installs it)
__device__ unsigned long long* g_fault_mailbox_compress = nullptr;
int set_fault_mailbox_compress(unsigned long long* slot) {
  TQ_CUDA_OK(cudaMemcpyToSymbol(g_fault_mailbox_compress, &slot, sizeof(slot)));
  return TQ_OK;
}

int read_compress_faults(unsigned long long* out) {
  TQ_CUDA_OK(cudaMemcpyFromSymbol(out, g_compress_faults, sizeof(*out)));
  return TQ_OK;
}

namespace {

__device__ __forceinline__ uint32_t bf16_bits(float v) {
  return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(v)));
}
__device__ __forceinline__ float bf16_value(uint32_t b) { return __uint_as_float(b << 16); }

// Copy a row-major fp32 [D, D] matrix into two canonical K-major bf16 operand tiles: hi = bf16(m),
// lo = bf16(m - hi).  Row j, 8-element chunk c at (j/8)*SBO + c*128 + (j%8)*16.
template <int D>
__device__ void load_split_matrix(const float* __restrict__ M, uint8_t* hi, uint8_t* lo, int tid, int nthreads) {
  constexpr int G = D / 8;
  constexpr uint32_t SBO = G * 128;
  for (int e = tid; e < D * G; e += nthreads) {
    const int j = e % 8 + 8 * (e / (8 * G)), c = (e / 8) % G;
    float v[8];
    load8<float>(M + j * D + c * 8, v);
    uint32_t h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t h0 = bf16_bits(v[2 * i]), h1 = bf16_bits(v[2 * i + 1]);
      h[i] = h0 | (h1 << 16);
      l[i] = bf16_bits(v[2 * i] - bf16_value(h0)) | (bf16_bits(v[2 * i + 1] - bf16_value(h1)) << 16);
    }
    const uint32_t off = (j / 8) * SBO + c * 128 + (j % 8) * 16;
    *reinterpret_cast<uint4*>(hi + off) = make_uint4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<uint4*>(lo + off) = make_uint4(l[0], l[1], l[2], l[3]);
  }
}

template <int D, int IB, bool IS_KEY>
__global__ void __launch_bounds__(4 * D, 1) compress_tc_kernel(const CompressArgs a) {
  constexpr int G = D / 8;
  constexpr int NP = D / 32;               // threads per row: each owns 32 consecutive coordinates
  constexpr int kThreads = 128 * NP;
  constexpr uint32_t SBO = G * 128;
  constexpr uint32_t MAT = D * D * 2;      // one bf16 matrix
  constexpr uint32_t TILE = 128 * D * 2;   // one bf16 A tile
  constexpr int NB = (1 << IB) - 1;
  constexpr int ROWB = D * IB / 8;         // packed index bytes per row (4 * IB of them per thread)
  constexpr int kCols = IS_KEY ? 2 * D : D;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* PiH = smem;
  uint8_t* PiL = PiH + MAT;
  uint8_t* SeH = PiL + MAT;                 // keys only
  uint8_t* SeL = SeH + (IS_KEY ? MAT : 0);
  uint8_t* A0 = SeL + (IS_KEY ? MAT : 0);   // X, later r_hi
  uint8_t* A1 = A0 + TILE;                  // r_lo (keys only)
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  __shared__ float cen_s[IS_KEY ? (1 << IB) : 1];
  __shared__ float ss_part[NP][128];        // partial squared norms of the row's parts
  __shared__ float rr_part[IS_KEY ? NP : 1][128];
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int row = (warp % 4) * 32 + lane;   // = tensor-memory lane
  const int part = warp / 4;                // coordinates [32 part, 32 part + 32)

  if (tid == 0) {
    s_abort = 0;
    tc::mbar_init(tc::smem_u32(&bar), 1);
    tc::fence_mbar_init();
  }
  if (warp == 0) tc::tmem_alloc(tc::smem_u32(&tmem_slot), kCols < 32 ? 32 : kCols);
  load_split_matrix<D>(a.Pi, PiH, PiL, tid, kThreads);
  if (IS_KEY) {
    load_split_matrix<D>(a.S_eff, SeH, SeL, tid, kThreads);
    if (tid < (1 << IB)) cen_s[tid] = a.centroids[tid];
  }
  float bnd[NB];
#pragma unroll
  for (int j = 0; j < NB; ++j) bnd[j] = __ldg(a.boundaries + j);
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t lane_base = (uint32_t)((warp % 4) * 32) << 16;
  const uint32_t bar_addr = tc::smem_u32(&bar);
  constexpr uint32_t idesc = tc::idesc_bf16(128, D, false, false);
  const uint64_t a0d = tc::smem_desc(tc::smem_u32(A0), 128, SBO), a1d = tc::smem_desc(tc::smem_u32(A1), 128, SBO);
  const uint64_t pihd = tc::smem_desc(tc::smem_u32(PiH), 128, SBO), pild = tc::smem_desc(tc::smem_u32(PiL), 128, SBO);
  const uint64_t sehd = tc::smem_desc(tc::smem_u32(SeH), 128, SBO), seld = tc::smem_desc(tc::smem_u32(SeL), 128, SBO);
  const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(a.src);
  const int64_t HS = a.H * a.S;
  uint32_t phase = 0;
  volatile int* abort_flag = &s_abort;

  uint4 rowbuf[4];  // this thread's 32 coordinates of its row of the tile about to be processed
  auto fetch = [&](int tile) {
    const int64_t n = static_cast<int64_t>(tile) * 128 + row;
    if (tile < a.num_tiles && n < a.n_vec) {
      const int64_t b = n / HS, rem = n % HS;
      const uint4* p = reinterpret_cast<const uint4*>(src + b * a.stride_b + (rem / a.S) * a.stride_h +
                                                      (rem % a.S) * a.stride_s) + 4 * part;
#pragma unroll
      for (int c = 0; c < 4; ++c) rowbuf[c] = p[c];
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c) rowbuf[c] = make_uint4(0, 0, 0, 0);
    }
  };
  fetch(blockIdx.x);

  for (int tile = blockIdx.x; tile < a.num_tiles; tile += gridDim.x) {
    const int64_t n = static_cast<int64_t>(tile) * 128 + row;
    const bool live = n < a.n_vec;
    const int64_t no = compress_out_row(a, n);  // where this vector's packed row goes
    // ---- 1. norm + A tile ------------------------------------------------------------------
    {
      float ss = 0.f;
      uint8_t* dst = A0 + (row / 8) * SBO + (row % 8) * 16 + 4 * part * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t w[4] = {rowbuf[c].x, rowbuf[c].y, rowbuf[c].z, rowbuf[c].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xffff0000u);
          ss = fmaf(lo, lo, ss);
          ss = fmaf(hi, hi, ss);
        }
        *reinterpret_cast<uint4*>(dst + c * 128) = rowbuf[c];
      }
      ss_part[part][row] = ss;
    }
    tc::fence_async_smem();
    tc::fence_before_sync();
    __syncthreads();
    // ---- 2. rotate ---------------------------------------------------------------------------
    if (tid == 0) {
      tc::fence_after_sync();
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks)
        tc::mma_bf16(tmem, a0d + (uint64_t)(ks * 256 >> 4), pihd + (uint64_t)(ks * 256 >> 4), idesc, ks > 0);
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks)
        tc::mma_bf16(tmem, a0d + (uint64_t)(ks * 256 >> 4), pild + (uint64_t)(ks * 256 >> 4), idesc, 1u);
      tc::mma_commit(bar_addr);
    }
    fetch(tile + gridDim.x);  // next tile's rows travel while this one is processed
    float ss = 0.f;  // summed in a fixed order, so that every part of the row sees the same norm
#pragma unroll
    for (int q = 0; q < NP; ++q) ss += ss_part[q][row];
    const float nv = sqrtf(ss), den = nv + 1e-8f;
    // y = y_raw / den is compared with the boundaries as y_raw > b * den (den > 0): one multiply per
    // boundary and row instead of one division per coordinate
    float bden[NB];
#pragma unroll
    for (int j = 0; j < NB; ++j) bden[j] = bnd[j] * den;
    if (!tc::mbar_wait_or_abort(bar_addr, phase, abort_flag)) break;
    phase ^= 1;
    tc::fence_after_sync();
    // ---- 3. index + pack (4. residual) ----------------------------------------------------------
    float rr = 0.f;
    uint32_t packed[IB];
#pragma unroll
    for (int i = 0; i < IB; ++i) packed[i] = 0;
    {
      uint32_t raw[32];
      tc::tmem_ld32(tmem + lane_base + 32 * part, raw);
      tc::wait_ld();
#pragma unroll
      for (int g8 = 0; g8 < 4; ++g8) {
        uint64_t word = 0;
        uint32_t rh[4], rl[4];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float yr = __uint_as_float(raw[g8 * 8 + e]);
          const int idx = count_below<NB>(yr, bden);
          word |= static_cast<uint64_t>(idx) << (e * IB);
          if (IS_KEY) {
            const float res = fmaf(-nv, cen_s[idx], yr);
            rr = fmaf(res, res, rr);
            const uint32_t hb = bf16_bits(res), lb = bf16_bits(res - bf16_value(hb));
            if (e & 1) { rh[e / 2] |= hb << 16; rl[e / 2] |= lb << 16; }
            else { rh[e / 2] = hb; rl[e / 2] = lb; }
          }
        }
        // the 8 fields of this group are IB whole bytes at byte offset g8*IB of the thread's 4*IB bytes
#pragma unroll
        for (int bt = 0; bt < IB; ++bt) {
          const int byte = g8 * IB + bt;
          packed[byte / 4] |= static_cast<uint32_t>((word >> (8 * bt)) & 0xffu) << (8 * (byte % 4));
        }
        if (IS_KEY) {
          const uint32_t off = (row / 8) * SBO + (4 * part + g8) * 128 + (row % 8) * 16;
          *reinterpret_cast<uint4*>(A0 + off) = make_uint4(rh[0], rh[1], rh[2], rh[3]);
          *reinterpret_cast<uint4*>(A1 + off) = make_uint4(rl[0], rl[1], rl[2], rl[3]);
        }
      }
    }
    if (live) {
      uint32_t* dst = reinterpret_cast<uint32_t*>(a.packed_idx + no * ROWB + 4 * IB * part);
      if constexpr (IB == 4) *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      else if constexpr (IB == 2) *reinterpret_cast<uint2*>(dst) = make_uint2(packed[0], packed[1]);
      else {
#pragma unroll
        for (int i = 0; i < IB; ++i) dst[i] = packed[i];
      }
      if (part == 0) a.vec_norms[no] = fp16_bits(nv);
    }
    if (IS_KEY) {
      // ---- QJL sketch of the residual --------------------------------------------------------
      rr_part[part][row] = rr;
      tc::fence_async_smem();
      tc::fence_before_sync();
      __syncthreads();
      if (tid == 0) {
        tc::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          tc::mma_bf16(tmem + D, a0d + (uint64_t)(ks * 256 >> 4), sehd + (uint64_t)(ks * 256 >> 4), idesc, ks > 0);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          tc::mma_bf16(tmem + D, a0d + (uint64_t)(ks * 256 >> 4), seld + (uint64_t)(ks * 256 >> 4), idesc, 1u);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          tc::mma_bf16(tmem + D, a1d + (uint64_t)(ks * 256 >> 4), sehd + (uint64_t)(ks * 256 >> 4), idesc, 1u);
        tc::mma_commit(bar_addr);
      }
      if (live && part == 0) {
        float rs = 0.f;
#pragma unroll
        for (int q = 0; q < NP; ++q) rs += rr_part[q][row];
        a.residual_norms[no] = fp16_bits(sqrtf(rs));
      }
      if (!tc::mbar_wait_or_abort(bar_addr, phase, abort_flag)) break;
      phase ^= 1;
      tc::fence_after_sync();
      uint32_t raw[32];
      tc::tmem_ld32(tmem + D + lane_base + 32 * part, raw);
      tc::wait_ld();
      uint32_t bits = 0;
#pragma unroll
      for (int e = 0; e < 32; ++e) bits |= (__uint_as_float(raw[e]) >= 0.f ? 1u : 0u) << e;
      if (live) *reinterpret_cast<uint32_t*>(a.packed_signs + no * (D / 8) + 4 * part) = bits;
    }
    tc::fence_before_sync();
    __syncthreads();  // the next tile overwrites the A tiles, the partial sums and the accumulators
  }
  if (s_abort) {
    if (tid == 0) {
      atomicAdd(&g_compress_faults, 1ull);
      notify_host_of_fault(g_fault_mailbox_compress);
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem, kCols < 32 ? 32 : kCols);
}

template <int D, int IB, bool IS_KEY>
int launch(const CompressArgs& a, cudaStream_t stream) {
  constexpr size_t smem_req = (size_t)(IS_KEY ? 4 : 2) * D * D * 2 + (size_t)(IS_KEY ? 2 : 1) * 128 * D * 2;
  // one CTA of 4 D threads per SM (16 warps at head_dim 128): the register file does not hold two
  constexpr int per_sm = 1;
  auto kern = compress_tc_kernel<D, IB, IS_KEY>;
  TQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_req));
  const int tiles = (int)((a.n_vec + 127) / 128);
  CompressArgs b = a;
  b.num_tiles = tiles;
  int grid = sm_count() * per_sm;
  if (grid > tiles) grid = tiles;
  {
    ProfScope prof(IS_KEY ? kProfCompressKeys : kProfCompressValues, stream);
    kern<<<grid, 4 * D, smem_req, stream>>>(b);
  }
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
}

}  // namespace

int compress_tc(bool is_key, int d, int ib, const CompressArgs& a, cudaStream_t stream) {
  if (is_key) {
    if (d == 128) return ib == 1 ? launch<128, 1, true>(a, stream) : ib == 2 ? launch<128, 2, true>(a, stream)
                                                                             : launch<128, 3, true>(a, stream);
    return ib == 1 ? launch<64, 1, true>(a, stream) : ib == 2 ? launch<64, 2, true>(a, stream)
                                                              : launch<64, 3, true>(a, stream);
  }
  if (d == 128) return ib == 2 ? launch<128, 2, false>(a, stream) : ib == 3 ? launch<128, 3, false>(a, stream)
                                                                            : launch<128, 4, false>(a, stream);
  return ib == 2 ? launch<64, 2, false>(a, stream) : ib == 3 ? launch<64, 3, false>(a, stream)
                                                             : launch<64, 4, false>(a, stream);
}

}  // namespace tq
