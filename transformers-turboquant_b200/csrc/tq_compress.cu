// Key / value compression, fp32 arithmetic on the CUDA cores (TQ_MODE_FP32).
//
// One persistent CTA per SM walks tiles of 64 vectors.  Per tile:
//   1. coalesced 16-byte loads of the vectors, row norms by half-warp shuffles,
//      x / (n + 1e-8) written to shared memory;
//   2. y = x Pi^T as a register-tiled fp32 GEMM (4 rows x 8 consecutive coordinates
//      per thread) against Pi^T held in shared memory;
//   3. Lloyd-Max index by boundary counting; the 8 indices a thread owns are exactly
//      `b` whole bytes of the row's LSB-first bit stream, stored without atomics;
//   4. keys only: residual in rotated coordinates r = (n + 1e-8) y - n C[idx] (equal to
//      (x - k_mse) Pi^T), its norm, and sign(r S_eff^T) from a second GEMM; 8 sign bits
//      = one byte per thread.
// Everything stays in rotated coordinates, so no back-rotation GEMM is needed.
//
// Follows TurboQuantCompressorV2.compress / TurboQuantCompressorMSE.compress of the
// reference (src/turboquant_pytorch/compressors.py:98-161, :270-294).
#include "tq_common.cuh"
#include "tq_simt.cuh"
#include "tq_compress.cuh"
#include "tq_attention.cuh"

namespace tq {

template <typename T, int D, int IB, bool IS_KEY>
__global__ void __launch_bounds__(16 * (D / 8)) compress_simt_kernel(const CompressArgs a) {
  constexpr int TX = D / 8;
  constexpr int NT = 16 * TX;
  constexpr int XS = D + 4;  // padded row stride of the tile
  constexpr int NB = (1 << IB) - 1;
  extern __shared__ __align__(16) float smem[];
  float* PiT = smem;                                  // [D][D] permuted columns
  float* SeT = PiT + D * D;                           // keys only
  float* X = SeT + (IS_KEY ? D * D : 0);              // [64][XS]
  float* nrm = X + kTileRows * XS;                    // [64] norms

  const int tid = threadIdx.x;
  const int tx = tid % TX, ty = tid / TX;
  const int row0 = ty * 4;

  load_matrix<D, true>(a.Pi, PiT, tid, NT);
  if (IS_KEY) load_matrix<D, true>(a.S_eff, SeT, tid, NT);
  float bnd[NB];
#pragma unroll
  for (int j = 0; j < NB; ++j) bnd[j] = __ldg(a.boundaries + j);
  float cen[IS_KEY ? (1 << IB) : 1];
  if (IS_KEY) {
#pragma unroll
    for (int j = 0; j < (1 << IB); ++j) cen[j] = __ldg(a.centroids + j);
  }
  const T* src = static_cast<const T*>(a.src);
  const int64_t HS = a.H * a.S;

  for (int tile = blockIdx.x; tile < a.num_tiles; tile += gridDim.x) {
    const int64_t base = static_cast<int64_t>(tile) * kTileRows;
    __syncthreads();  // previous tile's readers of X are done; also covers the matrix loads
    // ---- 1. load, norm, normalise --------------------------------------------------
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int64_t n = base + row0 + r;
      float v[8];
      if (n < a.n_vec) {
        const int64_t b = n / HS, rem = n % HS;
        const int64_t h = rem / a.S, s = rem % a.S;
        load8<T>(src + b * a.stride_b + h * a.stride_h + s * a.stride_s + tx * 8, v);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = 0.f;
      }
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss = fmaf(v[e], v[e], ss);
#pragma unroll
      for (int off = TX / 2; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
      const float nv = sqrtf(ss);
      const float inv_den = nv + 1e-8f;
      float* xr = X + (row0 + r) * XS + tx * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) xr[e] = v[e] / inv_den;
      if (tx == 0) nrm[row0 + r] = nv;
    }
    __syncthreads();
    // ---- 2. rotate -------------------------------------------------------------------
    float y[4][8];
    tile_gemm<D, XS>(X, PiT, row0, tx, y);
    if (IS_KEY) __syncthreads();  // X is about to be overwritten with the residual
    // ---- 3. index, pack, 4. residual ---------------------------------------------------
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int64_t n = base + row0 + r;
      const int64_t no = compress_out_row(a, n);
      int f[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) f[c] = count_below<NB>(y[r][c], bnd);
      if (n < a.n_vec) store_fields8<IB>(a.packed_idx + no * (D * IB / 8) + tx * IB, f);
      const float nv = nrm[row0 + r];
      if (IS_KEY) {
        const float np = nv + 1e-8f;
        float rr = 0.f;
        float* xr = X + (row0 + r) * XS + tx * 8;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float cv = cen[0];
#pragma unroll
          for (int j = 1; j < (1 << IB); ++j) cv = (f[c] == j) ? cen[j] : cv;
          const float res = fmaf(np, y[r][c], -nv * cv);
          xr[c] = res;
          rr = fmaf(res, res, rr);
        }
#pragma unroll
        for (int off = TX / 2; off > 0; off >>= 1) rr += __shfl_xor_sync(0xffffffffu, rr, off);
        if (tx == 0 && n < a.n_vec) {
          a.vec_norms[no] = fp16_bits(nv);
          a.residual_norms[no] = fp16_bits(sqrtf(rr));
        }
      } else if (tx == 0 && n < a.n_vec) {
        a.vec_norms[no] = fp16_bits(nv);
      }
    }
    if (IS_KEY) {
      __syncthreads();
      float p[4][8];
      tile_gemm<D, XS>(X, SeT, row0, tx, p);
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int64_t n = base + row0 + r;
        unsigned bits = 0;
#pragma unroll
        for (int c = 0; c < 8; ++c) bits |= (p[r][c] >= 0.f ? 1u : 0u) << c;
        if (n < a.n_vec) a.packed_signs[compress_out_row(a, n) * (D / 8) + tx] = static_cast<uint8_t>(bits);
      }
    }
  }
}

template <int D, bool IS_KEY>
constexpr size_t compress_smem_bytes() {
  return sizeof(float) * (size_t)((IS_KEY ? 2 : 1) * D * D + kTileRows * (D + 4) + kTileRows);
}

template <typename T, int D, int IB, bool IS_KEY>
static int launch_compress(const CompressArgs& a, cudaStream_t stream) {
  constexpr size_t smem = compress_smem_bytes<D, IS_KEY>();
  auto kern = compress_simt_kernel<T, D, IB, IS_KEY>;
  TQ_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int per_sm = smem > 110 * 1024 ? 1 : 2;
  int grid = sm_count() * per_sm;
  if (grid > a.num_tiles) grid = a.num_tiles;
  {
    ProfScope prof(IS_KEY ? kProfCompressKeys : kProfCompressValues, stream);
    kern<<<grid, 16 * (D / 8), smem, stream>>>(a);
  }
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
}

template <typename T, int D, bool IS_KEY>
static int dispatch_ib(int ib, const CompressArgs& a, cudaStream_t stream) {
  // keys index with bits-1 in 1..3 bits, values with bits in 2..4
  if constexpr (IS_KEY) {
    if (ib == 1) return launch_compress<T, D, 1, true>(a, stream);
  } else {
    if (ib == 4) return launch_compress<T, D, 4, false>(a, stream);
  }
  if (ib == 2) return launch_compress<T, D, 2, IS_KEY>(a, stream);
  if (ib == 3) return launch_compress<T, D, 3, IS_KEY>(a, stream);
  return fail(TQ_ERR_INVALID_ARG, "index width %d unsupported", ib);
}

template <bool IS_KEY>
static int dispatch_compress(int dtype, int d, int ib, const CompressArgs& a, int mode, cudaStream_t stream) {
  // tensor-core kernel: bf16 inputs are exact MMA operands; other input types keep the fp32 kernel
  if (mode == TQ_MODE_BF16 && dtype == TQ_BF16) return compress_tc(IS_KEY, d, ib, a, stream);
#define TQ_CASE(TYPE)                                               \
  if (d == 128) return dispatch_ib<TYPE, 128, IS_KEY>(ib, a, stream); \
  return dispatch_ib<TYPE, 64, IS_KEY>(ib, a, stream);
  if (dtype == TQ_F32) { TQ_CASE(float) }
  if (dtype == TQ_BF16) { TQ_CASE(__nv_bfloat16) }
  TQ_CASE(__half)
#undef TQ_CASE
}

static int check_states(const void* p, int dtype, int64_t B, int64_t H, int64_t S, int d,
                        int64_t sb, int64_t sh, int64_t ss, int bits) {
  TQ_REQUIRE(dtype == TQ_F32 || dtype == TQ_BF16 || dtype == TQ_F16, "unknown dtype %d", dtype);
  TQ_REQUIRE(valid_head_dim(d), "head_dim %d unsupported (64 or 128)", d);
  TQ_REQUIRE(valid_bits(bits), "bits %d unsupported (2, 3 or 4)", bits);
  TQ_REQUIRE(B >= 0 && H >= 0 && S >= 0, "negative size");
  TQ_REQUIRE(B * H * S < ((int64_t)1 << 31) * kTileRows, "too many vectors");
  if (B * H * S == 0) return TQ_OK;
  TQ_REQUIRE(p != nullptr, "NULL input pointer");
  const int64_t align_elems = 16 / elem_size(dtype);
  TQ_REQUIRE(aligned16(p), "input base pointer must be 16-byte aligned");
  TQ_REQUIRE(sb % align_elems == 0 && sh % align_elems == 0 && ss % align_elems == 0,
             "strides must keep every row 16-byte aligned");
  TQ_REQUIRE(ss >= d || S <= 1, "row stride %lld smaller than head_dim", (long long)ss);
  return TQ_OK;
}

}  // namespace tq

using namespace tq;

extern "C" {

static int compress_keys_entry(const void* keys, int dtype, int64_t B, int64_t H, int64_t S, int d,
                     int64_t stride_b, int64_t stride_h, int64_t stride_s, const float* Pi,
                     const float* S_eff, const float* centroids, const float* boundaries, int bits,
                     uint8_t* packed_idx, uint8_t* packed_signs, uint16_t* vec_norms,
                     uint16_t* residual_norms, int64_t out_stride, int64_t out_offset, int mode, void* stream) {
  if (int st = check_states(keys, dtype, B, H, S, d, stride_b, stride_h, stride_s, bits)) return st;
  TQ_REQUIRE(mode == TQ_MODE_FP32 || mode == TQ_MODE_BF16, "unknown mode %d", mode);
  const int64_t n = B * H * S;
  if (n == 0) return TQ_OK;
  TQ_REQUIRE(Pi && S_eff && centroids && boundaries, "NULL constant pointer");
  TQ_REQUIRE(packed_idx && packed_signs && vec_norms && residual_norms, "NULL output pointer");
  CallScope scope(keys, "keys", static_cast<cudaStream_t>(stream));
  if (scope.status()) return scope.status();
  CompressArgs a{keys, n, H, S, stride_b, stride_h, stride_s, Pi, S_eff, centroids, boundaries,
                 packed_idx, packed_signs, vec_norms, residual_norms,
                 (int)((n + kTileRows - 1) / kTileRows), out_stride, out_offset};
  return dispatch_compress<true>(dtype, d, bits - 1, a, mode, static_cast<cudaStream_t>(stream));
}

static int compress_values_entry(const void* values, int dtype, int64_t B, int64_t H, int64_t S, int d,
                       int64_t stride_b, int64_t stride_h, int64_t stride_s, const float* Pi,
                       const float* boundaries, int bits, uint8_t* packed_idx, uint16_t* vec_norms,
                       int64_t out_stride, int64_t out_offset, int mode, void* stream) {
  if (int st = check_states(values, dtype, B, H, S, d, stride_b, stride_h, stride_s, bits)) return st;
  TQ_REQUIRE(mode == TQ_MODE_FP32 || mode == TQ_MODE_BF16, "unknown mode %d", mode);
  const int64_t n = B * H * S;
  if (n == 0) return TQ_OK;
  TQ_REQUIRE(Pi && boundaries, "NULL constant pointer");
  TQ_REQUIRE(packed_idx && vec_norms, "NULL output pointer");
  CallScope scope(values, "values", static_cast<cudaStream_t>(stream));
  if (scope.status()) return scope.status();
  CompressArgs a{values, n, H, S, stride_b, stride_h, stride_s, Pi, nullptr, nullptr, boundaries,
                 packed_idx, nullptr, vec_norms, nullptr, (int)((n + kTileRows - 1) / kTileRows), out_stride, out_offset};
  return dispatch_compress<false>(dtype, d, bits, a, mode, static_cast<cudaStream_t>(stream));
}

int tq_compress_kv(const void* keys, const void* values, int dtype, int64_t B, int64_t H, int64_t S, int d,
                   int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s, int64_t v_stride_b,
                   int64_t v_stride_h, int64_t v_stride_s, const void* constants, int bits, uint8_t* key_idx,
                   uint8_t* key_signs, uint16_t* key_vec_norms, uint16_t* key_residual_norms, uint8_t* val_idx,
                   uint16_t* val_vec_norms, int64_t kv_capacity, int64_t kv_offset, int mode, void* stream) {
  TQ_REQUIRE(constants != nullptr && (reinterpret_cast<uintptr_t>(constants) & 255u) == 0,
             "constants must be a 256-byte aligned buffer filled by tq_prepare_constants");
  TQ_REQUIRE(kv_offset >= 0 && S >= 0 && kv_offset + S <= kv_capacity,
             "%lld new tokens behind %lld do not fit a cache of %lld", (long long)S, (long long)kv_offset,
             (long long)kv_capacity);
  TQ_REQUIRE(mode == TQ_MODE_FP32 || mode == TQ_MODE_BF16, "unknown mode %d", mode);
  if (keys != nullptr)
    if (int st = check_states(keys, dtype, B, H, S, d, k_stride_b, k_stride_h, k_stride_s, bits)) return st;
  if (values != nullptr)
    if (int st = check_states(values, dtype, B, H, S, d, v_stride_b, v_stride_h, v_stride_s, bits)) return st;
  if (keys == nullptr && values == nullptr) {
    TQ_REQUIRE(B * H * S == 0, "NULL input pointers");
    return check_states(nullptr, dtype, B, H, S, d, 0, 0, d, bits);
  }
  if (B * H * S == 0) return TQ_OK;
  TQ_REQUIRE(keys == nullptr || (key_idx && key_signs && key_vec_norms && key_residual_norms), "NULL key output pointer");
  TQ_REQUIRE(values == nullptr || (val_idx && val_vec_norms), "NULL value output pointer");
  const uint8_t* c = static_cast<const uint8_t*>(constants);
  if (compress_kv_applies(dtype, d, mode)) {
    CallScope scope(keys != nullptr ? keys : values, "keys/values", static_cast<cudaStream_t>(stream));
    if (scope.status()) return scope.status();
    const int64_t ks[3] = {k_stride_b, k_stride_h, k_stride_s}, vs[3] = {v_stride_b, v_stride_h, v_stride_s};
    const int st = compress_kv(keys, values, B, H, S, ks, vs, c, bits, key_idx, key_signs, key_vec_norms,
                               key_residual_norms, val_idx, val_vec_norms, kv_capacity, kv_offset,
                               static_cast<cudaStream_t>(stream));
    if (st != TQ_ERR_UNSUPPORTED) return st;  // strides no tensor map describes: the per-side kernels read them
  }
  const ConstLayout L = const_layout(d);
  auto f32 = [&](size_t off) { return reinterpret_cast<const float*>(c + off); };
  if (keys != nullptr)
    if (int st = compress_keys_entry(keys, dtype, B, H, S, d, k_stride_b, k_stride_h, k_stride_s, f32(L.pi_k),
                                     f32(L.s_eff), f32(L.cen_k), f32(L.bnd_k), bits, key_idx, key_signs,
                                     key_vec_norms, key_residual_norms, kv_capacity, kv_offset, mode, stream))
      return st;
  if (values != nullptr)
    return compress_values_entry(values, dtype, B, H, S, d, v_stride_b, v_stride_h, v_stride_s, f32(L.pi_v),
                                 f32(L.bnd_v), bits, val_idx, val_vec_norms, kv_capacity, kv_offset, mode, stream);
  return TQ_OK;
}

int tq_compress_keys(const void* keys, int dtype, int64_t B, int64_t H, int64_t S, int d,
                     int64_t stride_b, int64_t stride_h, int64_t stride_s, const float* Pi,
                     const float* S_eff, const float* centroids, const float* boundaries, int bits,
                     uint8_t* packed_idx, uint8_t* packed_signs, uint16_t* vec_norms,
                     uint16_t* residual_norms, int mode, void* stream) {
  return compress_keys_entry(keys, dtype, B, H, S, d, stride_b, stride_h, stride_s, Pi, S_eff, centroids, boundaries,
                             bits, packed_idx, packed_signs, vec_norms, residual_norms, S, 0, mode, stream);
}

int tq_compress_values(const void* values, int dtype, int64_t B, int64_t H, int64_t S, int d,
                       int64_t stride_b, int64_t stride_h, int64_t stride_s, const float* Pi,
                       const float* boundaries, int bits, uint8_t* packed_idx, uint16_t* vec_norms,
                       int mode, void* stream) {
  return compress_values_entry(values, dtype, B, H, S, d, stride_b, stride_h, stride_s, Pi, boundaries, bits,
                               packed_idx, vec_norms, S, 0, mode, stream);
}

int tq_append_keys(const void* keys, int dtype, int64_t B, int64_t H, int64_t S, int d,
                   int64_t stride_b, int64_t stride_h, int64_t stride_s, const float* Pi,
                   const float* S_eff, const float* centroids, const float* boundaries, int bits,
                   uint8_t* packed_idx, uint8_t* packed_signs, uint16_t* vec_norms,
                   uint16_t* residual_norms, int64_t kv_capacity, int64_t kv_offset, int mode, void* stream) {
  TQ_REQUIRE(kv_offset >= 0 && S >= 0 && kv_offset + S <= kv_capacity,
             "%lld new tokens behind %lld do not fit a cache of %lld", (long long)S, (long long)kv_offset,
             (long long)kv_capacity);
  return compress_keys_entry(keys, dtype, B, H, S, d, stride_b, stride_h, stride_s, Pi, S_eff, centroids, boundaries,
                             bits, packed_idx, packed_signs, vec_norms, residual_norms, kv_capacity, kv_offset, mode,
                             stream);
}

int tq_append_values(const void* values, int dtype, int64_t B, int64_t H, int64_t S, int d,
                     int64_t stride_b, int64_t stride_h, int64_t stride_s, const float* Pi,
                     const float* boundaries, int bits, uint8_t* packed_idx, uint16_t* vec_norms,
                     int64_t kv_capacity, int64_t kv_offset, int mode, void* stream) {
  TQ_REQUIRE(kv_offset >= 0 && S >= 0 && kv_offset + S <= kv_capacity,
             "%lld new tokens behind %lld do not fit a cache of %lld", (long long)S, (long long)kv_offset,
             (long long)kv_capacity);
  return compress_values_entry(values, dtype, B, H, S, d, stride_b, stride_h, stride_s, Pi, boundaries, bits,
                               packed_idx, vec_norms, kv_capacity, kv_offset, mode, stream);
}

}  // extern "C"
