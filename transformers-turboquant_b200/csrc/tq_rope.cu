// Rotary position embedding of the query and key heads of one attention layer in ONE launch.
//
// The reference's adapters call HF's apply_rotary_pos_emb before they compress the keys
// (src/transformers_turboquant/families/llama.py:98, qwen2.py:98): q*cos + rotate_half(q)*sin as four
// elementwise torch kernels and a concatenation per tensor, i.e. about ten passes over q and k.  This
// kernel reads every element once and writes it once, in the [B, H, S, D] layout the compression and
// attention kernels like best, and reproduces torch's arithmetic to the bit: every product and the sum
// are rounded to the tensor dtype, as the separate torch kernels round them.
//
// HBM-bound: 2 x (B (Hq + Hkv) S D) elements in + out, plus the cos/sin rows (shared by all heads: L2).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "tq_common.cuh"

namespace tq {
namespace {

struct RopeArgs {
  const void *q, *k, *cos, *sin;
  void *q_out, *k_out;
  int64_t B, Hq, Hkv, S;
  int64_t qsb, qsh, qss, ksb, ksh, kss, csb, css;  // element strides
  int d;
};

template <int DTYPE>
struct Elem;
template <>
struct Elem<TQ_BF16> {
  using T = __nv_bfloat16;
  static __device__ __forceinline__ float up(T v) { return __bfloat162float(v); }
  static __device__ __forceinline__ float rn(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
  static __device__ __forceinline__ T down(float v) { return __float2bfloat16_rn(v); }
};
template <>
struct Elem<TQ_F16> {
  using T = __half;
  static __device__ __forceinline__ float up(T v) { return __half2float(v); }
  static __device__ __forceinline__ float rn(float v) { return __half2float(__float2half_rn(v)); }
  static __device__ __forceinline__ T down(float v) { return __float2half_rn(v); }
};
template <>
struct Elem<TQ_F32> {
  using T = float;
  static __device__ __forceinline__ float up(T v) { return v; }
  static __device__ __forceinline__ float rn(float v) { return v; }
  static __device__ __forceinline__ T down(float v) { return v; }
};

// 16 bytes of a row
template <typename T>
struct alignas(16) Chunk {
  T v[16 / sizeof(T)];
};

// One work item = one 16-byte chunk of the first half of a row and its partner in the second half.
// Items are numbered in the memory order of the projection output ([B, S, H, D]: consecutive threads read
// consecutive bytes); each output row is written in two 16-byte-per-thread runs.
// IDX: uint32_t when the item count fits (64-bit divisions would otherwise dominate the instruction stream).
template <int DTYPE, typename IDX>
__global__ void __launch_bounds__(256) rope_kernel(const RopeArgs a) {
  using E = Elem<DTYPE>;
  using T = typename E::T;
  constexpr int N = 16 / (int)sizeof(T);  // elements per chunk
  const int half = a.d / 2;
  const IDX cpr = (IDX)(half / N);  // chunks per half row
  const IDX H = (IDX)(a.Hq + a.Hkv), S = (IDX)a.S;
  const IDX items = (IDX)a.B * S * H * cpr;
  for (IDX it = (IDX)blockIdx.x * blockDim.x + threadIdx.x; it < items; it += (IDX)gridDim.x * blockDim.x) {
    const int c = (int)(it % cpr);
    IDX r = it / cpr;
    const int64_t h = (int64_t)(r % H);
    r /= H;
    const int64_t s = (int64_t)(r % S), b = (int64_t)(r / S);
    const bool is_q = h < a.Hq;
    const int64_t hh = is_q ? h : h - a.Hq;
    const T* src = is_q ? static_cast<const T*>(a.q) + b * a.qsb + hh * a.qsh + s * a.qss
                        : static_cast<const T*>(a.k) + b * a.ksb + hh * a.ksh + s * a.kss;
    T* dst = is_q ? static_cast<T*>(a.q_out) + ((b * a.Hq + hh) * a.S + s) * a.d
                  : static_cast<T*>(a.k_out) + ((b * a.Hkv + hh) * a.S + s) * a.d;
    const T* cs = static_cast<const T*>(a.cos) + b * a.csb + s * a.css;
    const T* sn = static_cast<const T*>(a.sin) + b * a.csb + s * a.css;
    const Chunk<T> xlo = *reinterpret_cast<const Chunk<T>*>(src + c * N);
    const Chunk<T> xhi = *reinterpret_cast<const Chunk<T>*>(src + half + c * N);
    const Chunk<T> clo = *reinterpret_cast<const Chunk<T>*>(cs + c * N);
    const Chunk<T> chi = *reinterpret_cast<const Chunk<T>*>(cs + half + c * N);
    const Chunk<T> slo = *reinterpret_cast<const Chunk<T>*>(sn + c * N);
    const Chunk<T> shi = *reinterpret_cast<const Chunk<T>*>(sn + half + c * N);
    Chunk<T> olo, ohi;
#pragma unroll
    for (int e = 0; e < N; ++e) {
      const float lo = E::up(xlo.v[e]), hi = E::up(xhi.v[e]);
      // out[i] = x[i] cos[i] - x[i + d/2] sin[i];  out[i + d/2] = x[i + d/2] cos[i + d/2] + x[i] sin[i + d/2];
      // each product and the sum rounded to the tensor dtype (no fused multiply-add)
      olo.v[e] = E::down(__fadd_rn(E::rn(__fmul_rn(lo, E::up(clo.v[e]))), E::rn(__fmul_rn(-hi, E::up(slo.v[e])))));
      ohi.v[e] = E::down(__fadd_rn(E::rn(__fmul_rn(hi, E::up(chi.v[e]))), E::rn(__fmul_rn(lo, E::up(shi.v[e])))));
    }
    *reinterpret_cast<Chunk<T>*>(dst + c * N) = olo;
    *reinterpret_cast<Chunk<T>*>(dst + half + c * N) = ohi;
  }
}

inline bool aligned16p(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace tq

using namespace tq;

extern "C" int tq_rope(const void* q, const void* k, int dtype, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int d,
                       int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s, int64_t k_stride_b,
                       int64_t k_stride_h, int64_t k_stride_s, const void* cos, const void* sin, int64_t cs_stride_b,
                       int64_t cs_stride_s, void* q_out, void* k_out, void* stream) {
  TQ_REQUIRE(dtype == TQ_F32 || dtype == TQ_BF16 || dtype == TQ_F16, "unknown dtype %d", dtype);
  TQ_REQUIRE(B >= 0 && Hq >= 0 && Hkv >= 0 && S >= 0, "negative extent");
  TQ_REQUIRE(d > 0 && d % 32 == 0, "head_dim %d must be a positive multiple of 32", d);
  if (B == 0 || S == 0 || Hq + Hkv == 0) return TQ_OK;
  TQ_REQUIRE(cos && sin, "NULL cos / sin");
  TQ_REQUIRE((Hq == 0 || (q && q_out)) && (Hkv == 0 || (k && k_out)), "NULL pointer");
  const int n = dtype == TQ_F32 ? 4 : 8;  // elements per 16 bytes
  TQ_REQUIRE(aligned16p(q) && aligned16p(k) && aligned16p(cos) && aligned16p(sin) && aligned16p(q_out) && aligned16p(k_out),
             "all tensors must be 16-byte aligned");
  TQ_REQUIRE(q_stride_b % n == 0 && q_stride_h % n == 0 && q_stride_s % n == 0 && k_stride_b % n == 0 &&
                 k_stride_h % n == 0 && k_stride_s % n == 0 && cs_stride_b % n == 0 && cs_stride_s % n == 0,
             "strides must keep rows 16-byte aligned");
  TQ_REQUIRE(q_out != q && k_out != k, "outputs must not alias the inputs");
  const cudaStream_t s = static_cast<cudaStream_t>(stream);
  CallScope scope(Hq > 0 ? q : k, "q", s);
  if (scope.status()) return scope.status();
  const RopeArgs a{q, k, cos, sin, q_out, k_out, B, Hq, Hkv, S, q_stride_b, q_stride_h, q_stride_s,
                   k_stride_b, k_stride_h, k_stride_s, cs_stride_b, cs_stride_s, d};
  const int64_t items = B * S * (Hq + Hkv) * (d / 2 / n);
  int dev = 0, sms = 148;
  TQ_CUDA_OK(cudaGetDevice(&dev));
  TQ_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int64_t want = (items + 255) / 256, cap = (int64_t)sms * 8;  // 8 resident CTAs of 256 threads per SM
  const unsigned grid = (unsigned)(want < cap ? want : cap);
  const bool small = items + (int64_t)grid * 256 < (int64_t)0xffffffffu;  // the loop counter may overshoot once
  if (dtype == TQ_BF16) {
    if (small) rope_kernel<TQ_BF16, uint32_t><<<grid, 256, 0, s>>>(a);
    else rope_kernel<TQ_BF16, int64_t><<<grid, 256, 0, s>>>(a);
  } else if (dtype == TQ_F16) {
    if (small) rope_kernel<TQ_F16, uint32_t><<<grid, 256, 0, s>>>(a);
    else rope_kernel<TQ_F16, int64_t><<<grid, 256, 0, s>>>(a);
  } else {
    if (small) rope_kernel<TQ_F32, uint32_t><<<grid, 256, 0, s>>>(a);
    else rope_kernel<TQ_F32, int64_t><<<grid, 256, 0, s>>>(a);
  }
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
}
