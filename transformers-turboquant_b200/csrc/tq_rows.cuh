// Row-chunk loads and stores shared by the tensor-core kernels: 8 input elements of any supported
// dtype as one 16-byte bf16 chunk, and 32 fp32 accumulator values as 32 output elements of any dtype.
#pragma once
#include "tq_common.cuh"
#include "tq_tcgen05.cuh"

namespace tq {

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

}  // namespace tq
