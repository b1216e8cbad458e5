// Shared host/device helpers for libtq_b200: status + error text, argument checks,
// element loads, fp16 norm encoding and the LSB-first bit-stream packing rule.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "tq_b200.h"

namespace tq {

// ---- host: thread-local error text --------------------------------------------------
void set_error(const char* fmt, ...);
int fail(tq_status st, const char* fmt, ...);

#define TQ_REQUIRE(cond, ...)                                   \
  do {                                                          \
    if (!(cond)) return ::tq::fail(TQ_ERR_INVALID_ARG, __VA_ARGS__); \
  } while (0)

#define TQ_CUDA_OK(expr)                                                              \
  do {                                                                                \
    cudaError_t _e = (expr);                                                          \
    if (_e != cudaSuccess)                                                            \
      return ::tq::fail(TQ_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool valid_head_dim(int d) { return d == 64 || d == 128; }
inline bool valid_bits(int bits) { return bits >= 2 && bits <= 4; }
inline int elem_size(int dtype) { return dtype == TQ_F32 ? 4 : 2; }

// ---- host: which device a call runs on, and what earlier launches reported ----------------
//
// An entry point runs on the device that owns its first data pointer, whatever the thread's current device is:
// CallScope looks the owner up (cudaPointerGetAttributes), makes it current for the duration of the call and
// restores the previous device on the way out.  A pointer that is not device (or managed) memory is refused.
//
// It is also where a call learns that an EARLIER launch on that device gave up a bounded wait: the kernels raise a
// flag in a page of host memory that the library pins and maps once per process (static storage, 4 KB, no
// allocation), so the check is one read of host memory -- no synchronisation, legal during stream capture.  The
// page is installed on a device by the first call made there outside stream capture; until then, and if pinning
// is refused, only tq_device_fault_count() (which reads the device counters) reports expired waits.
class CallScope {
 public:
  CallScope(const void* data_ptr, const char* what, cudaStream_t stream);
  ~CallScope();
  CallScope(const CallScope&) = delete;
  CallScope& operator=(const CallScope&) = delete;
  int status() const { return status_; }  // TQ_OK, or the status the entry point must return at once
  int device() const { return device_; }

 private:
  int status_ = TQ_OK, device_ = -1, previous_ = -1;
};
constexpr int kMaxDevices = 64;
// installed by CallScope, one per translation unit that has bounded waits
int set_fault_mailbox_c2(unsigned long long* slot);
int set_fault_mailbox_tc(unsigned long long* slot);
int set_fault_mailbox_compress(unsigned long long* slot);
int set_fault_mailbox_compress_kv(unsigned long long* slot);
int set_fault_mailbox_selftest(unsigned long long* slot);

// Device side of the mailbox: `slot` is the translation unit's copy of the pointer (NULL until installed).
__device__ __forceinline__ void notify_host_of_fault(unsigned long long* slot) {
  if (slot != nullptr) {
    *reinterpret_cast<volatile unsigned long long*>(slot) = 1ull;
    __threadfence_system();
  }
}

// Copies the device counter of expired bounded waits (kept by the tensor-core
// translation unit) to the host.
int read_wait_faults(unsigned long long* out);
int read_compress_faults(unsigned long long* out);
int read_compress_kv_faults(unsigned long long* out);
int trace_enable(int on);
int trace_read(long long* host_buf, int max_records, int* n_out);

// ---- optional per-kernel timing (tq_profile_begin / tq_profile_end) ------------------
enum ProfKind { kProfCompressKeys = 0, kProfCompressValues = 1, kProfPrepareQueries = 2, kProfAttention = 3,
                kProfBackRotation = 4, kProfKinds = 5 };
// Record a CUDA event on `stream` before / after a kernel launch when profiling is on.
void prof_mark(int kind, bool is_end, cudaStream_t stream);
struct ProfScope {
  int kind;
  cudaStream_t stream;
  ProfScope(int k, cudaStream_t s) : kind(k), stream(s) { prof_mark(kind, false, stream); }
  ~ProfScope() { prof_mark(kind, true, stream); }
};

// ---- device helpers -------------------------------------------------------------------

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

// Load 8 consecutive elements (16-byte aligned for 2-byte types, 32 for fp32) as floats.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&out)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&out)[8]) {
  float4 a = reinterpret_cast<const float4*>(p)[0];
  float4 b = reinterpret_cast<const float4*>(p)[1];
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
  out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&out)[8]) {
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&out)[8]) {
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __half22float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ uint16_t fp16_bits(float v) { return __half_as_ushort(__float2half_rn(v)); }
__device__ __forceinline__ float fp16_value(uint16_t b) { return __half2float(__ushort_as_half(b)); }

// Number of ascending boundaries strictly below y: the Lloyd-Max index.
template <int NB>
__device__ __forceinline__ int count_below(float y, const float (&bnd)[NB]) {
  int idx = 0;
#pragma unroll
  for (int j = 0; j < NB; ++j) idx += (y > bnd[j]) ? 1 : 0;
  return idx;
}

// Pack 8 consecutive b-bit fields into the b bytes they occupy in the row's bit stream
// (field i at stream bits [i*b, i*b+b), LSB first) and store them at `dst`.
template <int BITS>
__device__ __forceinline__ void store_fields8(uint8_t* dst, const int (&f)[8]) {
  uint64_t word = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) word |= static_cast<uint64_t>(f[i] & ((1 << BITS) - 1)) << (i * BITS);
#pragma unroll
  for (int j = 0; j < BITS; ++j) dst[j] = static_cast<uint8_t>(word >> (8 * j));
}

// Extract field `i` (0..7) from the b bytes holding 8 consecutive fields.
template <int BITS>
__device__ __forceinline__ uint64_t load_fields8(const uint8_t* src) {
  uint64_t word = 0;
#pragma unroll
  for (int j = 0; j < BITS; ++j) word |= static_cast<uint64_t>(src[j]) << (8 * j);
  return word;
}

}  // namespace tq
