// Error plumbing, version, and the wire-format primitives: pack, unpack, Lloyd-Max
// quantise of rotated coordinates, centroid dequantise.  These are HBM-bound byte
// kernels; each thread owns 8 consecutive fields, i.e. exactly b whole bytes of the
// row's bit stream, so no atomics or pre-zeroed outputs are needed.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "tq_common.cuh"
#include "tq_attention.cuh"
#include "tq_tcgen05.cuh"

namespace tq {

static thread_local char t_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
}

int fail(tq_status st, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
  return st;
}

// ---- device selection and the host-visible status page -------------------------------------
namespace {
// One page of the library's own static storage, pinned and mapped into the devices' address space at first use.
// Slot d: an expired bounded wait on device d.  Slot kMaxDevices + d: the self-test's flag on device d.
struct alignas(4096) StatusPage {
  volatile unsigned long long slot[4096 / sizeof(unsigned long long)];
};
StatusPage g_status_page;
std::mutex g_setup_mutex;
int g_page_state = 0;                    // 0 = not tried yet, 1 = pinned and mapped, -1 = pinning was refused
bool g_device_ready[kMaxDevices] = {};   // mailbox pointers installed on this device
bool g_sticky_fault[kMaxDevices] = {};   // tq_device_fault_count has seen a non-zero device counter

__device__ unsigned long long* g_mailbox_selftest = nullptr;

// The first call on a device outside stream capture installs the mailbox pointers (four small synchronous
// copies to device symbols).  Nothing is allocated: the page is static storage, cudaHostRegister only pins it.
void install_status_page(int dev, cudaStream_t stream) {
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_device_ready[dev] || g_page_state < 0) return;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return;  // not now: synchronous set-up is illegal inside a capture; a later call installs it
  }
  if (g_page_state == 0) {
    const cudaError_t e = cudaHostRegister(&g_status_page, sizeof(g_status_page),
                                           cudaHostRegisterMapped | cudaHostRegisterPortable);
    if (e != cudaSuccess) {
      cudaGetLastError();
      g_page_state = -1;
      return;
    }
    g_page_state = 1;
  }
  void* dptr = nullptr;
  if (cudaHostGetDevicePointer(&dptr, const_cast<unsigned long long*>(&g_status_page.slot[0]), 0) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  unsigned long long* base = static_cast<unsigned long long*>(dptr);
  unsigned long long* self = base + kMaxDevices + dev;
  if (set_fault_mailbox_c2(base + dev) || set_fault_mailbox_tc(base + dev) || set_fault_mailbox_compress(base + dev) || set_fault_mailbox_compress_kv(base + dev) ||
      cudaMemcpyToSymbol(g_mailbox_selftest, &self, sizeof(self)) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  g_device_ready[dev] = true;
}
}  // namespace

CallScope::CallScope(const void* data_ptr, const char* what, cudaStream_t stream) {
  cudaPointerAttributes attr;
  cudaError_t e = cudaPointerGetAttributes(&attr, data_ptr);
  if (e != cudaSuccess) {
    cudaGetLastError();
    status_ = fail(TQ_ERR_CUDA, "cudaPointerGetAttributes(%s) failed: %s", what, cudaGetErrorString(e));
    return;
  }
  if (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged) {
    status_ = fail(TQ_ERR_INVALID_ARG, "%s is not a device pointer (the library has no host path)", what);
    return;
  }
  device_ = attr.device;
  if (device_ < 0 || device_ >= kMaxDevices) {
    status_ = fail(TQ_ERR_INVALID_ARG, "device ordinal %d outside 0..%d", device_, kMaxDevices - 1);
    return;
  }
  int current = -1;
  if ((e = cudaGetDevice(&current)) != cudaSuccess) {
    status_ = fail(TQ_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(e));
    return;
  }
  if (current != device_) {
    if ((e = cudaSetDevice(device_)) != cudaSuccess) {
      status_ = fail(TQ_ERR_CUDA, "cudaSetDevice(%d) failed: %s", device_, cudaGetErrorString(e));
      return;
    }
    previous_ = current;
  }
  if (!g_device_ready[device_]) install_status_page(device_, stream);
  if (g_status_page.slot[device_] != 0ull || g_sticky_fault[device_])
    status_ = fail(TQ_ERR_DEVICE_WAIT,
                   "a bounded device-side wait expired in an earlier launch on device %d: results computed since "
                   "then are not valid and nothing further is launched (tq_device_fault_count reads the counter; "
                   "the condition lasts until the process exits)", device_);
}

CallScope::~CallScope() {
  if (previous_ >= 0) cudaSetDevice(previous_);
}

int set_fault_mailbox_selftest(unsigned long long* slot) {
  TQ_CUDA_OK(cudaMemcpyToSymbol(g_mailbox_selftest, &slot, sizeof(slot)));
  return TQ_OK;
}

// Self-test of the expiry path (tq_selftest_wait_expiry): one CTA initialises an mbarrier that nobody arrives on
// and waits for it with the bounded wait the production kernels use, with a short limit.  The wait gives up,
// raises the CTA's abort flag, and thread 0 reports through the mailbox -- into the self-test's own slot, not
// the one that poisons later calls.  Nothing traps, faults or spins without bound.
__global__ void selftest_wait_kernel(long long limit_cycles, long long* waited_cycles) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    s_abort = 0;
    tc::mbar_init(tc::smem_u32(&bar), 1);
    tc::fence_mbar_init();
  }
  __syncthreads();
  const long long t0 = clock64();
  const bool ok = tc::mbar_wait_or_abort(tc::smem_u32(&bar), 0, &s_abort, limit_cycles);
  __syncthreads();
  if (threadIdx.x == 0) {
    *waited_cycles = clock64() - t0;
    if (!ok && s_abort) notify_host_of_fault(g_mailbox_selftest);
  }
}

// ---- per-kernel timing ------------------------------------------------------------------
namespace {
struct ProfState {
  bool on = false;
  int cap = 0;
  int used[kProfKinds] = {0, 0, 0, 0, 0};
  cudaEvent_t* ev[kProfKinds] = {nullptr, nullptr, nullptr, nullptr, nullptr};  // 2*cap each: begin,end pairs
};
ProfState g_prof;
}  // namespace

void prof_mark(int kind, bool is_end, cudaStream_t stream) {
  if (!g_prof.on) return;
  int& n = g_prof.used[kind];
  if (n >= g_prof.cap) return;
  cudaEventRecord(g_prof.ev[kind][2 * n + (is_end ? 1 : 0)], stream);
  if (is_end) ++n;
}

// ---- kernels ----------------------------------------------------------------------------

// One thread per group of 8 fields.  groups_per_row = d/8.
template <int BITS>
__global__ void pack_kernel(const int32_t* __restrict__ idx, int64_t n_groups, int groups_per_row,
                            uint8_t* __restrict__ out) {
  int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (g >= n_groups) return;
  const int4* src = reinterpret_cast<const int4*>(idx + g * 8);
  int4 a = src[0], b = src[1];
  int f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  store_fields8<BITS>(out + g * BITS, f);
}

template <int BITS>
__global__ void unpack_kernel(const uint8_t* __restrict__ packed, int64_t n_groups,
                              int32_t* __restrict__ idx) {
  int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (g >= n_groups) return;
  uint64_t w = load_fields8<BITS>(packed + g * BITS);
  int f[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = static_cast<int>((w >> (i * BITS)) & ((1u << BITS) - 1));
  int4* dst = reinterpret_cast<int4*>(idx + g * 8);
  dst[0] = make_int4(f[0], f[1], f[2], f[3]);
  dst[1] = make_int4(f[4], f[5], f[6], f[7]);
}

template <int BITS>
__global__ void quantize_kernel(const float* __restrict__ rotated, int64_t n_groups,
                                const float* __restrict__ boundaries, uint8_t* __restrict__ out) {
  constexpr int NB = (1 << BITS) - 1;
  float bnd[NB];
#pragma unroll
  for (int j = 0; j < NB; ++j) bnd[j] = __ldg(boundaries + j);
  int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (g >= n_groups) return;
  float y[8];
  load8<float>(rotated + g * 8, y);
  int f[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = count_below<NB>(y[i], bnd);
  store_fields8<BITS>(out + g * BITS, f);
}

template <int BITS>
__global__ void dequantize_kernel(const uint8_t* __restrict__ packed, int64_t n_groups,
                                  const float* __restrict__ centroids, float* __restrict__ out) {
  __shared__ float lut[1 << BITS];
  if (threadIdx.x < (1 << BITS)) lut[threadIdx.x] = centroids[threadIdx.x];
  __syncthreads();
  int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (g >= n_groups) return;
  uint64_t w = load_fields8<BITS>(packed + g * BITS);
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = lut[(w >> (i * BITS)) & ((1u << BITS) - 1)];
  float4* dst = reinterpret_cast<float4*>(out + g * 8);
  dst[0] = make_float4(v[0], v[1], v[2], v[3]);
  dst[1] = make_float4(v[4], v[5], v[6], v[7]);
}

template <template <int> class Launcher, typename... Args>
static int dispatch_bits(int b, Args... args) {
  switch (b) {
    case 1: return Launcher<1>::run(args...);
    case 2: return Launcher<2>::run(args...);
    case 3: return Launcher<3>::run(args...);
    case 4: return Launcher<4>::run(args...);
    case 5: return Launcher<5>::run(args...);
    case 6: return Launcher<6>::run(args...);
    case 7: return Launcher<7>::run(args...);
    case 8: return Launcher<8>::run(args...);
  }
  return fail(TQ_ERR_INVALID_ARG, "bit width %d outside 1..8", b);
}

static inline unsigned grid_for(int64_t n_groups) { return static_cast<unsigned>((n_groups + 255) / 256); }

template <int BITS>
struct PackL {
  static int run(const int32_t* idx, int64_t ng, int gpr, uint8_t* out, cudaStream_t s) {
    pack_kernel<BITS><<<grid_for(ng), 256, 0, s>>>(idx, ng, gpr, out);
    return TQ_OK;
  }
};
template <int BITS>
struct UnpackL {
  static int run(const uint8_t* p, int64_t ng, int32_t* idx, cudaStream_t s) {
    unpack_kernel<BITS><<<grid_for(ng), 256, 0, s>>>(p, ng, idx);
    return TQ_OK;
  }
};
template <int BITS>
struct QuantL {
  static int run(const float* r, int64_t ng, const float* b, uint8_t* out, cudaStream_t s) {
    quantize_kernel<BITS><<<grid_for(ng), 256, 0, s>>>(r, ng, b, out);
    return TQ_OK;
  }
};
template <int BITS>
struct DequantL {
  static int run(const uint8_t* p, int64_t ng, const float* c, float* out, cudaStream_t s) {
    dequantize_kernel<BITS><<<grid_for(ng), 256, 0, s>>>(p, ng, c, out);
    return TQ_OK;
  }
};

static int check_rows(int64_t n, int d, int b, int bmax) {
  TQ_REQUIRE(n >= 0, "row count %lld is negative", (long long)n);
  TQ_REQUIRE(d > 0 && d % 8 == 0, "row length %d must be a positive multiple of 8", d);
  TQ_REQUIRE(b >= 1 && b <= bmax, "bit width %d outside 1..%d", b, bmax);
  TQ_REQUIRE(n * (int64_t)(d / 8) < (int64_t)1 << 39, "problem too large");
  return TQ_OK;
}

}  // namespace tq

using namespace tq;

extern "C" {

int tq_version(void) { return 100; }

const char* tq_last_error(void) { return t_error; }

int tq_device_fault_count(void* stream, int64_t* count_host) {
  TQ_REQUIRE(count_host != nullptr, "count_host is NULL");
  unsigned long long v = 0;
  TQ_CUDA_OK(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  unsigned long long w = 0;
  if (int st = read_wait_faults(&v)) return st;
  if (int st = read_compress_faults(&w)) return st;
  unsigned long long x = 0, y = 0;
  if (int st = read_c2_faults(&x)) return st;
  if (int st = read_compress_kv_faults(&y)) return st;
  x += y;
  *count_host = static_cast<int64_t>(v + w + x);
  int dev = -1;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices && v + w + x != 0) g_sticky_fault[dev] = true;
  return TQ_OK;
}

int tq_selftest_wait_expiry(void* stream, int64_t limit_cycles, int64_t* waited_cycles_host) {
  TQ_REQUIRE(limit_cycles >= 1000 && limit_cycles <= 2000000000ll, "limit_cycles %lld outside 1e3..2e9",
             (long long)limit_cycles);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int dev = -1;
  TQ_CUDA_OK(cudaGetDevice(&dev));
  TQ_REQUIRE(dev >= 0 && dev < kMaxDevices, "device ordinal %d outside 0..%d", dev, kMaxDevices - 1);
  if (!g_device_ready[dev]) install_status_page(dev, s);
  if (!g_device_ready[dev])
    return fail(TQ_ERR_UNSUPPORTED, "the host-visible status page could not be installed on device %d", dev);
  volatile unsigned long long* flag = &g_status_page.slot[kMaxDevices + dev];
  long long* waited = const_cast<long long*>(reinterpret_cast<volatile long long*>(&g_status_page.slot[2 * kMaxDevices + dev]));
  void* waited_dev = nullptr;
  TQ_CUDA_OK(cudaHostGetDevicePointer(&waited_dev, waited, 0));
  *flag = 0ull;
  *waited = 0;
  selftest_wait_kernel<<<1, 64, 0, s>>>((long long)limit_cycles, static_cast<long long*>(waited_dev));
  TQ_CUDA_OK(cudaGetLastError());
  TQ_CUDA_OK(cudaStreamSynchronize(s));
  if (waited_cycles_host != nullptr) *waited_cycles_host = *waited;
  if (*flag == 0ull) return TQ_OK;  // the wait did not expire (it cannot succeed either: nobody arrives)
  *flag = 0ull;
  return fail(TQ_ERR_DEVICE_WAIT, "self-test: a bounded device-side wait gave up after %lld cycles (limit %lld) and "
              "reported it to the host", (long long)*waited, (long long)limit_cycles);
}

static bool trace_sm_pairs() {
  const char* e = getenv("TQ_B200_ATTN");
  return !(e != nullptr && e[0] == 'w');
}

int tq_trace_enable(int on) {
#ifndef TQ_B200_TRACE
  if (on) return fail(TQ_ERR_UNSUPPORTED, "this build carries no tracing kernels: rebuild with `build.py --trace`");
#endif
  if (int st = trace_enable(on)) return st;
  return trace_enable_c2(on);
}

int tq_trace_read(int64_t* records_host, int max_records, int* n_host) {
  TQ_REQUIRE(records_host && n_host && max_records > 0, "bad trace buffer");
  if (trace_sm_pairs()) return trace_read_c2(reinterpret_cast<long long*>(records_host), max_records, n_host);
  return trace_read(reinterpret_cast<long long*>(records_host), max_records, n_host);
}

int tq_profile_begin(int max_records) {
  TQ_REQUIRE(max_records > 0 && max_records <= 4096, "max_records %d outside 1..4096", max_records);
  TQ_REQUIRE(!g_prof.on, "profiling already active");
  for (int k = 0; k < kProfKinds; ++k) {
    g_prof.ev[k] = new cudaEvent_t[2 * max_records];
    for (int i = 0; i < 2 * max_records; ++i) TQ_CUDA_OK(cudaEventCreate(&g_prof.ev[k][i]));
    g_prof.used[k] = 0;
  }
  g_prof.cap = max_records;
  g_prof.on = true;
  return TQ_OK;
}

int tq_profile_end(float* ms_sum, int* launches) {
  TQ_REQUIRE(g_prof.on, "profiling is not active");
  TQ_REQUIRE(ms_sum && launches, "NULL output pointer");
  g_prof.on = false;
  int rc = TQ_OK;
  for (int k = 0; k < kProfKinds; ++k) {
    ms_sum[k] = 0.f;
    launches[k] = g_prof.used[k];
    for (int i = 0; i < g_prof.used[k]; ++i) {
      float ms = 0.f;
      cudaError_t e = cudaEventSynchronize(g_prof.ev[k][2 * i + 1]);
      if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, g_prof.ev[k][2 * i], g_prof.ev[k][2 * i + 1]);
      if (e != cudaSuccess) rc = fail(TQ_ERR_CUDA, "event timing failed: %s", cudaGetErrorString(e));
      ms_sum[k] += ms;
    }
    for (int i = 0; i < 2 * g_prof.cap; ++i) cudaEventDestroy(g_prof.ev[k][i]);
    delete[] g_prof.ev[k];
    g_prof.ev[k] = nullptr;
  }
  return rc;
}

int tq_pack_bits(const int32_t* indices, int64_t n, int d, int b, uint8_t* packed, void* stream) {
  if (int st = check_rows(n, d, b, 8)) return st;
  if (n == 0) return TQ_OK;
  TQ_REQUIRE(indices && packed, "NULL pointer");
  TQ_REQUIRE(aligned16(indices), "indices must be 16-byte aligned");
  CallScope scope(indices, "indices", static_cast<cudaStream_t>(stream));
  if (scope.status()) return scope.status();
  int st = dispatch_bits<PackL>(b, indices, n * (d / 8), d / 8, packed, static_cast<cudaStream_t>(stream));
  if (st) return st;
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
}

int tq_unpack_bits(const uint8_t* packed, int64_t n, int d, int b, int32_t* indices, void* stream) {
  if (int st = check_rows(n, d, b, 8)) return st;
  if (n == 0) return TQ_OK;
  TQ_REQUIRE(indices && packed, "NULL pointer");
  TQ_REQUIRE(aligned16(indices), "indices must be 16-byte aligned");
  CallScope scope(packed, "packed", static_cast<cudaStream_t>(stream));
  if (scope.status()) return scope.status();
  int st = dispatch_bits<UnpackL>(b, packed, n * (d / 8), indices, static_cast<cudaStream_t>(stream));
  if (st) return st;
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
}

int tq_quantize_rotated(const float* rotated, int64_t n, int d, const float* boundaries, int b_eff,
                        uint8_t* packed, void* stream) {
  if (int st = check_rows(n, d, b_eff, 4)) return st;
  if (n == 0) return TQ_OK;
  TQ_REQUIRE(rotated && boundaries && packed, "NULL pointer");
  TQ_REQUIRE(aligned16(rotated), "rotated must be 16-byte aligned");
  CallScope scope(rotated, "rotated", static_cast<cudaStream_t>(stream));
  if (scope.status()) return scope.status();
  const int64_t ng = n * (d / 8);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (b_eff) {  // boundaries live in registers, so only the widths the codebooks use
    case 1: QuantL<1>::run(rotated, ng, boundaries, packed, s); break;
    case 2: QuantL<2>::run(rotated, ng, boundaries, packed, s); break;
    case 3: QuantL<3>::run(rotated, ng, boundaries, packed, s); break;
    default: QuantL<4>::run(rotated, ng, boundaries, packed, s); break;
  }
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
}

int tq_dequantize(const uint8_t* packed, int64_t n, int d, const float* centroids, int b, float* out,
                  void* stream) {
  if (int st = check_rows(n, d, b, 8)) return st;
  if (n == 0) return TQ_OK;
  TQ_REQUIRE(packed && centroids && out, "NULL pointer");
  TQ_REQUIRE(aligned16(out), "out must be 16-byte aligned");
  CallScope scope(packed, "packed", static_cast<cudaStream_t>(stream));
  if (scope.status()) return scope.status();
  int st = dispatch_bits<DequantL>(b, packed, n * (d / 8), centroids, out, static_cast<cudaStream_t>(stream));
  if (st) return st;
  TQ_CUDA_OK(cudaGetLastError());
  return TQ_OK;
}

}  // extern "C"
