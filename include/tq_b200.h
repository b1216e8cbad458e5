/*
 * tq_b200.h -- C ABI of the B200 (sm_100a) TurboQuant KV-compression and
 * compressed-attention library (libtq_b200.so).
 *
 * Everything here takes plain pointers and sizes.  All data pointers of a call are DEVICE
 * pointers on ONE CUDA device unless a parameter says "host"; that device need not be the
 * thread's current one: an entry point finds the owner of its first data pointer, makes it
 * current for the duration of the call and restores the previous device (`stream` must
 * belong to the same device).  `stream` is a cudaStream_t passed as void* (NULL = the legacy
 * default stream).  Every
 * entry point validates its arguments on the host and returns a tq_status; on
 * anything but TQ_OK no kernel was launched and tq_last_error() describes the
 * problem.  No entry point allocates or frees device memory; scratch space is
 * supplied by the caller (see tq_attention_workspace_bytes).
 *
 * "Reference" citations are file:line in SrzStephen/transformers-turboquant, the
 * project whose interfaces these entry points replace.
 *
 * Wire format (shared by all entry points; reference
 * src/turboquant_pytorch/kernels/bit_ops.py:5-7 and compressors.py:132-138,
 * :281-285).  Vectors are numbered n = (batch*H + head)*S + position.
 *   packed indices : uint8 [N, ceil(d*b/8)], LSB-first bit stream per row: field i
 *                    occupies stream bits [i*b, i*b+b); stream bit g is bit g%8 of
 *                    byte g/8.  Keys use b = bits-1, values use b = bits.
 *   packed signs   : uint8 [N, d/8], one bit per sketch coordinate, 1 = (>= 0).
 *   norms          : IEEE fp16 bit patterns, uint16 [N].
 */
#ifndef TQ_B200_H
#define TQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  TQ_OK = 0,
  TQ_ERR_INVALID_ARG = 1,   /* bad size, unsupported bits/head_dim, NULL or misaligned pointer */
  TQ_ERR_CUDA = 2,          /* a CUDA runtime call failed; message holds cudaGetErrorString */
  TQ_ERR_UNSUPPORTED = 3,   /* valid request that this build does not implement */
  TQ_ERR_WORKSPACE = 4,     /* caller-supplied scratch buffer too small or misaligned */
  TQ_ERR_DEVICE_WAIT = 5    /* a bounded device-side wait gave up (see tq_device_fault_count) */
} tq_status;

typedef enum { TQ_F32 = 0, TQ_BF16 = 1, TQ_F16 = 2 } tq_dtype;

/* Arithmetic mode.  TQ_MODE_FP32: every contraction in fp32 on the CUDA cores, the
 * parity mode.  TQ_MODE_BF16: contractions on the tensor cores (tcgen05) from bf16
 * operands with fp32 accumulation, the throughput mode. */
typedef enum { TQ_MODE_FP32 = 0, TQ_MODE_BF16 = 1 } tq_mode;

/* Library version, major*10000 + minor*100 + patch. */
int tq_version(void);

/* Message of the last failing call made by this host thread ("" if none). */
const char* tq_last_error(void);

/* Number of bounded device-side waits that have expired on the current device since the library was
 * loaded (0 in a healthy process).  Reads a device counter; synchronises `stream`.
 *
 * Status contract: a kernel whose bounded wait expires unwinds cleanly and raises a flag in a page of host
 * memory (static storage of the library, pinned and mapped by the first call made on a device outside stream
 * capture; nothing is allocated).  From then on every launching entry point called for that device returns
 * TQ_ERR_DEVICE_WAIT without launching anything -- the check is one read of host memory, so it costs no
 * synchronisation and is legal during stream capture.  The call whose own kernel gave up has already returned
 * TQ_OK (launches are asynchronous); its output, and that of calls queued before the flag was seen, is invalid. */
int tq_device_fault_count(void* stream, int64_t* count_host);

/* Self-test of the expiry path of the bounded device-side waits (no counterpart in the reference).  Launches one
 * tiny CTA on the current device that waits, with the same bounded wait the attention and compression kernels
 * use, for an mbarrier nobody arrives on, with a limit of `limit_cycles` SM clocks (1e3 .. 2e9).  The wait gives
 * up, the kernel returns normally and reports the expiry to the host through the library's status page; the call
 * synchronises `stream` and then returns TQ_ERR_DEVICE_WAIT with a tq_last_error() text -- the same status every
 * launching entry point returns once a production kernel has given up a wait.  The self-test uses a flag of its
 * own: tq_device_fault_count stays 0 and later calls are not refused.  `waited_cycles_host` (optional) receives
 * the SM clocks the wait lasted.  TQ_ERR_UNSUPPORTED when the status page could not be pinned. */
int tq_selftest_wait_expiry(void* stream, int64_t limit_cycles, int64_t* waited_cycles_host);

/* Per-kernel device timing for benchmarks (no counterpart in the reference).  Between
 * tq_profile_begin and tq_profile_end every launch of the kernel kinds below is bracketed
 * by CUDA events on its own stream (up to max_records launches per kind, nothing is
 * synchronised while recording).  tq_profile_end waits for the recorded events and writes,
 * per kind, the summed milliseconds and the number of launches into two host arrays of
 * TQ_PROF_KINDS entries.  Process-wide, not thread-safe. */
enum {
  TQ_PROF_COMPRESS_KEYS = 0,
  TQ_PROF_COMPRESS_VALUES = 1,
  TQ_PROF_PREPARE_QUERIES = 2,
  TQ_PROF_ATTENTION = 3,
  TQ_PROF_BACK_ROTATION = 4,
  TQ_PROF_KINDS = 5
};
int tq_profile_begin(int max_records);
int tq_profile_end(float* ms_sum_host, int* launches_host);

/* Pipeline trace of the tensor-core attention kernel (diagnostics; no counterpart in the
 * reference).  While enabled, the CTA that handles the last query tile of (batch 0, head 0)
 * appends (tag, SM clock) pairs at each stage boundary of its softmax, producer and MMA
 * roles: tag = role << 32 | event << 16 | key tile.  tq_trace_read synchronises the device
 * and copies the first max_records slots of the 4096-slot buffer (2 int64 each; each role owns
 * one third of the slots, unused slots carry tag -1) to the host. */
/* The tracing instantiations are compiled only by `build.py --trace`; in the default build tq_trace_enable(1)
 * returns TQ_ERR_UNSUPPORTED. */
int tq_trace_enable(int on);
int tq_trace_read(int64_t* records_host, int max_records, int* n_host);

/* ---- wire-format primitives (test hooks and standalone operators) ------------- */

/* int32 [n, d] -> packed [n, ceil(d*b/8)], 1 <= b <= 8, d*b a multiple of 8.
 * Replaces pack_bits (src/turboquant_pytorch/kernels/bit_ops.py:173-199, :243-286). */
int tq_pack_bits(const int32_t* indices, int64_t n, int d, int b, uint8_t* packed, void* stream);

/* Inverse of tq_pack_bits.  Replaces unpack_bits (kernels/bit_ops.py:201-235, :288-326). */
int tq_unpack_bits(const uint8_t* packed, int64_t n, int d, int b, int32_t* indices, void* stream);

/* fp32 rotated coordinates [n, d] -> packed Lloyd-Max indices.  index = number of
 * boundaries strictly below the coordinate (first-minimum argmin, lower neighbour
 * on an exact tie).  `boundaries` holds 2^b_eff - 1 ascending fp32 values.
 * Replaces lloyd_max_quantize (kernels/quantize.py:201-247, :299-339) and the argmin
 * of compressors.py:141-142, :288-289. */
int tq_quantize_rotated(const float* rotated, int64_t n, int d, const float* boundaries, int b_eff,
                        uint8_t* packed, void* stream);

/* packed indices -> fp32 centroid values [n, d].  `centroids` holds 2^b fp32 values.
 * Replaces lloyd_max_dequantize (kernels/quantize.py:249-290, :341-369). */
int tq_dequantize(const uint8_t* packed, int64_t n, int d, const float* centroids, int b,
                  float* out, void* stream);

/* ---- per-compressor constants, prepared once ------------------------------------------- */

/* Everything a launch needs that depends only on a (key compressor, value compressor) pair -- the fp32 matrices
 * and codebooks and the operand images the tensor-core kernels copy into shared memory -- in one device buffer of
 * tq_constants_bytes(d, bits) bytes (256-byte aligned, owned by the caller), filled once per layer by
 * tq_prepare_constants.  The *_prepared / tq_compress_kv entry points read it and rebuild nothing, so a call is
 * its own kernels only.  Arguments as for tq_compress_keys / tq_compress_values / tq_attention_fwd:
 *   Pi_k, S_eff [d, d], centroids_k [2^(bits-1)], boundaries_k [2^(bits-1) - 1]   (key side)
 *   Pi_v [d, d], centroids_v [2^bits], boundaries_v [2^bits - 1]                  (value side)
 * Replaces the constants the reference's compressors hold as attributes and re-read in every call
 * (compressors.py:42-70, :230-246) and the per-call table builds of kernels/attention.py:300-330. */
size_t tq_constants_bytes(int d, int bits);
int tq_prepare_constants(const float* Pi_k, const float* S_eff, const float* centroids_k,
                         const float* boundaries_k, const float* Pi_v, const float* centroids_v,
                         const float* boundaries_v, int bits, int d, void* constants, size_t constants_bytes,
                         void* stream);

/* ---- rotary position embedding (the adapters' step before compression) ---------------- */

/* q_out = q * cos + rotate_half(q) * sin and the same for k, both in ONE launch: every element read once and
 * written once.  q: [B, Hq, S, d], k: [B, Hkv, S, d] of `dtype` with their own element strides (the transposed
 * view of a projection output is fine); cos, sin: [B or 1, S, d] of the same dtype, rows contiguous, element
 * strides cs_stride_b (0 for a broadcast batch) and cs_stride_s; q_out, k_out: contiguous [B, H, S, d], must not
 * alias the inputs.  rotate_half(x) = concat(-x[d/2:], x[:d/2]).  Each product and the sum are rounded to `dtype`
 * separately, which is what the separate torch kernels do: the result equals HF's to the bit.  All pointers
 * 16-byte aligned, strides multiples of 16 bytes, d a multiple of 32.  Either side may have zero heads.
 * Replaces apply_rotary_pos_emb as the family adapters call it (src/transformers_turboquant/families/llama.py:98,
 * qwen2.py:98). */
int tq_rope(const void* q, const void* k, int dtype, int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int d,
            int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
            int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
            const void* cos, const void* sin, int64_t cs_stride_b, int64_t cs_stride_s,
            void* q_out, void* k_out, void* stream);

/* ---- compression ---------------------------------------------------------------- */

/* Keys and values of one layer in ONE launch: tq_compress_keys(keys) and tq_compress_values(values) with the
 * constants taken from a prepared buffer.  keys, values: [B, H, S, d] of `dtype` with their own element strides;
 * either may be NULL, which skips that side.  Vector (b, h, s) goes to row (b*H + h)*kv_capacity + kv_offset + s
 * of every output array (kv_capacity = S, kv_offset = 0: the contiguous layout of the separate calls).
 * bf16 inputs of head_dim 128 in TQ_MODE_BF16 take the fused kernel (TMA-staged tiles, rotation and sketch on
 * tcgen05); anything else runs the per-side kernels, same bytes.
 * Replaces TurboQuantCompressorV2.compress + TurboQuantCompressorMSE.compress as the family adapters call them
 * back to back (src/transformers_turboquant/families/llama.py:103-104; compressors.py:98-161, :270-294). */
int tq_compress_kv(const void* keys, const void* values, int dtype, int64_t B, int64_t H, int64_t S, int d,
                   int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                   int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_s,
                   const void* constants, int bits,
                   uint8_t* key_idx, uint8_t* key_signs, uint16_t* key_vec_norms, uint16_t* key_residual_norms,
                   uint8_t* val_idx, uint16_t* val_vec_norms,
                   int64_t kv_capacity, int64_t kv_offset, int mode, void* stream);

/* Key compression: norm, normalise, rotate by Pi^T, Lloyd-Max index with bits-1 bits,
 * residual, its norm, and the sign of its QJL sketch, for every vector of
 * keys[B, H, S, d].  Strides are in elements; the innermost dimension is contiguous
 * and every row starts on a 16-byte boundary.
 *   Pi         fp32 [d, d]  rotation (rotated = x @ Pi^T)
 *   S_eff      fp32 [d, d]  sketch matrix in rotated coordinates, S @ Pi^T
 *   centroids  fp32 [2^(bits-1)], boundaries fp32 [2^(bits-1) - 1]
 * Outputs: packed_idx [N, d*(bits-1)/8], packed_signs [N, d/8], vec_norms [N],
 * residual_norms [N] (fp16 bit patterns), N = B*H*S.
 * Replaces TurboQuantCompressorV2.compress (compressors.py:98-161) with the packed
 * result layout of compressors.py:132-138. */
int tq_compress_keys(const void* keys, int dtype, int64_t B, int64_t H, int64_t S, int d,
                     int64_t stride_b, int64_t stride_h, int64_t stride_s,
                     const float* Pi, const float* S_eff, const float* centroids,
                     const float* boundaries, int bits,
                     uint8_t* packed_idx, uint8_t* packed_signs, uint16_t* vec_norms,
                     uint16_t* residual_norms, int mode, void* stream);

/* Value compression: norm, normalise, rotate, Lloyd-Max index with `bits` bits.
 * Replaces TurboQuantCompressorMSE.compress (compressors.py:270-294), packed layout
 * of compressors.py:281-285. */
int tq_compress_values(const void* values, int dtype, int64_t B, int64_t H, int64_t S, int d,
                       int64_t stride_b, int64_t stride_h, int64_t stride_s,
                       const float* Pi, const float* boundaries, int bits,
                       uint8_t* packed_idx, uint16_t* vec_norms, int mode, void* stream);

/* Packed values -> fp32 [N, d]: centroid lookup, back-rotation by Pi, times the norm.
 * Replaces TurboQuantCompressorMSE.decompress (compressors.py:296-317). */
int tq_decompress_values(const uint8_t* packed_idx, const uint16_t* vec_norms, int64_t n, int d,
                         const float* Pi, const float* centroids, int bits, float* out,
                         void* stream);

/* ---- attention -------------------------------------------------------------------- */

/* Unscaled, unmasked estimator scores, fp32 [B, Hq, Sq, Sk]:
 *   score = n_k <q Pi^T, C[idx_k]> + sqrt(pi/2)/d * rn_k <q Pi^T S_eff^T, +-1_k>.
 * Query head h reads key head h / (Hq/Hkv).  Materialises the full matrix: meant for
 * parity checks and small shapes.  `workspace` must hold tq_attention_workspace_bytes.
 * Replaces TurboQuantCompressorV2.asymmetric_attention_scores (compressors.py:163-224)
 * and kernels/attention.py:274-372. */
int tq_attention_scores(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d,
                        int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                        int64_t Hkv, int64_t Sk,
                        const uint8_t* key_idx, const uint8_t* key_signs,
                        const uint16_t* key_vec_norms, const uint16_t* key_residual_norms,
                        const float* Pi_k, const float* S_eff, const float* centroids_k, int bits,
                        float* scores, void* workspace, size_t workspace_bytes, int mode,
                        void* stream);

/* Query preparation, the per-query half of the estimator: q_cat[n, 0:d] = q Pi^T and
 * q_cat[n, d:2d] = sqrt(pi/2)/d * q S^T (S = S_eff Pi), row n = (b*Hq + h)*Sq + s.
 * q_cat is fp32 [N, 2d] in TQ_MODE_FP32 and bf16 [N, 2d] in TQ_MODE_BF16, where
 * `workspace` must hold 4*d*d bytes (256-byte aligned; unused in fp32 mode).
 * Replaces the q_rot / S_eff projections of compressors.py:186-189 and the per-query
 * projection loop of kernels/attention.py:158-167. */
int tq_prepare_queries(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d,
                       int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                       const float* Pi_k, const float* S_eff, void* q_cat,
                       void* workspace, size_t workspace_bytes, int mode, void* stream);

/* Scratch bytes tq_attention_scores / tq_attention_fwd need for the given problem. */
size_t tq_attention_workspace_bytes(int64_t B, int64_t Hq, int64_t Sq, int d, int mode);

/* Decode-sized calls (query rows per KV head (Hq/Hkv)*Sq <= 16, Sk >= 256, d = 128, TQ_MODE_BF16)
 * are served by a split-KV kernel that streams the packed bytes once; same arguments, same result.
 * The reference has no counterpart: it disables the KV cache (patch.py:80-81). */
/* Fused compressed attention: out = softmax(scores*sm_scale + mask) @ V_hat, computed
 * from packed keys and values without materialising scores or decompressed K/V.
 *   causal != 0 : query i (aligned to the end of the keys) sees keys <= i + Sk - Sq.
 *   mask        : optional additive fp32 mask, element (b, i, k) at
 *                 mask[b*mask_stride_b + i*mask_stride_q + k]; NULL for none.
 *   out         : [B, Hq, Sq, d] of `dtype` with the given element strides.
 * Replaces the attention core of the family adapters
 * (src/transformers_turboquant/families/llama.py:100-114, gpt2.py:90-110). */
int tq_attention_fwd(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d,
                     int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                     int64_t Hkv, int64_t Sk,
                     const uint8_t* key_idx, const uint8_t* key_signs,
                     const uint16_t* key_vec_norms, const uint16_t* key_residual_norms,
                     const uint8_t* val_idx, const uint16_t* val_vec_norms,
                     const float* Pi_k, const float* S_eff, const float* centroids_k,
                     const float* Pi_v, const float* centroids_v, int bits,
                     float sm_scale, int causal,
                     const float* mask, int64_t mask_stride_b, int64_t mask_stride_q,
                     void* out, int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s,
                     void* workspace, size_t workspace_bytes, int mode, void* stream);

/* tq_attention_fwd / tq_attention_fwd_cached with the constants taken from a prepared buffer: no operand is
 * rebuilt per call, and the scratch need drops to tq_attention_prepared_workspace_bytes -- zero for prefill-sized
 * calls in TQ_MODE_BF16 (`workspace` may then be NULL).  kv_capacity = Sk is the contiguous
 * layout; a larger capacity is the persistent-cache layout of tq_attention_fwd_cached (same shape limits).
 * Replaces the attention core of the family adapters (families/llama.py:100-114, gpt2.py:90-110). */
size_t tq_attention_prepared_workspace_bytes(int64_t B, int64_t Hq, int64_t Sq, int64_t Hkv, int64_t Sk,
                                             int64_t kv_capacity, int d, int mode);
int tq_attention_fwd_prepared(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d,
                              int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                              int64_t Hkv, int64_t Sk, int64_t kv_capacity,
                              const uint8_t* key_idx, const uint8_t* key_signs,
                              const uint16_t* key_vec_norms, const uint16_t* key_residual_norms,
                              const uint8_t* val_idx, const uint16_t* val_vec_norms,
                              const void* constants, int bits, float sm_scale, int causal,
                              const float* mask, int64_t mask_stride_b, int64_t mask_stride_q,
                              void* out, int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s,
                              void* workspace, size_t workspace_bytes, int mode, void* stream);

/* tq_attention_fwd for callers that cannot hand over scratch memory (no counterpart in the
 * reference).  Meant for hosts that may not call cudaMalloc or any other allocator: a plugin
 * inside a serving process whose device memory belongs to someone else, or a call site that
 * only holds borrowed input and output buffers.  Same arguments and results as tq_attention_fwd
 * minus `workspace`: the scratch is a fixed tq_static_scratch_bytes() (32 MiB) array compiled
 * into the library, resident on every GPU that loads it until the process exits.
 *   - A problem whose tq_attention_workspace_bytes exceeds that size is rejected with
 *     TQ_ERR_WORKSPACE and nothing is launched (at d=128 the array covers about 43 000 query
 *     rows B*Hq*Sq in bf16 mode, 32 000 in fp32 mode).
 *   - The first call on each device looks up the array's device address (one runtime query) and,
 *     like the first call of any entry point on a device, installs the library's status page
 *     (pinning 4 KB of the library's own static storage, a few small synchronous copies); neither
 *     allocates.  Make that first call outside any stream capture.  No call allocates or frees
 *     device memory.
 *   - All calls on a device share the one array.  Every byte a call reads from it was written
 *     earlier in the same call, so stale contents are harmless and nothing has to be cleared;
 *     but two calls that overlap on the GPU (different streams, or threads) race on it.
 *     Serialise them. */
size_t tq_static_scratch_bytes(void);
int tq_attention_fwd_static(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d,
                            int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                            int64_t Hkv, int64_t Sk,
                            const uint8_t* key_idx, const uint8_t* key_signs,
                            const uint16_t* key_vec_norms, const uint16_t* key_residual_norms,
                            const uint8_t* val_idx, const uint16_t* val_vec_norms,
                            const float* Pi_k, const float* S_eff, const float* centroids_k,
                            const float* Pi_v, const float* centroids_v, int bits,
                            float sm_scale, int causal,
                            const float* mask, int64_t mask_stride_b, int64_t mask_stride_q,
                            void* out, int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s,
                            int mode, void* stream);

/* tq_attention_fwd against a persistent packed KV cache (no counterpart in the reference, which
 * disables the cache and recompresses the whole prefix for every generated token: patch.py:80-81;
 * the concept is turboquant.py:199-286).  Every packed array has room for `kv_capacity` keys per
 * (batch, KV head) -- key k of pair (b, h) is row (b*Hkv + h)*kv_capacity + k -- of which the
 * first Sk are in use; new tokens are compressed by tq_compress_keys / tq_compress_values and
 * copied behind them.  Served by the split-KV kernel: head_dim 128, (Hq/Hkv)*Sq <= 16 query rows
 * per KV head, TQ_MODE_BF16, any Sk >= 1 (mask as in tq_attention_fwd); other shapes return
 * TQ_ERR_INVALID_ARG.
 * Workspace as for tq_attention_fwd in TQ_MODE_BF16. */
int tq_attention_fwd_cached(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d,
                            int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                            int64_t Hkv, int64_t Sk, int64_t kv_capacity,
                            const uint8_t* key_idx, const uint8_t* key_signs,
                            const uint16_t* key_vec_norms, const uint16_t* key_residual_norms,
                            const uint8_t* val_idx, const uint16_t* val_vec_norms,
                            const float* Pi_k, const float* S_eff, const float* centroids_k,
                            const float* Pi_v, const float* centroids_v, int bits,
                            float sm_scale, int causal,
                            const float* mask, int64_t mask_stride_b, int64_t mask_stride_q,
                            void* out, int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s,
                            void* workspace, size_t workspace_bytes, void* stream);

/* tq_compress_keys / tq_compress_values writing straight into a persistent cache (see
 * tq_attention_fwd_cached): input vector (b, h, s) goes to row (b*H + h)*kv_capacity + kv_offset + s
 * of every output array, i.e. behind the kv_offset tokens already stored.  Same arithmetic and the
 * same bytes as the contiguous calls; kv_offset + S must not exceed kv_capacity. */
int tq_append_keys(const void* keys, int dtype, int64_t B, int64_t H, int64_t S, int d,
                   int64_t stride_b, int64_t stride_h, int64_t stride_s,
                   const float* Pi, const float* S_eff, const float* centroids,
                   const float* boundaries, int bits,
                   uint8_t* packed_idx, uint8_t* packed_signs,
                   uint16_t* vec_norms, uint16_t* residual_norms,
                   int64_t kv_capacity, int64_t kv_offset, int mode, void* stream);
int tq_append_values(const void* values, int dtype, int64_t B, int64_t H, int64_t S, int d,
                     int64_t stride_b, int64_t stride_h, int64_t stride_s,
                     const float* Pi, const float* boundaries, int bits,
                     uint8_t* packed_idx, uint16_t* vec_norms,
                     int64_t kv_capacity, int64_t kv_offset, int mode, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TQ_B200_H */
