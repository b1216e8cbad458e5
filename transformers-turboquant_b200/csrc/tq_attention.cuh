// Argument block and entry points shared by the fp32 (CUDA-core) and bf16 (tcgen05)
// implementations of the fused compressed attention.
#pragma once
#include <cuda_bf16.h>

#include "tq_common.cuh"

namespace tq {

// Layout of the per-compressor constants buffer that tq_prepare_constants fills once: byte offsets of its parts
// (each a multiple of 256) for head_dim d.  Everything a launch needs that depends only on the compressor pair:
// the fp32 matrices and codebooks themselves, and the operand images the tensor-core kernels bulk-copy into
// shared memory (so that no call rebuilds them).
struct ConstLayout {
  size_t header;                                                  // magic, d, bits
  size_t pi_k, s_eff, pi_v, cen_k, bnd_k, cen_v, bnd_v;           // fp32 originals
  size_t w_cat_pair, w_unrot_pair, luts, w_cat_plain, w_unrot_plain;  // attention: bf16 operand images, fp16 pair tables
  size_t pik_hi, pik_lo, se_hi, se_lo, piv_hi, piv_lo;            // compression: split-bf16 K-major operand images
  size_t total;
};
constexpr uint32_t kConstMagic = 0x31425154u;  // "TQB1"
inline ConstLayout const_layout(int d) {
  ConstLayout L{};
  size_t off = 0;
  auto take = [&](size_t bytes) { const size_t at = off; off += (bytes + 255) & ~(size_t)255; return at; };
  const size_t m32 = (size_t)d * d * 4, m16 = (size_t)d * d * 2;
  L.header = take(256);
  L.pi_k = take(m32); L.s_eff = take(m32); L.pi_v = take(m32);
  L.cen_k = take(64); L.bnd_k = take(64); L.cen_v = take(64); L.bnd_v = take(64);
  L.w_cat_pair = take(2 * m16); L.w_unrot_pair = take(m16); L.luts = take(2048);
  L.w_cat_plain = take(2 * m16); L.w_unrot_plain = take(m16);
  L.pik_hi = take(m16); L.pik_lo = take(m16); L.se_hi = take(m16); L.se_lo = take(m16);
  L.piv_hi = take(m16); L.piv_lo = take(m16);
  L.total = off;
  return L;
}
int prepare_constants(const float* Pi_k, const float* S_eff, const float* cen_k, const float* bnd_k, const float* Pi_v,
                      const float* cen_v, const float* bnd_v, int bits, int d, void* constants, cudaStream_t stream);

struct AttnArgs {
  const void* q_cat;   // fp32 [n, 2d] (fp32 mode) or bf16 [n, 2d] (bf16 mode), row n = (b*Hq+h)*Sq+s
  int64_t Hq, Sq, Hkv, Sk;
  const uint8_t* key_idx;
  const uint8_t* key_sgn;
  const uint16_t* key_vn;
  const uint16_t* key_rn;
  const uint8_t* val_idx;
  const uint16_t* val_vn;
  const float* cen_k;
  const float* cen_v;
  const float* Pi_v;
  float sm_scale;
  int causal;
  const float* mask;
  int64_t mask_stride_b, mask_stride_q;
  void* out;
  int out_dtype;
  int64_t o_stride_b, o_stride_h, o_stride_s;
  // keys between the packed rows of consecutive (batch, KV head) pairs in every packed array: Sk for the
  // contiguous [B, Hkv, Sk] layout, the capacity of a persistent cache otherwise (split-KV kernel only)
  int64_t kv_stride;
};

int check_attention_args(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d, int64_t sb, int64_t sh,
                         int64_t ss, int64_t Hkv, int64_t Sk, int bits, int mode);

// fp32 mode: query preparation + CUDA-core flash kernel.  `workspace` holds q_cat fp32.
int attention_fwd_fp32(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d, int64_t sb, int64_t sh,
                       int64_t ss, const float* Pi_k, const float* S_eff, AttnArgs a, int bits, void* workspace,
                       cudaStream_t stream);

// bf16 mode: tcgen05 query preparation, tcgen05 flash kernel, tcgen05 back-rotation.
// `prepared` (optional): a constants buffer filled by prepare_constants for the same matrices; the operand images
// are then taken from it and nothing is rebuilt.
int attention_fwd_bf16(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d, int64_t sb, int64_t sh,
                       int64_t ss, const float* Pi_k, const float* S_eff, AttnArgs a, int bits, void* workspace,
                       cudaStream_t stream, const uint8_t* prepared = nullptr);
// scratch bytes of a bf16-mode call, by the kernel that will serve it (0 when the SM-pair kernel runs from a
// prepared constants buffer)
size_t workspace_bytes_bf16_prepared(int64_t B, int64_t Hq, int64_t Sq, int64_t Hkv, int64_t Sk, int64_t kv_stride,
                                     int d);

size_t workspace_bytes_bf16(int64_t BHq, int64_t Sq, int d);

// Decode-sized calls (few query rows per KV head, long keys; tq_attention_decode.cu), three launches: query
// preparation into `q_cat` (bf16 [n_q, 2d]), the split-KV kernel, then merge + back-rotation into a.out.
// `part_ws` holds decode_workspace_bytes(B * Hq).
bool decode_applies(const AttnArgs& a, int d);  // a.kv_stride != a.Sk: any key count
size_t decode_workspace_bytes(int64_t BHq);
int attention_decode(const AttnArgs& a, int64_t B, int bits, const void* q, int q_dtype, int64_t sb, int64_t sh,
                     int64_t ss, const float* Pi_k, const float* S_eff, void* q_cat, void* part_ws, cudaStream_t stream);

// Raw queries and the constant bf16 operands of the SM-pair kernel, which prepares its own query tile
// (q [Pi ; coeff S]^T) and rotates its output back (o Pi_v) on the tensor pipe.
struct PairArgs {
  const void* q;
  int q_dtype;
  int64_t q_stride_b, q_stride_h, q_stride_s;
  const __nv_bfloat16* w_cat;    // [2d, d] = [Pi ; coeff S]
  const __nv_bfloat16* w_unrot;  // [d, d]  = Pi_v^T
  const uint32_t* luts;          // pair tables: 4^(bits-1) key entries, then 4^bits value entries (bf16x2 words)
};

// SM-pair (2-CTA cluster) tensor-core kernel, head_dim 128; needs no per-query scratch.
int attention_c2(const AttnArgs& a, const PairArgs& x, int64_t B, int d, int bits, cudaStream_t stream);
int read_c2_faults(unsigned long long* out);
int trace_enable_c2(int on);
int trace_read_c2(long long* host_buf, int max_records, int* n_out);

int prepare_queries_bf16(const void* q, int dtype, int64_t B, int64_t Hq, int64_t Sq, int d, int64_t sb, int64_t sh,
                         int64_t ss, const float* Pi_k, const float* S_eff, void* w_cat_scratch, void* q_cat,
                         cudaStream_t stream, int q_cat_dtype = TQ_BF16);

}  // namespace tq
