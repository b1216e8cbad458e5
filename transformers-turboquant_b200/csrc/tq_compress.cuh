// Argument block shared by the fp32 (CUDA-core) and tensor-core compression kernels.
#pragma once
#include "tq_common.cuh"

namespace tq {

constexpr int kTileRows = 64;

struct CompressArgs {
  const void* src;
  int64_t n_vec, H, S;
  int64_t stride_b, stride_h, stride_s;
  const float* Pi;
  const float* S_eff;
  const float* centroids;
  const float* boundaries;
  uint8_t* packed_idx;
  uint8_t* packed_signs;
  uint16_t* vec_norms;
  uint16_t* residual_norms;
  int num_tiles;
  // Output row of input vector n = (b * H + h) * S + s: (b * H + h) * out_stride + out_offset + s.  out_stride = S
  // and out_offset = 0 give the contiguous layout; a persistent cache passes its capacity and its fill level.
  int64_t out_stride, out_offset;
};

__device__ __forceinline__ int64_t compress_out_row(const CompressArgs& a, int64_t n) {
  return a.out_stride == a.S ? n + a.out_offset : (n / a.S) * a.out_stride + a.out_offset + n % a.S;
}

// bf16 inputs, rotation and sketch projection on tcgen05 (tq_compress_tc.cu).
int compress_tc(bool is_key, int d, int index_bits, const CompressArgs& a, cudaStream_t stream);

// Keys and values in one launch, tiles staged by TMA, constants from a prepared buffer (tq_compress_kv.cu):
// bf16 inputs, head_dim 128, TQ_MODE_BF16.  Either input may be NULL (that side is skipped).  Strides in
// elements (batch, head, position).  TQ_ERR_UNSUPPORTED when the driver refuses a tensor map for the strides.
bool compress_kv_applies(int dtype, int d, int mode);
int compress_kv(const void* k, const void* v, int64_t B, int64_t H, int64_t S, const int64_t* k_strides,
                const int64_t* v_strides, const uint8_t* consts, int bits, uint8_t* key_idx, uint8_t* key_sgn,
                uint16_t* key_vn, uint16_t* key_rn, uint8_t* val_idx, uint16_t* val_vn, int64_t out_stride,
                int64_t out_offset, cudaStream_t stream);

}  // namespace tq
