// Host helpers shared by the tcgen05 GEMM launchers: tensor-map encoding
// through the driver entry point (no link-time dependency on libcuda) and the
// SM count of the current device.
#pragma once
#include "kernels.h"
#include <cuda.h>
#include <cuda_runtime.h>

namespace imex {
namespace tc_host {

using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                              const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                              const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return static_cast<EncodeFn>(nullptr);
    return reinterpret_cast<EncodeFn>(sym);
  }();
  return fn;
}

// 2-D row-major [outer, inner] 16-bit tensor with row pitch `pitch` elements,
// box [box_outer, 64], 128B swizzle.
inline bool make_map(CUtensorMap *m, const void *base, int in_dtype, int64_t inner, int64_t outer,
                     int box_outer, int64_t pitch = 0) {
  EncodeFn enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch > 0 ? pitch : inner) * 2};
  cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_outer)};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt =
      in_dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return enc(m, dt, 2, const_cast<void *>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 3-D [batch, rows, 64] 16-bit tensor, dense, box [1, box_rows, 64], 128B swizzle: the batches
// (attention heads) are a dimension of their own, so rows past `rows` read zeros instead of the
// next batch's first rows.
inline bool make_map_batched(CUtensorMap *m, const void *base, int in_dtype, int64_t rows, int64_t batch,
                             int box_rows) {
  EncodeFn enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[2] = {64 * 2, static_cast<cuuint64_t>(rows) * 64 * 2};
  cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapDataType dt =
      in_dtype == kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return enc(m, dt, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 2-D row-major [rows, cols] f32 tensor with row pitch `pitch` elements, box
// [32 rows, 32 cols] (128 bytes wide), 128B swizzle: the store side of the GEMM.
inline bool make_map_f32_out(CUtensorMap *m, const void *base, int64_t cols, int64_t rows,
                             int64_t pitch) {
  EncodeFn enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch > 0 ? pitch : cols) * 4};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(base), dims, strides, box,
             estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

inline int sm_count() {
  static int n = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  return n;
}


} // namespace tc_host
} // namespace imex
