// Tensor maps and tiled TMA loads for row-major int8 matrices (K-major tiles, 128-byte swizzle).
#pragma once

#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace lsvd {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// Tensor map of an int8 matrix [rows, k] (row stride in bytes, a multiple of 16; base 16-byte aligned) read in
// boxes of box_rows rows x 128 bytes with the 128-byte swizzle; elements outside the matrix read as zero.
inline int make_map_k128(CUtensorMap* map, const int8_t* base, int64_t rows, int64_t k, int64_t row_stride, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return LSVD_ERR_CUDA;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_stride)};
  const cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1u, 1u};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LSVD_OK : LSVD_ERR_CUDA;
}

// Tensor map of int8 activations [m, k] (row stride in bytes, a multiple of 16) seen as [K block][token][128 bytes]:
// boxes of box_kb K blocks x 16 tokens x 128 bytes, 128-byte swizzle; tokens beyond m and blocks beyond K read as zero.
inline int make_map_act(CUtensorMap* map, const int8_t* base, int64_t m, int64_t k, int64_t row_stride, int box_kb) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return LSVD_ERR_CUDA;
  const cuuint64_t dims[3] = {128u, static_cast<cuuint64_t>(m), static_cast<cuuint64_t>((k + 127) / 128)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(row_stride), 128u};
  const cuuint32_t box[3] = {128u, 16u, static_cast<cuuint32_t>(box_kb)};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LSVD_OK : LSVD_ERR_CUDA;
}

#ifdef __CUDACC__
// One box of a 2-D tensor map into shared memory; x (bytes along K) must be a multiple of 16.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
#endif

}  // namespace lsvd
