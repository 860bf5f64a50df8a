// Small data-movement kernels of the tensor-parallel layer.
#include "common.cuh"

#include "../../include/lsvd_b200.h"

namespace lsvd {

constexpr int kMaxSegments = 32;

struct GatherSegParams {
  const uint8_t* src;
  uint8_t* dst;
  int64_t dst_row_stride;                 // bytes
  int32_t rows, nseg;
  int64_t src_off[kMaxSegments];          // bytes: first byte of the segment in row 0
  int64_t src_row_stride[kMaxSegments];   // bytes between two rows of the segment
  int64_t dst_off[kMaxSegments];          // bytes: where the segment starts in a destination row
  int32_t len[kMaxSegments];              // bytes, a multiple of 16
};

// grid (segments, rows): 16-byte copies
__global__ void __launch_bounds__(256) gather_segments_kernel(const __grid_constant__ GatherSegParams p) {
  const int s = blockIdx.x, r = blockIdx.y;
  const uint4* src = reinterpret_cast<const uint4*>(p.src + p.src_off[s] + r * p.src_row_stride[s]);
  uint4* dst = reinterpret_cast<uint4*>(p.dst + r * p.dst_row_stride + p.dst_off[s]);
  for (int i = threadIdx.x; i < (p.len[s] >> 4); i += blockDim.x) dst[i] = __ldcg(src + i);
}

}  // namespace lsvd

extern "C" int lsvd_gather_segments(const void* src, void* dst, int64_t dst_row_stride_bytes, int32_t rows, int32_t nseg,
                                    const int64_t* src_off_bytes, const int64_t* src_row_stride_bytes,
                                    const int64_t* dst_off_bytes, const int32_t* len_bytes, void* stream) {
  using namespace lsvd;
  if (rows < 0 || nseg <= 0 || nseg > kMaxSegments || !src_off_bytes || !src_row_stride_bytes || !dst_off_bytes || !len_bytes)
    return LSVD_ERR_INVALID_ARG;
  if (rows == 0) return LSVD_OK;
  if (src == nullptr || dst == nullptr || rows > 65535 || !aligned(src, 16) || !aligned(dst, 16) || (dst_row_stride_bytes % 16))
    return LSVD_ERR_INVALID_ARG;
  GatherSegParams p{};
  p.src = static_cast<const uint8_t*>(src);
  p.dst = static_cast<uint8_t*>(dst);
  p.dst_row_stride = dst_row_stride_bytes;
  p.rows = rows;
  p.nseg = nseg;
  for (int s = 0; s < nseg; ++s) {
    if ((src_off_bytes[s] % 16) || (src_row_stride_bytes[s] % 16) || (dst_off_bytes[s] % 16) || (len_bytes[s] % 16) ||
        len_bytes[s] < 0 || src_off_bytes[s] < 0 || dst_off_bytes[s] < 0 || dst_off_bytes[s] + len_bytes[s] > dst_row_stride_bytes)
      return LSVD_ERR_INVALID_ARG;
    p.src_off[s] = src_off_bytes[s];
    p.src_row_stride[s] = src_row_stride_bytes[s];
    p.dst_off[s] = dst_off_bytes[s];
    p.len[s] = len_bytes[s];
  }
  gather_segments_kernel<<<dim3(nseg, rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  LSVD_CUDA_TRY(cudaGetLastError());
  return LSVD_OK;
}
