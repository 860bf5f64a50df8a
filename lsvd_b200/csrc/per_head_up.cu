// Ragged per-head up-projection of a latent: y[t, h * cout + c] = sum_r A_h[c, r] * z[t, off_h + r] (+ bias).
//
// The arithmetic of SVDLinear.forward for per-head factors with a rank split
// (fake_quant/utils/svd_utils.py:1978-2015): there the latents and the factors are padded to the largest rank and
// multiplied by one einsum; here every head reads exactly its own r_h columns.  fp16 operands, fp32 accumulation, one
// rounding to fp16 at the end (the bias, if any, is added to the rounded product in fp16 like the reference's
// `y + bias`).
#include "common.cuh"

#include <cuda_fp16.h>

#include "../../include/lsvd_b200.h"

namespace lsvd {

constexpr int kPhuThreads = 256;
constexpr int kPhuTokens = 8;       // tokens per block: the factor of a head is read once for all of them

struct PerHeadUpParams {
  const __half* z; int64_t z_row_stride;
  const __half* a;                   // the factors, head after head, each [cout, r_h] row-major
  const __half* bias;                // [num_heads * cout] or NULL
  __half* y; int64_t y_row_stride;
  int32_t tokens, num_heads, cout;
  int32_t off[LSVD_MAX_HEADS + 1];   // first latent column of every head
};

// grid (heads, ceil(tokens / 8)); a warp owns output channels warp, warp + 8, ...: its lanes split the rank (coalesced
// reads of the factor's row), every lane keeps the partial dot products of the block's 8 tokens.
__global__ void __launch_bounds__(kPhuThreads) per_head_up_kernel(const PerHeadUpParams p) {
  extern __shared__ __half zs[];     // [8][r_h]
  const int h = blockIdx.x;
  const int t0 = blockIdx.y * kPhuTokens;
  const int nt = min(kPhuTokens, p.tokens - t0);
  const int c0 = p.off[h], r = p.off[h + 1] - c0;
  for (int i = threadIdx.x; i < kPhuTokens * r; i += blockDim.x) {
    const int t = i / r, j = i - t * r;
    zs[i] = t < nt ? p.z[(t0 + t) * p.z_row_stride + c0 + j] : __float2half(0.f);
  }
  __syncthreads();
  const __half* a = p.a + static_cast<int64_t>(c0) * p.cout;    // sum_{g < h} cout * r_g elements precede head h
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int c = warp; c < p.cout; c += kPhuThreads / 32) {
    const __half* row = a + static_cast<int64_t>(c) * r;
    float acc[kPhuTokens];
#pragma unroll
    for (int t = 0; t < kPhuTokens; ++t) acc[t] = 0.f;
    for (int j = lane; j < r; j += 32) {
      const float w = __half2float(row[j]);
#pragma unroll
      for (int t = 0; t < kPhuTokens; ++t) acc[t] = fmaf(w, __half2float(zs[t * r + j]), acc[t]);
    }
#pragma unroll
    for (int t = 0; t < kPhuTokens; ++t) acc[t] = warp_sum(acc[t]);
    if (lane < nt) {
      float v = acc[0];
#pragma unroll
      for (int t = 1; t < kPhuTokens; ++t) v = lane == t ? acc[t] : v;
      __half o = __float2half_rn(v);
      const int col = h * p.cout + c;
      if (p.bias != nullptr) o = __hadd(o, p.bias[col]);
      p.y[(t0 + lane) * p.y_row_stride + col] = o;
    }
  }
}

}  // namespace lsvd

extern "C" int lsvd_per_head_up(const void* z, int64_t z_row_stride, const void* factors, const int32_t* rank_off,
                                const void* bias, void* y, int64_t y_row_stride, int32_t tokens, int32_t num_heads,
                                int32_t cout, void* stream) {
  using namespace lsvd;
  if (tokens < 0 || num_heads <= 0 || num_heads > LSVD_MAX_HEADS || cout <= 0 || rank_off == nullptr) return LSVD_ERR_INVALID_ARG;
  if (tokens == 0) return LSVD_OK;
  if (z == nullptr || factors == nullptr || y == nullptr) return LSVD_ERR_INVALID_ARG;
  PerHeadUpParams p{};
  int rmax = 0;
  for (int h = 0; h <= num_heads; ++h) {
    p.off[h] = rank_off[h];
    if (h > 0) {
      if (rank_off[h] < rank_off[h - 1]) return LSVD_ERR_INVALID_ARG;
      rmax = std::max(rmax, rank_off[h] - rank_off[h - 1]);
    }
  }
  if (rank_off[0] != 0 || z_row_stride < rank_off[num_heads] || y_row_stride < static_cast<int64_t>(num_heads) * cout)
    return LSVD_ERR_INVALID_ARG;
  const size_t smem = static_cast<size_t>(kPhuTokens) * std::max(rmax, 1) * sizeof(__half);
  if (smem > 200 * 1024) return LSVD_ERR_UNSUPPORTED;
  p.z = static_cast<const __half*>(z);
  p.z_row_stride = z_row_stride;
  p.a = static_cast<const __half*>(factors);
  p.bias = static_cast<const __half*>(bias);
  p.y = static_cast<__half*>(y);
  p.y_row_stride = y_row_stride;
  p.tokens = tokens;
  p.num_heads = num_heads;
  p.cout = cout;
  if (smem > 48 * 1024) LSVD_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(per_head_up_kernel), smem));
  const dim3 grid(num_heads, (tokens + kPhuTokens - 1) / kPhuTokens);
  if (grid.y > 65535u) return LSVD_ERR_UNSUPPORTED;
  per_head_up_kernel<<<grid, kPhuThreads, smem, static_cast<cudaStream_t>(stream)>>>(p);
  LSVD_CUDA_TRY(cudaGetLastError());
  return LSVD_OK;
}
