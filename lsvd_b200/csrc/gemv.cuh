// Shared by the two forms of the weight-streaming W8A8 product: parameters, the int8 MMA and the epilogue.
#pragma once

#include "common.cuh"

namespace lsvd {

struct GemvParams {
  const int8_t* w;  int64_t w_row_stride;  const float* w_scale;
  const int8_t* w2; int64_t w2_row_stride; const float* w2_scale;
  const int8_t* a;  int64_t a_row_stride;  const float* a_scale;  int64_t a_scale_stride;
  const int8_t* a2; int64_t a2_row_stride; const float* a2_scale; int64_t a2_scale_stride;
  __half* out; int64_t out_row_stride; int32_t out_col;
  const __half* residual; int64_t residual_row_stride;
  int32_t* acc_out; int32_t* acc2_out;
  int32_t* status_word;
  int32_t m, n, k, epilogue;
  // optional per-token maximum of |fp32 value| over the output channels, kept as the bit pattern of a non-negative
  // float (ordered like an unsigned integer): slot 0 for channels below absmax_split, slot 1 from there on
  uint32_t* row_absmax; int64_t row_absmax_stride; int32_t absmax_split;
  int32_t prefetch;          // pull the block's weight rows toward L2 before waiting for the previous kernel
  float* out_f32;            // optional [m, n]: (acc * a_scale) * w_scale before any fp16 rounding (single products)
};

// The TMA-fed persistent form (gemv_tma.cu), for at most 16 tokens.
int launch_gemv_streamed(const GemvParams& p, bool dual, bool split, cudaStream_t st);
// The TMA-fed form for 17..64 tokens: token rows shared by the block's warps through shared memory.
int launch_gemv_wide(const GemvParams& p, bool dual, bool split, cudaStream_t st);

#ifdef __CUDACC__
__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_u4(const int8_t* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + expf(-g)); }

// Dequantise, gate, add the residual and store one element; sum1 / the second scales are used by gate/up pairs.
// Returns |fp32 value| before it is rounded to fp16 (the quantity the all-fp32 pipeline takes its next scale from).
// MIX: the all-fp32 conventions (epilogue 2 for a pair; the returned maximum is used).
template <bool DUAL, bool SPLIT_B, bool MIX = false>
__device__ __forceinline__ float gemv_store(const GemvParams& p, int tok, int row, int sum0, int sum1) {
  if (p.acc_out != nullptr) p.acc_out[static_cast<int64_t>(tok) * p.n + row] = sum0;
  if (DUAL && p.acc2_out != nullptr) p.acc2_out[static_cast<int64_t>(tok) * p.n + row] = sum1;
  if (!DUAL && p.out_f32 != nullptr)
    p.out_f32[static_cast<int64_t>(tok) * p.n + row] = (static_cast<float>(sum0) * p.a_scale[tok * p.a_scale_stride]) * p.w_scale[row];
  if (p.out == nullptr) return 0.f;
  const float sa = p.a_scale[tok * p.a_scale_stride];
  const float f0 = (static_cast<float>(sum0) * sa) * p.w_scale[row];
  float f = f0;
  __half res = __float2half_rn(f0);
  if (DUAL) {
    const float sb = SPLIT_B ? p.a2_scale[tok * p.a2_scale_stride] : sa;
    const float f1 = (static_cast<float>(sum1) * sb) * p.w2_scale[row];
    if (MIX) {
      // all in fp32, one rounding: up * (gate * sigmoid(gate))
      f = f1 * (f0 * (1.0f / (1.0f + expf(-f0))));
      res = __float2half_rn(f);
    } else {
      const __half u = __float2half_rn(f1);
      // silu in fp32 rounded to fp16, then an fp16 product: how PyTorch evaluates F.silu(g) * u on fp16 tensors
      const __half sg = __float2half_rn(silu_f(__half2float(res)));
      res = __float2half_rn(__half2float(sg) * __half2float(u));
    }
  }
  if (p.residual != nullptr)       // fp16 add of the fp16 result and the residual, as the reference's `x @ W + residual`
    res = __float2half_rn(__half2float(res) + __half2float(p.residual[static_cast<int64_t>(tok) * p.residual_row_stride + row]));
  p.out[static_cast<int64_t>(tok) * p.out_row_stride + p.out_col + row] = res;
  return fabsf(f);
}
#endif

}  // namespace lsvd
