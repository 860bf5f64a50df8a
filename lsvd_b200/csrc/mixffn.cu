// Quantisers of the all-fp32 "mixffn" W8A8 pipeline: RMSNorm + per-token quantiser, quantiser of fp16 rows with a
// maximum collected by the preceding product, and quantiser of int32 accumulators.  One block per token row; rows are
// a few KB and stay in L1/L2 between the passes, so the kernels are launch-bound at decode sizes.
//
// Arithmetic (fixed so that codes match the CPU statement bit for bit): every product and quotient is a single
// rounded fp32 operation in the written order; scale = max(absmax / 127, 1e-8); code = clamp(trunc(v / scale +- 0.5)).
#include "common.cuh"

namespace lsvd {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();                       // red may still be read from an earlier reduction
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int i = 1; i < kThreads / 32; ++i) r = fmaxf(r, red[i]);
  return r;
}

__device__ __forceinline__ float scale_of(float absmax) { return fmaxf(__fdiv_rn(absmax, 127.0f), 1e-8f); }

__device__ __forceinline__ int code_of(float v, float scale) {
  const float s = __fdiv_rn(v, scale);
  const int r = __float2int_rz(s >= 0.f ? __fadd_rn(s, 0.5f) : __fsub_rn(s, 0.5f));
  return max(-128, min(127, r));
}

struct RmsParams {
  const __half* x; int64_t x_row_stride; const __half* w; float eps;
  int8_t* q; int64_t q_row_stride; float* scale; uint32_t* clear_words; int32_t clear_per_row; int32_t cols;
};

__global__ void __launch_bounds__(kThreads) mix_rmsnorm_quant_kernel(RmsParams p) {
  __shared__ double red_d[kThreads / 32];
  __shared__ float red_f[kThreads / 32];
  grid_dependency_sync();
  const int row = blockIdx.x;
  const __half* x = p.x + row * p.x_row_stride;
  if (p.clear_words != nullptr)
    for (int i = threadIdx.x; i < p.clear_per_row; i += kThreads) p.clear_words[static_cast<int64_t>(row) * p.clear_per_row + i] = 0u;
  // sum of squares: squares of fp16 values are exact in fp32 and their sum is carried in fp64, so the statistic is the
  // correctly rounded one whatever the order of the additions
  double ss = 0.0;
  for (int c = threadIdx.x; c < p.cols; c += kThreads) {
    const float v = __half2float(x[c]);
    ss += static_cast<double>(v * v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red_d[threadIdx.x >> 5] = ss;
  __syncthreads();
  double tot = 0.0;
#pragma unroll
  for (int i = 0; i < kThreads / 32; ++i) tot += red_d[i];
  const float sumsq = static_cast<float>(tot);
  const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sumsq, static_cast<float>(p.cols)), p.eps)));
  float mx = 0.f;
  for (int c = threadIdx.x; c < p.cols; c += kThreads)
    mx = fmaxf(mx, fabsf(__fmul_rn(__fmul_rn(__half2float(x[c]), inv), __half2float(p.w[c]))));
  mx = block_max(mx, red_f);
  const float scale = scale_of(mx);
  int8_t* q = p.q + row * p.q_row_stride;
  for (int c = threadIdx.x; c < p.cols; c += kThreads)
    q[c] = static_cast<int8_t>(code_of(__fmul_rn(__fmul_rn(__half2float(x[c]), inv), __half2float(p.w[c])), scale));
  if (threadIdx.x == 0) p.scale[row] = __half2float(__float2half_rn(scale));
}

struct GroupParams {
  const __half* x; int64_t x_row_stride; const uint32_t* absmax; int64_t absmax_stride;
  int8_t* q; int64_t q_row_stride; float* scale; int64_t scale_stride; int32_t cols, split, shared, vec;
};

__global__ void __launch_bounds__(kThreads) mix_group_quant_kernel(GroupParams p) {
  grid_dependency_sync();
  const int row = blockIdx.x;
  const bool two = p.split < p.cols;
  float m0 = __uint_as_float(p.absmax[row * p.absmax_stride]);
  float m1 = two ? __uint_as_float(p.absmax[row * p.absmax_stride + 1]) : m0;
  if (p.shared) m0 = m1 = fmaxf(m0, m1);
  const float s0 = scale_of(m0), s1 = scale_of(m1);
  const __half* x = p.x + row * p.x_row_stride;
  int8_t* q = p.q + row * p.q_row_stride;
  if (p.vec) {                                         // eight columns per step; split is a multiple of 8
    for (int c = threadIdx.x * 8; c < p.cols; c += kThreads * 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(x + c);
      const __half2* h = reinterpret_cast<const __half2*>(&raw);
      const float s = c < p.split ? s0 : s1;
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        const uint32_t pair = (static_cast<uint32_t>(code_of(f.x, s)) & 0xffu) | ((static_cast<uint32_t>(code_of(f.y, s)) & 0xffu) << 8);
        if (i < 2) lo |= pair << (16 * i); else hi |= pair << (16 * (i - 2));
      }
      *reinterpret_cast<uint2*>(q + c) = make_uint2(lo, hi);
    }
  } else {
    for (int c = threadIdx.x; c < p.cols; c += kThreads)
      q[c] = static_cast<int8_t>(code_of(__half2float(x[c]), c < p.split ? s0 : s1));
  }
  if (threadIdx.x == 0) {
    p.scale[row * p.scale_stride] = s0;
    if (two && !p.shared) p.scale[row * p.scale_stride + 1] = s1;
  }
}

struct AccParams {
  const int32_t* acc; int64_t acc_row_stride; const float* row_scale; int64_t row_scale_stride; const float* col_scale;
  int8_t* q; int64_t q_row_stride; float* scale; int32_t cols;
};

__global__ void __launch_bounds__(kThreads) mix_acc_quant_kernel(AccParams p) {
  __shared__ float red_f[kThreads / 32];
  grid_dependency_sync();
  const int row = blockIdx.x;
  const int32_t* acc = p.acc + row * p.acc_row_stride;
  const float rs = p.row_scale[row * p.row_scale_stride];
  float mx = 0.f;
  for (int c = threadIdx.x; c < p.cols; c += kThreads)
    mx = fmaxf(mx, fabsf(__fmul_rn(__fmul_rn(static_cast<float>(acc[c]), rs), p.col_scale[c])));
  mx = block_max(mx, red_f);
  const float scale = scale_of(mx);
  int8_t* q = p.q + row * p.q_row_stride;
  for (int c = threadIdx.x; c < p.cols; c += kThreads)
    q[c] = static_cast<int8_t>(code_of(__fmul_rn(__fmul_rn(static_cast<float>(acc[c]), rs), p.col_scale[c]), scale));
  if (threadIdx.x == 0) p.scale[row] = scale;
}

}  // namespace
}  // namespace lsvd

extern "C" int lsvd_mix_rmsnorm_quant(const lsvd_mix_rmsnorm_quant_args* a, void* stream) {
  using namespace lsvd;
  if (a == nullptr || a->rows <= 0 || a->cols <= 0 || !a->x || !a->norm_weight || !a->q || !a->scale) return LSVD_ERR_INVALID_ARG;
  if (a->clear_words != nullptr && a->clear_per_row <= 0) return LSVD_ERR_INVALID_ARG;
  RmsParams p{static_cast<const __half*>(a->x), a->x_row_stride, static_cast<const __half*>(a->norm_weight), a->eps,
              a->q, a->q_row_stride, a->scale, a->clear_words, a->clear_per_row, a->cols};
  LSVD_CUDA_TRY(launch_chained(mix_rmsnorm_quant_kernel, dim3(a->rows), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), 1,
                               ffn_chain_enabled(), p));
  return LSVD_OK;
}

extern "C" int lsvd_mix_group_quant(const lsvd_mix_group_quant_args* a, void* stream) {
  using namespace lsvd;
  if (a == nullptr || a->rows <= 0 || a->cols <= 0 || a->split <= 0 || a->split > a->cols) return LSVD_ERR_INVALID_ARG;
  if (!a->x || !a->absmax || !a->q || !a->scale) return LSVD_ERR_INVALID_ARG;
  const bool vec = (a->cols % 8) == 0 && (a->split % 8) == 0 && aligned(a->x, 16) && (a->x_row_stride % 8) == 0 &&
                   aligned(a->q, 8) && (a->q_row_stride % 8) == 0;
  GroupParams p{static_cast<const __half*>(a->x), a->x_row_stride, a->absmax, a->absmax_stride, a->q, a->q_row_stride,
                a->scale, a->scale_stride, a->cols, a->split, a->shared, vec ? 1 : 0};
  LSVD_CUDA_TRY(launch_chained(mix_group_quant_kernel, dim3(a->rows), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), 1,
                               ffn_chain_enabled(), p));
  return LSVD_OK;
}

extern "C" int lsvd_mix_acc_quant(const lsvd_mix_acc_quant_args* a, void* stream) {
  using namespace lsvd;
  if (a == nullptr || a->rows <= 0 || a->cols <= 0 || !a->acc || !a->row_scale || !a->col_scale || !a->q || !a->scale)
    return LSVD_ERR_INVALID_ARG;
  AccParams p{a->acc, a->acc_row_stride, a->row_scale, a->row_scale_stride, a->col_scale, a->q, a->q_row_stride, a->scale,
              a->cols};
  LSVD_CUDA_TRY(launch_chained(mix_acc_quant_kernel, dim3(a->rows), dim3(kThreads), 0, static_cast<cudaStream_t>(stream), 1,
                               ffn_chain_enabled(), p));
  return LSVD_OK;
}
