// Device functions shared by the stand-alone kernels and the fused decode kernel: the per-token activation
// quantiser (plain, RMSNorm and sign-FWHT forms), the cache-append rounding, small MMA wrappers.  Each function
// is the arithmetic of one reference routine; a kernel that calls it produces the same bits whatever launch
// it sits in.
#pragma once

#include "common.cuh"

namespace lsvd {

#ifdef __CUDACC__

// ----------------------------------------------------------------------------------------------
// per-token quantisation, optional power-of-two rotation
//   fake_quant/utils/quant_utils.py:201-212,30-33 (ActQuantizer), hadamard_utils.py:99-104 (rotation),
//   kernels/layer_bench/ffn_kernel/utils.py:560-565 (RMSNorm)
// ----------------------------------------------------------------------------------------------
struct ActQuantParams {
  const __half* x;
  int64_t x_row_stride;
  const __half* sign;
  const __half* norm_weight;   // RMSNorm weight [cols] or NULL
  float norm_eps;
  int8_t* q;
  int64_t q_row_stride;
  float* scale;
  __half* x_rot;
  int32_t rows, cols, rotate;
  int32_t vec8;              // rows of x, sign and q allow 16 / 8-byte accesses
  float rot_scale;           // 1 / sqrt(cols)
  // optional: the row is fp16(x32[r, i] + add16[r, i]) instead of x (a reduced fp32 partial sum plus its fp16
  // residual); sum_out receives that fp16 row
  const float* x32;
  const __half* add16;
  __half* sum_out;
  __half* fake;              // optional [rows, cols] (contiguous): the fake-quantised row fp16(scale * code)
};

__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < (blockDim.x >> 5)) ? red[lane] : 0.f;
  r = warp_max(r);
  return r;
}

// scale = absmax / 127 (1 for a zero row), both divisions IEEE: the codes must match the reference bit for bit.
__device__ __forceinline__ float act_scale_of(float amax) { return amax > 0.f ? __fdiv_rn(amax, 127.f) : 1.f; }

__device__ __forceinline__ int8_t act_code(float x, float s) {
  const float y = rintf(__fdiv_rn(x, s));
  return static_cast<int8_t>(fminf(fmaxf(y, -128.f), 127.f));
}

// One row by one thread block.  `row`: cols floats of shared memory, `red`: 8 floats.  Every thread of the block
// must call it (block barriers inside); any block size that is a multiple of 32 up to 256.
__device__ __forceinline__ void act_quant_row(const ActQuantParams& p, int r, float* row, float* red) {
  const __half* x = p.x + r * p.x_row_stride;
  if (p.x32 != nullptr) {
    const int64_t base = static_cast<int64_t>(r) * p.cols;
    if ((p.cols & 3) == 0) {
      // four entries per thread and pass (rows start 16-byte aligned: contiguous tensors, cols a multiple of 4), all of a
      // thread's loads requested before the first use
      const int quads = p.cols >> 2;
      for (int c0 = threadIdx.x; c0 < quads; c0 += 4 * blockDim.x) {
        float4 xv[4];
        uint2 av[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = c0 + u * blockDim.x;
          if (c < quads) {
            xv[u] = __ldcg(reinterpret_cast<const float4*>(p.x32 + base) + c);
            if (p.add16 != nullptr) av[u] = __ldg(reinterpret_cast<const uint2*>(p.add16 + base) + c);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = c0 + u * blockDim.x;
          if (c < quads) {
            float v[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w};
            if (p.add16 != nullptr) {
              const float2 a0 = __half22float2(*reinterpret_cast<const __half2*>(&av[u].x));
              const float2 a1 = __half22float2(*reinterpret_cast<const __half2*>(&av[u].y));
              v[0] += a0.x; v[1] += a0.y; v[2] += a1.x; v[3] += a1.y;
            }
            const __half2 h0 = __floats2half2_rn(v[0], v[1]), h1 = __floats2half2_rn(v[2], v[3]);
            if (p.sum_out != nullptr) {
              uint2 o;
              o.x = *reinterpret_cast<const uint32_t*>(&h0);
              o.y = *reinterpret_cast<const uint32_t*>(&h1);
              reinterpret_cast<uint2*>(p.sum_out + base)[c] = o;
            }
            const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
            row[4 * c] = f0.x; row[4 * c + 1] = f0.y; row[4 * c + 2] = f1.x; row[4 * c + 3] = f1.y;
          }
        }
      }
    } else {
      for (int i = threadIdx.x; i < p.cols; i += blockDim.x) {
        const int64_t o = base + i;
        float v = __ldcg(p.x32 + o);
        if (p.add16 != nullptr) v += __half2float(p.add16[o]);
        const __half hv = __float2half_rn(v);
        if (p.sum_out != nullptr) p.sum_out[o] = hv;
        row[i] = __half2float(hv);
      }
    }
  } else if (p.vec8) {
    // 16-byte loads, all of a thread's chunks in flight before the first use
    const int chunks = p.cols >> 3;
    for (int c0 = threadIdx.x; c0 < chunks; c0 += 4 * blockDim.x) {
      uint4 xv[4], sv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * blockDim.x;
        if (c < chunks) {
          xv[u] = __ldcg(reinterpret_cast<const uint4*>(x) + c);
          if (p.sign != nullptr) sv[u] = __ldg(reinterpret_cast<const uint4*>(p.sign) + c);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * blockDim.x;
        if (c < chunks) {
          const __half2* xh = reinterpret_cast<const __half2*>(&xv[u]);
          const __half2* sh = reinterpret_cast<const __half2*>(&sv[u]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float2 f = __half22float2(xh[e]);
            if (p.sign != nullptr) {
              const float2 g2 = __half22float2(sh[e]);
              f.x *= g2.x;
              f.y *= g2.y;
            }
            row[c * 8 + 2 * e] = f.x;
            row[c * 8 + 2 * e + 1] = f.y;
          }
        }
      }
    }
  } else {
    for (int i = threadIdx.x; i < p.cols; i += blockDim.x) {
      float v = __half2float(x[i]);
      if (p.sign != nullptr) v *= __half2float(p.sign[i]);
      row[i] = v;
    }
  }
  __syncthreads();
  if (p.norm_weight != nullptr) {
    // RMSNorm as kernels/layer_bench/ffn_kernel/utils.py:560-565: fp32 statistics, the normalised value
    // rounded to fp16, then an fp16 product with the weight.
    float ss = 0.f;
    for (int i = threadIdx.x; i < p.cols; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
    ss = warp_sum(ss);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int wi = 0; wi < (blockDim.x >> 5); ++wi) tot += red[wi];
    const float inv = rsqrtf(tot / static_cast<float>(p.cols) + p.norm_eps);
    for (int i = threadIdx.x; i < p.cols; i += blockDim.x) {
      const __half xn = __float2half_rn(row[i] * inv);
      const __half hv = __float2half_rn(__half2float(xn) * __half2float(p.norm_weight[i]));
      row[i] = __half2float(hv);
      if (p.x_rot != nullptr) p.x_rot[static_cast<int64_t>(r) * p.cols + i] = hv;
    }
    __syncthreads();
  }
  if (p.rotate) {
    // Sylvester butterflies in fp32, stride 1 first: the same additions in the same order as the
    // reference's butterfly loop, so the rotated row is bit-identical.
    int lg = 0;
    for (int h = 1; h < p.cols; h <<= 1, ++lg) {
      for (int i = threadIdx.x; i < (p.cols >> 1); i += blockDim.x) {
        const int j = ((i >> lg) << (lg + 1)) + (i & (h - 1));
        const float a = row[j], b = row[j + h];
        row[j] = a + b;
        row[j + h] = a - b;
      }
      __syncthreads();
    }
    for (int i = threadIdx.x; i < p.cols; i += blockDim.x) {
      const __half hv = __float2half_rn(row[i] * p.rot_scale);
      row[i] = __half2float(hv);
      if (p.x_rot != nullptr) p.x_rot[static_cast<int64_t>(r) * p.cols + i] = hv;
    }
    __syncthreads();
  }
  float amax = 0.f;
  for (int i = threadIdx.x; i < p.cols; i += blockDim.x) amax = fmaxf(amax, fabsf(row[i]));
  amax = block_max(amax, red);
  const float s = act_scale_of(amax);
  if (threadIdx.x == 0) p.scale[r] = s;
  int8_t* q = p.q + r * p.q_row_stride;
  if (p.vec8) {
    for (int c = threadIdx.x; c < (p.cols >> 3); c += blockDim.x) {
      uint32_t lo = 0u, hi = 0u;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        lo |= static_cast<uint32_t>(static_cast<uint8_t>(act_code(row[c * 8 + e], s))) << (8 * e);
        hi |= static_cast<uint32_t>(static_cast<uint8_t>(act_code(row[c * 8 + 4 + e], s))) << (8 * e);
      }
      *reinterpret_cast<uint2*>(q + c * 8) = make_uint2(lo, hi);
    }
  } else {
    for (int i = threadIdx.x; i < p.cols; i += blockDim.x) q[i] = act_code(row[i], s);
  }
  if (p.fake != nullptr) {
    // what the reference's quantiser returns from forward(): scale * code in fp32, rounded to fp16
    // (fake_quant/utils/quant_utils.py:41-46)
    __half* f = p.fake + static_cast<int64_t>(r) * p.cols;
    for (int i = threadIdx.x; i < p.cols; i += blockDim.x) f[i] = __float2half_rn(s * static_cast<float>(act_code(row[i], s)));
  }
}

// ----------------------------------------------------------------------------------------------
// The input rotation for rows of 4096 entries (the 7B hidden size): radix-16 butterflies in registers
// ----------------------------------------------------------------------------------------------
// 256 threads x 16 entries.  Three rounds of four butterfly stages each run in registers (strides 1..8 on 16
// consecutive entries, 16..128 and 256..2048 after an exchange through shared memory): the same additions in the
// same order as the stage-by-stage loop of act_quant_row, with 5 block barriers instead of 14.
__device__ __forceinline__ int rot_slot(int j) { return j + (j >> 4); }      // one pad word per 16: conflict-free exchanges

__device__ __forceinline__ void butterflies16(float (&e)[16]) {
#pragma unroll
  for (int h = 1; h < 16; h <<= 1)
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if ((i & h) == 0) {
        const float a = e[i], b = e[i + h];
        e[i] = a + b;
        e[i + h] = a - b;
      }
}

// `row`: 4096 + 256 floats of shared memory, `red`: 8 floats; exactly 256 threads.
__device__ __forceinline__ void act_quant_rot4096_row(const ActQuantParams& p, int r, float* row, float* red) {
  const int T = threadIdx.x;
  const __half* x = p.x + r * p.x_row_stride;
  float e[16];
  {
    const uint4 v0 = __ldcg(reinterpret_cast<const uint4*>(x) + 2 * T), v1 = __ldcg(reinterpret_cast<const uint4*>(x) + 2 * T + 1);
    uint4 s0 = make_uint4(0u, 0u, 0u, 0u), s1 = s0;
    if (p.sign != nullptr) {
      s0 = __ldg(reinterpret_cast<const uint4*>(p.sign) + 2 * T);
      s1 = __ldg(reinterpret_cast<const uint4*>(p.sign) + 2 * T + 1);
    }
    const __half2* xa = reinterpret_cast<const __half2*>(&v0);
    const __half2* xb = reinterpret_cast<const __half2*>(&v1);
    const __half2* sa = reinterpret_cast<const __half2*>(&s0);
    const __half2* sb = reinterpret_cast<const __half2*>(&s1);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(xa[i]), g2 = __half22float2(xb[i]);
      if (p.sign != nullptr) {
        const float2 u = __half22float2(sa[i]), w = __half22float2(sb[i]);
        f.x *= u.x; f.y *= u.y; g2.x *= w.x; g2.y *= w.y;
      }
      e[2 * i] = f.x; e[2 * i + 1] = f.y; e[8 + 2 * i] = g2.x; e[8 + 2 * i + 1] = g2.y;
    }
  }
  butterflies16(e);                                            // strides 1, 2, 4, 8: entries 16 T + i
#pragma unroll
  for (int i = 0; i < 16; ++i) row[rot_slot(16 * T + i)] = e[i];
  __syncthreads();
  const int j2 = (T >> 4) * 256 + (T & 15);                    // strides 16 .. 128: entries j2 + 16 i
#pragma unroll
  for (int i = 0; i < 16; ++i) e[i] = row[rot_slot(j2 + 16 * i)];
  butterflies16(e);
#pragma unroll
  for (int i = 0; i < 16; ++i) row[rot_slot(j2 + 16 * i)] = e[i];
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 16; ++i) e[i] = row[rot_slot(T + 256 * i)];   // strides 256 .. 2048: entries T + 256 i
  butterflies16(e);
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    e[i] = __half2float(__float2half_rn(e[i] * p.rot_scale));
    amax = fmaxf(amax, fabsf(e[i]));
    row[rot_slot(T + 256 * i)] = e[i];
  }
  amax = block_max(amax, red);                                 // its barriers also publish the rotated row
  const float s = act_scale_of(amax);
  if (T == 0) p.scale[r] = s;
  // 16 consecutive entries per thread again: one 16-byte store of codes (and two of fp16 values if wanted)
  __align__(16) int8_t codes[16];
  __align__(16) __half hv[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float v = row[rot_slot(16 * T + i)];
    codes[i] = act_code(v, s);
    hv[i] = __float2half_rn(v);
  }
  *reinterpret_cast<uint4*>(p.q + r * p.q_row_stride + 16 * T) = *reinterpret_cast<const uint4*>(codes);
  if (p.x_rot != nullptr) {
    uint4* dst = reinterpret_cast<uint4*>(p.x_rot + static_cast<int64_t>(r) * p.cols + 16 * T);
    dst[0] = reinterpret_cast<const uint4*>(hv)[0];
    dst[1] = reinterpret_cast<const uint4*>(hv)[1];
  }
}

// True when act_quant_rot4096_row can take the row (the host-side test of lsvd_act_quant).
__host__ __device__ inline bool act_quant_rot4096_ok(const ActQuantParams& p) {
  return p.rotate && p.cols == 4096 && p.vec8 && p.norm_weight == nullptr && p.fake == nullptr &&
         (reinterpret_cast<uintptr_t>(p.q) & 15) == 0 && (p.q_row_stride % 16) == 0 &&
         (p.x_rot == nullptr || (reinterpret_cast<uintptr_t>(p.x_rot) & 15) == 0);
}

// ----------------------------------------------------------------------------------------------
// cache-append rounding (kernels/layer_bench/benchmark_triton_int8_layer.py:107-109,
// fd_kernel/destindex_copy_quantize_latent.py:26-29)
// ----------------------------------------------------------------------------------------------
// `r` = the correctly rounded reciprocal of the scale (__frcp_rn), used by the fp16-division form only.
template <int kRounding>
__device__ __forceinline__ int quantise_one(float x, float s, float r) {
  if (kRounding == LSVD_ROUND_TORCH) {
    // fp16 division = exact quotient rounded once to fp16; then round half to even.  Both roundings are done with
    // additions instead of conversions (the conversion unit is what bounds the append kernel at prefill sizes):
    //   * to 11 significant bits: add and subtract 1.5 * 2^(e + 13), e the exponent of y -- the sum lies in the binade
    //     whose spacing is 2^(e - 10), the spacing of fp16 numbers around y, and fp32 addition rounds ties to even.
    //     (Below 2^-14, where fp16 is coarser than that, the code is 0 either way.)  Quotients beyond +-256 end at a
    //     clamp bound whatever their rounding, so they are clamped first, which also keeps e + 13 in range;
    //   * to an integer: add 1.5 * 2^23 and read the low mantissa bits.
    // The quotient: x and s are fp16 numbers, so x / s is a ratio of two 11-bit integers and stays at least two fp32
    // spacings away from every fp16 rounding boundary it does not hit exactly.  A quotient within one spacing of the
    // exact one therefore rounds to the same fp16 number as the IEEE quotient: q0 = x r, one residual, one correction
    // (three FMA-pipe operations instead of a division per entry); a boundary that is hit exactly is representable
    // and comes out exact.
    const float q0 = __fmul_rn(x, r);
    float y = __fmaf_rn(__fmaf_rn(-s, q0, x), r, q0);
    y = fminf(fmaxf(y, -256.f), 256.f);
    const float c = __uint_as_float(((__float_as_uint(y) & 0x7f800000u) + (13u << 23)) | 0x00400000u);
    y = __fsub_rn(__fadd_rn(y, c), c);
    const int q = __float_as_int(__fadd_rn(y, 12582912.f)) - 0x4b400000;
    return min(max(q, -128), 127);
  } else {
    float y = __fdiv_rn(x, s);
    int r2 = static_cast<int>(y >= 0.f ? y + 0.5f : y - 0.5f);   // conversion truncates toward zero
    return min(max(r2, -128), 127);
  }
}

// Scale of a (token, head) unit of the latent cache from its absmax: fp16(max(absmax / 128, 1e-4)).
__device__ __forceinline__ __half latent_scale_of(float amax) {
  __half s16 = __float2half_rn(amax * 0.0078125f);       // absmax is an fp16 value; /128 in fp16 is one rounding
  const __half floor16 = __float2half_rn(1e-4f);
  if (__half2float(s16) < __half2float(floor16)) s16 = floor16;
  return s16;
}

// (H_K kron H_nb) rotation + per-token quantisation: parameters shared by its kernels.
struct HadQuantParams {
  const __half* x;
  int64_t x_row_stride;
  const uint4* packed;       // had_K in MMA A-fragment order: [m tile][k tile][lane] x {a0, a1, a2, a3}
  int8_t* q;
  int64_t q_row_stride;
  float* scale;
  __half* y;
  int32_t rows, cols, K, nb; // nb = cols / K, a power of two in [8, 128]
  int32_t Kp, ld;            // K rounded up to 16; leading dimension (halves) of the staged columns
  int32_t cluster, ntile_per;   // blocks per token, 8-column tiles per block
  int32_t x_vec16;              // rows of x are 16-byte aligned
  float rot_scale;           // 1 / sqrt(cols)
};

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col).  Lane (g, t):
//   a0: row g, k 2t..2t+1   a1: row g+8, k 2t..   a2: row g, k 2t+8..   a3: row g+8, k 2t+8..
//   b0: k 2t..2t+1, col g   b1: k 2t+8.., col g   d0,d1: row g, cols 2t,2t+1   d2,d3: row g+8
__device__ __forceinline__ void mma_f16_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

#endif  // __CUDACC__

}  // namespace lsvd
