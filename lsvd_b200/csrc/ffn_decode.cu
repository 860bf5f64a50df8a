// Hybrid SVD/RTN FFN for decode batches (1..64 tokens): per-token int8 quantisation (with the input and
// the d_ffn Hadamard rotations), and the weight-streaming W8A8 products.
//
// The products are HBM streams of int8 weights: 100 MB per FFN call at the 7B shape whatever the batch.
// A block owns 16 output channels (of one matrix, or of a gate/up pair); its eight warps split K, each
// lane loads 16 contiguous weight bytes per instruction straight into the A fragments of exact int8
// tensor-core MMAs (m16n8k32, int32 accumulators) whose B fragments are the tokens' int8 activations
// (L1/L2 resident), and the warps' partial sums meet in shared memory for the dequantising epilogue.
//
// Reference semantics: fake_quant/utils/hybrid_ffn_utils.py:956-984 (module forward),
// fake_quant/utils/quant_utils.py:201-212,30-33 (activation quantiser), :319-338 (wrapped Linear),
// fake_quant/utils/hadamard_utils.py:99-113 (rotations).
#include <algorithm>
#include <cmath>

#include "common.cuh"
#include "devfn.cuh"
#include "gemv.cuh"

namespace lsvd {

// ----------------------------------------------------------------------------------------------
// per-token quantisation, optional power-of-two rotation: one block per row (the row functions live in devfn.cuh)
// ----------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) act_quant_kernel(const __grid_constant__ ActQuantParams p) {
  extern __shared__ float row[];          // cols floats
  __shared__ float red[8];
  grid_dependency_sync();
  act_quant_row(p, blockIdx.x, row, red);
}

__global__ void __launch_bounds__(256) act_quant_rot4096_kernel(const __grid_constant__ ActQuantParams p) {
  __shared__ float row[4096 + 256];
  __shared__ float red[8];
  grid_dependency_sync();
  act_quant_rot4096_row(p, blockIdx.x, row, red);
}

// ----------------------------------------------------------------------------------------------
// per-token quantisation of MANY rows (prefill): one warp per row, the row in registers
// ----------------------------------------------------------------------------------------------
// The block-per-row kernel passes a row through shared memory with five block barriers: about 12 us per row, which a
// prefill's 32 768 rows turn into 340 us for 0.67 GB (RMSNorm + A8 of the hidden states).  Here a lane holds NCH 16-byte
// chunks of the row (cols = 256 NCH), the reductions are warp shuffles, nothing is staged.  No rotation, no fp32 input;
// the same scale and code functions as act_quant_row, so the codes are the same bits; with the RMSNorm the sum of squares
// is added in another order (lane-wise, then across the warp).
template <int NCH>
__global__ void __launch_bounds__(256, (NCH <= 16 ? 2 : 1)) act_quant_rows_kernel(const __grid_constant__ ActQuantParams p) {
  grid_dependency_sync();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= p.rows) return;
  const uint4* x = reinterpret_cast<const uint4*>(p.x + r * p.x_row_stride);
  uint4 xv[NCH];
#pragma unroll
  for (int c = 0; c < NCH; ++c) xv[c] = __ldcg(x + c * 32 + lane);
  if (p.norm_weight != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const __half2* h = reinterpret_cast<const __half2*>(&xv[c]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h[e]);
        ss = fmaf(f.x, f.x, ss);
        ss = fmaf(f.y, f.y, ss);
      }
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / static_cast<float>(p.cols) + p.norm_eps);
    const uint4* w = reinterpret_cast<const uint4*>(p.norm_weight);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const uint4 wv = __ldg(w + c * 32 + lane);
      __half2* h = reinterpret_cast<__half2*>(&xv[c]);
      const __half2* wh = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h[e]);
        const float2 g = __half22float2(wh[e]);
        // fp32 statistics, the normalised value rounded to fp16, then an fp16 product with the weight (act_quant_row)
        const __half a = __float2half_rn(f.x * inv), b = __float2half_rn(f.y * inv);
        h[e] = __halves2half2(__float2half_rn(__half2float(a) * g.x), __float2half_rn(__half2float(b) * g.y));
      }
      if (p.x_rot != nullptr) reinterpret_cast<uint4*>(p.x_rot + static_cast<int64_t>(r) * p.cols)[c * 32 + lane] = xv[c];
    }
  }
  float amax = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const __half2* h = reinterpret_cast<const __half2*>(&xv[c]);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __half22float2(h[e]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  amax = warp_max(amax);
  const float s = act_scale_of(amax);
  if (lane == 0) p.scale[r] = s;
  uint2* q = reinterpret_cast<uint2*>(p.q + r * p.q_row_stride);
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const __half2* h = reinterpret_cast<const __half2*>(&xv[c]);
    uint32_t w2[2] = {0u, 0u};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __half22float2(h[e]);
      w2[e >> 1] |= static_cast<uint32_t>(static_cast<uint8_t>(act_code(f.x, s))) << (16 * (e & 1));
      w2[e >> 1] |= static_cast<uint32_t>(static_cast<uint8_t>(act_code(f.y, s))) << (16 * (e & 1) + 8);
    }
    q[c * 32 + lane] = make_uint2(w2[0], w2[1]);
  }
}

// ----------------------------------------------------------------------------------------------
// Hadamard across heads + per-token quantisation (the online rotation in front of o_proj)
// ----------------------------------------------------------------------------------------------
// A row is [H][D]; every column d is transformed over its H entries (H a power of two), scale 1 / sqrt(H), fp16
// rounding, then the row is quantised like any activation.  A thread owns two adjacent columns and keeps their
// 2 H entries in registers: the butterflies need no exchange at all.
struct HeadsHadParams {
  const __half* x;
  int64_t x_row_stride;
  int8_t* q;
  int64_t q_row_stride;
  float* scale;
  __half* y;
  int32_t rows, heads, head_dim;
  float rot_scale;
};

template <int H>
__global__ void __launch_bounds__(128) heads_hadamard_quant_kernel(const __grid_constant__ HeadsHadParams p) {
  __shared__ float red[8];
  grid_dependency_sync();
  const int r = blockIdx.x, D = p.head_dim;
  const __half* x = p.x + r * p.x_row_stride;
  const int c = 2 * threadIdx.x;                  // columns c, c + 1
  const bool on = c < D;
  float e0[H], e1[H];
#pragma unroll
  for (int h = 0; h < H; ++h) {
    e0[h] = e1[h] = 0.f;
    if (on) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(x + h * D + c));
      e0[h] = f.x;
      e1[h] = f.y;
    }
  }
#pragma unroll
  for (int s = 1; s < H; s <<= 1)
#pragma unroll
    for (int h = 0; h < H; ++h)
      if ((h & s) == 0) {
        const float a0 = e0[h], b0 = e0[h + s], a1 = e1[h], b1 = e1[h + s];
        e0[h] = a0 + b0; e0[h + s] = a0 - b0;
        e1[h] = a1 + b1; e1[h + s] = a1 - b1;
      }
  float amax = 0.f;
#pragma unroll
  for (int h = 0; h < H; ++h) {
    e0[h] = __half2float(__float2half_rn(e0[h] * p.rot_scale));
    e1[h] = __half2float(__float2half_rn(e1[h] * p.rot_scale));
    amax = fmaxf(amax, fmaxf(fabsf(e0[h]), fabsf(e1[h])));
  }
  amax = block_max(amax, red);
  const float s = act_scale_of(amax);
  if (threadIdx.x == 0) p.scale[r] = s;
  if (!on) return;
  int8_t* q = p.q + r * p.q_row_stride;
#pragma unroll
  for (int h = 0; h < H; ++h) {
    const uint16_t packed = static_cast<uint16_t>(static_cast<uint8_t>(act_code(e0[h], s))) |
                            (static_cast<uint16_t>(static_cast<uint8_t>(act_code(e1[h], s))) << 8);
    *reinterpret_cast<uint16_t*>(q + h * D + c) = packed;
    if (p.y != nullptr)
      *reinterpret_cast<__half2*>(p.y + static_cast<int64_t>(r) * H * D + h * D + c) = __floats2half2_rn(e0[h], e1[h]);
  }
}

// The same for a head count that is not a power of two (H = K, e.g. 28): y = fp16(fp16(had_K x) / sqrt(H)), the
// reference's fp16 matmul followed by its fp16-tensor-by-scalar division.  A thread owns two adjacent columns,
// keeps their 2 H inputs in registers, reads had_K (staged as +-1 floats) from shared memory, and parks the fp16
// results in shared memory until the row's scale is known.
constexpr int kHeadsMax = 64;

__global__ void __launch_bounds__(128) heads_hadk_quant_kernel(const __grid_constant__ HeadsHadParams p, const __half* had_K) {
  extern __shared__ __align__(16) uint8_t hh_smem[];
  float* hk = reinterpret_cast<float*>(hh_smem);                       // [H][H]
  __half2* ys = reinterpret_cast<__half2*>(hk + p.heads * p.heads);    // [H][D / 2]
  __shared__ float red[8];
  grid_dependency_sync();
  const int r = blockIdx.x, D = p.head_dim, H = p.heads;
  for (int i = threadIdx.x; i < H * H; i += blockDim.x) hk[i] = __half2float(had_K[i]);
  const __half* x = p.x + r * p.x_row_stride;
  const int c = 2 * threadIdx.x;
  const bool on = c < D;
  float e0[kHeadsMax], e1[kHeadsMax];
#pragma unroll
  for (int h = 0; h < kHeadsMax; ++h) {
    e0[h] = e1[h] = 0.f;
    if (on && h < H) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(x + h * D + c));
      e0[h] = f.x;
      e1[h] = f.y;
    }
  }
  __syncthreads();
  float amax = 0.f;
  const float root = sqrtf(static_cast<float>(H));
  if (on) {
    for (int o = 0; o < H; ++o) {
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int h = 0; h < kHeadsMax; ++h)
        if (h < H) {
          const float w = hk[o * H + h];
          a0 = fmaf(w, e0[h], a0);
          a1 = fmaf(w, e1[h], a1);
        }
      const float y0 = __half2float(__float2half_rn(__fdiv_rn(__half2float(__float2half_rn(a0)), root)));
      const float y1 = __half2float(__float2half_rn(__fdiv_rn(__half2float(__float2half_rn(a1)), root)));
      amax = fmaxf(amax, fmaxf(fabsf(y0), fabsf(y1)));
      ys[o * (D >> 1) + threadIdx.x] = __floats2half2_rn(y0, y1);
    }
  }
  amax = block_max(amax, red);
  const float s = act_scale_of(amax);
  if (threadIdx.x == 0) p.scale[r] = s;
  if (!on) return;
  int8_t* q = p.q + r * p.q_row_stride;
  for (int o = 0; o < H; ++o) {
    const __half2 v = ys[o * (D >> 1) + threadIdx.x];               // written by this thread
    const float2 f = __half22float2(v);
    const uint16_t packed = static_cast<uint16_t>(static_cast<uint8_t>(act_code(f.x, s))) |
                            (static_cast<uint16_t>(static_cast<uint8_t>(act_code(f.y, s))) << 8);
    *reinterpret_cast<uint16_t*>(q + o * D + c) = packed;
    if (p.y != nullptr) *reinterpret_cast<__half2*>(p.y + static_cast<int64_t>(r) * H * D + o * D + c) = v;
  }
}

// ----------------------------------------------------------------------------------------------
// (H_K kron H_nb) rotation + per-token quantisation: a thread-block cluster per token
// ----------------------------------------------------------------------------------------------
// y[k', j] = sum_k had_K[k', k] * fwht(x[k, :])[j] / sqrt(cols).  The blocks of a cluster split the nb
// columns j (8 per MMA tile); each block rotates all K power-of-two blocks with warp shuffles (cheap),
// keeps the columns it owns, multiplies by had_K on the fp16 tensor cores (A fragments come pre-packed in
// fragment order, so a lane loads 16 bytes per MMA and every had_K element is read once per block), and
// the row's absmax is exchanged through distributed shared memory between two cluster barriers.
// Pack had_K [K, K] (fp16, row-major) into A-fragment order, zero padded to multiples of 16.
__global__ void hadamard_pack_kernel(const __half* had_K, int K, int Kp, uint4* out) {
  const int tiles = Kp >> 4;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= tiles * tiles * 32) return;
  const int lane = idx & 31, kt = (idx >> 5) % tiles, mt = (idx >> 5) / tiles;
  const int g = lane >> 2, t = lane & 3;
  auto at = [&](int r, int c) -> uint32_t {
    const __half lo = (r < K && c < K) ? had_K[r * K + c] : __float2half_rn(0.f);
    const __half hi = (r < K && c + 1 < K) ? had_K[r * K + c + 1] : __float2half_rn(0.f);
    return static_cast<uint32_t>(__half_as_ushort(lo)) | (static_cast<uint32_t>(__half_as_ushort(hi)) << 16);
  };
  const int r0 = mt * 16 + g, c0 = kt * 16 + 2 * t;
  out[idx] = make_uint4(at(r0, c0), at(r0 + 8, c0), at(r0, c0 + 8), at(r0 + 8, c0 + 8));
}

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Read a float from the same shared-memory offset in block `rank` of the cluster.
__device__ __forceinline__ float cluster_peer_float(const float* local, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

constexpr int kHadMaxTilesPerWarp = 2;     // m tiles a warp keeps in registers: Kp <= 256 with 8 warps
// 8-column tiles per block (template parameter NTP): 2 covers nb <= 128 with a cluster of 8 blocks per token, the
// latency-oriented form of decode batches; 8 lets one block (nb <= 64) or two (nb = 128) take a whole token, the
// throughput-oriented form of prefill batches, where tokens outnumber the SMs by far.

template <int kHadMaxNtilePer>
__global__ void __launch_bounds__(256) hadamard_quant_kernel(const __grid_constant__ HadQuantParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __half* Tt = reinterpret_cast<__half*>(smem_raw);          // [ntile_per * 8][ld]: my columns of the rotated blocks
  __half* xs = Tt + p.ntile_per * 8 * p.ld;                  // [cols]: the token's row, staged with wide loads
  __shared__ float red[8];
  grid_dependency_sync();
  __shared__ float my_max;
  const int crank = static_cast<int>(cluster_rank());
  const int r = blockIdx.x / p.cluster;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = p.K, nb = p.nb, ld = p.ld;
  const int col0 = crank * p.ntile_per * 8, ncols = p.ntile_per * 8;     // columns [col0, col0 + ncols) are mine

  for (int i = threadIdx.x; i < ncols * ld; i += blockDim.x) Tt[i] = __float2half_rn(0.f);
  {
    const __half* xg = p.x + r * p.x_row_stride;
    if (p.x_vec16) {
      // only the blocks this cluster member rotates: k = crank, crank + cluster, ...
      const int per_blk = nb >> 3, nmine = (K - crank + p.cluster - 1) / p.cluster;
      for (int i = threadIdx.x; i < nmine * per_blk; i += blockDim.x) {
        const int kb = i / per_blk, c = i - kb * per_blk;
        const int o = (((crank + kb * p.cluster) * nb) >> 3) + c;
        reinterpret_cast<uint4*>(xs)[o] = __ldg(reinterpret_cast<const uint4*>(xg) + o);
      }
    } else {
      for (int i = threadIdx.x; i < p.cols; i += blockDim.x) xs[i] = xg[i];
    }
  }
  cluster_barrier();        // every block's Tt is cleared before any peer writes into it

  // ---- power-of-two part: each warp rotates whole blocks of nb entries; a lane holds entries lane + 32 i ----
  const __half* x = xs;
  const int per = nb >= 32 ? (nb >> 5) : 1;         // 1, 2 or 4 entries per lane (lanes >= nb idle when nb < 32)
  const bool lane_on = lane < nb;
  // Block c of the cluster rotates the blocks k = c, c + cluster, ... and sends each peer the columns it owns
  // (distributed shared memory); a cluster barrier then makes every block's Tt complete.
  for (int k = crank + warp * p.cluster; k < K; k += (blockDim.x >> 5) * p.cluster) {
    float e[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) e[i] = (i < per && lane_on) ? __half2float(x[k * nb + i * 32 + lane]) : 0.f;
    // strides 1..16 cross lanes; the entry with the stride bit clear gets a + b, the other a - b
#pragma unroll
    for (int h = 1; h < 32; h <<= 1) {
      if (h >= nb) break;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (i < per) {
          const float o = __shfl_xor_sync(0xffffffffu, e[i], h);
          e[i] = (lane & h) ? o - e[i] : e[i] + o;
        }
      }
    }
    if (per >= 2) {                        // stride 32
      const float a0 = e[0], a1 = e[1];
      e[0] = a0 + a1; e[1] = a0 - a1;
      if (per == 4) { const float b0 = e[2], b1 = e[3]; e[2] = b0 + b1; e[3] = b0 - b1; }
    }
    if (per == 4) {                        // stride 64
      const float a0 = e[0], a2 = e[2], a1 = e[1], a3 = e[3];
      e[0] = a0 + a2; e[2] = a0 - a2; e[1] = a1 + a3; e[3] = a1 - a3;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int j = i * 32 + lane;
      if (i < per && lane_on) {
        const int owner = j / ncols, local = j - owner * ncols;
        const __half hv = __float2half_rn(e[i] * p.rot_scale);
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(Tt + local * ld + k)), "r"(owner));
        asm volatile("st.shared::cluster.b16 [%0], %1;" ::"r"(remote), "h"(__half_as_ushort(hv)) : "memory");
      }
    }
  }
  cluster_barrier();

  // ---- had_K part on the tensor cores: warp w owns m tiles w, w + 8; results stay in registers ----
  const int g = lane >> 2, t = lane & 3;
  const int tiles = p.Kp >> 4;
  float d[kHadMaxTilesPerWarp][kHadMaxNtilePer][4];
  float amax = 0.f;
#pragma unroll
  for (int mi = 0; mi < kHadMaxTilesPerWarp; ++mi) {
    const int mt = warp + mi * 8;
#pragma unroll
    for (int ni = 0; ni < kHadMaxNtilePer; ++ni)
#pragma unroll
      for (int c = 0; c < 4; ++c) d[mi][ni][c] = 0.f;
    if (mt < tiles) {
      const uint4* ap = p.packed + (static_cast<int64_t>(mt) * tiles) * 32 + lane;
      // decode form: every k tile of this m tile requested together (one memory round trip); prefill form: one
      // at a time (they stay in L1 for the next tokens of the SM, and the registers hold more accumulators instead)
      constexpr int kAhead = kHadMaxNtilePer <= 2 ? 16 : 1;
      uint4 a[kAhead];
      if (kAhead == 16) {
#pragma unroll
        for (int kt = 0; kt < kAhead; ++kt) a[kt] = kt < tiles ? __ldg(ap + kt * 32) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int kt = 0; kt < 16; ++kt) {
        if (kt < tiles) {
          if (kAhead == 1) a[0] = __ldg(ap + kt * 32);
          const uint4 af = a[kAhead == 16 ? kt : 0];
#pragma unroll
          for (int ni = 0; ni < kHadMaxNtilePer; ++ni) {
            if (ni < p.ntile_per) {
              const __half* brow = Tt + (ni * 8 + g) * ld + kt * 16 + 2 * t;
              const uint32_t b0 = *reinterpret_cast<const uint32_t*>(brow);
              const uint32_t b1 = *reinterpret_cast<const uint32_t*>(brow + 8);
              mma_f16_16x8x16(d[mi][ni], af.x, af.y, af.z, af.w, b0, b1);
            }
          }
        }
      }
#pragma unroll
      for (int ni = 0; ni < kHadMaxNtilePer; ++ni)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          d[mi][ni][c] = __half2float(__float2half_rn(d[mi][ni][c]));        // the reference's fp16 result
          const int row = mt * 16 + g + 8 * (c >> 1);
          if (ni < p.ntile_per && row < K) amax = fmaxf(amax, fabsf(d[mi][ni][c]));
        }
    }
  }
  amax = block_max(amax, red);
  if (threadIdx.x == 0) my_max = amax;
  cluster_barrier();
  float row_max = 0.f;
  for (int c = 0; c < p.cluster; ++c) row_max = fmaxf(row_max, cluster_peer_float(&my_max, c));
  cluster_barrier();                        // nobody leaves while a peer may still read its my_max
  const float s = act_scale_of(row_max);
  if (crank == 0 && threadIdx.x == 0) p.scale[r] = s;

  // ---- quantise and store my columns ----
  int8_t* q = p.q + r * p.q_row_stride;
#pragma unroll
  for (int mi = 0; mi < kHadMaxTilesPerWarp; ++mi) {
    const int mt = warp + mi * 8;
    if (mt >= tiles) continue;
#pragma unroll
    for (int ni = 0; ni < kHadMaxNtilePer; ++ni) {
      if (ni >= p.ntile_per) continue;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int row = mt * 16 + g + 8 * hf;
        if (row >= K) continue;
        const int col = col0 + ni * 8 + 2 * t;
        const float v0 = d[mi][ni][2 * hf], v1 = d[mi][ni][2 * hf + 1];
        const int64_t o = static_cast<int64_t>(row) * nb + col;
        const uint16_t packed = static_cast<uint16_t>(static_cast<uint8_t>(act_code(v0, s))) |
                                (static_cast<uint16_t>(static_cast<uint8_t>(act_code(v1, s))) << 8);
        *reinterpret_cast<uint16_t*>(q + o) = packed;
        if (p.y != nullptr) {
          __half* yo = p.y + static_cast<int64_t>(r) * p.cols + o;
          *reinterpret_cast<__half2*>(yo) = __floats2half2_rn(v0, v1);
        }
      }
    }
  }
}

// ----------------------------------------------------------------------------------------------
// The same rotation + quantisation for many tokens (prefill): one block per token, built for throughput
// ----------------------------------------------------------------------------------------------
// nb = 64.  A warp rotates four 64-entry blocks at a time: a lane holds eight consecutive entries of one block
// (one 16-byte load), does the strides 1, 2, 4 in registers and the strides 8, 16, 32 with three rounds of
// shuffles: the same additions in the same order as the butterfly loop.  The had_K product and the fp16
// roundings are those of hadamard_quant_kernel; the int8 codes are staged in shared memory and leave as
// 16-byte stores.
constexpr int kRowsNb = 64;

__global__ void __launch_bounds__(512) hadamard_quant_rows_kernel(const __grid_constant__ HadQuantParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __shared__ float red[16];
  const int K = p.K, ld = p.ld;                              // ld = Kp + 10 halves here
  __half* Tt = reinterpret_cast<__half*>(smem_raw);           // [64][ld]: column j of every rotated block
  uint8_t* Tq = smem_raw;                                     // [Kp][80] int8 codes, after the product (same bytes)
  const int r = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nw = blockDim.x >> 5;                              // one warp per 16-row tile of had_K: Kp / 16 warps
  const __half* xg = p.x + r * p.x_row_stride;

  // columns K .. Kp of Tt meet zero entries of had_K in the product: they must hold numbers, not leftovers
  for (int i = threadIdx.x; i < kRowsNb * (p.Kp - K); i += blockDim.x) {
    const int j = i / (p.Kp - K), k = K + (i - j * (p.Kp - K));
    Tt[j * ld + k] = __float2half_rn(0.f);
  }
  {
    const int sub = lane & 7, quad = lane >> 3;
    constexpr int kMaxIter = 4;                     // K / 4 groups of four blocks over Kp / 16 warps: at most 4 each
    uint4 xv[kMaxIter];
#pragma unroll
    for (int it = 0; it < kMaxIter; ++it) {         // every load of this lane in flight before the first use
      const int k = (warp + it * nw) * 4 + quad;
      xv[it] = make_uint4(0u, 0u, 0u, 0u);
      if (k < K) xv[it] = __ldg(reinterpret_cast<const uint4*>(xg + k * kRowsNb) + sub);
    }
#pragma unroll
    for (int it = 0; it < kMaxIter; ++it) {
      const int k = (warp + it * nw) * 4 + quad;
      if ((warp + it * nw) * 4 >= K) break;
      float e[8];
      {
        const __half2* h2 = reinterpret_cast<const __half2*>(&xv[it]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __half22float2(h2[i]);
          e[2 * i] = f.x;
          e[2 * i + 1] = f.y;
        }
      }
#pragma unroll
      for (int h = 1; h < 8; h <<= 1)
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if ((i & h) == 0) {
            const float a = e[i], b = e[i + h];
            e[i] = a + b;
            e[i + h] = a - b;
          }
#pragma unroll
      for (int h = 1; h < 8; h <<= 1)              // strides 8, 16, 32 <-> lane bits 0, 1, 2
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float o = __shfl_xor_sync(0xffffffffu, e[i], h);
          e[i] = (sub & h) ? o - e[i] : e[i] + o;
        }
      if (k < K) {
#pragma unroll
        for (int i = 0; i < 8; ++i) Tt[(sub * 8 + i) * ld + k] = __float2half_rn(e[i] * p.rot_scale);
      }
    }
  }
  __syncthreads();

  // ---- had_K product: warp w owns m tile w ----
  const int g = lane >> 2, t = lane & 3;
  const int tiles = p.Kp >> 4;
  const int mt = warp;
  float d[8][4];
  float amax = 0.f;
#pragma unroll
  for (int ni = 0; ni < 8; ++ni)
#pragma unroll
    for (int c = 0; c < 4; ++c) d[ni][c] = 0.f;
  {
    const uint4* ap = p.packed + (static_cast<int64_t>(mt) * tiles) * 32 + lane;
    uint4 af[4];                                 // four fragments of had_K in flight
#pragma unroll
    for (int u = 0; u < 4; ++u) af[u] = u < tiles ? __ldg(ap + u * 32) : make_uint4(0u, 0u, 0u, 0u);
    for (int kt0 = 0; kt0 < tiles; kt0 += 4) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int kt = kt0 + u;
        if (kt < tiles) {
          const uint4 a4 = af[u];
          if (kt + 4 < tiles) af[u] = __ldg(ap + (kt + 4) * 32);
#pragma unroll
          for (int ni = 0; ni < 8; ++ni) {
            const __half* brow = Tt + (ni * 8 + g) * ld + kt * 16 + 2 * t;
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(brow);
            const uint32_t b1 = *reinterpret_cast<const uint32_t*>(brow + 8);
            mma_f16_16x8x16(d[ni], a4.x, a4.y, a4.z, a4.w, b0, b1);
          }
        }
      }
    }
#pragma unroll
    for (int ni = 0; ni < 8; ++ni)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        d[ni][c] = __half2float(__float2half_rn(d[ni][c]));        // the reference's fp16 result
        if (mt * 16 + g + 8 * (c >> 1) < K) amax = fmaxf(amax, fabsf(d[ni][c]));
      }
  }
  amax = block_max(amax, red);                // its barriers also end every warp's reads of Tt
  const float s = act_scale_of(amax);
  if (threadIdx.x == 0) p.scale[r] = s;

  // ---- quantise into shared memory (rows of 80 bytes: conflict-free 2-byte stores, 16-byte aligned rows) ----
#pragma unroll
  for (int ni = 0; ni < 8; ++ni)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int row = mt * 16 + g + 8 * hf;
      const uint16_t packed = static_cast<uint16_t>(static_cast<uint8_t>(act_code(d[ni][2 * hf], s))) |
                              (static_cast<uint16_t>(static_cast<uint8_t>(act_code(d[ni][2 * hf + 1], s))) << 8);
      *reinterpret_cast<uint16_t*>(Tq + row * 80 + ni * 8 + 2 * t) = packed;
    }
  __syncthreads();
  int8_t* q = p.q + r * p.q_row_stride;
  if ((reinterpret_cast<uintptr_t>(q) & 15) == 0) {
    for (int i = threadIdx.x; i < K * 4; i += blockDim.x) {
      const int row = i >> 2, c = i & 3;
      reinterpret_cast<uint4*>(q)[i] = *reinterpret_cast<const uint4*>(Tq + row * 80 + c * 16);
    }
  } else {
    for (int i = threadIdx.x; i < K * kRowsNb; i += blockDim.x) q[i] = static_cast<int8_t>(Tq[(i >> 6) * 80 + (i & 63)]);
  }
}

// ----------------------------------------------------------------------------------------------
// weight-streaming W8A8 product
// ----------------------------------------------------------------------------------------------
constexpr int kGemvWarps = 8;

// NT = token tiles of 8 (tokens beyond m read as zero); DUAL = a gate/up pair of matrices in one pass;
// SPLIT_B = the second matrix has its own activations.
// MIX = the all-fp32 epilogue conventions and the per-token maxima (their own instantiations: the other products keep
// their register budget, which for 17..32 tokens is capped so that three blocks share an SM -- 78 -> 68 us per FFN call).
template <int NT, bool DUAL, bool SPLIT_B, bool MIX>
__global__ void __launch_bounds__(kGemvWarps * 32, (NT == 4 && !MIX) ? 3 : 0) w8a8_gemv_kernel(const __grid_constant__ GemvParams p) {
  extern __shared__ __align__(16) int red[];      // [warp][matrix][NT][4][32]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * 16;
  constexpr int NMAT = DUAL ? 2 : 1;
  grid_dependency_release();
  if (p.prefetch) {
    // The weights do not depend on the kernel before this one: while that kernel drains, ask for this block's 16
    // rows (of each matrix) line by line, so that the loads after the wait find them in L2.
    const int lines = (p.k + 127) >> 7;
    for (int i = threadIdx.x; i < 16 * lines; i += blockDim.x) {
      const int r = i / lines, c = i - r * lines;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(p.w + (row0 + r) * p.w_row_stride + c * 128));
      if (DUAL) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.w2 + (row0 + r) * p.w2_row_stride + c * 128));
    }
  }
  grid_dependency_wait();

  int acc[NMAT][NT][4];
#pragma unroll
  for (int mtx = 0; mtx < NMAT; ++mtx)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[mtx][j][c] = 0;

  // K is cut into spans of 64 bytes (a lane's 16 bytes per row cover two 32-wide MMA steps).  Runs of kUnroll
  // spans are dealt to the warps round-robin, so at any moment the block reads one contiguous stretch of each
  // of its rows (8 warps x kUnroll x 64 bytes) instead of eight distant ones: DRAM pages stay open.
  const int spans = p.k >> 6;
  const int8_t* wr0 = p.w + (row0 + g) * p.w_row_stride + 16 * t;
  const int8_t* wr1 = wr0 + 8 * p.w_row_stride;
  const int8_t* w2r0 = DUAL ? p.w2 + (row0 + g) * p.w2_row_stride + 16 * t : nullptr;
  const int8_t* w2r1 = DUAL ? w2r0 + 8 * p.w2_row_stride : nullptr;

  constexpr int kUnroll = NT <= 2 ? 4 : (NT == 4 ? 2 : 1);     // spans whose loads are issued together
  auto span = [&](int ko, bool on) {
    // `on` is false only for the lanes past the end of a last, partial span (K a multiple of 16, not of 64)
    uint4 x0 = make_uint4(0u, 0u, 0u, 0u), x1 = x0, y0 = x0, y1 = x0;
    if (on) {
      x0 = ldg_u4(wr0 + ko);
      x1 = ldg_u4(wr1 + ko);
      if (DUAL) {
        y0 = ldg_u4(w2r0 + ko);
        y1 = ldg_u4(w2r1 + ko);
      }
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int tok = j * 8 + g;
      uint4 bv = make_uint4(0u, 0u, 0u, 0u);
      if (on && tok < p.m) bv = ldg_u4(p.a + tok * p.a_row_stride + ko + 16 * t);
      // the MMA's k index is a permutation of the 32 columns that A and B share: k 4t..4t+3 <-> the first
      // four of a lane's bytes, k 16+4t.. <-> the next four
      mma_s8(acc[0][j], x0.x, x1.x, x0.y, x1.y, bv.x, bv.y);
      mma_s8(acc[0][j], x0.z, x1.z, x0.w, x1.w, bv.z, bv.w);
      if (DUAL) {
        uint4 bw = bv;
        if (SPLIT_B) {
          bw = make_uint4(0u, 0u, 0u, 0u);
          if (on && tok < p.m) bw = ldg_u4(p.a2 + tok * p.a2_row_stride + ko + 16 * t);
        }
        mma_s8(acc[NMAT - 1][j], y0.x, y1.x, y0.y, y1.y, bw.x, bw.y);
        mma_s8(acc[NMAT - 1][j], y0.z, y1.z, y0.w, y1.w, bw.z, bw.w);
      }
    }
  };
  if (spans >= kGemvWarps * kUnroll) {
    for (int s0 = warp * kUnroll; s0 < spans; s0 += kGemvWarps * kUnroll) {
      if (s0 + kUnroll <= spans) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) span((s0 + u) * 64, true);
      } else {
        for (int s = s0; s < spans; ++s) span(s * 64, true);
      }
    }
  } else {                                   // short K: single spans, so that every warp gets some
    for (int s = warp; s < spans; s += kGemvWarps) span(s * 64, true);
  }
  if ((p.k & 63) != 0 && warp == kGemvWarps - 1) span(spans * 64, 16 * t < (p.k & 63));

  // ---- sum the warps' shares ----
  int* mine = red + warp * (NMAT * NT * 4 * 32);
#pragma unroll
  for (int mtx = 0; mtx < NMAT; ++mtx)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) mine[((mtx * NT + j) * 4 + c) * 32 + lane] = acc[mtx][j][c];
  __syncthreads();

  // element e of a matrix: (j, c, lane) -> row = g + 8 (c >> 1), token = 8 j + 2 t + (c & 1)
  for (int e = threadIdx.x; e < NT * 4 * 32; e += blockDim.x) {
    const int el = e & 31, c = (e >> 5) & 3, j = e >> 7;
    const int row = row0 + (el >> 2) + 8 * (c >> 1);
    const int tok = j * 8 + 2 * (el & 3) + (c & 1);
    int sum0 = 0, sum1 = 0;
#pragma unroll
    for (int wi = 0; wi < kGemvWarps; ++wi) {
      sum0 += red[wi * (NMAT * NT * 4 * 32) + e];
      if (DUAL) sum1 += red[wi * (NMAT * NT * 4 * 32) + NT * 4 * 32 + e];
    }
    float av = 0.f;
    if (tok < p.m) av = gemv_store<DUAL, SPLIT_B, MIX>(p, tok, row, sum0, sum1);
    if (MIX && p.row_absmax != nullptr) {
      // the eight lanes that share (el & 3) hold one token's values of eight channels (e >> 5 is uniform in a warp)
      av = fmaxf(av, __shfl_xor_sync(0xffffffffu, av, 4));
      av = fmaxf(av, __shfl_xor_sync(0xffffffffu, av, 8));
      av = fmaxf(av, __shfl_xor_sync(0xffffffffu, av, 16));
      if (el < 4 && tok < p.m)
        atomicMax(p.row_absmax + tok * p.row_absmax_stride + (row0 >= p.absmax_split ? 1 : 0), __float_as_uint(av));
    }
  }
}

// ----------------------------------------------------------------------------------------------
// host
// ----------------------------------------------------------------------------------------------
static bool is_pow2(int n) { return n > 0 && (n & (n - 1)) == 0; }

template <int NT, bool DUAL, bool SPLIT_B, bool MIX>
static int launch_gemv(const GemvParams& p, cudaStream_t st) {
  const int smem = kGemvWarps * (DUAL ? 2 : 1) * NT * 4 * 32 * 4;
  auto kern = w8a8_gemv_kernel<NT, DUAL, SPLIT_B, MIX>;
  if (smem > 48 * 1024) LSVD_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem));
  LSVD_CUDA_TRY(launch_chained(kern, dim3(p.n / 16), dim3(kGemvWarps * 32), smem, st, 1, p.prefetch != 0, p));
  return LSVD_OK;
}

template <int NT, bool MIX>
static int launch_gemv_form(const GemvParams& p, bool dual, bool split, cudaStream_t st) {
  if (!dual) return launch_gemv<NT, false, false, MIX>(p, st);
  if (split) return launch_gemv<NT, true, true, MIX>(p, st);
  return launch_gemv<NT, true, false, MIX>(p, st);
}

template <int NT>
static int launch_gemv_nt(const GemvParams& p, bool dual, bool split, cudaStream_t st) {
  const bool mix = p.epilogue == 2 || p.row_absmax != nullptr;
  return mix ? launch_gemv_form<NT, true>(p, dual, split, st) : launch_gemv_form<NT, false>(p, dual, split, st);
}

}  // namespace lsvd

namespace lsvd {
__global__ void dequant_residual_kernel(const int32_t* acc, const float* a_scale, const float* w_scale, const __half* residual,
                                        int64_t res_stride, __half* out, int64_t out_stride, int m, int n) {
  grid_dependency_sync();
  const int64_t total = static_cast<int64_t>(m) * n;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int tok = static_cast<int>(i / n), ch = static_cast<int>(i - static_cast<int64_t>(tok) * n);
    __half v = __float2half_rn((static_cast<float>(acc[i]) * a_scale[tok]) * w_scale[ch]);
    if (residual != nullptr) v = __float2half_rn(__half2float(v) + __half2float(residual[tok * res_stride + ch]));
    out[tok * out_stride + ch] = v;
  }
}
}  // namespace lsvd

extern "C" int lsvd_dequant_residual(const int32_t* acc, const float* a_scale, const float* w_scale, const void* residual,
                                     int64_t residual_row_stride, void* out, int64_t out_row_stride, int32_t m, int32_t n, void* stream) {
  using namespace lsvd;
  if (!acc || !a_scale || !w_scale || !out || m <= 0 || n <= 0) return LSVD_ERR_INVALID_ARG;
  const int64_t total = static_cast<int64_t>(m) * n;
  const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 4 * std::max(1, device_sm_count())));
  LSVD_CUDA_TRY(launch_chained(dequant_residual_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream), 1, false, acc,
                               a_scale, w_scale, static_cast<const __half*>(residual), residual_row_stride, static_cast<__half*>(out),
                               out_row_stride, static_cast<int>(m), static_cast<int>(n)));
  return LSVD_OK;
}

extern "C" int lsvd_act_quant(const lsvd_act_quant_args* a, void* stream) {
  using namespace lsvd;
  if (a == nullptr || a->rows < 0 || a->cols <= 0 || a->cols > 16384) return LSVD_ERR_INVALID_ARG;
  if (a->rows == 0) return LSVD_OK;
  if ((!a->x && !a->x_f32) || !a->q || !a->scale) return LSVD_ERR_INVALID_ARG;
  if (a->x_f32 != nullptr && (a->sign != nullptr || a->fwht != 0)) return LSVD_ERR_UNSUPPORTED;
  // the fp32 rows are read four entries at a time when cols allows it: 16-byte aligned rows (8 for the fp16 companions)
  if (a->x_f32 != nullptr && (a->cols % 4) == 0 &&
      (!aligned(a->x_f32, 16) || (a->add != nullptr && !aligned(a->add, 8)) || (a->sum_out != nullptr && !aligned(a->sum_out, 8))))
    return LSVD_ERR_INVALID_ARG;
  const bool rotate = a->sign != nullptr || a->fwht != 0;
  if (rotate && !is_pow2(a->cols)) return LSVD_ERR_INVALID_ARG;
  ActQuantParams p{};
  p.x = static_cast<const __half*>(a->x);
  p.x_row_stride = a->x_row_stride;
  p.sign = static_cast<const __half*>(a->sign);
  p.norm_weight = static_cast<const __half*>(a->norm_weight);
  p.norm_eps = a->norm_eps;
  if (p.norm_weight != nullptr && a->sign != nullptr) return LSVD_ERR_UNSUPPORTED;
  p.q = a->q;
  p.q_row_stride = a->q_row_stride;
  p.scale = a->scale;
  p.x_rot = static_cast<__half*>(a->x_rot);
  p.rows = a->rows;
  p.cols = a->cols;
  p.rotate = rotate ? 1 : 0;
  p.rot_scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(a->cols)));
  p.x32 = a->x_f32;
  p.add16 = static_cast<const __half*>(a->add);
  p.sum_out = static_cast<__half*>(a->sum_out);
  p.fake = static_cast<__half*>(a->fake);
  p.vec8 = ((a->cols % 8) == 0 && aligned(a->x, 16) && (a->x_row_stride % 8) == 0 && aligned(a->q, 8) &&
            (a->q_row_stride % 8) == 0 && (a->sign == nullptr || aligned(a->sign, 16))) ? 1 : 0;
  if (rotate && a->cols == 4096 && p.vec8 && p.norm_weight == nullptr && p.fake == nullptr && aligned(a->q, 16) && (a->q_row_stride % 16) == 0 &&
      (p.x_rot == nullptr || aligned(p.x_rot, 16))) {
    LSVD_CUDA_TRY(launch_chained(act_quant_rot4096_kernel, dim3(a->rows), dim3(256), 0, static_cast<cudaStream_t>(stream), 1,
                                 false, p));
    return LSVD_OK;
  }
  // many rows of a width the warp-per-row kernel is built for (a prefill): no shared memory, no block barriers
  if (!rotate && a->x_f32 == nullptr && p.fake == nullptr && p.vec8 && a->rows >= 512 && (a->cols % 256) == 0 &&
      aligned(a->q, 8) && (p.x_rot == nullptr || aligned(p.x_rot, 16)) &&
      (p.norm_weight == nullptr || aligned(p.norm_weight, 16))) {
    void (*kern)(ActQuantParams) = nullptr;
    switch (a->cols / 256) {
      case 2: kern = act_quant_rows_kernel<2>; break;
      case 4: kern = act_quant_rows_kernel<4>; break;
      case 8: kern = act_quant_rows_kernel<8>; break;
      case 10: kern = act_quant_rows_kernel<10>; break;
      case 16: kern = act_quant_rows_kernel<16>; break;
      case 20: kern = act_quant_rows_kernel<20>; break;
      default: break;
    }
    if (kern != nullptr) {
      LSVD_CUDA_TRY(launch_chained(kern, dim3((a->rows + 7) / 8), dim3(256), 0, static_cast<cudaStream_t>(stream), 1, false, p));
      return LSVD_OK;
    }
  }
  const int smem = a->cols * 4;
  if (smem > 48 * 1024) LSVD_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(act_quant_kernel), smem));
  LSVD_CUDA_TRY(launch_chained(act_quant_kernel, dim3(a->rows), dim3(256), smem, static_cast<cudaStream_t>(stream), 1, false, p));
  return LSVD_OK;
}

extern "C" int lsvd_heads_hadamard_quant(const lsvd_heads_hadamard_quant_args* a, void* stream) {
  using namespace lsvd;
  if (a == nullptr || a->rows < 0 || a->heads <= 1 || a->head_dim <= 0 || (a->head_dim % 2) || a->head_dim > 256)
    return LSVD_ERR_INVALID_ARG;
  if (a->rows == 0) return LSVD_OK;
  if (!a->x || !a->q || !a->scale) return LSVD_ERR_INVALID_ARG;
  if (!aligned(a->x, 4) || (a->x_row_stride % 2) || !aligned(a->q, 2) || (a->q_row_stride % 2) || (a->y && !aligned(a->y, 4)))
    return LSVD_ERR_INVALID_ARG;
  HeadsHadParams p{};
  p.x = static_cast<const __half*>(a->x); p.x_row_stride = a->x_row_stride;
  p.q = a->q; p.q_row_stride = a->q_row_stride; p.scale = a->scale; p.y = static_cast<__half*>(a->y);
  p.rows = a->rows; p.heads = a->heads; p.head_dim = a->head_dim;
  p.rot_scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(a->heads)));
  void (*kern)(HeadsHadParams) = nullptr;
  switch (a->heads) {
    case 2: kern = heads_hadamard_quant_kernel<2>; break;
    case 4: kern = heads_hadamard_quant_kernel<4>; break;
    case 8: kern = heads_hadamard_quant_kernel<8>; break;
    case 16: kern = heads_hadamard_quant_kernel<16>; break;
    case 32: kern = heads_hadamard_quant_kernel<32>; break;
    case 64: kern = heads_hadamard_quant_kernel<64>; break;
    default: break;
  }
  if (a->had_K != nullptr) {                    // the had_K @ x form (head counts that are not a power of two)
    if (a->heads > kHeadsMax) return LSVD_ERR_UNSUPPORTED;
    const int smem = a->heads * a->heads * 4 + a->heads * a->head_dim * 2;
    if (smem > 48 * 1024) LSVD_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(heads_hadk_quant_kernel), smem));
    LSVD_CUDA_TRY(launch_chained(heads_hadk_quant_kernel, dim3(a->rows), dim3(128), smem, static_cast<cudaStream_t>(stream), 1,
                                 false, p, static_cast<const __half*>(a->had_K)));
    return LSVD_OK;
  }
  if (kern == nullptr) return LSVD_ERR_UNSUPPORTED;       // not a power of two and no had_K given
  LSVD_CUDA_TRY(launch_chained(kern, dim3(a->rows), dim3(128), 0, static_cast<cudaStream_t>(stream), 1, false, p));
  return LSVD_OK;
}

// ----------------------------------------------------------------------------------------------
// Hadamard across heads when the heads are sharded over tensor-parallel ranks
// ----------------------------------------------------------------------------------------------
// The transform is linear in its input heads: y[h', d] = s * sum_h S[h', h] x[h, d].  A rank that holds the heads
// head_ids[0..n_local) adds their terms for EVERY output head h' into an fp32 row; the sum of the ranks' rows (one
// all-reduce) is the rotated row, which lsvd_act_quant (x_f32) rounds to fp16 once and quantises.
struct HeadsHadPartialParams {
  const __half* x; int64_t x_row_stride;
  const __half* had_K;             // [heads, heads] +-1, or NULL: Sylvester signs (-1)^popcount(h' & h)
  float* out;                      // [rows, heads * head_dim]
  int32_t rows, heads, head_dim, n_local;
  float scale;
  int32_t head_ids[LSVD_MAX_HEADS];
};

__global__ void __launch_bounds__(256) heads_hadamard_partial_kernel(const __grid_constant__ HeadsHadPartialParams p) {
  const int r = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;            // output column h' * head_dim + d
  if (i >= p.heads * p.head_dim) return;
  const int ho = i / p.head_dim, d = i - ho * p.head_dim;
  const __half* x = p.x + r * p.x_row_stride + d;
  float acc = 0.f;
  for (int j = 0; j < p.n_local; ++j) {
    const int h = p.head_ids[j];
    const float v = __half2float(x[j * p.head_dim]);
    const bool neg = p.had_K != nullptr ? (__half2float(p.had_K[ho * p.heads + h]) < 0.f) : ((__popc(ho & h) & 1) != 0);
    acc += neg ? -v : v;
  }
  p.out[static_cast<int64_t>(r) * p.heads * p.head_dim + i] = acc * p.scale;
}

extern "C" int lsvd_heads_hadamard_partial(const void* x, int64_t x_row_stride, const int32_t* head_ids, int32_t n_local,
                                           int32_t heads, int32_t head_dim, const void* had_K, float* out, int32_t rows,
                                           void* stream) {
  using namespace lsvd;
  if (rows < 0 || heads <= 1 || heads > LSVD_MAX_HEADS || head_dim <= 0 || n_local < 0 || n_local > heads || head_ids == nullptr)
    return LSVD_ERR_INVALID_ARG;
  if (rows == 0) return LSVD_OK;
  if (x == nullptr || out == nullptr || rows > 65535) return LSVD_ERR_INVALID_ARG;
  if (had_K == nullptr && !is_pow2(heads)) return LSVD_ERR_UNSUPPORTED;
  HeadsHadPartialParams p{};
  p.x = static_cast<const __half*>(x); p.x_row_stride = x_row_stride;
  p.had_K = static_cast<const __half*>(had_K);
  p.out = out;
  p.rows = rows; p.heads = heads; p.head_dim = head_dim; p.n_local = n_local;
  p.scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(heads)));
  for (int j = 0; j < n_local; ++j) {
    if (head_ids[j] < 0 || head_ids[j] >= heads) return LSVD_ERR_INVALID_ARG;
    p.head_ids[j] = head_ids[j];
  }
  const int cols = heads * head_dim;
  heads_hadamard_partial_kernel<<<dim3((cols + 255) / 256, rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  LSVD_CUDA_TRY(cudaGetLastError());
  return LSVD_OK;
}

extern "C" size_t lsvd_hadamard_packed_bytes(int32_t K) {
  if (K <= 1 || K > 256) return 0;
  const size_t tiles = (static_cast<size_t>(K) + 15) / 16;
  return tiles * tiles * 32 * 16;
}

extern "C" int lsvd_hadamard_pack(const void* had_K, int32_t K, void* packed, void* stream) {
  using namespace lsvd;
  if (had_K == nullptr || packed == nullptr || K <= 1 || K > 256 || !aligned(packed, 16)) return LSVD_ERR_INVALID_ARG;
  const int Kp = (K + 15) / 16 * 16;
  const int n = (Kp / 16) * (Kp / 16) * 32;
  hadamard_pack_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(had_K), K, Kp, static_cast<uint4*>(packed));
  LSVD_CUDA_TRY(cudaGetLastError());
  return LSVD_OK;
}

extern "C" int lsvd_hadamard_quant(const lsvd_hadamard_quant_args* a, void* stream) {
  using namespace lsvd;
  if (a == nullptr || a->rows < 0 || a->cols <= 0 || a->K <= 1 || a->K > 256) return LSVD_ERR_INVALID_ARG;
  if (a->rows == 0) return LSVD_OK;
  if (!a->x || !a->had_K_packed || !a->q || !a->scale || !aligned(a->had_K_packed, 16)) return LSVD_ERR_INVALID_ARG;
  if (a->cols % a->K) return LSVD_ERR_INVALID_ARG;
  const int nb = a->cols / a->K;
  if (!is_pow2(nb) || nb < 8 || nb > 128) return LSVD_ERR_UNSUPPORTED;
  if ((a->q_row_stride % 2) || !aligned(a->q, 2) || (a->y && !aligned(a->y, 4))) return LSVD_ERR_INVALID_ARG;
  HadQuantParams p{};
  p.x = static_cast<const __half*>(a->x);
  p.x_row_stride = a->x_row_stride;
  p.packed = static_cast<const uint4*>(a->had_K_packed);
  p.q = a->q;
  p.q_row_stride = a->q_row_stride;
  p.scale = a->scale;
  p.y = static_cast<__half*>(a->y);
  p.rows = a->rows;
  p.cols = a->cols;
  p.K = a->K;
  p.nb = nb;
  p.Kp = (a->K + 15) / 16 * 16;
  p.ld = p.Kp + 8;
  const int ntiles = nb / 8;
  // Few tokens: a cluster of up to 8 blocks per token shortens the critical path.  Many tokens: one block (two
  // for nb = 128) per token keeps every SM busy without the cluster's redundant staging.
  // a cluster of 8 blocks per token stops paying once the clusters no longer fit on the GPU together
  const bool many = a->rows * 8 > 2 * std::max(1, device_sm_count());
  if (many) {
    p.cluster = ntiles <= 8 ? 1 : ntiles / 8;
  } else {
    p.cluster = ntiles < 8 ? ntiles : 8;
  }
  p.ntile_per = ntiles / p.cluster;
  p.rot_scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(a->cols)));
  const int smem = (p.ntile_per * 8 * p.ld + a->cols) * 2;
  p.x_vec16 = (aligned(a->x, 16) && (a->x_row_stride % 8) == 0 && (a->cols % 8) == 0) ? 1 : 0;
  if (many && nb == kRowsNb && a->y == nullptr && p.x_vec16 && (a->x_row_stride % 8) == 0) {
    p.ld = p.Kp + 10;
    const int smem_rows = std::max(kRowsNb * p.ld * 2, p.Kp * 80);
    if (smem_rows > 48 * 1024)
      LSVD_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(hadamard_quant_rows_kernel), smem_rows));
    LSVD_CUDA_TRY(launch_chained(hadamard_quant_rows_kernel, dim3(static_cast<unsigned>(a->rows)), dim3(p.Kp * 2), smem_rows,
                                 static_cast<cudaStream_t>(stream), 1, false, p));
    return LSVD_OK;
  }
  void (*kern)(HadQuantParams) = p.ntile_per <= 2 ? hadamard_quant_kernel<2> : hadamard_quant_kernel<8>;
  if (smem > 48 * 1024) LSVD_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem));
  LSVD_CUDA_TRY(launch_chained(kern, dim3(static_cast<unsigned>(a->rows * p.cluster)), dim3(256), smem,
                               static_cast<cudaStream_t>(stream), p.cluster, false, p));
  return LSVD_OK;
}

extern "C" int lsvd_w8a8_gemv(const lsvd_gemv_args* a, void* stream) {
  using namespace lsvd;
  if (a == nullptr || a->m <= 0 || a->m > 64 || a->n <= 0 || (a->n % 16) || a->k <= 0 || (a->k % 16))
    return LSVD_ERR_INVALID_ARG;
  if (!a->w || !a->a) return LSVD_ERR_INVALID_ARG;
  if ((a->out != nullptr || a->out_f32 != nullptr) && (!a->w_scale || !a->a_scale)) return LSVD_ERR_INVALID_ARG;
  const bool dual = a->w2 != nullptr;
  if (dual != (a->epilogue == 1 || a->epilogue == 2) || a->epilogue < 0 || a->epilogue > 2) return LSVD_ERR_INVALID_ARG;
  const bool fp32_form = a->epilogue == 2 || a->row_absmax != nullptr;     // built into the register-fed kernel only
  if (fp32_form && (a->form == 1 || a->form == 2)) return LSVD_ERR_UNSUPPORTED;
  if (a->row_absmax != nullptr && (a->out == nullptr || a->absmax_split < 0 || (a->absmax_split % 16))) return LSVD_ERR_INVALID_ARG;
  if (dual && a->out != nullptr && !a->w2_scale) return LSVD_ERR_INVALID_ARG;
  const bool split = dual && a->a2 != nullptr;
  if (split && a->out != nullptr && !a->a2_scale) return LSVD_ERR_INVALID_ARG;
  if (!aligned(a->w, 16) || (a->w_row_stride % 16) || !aligned(a->a, 16) || (a->a_row_stride % 16)) return LSVD_ERR_INVALID_ARG;
  if (dual && (!aligned(a->w2, 16) || (a->w2_row_stride % 16))) return LSVD_ERR_INVALID_ARG;
  if (split && (!aligned(a->a2, 16) || (a->a2_row_stride % 16))) return LSVD_ERR_INVALID_ARG;
  GemvParams p{};
  p.w = a->w; p.w_row_stride = a->w_row_stride; p.w_scale = a->w_scale;
  p.w2 = a->w2; p.w2_row_stride = a->w2_row_stride; p.w2_scale = a->w2_scale;
  p.a = a->a; p.a_row_stride = a->a_row_stride; p.a_scale = a->a_scale; p.a_scale_stride = a->a_scale_stride;
  p.a2 = a->a2; p.a2_row_stride = a->a2_row_stride; p.a2_scale = a->a2_scale; p.a2_scale_stride = a->a2_scale_stride;
  p.out = static_cast<__half*>(a->out); p.out_row_stride = a->out_row_stride; p.out_col = a->out_col;
  p.residual = static_cast<const __half*>(a->residual); p.residual_row_stride = a->residual_row_stride;
  p.acc_out = a->acc_out; p.acc2_out = a->acc2_out;
  p.status_word = a->status_word;
  p.m = a->m; p.n = a->n; p.k = a->k; p.epilogue = a->epilogue;
  p.row_absmax = a->row_absmax; p.row_absmax_stride = a->row_absmax_stride;
  p.absmax_split = a->absmax_split > 0 ? a->absmax_split : a->n;
  p.prefetch = (a->prefetch_weights != 0 && ffn_chain_enabled()) ? 1 : 0;
  p.out_f32 = a->out_f32;
  if (a->out_f32 != nullptr && (dual || a->form == 1 || a->form == 2)) return LSVD_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->form == 1) return a->m <= 16 ? launch_gemv_streamed(p, dual, split, st) : LSVD_ERR_UNSUPPORTED;
  if (a->form == 2) return launch_gemv_wide(p, dual, split, st);
  if (a->form != 0 && a->form != 3) return LSVD_ERR_INVALID_ARG;
  // more than 32 tokens: the form that shares the token rows between a block's warps (measured: 35.6 vs 48.9 us for the
  // 45 MB gate/up pair at 64 tokens; no gain at 32 tokens).  Its blocks split K between their warps when the matrix
  // has few channels, which is what a tensor-parallel rank's column slice looks like (a 9.8 MB latent projection slice
  // took 38 us in the register-fed form, more than the whole 39 MB matrix in this one); short reductions stay
  // register-fed.
  const int64_t weight_bytes = static_cast<int64_t>(a->n) * a->k * (dual ? 2 : 1);
  if (a->form == 0 && !fp32_form && a->out_f32 == nullptr && a->m > 32 && weight_bytes >= (4ll << 20) && a->k >= 2048)
    return launch_gemv_wide(p, dual, split, st);
  if (a->m <= 8) return launch_gemv_nt<1>(p, dual, split, st);
  if (a->m <= 16) return launch_gemv_nt<2>(p, dual, split, st);
  if (a->m <= 32) return launch_gemv_nt<4>(p, dual, split, st);
  return launch_gemv_nt<8>(p, dual, split, st);
}
