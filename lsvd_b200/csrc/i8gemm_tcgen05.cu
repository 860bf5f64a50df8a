// W8A8 GEMM for prefill and large batches on the fifth-generation tensor cores:
//   acc[m, n] = sum_k a[m, k] * w[n, k]   (int8 x int8 -> int32, exact), dequantised to fp16 in the epilogue.
//
// Persistent: one block per SM walks 128 (tokens) x 256 (channels) tiles.  Warp 0 (one elected lane) streams the
// A and B tiles with TMA (cp.async.bulk.tensor, 128-byte swizzle, every block loads its own tiles) into a four-stage shared-memory
// ring; warp 1 (one elected lane) issues tcgen05.mma kind::i8 (M 128, N 256, K 32 per instruction) into one of
// two accumulators in tensor memory (2 x 256 columns of 32 bits, allocated by warp 1); tcgen05.commit hands each
// ring stage back to the producer and, after a tile's last MMA, hands the accumulator to the eight epilogue warps,
// which read it with tcgen05.ld (lane = token row, 32 columns at a time), apply token and channel scales (and
// SiLU gating / a residual) and store fp16 while the MMAs of the next tile fill the other accumulator.  Every
// mbarrier wait is bounded; a wait that gives up sets the status word and the block still releases its tensor
// memory.
//
// Replaces the Triton tl.dot int8 kernels of the reference for M >> 64
// (kernels/layer_bench/ffn_kernel/mix_ffn_kernel.py:410-500, 903-1021, 1152-1338) and produces the same values as
// the decode-sized lsvd_w8a8_gemv.
#include <algorithm>
#include <cmath>

#include "common.cuh"
#include "tc5.cuh"
#include "tma.cuh"

namespace lsvd {

constexpr int kBM = 128, kBN = 256, kBK = 128, kMaxStages = 4;
constexpr int kATile = kBM * kBK, kBTile = kBN * kBK;                     // bytes (int8)
constexpr int kEpiWarps = 8;                                               // two per quarter of the TMEM lanes
constexpr int kGemmThreads = 64 + kEpiWarps * 32;                          // producer, MMA issuer, epilogue warps
constexpr int kGemmSmem = kMaxStages * (kATile + kBTile) + 1024 /*alignment slack*/ + 256 /*barriers*/ + 2 * kBN * 4 /*scales*/;
constexpr uint32_t kTmemCols = 512;                                        // two accumulators of kBN columns

struct GemmParams {
  const float* a_scale;
  int64_t a_scale_stride;
  const float* w_scale;
  const float* w2_scale;
  __half* out;
  int64_t out_row_stride;
  int32_t out_col;
  const __half* gate;        // epilogue of a lone "up" product: out = fp16(fp16(silu(gate)) * value)
  int64_t gate_row_stride;
  int32_t gate_col;
  const __half* residual;    // fp16 add of the fp16 result and the residual (single product)
  int64_t residual_row_stride;
  int32_t* acc_out;          // optional raw accumulators [m, n] (single-matrix form only)
  int32_t* status_word;
  int32_t m, n, k, dual;     // dual: the B tile is 128 gate channels followed by their 128 up channels
  int32_t split;             // dual with separate activations for the up half: a second A tile per stage, two N = 128 MMAs
  const float* a2_scale;
  int64_t a2_scale_stride;
  int32_t m_tiles, n_tiles;
};

// Instruction descriptor: D = S32 (2 at bit 4), A = S8 (1 at bit 7), B = S8 (1 at bit 10), both K-major,
// N >> 3 at bit 17, M >> 4 at bit 24.
constexpr uint32_t kIdescHalf = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>((kBN / 2) >> 3) << 17) |
                                (static_cast<uint32_t>(kBM >> 4) << 24);
constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kBN >> 3) << 17) |
                            (static_cast<uint32_t>(kBM >> 4) << 24);

__device__ __forceinline__ float silu_pf(float g) { return g / (1.0f + expf(-g)); }

// Eight consecutive fp16 values: one 16-byte load when the address allows it.
__device__ __forceinline__ void load8_halves(__half (&dst)[8], const __half* src) {
  if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    *reinterpret_cast<uint4*>(dst) = __ldg(reinterpret_cast<const uint4*>(src));
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) dst[e] = src[e];
  }
}

__global__ void __launch_bounds__(kGemmThreads, 1)
i8gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_a2,
                      const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_b2,
                      const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  // a stage: [A tile][second A tile, split form only][B tile]; 4 stages of 48 KB or 3 of 64 KB
  const int kStages = p.split ? 3 : 4;
  const int a_tiles = p.split ? 2 : 1;
  const int stage_bytes = a_tiles * kATile + kBTile;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + kMaxStages * (kATile + kBTile));
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* acc_full = empty_bar + kMaxStages;     // [2] accumulator ready for the epilogue
  uint64_t* acc_empty = acc_full + 2;              // [2] accumulator drained by the epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* col_scale = reinterpret_cast<float*>(tmem_slot + 4);       // [2][kBN] channel scales of the tiles in flight

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kiters = (p.k + kBK - 1) / kBK;
  const int ntile_cols = p.dual ? kBN / 2 : kBN;   // channels per tile (per matrix when dual)
  const int total_tiles = p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], kEpiWarps);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Tiles in channel-fastest order: the blocks that run together share a few token tiles and all weight tiles.
  if (warp == 0) {
    if (lane == 0) {
      // ================= TMA producer =================
      int it = 0;
      for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        const int m0 = (tile / p.n_tiles) * kBM, n0 = (tile % p.n_tiles) * ntile_cols;
        for (int kk = 0; kk < kiters; ++kk, ++it) {
          const int s = it % kStages;
          if (*abort_flag || !mbar_wait_bounded(&empty_bar[s], ((it / kStages) & 1) ^ 1)) {
            report_status(p.status_word, LSVD_ERR_TIMEOUT);
            *abort_flag = 1;
            break;
          }
          uint8_t* stA = tiles + s * stage_bytes;
          uint8_t* stB = stA + a_tiles * kATile;
          mbar_arrive_expect_tx(&full_bar[s], stage_bytes);
          tma_load_2d(stA, &tm_a, kk * kBK, m0, &full_bar[s]);
          if (p.split) tma_load_2d(stA + kATile, &tm_a2, kk * kBK, m0, &full_bar[s]);
          if (p.dual) {
            tma_load_2d(stB, &tm_b, kk * kBK, n0, &full_bar[s]);
            tma_load_2d(stB + kBTile / 2, &tm_b2, kk * kBK, n0, &full_bar[s]);
          } else {
            tma_load_2d(stB, &tm_b, kk * kBK, n0, &full_bar[s]);
            tma_load_2d(stB + kBTile / 2, &tm_b, kk * kBK, n0 + kBN / 2, &full_bar[s]);
          }
        }
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ================= MMA issuer =================
      int it = 0, li = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++li) {
        const int buf = li & 1;
        if (!mbar_wait_bounded(&acc_empty[buf], ((li >> 1) & 1) ^ 1)) {
          report_status(p.status_word, LSVD_ERR_TIMEOUT);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * kBN);
        for (int kk = 0; kk < kiters; ++kk, ++it) {
          const int s = it % kStages;
          if (*abort_flag || !mbar_wait_bounded(&full_bar[s], (it / kStages) & 1)) {
            report_status(p.status_word, LSVD_ERR_TIMEOUT);
            *abort_flag = 1;
            break;
          }
          tc_fence_after();
          const uint8_t* stA = tiles + s * stage_bytes;
          const uint8_t* stB = stA + a_tiles * kATile;
          const uint64_t adesc = smem_desc_k_major_sw128(stA);
          const uint64_t bdesc = smem_desc_k_major_sw128(stB);
          if (!p.split) {
#pragma unroll
            for (int q = 0; q < kBK / 32; ++q)       // 32 int8 of K per instruction: 32 bytes further inside the swizzled row
              umma_i8(tmem_d, adesc + static_cast<uint64_t>(q * 32 >> 4), bdesc + static_cast<uint64_t>(q * 32 >> 4), kIdesc,
                      (kk > 0 || q > 0) ? 1u : 0u);
          } else {
            // gate half: A x B rows 0..127 into columns 0..127; up half: second A x B rows 128..255 into columns 128..255
            const uint64_t a2desc = smem_desc_k_major_sw128(stA + kATile);
            const uint64_t b2desc = smem_desc_k_major_sw128(stB + kBTile / 2);
#pragma unroll
            for (int q = 0; q < kBK / 32; ++q) {
              const uint64_t off = static_cast<uint64_t>(q * 32 >> 4);
              const uint32_t accumulate = (kk > 0 || q > 0) ? 1u : 0u;
              umma_i8(tmem_d, adesc + off, bdesc + off, kIdescHalf, accumulate);
              umma_i8(tmem_d + kBN / 2, a2desc + off, b2desc + off, kIdescHalf, accumulate);
            }
          }
          umma_commit(&empty_bar[s]);                // the stage is free once these MMAs have read it
        }
        umma_commit(&acc_full[buf]);                 // arrives when every MMA above has finished (also after an abort)
      }
    }
  } else {
    // ================= epilogue: warps 2..9; a warp reads the TMEM lanes 32 * (warp % 4) .. + 31, and the two
    // warps of a quarter take alternate 32-column chunks =================
    const int quarter = warp & 3;
    const int half_id = (warp - 2) >> 2;             // 0 or 1: which of the quarter's two warps
    const int et = threadIdx.x - 64;                 // 0..255 among the epilogue threads
    int li = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++li) {
      const int buf = li & 1;
      const int m0 = (tile / p.n_tiles) * kBM, n0 = (tile % p.n_tiles) * ntile_cols;
      // Channel scales of the tile, in accumulator column order, staged once per tile: the inner loops then
      // read them from shared memory instead of waiting on global loads value by value.
      float* cs = col_scale + buf * kBN;
#pragma unroll
      for (int i = et; i < kBN; i += kEpiWarps * 32) {
        float v = 0.f;
        if (p.dual) {
          const int col = n0 + (i & (kBN / 2 - 1));
          if (col < p.n) v = (i < kBN / 2) ? p.w_scale[col] : p.w2_scale[col];
        } else if (n0 + i < p.n) {
          v = p.w_scale[n0 + i];
        }
        cs[i] = v;
      }
      // Every epilogue warp attends the named barrier whatever its own wait returned; the barrier also ORs "a wait gave
      // up or the block is aborting" over the eight warps, so they go on together or leave together (and an aborted
      // tile's partial accumulator is never stored).
      bool bad = false;
      if (!mbar_wait_bounded(&acc_full[buf], (li >> 1) & 1)) {
        report_status(p.status_word, LSVD_ERR_TIMEOUT);
        *abort_flag = 1;
        bad = true;
      }
      // the staged scales are visible; tile li - 2's readers are done
      if (named_barrier_or(1, kEpiWarps * 32, bad || *abort_flag != 0)) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const bool row_ok = row < p.m;
      const float sa = row_ok ? p.a_scale[row * p.a_scale_stride] : 0.f;
      const float sa2 = (row_ok && p.split) ? p.a2_scale[row * p.a2_scale_stride] : sa;
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buf * kBN);
      __half* orow = p.out != nullptr ? p.out + static_cast<int64_t>(row) * p.out_row_stride + p.out_col : nullptr;
      const __half* grow = p.gate != nullptr ? p.gate + static_cast<int64_t>(row) * p.gate_row_stride + p.gate_col : nullptr;
      const __half* rrow = p.residual != nullptr ? p.residual + static_cast<int64_t>(row) * p.residual_row_stride : nullptr;
      const int chunks = p.dual ? kBN / 64 : kBN / 32;
      // Gate / residual values come from DRAM with a row per lane: the 64 bytes a lane needs for a chunk of 32
      // channels are requested together, before the accumulator is read.
      uint4 gq[4], rq[4];
      auto fetch_side = [&](int c) {
        const int col0 = n0 + c * 32;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          gq[q] = rq[q] = make_uint4(0u, 0u, 0u, 0u);
          if (row_ok && col0 + q * 8 < p.n) {
            if (grow != nullptr) load8_halves(reinterpret_cast<__half(&)[8]>(gq[q]), grow + col0 + q * 8);
            if (rrow != nullptr) load8_halves(reinterpret_cast<__half(&)[8]>(rq[q]), rrow + col0 + q * 8);
          }
        }
      };
      const bool side = grow != nullptr || rrow != nullptr;
#pragma unroll 1
      for (int c = half_id; c < chunks; c += 2) {
        uint32_t v[32], u[32];
        if (side) fetch_side(c);
        __syncwarp();
        tmem_ld32(lane_addr + c * 32, v);
        if (p.dual) tmem_ld32(lane_addr + kBN / 2 + c * 32, u);
        const int col0 = n0 + c * 32;
        if (!row_ok || col0 >= p.n) continue;
        if (p.acc_out != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.n) p.acc_out[static_cast<int64_t>(row) * p.n + col0 + j] = static_cast<int>(v[j]);
        }
        if (orow == nullptr) continue;
#pragma unroll
        for (int j0 = 0; j0 < 32; j0 += 8) {         // eight channels = one 16-byte store; n is a multiple of 16
          const int col = col0 + j0;
          if (col >= p.n) break;
          __align__(16) __half r[8];
#pragma unroll
          for (int e = 0; e < 8; ++e)
            r[e] = __float2half_rn((static_cast<float>(static_cast<int>(v[j0 + e])) * sa) * cs[c * 32 + j0 + e]);
          if (p.dual) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const __half u16 = __float2half_rn((static_cast<float>(static_cast<int>(u[j0 + e])) * sa2) * cs[kBN / 2 + c * 32 + j0 + e]);
              const __half sg = __float2half_rn(silu_pf(__half2float(r[e])));
              r[e] = __float2half_rn(__half2float(sg) * __half2float(u16));
            }
          }
          if (grow != nullptr) {
            const __half* gt = reinterpret_cast<const __half*>(&gq[j0 >> 3]);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const __half sg = __float2half_rn(silu_pf(__half2float(gt[e])));
              r[e] = __float2half_rn(__half2float(sg) * __half2float(r[e]));
            }
          }
          if (rrow != nullptr) {
            const __half* rs = reinterpret_cast<const __half*>(&rq[j0 >> 3]);
#pragma unroll
            for (int e = 0; e < 8; ++e) r[e] = __float2half_rn(__half2float(r[e]) + __half2float(rs[e]));
          }
          if ((reinterpret_cast<uintptr_t>(orow + col) & 15) == 0) {
            *reinterpret_cast<uint4*>(orow + col) = *reinterpret_cast<const uint4*>(r);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) orow[col + e] = r[e];
          }
        }
      }
      // this warp's reads of the accumulator are complete (tcgen05.wait::ld in tmem_ld32): hand it back
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace lsvd

extern "C" int lsvd_i8gemm_prefill(const lsvd_i8gemm_args* a, void* stream) {
  using namespace lsvd;
  if (a == nullptr || a->m <= 0 || a->n <= 0 || (a->n % 16) || a->k <= 0 || (a->k % 16)) return LSVD_ERR_INVALID_ARG;
  if (!a->a || !a->w || !a->a_scale || !a->w_scale) return LSVD_ERR_INVALID_ARG;
  if (a->out == nullptr && a->acc_out == nullptr) return LSVD_ERR_INVALID_ARG;
  const bool dual = a->w2 != nullptr;
  if (dual && (!a->w2_scale || a->out == nullptr || a->acc_out != nullptr || a->gate != nullptr || a->residual != nullptr))
    return LSVD_ERR_INVALID_ARG;
  if ((a->gate != nullptr || a->residual != nullptr) && a->out == nullptr) return LSVD_ERR_INVALID_ARG;
  if (!aligned(a->a, 16) || (a->a_row_stride % 16) || !aligned(a->w, 16) || (a->w_row_stride % 16)) return LSVD_ERR_INVALID_ARG;
  if (dual && (!aligned(a->w2, 16) || (a->w2_row_stride % 16))) return LSVD_ERR_INVALID_ARG;
  if (a->out && (!aligned(a->out, 4) || (a->out_row_stride % 2) || (a->out_col % 2))) return LSVD_ERR_INVALID_ARG;
  const bool split = dual && a->a2 != nullptr;
  if (a->a2 != nullptr && !dual) return LSVD_ERR_INVALID_ARG;
  if (split && (!a->a2_scale || !aligned(a->a2, 16) || (a->a2_row_stride % 16))) return LSVD_ERR_INVALID_ARG;
  CUtensorMap ma, ma2, mb, mb2;
  int rc = make_map_k128(&ma, a->a, a->m, a->k, a->a_row_stride, kBM);
  if (rc != LSVD_OK) return rc;
  rc = make_map_k128(&ma2, split ? a->a2 : a->a, a->m, a->k, split ? a->a2_row_stride : a->a_row_stride, kBM);
  if (rc != LSVD_OK) return rc;
  rc = make_map_k128(&mb, a->w, a->n, a->k, a->w_row_stride, kBN / 2);
  if (rc != LSVD_OK) return rc;
  rc = make_map_k128(&mb2, dual ? a->w2 : a->w, a->n, a->k, dual ? a->w2_row_stride : a->w_row_stride, kBN / 2);
  if (rc != LSVD_OK) return rc;
  GemmParams p{};
  p.a_scale = a->a_scale;
  p.a_scale_stride = a->a_scale_stride > 0 ? a->a_scale_stride : 1;
  p.w_scale = a->w_scale;
  p.w2_scale = a->w2_scale;
  p.out = static_cast<__half*>(a->out);
  p.out_row_stride = a->out_row_stride;
  p.out_col = a->out_col;
  p.gate = static_cast<const __half*>(a->gate);
  p.gate_row_stride = a->gate_row_stride;
  p.gate_col = a->gate_col;
  p.residual = static_cast<const __half*>(a->residual);
  p.residual_row_stride = a->residual_row_stride;
  p.acc_out = a->acc_out;
  p.status_word = a->status_word;
  p.m = a->m; p.n = a->n; p.k = a->k; p.dual = dual ? 1 : 0;
  p.split = split ? 1 : 0;
  p.a2_scale = a->a2_scale;
  p.a2_scale_stride = a->a2_scale_stride > 0 ? a->a2_scale_stride : 1;
  const int ntile = dual ? kBN / 2 : kBN;
  p.m_tiles = (a->m + kBM - 1) / kBM;
  p.n_tiles = (a->n + ntile - 1) / ntile;
  const int64_t tiles = static_cast<int64_t>(p.m_tiles) * p.n_tiles;
  if (tiles > 0x7fffffffLL) return LSVD_ERR_UNSUPPORTED;
  LSVD_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(i8gemm_tcgen05_kernel), kGemmSmem));
  const int grid = static_cast<int>(std::min<int64_t>(tiles, std::max(1, device_sm_count())));
  i8gemm_tcgen05_kernel<<<grid, kGemmThreads, kGemmSmem, static_cast<cudaStream_t>(stream)>>>(ma, ma2, mb, mb2, p);
  LSVD_CUDA_TRY(cudaGetLastError());
  return LSVD_OK;
}
