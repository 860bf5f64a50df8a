// W8A8 GEMM for prefill and large batches on the fifth-generation tensor cores:
//   acc[m, n] = sum_k a[m, k] * w[n, k]   (int8 x int8 -> int32, exact), dequantised to fp16 in the epilogue.
//
// One thread block computes a 128 (tokens) x 256 (channels) tile.  Warp 0 (one elected lane) streams the A and B
// tiles with TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast) into a four-stage shared-memory ring;
// warp 1 (one elected lane) issues tcgen05.mma kind::i8 (M 128, N 256, K 32 per instruction) whose accumulator
// lives in tensor memory (256 columns of 32 bits, allocated by warp 1); tcgen05.commit hands each ring stage
// back to the producer and finally signals the four epilogue warps, which read the accumulator with
// tcgen05.ld (lane = token row, 32 columns at a time), apply token and channel scales (and SiLU gating for a
// gate/up pair) and store fp16.  Every mbarrier wait is bounded; a wait that gives up sets the status word and
// the block still releases its tensor memory.
//
// Replaces the Triton tl.dot int8 kernels of the reference for M >> 64
// (kernels/layer_bench/ffn_kernel/mix_ffn_kernel.py:410-500, 903-1021, 1152-1338) and produces the same values as
// the decode-sized lsvd_w8a8_gemv.
#include <cuda.h>

#include <cmath>
#include <mutex>

#include "common.cuh"

namespace lsvd {

constexpr int kBM = 128, kBN = 256, kBK = 128, kStages = 4;
constexpr int kATile = kBM * kBK, kBTile = kBN * kBK;                     // bytes (int8)
constexpr int kGemmThreads = 192;                                          // producer, MMA issuer, four epilogue warps
constexpr int kGemmSmem = kStages * (kATile + kBTile) + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr uint32_t kTmemCols = 256;

struct GemmParams {
  const float* a_scale;
  const float* w_scale;
  const float* w2_scale;
  __half* out;
  int64_t out_row_stride;
  int32_t out_col;
  int32_t* acc_out;          // optional raw accumulators [m, n] (single-matrix form only)
  int32_t* status_word;
  int32_t m, n, k, dual;     // dual: the B tile is 128 gate channels followed by their 128 up channels
};

// ---- PTX wrappers -----------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile written by TMA with the 128-byte swizzle: rows of 128 bytes,
// groups of 8 rows (1024 bytes) apart by the stride offset; descriptor version 1 (sm_100), layout type 2 (128 B).
__device__ __forceinline__ uint64_t smem_desc_k_major_sw128(const void* tile) {
  const uint64_t addr = smem_u32(tile);
  return ((addr & 0x3FFFFull) >> 4) | (1ull << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: D = S32 (2 at bit 4), A = S8 (1 at bit 7), B = S8 (1 at bit 10), both K-major,
// N >> 3 at bit 17, M >> 4 at bit 24.
constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kBN >> 3) << 17) |
                            (static_cast<uint32_t>(kBM >> 4) << 24);

__device__ __forceinline__ float silu_pf(float g) { return g / (1.0f + expf(-g)); }

__global__ void __launch_bounds__(kGemmThreads, 1)
i8gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                      const __grid_constant__ CUtensorMap tm_b2, const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sA = tiles;
  uint8_t* sB = tiles + kStages * kATile;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + kStages * (kATile + kBTile));
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* acc_bar = empty_bar + kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * kBM;
  const int n0 = blockIdx.x * (p.dual ? kBN / 2 : kBN);       // first channel of the tile (per matrix when dual)
  const int kiters = (p.k + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // ================= TMA producer =================
      for (int it = 0; it < kiters; ++it) {
        const int s = it % kStages;
        if (!mbar_wait_bounded(&empty_bar[s], ((it / kStages) & 1) ^ 1)) {
          report_status(p.status_word, LSVD_ERR_TIMEOUT);
          *abort_flag = 1;
          break;
        }
        mbar_arrive_expect_tx(&full_bar[s], kATile + kBTile);
        tma_load_2d(sA + s * kATile, &tm_a, it * kBK, m0, &full_bar[s]);
        if (p.dual) {
          tma_load_2d(sB + s * kBTile, &tm_b, it * kBK, n0, &full_bar[s]);
          tma_load_2d(sB + s * kBTile + kBTile / 2, &tm_b2, it * kBK, n0, &full_bar[s]);
        } else {
          tma_load_2d(sB + s * kBTile, &tm_b, it * kBK, n0, &full_bar[s]);
          tma_load_2d(sB + s * kBTile + kBTile / 2, &tm_b, it * kBK, n0 + kBN / 2, &full_bar[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ================= MMA issuer =================
      bool ok = true;
      for (int it = 0; it < kiters && ok; ++it) {
        const int s = it % kStages;
        if (*abort_flag || !mbar_wait_bounded(&full_bar[s], (it / kStages) & 1)) {
          report_status(p.status_word, LSVD_ERR_TIMEOUT);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t adesc = smem_desc_k_major_sw128(sA + s * kATile);
        const uint64_t bdesc = smem_desc_k_major_sw128(sB + s * kBTile);
#pragma unroll
        for (int kk = 0; kk < kBK / 32; ++kk)        // 32 int8 of K per instruction: 32 bytes further inside the swizzled row
          umma_i8(tmem_base, adesc + static_cast<uint64_t>(kk * 32 >> 4), bdesc + static_cast<uint64_t>(kk * 32 >> 4), kIdesc,
                  (it > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&empty_bar[s]);                  // the stage is free once these MMAs have read it
      }
      umma_commit(acc_bar);                          // arrives when every MMA above has finished (also after an abort)
    }
  } else {
    // ================= epilogue: warps 2..5, TMEM lanes 32 * (warp % 4) .. + 31 =================
    const int quarter = warp & 3;
    const bool ok = mbar_wait_bounded(acc_bar, 0) && *abort_flag == 0;
    if (!ok) report_status(p.status_word, LSVD_ERR_TIMEOUT);
    tc_fence_after();
    const int row = m0 + quarter * 32 + lane;
    const float sa = (ok && row < p.m) ? p.a_scale[row] : 0.f;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    if (ok) {
      if (!p.dual) {
#pragma unroll 1
        for (int c = 0; c < kBN / 32; ++c) {
          uint32_t v[32];
          tmem_ld32(lane_addr + c * 32, v);
          const int col0 = n0 + c * 32;
          if (row < p.m) {
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const int col = col0 + j;
              if (col < p.n) {        // n is even: a pair is inside or outside together
                if (p.acc_out != nullptr) {
                  p.acc_out[static_cast<int64_t>(row) * p.n + col] = static_cast<int>(v[j]);
                  p.acc_out[static_cast<int64_t>(row) * p.n + col + 1] = static_cast<int>(v[j + 1]);
                }
                if (p.out != nullptr) {
                  const float f0 = (static_cast<float>(static_cast<int>(v[j])) * sa) * p.w_scale[col];
                  const float f1 = (static_cast<float>(static_cast<int>(v[j + 1])) * sa) * p.w_scale[col + 1];
                  *reinterpret_cast<__half2*>(p.out + static_cast<int64_t>(row) * p.out_row_stride + p.out_col + col) =
                      __floats2half2_rn(f0, f1);
                }
              }
            }
          }
        }
      } else {
        // columns 0..127: gate channels n0.., columns 128..255: the same channels of the up matrix
#pragma unroll 1
        for (int c = 0; c < kBN / 64; ++c) {
          uint32_t gv[32], uv[32];
          tmem_ld32(lane_addr + c * 32, gv);
          tmem_ld32(lane_addr + kBN / 2 + c * 32, uv);
          const int col0 = n0 + c * 32;
          if (row < p.m) {
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const int col = col0 + j;
              if (col < p.n) {
                float h[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                  const __half g16 = __float2half_rn((static_cast<float>(static_cast<int>(gv[j + e])) * sa) * p.w_scale[col + e]);
                  const __half u16 = __float2half_rn((static_cast<float>(static_cast<int>(uv[j + e])) * sa) * p.w2_scale[col + e]);
                  const __half sg = __float2half_rn(silu_pf(__half2float(g16)));
                  h[e] = __half2float(sg) * __half2float(u16);
                }
                *reinterpret_cast<__half2*>(p.out + static_cast<int64_t>(row) * p.out_row_stride + p.out_col + col) =
                    __floats2half2_rn(h[0], h[1]);
              }
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host --------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
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

// Tensor map of an int8 matrix [rows, k] (row stride in bytes), boxes of 128 rows x 128 bytes, 128-byte swizzle,
// out-of-range elements read as zero.
static int make_map(CUtensorMap* map, const int8_t* base, int64_t rows, int64_t k, int64_t row_stride) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return LSVD_ERR_CUDA;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_stride)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), 128u};
  const cuuint32_t estr[2] = {1u, 1u};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LSVD_OK : LSVD_ERR_CUDA;
}

}  // namespace lsvd

extern "C" int lsvd_i8gemm_prefill(const lsvd_i8gemm_args* a, void* stream) {
  using namespace lsvd;
  if (a == nullptr || a->m <= 0 || a->n <= 0 || (a->n % 16) || a->k <= 0 || (a->k % 16)) return LSVD_ERR_INVALID_ARG;
  if (!a->a || !a->w || !a->a_scale || !a->w_scale) return LSVD_ERR_INVALID_ARG;
  if (a->out == nullptr && a->acc_out == nullptr) return LSVD_ERR_INVALID_ARG;
  const bool dual = a->w2 != nullptr;
  if (dual && (!a->w2_scale || a->out == nullptr || a->acc_out != nullptr)) return LSVD_ERR_INVALID_ARG;
  if (!aligned(a->a, 16) || (a->a_row_stride % 16) || !aligned(a->w, 16) || (a->w_row_stride % 16)) return LSVD_ERR_INVALID_ARG;
  if (dual && (!aligned(a->w2, 16) || (a->w2_row_stride % 16))) return LSVD_ERR_INVALID_ARG;
  if (a->out && (!aligned(a->out, 4) || (a->out_row_stride % 2) || (a->out_col % 2))) return LSVD_ERR_INVALID_ARG;
  CUtensorMap ma, mb, mb2;
  int rc = make_map(&ma, a->a, a->m, a->k, a->a_row_stride);
  if (rc != LSVD_OK) return rc;
  rc = make_map(&mb, a->w, a->n, a->k, a->w_row_stride);
  if (rc != LSVD_OK) return rc;
  rc = make_map(&mb2, dual ? a->w2 : a->w, a->n, a->k, dual ? a->w2_row_stride : a->w_row_stride);
  if (rc != LSVD_OK) return rc;
  GemmParams p{};
  p.a_scale = a->a_scale;
  p.w_scale = a->w_scale;
  p.w2_scale = a->w2_scale;
  p.out = static_cast<__half*>(a->out);
  p.out_row_stride = a->out_row_stride;
  p.out_col = a->out_col;
  p.acc_out = a->acc_out;
  p.status_word = a->status_word;
  p.m = a->m; p.n = a->n; p.k = a->k; p.dual = dual ? 1 : 0;
  LSVD_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(i8gemm_tcgen05_kernel), kGemmSmem));
  const int ntile = dual ? kBN / 2 : kBN;
  dim3 grid((a->n + ntile - 1) / ntile, (a->m + kBM - 1) / kBM);
  i8gemm_tcgen05_kernel<<<grid, kGemmThreads, kGemmSmem, static_cast<cudaStream_t>(stream)>>>(ma, mb, mb2, p);
  LSVD_CUDA_TRY(cudaGetLastError());
  return LSVD_OK;
}
