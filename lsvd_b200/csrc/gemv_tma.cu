// Weight-streaming W8A8 product for decode batches of at most 16 tokens, fed by TMA:
//   acc[tok, row] = sum_k a[tok, k] * w[row, k]      (int8 x int8 -> int32 on mma.sync m16n8k32)
//
// A decode GEMV is a pure HBM stream, and on this part a stream only runs at full rate with on the order of
// 100 KB in flight per SM: more than the register file can hold as load destinations.  So the loads go
// through shared memory.  One persistent block per SM walks its share of the 16-row tiles; a producer warp
// (one elected lane) issues tiled TMA copies (cp.async.bulk.tensor.2d, 128-byte swizzle, every block loads its own tiles) of the
// next 1 KB of K of the tile's rows of every weight matrix and of the token rows into a ring of stages; eight
// consumer warps each take one 128-byte chunk of the stage, read it with conflict-free 16-byte shared loads in
// MMA fragment order and accumulate; after the last stage of a tile their shares are summed through shared
// memory and dequantised while the producer already streams the next tile.  Every mbarrier wait is bounded.
//
// Same values as the register-fed form in ffn_decode.cu (w8a8_gemv_kernel), which serves larger batches.
#include <algorithm>
#include <cstdlib>

#include "gemv.cuh"
#include "tma.cuh"

namespace lsvd {

constexpr int kTgConsumers = 8;                       // consumer warps = 128-byte chunks of a stage
constexpr int kTgThreads = (kTgConsumers + 1) * 32;   // + the producer warp
constexpr int kTgStageK = kTgConsumers * 128;         // bytes of K per stage
constexpr int kTgRows = 16;                           // weight rows per tile and matrix
constexpr int kTgMaxStages = 12;

template <int NT, bool DUAL, bool SPLIT_B>
struct TgLayout {
  static constexpr int kW = kTgConsumers * kTgRows * 128;               // one matrix' rows of a stage
  static constexpr int kA = kTgConsumers * NT * 8 * 128;                // the token rows of a stage
  static constexpr int kStage = kW * (DUAL ? 2 : 1) + kA * (SPLIT_B ? 2 : 1);
  static constexpr int kRed = kTgConsumers * (DUAL ? 2 : 1) * NT * 4 * 32 * 4;
};

__device__ __forceinline__ uint4 lds_u4(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }

// Named barrier of the consumer warps only: the producer never joins it.
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kTgConsumers * 32) : "memory"); }

template <int NT, bool DUAL, bool SPLIT_B>
__global__ void __launch_bounds__(kTgThreads, 1)
w8a8_gemv_tma_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_w2,
                     const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_a2,
                     const __grid_constant__ GemvParams p, const int stages) {
  using L = TgLayout<NT, DUAL, SPLIT_B>;
  constexpr int NMAT = DUAL ? 2 : 1;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  int* red = reinterpret_cast<int*>(ring + static_cast<size_t>(stages) * L::kStage);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(red) + L::kRed);
  uint64_t* empty_bar = full_bar + kTgMaxStages;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kTgConsumers);
    }
    fence_mbar_init();
  }
  __syncthreads();

  const int tiles = p.n / kTgRows;
  const int ksteps = (p.k + kTgStageK - 1) / kTgStageK;

  if (warp == kTgConsumers) {
    // ================= producer =================
    if (lane == 0) {
      // Weights do not depend on the kernel before this one; the token rows do.
      grid_dependency_wait();
      int it = 0;
      for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int row0 = tile * kTgRows;
        for (int ks = 0; ks < ksteps; ++ks, ++it) {
          const int s = it % stages;
          if (!mbar_wait_bounded(&empty_bar[s], ((it / stages) & 1) ^ 1)) {
            report_status(p.status_word, LSVD_ERR_TIMEOUT);
            return;
          }
          uint8_t* st = ring + static_cast<size_t>(s) * L::kStage;
          mbar_arrive_expect_tx(&full_bar[s], L::kStage);
          const int k0 = ks * kTgStageK;
#pragma unroll
          for (int c = 0; c < kTgConsumers; ++c) {
            tma_load_2d(st + c * (kTgRows * 128), &tm_w, k0 + c * 128, row0, &full_bar[s]);
            if (DUAL) tma_load_2d(st + L::kW + c * (kTgRows * 128), &tm_w2, k0 + c * 128, row0, &full_bar[s]);
            tma_load_2d(st + NMAT * L::kW + c * (NT * 8 * 128), &tm_a, k0 + c * 128, 0, &full_bar[s]);
            if (SPLIT_B) tma_load_2d(st + NMAT * L::kW + L::kA + c * (NT * 8 * 128), &tm_a2, k0 + c * 128, 0, &full_bar[s]);
          }
        }
      }
    }
    return;
  }

  // ================= consumers =================
  const int g = lane >> 2, t = lane & 3;
  int it = 0;
  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    int acc[NMAT][NT][4];
#pragma unroll
    for (int mtx = 0; mtx < NMAT; ++mtx)
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[mtx][j][c] = 0;

    bool bad = false;
    for (int ks = 0; ks < ksteps; ++ks, ++it) {
      const int s = it % stages;
      if (!mbar_wait_bounded(&full_bar[s], (it / stages) & 1)) {
        report_status(p.status_word, LSVD_ERR_TIMEOUT);
        bad = true;              // leave the K loop, but still attend the named barrier below
        break;
      }
      const uint8_t* st = ring + static_cast<size_t>(s) * L::kStage;
      const uint8_t* wc = st + warp * (kTgRows * 128);                      // this warp's 128-byte chunk: [16 rows][128]
      const uint8_t* ac = st + NMAT * L::kW + warp * (NT * 8 * 128);        // [NT * 8 tokens][128]
      // 128-byte swizzle: the 16-byte unit j of row r sits at unit j ^ (r & 7); rows g and g + 8 share g & 7
#pragma unroll
      for (int sp = 0; sp < 2; ++sp) {
        const int unit = ((4 * sp + t) ^ g) << 4;
        const uint4 x0 = lds_u4(wc + g * 128 + unit), x1 = lds_u4(wc + (g + 8) * 128 + unit);
        uint4 y0 = x0, y1 = x1;
        if (DUAL) {
          y0 = lds_u4(wc + L::kW + g * 128 + unit);
          y1 = lds_u4(wc + L::kW + (g + 8) * 128 + unit);
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const uint4 bv = lds_u4(ac + (j * 8 + g) * 128 + unit);
          // the MMA's k index is a permutation of the 32 columns that A and B share: k 4t..4t+3 <-> the first
          // four of a lane's bytes, k 16+4t.. <-> the next four
          mma_s8(acc[0][j], x0.x, x1.x, x0.y, x1.y, bv.x, bv.y);
          mma_s8(acc[0][j], x0.z, x1.z, x0.w, x1.w, bv.z, bv.w);
          if (DUAL) {
            uint4 bw = bv;
            if (SPLIT_B) bw = lds_u4(ac + L::kA + (j * 8 + g) * 128 + unit);
            mma_s8(acc[NMAT - 1][j], y0.x, y1.x, y0.y, y1.y, bw.x, bw.y);
            mma_s8(acc[NMAT - 1][j], y0.z, y1.z, y0.w, y1.w, bw.z, bw.w);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }

    // ---- sum the warps' shares, dequantise, store ----
    int* mine = red + warp * (NMAT * NT * 4 * 32);
#pragma unroll
    for (int mtx = 0; mtx < NMAT; ++mtx)
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) mine[((mtx * NT + j) * 4 + c) * 32 + lane] = acc[mtx][j][c];
    // the barrier ORs "a wait gave up" over the consumer warps: they all stop here or none does
    if (named_barrier_or(1, kTgConsumers * 32, bad)) return;
    const int row0 = tile * kTgRows;
    // element e of a matrix: (j, c, lane) -> row = g + 8 (c >> 1), token = 8 j + 2 t + (c & 1)
    for (int e = threadIdx.x; e < NT * 4 * 32; e += kTgConsumers * 32) {
      const int el = e & 31, c = (e >> 5) & 3, j = e >> 7;
      const int row = row0 + (el >> 2) + 8 * (c >> 1);
      const int tok = j * 8 + 2 * (el & 3) + (c & 1);
      int sum0 = 0, sum1 = 0;
#pragma unroll
      for (int wi = 0; wi < kTgConsumers; ++wi) {
        sum0 += red[wi * (NMAT * NT * 4 * 32) + e];
        if (DUAL) sum1 += red[wi * (NMAT * NT * 4 * 32) + NT * 4 * 32 + e];
      }
      if (tok < p.m) gemv_store<DUAL, SPLIT_B>(p, tok, row, sum0, sum1);
    }
    consumer_sync();                   // the shares are read before the next tile overwrites them
  }
}

// ----------------------------------------------------------------------------------------------
// 17..64 tokens: the token rows are as large as a block's weight rows, so they are shared
// ----------------------------------------------------------------------------------------------
// With more tokens the register-fed form re-reads every token row once per 16 output channels (L1-bound:
// 68 us for the 45 MB gate/up pair at 64 tokens).  Here a block owns up to 64 channels (one consumer warp per 16)
// and a stage holds 256 bytes of K of those weight rows and of ALL token rows, fetched once per block by TMA;
// every consumer warp reads the whole token tile from shared memory and only its own weight rows, keeps complete
// sums for its channels in registers, and stores them itself: no reduction across warps.
// When the matrix has too few channels to give every SM a block of 64 (a tensor-parallel rank's column slice), a block
// takes 16 or 32 channels and its four consumer warps split every stage's K instead (`kw` warps per 16-channel tile, each
// taking every kw-th 64-byte span): a single warp's chain of dependent MMAs on one tile leaves three quarters of the SM's
// tensor issue idle (measured: 46 us for a 2 x 1728 x 5120 pair on 108 one-warp blocks, the same as for 4 x the channels).
// The kw partial sums of a tile meet in shared memory; each of the kw warps then finishes the token columns j = kq mod kw.
constexpr int kWideStageK = 256;                      // bytes of K per stage: two 128-byte chunks
constexpr int kWideMaxWarps = 4;

template <int NT, bool DUAL, bool SPLIT_B, int KW>
__global__ void __launch_bounds__((kWideMaxWarps + 1) * 32, 1)
w8a8_gemv_wide_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_w2,
                      const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_a2,
                      const __grid_constant__ GemvParams p, const int stages, const int warps) {
  constexpr int NMAT = DUAL ? 2 : 1;
  constexpr int kw = KW;                              // warps that share a 16-channel tile's K
  extern __shared__ uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int rows = warps * 16;                        // channels per block (and matrix): `warps` 16-channel tiles
  const int consumers = warps * kw;                   // kw warps share a tile's K
  const int w_bytes = 2 * rows * 128;                 // one matrix' rows of a stage: [2 chunks][rows][128]
  const int a_bytes = 2 * NT * 8 * 128;               // the token rows of a stage: [2 chunks][NT * 8][128]
  const int stage_bytes = NMAT * w_bytes + (SPLIT_B ? 2 : 1) * a_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ring + static_cast<size_t>(stages) * stage_bytes);
  uint64_t* empty_bar = full_bar + kTgMaxStages;
  int* red = reinterpret_cast<int*>(empty_bar + kTgMaxStages);      // kw > 1: [consumers][NMAT * NT * 4 * 32] partial sums

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], consumers);
    }
    fence_mbar_init();
  }
  __syncthreads();
  const int tiles = (p.n + rows - 1) / rows;
  const int ksteps = (p.k + kWideStageK - 1) / kWideStageK;

  if (warp == consumers) {
    // ================= producer =================
    if (lane == 0) {
      grid_dependency_wait();
      int it = 0;
      for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int row0 = tile * rows;
        for (int ks = 0; ks < ksteps; ++ks, ++it) {
          const int s = it % stages;
          if (!mbar_wait_bounded(&empty_bar[s], ((it / stages) & 1) ^ 1)) {
            report_status(p.status_word, LSVD_ERR_TIMEOUT);
            return;
          }
          uint8_t* st = ring + static_cast<size_t>(s) * stage_bytes;
          mbar_arrive_expect_tx(&full_bar[s], stage_bytes);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int k0 = ks * kWideStageK + c * 128;
            tma_load_2d(st + c * (rows * 128), &tm_w, k0, row0, &full_bar[s]);
            if (DUAL) tma_load_2d(st + w_bytes + c * (rows * 128), &tm_w2, k0, row0, &full_bar[s]);
            tma_load_2d(st + NMAT * w_bytes + c * (NT * 8 * 128), &tm_a, k0, 0, &full_bar[s]);
            if (SPLIT_B) tma_load_2d(st + NMAT * w_bytes + a_bytes + c * (NT * 8 * 128), &tm_a2, k0, 0, &full_bar[s]);
          }
        }
      }
    }
    return;
  }
  if (warp > consumers) return;

  // ========== consumers: warp w works on channels 16 rt .. 16 rt + 15 of the block's tile, K spans kq mod kw ==========
  const int g = lane >> 2, t = lane & 3;
  const int rt = warp / kw, kq = warp - rt * kw;
  bool bad = false;
  int it = 0;
  for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    int acc[NMAT][NT][4];
#pragma unroll
    for (int mtx = 0; mtx < NMAT; ++mtx)
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[mtx][j][c] = 0;
    for (int ks = 0; ks < ksteps; ++ks, ++it) {
      const int s = it % stages;
      if (!mbar_wait_bounded(&full_bar[s], (it / stages) & 1)) {
        report_status(p.status_word, LSVD_ERR_TIMEOUT);
        bad = true;
        break;
      }
      const uint8_t* st = ring + static_cast<size_t>(s) * stage_bytes;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const uint8_t* wc = st + c * (rows * 128) + rt * (16 * 128);          // [16 rows of this warp's tile][128], swizzled
        const uint8_t* ac = st + NMAT * w_bytes + c * (NT * 8 * 128);         // [NT * 8 tokens][128]
#pragma unroll
        for (int sp = 0; sp < 2; ++sp) {
          if (KW > 1 && ((2 * c + sp) % KW) != kq) continue;                  // another warp of the tile takes this span
          const int unit = ((4 * sp + t) ^ g) << 4;
          const uint4 x0 = lds_u4(wc + g * 128 + unit), x1 = lds_u4(wc + (g + 8) * 128 + unit);
          uint4 y0 = x0, y1 = x1;
          if (DUAL) {
            y0 = lds_u4(wc + w_bytes + g * 128 + unit);
            y1 = lds_u4(wc + w_bytes + (g + 8) * 128 + unit);
          }
#pragma unroll
          for (int j = 0; j < NT; ++j) {
            const uint4 bv = lds_u4(ac + (j * 8 + g) * 128 + unit);
            mma_s8(acc[0][j], x0.x, x1.x, x0.y, x1.y, bv.x, bv.y);
            mma_s8(acc[0][j], x0.z, x1.z, x0.w, x1.w, bv.z, bv.w);
            if (DUAL) {
              uint4 bw = bv;
              if (SPLIT_B) bw = lds_u4(ac + a_bytes + (j * 8 + g) * 128 + unit);
              mma_s8(acc[NMAT - 1][j], y0.x, y1.x, y0.y, y1.y, bw.x, bw.y);
              mma_s8(acc[NMAT - 1][j], y0.z, y1.z, y0.w, y1.w, bw.z, bw.w);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }
    if (kw == 1) {
      if (bad) return;
    } else {
      // the tile's kw partial sums meet in shared memory; this warp goes on with the token columns j = kq mod kw
      int* mine = red + warp * (NMAT * NT * 4 * 32);
#pragma unroll
      for (int mtx = 0; mtx < NMAT; ++mtx)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
          for (int c = 0; c < 4; ++c) mine[((mtx * NT + j) * 4 + c) * 32 + lane] = acc[mtx][j][c];
      // the barrier ORs "a wait gave up" over the consumer warps: they all stop here or none does
      if (named_barrier_or(1, consumers * 32, bad)) return;
#pragma unroll
      for (int mtx = 0; mtx < NMAT; ++mtx)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            int sum = 0;
            if ((j % kw) == kq)
              for (int q = 0; q < kw; ++q) sum += red[(rt * kw + q) * (NMAT * NT * 4 * 32) + ((mtx * NT + j) * 4 + c) * 32 + lane];
            acc[mtx][j][c] = sum;
          }
    }
    // ---- complete sums of channels (g, g + 8) x tokens (8 j + 2 t, + 1): dequantise and store ----
    // Scales and residuals are requested for all of a lane's 4 NT values before the first one is used: an
    // epilogue that waits on a global load per value costs more than the tile's whole stream.
    const int row_base = tile * rows + rt * 16;
    const int r0 = row_base + g, r1 = r0 + 8;
    const bool ok0 = r0 < p.n, ok1 = r1 < p.n;
    if (p.acc_out != nullptr || (DUAL && p.acc2_out != nullptr)) {
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int row = (c >> 1) ? r1 : r0, tok = j * 8 + 2 * t + (c & 1);
          if (row < p.n && tok < p.m && (j % kw) == kq) {
            if (p.acc_out != nullptr) p.acc_out[static_cast<int64_t>(tok) * p.n + row] = acc[0][j][c];
            if (DUAL && p.acc2_out != nullptr) p.acc2_out[static_cast<int64_t>(tok) * p.n + row] = acc[NMAT - 1][j][c];
          }
        }
    }
    if (p.out != nullptr) {
      float sw[2] = {0.f, 0.f}, sw2[2] = {0.f, 0.f};
      if (ok0) sw[0] = p.w_scale[r0];
      if (ok1) sw[1] = p.w_scale[r1];
      if (DUAL) {
        if (ok0) sw2[0] = p.w2_scale[r0];
        if (ok1) sw2[1] = p.w2_scale[r1];
      }
      float sa[NT][2], sb[NT][2];
      __half res[NT][4];
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tok = j * 8 + 2 * t + e;
          sa[j][e] = sb[j][e] = 0.f;
          if (tok < p.m) {
            sa[j][e] = p.a_scale[tok * p.a_scale_stride];
            sb[j][e] = (DUAL && SPLIT_B) ? p.a2_scale[tok * p.a2_scale_stride] : sa[j][e];
          }
        }
      if (p.residual != nullptr) {
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int row = (c >> 1) ? r1 : r0, tok = j * 8 + 2 * t + (c & 1);
            res[j][c] = __float2half(0.f);
            if (row < p.n && tok < p.m) res[j][c] = p.residual[static_cast<int64_t>(tok) * p.residual_row_stride + row];
          }
      }
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int hi = c >> 1, e = c & 1;
          const int row = hi ? r1 : r0, tok = j * 8 + 2 * t + e;
          if (row >= p.n || tok >= p.m || (j % kw) != kq) continue;
          const __half v0 = __float2half_rn((static_cast<float>(acc[0][j][c]) * sa[j][e]) * sw[hi]);
          __half out = v0;
          if (DUAL) {
            const __half u = __float2half_rn((static_cast<float>(acc[NMAT - 1][j][c]) * sb[j][e]) * sw2[hi]);
            const __half sg = __float2half_rn(silu_f(__half2float(v0)));
            out = __float2half_rn(__half2float(sg) * __half2float(u));
          }
          if (p.residual != nullptr) out = __float2half_rn(__half2float(out) + __half2float(res[j][c]));
          p.out[static_cast<int64_t>(tok) * p.out_row_stride + p.out_col + row] = out;
        }
    }
    if (kw > 1) named_barrier_or(1, consumers * 32, false);      // the shares are read before the next tile overwrites them
  }
}

template <int NT, bool DUAL, bool SPLIT_B>
static int launch_wide(const GemvParams& p, cudaStream_t st) {
  constexpr int NMAT = DUAL ? 2 : 1;
  const int sms = std::max(1, device_sm_count());
  const int row_tiles = (p.n + 15) / 16;
  const int warps = std::max(1, std::min(kWideMaxWarps, (row_tiles + sms - 1) / sms));    // 16-channel tiles per block
  int kw = warps == 1 ? 4 : (warps == 2 ? 2 : 1);                                          // warps that share a tile's K
  {
    // measurement knob: LSVD_GEMV_WIDE_KW = 1 | 2 | 4 forces the split where the block shape allows it
    static const int forced = [] { const char* e = std::getenv("LSVD_GEMV_WIDE_KW"); return e ? std::atoi(e) : 0; }();
    if ((forced == 1 || forced == 2 || forced == 4) && warps * forced <= kWideMaxWarps) kw = forced;
  }
  const int rows = warps * 16;
  CUtensorMap mw, mw2, ma, ma2;
  int rc = make_map_k128(&mw, p.w, p.n, p.k, p.w_row_stride, rows);
  if (rc != LSVD_OK) return rc;
  rc = make_map_k128(&mw2, DUAL ? p.w2 : p.w, p.n, p.k, DUAL ? p.w2_row_stride : p.w_row_stride, rows);
  if (rc != LSVD_OK) return rc;
  rc = make_map_k128(&ma, p.a, p.m, p.k, p.a_row_stride, NT * 8);
  if (rc != LSVD_OK) return rc;
  rc = make_map_k128(&ma2, SPLIT_B ? p.a2 : p.a, p.m, p.k, SPLIT_B ? p.a2_row_stride : p.a_row_stride, NT * 8);
  if (rc != LSVD_OK) return rc;
  const int stage_bytes = NMAT * 2 * rows * 128 + (SPLIT_B ? 2 : 1) * 2 * NT * 8 * 128;
  const int red_bytes = kw > 1 ? warps * kw * NMAT * NT * 4 * 32 * 4 : 0;
  const int fixed = 1024 + 2 * kTgMaxStages * 8 + 16 + red_bytes;
  const int budget = device_max_smem_optin() - 4096;
  const int tiles = (p.n + rows - 1) / rows;
  const int ksteps = (p.k + kWideStageK - 1) / kWideStageK;
  const int grid = std::min(tiles, sms);
  const int per_block = ((tiles + grid - 1) / grid) * ksteps;
  const int stages = std::max(1, std::min(std::min((budget - fixed) / stage_bytes, kTgMaxStages), per_block));
  if (fixed + stage_bytes > budget) return LSVD_ERR_UNSUPPORTED;
  const int smem = fixed + stages * stage_bytes;
  void (*kern)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, GemvParams, int, int) =
      kw == 4 ? w8a8_gemv_wide_kernel<NT, DUAL, SPLIT_B, 4>
              : (kw == 2 ? w8a8_gemv_wide_kernel<NT, DUAL, SPLIT_B, 2> : w8a8_gemv_wide_kernel<NT, DUAL, SPLIT_B, 1>);
  LSVD_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem));
  LSVD_CUDA_TRY(launch_chained(kern, dim3(grid), dim3((kWideMaxWarps + 1) * 32), smem, st, 1, false, mw, mw2, ma, ma2, p,
                               stages, warps));
  return LSVD_OK;
}

int launch_gemv_wide(const GemvParams& p, bool dual, bool split, cudaStream_t st) {
  if (p.m <= 32) {
    if (!dual) return launch_wide<4, false, false>(p, st);
    return split ? launch_wide<4, true, true>(p, st) : launch_wide<4, true, false>(p, st);
  }
  if (!dual) return launch_wide<8, false, false>(p, st);
  return split ? launch_wide<8, true, true>(p, st) : launch_wide<8, true, false>(p, st);
}

template <int NT, bool DUAL, bool SPLIT_B>
static int launch_tg(const GemvParams& p, cudaStream_t st) {
  using L = TgLayout<NT, DUAL, SPLIT_B>;
  CUtensorMap mw, mw2, ma, ma2;
  int rc = make_map_k128(&mw, p.w, p.n, p.k, p.w_row_stride, kTgRows);
  if (rc != LSVD_OK) return rc;
  rc = make_map_k128(&mw2, DUAL ? p.w2 : p.w, p.n, p.k, DUAL ? p.w2_row_stride : p.w_row_stride, kTgRows);
  if (rc != LSVD_OK) return rc;
  rc = make_map_k128(&ma, p.a, p.m, p.k, p.a_row_stride, NT * 8);
  if (rc != LSVD_OK) return rc;
  rc = make_map_k128(&ma2, SPLIT_B ? p.a2 : p.a, p.m, p.k, SPLIT_B ? p.a2_row_stride : p.a_row_stride, NT * 8);
  if (rc != LSVD_OK) return rc;
  const int fixed = 1024 /*alignment*/ + L::kRed + 2 * kTgMaxStages * 8 + 16;
  const int budget = device_max_smem_optin() - 4096;
  int stages = (budget - fixed) / L::kStage;
  const int ksteps = (p.k + kTgStageK - 1) / kTgStageK;
  const int tiles = p.n / kTgRows;
  const int sms = std::max(1, device_sm_count());
  const int grid = std::min(tiles, sms);
  const int per_block = ((tiles + grid - 1) / grid) * ksteps;      // stages a block ever fills
  stages = std::max(1, std::min(std::min(stages, kTgMaxStages), per_block));
  if (stages < 1 || fixed + L::kStage > budget) return LSVD_ERR_UNSUPPORTED;
  const int smem = fixed + stages * L::kStage;
  auto kern = w8a8_gemv_tma_kernel<NT, DUAL, SPLIT_B>;
  LSVD_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem));
  LSVD_CUDA_TRY(launch_chained(kern, dim3(grid), dim3(kTgThreads), smem, st, 1, false, mw, mw2, ma, ma2, p, stages));
  return LSVD_OK;
}

int launch_gemv_streamed(const GemvParams& p, bool dual, bool split, cudaStream_t st) {
  if (p.m <= 8) {
    if (!dual) return launch_tg<1, false, false>(p, st);
    return split ? launch_tg<1, true, true>(p, st) : launch_tg<1, true, false>(p, st);
  }
  if (!dual) return launch_tg<2, false, false>(p, st);
  return split ? launch_tg<2, true, true>(p, st) : launch_tg<2, true, false>(p, st);
}

}  // namespace lsvd
