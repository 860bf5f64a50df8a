// The decode step of a layer as persistent kernels: one thread block per SM walks a short program of stages
// (quantisers, weight-streaming products, the attention merge, the cache append) separated by grid barriers,
// instead of one launch per stage.
//
// Why: at decode sizes every stage is a few microseconds long, and a chain of 14 launches spends more time
// between and at the edges of its kernels than inside them.  Here the weights of ALL products of the program
// flow through one ring of shared memory (TMA boxes of 128 rows x 128 bytes, nine stages = 144 KB per SM in
// flight), and the ring runs ahead of the stages: weights do not depend on anything computed in the step, so
// while the blocks meet at a barrier or a few of them run a quantiser, the ring already holds the first tiles
// of the next product, and HBM stays busy.
//
//   product      tcgen05.mma kind::i8 with the WEIGHTS as the 128-row operand and the tokens (at most 16) as the
//                16-column operand: D[128 channels x 16 tokens] in tensor memory.  A product is cut into
//                (128-row tile, 128-byte K block) units; every block takes an equal contiguous run of them, so
//                all SMs stream the same number of bytes whatever the matrix shape.  A block's run covers parts
//                of at most a few row tiles ("pieces"), each with its own 16 accumulator columns; finished pieces
//                are read with tcgen05.ld and ADDED (red.add.s32, exact and order-independent) to global int32
//                accumulators that the program's first stage cleared.  The tokens' int8 activations for the
//                block's K blocks are written by the threads into a swizzled shared-memory panel when the product
//                starts.  Roles: one lane issues TMA, one lane issues MMAs, four warps drain accumulators.
//   finalisers   the dequantising epilogues of the stand-alone products (gemv.cuh) as elementwise stages on
//                the int32 accumulators: latent quantiser, SwiGLU, output + residual.
//   quantisers   the row functions of the stand-alone kernels (devfn.cuh), one token per block; the d_ffn
//                rotation as (token, 8 columns) units.
//   barriers     counters in a caller-provided sync block; every wait (grid barrier, mbarrier) is bounded and
//                reports LSVD_ERR_TIMEOUT; after a timeout the block skips its work but still arrives at every
//                later barrier, so the counters stay consistent for the next launch; tensor memory is released
//                on every path.
//
// (A first version fed the ring with 16-byte cp.async copies and multiplied with mma.sync: measured on B200 the
// copies stalled at issue -- 150 cycles per instruction -- and held up the shared-memory loads behind them; the
// products ran at 1.8 TB/s.  Bulk tensor copies do not pass through the load/store unit at all.)
//
// Values are those of the stand-alone entry points (same device functions, same epilogue arithmetic):
// lsvd_act_quant, lsvd_w8a8_gemv, lsvd_hadamard_quant, lsvd_cache_append, the absorb / merge kernels of
// lsvd_attn_decode.  What it replaces in the reference is what those replace:
// fake_quant/utils/hybrid_ffn_utils.py:956-984 (FFN), kernels/layer_bench/ffn_kernel/baseline_kernel.py:107-145
// (attention block around the decode attention), fd_kernel/destindex_copy_quantize_latent.py:7-50,
// fd_kernel/flash_latent_per_head_decoding_stage2.py:7-48.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>

#include "fused.cuh"
#include "gemv.cuh"
#include "tc5.cuh"
#include "tma.cuh"

namespace lsvd {

// ----------------------------------------------------------------------------------------------
// small device helpers
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Writes to shared memory by ordinary stores become visible to the tensor core's reads (async proxy).
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ----------------------------------------------------------------------------------------------
// grid barriers on monotonic counters
// ----------------------------------------------------------------------------------------------
// sync[0] = number of launches completed on this block of words (epoch), sync[1] = blocks that have left (all
// launches), sync[2] = epoch + 1 of a launch that gave up, sync[8 + i] = arrivals at barrier i (all launches),
// sync[32 + t] = arrivals of the rotation units of token t.  Nothing is ever reset: launch e waits for counter i to
// reach (e + 1) * gridDim.x.  All launches that share a sync block must have the same grid size and be ordered on a stream.
constexpr uint64_t kGridWaitNs = 1000000000ull;

struct GridSync {
  uint32_t* w;
  uint32_t epoch, nblocks;
  int32_t* status_word;
  volatile int* aborted;   // shared-memory flag of this block
};

__device__ __forceinline__ void grid_arrive(const GridSync& gs, int i) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(&gs.w[8 + i], 1u);
  }
}

__device__ __forceinline__ void grid_wait(const GridSync& gs, int i) {
  if (threadIdx.x == 0 && *gs.aborted == 0) {
    const uint32_t target = (gs.epoch + 1u) * gs.nblocks;
    const uint64_t t0 = global_timer_ns();
    uint32_t polls = 0;
    for (;;) {
      const uint32_t v = ld_acquire_u32(&gs.w[8 + i]);
      if (static_cast<int32_t>(v - target) >= 0) break;
      if ((++polls & 63u) == 0u) {
        if (ld_acquire_u32(&gs.w[2]) == gs.epoch + 1u) {     // another block gave up
          *gs.aborted = 1;
          break;
        }
        if (global_timer_ns() - t0 > kGridWaitNs || polls > (1u << 26)) {
          atomicExch(&gs.w[2], gs.epoch + 1u);
          report_status(gs.status_word, LSVD_ERR_TIMEOUT);
          *gs.aborted = 1;
          break;
        }
      }
      __nanosleep(32);
    }
  }
  __syncthreads();
}

__device__ __forceinline__ void grid_barrier(const GridSync& gs, int i) {
  grid_arrive(gs, i);
  grid_wait(gs, i);
}

// ----------------------------------------------------------------------------------------------
// the product engine: TMA ring of weight boxes, tcgen05.mma into tensor memory, red.add epilogue
// ----------------------------------------------------------------------------------------------
struct EngineShared {
  uint64_t full[kFStages], empty[kFStages], acc_full[kFMaxPieces], panel_full;
  uint32_t tmem_base;
};

struct UnitCursor {
  int op, u, u1;        // next unit of this block inside product `op`, end of the block's run
  uint32_t count;       // units passed so far (ring stage = count % kFStages)
};

__device__ __forceinline__ void unit_range(const FOp& o, int& u0, int& u1) {
  const int64_t units = static_cast<int64_t>(o.tiles) * o.kblocks;
  u0 = static_cast<int>(units * blockIdx.x / gridDim.x);
  u1 = static_cast<int>(units * (blockIdx.x + 1) / gridDim.x);
}

__device__ __forceinline__ void cursor_seek(const FusedParams& p, UnitCursor& c, int op) {
  while (op < p.nops) {
    int u0, u1;
    unit_range(p.op[op], u0, u1);
    if (u0 < u1) {
      c.op = op;
      c.u = u0;
      c.u1 = u1;
      return;
    }
    ++op;
  }
  c.op = p.nops;
  c.u = c.u1 = 0;
}

// Issue weight boxes until `upto` units have been asked for in total (or the program has no more).  One thread.
__device__ __forceinline__ void produce(const FusedParams& p, const FMaps& maps, EngineShared& es, uint8_t* ring, UnitCursor& pc,
                                        uint32_t upto, volatile int* aborted) {
  while (pc.op < p.nops && pc.count < upto && *aborted == 0) {
    const uint32_t s = pc.count % kFStages, round = pc.count / kFStages;
    if (round > 0 && !mbar_wait_bounded(&es.empty[s], (round - 1u) & 1u)) {
      report_status(p.status_word, LSVD_ERR_TIMEOUT);
      *aborted = 1;
      return;
    }
    const FOp& o = p.op[pc.op];
    const int tile = pc.u / o.kblocks, kb = pc.u - tile * o.kblocks;
    mbar_arrive_expect_tx(&es.full[s], kFStageBytes);
    tma_load_2d(ring + s * kFStageBytes, &maps.w[pc.op], kb * 128, tile * 128, &es.full[s]);
    ++pc.count;
    if (++pc.u >= pc.u1) cursor_seek(p, pc, pc.op + 1);
  }
}

// ---- the activation panel: tcgen05 B tiles of 16 rows (tokens) x 128 bytes of K, rows of absent tokens and bytes
// beyond K zero, 16-byte pieces swizzled like TMA would (piece j of row r at j ^ (r & 7)) ----
__device__ __forceinline__ uint8_t* panel_piece(uint8_t* panel, int tile, int r, int j) {
  return panel + tile * 2048 + r * 128 + ((j ^ (r & 7)) << 4);
}

__device__ __forceinline__ uint4 quantise16(const uint4& v0, const uint4& v1, float sc) {
  const __half2* h0 = reinterpret_cast<const __half2*>(&v0);
  const __half2* h1 = reinterpret_cast<const __half2*>(&v1);
  uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 a = __half22float2(h0[e]), b = __half22float2(h1[e]);
    w[e >> 1] |= static_cast<uint32_t>(static_cast<uint8_t>(act_code(a.x, sc))) << (16 * (e & 1));
    w[e >> 1] |= static_cast<uint32_t>(static_cast<uint8_t>(act_code(a.y, sc))) << (16 * (e & 1) + 8);
    w[2 + (e >> 1)] |= static_cast<uint32_t>(static_cast<uint8_t>(act_code(b.x, sc))) << (16 * (e & 1));
    w[2 + (e >> 1)] |= static_cast<uint32_t>(static_cast<uint8_t>(act_code(b.y, sc))) << (16 * (e & 1) + 8);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// `ntiles` panel tiles; tile i holds K block kb_of(i).  All loads of a batch of eight pieces per thread are in
// flight together: a dependent global load costs a microsecond while the weight stream runs.
template <typename KbOf>
__device__ __forceinline__ void write_panel(const FOp& o, int m, int ntiles, KbOf kb_of, uint8_t* panel) {
  const int pieces = ntiles * 128;
  constexpr int kBatch = 8;
  for (int p0 = threadIdx.x; p0 < pieces; p0 += kBatch * blockDim.x) {
    uint4 v[kBatch], v2[kBatch];
    float sc[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int pi = p0 + u * blockDim.x;
      v[u] = v2[u] = make_uint4(0u, 0u, 0u, 0u);
      sc[u] = 1.f;
      if (pi < pieces) {
        const int i = pi >> 7, r = (pi >> 3) & 15, j = pi & 7;
        const int col = kb_of(i) * 128 + j * 16;
        if (r < m && col < o.panel_k) {
          if (o.act_kind == 0) {
            v[u] = __ldcg(reinterpret_cast<const uint4*>(o.a + r * o.a_stride + col));
          } else {
            const uint4* src = reinterpret_cast<const uint4*>(o.a16 + r * o.a16_stride + col);
            v[u] = __ldcg(src);
            v2[u] = __ldcg(src + 1);
            sc[u] = act_scale_of(__uint_as_float(__ldcg(o.a_amax + r * o.a_amax_stride)));
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int pi = p0 + u * blockDim.x;
      if (pi < pieces) {
        const int i = pi >> 7, r = (pi >> 3) & 15, j = pi & 7;
        *reinterpret_cast<uint4*>(panel_piece(panel, i, r, j)) = o.act_kind == 0 ? v[u] : quantise16(v[u], v2[u], sc[u]);
      }
    }
  }
}

// One box of a 3-D tensor map (128 bytes x tokens x K blocks) into shared memory.
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}

struct EngineState {
  UnitCursor load;          // producer position (thread 0)
  uint32_t consumed;        // units of all products finished so far by this block (same in every thread)
  uint32_t acc_phase;       // bit i: parity of the next completion of acc_full[i]
  uint32_t panel_phase;     // parity of the next completion of panel_full
};

// This block's units of the products k0 .. k0 + nk - 1, which share one activation panel.  All threads enter and
// leave together.  With arrive_after > 0 the block arrives at grid barrier `arrive_bar` as soon as its additions for the
// group's first arrive_after products are done (the others need not wait for that).
__device__ __forceinline__ void run_group(const FusedParams& p, const FMaps& maps, int k0, int nk, EngineShared& es, EngineState& st,
                                          uint8_t* ring, uint8_t* panel, float* zscale, volatile int* aborted, const GridSync& gs,
                                          int arrive_after, int arrive_bar) {
  const FOp& o0 = p.op[k0];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int total_units = 0, total_pieces = 0;
  for (int k = k0; k < k0 + nk; ++k) {
    int u0, u1;
    unit_range(p.op[k], u0, u1);
    total_units += u1 - u0;
    if (u1 > u0) total_pieces += (u1 - 1) / p.op[k].kblocks - u0 / p.op[k].kblocks + 1;
  }
  // ---- the panel: bulk tensor copies issued by one thread (the MMA issuer waits for them on an mbarrier), or written
  // by all threads when the codes are made on the way in ----
  int rel_u0 = 0, rel_n = 0;
  if (!o0.panel_full) {
    int u0, u1;
    unit_range(o0, u0, u1);
    rel_u0 = u0;
    rel_n = u1 - u0;
  }
  if (o0.panel_tma) {
    if (threadIdx.x == 0 && total_units > 0) {
      if (o0.panel_full) {
        const int boxes = ((o0.panel_k + 127) / 128 + 7) / 8;
        mbar_arrive_expect_tx(&es.panel_full, static_cast<uint32_t>(boxes) * 8u * 2048u);
        for (int bx = 0; bx < boxes; ++bx) tma_load_3d(panel + bx * 8 * 2048, &maps.a8[k0], 0, 0, bx * 8, &es.panel_full);
      } else {
        mbar_arrive_expect_tx(&es.panel_full, static_cast<uint32_t>(rel_n) * 2048u);
        for (int i = 0; i < rel_n; ++i)
          tma_load_3d(panel + i * 2048, &maps.a1[k0], 0, 0, (rel_u0 + i) % o0.kblocks, &es.panel_full);
      }
    }
  } else {
    if (o0.panel_full) {
      write_panel(o0, p.m, (o0.panel_k + 127) >> 7, [](int i) { return i; }, panel);
    } else {
      const int u0 = rel_u0, kblocks = o0.kblocks;
      write_panel(o0, p.m, rel_n, [u0, kblocks](int i) { return (u0 + i) % kblocks; }, panel);
    }
    fence_proxy_async_smem();
    __syncthreads();
  }

  if (warp == 0) {
    if (lane == 0) produce(p, maps, es, ring, st.load, st.consumed + static_cast<uint32_t>(total_units) + kFStages, aborted);
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_i8(128, 16);
      uint32_t cnt = st.consumed;
      int piece = -1;
      bool ok = true;
      if (o0.panel_tma && total_units > 0 && !mbar_wait_bounded(&es.panel_full, st.panel_phase & 1u)) {
        report_status(p.status_word, LSVD_ERR_TIMEOUT);
        *aborted = 1;
        ok = false;
      }
      const uint64_t ring_desc = smem_desc_k_major_sw128(ring), panel_desc = smem_desc_k_major_sw128(panel);
      uint32_t s = cnt % kFStages, par = (cnt / kFStages) & 1u;
      for (int k = k0; k < k0 + nk && ok; ++k) {
        const FOp& o = p.op[k];
        int u0, u1;
        unit_range(o, u0, u1);
        if (u0 >= u1) continue;
        int tile = u0 / o.kblocks, kb = u0 - tile * o.kblocks;
        bool first = true;
        for (int u = u0; u < u1; ++u) {
          if (first) ++piece;
          if (!mbar_try_wait(&es.full[s], par) && (*aborted != 0 || !mbar_wait_bounded(&es.full[s], par))) {
            report_status(p.status_word, LSVD_ERR_TIMEOUT);
            *aborted = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const int ptile = o0.panel_full ? o.a_kb0 + kb : u - rel_u0;
          const uint64_t adesc = ring_desc + static_cast<uint64_t>(s * (kFStageBytes >> 4));
          const uint64_t bdesc = panel_desc + static_cast<uint64_t>(ptile * (2048 >> 4));
          const uint32_t tmem_d = es.tmem_base + static_cast<uint32_t>(piece * 16);
          // 32 int8 of K per instruction: 32 bytes (two 16-byte units) further inside the swizzled row
          umma_i8(tmem_d, adesc, bdesc, idesc, first ? 0u : 1u);
          umma_i8(tmem_d, adesc + 2, bdesc + 2, idesc, 1u);
          umma_i8(tmem_d, adesc + 4, bdesc + 4, idesc, 1u);
          umma_i8(tmem_d, adesc + 6, bdesc + 6, idesc, 1u);
          umma_commit(&es.empty[s]);                                        // the stage is free once these MMAs have read it
          first = false;
          if (++kb == o.kblocks) {
            kb = 0;
            ++tile;
            first = true;
          }
          if (first || u + 1 == u1) umma_commit(&es.acc_full[piece]);
          if (++s == kFStages) {
            s = 0;
            par ^= 1u;
          }
        }
      }
    }
  } else if (warp >= 4) {
    // ---- accumulators of finished pieces: lane = channel, 16 columns = tokens; added to the global accumulators ----
    const int quarter = warp & 3;
    int piece = 0;
    bool ok = true;
    for (int k = k0; k < k0 + nk; ++k) {
      const FOp& o = p.op[k];
      int u0, u1;
      unit_range(o, u0, u1);
      if (ok && u1 > u0) {
        const int tile0 = u0 / o.kblocks, tile1 = (u1 - 1) / o.kblocks;
        for (int tile = tile0; tile <= tile1; ++tile, ++piece) {
          if (*aborted != 0 || !mbar_wait_bounded(&es.acc_full[piece], (st.acc_phase >> piece) & 1u)) {
            report_status(p.status_word, LSVD_ERR_TIMEOUT);
            *aborted = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          uint32_t v[16];
          tmem_ld16(es.tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(piece * 16), v);
          const int row = tile * 128 + quarter * 32 + lane;
          if (row < o.n) {
#pragma unroll
            for (int j = 0; j < kFMaxTokens; ++j)
              if (j < p.m) atomicAdd(o.acc + j * o.acc_stride + row, static_cast<int>(v[j]));
          }
        }
      }
      if (arrive_after > 0 && k == k0 + arrive_after - 1) {
        // the four epilogue warps are done with the first products: one of their threads arrives for the block
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (threadIdx.x == 128) {
          __threadfence();
          atomicAdd(&gs.w[8 + arrive_bar], 1u);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  st.consumed += static_cast<uint32_t>(total_units);
  st.acc_phase ^= (1u << total_pieces) - 1u;
  if (o0.panel_tma && total_units > 0) st.panel_phase ^= 1u;
}

// ----------------------------------------------------------------------------------------------
// finalisers: the epilogues of gemv_store (gemv.cuh) on the int32 accumulators
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ __half dequant16(int acc, float sa, float sw) { return __float2half_rn((static_cast<float>(acc) * sa) * sw); }

__device__ __forceinline__ __half swiglu16(__half g, __half u) {
  const __half sg = __float2half_rn(silu_f(__half2float(g)));
  return __float2half_rn(__half2float(sg) * __half2float(u));
}

// Latents of the SVD branch: one (token, gate | up) unit per block: lat = fp16((acc x_s) U_s), per-unit absmax, codes.
__device__ __forceinline__ void latent_quant_unit(const FusedParams& p, const FOp& oU, int tok, int half, float* buf, float* red) {
  const int r = p.rank;
  const float xs = __ldcg(p.x_scale + tok);
  float amax = 0.f;
  for (int i = threadIdx.x; i < r; i += blockDim.x) {
    const int ch = half * r + i;
    const float v = __half2float(dequant16(__ldcg(oU.acc + tok * oU.acc_stride + ch), xs, __ldg(p.U_s + ch)));
    buf[i] = v;
    amax = fmaxf(amax, fabsf(v));
  }
  amax = block_max(amax, red);
  const float s = act_scale_of(amax);
  if (threadIdx.x == 0) p.z_s[tok * 2 + half] = s;
  for (int i = threadIdx.x; i < r; i += blockDim.x) p.z_q[static_cast<int64_t>(tok) * 2 * r + half * r + i] = act_code(buf[i], s);
  __syncthreads();
}

// (H_K kron H_64) rotation + per-token quantisation, one (token, group of 8 columns) unit per block: the arithmetic
// of hadamard_quant_rows_kernel (ffn_decode.cu).  Every unit rotates all K blocks of 64 entries (cheap) and keeps the
// 8 columns it owns, multiplies them by had_K on the tensor cores (the fragments of had_K are requested before
// anything else, so that their latency hides behind the rotation), and the 8 units of a token agree on the row's
// absmax through one atomic maximum and a counter they alone wait on (bounded), then quantise from registers.
constexpr int kHadIter = 6;     // groups of four 64-entry blocks per warp: K <= 192
constexpr int kHadTiles = 12;   // 16-row tiles of had_K: Kp <= 192

__device__ __forceinline__ void hadamard_unit(const HadQuantParams& p, int r, int cg, uint8_t* scratch, float* red,
                                              uint32_t* amax_word, uint32_t* count_word, uint32_t count_target,
                                              int32_t* status_word, int* flag) {
  const int K = p.K, ld = p.ld;
  __half* Tt = reinterpret_cast<__half*>(scratch);             // [8][ld]: my columns of every rotated block
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int tiles = p.Kp >> 4;
  // ---- fragments of had_K for this warp's (at most two) row tiles: all requested now ----
  uint4 af[2][kHadTiles];
#pragma unroll
  for (int mi = 0; mi < 2; ++mi) {
    const int mt = warp + mi * kFWarps;
    const uint4* ap = p.packed + (static_cast<int64_t>(mt) * tiles) * 32 + lane;
#pragma unroll
    for (int kt = 0; kt < kHadTiles; ++kt)
      af[mi][kt] = (mt < tiles && kt < tiles) ? __ldg(ap + kt * 32) : make_uint4(0u, 0u, 0u, 0u);
  }
  const __half* xg = p.x + r * p.x_row_stride;
  for (int i = threadIdx.x; i < 8 * (p.Kp - K); i += blockDim.x) {
    const int j = i / (p.Kp - K), k = K + (i - j * (p.Kp - K));
    Tt[j * ld + k] = __float2half_rn(0.f);
  }
  {
    const int sub = lane & 7, quad = lane >> 3;
    uint4 xv[kHadIter];
#pragma unroll
    for (int it = 0; it < kHadIter; ++it) {
      const int k = (warp + it * kFWarps) * 4 + quad;
      xv[it] = make_uint4(0u, 0u, 0u, 0u);
      if (k < K) xv[it] = __ldcg(reinterpret_cast<const uint4*>(xg + k * 64) + sub);
    }
#pragma unroll
    for (int it = 0; it < kHadIter; ++it) {
      const int k = (warp + it * kFWarps) * 4 + quad;
      if ((warp + it * kFWarps) * 4 >= K) break;
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
          const float o2 = __shfl_xor_sync(0xffffffffu, e[i], h);
          e[i] = (sub & h) ? o2 - e[i] : e[i] + o2;
        }
      if (k < K && sub == cg) {                    // entries 8 sub .. 8 sub + 7 of block k: my columns
#pragma unroll
        for (int i = 0; i < 8; ++i) Tt[i * ld + k] = __float2half_rn(e[i] * p.rot_scale);
      }
    }
  }
  __syncthreads();

  float d[2][4];
  float amax = 0.f;
#pragma unroll
  for (int mi = 0; mi < 2; ++mi) {
    const int mt = warp + mi * kFWarps;
#pragma unroll
    for (int c = 0; c < 4; ++c) d[mi][c] = 0.f;
    if (mt < tiles) {
#pragma unroll
      for (int kt = 0; kt < kHadTiles; ++kt) {
        if (kt < tiles) {
          const __half* brow = Tt + g * ld + kt * 16 + 2 * t;
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(brow);
          const uint32_t b1 = *reinterpret_cast<const uint32_t*>(brow + 8);
          mma_f16_16x8x16(d[mi], af[mi][kt].x, af[mi][kt].y, af[mi][kt].z, af[mi][kt].w, b0, b1);
        }
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        d[mi][c] = __half2float(__float2half_rn(d[mi][c]));        // the reference's fp16 result
        if (mt * 16 + g + 8 * (c >> 1) < K) amax = fmaxf(amax, fabsf(d[mi][c]));
      }
    }
  }
  amax = block_max(amax, red);
  // ---- the row's absmax: eight units, one word, one counter ----
  if (threadIdx.x == 0) {
    atomicMax(amax_word, __float_as_uint(amax));
    __threadfence();
    atomicAdd(count_word, 1u);
    const uint64_t t0 = global_timer_ns();
    uint32_t polls = 0;
    while (static_cast<int32_t>(ld_acquire_u32(count_word) - count_target) < 0) {
      if ((++polls & 63u) == 0u && (global_timer_ns() - t0 > kGridWaitNs || polls > (1u << 26))) {
        report_status(status_word, LSVD_ERR_TIMEOUT);
        break;
      }
      __nanosleep(20);
    }
    *flag = static_cast<int>(ld_acquire_u32(amax_word));
  }
  __syncthreads();
  const float s = act_scale_of(__int_as_float(*flag));
  if (cg == 0 && threadIdx.x == 0) p.scale[r] = s;
  int8_t* q = p.q + r * p.q_row_stride;
#pragma unroll
  for (int mi = 0; mi < 2; ++mi) {
    const int mt = warp + mi * kFWarps;
    if (mt < tiles) {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int row = mt * 16 + g + 8 * hf;
        if (row < K) {
          const uint16_t packed = static_cast<uint16_t>(static_cast<uint8_t>(act_code(d[mi][2 * hf], s))) |
                                  (static_cast<uint16_t>(static_cast<uint8_t>(act_code(d[mi][2 * hf + 1], s))) << 8);
          *reinterpret_cast<uint16_t*>(q + row * 64 + cg * 8 + 2 * t) = packed;
        }
      }
    }
  }
  __syncthreads();
}

// Merge of the partial results of a (request, head): one warp per unit.
__device__ __forceinline__ void merge_units(const FMerge& mg, int m, int warp, int lane) {
  const int units = m * mg.num_heads;
  for (int u = blockIdx.x * kFWarps + warp; u < units; u += gridDim.x * kFWarps) {
    const int b = u / mg.num_heads, h = u - b * mg.num_heads;
    const int v0 = mg.v_off[h], rv = mg.v_off[h + 1] - v0;
    const int ntiles = (__ldg(mg.b_seq_len + b) + 31) / 32;
    int nparts = (ntiles + mg.chunk_tiles[h] - 1) / mg.chunk_tiles[h];
    if (nparts > mg.parts[h]) nparts = mg.parts[h];
    const float* ml = mg.part_ml + (static_cast<int64_t>(b) * mg.items_per_request + mg.part_off[h]) * 2;
    float M = -INFINITY;
    for (int k = lane; k < nparts; k += 32) M = fmaxf(M, __ldcg(ml + k * 2));
    M = warp_max(M);
    float denom = 0.f;
    for (int k = lane; k < nparts; k += 32) denom += __ldcg(ml + k * 2 + 1) * exp2f(__ldcg(ml + k * 2) - M);
    denom = warp_sum(denom);
    const float* pa = mg.part_acc + static_cast<int64_t>(b) * mg.acc_per_request + mg.acc_off[h];
    float num[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < nparts; ++k) {
      const float w = exp2f(__ldcg(ml + k * 2) - M);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (lane + 32 * i < rv) num[i] = fmaf(__ldcg(pa + static_cast<int64_t>(k) * rv + lane + 32 * i), w, num[i]);
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (lane + 32 * i < rv) {
        const __half o = __float2half_rn(nparts > 0 ? num[i] / denom : 0.f);
        mg.out_latent[b * mg.out_latent_stride + v0 + lane + 32 * i] = o;
        amax = fmaxf(amax, fabsf(__half2float(o)));
      }
    amax = warp_max(amax);
    if (lane == 0 && mg.amax != nullptr) atomicMax(mg.amax + b, __float_as_uint(amax));
  }
}


// Cache append (K and V) and query absorption of a (request, head): one warp per unit.  The arithmetic of
// cache_append_kernel (cache_append.cu) and of absorb_query_kernel (attn_decode.cu); the latents are dequantised
// from the latent projection's accumulators on the way in.
__device__ __forceinline__ float latent_value(const FAppend& ap, int b, int col) {
  return __half2float(dequant16(__ldcg(ap.lat_acc + static_cast<int64_t>(b) * ap.lat_stride + col), __ldcg(ap.x_scale + b),
                                __ldg(ap.w_scale + col)));
}

template <int kRounding>
__device__ __forceinline__ void append_side(const FAppend& ap, int b, int h, int dest, int lane, bool is_v) {
  const int r0 = is_v ? ap.v_off[h] : ap.k_off[h];
  const int rank = (is_v ? ap.v_off[h + 1] : ap.k_off[h + 1]) - r0;
  const int i0 = lane * 4;
  const bool active = i0 < rank;
  float x[4] = {0.f, 0.f, 0.f, 0.f};
  if (active) {
    const int col = (is_v ? ap.v_col : ap.k_col) + r0 + i0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      x[j] = latent_value(ap, b, col + j);
      if (ap.lat_out != nullptr) ap.lat_out[static_cast<int64_t>(b) * ap.lat_stride + col + j] = __float2half_rn(x[j]);
    }
  }
  float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
  amax = warp_max(amax);
  const __half s16 = latent_scale_of(amax);
  const float sf = __half2float(s16), rsf = __frcp_rn(sf);
  int8_t* cache = is_v ? ap.cache_v : ap.cache_k;
  const int64_t row_stride = is_v ? ap.cache_v_row_stride : ap.cache_k_row_stride;
  __half* scale = is_v ? ap.scale_v : ap.scale_k;
  const int64_t scale_stride = is_v ? ap.scale_v_row_stride : ap.scale_k_row_stride;
  if (dest < 0) return;              // slot out of range: reported by the caller, nothing written
  if (active) {
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) packed |= (static_cast<uint32_t>(quantise_one<kRounding>(x[j], sf, rsf)) & 0xffu) << (8 * j);
    int8_t* dst = ap.head_major ? cache + static_cast<int64_t>(r0) * ap.num_slots + static_cast<int64_t>(dest) * rank + i0
                                : cache + static_cast<int64_t>(dest) * row_stride + r0 + i0;
    *reinterpret_cast<uint32_t*>(dst) = packed;
  }
  if (lane == 0) {
    if (ap.head_major) scale[static_cast<int64_t>(h) * ap.num_slots + dest] = s16;
    else scale[static_cast<int64_t>(dest) * scale_stride + h] = s16;
  }
}

constexpr int kLimbMaxF = 63 * (16384 + 128 + 1);

__device__ __forceinline__ void append_absorb_units(const FAppend& ap, int m, int32_t* status_word, float* qbuf, int warp, int lane) {
  if (blockIdx.x == 0 && threadIdx.x == 0) *ap.queue = 0;
  const int units = m * ap.num_heads;
  float* qs = qbuf + warp * 256;
  for (int u = blockIdx.x * kFWarps + warp; u < units; u += gridDim.x * kFWarps) {
    const int b = u / ap.num_heads, h = u - b * ap.num_heads;
    int dest = __ldg(ap.dest_loc + b);
    if (dest < 0 || dest >= ap.num_slots) {
      if (lane == 0) report_status(status_word, LSVD_ERR_BOUNDS);
      dest = -1;
    }
    if (ap.rounding == LSVD_ROUND_TORCH) {
      append_side<LSVD_ROUND_TORCH>(ap, b, h, dest, lane, false);
      append_side<LSVD_ROUND_TORCH>(ap, b, h, dest, lane, true);
    } else {
      append_side<LSVD_ROUND_TRITON>(ap, b, h, dest, lane, false);
      append_side<LSVD_ROUND_TRITON>(ap, b, h, dest, lane, true);
    }
    // ---- absorbed query: q~ = C_h q_lat, then three balanced base-128 limbs per entry and one step per head ----
    const int D = ap.rank_q;
    __syncwarp();
    for (int d = lane; d < D; d += 32) {
      const float v = latent_value(ap, b, ap.q_col + h * D + d);
      qs[d] = v;
      if (ap.lat_out != nullptr) ap.lat_out[static_cast<int64_t>(b) * ap.lat_stride + ap.q_col + h * D + d] = __float2half_rn(v);
    }
    __syncwarp();
    const int r0 = ap.k_off[h], r = ap.k_off[h + 1] - r0;
    float qt[4];
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = lane + 32 * i;
      qt[i] = 0.f;
      if (e < r) {
        const __half* row = ap.up_k + static_cast<int64_t>(r0 + e) * ap.up_k_row_stride;
        float acc = 0.f;
        for (int d0 = 0; d0 < D; d0 += 8) {
          const uint4 v = __ldg(reinterpret_cast<const uint4*>(row + d0));
          const __half2* h2 = reinterpret_cast<const __half2*>(&v);
#pragma unroll
          for (int e2 = 0; e2 < 4; ++e2) {
            const float2 f = __half22float2(h2[e2]);
            acc = fmaf(f.x, qs[d0 + 2 * e2], acc);
            acc = fmaf(f.y, qs[d0 + 2 * e2 + 1], acc);
          }
        }
        qt[i] = acc;
        a = fmaxf(a, fabsf(acc));
      }
    }
    const float amax = warp_max(a);
    const float inv = amax > 0.f ? static_cast<float>(kLimbMaxF) / amax : 0.f;
    if (lane == 0) ap.qstep[b * ap.num_heads + h] = (amax > 0.f ? amax / static_cast<float>(kLimbMaxF) : 0.f) * ap.score_scale;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = lane + 32 * i;
      if (e < r) {
        int Q = __float2int_rn(qt[i] * inv);
        Q = max(-kLimbMaxF, min(kLimbMaxF, Q));
        int c0 = Q & 127; if (c0 >= 64) c0 -= 128;
        const int Q1 = (Q - c0) >> 7;
        int c1 = Q1 & 127; if (c1 >= 64) c1 -= 128;
        const int c2 = (Q1 - c1) >> 7;
        int8_t* out = reinterpret_cast<int8_t*>(ap.qlimb + (static_cast<int64_t>(b) * (ap.sum_rk / 16) + (r0 + e) / 16) * 3);
        out[0 * 16 + (e & 15)] = static_cast<int8_t>(c0);
        out[1 * 16 + (e & 15)] = static_cast<int8_t>(c1);
        out[2 * 16 + (e & 15)] = static_cast<int8_t>(c2);
      }
    }
  }
}

// ----------------------------------------------------------------------------------------------
// the kernel
// ----------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kFThreads, 1)
fused_decode_kernel(const __grid_constant__ FusedParams p, const __grid_constant__ FMaps maps, const __grid_constant__ FMerge mg,
                    const __grid_constant__ FAppend ap) {
  extern __shared__ uint8_t fsmem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fsmem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* panel = ring + kFRing;
  uint8_t* scratch = panel + kFPanel;
  __shared__ EngineShared es;
  __shared__ float red8[8];
  __shared__ float zscale[kFMaxTokens * 2];
  __shared__ volatile int aborted;
  __shared__ int flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    aborted = 0;
    for (int s = 0; s < kFStages; ++s) {
      mbar_init(&es.full[s], 1);
      mbar_init(&es.empty[s], 1);
    }
    for (int i = 0; i < kFMaxPieces; ++i) mbar_init(&es.acc_full[i], 1);
    mbar_init(&es.panel_full, 1);
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(&es.tmem_base, 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  // ---- the ring starts before anything else: weights depend on nothing ----
  grid_dependency_release();
  EngineState st;
  st.consumed = 0;
  st.acc_phase = 0;
  st.panel_phase = 0;
  st.load.count = 0;
  cursor_seek(p, st.load, 0);
  if (threadIdx.x == 0) produce(p, maps, es, ring, st.load, 3, &aborted);      // a short start: the first stage's own loads come first
  grid_dependency_wait();
  __syncthreads();
  GridSync gs;
  gs.w = p.sync;
  gs.epoch = ld_acquire_u32(&p.sync[0]);
  gs.nblocks = gridDim.x;
  gs.status_word = p.status_word;
  gs.aborted = &aborted;
  int bar = 0, opi = 0;
  int prof_i = 0;
  auto stamp = [&]() {
    if (p.prof != nullptr && threadIdx.x == 0 && prof_i < kFProfSlots) p.prof[blockIdx.x * kFProfSlots + prof_i] = global_timer_ns();
    ++prof_i;
  };
  stamp();
  // ---- accumulators and absmax words of this launch start at zero (the first additions come after the first barrier) ----
  for (int z = 0; z < kFMaxZero; ++z)
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < p.zero_count[z]; i += gridDim.x * blockDim.x)
      p.zero_ptr[z][i] = make_uint4(0u, 0u, 0u, 0u);

  if (p.stages & FST_MERGE) {
    merge_units(mg, p.m, warp, lane);
    stamp();
    grid_barrier(gs, bar++);
    stamp();
  }
  if (p.stages & FST_PROJ) {
    if (!aborted) run_group(p, maps, opi, 1, es, st, ring, panel, zscale, &aborted, gs, 0, 0);
    stamp();
    grid_barrier(gs, bar++);
    stamp();
    if (!aborted) {
      const FOp& o = p.op[opi];
      const int total = p.m * o.n;
      for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int tok = i / o.n, ch = i - tok * o.n;
        const float sa = act_scale_of(__uint_as_float(__ldcg(o.a_amax + tok * o.a_amax_stride)));
        __half v = dequant16(__ldcg(o.acc + tok * o.acc_stride + ch), sa, __ldg(p.proj_w_scale + ch));
        if (p.proj_residual != nullptr)
          v = __float2half_rn(__half2float(v) + __half2float(__ldcg(p.proj_residual + static_cast<int64_t>(tok) * p.proj_res_stride + ch)));
        p.proj_out[static_cast<int64_t>(tok) * p.proj_out_stride + ch] = v;
      }
    }
    ++opi;
    stamp();
    grid_barrier(gs, bar++);
    stamp();
    if (blockIdx.x == 0)
      for (int i = threadIdx.x; i < p.clear_late_count; i += blockDim.x) p.clear_late[i] = 0u;
  }
  if (p.stages & FST_QIN) {
    if (!aborted) {
      float* row = reinterpret_cast<float*>(scratch);
      const bool rot = act_quant_rot4096_ok(p.q_in);
      // tokens are spread over the SMs (block t * stride takes token t)
      const int stride = max(1, static_cast<int>(gridDim.x) / max(1, p.q_in.rows));
      if (blockIdx.x % stride == 0) {
        for (int r = blockIdx.x / stride; r < p.q_in.rows; r += (gridDim.x + stride - 1) / stride) {
          if (rot) act_quant_rot4096_row(p.q_in, r, row, red8);
          else act_quant_row(p.q_in, r, row, red8);
          __syncthreads();
        }
      }
    }
    if (threadIdx.x == 0) produce(p, maps, es, ring, st.load, kFStages, &aborted);
    stamp();
    grid_barrier(gs, bar++);
    stamp();
  }
  if (p.stages & FST_LATPROJ) {
    if (!aborted) run_group(p, maps, opi, 1, es, st, ring, panel, zscale, &aborted, gs, 0, 0);
    ++opi;
    stamp();
    grid_barrier(gs, bar++);
    stamp();
    if (!aborted) append_absorb_units(ap, p.m, p.status_word, reinterpret_cast<float*>(scratch), warp, lane);
    stamp();
  }
  if (p.stages & FST_FFN) {
    // products U | W_gate | W_up as one group on one panel; the block arrives at U's barrier as soon as its own
    // additions to U's accumulators are done, and meets it after the group
    const int bar_u = bar++;
    if (!aborted) run_group(p, maps, opi, 3, es, st, ring, panel, zscale, &aborted, gs, 1, bar_u);
    else grid_arrive(gs, bar_u);
    stamp();
    grid_wait(gs, bar_u);
    stamp();
    // latents: dequantise, per-(token, half) absmax, codes
    if (!aborted && static_cast<int>(blockIdx.x) < 2 * p.m)
      latent_quant_unit(p, p.op[opi], blockIdx.x >> 1, blockIdx.x & 1, reinterpret_cast<float*>(scratch), red8);
    stamp();
    grid_barrier(gs, bar++);
    stamp();
    // V_gate | V_up on the two halves of the latent codes
    if (!aborted) run_group(p, maps, opi + 3, 2, es, st, ring, panel, zscale, &aborted, gs, 0, 0);
    stamp();
    grid_barrier(gs, bar++);
    stamp();
    // hidden vector: h = fp16(fp16(silu(g)) u) with g, u dequantised from the gate / up accumulators
    if (!aborted) {
      const FOp& og = p.op[opi + 1];
      const FOp& ou = p.op[opi + 2];
      const FOp& vg = p.op[opi + 3];
      const FOp& vu = p.op[opi + 4];
      const int total = p.m * p.d_ffn;
      for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int tok = i / p.d_ffn, c = i - tok * p.d_ffn;
        __half g, u;
        if (c < p.n_svd) {
          g = dequant16(__ldcg(vg.acc + tok * vg.acc_stride + c), __ldcg(p.z_s + tok * 2), __ldg(p.Vg_s + c));
          u = dequant16(__ldcg(vu.acc + tok * vu.acc_stride + c), __ldcg(p.z_s + tok * 2 + 1), __ldg(p.Vu_s + c));
        } else {
          const int cq = c - p.n_svd;
          const float xs = __ldcg(p.x_scale + tok);
          g = dequant16(__ldcg(og.acc + tok * og.acc_stride + cq), xs, __ldg(p.Wg_s + cq));
          u = dequant16(__ldcg(ou.acc + tok * ou.acc_stride + cq), xs, __ldg(p.Wu_s + cq));
        }
        p.h16[static_cast<int64_t>(tok) * p.d_ffn + c] = swiglu16(g, u);
      }
    }
    stamp();
    grid_barrier(gs, bar++);
    stamp();
    // hidden vector: rotation + quantiser
    if (!aborted) {
      if (p.hq_kind) {
        // one (token, 8 columns) unit per block: the eight units of a token wait for each other, so a block never takes two
        if (static_cast<int>(blockIdx.x) < p.hq.rows * 8) {
          const int r = blockIdx.x >> 3;
          hadamard_unit(p.hq, r, blockIdx.x & 7, scratch, red8, p.hq_amax + r, &p.sync[32 + r], (gs.epoch + 1u) * 8u,
                        p.status_word, &flag);
        }
      } else {
        const int rows = p.hq_plain.rows;
        const int stride = max(1, static_cast<int>(gridDim.x) / max(1, rows));
        if (blockIdx.x % stride == 0) {
          for (int r = blockIdx.x / stride; r < rows; r += (gridDim.x + stride - 1) / stride) {
            act_quant_row(p.hq_plain, r, reinterpret_cast<float*>(scratch), red8);
            __syncthreads();
          }
        }
      }
    }
    stamp();
    grid_barrier(gs, bar++);
    stamp();
    if (!aborted) run_group(p, maps, opi + 5, 1, es, st, ring, panel, zscale, &aborted, gs, 0, 0);
    stamp();
    grid_barrier(gs, bar++);
    stamp();
    if (!aborted) {
      const FOp& o = p.op[opi + 5];
      const int total = p.m * p.d_out;
      for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int tok = i / p.d_out, ch = i - tok * p.d_out;
        __half v = dequant16(__ldcg(o.acc + tok * o.acc_stride + ch), __ldcg(p.h_scale + tok), __ldg(p.Wd_s + ch));
        if (p.out_residual != nullptr)
          v = __float2half_rn(__half2float(v) + __half2float(__ldcg(p.out_residual + static_cast<int64_t>(tok) * p.out_res_stride + ch)));
        p.out[static_cast<int64_t>(tok) * p.out_stride + ch] = v;
      }
    }
    opi += 6;
  }
  stamp();
  // ---- leave: boxes still on their way are waited for (bounded), tensor memory is released, the last block out closes the epoch ----
  if (threadIdx.x == 0 && aborted) {
    for (uint32_t c = st.consumed; c < st.load.count; ++c)
      if (!mbar_wait_bounded(&es.full[c % kFStages], (c / kFStages) & 1u)) break;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(es.tmem_base, 128);
  }
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t old = atomicAdd(&p.sync[1], 1u);
    if (old + 1u == (gs.epoch + 1u) * gs.nblocks) {
      __threadfence();
      atomicExch(&p.sync[0], gs.epoch + 1u);
    }
  }
}

// ----------------------------------------------------------------------------------------------
// host
// ----------------------------------------------------------------------------------------------
bool fused_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("LSVD_FUSED");
    return !(v != nullptr && v[0] == '0');
  }();
  return on;
}

// Tensor maps are made once per (weights, shape) and kept: encoding one costs a driver call.
static std::mutex g_map_mu;
static std::map<std::tuple<const void*, int64_t, int64_t, int64_t>, CUtensorMap> g_maps;

bool fused_prepare_op(FusedParams& p, FMaps& maps, int i, const int8_t* w, int64_t w_stride) {
  FOp& o = p.op[i];
  if (o.k <= 0 || (o.k % 16) != 0 || o.n <= 0 || !aligned(w, 16) || (w_stride % 16) != 0) return false;
  if (o.act_kind == 0 && (!aligned(o.a, 16) || (o.a_stride % 16) != 0)) return false;
  if (o.act_kind == 1 && (!aligned(o.a16, 16) || (o.a16_stride % 8) != 0)) return false;
  o.tiles = (o.n + 127) / 128;
  o.kblocks = (o.k + 127) / 128;
  const int sms = device_sm_count();
  if (sms <= 0) return false;
  const auto key = std::make_tuple(static_cast<const void*>(w), static_cast<int64_t>(o.n), static_cast<int64_t>(o.k), w_stride);
  std::lock_guard<std::mutex> lock(g_map_mu);
  auto it = g_maps.find(key);
  if (it == g_maps.end()) {
    CUtensorMap m;
    if (make_map_k128(&m, w, o.n, o.k, w_stride, 128) != LSVD_OK) return false;
    it = g_maps.emplace(key, m).first;
  }
  maps.w[i] = it->second;
  return true;
}

// Tensor maps of the int8 activations of the group that starts at product k0 (kept like the weight maps).  When the
// driver refuses the layout the panel is written by the threads instead.
static std::map<std::tuple<const void*, int64_t, int64_t, int64_t, int>, CUtensorMap> g_act_maps;

void fused_prepare_panel(FusedParams& p, FMaps& maps, int k0) {
  FOp& o = p.op[k0];
  o.panel_tma = 0;
  if (o.act_kind != 0) return;
  CUtensorMap* dst[2] = {&maps.a8[k0], &maps.a1[k0]};
  const int box[2] = {8, 1};
  std::lock_guard<std::mutex> lock(g_map_mu);
  for (int i = 0; i < 2; ++i) {
    const auto key = std::make_tuple(static_cast<const void*>(o.a), static_cast<int64_t>(p.m), static_cast<int64_t>(o.panel_k),
                                     o.a_stride, box[i]);
    auto it = g_act_maps.find(key);
    if (it == g_act_maps.end()) {
      CUtensorMap m;
      if (make_map_act(&m, o.a, p.m, o.panel_k, o.a_stride, box[i]) != LSVD_OK) return;
      it = g_act_maps.emplace(key, m).first;
    }
    *dst[i] = it->second;
  }
  o.panel_tma = 1;
}

// A group of products on one panel: exact check, over all blocks of the launch, that the pieces fit the tensor
// memory columns and (for a panel that holds a block's own run) that the run fits the panel.
bool fused_check_group(const FusedParams& p, int k0, int nk) {
  const int sms = device_sm_count();
  if (sms <= 0 || nk < 1 || k0 + nk > p.nops) return false;
  const FOp& o0 = p.op[k0];
  if (o0.panel_full) {
    if (o0.panel_k > kFPanelUnits * 128) return false;
    for (int k = k0; k < k0 + nk; ++k)
      if (p.op[k].a_kb0 * 128 + p.op[k].k > o0.panel_k) return false;
  } else if (nk != 1) {
    return false;
  }
  for (int b = 0; b < sms; ++b) {
    int pieces = 0;
    for (int k = k0; k < k0 + nk; ++k) {
      const FOp& o = p.op[k];
      const int64_t units = static_cast<int64_t>(o.tiles) * o.kblocks;
      const int u0 = static_cast<int>(units * b / sms), u1 = static_cast<int>(units * (b + 1) / sms);
      if (u1 > u0) pieces += (u1 - 1) / o.kblocks - u0 / o.kblocks + 1;
      if (!o0.panel_full && u1 - u0 > kFPanelUnits) return false;
    }
    if (pieces > kFMaxPieces) return false;
  }
  return true;
}

static unsigned long long* g_profile = nullptr;

int launch_fused(const FusedParams& p_in, const FMaps& maps, const FMerge* mg, const FAppend* ap, cudaStream_t st, bool chain) {
  FusedParams p = p_in;
  p.prof = g_profile;
  const int sms = device_sm_count();
  if (sms <= 0) return LSVD_ERR_CUDA;
  if (p.m < 1 || p.m > kFMaxTokens || p.nops < 0 || p.nops > kFMaxOps || p.sync == nullptr) return LSVD_ERR_INVALID_ARG;
  if ((p.stages & FST_FFN) && p.hq_kind && p.hq.rows * 8 > sms) return LSVD_ERR_UNSUPPORTED;
  if ((p.stages & FST_FFN) && 2 * p.m > sms) return LSVD_ERR_UNSUPPORTED;
  static const FMerge kNoMerge{};
  static const FAppend kNoAppend{};
  LSVD_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(fused_decode_kernel), kFSmem));
  LSVD_CUDA_TRY(launch_chained(fused_decode_kernel, dim3(sms), dim3(kFThreads), kFSmem, st, 1, chain, p, maps, mg ? *mg : kNoMerge,
                               ap ? *ap : kNoAppend));
  return LSVD_OK;
}

}  // namespace lsvd

extern "C" void lsvd_fused_set_profile(void* device_buffer) { lsvd::g_profile = static_cast<unsigned long long*>(device_buffer); }
