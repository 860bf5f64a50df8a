// int8 latent flash-decoding attention for one query token per request ("absorb" form).
//
// Three kernels per call:
//   1. absorb_query_kernel   q~_h = B_k,h q_h (fp32), stored as three balanced base-128 int8 limbs per
//                            entry plus one fp32 step per head, so that the per-token score is an exact
//                            integer dot product of int8 latents with int8 limbs (dp4a).
//   2. latent_stream_kernel  the HBM stream: persistent blocks walk a flattened (request, head group,
//                            32-token tile) space in equal contiguous shares; a producer warp stages each
//                            tile's K and V row segments with bulk copies (TMA) into a multi-stage shared
//                            memory ring, eight consumer warps score (lane = token), keep an online
//                            softmax per head and accumulate p * scale_v * z_v in registers.
//   3. merge_up_kernel       log-sum-exp merge of the partial results of every block that touched a
//                            (request, head), optional fp16 latent output, V up-projection o = B_v^T o_lat.
//
// What it replaces in the reference: stage 1
// (kernels/layer_bench/fd_kernel/flash_int8_latent_per_head_decoding_rope_stage1.py:32-194) rebuilds every
// key as (z_k . W_uk) * scales and dots it with the query; without a rotary embedding between them the
// up-factor can be applied to the query once instead (r_k multiply-adds per token instead of r_k * D).
// Stage 2 (flash_latent_per_head_decoding_stage2.py:7-48) is the same merge, followed here by the V
// up-projection the reference leaves to a later GEMM (ffn_kernel/baseline_kernel.py:96-99,144-145).
#include <algorithm>
#include <cmath>
#include <cstring>

#include "common.cuh"

namespace lsvd {

constexpr int kTileTokens = 32;          // tokens per tile: one per lane
constexpr int kConsumerWarps = 8;
constexpr int kStreamThreads = (kConsumerWarps + 1) * 32;
constexpr int kMaxGroups = 16;
constexpr int kMaxGroupHeads = 16;
constexpr int kMaxStages = 4;
constexpr int kMaxGroupBytes = 2048;     // K + V bytes of one token inside one head group
constexpr int kAccSlots = 8;             // 16-entry V chunks a consumer warp can accumulate
constexpr int kLimbMax = 63 * (16384 + 128 + 1);   // largest integer three balanced base-128 limbs hold
constexpr float kLog2e = 1.4426950408889634f;

struct WarpPlan {          // what one consumer warp owns inside a head group (at most two heads)
  int16_t head[2];         // global head index, -1 = none
  int16_t local[2];        // index of the head inside its group (row of the staged scale arrays)
  int16_t k_col[2];        // byte offset of the head's K latents inside the group's K segment
  int16_t k_chunks[2];     // r_k / 16
  int16_t v_col[2];
  int16_t v_chunks[2];     // r_v / 16
};

struct GroupPlan {
  int32_t h0, nh;
  int32_t k_seg_off, k_seg_bytes;   // inside a K cache row
  int32_t v_seg_off, v_seg_bytes;
  WarpPlan warp[kConsumerWarps];
};

struct StreamParams {
  const int8_t* cache_k;
  const int8_t* cache_v;
  const __half* scale_k;
  const __half* scale_v;
  int64_t cache_k_row_stride, cache_v_row_stride, scale_k_row_stride, scale_v_row_stride;
  const int32_t* req_to_token;
  int64_t req_to_token_stride;
  const int32_t* b_req_idx;
  const int32_t* b_seq_len;
  const uint4* qlimb;        // [batch][sum_rk/16][3] 16-byte limb vectors
  const float* qstep;        // [batch][H] : step of the limb grid times sm_scale * log2(e)
  float* part_ml;            // [batch][max_parts][H][2]  running max (log2 domain) and sum
  float* part_acc;           // [batch][max_parts][sum_rv] unnormalised accumulators
  int32_t* status_word;
  int32_t batch, num_heads, num_slots, sum_rk, sum_rv;
  int32_t tiles_per_block, max_parts, num_stages;
  int32_t k_tile_bytes, v_tile_bytes, stage_bytes;   // shared memory sizes (rows padded)
  int32_t ngroups;
  GroupPlan g[kMaxGroups];
};

// ----------------------------------------------------------------------------------------------
// 1. query absorption + limb split
// ----------------------------------------------------------------------------------------------
struct AbsorbParams {
  const __half* q;
  int64_t q_stride_b, q_stride_h;
  const __half* up_k;
  int64_t up_k_row_stride;
  uint4* qlimb;
  float* qstep;
  float score_scale;       // sm_scale * log2(e)
  int32_t num_heads, head_dim, sum_rk;
  int32_t k_off[LSVD_MAX_HEADS + 1];
};

__global__ void __launch_bounds__(128) absorb_query_kernel(const __grid_constant__ AbsorbParams p) {
  __shared__ float qs[256];
  __shared__ float qt[LSVD_MAX_RANK];
  __shared__ float wmax[4];
  const int h = blockIdx.x, b = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r0 = p.k_off[h], r = p.k_off[h + 1] - r0;
  const __half* qp = p.q + b * p.q_stride_b + h * p.q_stride_h;
  for (int d = threadIdx.x; d < p.head_dim; d += blockDim.x) qs[d] = __half2float(qp[d]);
  __syncthreads();
  for (int i = warp; i < r; i += 4) {
    const __half* row = p.up_k + static_cast<int64_t>(r0 + i) * p.up_k_row_stride;
    float acc = 0.f;
    for (int d = lane; d < p.head_dim; d += 32) acc = fmaf(__half2float(row[d]), qs[d], acc);
    acc = warp_sum(acc);
    if (lane == 0) qt[i] = acc;
  }
  __syncthreads();
  float a = (threadIdx.x < r) ? fabsf(qt[threadIdx.x]) : 0.f;
  a = warp_max(a);
  if (lane == 0) wmax[warp] = a;
  __syncthreads();
  const float amax = fmaxf(fmaxf(wmax[0], wmax[1]), fmaxf(wmax[2], wmax[3]));
  const float inv = amax > 0.f ? static_cast<float>(kLimbMax) / amax : 0.f;
  if (threadIdx.x == 0)
    p.qstep[b * p.num_heads + h] = (amax > 0.f ? amax / static_cast<float>(kLimbMax) : 0.f) * p.score_scale;
  if (threadIdx.x < r) {
    int Q = __float2int_rn(qt[threadIdx.x] * inv);
    Q = max(-kLimbMax, min(kLimbMax, Q));
    int c0 = Q & 127; if (c0 >= 64) c0 -= 128;
    const int Q1 = (Q - c0) >> 7;
    int c1 = Q1 & 127; if (c1 >= 64) c1 -= 128;
    const int c2 = (Q1 - c1) >> 7;
    const int i = threadIdx.x;
    int8_t* out = reinterpret_cast<int8_t*>(p.qlimb + (static_cast<int64_t>(b) * (p.sum_rk / 16) + (r0 + i) / 16) * 3);
    out[0 * 16 + (i & 15)] = static_cast<int8_t>(c0);
    out[1 * 16 + (i & 15)] = static_cast<int8_t>(c1);
    out[2 * 16 + (i & 15)] = static_cast<int8_t>(c2);
  }
}

// ----------------------------------------------------------------------------------------------
// 2. the stream
// ----------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ int tiles_of(int len) { return (len + kTileTokens - 1) / kTileTokens; }

// Row stride of a staged tile: segment bytes rounded so that (stride / 16) is odd, which makes the
// 16-byte accesses of 8 consecutive lanes (one token each) fall into distinct bank groups.
__host__ __device__ __forceinline__ int padded_row(int seg_bytes) { return ((seg_bytes >> 4) | 1) << 4; }

__device__ __forceinline__ int dp4a_s8(uint32_t a, uint32_t b, int c) {
  return __dp4a(static_cast<int>(a), static_cast<int>(b), c);
}

__global__ void __launch_bounds__(kStreamThreads, 1) latent_stream_kernel(const __grid_constant__ StreamParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);                 // [kMaxStages]
  uint64_t* empty_bar = full_bar + kMaxStages;                            // [kMaxStages]
  uint4* limb_scratch = reinterpret_cast<uint4*>(smem + 128);             // [warp][2 heads][8 chunks][3]
  uint8_t* stage_base = smem + 128 + kConsumerWarps * 2 * 8 * 3 * 16;     // 128 + 6144

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.num_stages; ++s) {
      mbar_init(&full_bar[s], 32);
      mbar_init(&empty_bar[s], kConsumerWarps);
    }
    fence_mbar_init();
  }
  __syncthreads();

  // This block's share of the flattened tile space.  The host bounds the space with max_len_in_batch;
  // the real lengths are read here, so trailing blocks may find nothing.
  const int64_t first = static_cast<int64_t>(blockIdx.x) * p.tiles_per_block;
  const int64_t last = first + p.tiles_per_block;      // exclusive
  // Locate `first`: requests in order, groups inside a request, tiles inside a group.
  int b = 0, g = 0, tile = 0, len = 0, ntiles = 0;
  int64_t base = 0;          // flattened index of tile 0 of request b, group 0
  bool found = false;
  for (; b < p.batch; ++b) {
    len = p.b_seq_len[b];
    ntiles = tiles_of(len);
    const int64_t span = static_cast<int64_t>(ntiles) * p.ngroups;
    if (first < base + span) {
      const int64_t off = first - base;
      g = static_cast<int>(off / ntiles);
      tile = static_cast<int>(off - static_cast<int64_t>(g) * ntiles);
      found = true;
      break;
    }
    base += span;
  }
  if (!found) return;

  int64_t cur = first;       // flattened index of (b, g, tile)
  uint32_t it = 0;           // tiles pushed through the ring by this block so far
  bool ok = true;

  while (ok && cur < last && b < p.batch) {
    // ---- one item: tiles [tile, tile_end) of (b, g) ----
    const int64_t room = tile + (last - cur);
    const int tile_end = room < ntiles ? static_cast<int>(room) : ntiles;
    const GroupPlan& G = p.g[g];
    const int k_stride = padded_row(G.k_seg_bytes), v_stride = padded_row(G.v_seg_bytes);
    // part index of this block for (b, g): blocks are numbered from the one holding tile 0.
    const int64_t seq_start = base + static_cast<int64_t>(g) * ntiles;
    const int part = static_cast<int>(blockIdx.x - seq_start / p.tiles_per_block);

    if (warp == kConsumerWarps) {
      // ================= producer =================
      const int req = p.b_req_idx[b];
      const int32_t* r2t = p.req_to_token + static_cast<int64_t>(req) * p.req_to_token_stride;
      int tok = tile * kTileTokens + lane;
      int slot_next = (tok < len) ? r2t[tok] : -1;
      for (int t = tile; t < tile_end; ++t, ++it) {
        const int slot = slot_next;
        tok = (t + 1) * kTileTokens + lane;
        slot_next = (t + 1 < tile_end && tok < len) ? r2t[tok] : -1;
        const int stage = it % p.num_stages;
        const uint32_t phase = (it / p.num_stages) & 1u;
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&empty_bar[stage], phase ^ 1u))) {
          report_status(p.status_word, LSVD_ERR_TIMEOUT);
          ok = false;
          break;
        }
        uint8_t* st = stage_base + static_cast<size_t>(stage) * p.stage_bytes;
        __half* sk = reinterpret_cast<__half*>(st + p.k_tile_bytes + p.v_tile_bytes);
        __half* sv = sk + kMaxGroupHeads * kTileTokens;
        bool valid = slot >= 0;
        if (valid && slot >= p.num_slots) {
          report_status(p.status_word, LSVD_ERR_BOUNDS);
          valid = false;
        }
        uint32_t bytes = 0;
        if (valid) {
          bulk_g2s(st + lane * k_stride, p.cache_k + static_cast<int64_t>(slot) * p.cache_k_row_stride + G.k_seg_off,
                   G.k_seg_bytes, &full_bar[stage]);
          bulk_g2s(st + p.k_tile_bytes + lane * v_stride,
                   p.cache_v + static_cast<int64_t>(slot) * p.cache_v_row_stride + G.v_seg_off, G.v_seg_bytes,
                   &full_bar[stage]);
          bytes = G.k_seg_bytes + G.v_seg_bytes;
          const __half* gk = p.scale_k + static_cast<int64_t>(slot) * p.scale_k_row_stride + G.h0;
          const __half* gv = p.scale_v + static_cast<int64_t>(slot) * p.scale_v_row_stride + G.h0;
#pragma unroll 4
          for (int j = 0; j < G.nh; ++j) {
            sk[j * kTileTokens + lane] = gk[j];
            sv[j * kTileTokens + lane] = gv[j];
          }
        } else {
          // A lane past the end of the request: zero scales make its token contribute nothing.
          for (int j = 0; j < G.nh; ++j) {
            sk[j * kTileTokens + lane] = __float2half_rn(0.f);
            sv[j * kTileTokens + lane] = __float2half_rn(0.f);
          }
        }
        mbar_arrive_expect_tx(&full_bar[stage], bytes);
      }
    } else {
      // ================= consumers =================
      const WarpPlan& W = G.warp[warp];
      const int nv0 = W.head[0] >= 0 ? W.v_chunks[0] : 0;
      const int nv1 = W.head[1] >= 0 ? W.v_chunks[1] : 0;
      float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f}, step[2] = {0.f, 0.f};
      float acc[kAccSlots][16];
#pragma unroll
      for (int s = 0; s < kAccSlots; ++s)
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[s][i] = 0.f;

      // Stage this request's limb vectors for the warp's heads in its private scratch.
      uint4* scratch = limb_scratch + warp * (2 * 8 * 3);
      __syncwarp();
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        if (W.head[hh] >= 0) {
          const uint4* src = p.qlimb + (static_cast<int64_t>(b) * (p.sum_rk / 16) +
                                        (G.k_seg_off + W.k_col[hh]) / 16) * 3;
          for (int i = lane; i < W.k_chunks[hh] * 3; i += 32) scratch[hh * 24 + i] = src[i];
          step[hh] = p.qstep[b * p.num_heads + W.head[hh]];
        }
      }
      __syncwarp();

      for (int t = tile; t < tile_end; ++t, ++it) {
        const int stage = it % p.num_stages;
        const uint32_t phase = (it / p.num_stages) & 1u;
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&full_bar[stage], phase))) {
          report_status(p.status_word, LSVD_ERR_TIMEOUT);
          ok = false;
          break;
        }
        const uint8_t* st = stage_base + static_cast<size_t>(stage) * p.stage_bytes;
        const __half* sk = reinterpret_cast<const __half*>(st + p.k_tile_bytes + p.v_tile_bytes);
        const __half* sv = sk + kMaxGroupHeads * kTileTokens;
        const bool tok_valid = (t * kTileTokens + lane) < len;

#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          if (W.head[hh] < 0) continue;
          // ---- scores: exact integer dot of the token's int8 latents with the three limb vectors ----
          const uint8_t* krow = st + lane * k_stride + W.k_col[hh];
          const uint4* ql = scratch + hh * 24;
          int a0 = 0, a1 = 0, a2 = 0;
          const int nk = W.k_chunks[hh];
          for (int c = 0; c < nk; ++c) {
            const uint4 z = *reinterpret_cast<const uint4*>(krow + c * 16);
            const uint4 l0 = ql[c * 3 + 0], l1 = ql[c * 3 + 1], l2 = ql[c * 3 + 2];
            a0 = dp4a_s8(z.x, l0.x, a0); a0 = dp4a_s8(z.y, l0.y, a0); a0 = dp4a_s8(z.z, l0.z, a0); a0 = dp4a_s8(z.w, l0.w, a0);
            a1 = dp4a_s8(z.x, l1.x, a1); a1 = dp4a_s8(z.y, l1.y, a1); a1 = dp4a_s8(z.z, l1.z, a1); a1 = dp4a_s8(z.w, l1.w, a1);
            a2 = dp4a_s8(z.x, l2.x, a2); a2 = dp4a_s8(z.y, l2.y, a2); a2 = dp4a_s8(z.z, l2.z, a2); a2 = dp4a_s8(z.w, l2.w, a2);
          }
          const float dot = fmaf(16384.f, static_cast<float>(a2), fmaf(128.f, static_cast<float>(a1), static_cast<float>(a0)));
          const float ks = __half2float(sk[W.local[hh] * kTileTokens + lane]);
          float s = tok_valid ? dot * (ks * step[hh]) : -INFINITY;     // log2 domain
          // ---- online softmax, maximum shared by the warp ----
          const float mx = warp_max_redux(s);
          const int lo = hh == 0 ? 0 : nv0;
          const int hi = hh == 0 ? nv0 : nv0 + nv1;
          if (mx > m[hh]) {
            const float corr = exp2f(m[hh] - mx);
            l[hh] *= corr;
#pragma unroll
            for (int sl = 0; sl < kAccSlots; ++sl) {
              if (sl >= lo && sl < hi) {
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[sl][i] *= corr;
              }
            }
            m[hh] = mx;
          }
          const float pr = exp2f(s - m[hh]);
          l[hh] += pr;
          const float w = pr * __half2float(sv[W.local[hh] * kTileTokens + lane]);
          // ---- latent V accumulation ----
          const uint8_t* vrow = st + p.k_tile_bytes + lane * v_stride + W.v_col[hh];
#pragma unroll
          for (int sl = 0; sl < kAccSlots; ++sl) {
            if (sl >= lo && sl < hi) {
              const uint4 z = *reinterpret_cast<const uint4*>(vrow + (sl - lo) * 16);
              acc[sl][0] = fmaf(w, s8_to_f32<0>(z.x), acc[sl][0]);
              acc[sl][1] = fmaf(w, s8_to_f32<1>(z.x), acc[sl][1]);
              acc[sl][2] = fmaf(w, s8_to_f32<2>(z.x), acc[sl][2]);
              acc[sl][3] = fmaf(w, s8_to_f32<3>(z.x), acc[sl][3]);
              acc[sl][4] = fmaf(w, s8_to_f32<0>(z.y), acc[sl][4]);
              acc[sl][5] = fmaf(w, s8_to_f32<1>(z.y), acc[sl][5]);
              acc[sl][6] = fmaf(w, s8_to_f32<2>(z.y), acc[sl][6]);
              acc[sl][7] = fmaf(w, s8_to_f32<3>(z.y), acc[sl][7]);
              acc[sl][8] = fmaf(w, s8_to_f32<0>(z.z), acc[sl][8]);
              acc[sl][9] = fmaf(w, s8_to_f32<1>(z.z), acc[sl][9]);
              acc[sl][10] = fmaf(w, s8_to_f32<2>(z.z), acc[sl][10]);
              acc[sl][11] = fmaf(w, s8_to_f32<3>(z.z), acc[sl][11]);
              acc[sl][12] = fmaf(w, s8_to_f32<0>(z.w), acc[sl][12]);
              acc[sl][13] = fmaf(w, s8_to_f32<1>(z.w), acc[sl][13]);
              acc[sl][14] = fmaf(w, s8_to_f32<2>(z.w), acc[sl][14]);
              acc[sl][15] = fmaf(w, s8_to_f32<3>(z.w), acc[sl][15]);
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
      }

      // ---- write this block's partial result for (b, g) ----
      if (ok && part >= 0 && part < p.max_parts) {
        float* ml = p.part_ml + (static_cast<int64_t>(b) * p.max_parts + part) * p.num_heads * 2;
        float* pa = p.part_acc + (static_cast<int64_t>(b) * p.max_parts + part) * p.sum_rv;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          if (W.head[hh] >= 0) {
            const float lsum = warp_sum(l[hh]);
            if (lane == 0) {
              ml[W.head[hh] * 2 + 0] = m[hh];
              ml[W.head[hh] * 2 + 1] = lsum;
            }
          }
        }
#pragma unroll
        for (int sl = 0; sl < kAccSlots; ++sl) {
          if (sl < nv0 + nv1) {
            // Sum the 16 entries of this slot over the 32 lanes (tokens): at each step a lane hands the
            // half it does not keep to its partner, so after five steps lane L holds entry (L >> 1) & 15.
            float* a = acc[sl];
            { const bool up = lane & 16;
#pragma unroll
              for (int i = 0; i < 8; ++i) { const float send = up ? a[i] : a[i + 8]; const float keep = up ? a[i + 8] : a[i];
                a[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16); } }
            { const bool up = lane & 8;
#pragma unroll
              for (int i = 0; i < 4; ++i) { const float send = up ? a[i] : a[i + 4]; const float keep = up ? a[i + 4] : a[i];
                a[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8); } }
            { const bool up = lane & 4;
#pragma unroll
              for (int i = 0; i < 2; ++i) { const float send = up ? a[i] : a[i + 2]; const float keep = up ? a[i + 2] : a[i];
                a[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4); } }
            { const bool up = lane & 2;
              const float send = up ? a[0] : a[1]; const float keep = up ? a[1] : a[0];
              a[0] = keep + __shfl_xor_sync(0xffffffffu, send, 2); }
            a[0] += __shfl_xor_sync(0xffffffffu, a[0], 1);
            const int hh = sl < nv0 ? 0 : 1;
            const int col = G.v_seg_off + W.v_col[hh] + (sl - (hh == 0 ? 0 : nv0)) * 16 + ((lane >> 1) & 15);
            if ((lane & 1) == 0) pa[col] = a[0];
          }
        }
      } else if (ok && lane == 0) {
        report_status(p.status_word, LSVD_ERR_BOUNDS);
      }
    }

    // ---- advance to the next (b, g) ----
    cur += tile_end - tile;
    if (tile_end == ntiles) {
      tile = 0;
      if (++g == p.ngroups) {
        g = 0;
        base += static_cast<int64_t>(ntiles) * p.ngroups;
        for (++b; b < p.batch; ++b) {      // skip empty requests
          len = p.b_seq_len[b];
          ntiles = tiles_of(len);
          if (ntiles > 0) break;
        }
      }
    } else {
      tile = tile_end;
    }
  }

  // A producer that gave up still owns copies in flight: let them land (bounded) before the block's
  // shared memory is released.
  if (!ok && warp == kConsumerWarps) {
    const uint32_t pending = it < static_cast<uint32_t>(p.num_stages) ? it : static_cast<uint32_t>(p.num_stages);
    for (uint32_t k = 0; k < pending; ++k) {
      const uint32_t j = it - 1 - k;
      mbar_wait_bounded(&full_bar[j % p.num_stages], (j / p.num_stages) & 1u);
    }
  }
}

// ----------------------------------------------------------------------------------------------
// 3. merge + V up-projection
// ----------------------------------------------------------------------------------------------
struct MergeParams {
  const float* part_ml;
  const float* part_acc;
  const int32_t* b_seq_len;
  const __half* up_v;
  int64_t up_v_row_stride;
  __half* out;
  int64_t out_stride_b, out_stride_h;
  __half* out_latent;
  int64_t out_latent_stride_b;
  int32_t batch, num_heads, head_dim, sum_rv, ngroups, tiles_per_block, max_parts;
  int32_t v_off[LSVD_MAX_HEADS + 1];
  int16_t head_group[LSVD_MAX_HEADS];
};

__global__ void __launch_bounds__(128) merge_up_kernel(const __grid_constant__ MergeParams p) {
  __shared__ float olat[LSVD_MAX_RANK];
  const int h = blockIdx.x, b = blockIdx.y;
  const int g = p.head_group[h];
  const int v0 = p.v_off[h], rv = p.v_off[h + 1] - v0;
  // Which blocks of the stream kernel touched (b, g): same arithmetic as the stream kernel.
  int64_t base = 0;
  for (int bb = 0; bb < b; ++bb) base += static_cast<int64_t>(tiles_of(p.b_seq_len[bb])) * p.ngroups;
  const int ntiles = tiles_of(p.b_seq_len[b]);
  const int64_t seq_start = base + static_cast<int64_t>(g) * ntiles;
  int nparts = 0;
  if (ntiles > 0) {
    const int64_t c_first = seq_start / p.tiles_per_block;
    const int64_t c_last = (seq_start + ntiles - 1) / p.tiles_per_block;
    nparts = static_cast<int>(c_last - c_first + 1);
    if (nparts > p.max_parts) nparts = p.max_parts;
  }
  const float* ml = p.part_ml + static_cast<int64_t>(b) * p.max_parts * p.num_heads * 2 + h * 2;
  float M = -INFINITY;
  for (int k = 0; k < nparts; ++k) M = fmaxf(M, ml[static_cast<int64_t>(k) * p.num_heads * 2]);
  float denom = 0.f;
  for (int k = 0; k < nparts; ++k)
    denom += ml[static_cast<int64_t>(k) * p.num_heads * 2 + 1] * exp2f(ml[static_cast<int64_t>(k) * p.num_heads * 2] - M);
  const int i = threadIdx.x;
  if (i < rv) {
    float num = 0.f;
    const float* pa = p.part_acc + static_cast<int64_t>(b) * p.max_parts * p.sum_rv + v0 + i;
    for (int k = 0; k < nparts; ++k)
      num += pa[static_cast<int64_t>(k) * p.sum_rv] * exp2f(ml[static_cast<int64_t>(k) * p.num_heads * 2] - M);
    const float o = nparts > 0 ? num / denom : 0.f;
    olat[i] = o;
    if (p.out_latent != nullptr) p.out_latent[b * p.out_latent_stride_b + v0 + i] = __float2half_rn(o);
  }
  __syncthreads();
  if (p.out != nullptr) {
    for (int d = threadIdx.x; d < p.head_dim; d += blockDim.x) {
      float acc = 0.f;
      const __half* col = p.up_v + static_cast<int64_t>(v0) * p.up_v_row_stride + d;
      for (int r = 0; r < rv; ++r) acc = fmaf(olat[r], __half2float(col[static_cast<int64_t>(r) * p.up_v_row_stride]), acc);
      p.out[b * p.out_stride_b + h * p.out_stride_h + d] = __float2half_rn(acc);
    }
  }
}

// ----------------------------------------------------------------------------------------------
// host: planning, validation, launch
// ----------------------------------------------------------------------------------------------
struct HostPlan {
  int ngroups = 0;
  GroupPlan g[kMaxGroups];
  int16_t head_group[LSVD_MAX_HEADS];
  int max_k_seg = 0, max_v_seg = 0;
  int num_stages = 0, stage_bytes = 0, k_tile_bytes = 0, v_tile_bytes = 0, smem_bytes = 0;
  int num_blocks = 0, tiles_per_block = 0, max_parts = 0;
};

// Distribute heads [h0, h0+n) over the consumer warps: longest first onto the least loaded warp that
// still has a free head slot and enough accumulator slots.  Returns false if some head finds no warp.
static bool assign_warps(const int32_t* k_off, const int32_t* v_off, int h0, int n, GroupPlan* out) {
  int order[kMaxGroupHeads];
  for (int i = 0; i < n; ++i) order[i] = h0 + i;
  std::sort(order, order + n, [&](int a, int b) {
    const int la = (k_off[a + 1] - k_off[a]) + (v_off[a + 1] - v_off[a]);
    const int lb = (k_off[b + 1] - k_off[b]) + (v_off[b + 1] - v_off[b]);
    return la != lb ? la > lb : a < b;
  });
  int load[kConsumerWarps] = {0}, cnt[kConsumerWarps] = {0}, vslots[kConsumerWarps] = {0};
  WarpPlan wp[kConsumerWarps];
  for (auto& w : wp) { w.head[0] = w.head[1] = -1; }
  for (int i = 0; i < n; ++i) {
    const int h = order[i];
    const int rk = k_off[h + 1] - k_off[h], rv = v_off[h + 1] - v_off[h];
    int best = -1;
    for (int w = 0; w < kConsumerWarps; ++w) {
      if (cnt[w] >= 2 || vslots[w] + rv / 16 > kAccSlots) continue;
      if (best < 0 || load[w] < load[best]) best = w;
    }
    if (best < 0) return false;
    const int j = cnt[best]++;
    load[best] += rk + rv;
    vslots[best] += rv / 16;
    wp[best].head[j] = static_cast<int16_t>(h);
    wp[best].local[j] = static_cast<int16_t>(h - h0);
    wp[best].k_col[j] = static_cast<int16_t>(k_off[h] - k_off[h0]);
    wp[best].k_chunks[j] = static_cast<int16_t>(rk / 16);
    wp[best].v_col[j] = static_cast<int16_t>(v_off[h] - v_off[h0]);
    wp[best].v_chunks[j] = static_cast<int16_t>(rv / 16);
  }
  if (out != nullptr) {
    out->h0 = h0;
    out->nh = n;
    out->k_seg_off = k_off[h0];
    out->k_seg_bytes = k_off[h0 + n] - k_off[h0];
    out->v_seg_off = v_off[h0];
    out->v_seg_bytes = v_off[h0 + n] - v_off[h0];
    for (int w = 0; w < kConsumerWarps; ++w) out->warp[w] = wp[w];
  }
  return true;
}

static int validate_offsets(const int32_t* off, int num_heads) {
  if (off == nullptr || off[0] != 0) return LSVD_ERR_INVALID_ARG;
  for (int h = 0; h < num_heads; ++h) {
    const int r = off[h + 1] - off[h];
    if (r <= 0 || r > LSVD_MAX_RANK || (r % 16) != 0) return LSVD_ERR_INVALID_ARG;
  }
  return LSVD_OK;
}

static int make_plan(int batch, int num_heads, const int32_t* k_off, const int32_t* v_off, int max_len, HostPlan* hp) {
  if (batch <= 0 || num_heads <= 0 || num_heads > LSVD_MAX_HEADS || max_len < 0) return LSVD_ERR_INVALID_ARG;
  int rc = validate_offsets(k_off, num_heads);
  if (rc != LSVD_OK) return rc;
  rc = validate_offsets(v_off, num_heads);
  if (rc != LSVD_OK) return rc;
  // Greedy contiguous head groups.
  int h = 0;
  hp->ngroups = 0;
  while (h < num_heads) {
    int n = 1;
    while (h + n < num_heads && n < kMaxGroupHeads) {
      const int bytes = (k_off[h + n + 1] - k_off[h]) + (v_off[h + n + 1] - v_off[h]);
      if (bytes > kMaxGroupBytes) break;
      if (!assign_warps(k_off, v_off, h, n + 1, nullptr)) break;
      ++n;
    }
    if (hp->ngroups >= kMaxGroups) return LSVD_ERR_UNSUPPORTED;
    if (!assign_warps(k_off, v_off, h, n, &hp->g[hp->ngroups])) return LSVD_ERR_UNSUPPORTED;
    for (int i = 0; i < n; ++i) hp->head_group[h + i] = static_cast<int16_t>(hp->ngroups);
    hp->max_k_seg = std::max(hp->max_k_seg, hp->g[hp->ngroups].k_seg_bytes);
    hp->max_v_seg = std::max(hp->max_v_seg, hp->g[hp->ngroups].v_seg_bytes);
    ++hp->ngroups;
    h += n;
  }
  hp->k_tile_bytes = ((kTileTokens * padded_row(hp->max_k_seg)) + 127) / 128 * 128;
  hp->v_tile_bytes = ((kTileTokens * padded_row(hp->max_v_seg)) + 127) / 128 * 128;
  hp->stage_bytes = hp->k_tile_bytes + hp->v_tile_bytes + 2 * kMaxGroupHeads * kTileTokens * 2;
  const int fixed = 128 + kConsumerWarps * 2 * 8 * 3 * 16;
  const int budget = device_max_smem_optin();
  if (budget <= 0) return LSVD_ERR_CUDA;
  int stages = (budget - fixed) / hp->stage_bytes;
  stages = std::min(stages, kMaxStages);
  if (stages < 2) return LSVD_ERR_UNSUPPORTED;
  hp->num_stages = stages;
  hp->smem_bytes = fixed + stages * hp->stage_bytes;
  // Equal contiguous shares of the flattened (request, group, tile) space, bounded with max_len.
  const int ntiles_max = (max_len + kTileTokens - 1) / kTileTokens;
  const int64_t total = static_cast<int64_t>(batch) * hp->ngroups * ntiles_max;
  const int sms = device_sm_count();
  if (sms <= 0) return LSVD_ERR_CUDA;
  const int64_t blocks = std::max<int64_t>(1, std::min<int64_t>(sms, total));
  hp->tiles_per_block = static_cast<int>(std::max<int64_t>(1, (total + blocks - 1) / blocks));
  hp->num_blocks = static_cast<int>(std::max<int64_t>(1, (total + hp->tiles_per_block - 1) / hp->tiles_per_block));
  hp->max_parts = (ntiles_max + hp->tiles_per_block - 1) / hp->tiles_per_block + 1;
  return LSVD_OK;
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct WorkspaceLayout {
  size_t qlimb, qstep, part_ml, part_acc, total;
};

static WorkspaceLayout workspace_layout(int batch, int num_heads, int sum_rk, int sum_rv, int max_parts) {
  WorkspaceLayout w{};
  size_t off = 0;
  w.qlimb = off; off = align_up(off + static_cast<size_t>(batch) * (sum_rk / 16) * 48, 256);
  w.qstep = off; off = align_up(off + static_cast<size_t>(batch) * num_heads * 4, 256);
  w.part_ml = off; off = align_up(off + static_cast<size_t>(batch) * max_parts * num_heads * 8, 256);
  w.part_acc = off; off = align_up(off + static_cast<size_t>(batch) * max_parts * sum_rv * 4, 256);
  w.total = off;
  return w;
}

}  // namespace lsvd

extern "C" size_t lsvd_attn_decode_workspace_bytes(int32_t batch, int32_t num_heads, int32_t sum_rank_k,
                                                   int32_t sum_rank_v, int32_t max_len_in_batch) {
  using namespace lsvd;
  if (batch <= 0 || num_heads <= 0 || sum_rank_k <= 0 || sum_rank_v <= 0 || max_len_in_batch < 0) return 0;
  // The number of partial results per request shrinks as head groups are added; one group bounds it.
  const int ntiles_max = (max_len_in_batch + kTileTokens - 1) / kTileTokens;
  const int64_t total = static_cast<int64_t>(batch) * ntiles_max;
  const int sms = std::max(1, device_sm_count());
  const int64_t blocks = std::max<int64_t>(1, std::min<int64_t>(sms, total));
  const int tiles_per_block = static_cast<int>(std::max<int64_t>(1, (total + blocks - 1) / blocks));
  const int max_parts = (ntiles_max + tiles_per_block - 1) / tiles_per_block + 1;
  return workspace_layout(batch, num_heads, sum_rank_k, sum_rank_v, max_parts).total;
}

extern "C" int lsvd_attn_decode_plan(int32_t batch, int32_t num_heads, const int32_t* k_off, const int32_t* v_off,
                                     int32_t max_len_in_batch, int32_t* num_splits, int32_t* num_groups,
                                     int32_t* num_stages, int32_t* num_blocks) {
  lsvd::HostPlan hp;
  const int rc = lsvd::make_plan(batch, num_heads, k_off, v_off, max_len_in_batch, &hp);
  if (rc != LSVD_OK) return rc;
  if (num_splits) *num_splits = hp.max_parts;
  if (num_groups) *num_groups = hp.ngroups;
  if (num_stages) *num_stages = hp.num_stages;
  if (num_blocks) *num_blocks = hp.num_blocks;
  return LSVD_OK;
}

extern "C" int lsvd_attn_decode(const lsvd_attn_decode_args* a, void* stream) {
  using namespace lsvd;
  if (a == nullptr) return LSVD_ERR_INVALID_ARG;
  if (a->batch <= 0 || a->head_dim <= 0 || a->head_dim > 256 || (a->head_dim % 8) != 0) return LSVD_ERR_INVALID_ARG;
  if (a->num_slots <= 0 || a->max_len_in_batch < 0) return LSVD_ERR_INVALID_ARG;
  if (!a->q || !a->cache_k || !a->cache_v || !a->scale_k || !a->scale_v || !a->up_k || !a->req_to_token ||
      !a->b_req_idx || !a->b_seq_len)
    return LSVD_ERR_INVALID_ARG;
  if (a->out == nullptr && a->out_latent == nullptr) return LSVD_ERR_INVALID_ARG;
  if (a->out != nullptr && a->up_v == nullptr) return LSVD_ERR_INVALID_ARG;
  HostPlan hp;
  int rc = make_plan(a->batch, a->num_heads, a->k_off, a->v_off, a->max_len_in_batch, &hp);
  if (rc != LSVD_OK) return rc;
  const int sum_rk = a->k_off[a->num_heads], sum_rv = a->v_off[a->num_heads];
  if (!aligned(a->cache_k, 16) || !aligned(a->cache_v, 16) || (a->cache_k_row_stride % 16) != 0 ||
      (a->cache_v_row_stride % 16) != 0 || a->cache_k_row_stride < sum_rk || a->cache_v_row_stride < sum_rv)
    return LSVD_ERR_INVALID_ARG;
  if (a->scale_k_row_stride < a->num_heads || a->scale_v_row_stride < a->num_heads) return LSVD_ERR_INVALID_ARG;
  if (!aligned(a->q, 2) || !aligned(a->up_k, 2) || !aligned(a->scale_k, 2) || !aligned(a->scale_v, 2))
    return LSVD_ERR_INVALID_ARG;
  const WorkspaceLayout wl = workspace_layout(a->batch, a->num_heads, sum_rk, sum_rv, hp.max_parts);
  if (a->workspace == nullptr || a->workspace_bytes < wl.total || !aligned(a->workspace, 256)) return LSVD_ERR_WORKSPACE;
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float sm_scale = a->sm_scale > 0.f ? a->sm_scale : 1.0f / std::sqrt(static_cast<float>(a->head_dim));

  AbsorbParams ap{};
  ap.q = static_cast<const __half*>(a->q);
  ap.q_stride_b = a->q_stride_b;
  ap.q_stride_h = a->q_stride_h;
  ap.up_k = static_cast<const __half*>(a->up_k);
  ap.up_k_row_stride = a->up_k_row_stride;
  ap.qlimb = reinterpret_cast<uint4*>(ws + wl.qlimb);
  ap.qstep = reinterpret_cast<float*>(ws + wl.qstep);
  ap.score_scale = sm_scale * kLog2e;
  ap.num_heads = a->num_heads;
  ap.head_dim = a->head_dim;
  ap.sum_rk = sum_rk;
  std::memcpy(ap.k_off, a->k_off, sizeof(int32_t) * (a->num_heads + 1));
  absorb_query_kernel<<<dim3(a->num_heads, a->batch), 128, 0, st>>>(ap);
  LSVD_CUDA_TRY(cudaGetLastError());

  if (a->max_len_in_batch > 0) {
    StreamParams sp{};
    sp.cache_k = a->cache_k;
    sp.cache_v = a->cache_v;
    sp.scale_k = static_cast<const __half*>(a->scale_k);
    sp.scale_v = static_cast<const __half*>(a->scale_v);
    sp.cache_k_row_stride = a->cache_k_row_stride;
    sp.cache_v_row_stride = a->cache_v_row_stride;
    sp.scale_k_row_stride = a->scale_k_row_stride;
    sp.scale_v_row_stride = a->scale_v_row_stride;
    sp.req_to_token = a->req_to_token;
    sp.req_to_token_stride = a->req_to_token_stride;
    sp.b_req_idx = a->b_req_idx;
    sp.b_seq_len = a->b_seq_len;
    sp.qlimb = ap.qlimb;
    sp.qstep = ap.qstep;
    sp.part_ml = reinterpret_cast<float*>(ws + wl.part_ml);
    sp.part_acc = reinterpret_cast<float*>(ws + wl.part_acc);
    sp.status_word = a->status_word;
    sp.batch = a->batch;
    sp.num_heads = a->num_heads;
    sp.num_slots = a->num_slots;
    sp.sum_rk = sum_rk;
    sp.sum_rv = sum_rv;
    sp.tiles_per_block = hp.tiles_per_block;
    sp.max_parts = hp.max_parts;
    sp.num_stages = hp.num_stages;
    sp.k_tile_bytes = hp.k_tile_bytes;
    sp.v_tile_bytes = hp.v_tile_bytes;
    sp.stage_bytes = hp.stage_bytes;
    sp.ngroups = hp.ngroups;
    for (int g = 0; g < hp.ngroups; ++g) sp.g[g] = hp.g[g];
    LSVD_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(latent_stream_kernel), hp.smem_bytes));
    if (a->ev_stream_begin) LSVD_CUDA_TRY(cudaEventRecord(static_cast<cudaEvent_t>(a->ev_stream_begin), st));
    latent_stream_kernel<<<hp.num_blocks, kStreamThreads, hp.smem_bytes, st>>>(sp);
    LSVD_CUDA_TRY(cudaGetLastError());
    if (a->ev_stream_end) LSVD_CUDA_TRY(cudaEventRecord(static_cast<cudaEvent_t>(a->ev_stream_end), st));
  }

  MergeParams mp{};
  mp.part_ml = reinterpret_cast<const float*>(ws + wl.part_ml);
  mp.part_acc = reinterpret_cast<const float*>(ws + wl.part_acc);
  mp.b_seq_len = a->b_seq_len;
  mp.up_v = static_cast<const __half*>(a->up_v);
  mp.up_v_row_stride = a->up_v_row_stride;
  mp.out = static_cast<__half*>(a->out);
  mp.out_stride_b = a->out_stride_b;
  mp.out_stride_h = a->out_stride_h;
  mp.out_latent = static_cast<__half*>(a->out_latent);
  mp.out_latent_stride_b = a->out_latent_stride_b;
  mp.batch = a->batch;
  mp.num_heads = a->num_heads;
  mp.head_dim = a->head_dim;
  mp.sum_rv = sum_rv;
  mp.ngroups = hp.ngroups;
  mp.tiles_per_block = hp.tiles_per_block;
  mp.max_parts = hp.max_parts;
  std::memcpy(mp.v_off, a->v_off, sizeof(int32_t) * (a->num_heads + 1));
  std::memcpy(mp.head_group, hp.head_group, sizeof(int16_t) * a->num_heads);
  merge_up_kernel<<<dim3(a->num_heads, a->batch), 128, 0, st>>>(mp);
  LSVD_CUDA_TRY(cudaGetLastError());
  return LSVD_OK;
}
