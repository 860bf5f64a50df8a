// int8 latent flash-decoding attention for one query token per request ("absorb" form).
//
// Three kernels per call:
//   1. absorb_query_kernel   q~_h = B_k,h q_h (fp32), stored as three balanced base-128 int8 limbs per
//                            entry plus one fp32 step per head, so that the per-token score is an exact
//                            integer dot product of int8 latents with int8 limbs (dp4a).
//   2. latent_stream_kernel  the HBM stream.  The work is cut into items (request, head, run of 32-token
//                            tiles) of roughly equal byte size, whatever the head's rank; every warp of a
//                            persistent grid takes items from a global counter and streams them on its own:
//                            128-bit loads straight from the cache rows into registers (consecutive lanes
//                            cover one token's bytes of the head, so a warp instruction reads whole 32-byte
//                            sectors), integer scores reduced with warp shuffles, an online softmax, and
//                            p * scale_v * z_v accumulated in 16 registers per lane.  There is no shared
//                            memory staging and no block-level synchronisation: latency is hidden by the
//                            16 independent warps per SM.  (Cache rows are scattered by the slot table and a
//                            head owns 16..128 bytes of a row: bulk/TMA copies of such pieces reached a
//                            quarter of this form's bandwidth.)
//   3. merge_up_kernel       log-sum-exp merge of the partial results of the items of a (request, head),
//                            optional fp16 latent output, V up-projection o = B_v^T o_lat.
//
// What it replaces in the reference: stage 1
// (kernels/layer_bench/fd_kernel/flash_int8_latent_per_head_decoding_rope_stage1.py:32-194) rebuilds every
// key as (z_k . W_uk) * scales and dots it with the query; without a rotary embedding between them the
// up-factor can be applied to the query once instead (r_k multiply-adds per token instead of r_k * D).
// Stage 2 (flash_latent_per_head_decoding_stage2.py:7-48) is the same merge, followed here by the V
// up-projection the reference leaves to a later GEMM (ffn_kernel/baseline_kernel.py:96-99,144-145).
#include <algorithm>
#include <cstdlib>
#include <cmath>
#include <cstring>
#include <mutex>

#include "attn.cuh"

namespace lsvd {

constexpr int kTileTokens = 32;          // tokens per tile
constexpr int kStreamWarps = 16;         // warps per block (one block per SM)
constexpr int kStreamThreads = kStreamWarps * 32;
constexpr int kItemBytes = 40 * 1024;    // target size of a work item (K + V bytes of its tokens): five steps of a 128 + 128-rank head
constexpr int kMaxItemTiles = 8;         // and its largest number of 32-token steps: a step costs a memory round trip
                                         // whatever the head's rank, and the last items of a call run alone
constexpr int kLimbMax = 63 * (16384 + 128 + 1);   // largest integer three balanced base-128 limbs hold
constexpr float kLog2e = 1.4426950408889634f;


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
  float* part_ml;            // [batch][items_per_request][2]  running max (log2 domain) and sum
  float* part_acc;           // [batch][acc_per_request]       unnormalised accumulators
  int32_t* queue;            // work counter, zeroed by the absorb kernel
  int32_t* status_word;
  int32_t batch, num_heads, num_slots, sum_rk;
  int32_t items_per_request, acc_per_request, total_items;
  int32_t head_major;        // cache layout: 0 = [slot][sum r] + scales [slot][H]; 1 = [head][slot][r_h] + scales [H][slot]
  HeadPlan head[LSVD_MAX_HEADS];
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
  int32_t* queue;          // work counter of the stream kernel that follows: reset here
  float score_scale;       // sm_scale * log2(e)
  int32_t num_heads, head_dim, sum_rk;
  int32_t up_k_vec16;      // rows of up_k are 16-byte aligned
  // checked copies of the batch bookkeeping for the kernels that follow: a request row outside the table becomes an empty
  // request, a length beyond the bound the work items were cut for becomes that bound; both are reported
  const int32_t* b_req_idx; const int32_t* b_seq_len;
  int32_t* san_req; int32_t* san_len; int32_t* status_word;
  int32_t max_len, r2t_rows;
  int32_t k_off[LSVD_MAX_HEADS + 1];
};

__global__ void __launch_bounds__(128) absorb_query_kernel(const __grid_constant__ AbsorbParams p) {
  __shared__ float qs[256];
  __shared__ float qt[LSVD_MAX_RANK];
  __shared__ float wmax[4];
  grid_dependency_release();
  const int h = blockIdx.x, b = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r0 = p.k_off[h], r = p.k_off[h + 1] - r0;
  // one thread per latent entry: its up-factor row is head_dim contiguous fp16 values.  The factor is a weight:
  // its first eight 16-byte pieces are requested before this kernel waits for the one before it.
  const __half* row = p.up_k + static_cast<int64_t>(r0 + min(static_cast<int>(threadIdx.x), r - 1)) * p.up_k_row_stride;
  uint4 v0[8];
  const bool pre = p.up_k_vec16 && threadIdx.x < r;
  if (pre) {
#pragma unroll
    for (int c = 0; c < 8; ++c)
      v0[c] = (c < (p.head_dim >> 3)) ? __ldg(reinterpret_cast<const uint4*>(row) + c) : make_uint4(0u, 0u, 0u, 0u);
  }
  grid_dependency_wait();
  if (h == 0 && b == 0 && threadIdx.x == 0) *p.queue = 0;
  if (h == 0 && threadIdx.x == 0) {
    int req = p.b_req_idx[b], len = p.b_seq_len[b];
    if (p.r2t_rows > 0 && static_cast<uint32_t>(req) >= static_cast<uint32_t>(p.r2t_rows)) {
      report_status(p.status_word, LSVD_ERR_BOUNDS);
      req = 0;
      len = 0;
    }
    if (len > p.max_len) {
      report_status(p.status_word, LSVD_ERR_BOUNDS);
      len = p.max_len;
    }
    p.san_req[b] = req;
    p.san_len[b] = len < 0 ? 0 : len;
  }
  const __half* qp = p.q + b * p.q_stride_b + h * p.q_stride_h;
  for (int d = threadIdx.x; d < p.head_dim; d += blockDim.x) qs[d] = __half2float(qp[d]);
  __syncthreads();
  if (threadIdx.x < r) {
    float acc = 0.f;
    if (p.up_k_vec16) {
      const uint4* rv = reinterpret_cast<const uint4*>(row);
      for (int c0 = 0; c0 < (p.head_dim >> 3); c0 += 8) {
        uint4 v[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          if (c0 == 0) v[c] = v0[c];
          else v[c] = (c0 + c < (p.head_dim >> 3)) ? __ldg(rv + c0 + c) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          if (c0 + c < (p.head_dim >> 3)) {
            const __half2* h2 = reinterpret_cast<const __half2*>(&v[c]);
            const float* qv = qs + (c0 + c) * 8;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __half22float2(h2[e]);
              acc = fmaf(f.x, qv[2 * e], acc);
              acc = fmaf(f.y, qv[2 * e + 1], acc);
            }
          }
        }
      }
    } else {
      for (int d = 0; d < p.head_dim; ++d) acc = fmaf(__half2float(row[d]), qs[d], acc);
    }
    qt[threadIdx.x] = acc;
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

// D(16x8, s32) += A(16x32, s8, row) * B(32x8, s8, col) on the tensor cores.  Lane (g = lane / 4, t = lane % 4)
// holds  a0: row g,   k 4t..4t+3     a1: row g+8, k 4t..4t+3     a2: row g,   k 16+4t..     a3: row g+8, k 16+4t..
//        b0: k 4t..4t+3, col g       b1: k 16+4t.., col g        d0,d1: row g, cols 2t,2t+1   d2,d3: row g+8.
__device__ __forceinline__ void mma_s8_16x8x32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Same with a zero accumulator on input (no registers to clear first).
__device__ __forceinline__ void mma_s8_16x8x32_zero(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                    uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// A signed (latents), B unsigned (softmax weights), zero accumulator on input.
__device__ __forceinline__ void mma_s8u8_16x8x32_zero(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                      uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ uint4 ldg128(const int8_t* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint2 ldg64(const int8_t* p) { return __ldg(reinterpret_cast<const uint2*>(p)); }

__device__ __forceinline__ int log2_ceil_chunks(int n) { return n > 4 ? 3 : (n > 2 ? 2 : (n > 1 ? 1 : 0)); }

// 4 x 4 byte transpose: out[r] = { x0.byte r, x1.byte r, x2.byte r, x3.byte r }.
__device__ __forceinline__ void transpose4x4_bytes(uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3, uint32_t (&out)[4]) {
  const uint32_t a_lo = __byte_perm(x0, x1, 0x5140), a_hi = __byte_perm(x0, x1, 0x7362);
  const uint32_t b_lo = __byte_perm(x2, x3, 0x5140), b_hi = __byte_perm(x2, x3, 0x7362);
  out[0] = __byte_perm(a_lo, b_lo, 0x5410);
  out[1] = __byte_perm(a_lo, b_lo, 0x7632);
  out[2] = __byte_perm(a_hi, b_hi, 0x5410);
  out[3] = __byte_perm(a_hi, b_hi, 0x7632);
}

// One work item: tiles [t0, t1) of request b for head h, streamed by one warp in steps of 32 tokens.
// Both contractions run as exact int8 tensor-core MMAs (m16n8k32, int32 accumulators), lane = (g, t):
//   scores   A = K latents, rows = tokens (two tiles of 16), k = 32 ranks per block; lane (g, t) loads the 8 bytes
//            at ranks 8t..8t+7 of the block for tokens g and g+8 of each tile (four lanes = one 32-byte sector);
//            B = the three int8 limbs of the absorbed query in columns 0..2.
//   values   A = V latents transposed, rows = ranks, k = the 32 tokens; lane (g, t) loads the 8 bytes at ranks
//            8g..8g+7 of a 64-rank group for tokens 8t..8t+7 and transposes 4 x 4 byte blocks in registers, which
//            feeds four MMAs (row g <-> rank 8g+r, row g+8 <-> rank 8g+4+r); B = the softmax weights
//            p * scale_v of the 32 tokens, quantised per step to two unsigned base-256 limbs against the step's
//            largest weight (16 bits), columns 0..1.  The int32 results are scaled back into fp32 accumulators.
template <bool kHeadMajor>
__device__ __forceinline__ void stream_item(const StreamParams& p, const HeadPlan& H, int b, int h, int rem, int k,
                                            int len, int t0, int t1, uint4* scratch, uint8_t* wlimb, int lane) {
  const int nk = H.nk, nv = H.nv;
  const int nkb = (nk + 1) >> 1;                 // 32-rank blocks of K
  const int nvg = (nv + 3) >> 2;                 // 64-rank groups of V
  const int g = lane >> 2, t4 = lane & 3;
  // head-major layout: a head's rows of consecutive slots are contiguous (r_h bytes apart), and so are its scales
  const int8_t* kbase = p.cache_k + (kHeadMajor ? static_cast<int64_t>(H.k_col) * p.num_slots : H.k_col) + t4 * 8;
  const int8_t* vbase = p.cache_v + (kHeadMajor ? static_cast<int64_t>(H.v_col) * p.num_slots : H.v_col) + g * 8;
  const bool v_ok0 = g * 8 < nv * 16, v_ok1 = 64 + g * 8 < nv * 16;
  const __half* ksc = kHeadMajor ? p.scale_k + static_cast<int64_t>(h) * p.num_slots : p.scale_k + h;
  const __half* vsc = kHeadMajor ? p.scale_v + static_cast<int64_t>(h) * p.num_slots : p.scale_v + h;
  const int32_t* r2t = p.req_to_token + static_cast<int64_t>(p.b_req_idx[b]) * p.req_to_token_stride;
  const float step = p.qstep[b * p.num_heads + h];
  // row strides fit 32 bits (checked by the host): a row address is one 32 x 32 + 64-bit multiply-add
  const uint32_t kstride = kHeadMajor ? static_cast<uint32_t>(nk * 16) : static_cast<uint32_t>(p.cache_k_row_stride);
  const uint32_t vstride = kHeadMajor ? static_cast<uint32_t>(nv * 16) : static_cast<uint32_t>(p.cache_v_row_stride);

  __syncwarp();
  {
    const uint4* src = p.qlimb + (static_cast<int64_t>(b) * (p.sum_rk / 16) + H.k_col / 16) * 3;
    if (lane < nk * 3) scratch[lane] = src[lane];
  }
  __syncwarp();
  // B operand of the score MMAs: column g is limb g of the absorbed query (columns 3..7 are zero).  The k
  // index of the MMA is a permutation of the ranks that matches how the A bytes are loaded:
  // k 4t..4t+3 <-> ranks 8t..8t+3 of the block, k 16+4t.. <-> ranks 8t+4..8t+7.
  uint32_t limb_b0[4], limb_b1[4];
#pragma unroll
  for (int kb = 0; kb < 4; ++kb) {
    limb_b0[kb] = limb_b1[kb] = 0u;
    const int chunk = kb * 2 + (t4 >> 1);
    if (chunk < nk && g < 3) {
      const uint32_t* w = reinterpret_cast<const uint32_t*>(scratch + chunk * 3 + g) + (t4 & 1) * 2;
      limb_b0[kb] = w[0];
      limb_b1[kb] = w[1];
    }
  }

  float m = -INFINITY, l = 0.f;
  float acc[2][4][2];                // [64-rank group][r][row g | row g+8]: this lane's share of the sums
#pragma unroll
  for (int gi = 0; gi < 2; ++gi)
#pragma unroll
    for (int r = 0; r < 4; ++r) acc[gi][r][0] = acc[gi][r][1] = 0.f;

  const int tok_begin = t0 * kTileTokens, tok_end = min(len, t1 * kTileTokens);
  // Software pipeline: the K latents of step i+1 are requested right after the score MMAs of step i have
  // consumed their registers, so they travel during the softmax and the value MMAs; the V latents of step i
  // are requested at the top of the step and travel during its score MMAs.  Slot numbers run two steps ahead.
  uint2 ka[4][4];                    // [token g + 8j][32-rank block]
  auto resolve = [&](int slot, bool& valid, int& rslot) {
    valid = slot >= 0;
    if (valid && slot >= p.num_slots) {
      report_status(p.status_word, LSVD_ERR_BOUNDS);
      valid = false;
    }
    // Lanes without a token read the row of the step's first token instead (always a real row): what they
    // load meets a zero weight or a masked score, and no load needs a validity predicate.
    const int slot0 = __shfl_sync(0xffffffffu, valid ? slot : -1, 0);
    rslot = valid ? slot : max(slot0, 0);
  };
  auto load_k = [&](int rslot) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int slot = __shfl_sync(0xffffffffu, rslot, g + 8 * j);
      const int8_t* row = kbase + static_cast<uint64_t>(static_cast<uint32_t>(slot)) * kstride;
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) {
        ka[j][kb] = make_uint2(0u, 0u);
        if (kb * 2 + (t4 >> 1) < nk) ka[j][kb] = ldg64(row + kb * 32);
      }
    }
  };
  bool valid;
  int rslot;
  {
    int s0 = -1;
    if (tok_begin + lane < tok_end) s0 = r2t[tok_begin + lane];
    resolve(s0, valid, rslot);
  }
  load_k(rslot);
  // The K and the V scale of a step's token are both needed by the softmax, long before the V latents are: both are
  // requested one step ahead, with the K latents (the V scale, requested at the top of its own step, sat on the step's
  // critical path: 8 us per call), and wait in ONE register as two fp16 bit patterns.
  auto load_scales = [&](int rs) {
    const uint32_t a = __half_as_ushort(ksc[kHeadMajor ? static_cast<int64_t>(rs) : rs * p.scale_k_row_stride]);
    const uint32_t c = __half_as_ushort(vsc[kHeadMajor ? static_cast<int64_t>(rs) : rs * p.scale_v_row_stride]);
    return a | (c << 16);
  };
  uint32_t kvs = load_scales(rslot);
  int slot_n1 = -1;                  // slot of "my" token of the next step (lane = token role)
  if (tok_begin + kTileTokens + lane < tok_end) slot_n1 = r2t[tok_begin + kTileTokens + lane];

  for (int tb = tok_begin; tb < tok_end; tb += kTileTokens) {
    int slot_n2 = -1;
    if (tb + 2 * kTileTokens + lane < tok_end) slot_n2 = r2t[tb + 2 * kTileTokens + lane];
    // ---- request the V latents of this step ----
    uint2 va[8], vb[8];              // [token 8t + i] of the first / second 64-rank group
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int slot = __shfl_sync(0xffffffffu, rslot, t4 * 8 + i);
      const int8_t* row = vbase + static_cast<uint64_t>(static_cast<uint32_t>(slot)) * vstride;
      va[i] = vb[i] = make_uint2(0u, 0u);
      if (v_ok0) va[i] = ldg64(row);
      if (v_ok1) vb[i] = ldg64(row + 64);
    }

    // ---- scores ----
    float sc[4];                     // score of token g + 8j, in lanes t = 0, 1 of the quad
#pragma unroll
    for (int rt = 0; rt < 2; ++rt) {
      int d[4];
      mma_s8_16x8x32_zero(d, ka[2 * rt][0].x, ka[2 * rt + 1][0].x, ka[2 * rt][0].y, ka[2 * rt + 1][0].y, limb_b0[0], limb_b1[0]);
#pragma unroll
      for (int kb = 1; kb < 4; ++kb) {
        if (kb < nkb)
          mma_s8_16x8x32(d, ka[2 * rt][kb].x, ka[2 * rt + 1][kb].x, ka[2 * rt][kb].y, ka[2 * rt + 1][kb].y,
                         limb_b0[kb], limb_b1[kb]);
      }
      float lo, hi;                  // columns 0, 1 (lane t = 0) and 2 (lane t = 1) are the three limbs
      if (t4 == 0) {
        lo = fmaf(128.f, static_cast<float>(d[1]), static_cast<float>(d[0]));
        hi = fmaf(128.f, static_cast<float>(d[3]), static_cast<float>(d[2]));
      } else {
        lo = 16384.f * static_cast<float>(d[0]);
        hi = 16384.f * static_cast<float>(d[2]);
      }
      sc[2 * rt] = lo + __shfl_xor_sync(0xffffffffu, lo, 1);
      sc[2 * rt + 1] = hi + __shfl_xor_sync(0xffffffffu, hi, 1);
    }
    float s_raw = 0.f;               // token T = lane: its score is sc[T >> 3] of the quad g = T & 7
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float got = __shfl_sync(0xffffffffu, sc[j], (lane & 7) << 2);
      if ((lane >> 3) == j) s_raw = got;
    }
    const float ks = __half2float(__ushort_as_half(static_cast<unsigned short>(kvs & 0xffffu)));
    const float vs_cur = __half2float(__ushort_as_half(static_cast<unsigned short>(kvs >> 16)));
    const float s = valid ? s_raw * (ks * step) : -INFINITY;      // log2 domain
    // ---- request the K latents of the next step (their registers are free now) ----
    const bool valid_cur = valid;
    if (tb + kTileTokens < tok_end) {
      resolve(slot_n1, valid, rslot);
      load_k(rslot);
      kvs = load_scales(rslot);
    }
    // ---- online softmax; the running maximum is shared by the warp ----
    const float mx = fmaxf(m, warp_max_redux(s));
    const float corr = exp2f(m - mx);
    m = mx;
    const float pr = exp2f(s - mx);
    l = fmaf(l, corr, pr);
    const float w = valid_cur ? pr * vs_cur : 0.f;
    // ---- weights of the 32 tokens as two unsigned base-256 limbs against the step's largest weight (16 bits) ----
    const float wmax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(w)));   // w >= 0
    const float winv = wmax > 0.f ? 65535.f / wmax : 0.f;
    const float wsc = wmax * (1.0f / 65535.f);
    {
      const uint32_t Q = static_cast<uint32_t>(min(65535, __float2int_rn(w * winv)));
      __syncwarp();
      wlimb[lane] = static_cast<uint8_t>(Q & 255u);
      wlimb[32 + lane] = static_cast<uint8_t>(Q >> 8);
      __syncwarp();
    }
    uint32_t wb0 = 0u, wb1 = 0u;     // B operand: k 4t..4t+3 <-> tokens 8t..8t+3, k 16+4t.. <-> tokens 8t+4..8t+7
    if (g < 2) {                     // column 0: low limb, column 1: high limb; both land in lane t = 0 of a quad
      const uint32_t* wl = reinterpret_cast<const uint32_t*>(wlimb + g * 32 + t4 * 8);
      wb0 = wl[0];
      wb1 = wl[1];
    }
    // ---- values ----
#pragma unroll
    for (int gi = 0; gi < 2; ++gi) {
      if (gi < nvg) {
        uint32_t x0[4], y0[4], x1[4], y1[4];
        if (gi == 0) {
          transpose4x4_bytes(va[0].x, va[1].x, va[2].x, va[3].x, x0);
          transpose4x4_bytes(va[0].y, va[1].y, va[2].y, va[3].y, y0);
          transpose4x4_bytes(va[4].x, va[5].x, va[6].x, va[7].x, x1);
          transpose4x4_bytes(va[4].y, va[5].y, va[6].y, va[7].y, y1);
        } else {
          transpose4x4_bytes(vb[0].x, vb[1].x, vb[2].x, vb[3].x, x0);
          transpose4x4_bytes(vb[0].y, vb[1].y, vb[2].y, vb[3].y, y0);
          transpose4x4_bytes(vb[4].x, vb[5].x, vb[6].x, vb[7].x, x1);
          transpose4x4_bytes(vb[4].y, vb[5].y, vb[6].y, vb[7].y, y1);
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          int d[4];
          mma_s8u8_16x8x32_zero(d, x0[r], y0[r], x1[r], y1[r], wb0, wb1);
          // lane t = 0 holds both limb columns; the other lanes of the quad compute on zero columns
          const float lo = static_cast<float>(d[0] + d[1] * 256), hi = static_cast<float>(d[2] + d[3] * 256);
          acc[gi][r][0] = fmaf(acc[gi][r][0], corr, wsc * lo);
          acc[gi][r][1] = fmaf(acc[gi][r][1], corr, wsc * hi);
        }
      }
    }
    slot_n1 = slot_n2;
  }

  // ---- this item's partial result ----
  const float lsum = warp_sum(l);
  float* ml = p.part_ml + (static_cast<int64_t>(b) * p.items_per_request + rem) * 2;
  if (lane == 0) {
    ml[0] = m;
    ml[1] = lsum;
  }
  float* pa = p.part_acc + static_cast<int64_t>(b) * p.acc_per_request + H.acc_off + k * nv * 16;
#pragma unroll
  for (int gi = 0; gi < 2; ++gi) {
    float v[8];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      v[r] = acc[gi][r][0];            // complete in lane t = 0 of each quad
      v[4 + r] = acc[gi][r][1];
    }
    if (t4 == 0 && gi * 64 + g * 8 < nv * 16) {
      float4* dst = reinterpret_cast<float4*>(pa + gi * 64 + g * 8);     // ranks 8g .. 8g+7 of the group
      dst[0] = make_float4(v[0], v[1], v[2], v[3]);
      dst[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
  }
}

template <bool kHeadMajor>
__global__ void __launch_bounds__(kStreamThreads, 1) latent_stream_kernel(const __grid_constant__ StreamParams p) {
  __shared__ uint4 limb_scratch[kStreamWarps][8 * 3];
  __shared__ __align__(16) uint8_t weight_limbs[kStreamWarps][96];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  grid_dependency_sync();

  for (;;) {
    // ---- take the next item: (request b, head h, part k) ----
    int item = 0;
    if (lane == 0) item = atomicAdd(p.queue, 1);
    item = __shfl_sync(0xffffffffu, item, 0);
    if (item >= p.total_items) break;
    const int b = item / p.items_per_request;
    const int rem = item - b * p.items_per_request;
    int below = 0;
    for (int i = lane; i < p.num_heads; i += 32) below += (p.head[i].part_off <= rem) ? 1 : 0;
    const int h = __reduce_add_sync(0xffffffffu, below) - 1;
    const HeadPlan& H = p.head[h];
    const int k = rem - H.part_off;
    const int len = p.b_seq_len[b];               // the checked copies written by the absorb kernel
    const int ntiles = tiles_of(len);
    const int t0 = k * H.chunk_tiles;
    const int t1 = min(ntiles, t0 + H.chunk_tiles);
    if (t0 >= t1) continue;                       // this request is shorter than the bound the items were cut for
    stream_item<kHeadMajor>(p, H, b, h, rem, k, len, t0, t1, limb_scratch[warp], weight_limbs[warp], lane);
  }
}

// ----------------------------------------------------------------------------------------------
// 2b. the same item over a shared-memory ring (head-major cache)
// ----------------------------------------------------------------------------------------------
// In the head-major layout the rows of a head for consecutive slots are one contiguous run, so a step's 32 K rows and
// 32 V rows are ONE bulk copy each (cp.async.bulk, no tensor map, no multicast) when the page table maps the step's
// tokens to consecutive slots -- checked per step by the warp -- and gathered 16-byte cp.async copies otherwise.  The rows
// land in a per-warp ring of up to four steps and complete on a per-stage mbarrier, so a warp keeps several steps of
// latents in flight without holding them in registers, the K fragments come from shared memory with constant offsets
// and the V fragments by ldmatrix.trans on bytes (no byte transposes in registers): 78 registers instead of 127, so 24
// warps per SM instead of 16.  Measured on B200 (batch 16 x 4097 tokens, ragged ranks): 61.4 us against 66.7 us for the
// register-fed kernel; at batch 64 x 8192 tokens, 40 heads: 0.97 of the measured HBM bandwidth against 0.79.  With
// byte transposes in registers as above, 12 / 16 / 20 / 24 warps took 90.6 / 77.4 / 72.3 / 69.3 us: what bounds both
// forms at the smaller size is a warp's own instruction stream per step, which more resident warps hide better.
// A step whose slots are not one run (always, on the slot-major cache) is gathered with 16-byte cp.async copies in
// commit groups instead (one bulk copy per row, 64 per step, took 116.5 us): 87 us against 80 us for the register-fed
// kernel, which LSVD_STREAM_RING=0 selects.
// Waits are bounded: a wait that runs out reports LSVD_ERR_TIMEOUT and the warp stops taking items.
constexpr int kRingWarps = 24;
constexpr int kRingThreads = kRingWarps * 32;
constexpr int kRingBytesPerWarp = 9088;              // two steps of a 64 + 64-rank head
constexpr int kRingMaxStages = 4;

__device__ __forceinline__ uint4 lds128(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }
// 16 bytes global -> shared without a register in between; a thread's copies complete in commit groups.
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Waits until at most `newer` of this thread's commit groups are still in flight (newer = 0..3).
__device__ __forceinline__ void cp_async_wait_newer(int newer) {
  switch (newer) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
  }
}
__device__ __forceinline__ uint2 lds64(const uint8_t* p) { return *reinterpret_cast<const uint2*>(p); }

// Two 16 x 16 byte matrices (rows given by lanes 0..15 and 16..31, 16 bytes each) transposed into registers: lane (g, t)
// receives, per matrix, bytes [4t..4t+3][g] and [4t..4t+3][g + 8] (layout measured on B200).
__device__ __forceinline__ void ldmatrix_x2_trans_b8(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const uint8_t* row) {
  asm volatile("ldmatrix.sync.aligned.m16n16.x2.trans.shared.b8 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(smem_u32(row)));
}

// A tile's 32 gathered rows of n 16-byte pieces into dst[32][n * 16]: consecutive lanes copy consecutive pieces (piece q
// belongs to row q / n), rows of lanes without a token are skipped.  Not inlined: it runs only for steps whose slots
// are not one run, and must not cost the streaming loop registers.
__device__ __noinline__ void ring_gather_rows(uint8_t* dst, const int8_t* base, int64_t row_stride, int n, int slot,
                                              uint32_t valid_mask, int lane) {
  const int inv = (65536 + n - 1) / n;           // q / n = (q * inv) >> 16 for q < 256
  for (int q0 = 0; q0 < kTileTokens * n; q0 += 32) {
    const int q = q0 + lane;
    const int row = (q * inv) >> 16, col = q - row * n;
    const int rslot = __shfl_sync(0xffffffffu, slot, row);
    if ((valid_mask >> row) & 1u) cp_async16(dst + q * 16, base + static_cast<int64_t>(rslot) * row_stride + col * 16);
  }
}

template <bool kHeadMajor>
__device__ __forceinline__ bool stream_item_ring(const StreamParams& p, const HeadPlan& H, int b, int h, int rem, int k,
                                                 int len, int t0, int t1, uint4* scratch, uint8_t* wlimb, uint8_t* ring,
                                                 uint64_t* bars, uint32_t& phases, int lane) {
  const int nk = H.nk, nv = H.nv;
  const int nvg = (nv + 3) >> 2;                 // 64-rank groups of V
  const int g = lane >> 2, t4 = lane & 3;
  const int rkb = nk * 16, rvb = nv * 16;        // bytes of a K / V row of this head
  const int stage_bytes = kTileTokens * (rkb + rvb);
  const int S = min(kRingMaxStages, kRingBytesPerWarp / stage_bytes);       // >= 2: a stage is at most 8 KB
  // head-major: a head's rows of consecutive slots are contiguous (r_h bytes apart), and so are its scales;
  // slot-major: a row sits at slot * row stride + the head's column, every row is its own copy
  const int8_t* kbase = p.cache_k + (kHeadMajor ? static_cast<int64_t>(H.k_col) * p.num_slots : H.k_col);
  const int8_t* vbase = p.cache_v + (kHeadMajor ? static_cast<int64_t>(H.v_col) * p.num_slots : H.v_col);
  const int64_t kstride = kHeadMajor ? rkb : p.cache_k_row_stride, vstride = kHeadMajor ? rvb : p.cache_v_row_stride;
  const __half* ksc = kHeadMajor ? p.scale_k + static_cast<int64_t>(h) * p.num_slots : p.scale_k + h;
  const __half* vsc = kHeadMajor ? p.scale_v + static_cast<int64_t>(h) * p.num_slots : p.scale_v + h;
  const int32_t* r2t = p.req_to_token + static_cast<int64_t>(p.b_req_idx[b]) * p.req_to_token_stride;
  const float step = p.qstep[b * p.num_heads + h];

  __syncwarp();
  {
    const uint4* src = p.qlimb + (static_cast<int64_t>(b) * (p.sum_rk / 16) + H.k_col / 16) * 3;
    if (lane < nk * 3) scratch[lane] = src[lane];
  }
  __syncwarp();
  // B operand of the score MMAs: column g is limb g of the absorbed query (columns 3..7 are zero).  Lane (g, t)
  // reads the 16 bytes 16t..16t+15 of a 64-rank group of a token row, and MMA s of the group (s = 0, 1) takes
  // k 4t..4t+3 <-> ranks 16t+8s..+3, k 16+4t.. <-> ranks 16t+8s+4..+7; the query limbs follow the same order.
  uint32_t limb_b0[4], limb_b1[4];   // [2 * group + s]
#pragma unroll
  for (int kb = 0; kb < 4; ++kb) {
    limb_b0[kb] = limb_b1[kb] = 0u;
    const int chunk = (kb >> 1) * 4 + t4;
    if (chunk < nk && g < 3) {
      const uint32_t* w = reinterpret_cast<const uint32_t*>(scratch + chunk * 3 + g) + (kb & 1) * 2;
      limb_b0[kb] = w[0];
      limb_b1[kb] = w[1];
    }
  }

  float m = -INFINITY, l = 0.f;
  float acc[2][4][2];                // [64-rank group][r][row g | row g+8]: this lane's share of the sums
#pragma unroll
  for (int gi = 0; gi < 2; ++gi)
#pragma unroll
    for (int r = 0; r < 4; ++r) acc[gi][r][0] = acc[gi][r][1] = 0.f;

  const int koff0 = t4 < nk ? 16 * t4 : 0, koff1 = 4 + t4 < nk ? 64 + 16 * t4 : 0;
  // stages filled by gathered cp.async copies: a bit per stage, the commit-group number of each (8 bits per stage) and
  // the number of groups committed so far
  uint32_t gather_mask = 0u, gather_seq_of = 0u, gather_seq = 0u;
  const int tok_begin = t0 * kTileTokens, tok_end = min(len, t1 * kTileTokens);
  const int nsteps = (tok_end - tok_begin + kTileTokens - 1) / kTileTokens;
  auto slot_of = [&](int j) {        // slot of this lane's token of step j (-1: no token)
    const int tok = tok_begin + j * kTileTokens + lane;
    return (j < nsteps && tok < tok_end) ? r2t[tok] : -1;
  };
  // what a lane keeps about its token of every step in flight: validity (a bit) and the two scales (two fp16)
  uint32_t q0 = 0u, q1 = 0u, q2 = 0u, q3 = 0u, vbits = 0u;
  int inflight = 0, ist = 0;         // steps in flight, stage of the next step to request
  auto issue = [&](int slot) {
    bool valid = slot >= 0;
    if (valid && slot >= p.num_slots) {
      report_status(p.status_word, LSVD_ERR_BOUNDS);
      valid = false;
    }
    const uint32_t mask = __ballot_sync(0xffffffffu, valid);
    const int n = __popc(mask);
    const int slot0 = __shfl_sync(0xffffffffu, slot, 0);
    const bool run = kHeadMajor && mask == (n == 32 ? 0xffffffffu : ((1u << n) - 1u)) &&
                     __all_sync(0xffffffffu, !valid || slot == slot0 + lane);
    uint8_t* kst = ring + ist * stage_bytes;
    uint8_t* vst = kst + kTileTokens * rkb;
    uint64_t* bar = bars + ist;
    if (run) {
      // one bulk copy per tile, counted in bytes on the stage's barrier
      if (lane == 0) {
        mbar_arrive_expect_tx(bar, static_cast<uint32_t>(n * (rkb + rvb)));
        if (n > 0) {
          bulk_g2s(kst, kbase + static_cast<int64_t>(slot0) * rkb, static_cast<uint32_t>(n * rkb), bar);
          bulk_g2s(vst, vbase + static_cast<int64_t>(slot0) * rvb, static_cast<uint32_t>(n * rvb), bar);
        }
      }
      gather_mask &= ~(1u << ist);
    } else {
      // gathered rows (64 bulk copies of one row each cost more than they bring): consecutive lanes copy consecutive
      // 16-byte pieces with cp.async (piece q of a tile = row q / pieces-per-row), one commit group per lane and step;
      // the barrier's phase is completed at once and the consumer waits for the group instead
      if (lane == 0) mbar_arrive(bar);
      ring_gather_rows(kst, kbase, kstride, nk, slot, mask, lane);
      ring_gather_rows(vst, vbase, vstride, nv, slot, mask, lane);
      cp_async_commit();
      gather_mask |= 1u << ist;
      gather_seq_of = (gather_seq_of & ~(0xffu << (8 * ist))) | ((gather_seq & 0xffu) << (8 * ist));
      ++gather_seq;
    }
    uint32_t sc = 0u;
    if (valid) {
      const uint32_t a = __half_as_ushort(ksc[kHeadMajor ? static_cast<int64_t>(slot) : slot * p.scale_k_row_stride]);
      const uint32_t c = __half_as_ushort(vsc[kHeadMajor ? static_cast<int64_t>(slot) : slot * p.scale_v_row_stride]);
      sc = a | (c << 16);
    }
    if (inflight == 0) q0 = sc;
    else if (inflight == 1) q1 = sc;
    else if (inflight == 2) q2 = sc;
    else q3 = sc;
    vbits |= (valid ? 1u : 0u) << inflight;
    ++inflight;
    ist = (ist + 1 == S) ? 0 : ist + 1;
  };

  // the first S steps are requested at once (their slot numbers by independent loads)
  int cst = ist;                     // stage of the next step to consume
  {
    int s_first[kRingMaxStages];
#pragma unroll
    for (int j = 0; j < kRingMaxStages; ++j) s_first[j] = (j < S) ? slot_of(j) : -1;
#pragma unroll
    for (int j = 0; j < kRingMaxStages; ++j)
      if (j < S && j < nsteps) issue(s_first[j]);
  }
  int slot_pref = slot_of(S);

  for (int j = 0; j < nsteps; ++j) {
    if (!mbar_wait_bounded(bars + cst, (phases >> cst) & 1u)) {
      report_status(p.status_word, LSVD_ERR_TIMEOUT);
      return false;
    }
    phases ^= 1u << cst;
    if ((gather_mask >> cst) & 1u) {
      cp_async_wait_newer(static_cast<int>((gather_seq - 1u - (gather_seq_of >> (8 * cst))) & 0xffu));
      __syncwarp();
    }
    const uint8_t* kst = ring + cst * stage_bytes;
    const uint8_t* vst = kst + kTileTokens * rkb;
    const bool valid = (vbits & 1u) != 0u;
    const uint32_t kvs = q0;
    vbits >>= 1;
    q0 = q1; q1 = q2; q2 = q3;
    --inflight;

    // ---- scores ----
    float sc[4];                     // score of token g + 8j, in lanes t = 0, 1 of the quad
#pragma unroll
    for (int rt = 0; rt < 2; ++rt) {
      // a 16-byte piece past the head's rank meets zero query limbs: it is read from piece 0 instead (any bytes do)
      const uint8_t* r0 = kst + (g + 16 * rt) * rkb;
      const uint8_t* r1 = r0 + 8 * rkb;
      const uint4 a0 = lds128(r0 + koff0), a1 = lds128(r1 + koff0);
      int d[4];
      mma_s8_16x8x32_zero(d, a0.x, a1.x, a0.y, a1.y, limb_b0[0], limb_b1[0]);
      mma_s8_16x8x32(d, a0.z, a1.z, a0.w, a1.w, limb_b0[1], limb_b1[1]);
      if (nk > 4) {
        const uint4 c0 = lds128(r0 + koff1), c1 = lds128(r1 + koff1);
        mma_s8_16x8x32(d, c0.x, c1.x, c0.y, c1.y, limb_b0[2], limb_b1[2]);
        mma_s8_16x8x32(d, c0.z, c1.z, c0.w, c1.w, limb_b0[3], limb_b1[3]);
      }
      float lo, hi;                  // columns 0, 1 (lane t = 0) and 2 (lane t = 1) are the three limbs
      if (t4 == 0) {
        lo = fmaf(128.f, static_cast<float>(d[1]), static_cast<float>(d[0]));
        hi = fmaf(128.f, static_cast<float>(d[3]), static_cast<float>(d[2]));
      } else {
        lo = 16384.f * static_cast<float>(d[0]);
        hi = 16384.f * static_cast<float>(d[2]);
      }
      sc[2 * rt] = lo + __shfl_xor_sync(0xffffffffu, lo, 1);
      sc[2 * rt + 1] = hi + __shfl_xor_sync(0xffffffffu, hi, 1);
    }
    float s_raw = 0.f;               // token T = lane: its score is sc[T >> 3] of the quad g = T & 7
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const float got = __shfl_sync(0xffffffffu, sc[jj], (lane & 7) << 2);
      if ((lane >> 3) == jj) s_raw = got;
    }
    const float ks = __half2float(__ushort_as_half(static_cast<unsigned short>(kvs & 0xffffu)));
    const float vs_cur = __half2float(__ushort_as_half(static_cast<unsigned short>(kvs >> 16)));
    const float s = valid ? s_raw * (ks * step) : -INFINITY;      // log2 domain
    // ---- online softmax; the running maximum is shared by the warp ----
    const float mx = fmaxf(m, warp_max_redux(s));
    const float corr = exp2f(m - mx);
    m = mx;
    const float pr = exp2f(s - mx);
    l = fmaf(l, corr, pr);
    const float w = valid ? pr * vs_cur : 0.f;
    // ---- weights of the 32 tokens as two unsigned base-256 limbs against the step's largest weight (16 bits) ----
    const float wmax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(w)));   // w >= 0
    const float winv = wmax > 0.f ? 65535.f / wmax : 0.f;
    const float wsc = wmax * (1.0f / 65535.f);
    {
      const uint32_t Q = static_cast<uint32_t>(min(65535, __float2int_rn(w * winv)));
      __syncwarp();
      wlimb[lane] = static_cast<uint8_t>(Q & 255u);
      wlimb[32 + lane] = static_cast<uint8_t>(Q >> 8);
      __syncwarp();
    }
    uint32_t wb0 = 0u, wb1 = 0u;     // B operand: k 4t..4t+3 <-> tokens 4t..4t+3, k 16+4t.. <-> tokens 16+4t..16+4t+3
    if (g < 2) {                     // column 0: low limb, column 1: high limb; both land in lane t = 0 of a quad
      const uint32_t* wl = reinterpret_cast<const uint32_t*>(wlimb + g * 32 + t4 * 4);
      wb0 = wl[0];
      wb1 = wl[4];
    }
    // ---- values: A = V transposed (rows = 16 ranks, k = the step's 32 tokens), fetched in fragment order by
    // ldmatrix.trans on bytes: lane l gives the address of token l's 16 ranks; registers 0, 1 = tokens 0..15 at ranks
    // g and g + 8, registers 2, 3 = tokens 16..31 -- the four A registers of the MMA, in order ----
    const uint8_t* vlane = vst + lane * rvb;
#pragma unroll
    for (int gi = 0; gi < 2; ++gi) {
      if (gi < nvg) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          if (gi * 4 + r < nv) {
            uint32_t a0, a1, a2, a3;
            ldmatrix_x2_trans_b8(a0, a1, a2, a3, vlane + 64 * gi + 16 * r);
            int d[4];
            mma_s8u8_16x8x32_zero(d, a0, a1, a2, a3, wb0, wb1);
            // lane t = 0 holds both limb columns; the other lanes of the quad compute on zero columns
            const float lo = static_cast<float>(d[0] + d[1] * 256), hi = static_cast<float>(d[2] + d[3] * 256);
            acc[gi][r][0] = fmaf(acc[gi][r][0], corr, wsc * lo);      // rank 64 gi + 16 r + g
            acc[gi][r][1] = fmaf(acc[gi][r][1], corr, wsc * hi);      // rank 64 gi + 16 r + g + 8
          }
        }
      }
    }
    // ---- the stage is read: request the step S ahead into it ----
    __syncwarp();
    cst = (cst + 1 == S) ? 0 : cst + 1;
    if (j + S < nsteps) {
      issue(slot_pref);
      slot_pref = slot_of(j + S + 1);
    }
  }

  // ---- this item's partial result ----
  const float lsum = warp_sum(l);
  float* ml = p.part_ml + (static_cast<int64_t>(b) * p.items_per_request + rem) * 2;
  if (lane == 0) {
    ml[0] = m;
    ml[1] = lsum;
  }
  float* pa = p.part_acc + static_cast<int64_t>(b) * p.acc_per_request + H.acc_off + k * nv * 16;
  if (t4 == 0) {                       // complete in lane t = 0 of each quad
#pragma unroll
    for (int gi = 0; gi < 2; ++gi)
#pragma unroll
      for (int r = 0; r < 4; ++r)
        if (gi * 4 + r < nv) {
          pa[64 * gi + 16 * r + g] = acc[gi][r][0];
          pa[64 * gi + 16 * r + g + 8] = acc[gi][r][1];
        }
  }
  return true;
}

template <bool kHeadMajor>
__global__ void __launch_bounds__(kRingThreads, 1) latent_stream_ring_kernel(const __grid_constant__ StreamParams p) {
  extern __shared__ __align__(128) uint8_t ring_smem[];                   // [kRingWarps][kRingBytesPerWarp]
  __shared__ uint4 limb_scratch[kRingWarps][8 * 3];
  __shared__ __align__(16) uint8_t weight_limbs[kRingWarps][96];
  __shared__ __align__(8) uint64_t bars[kRingWarps][kRingMaxStages];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kRingMaxStages; ++s) mbar_init(&bars[warp][s], 1);
    fence_mbar_init();
  }
  __syncwarp();
  grid_dependency_sync();
  uint32_t phases = 0u;              // bit s: the parity of stage s's next completion

  for (;;) {
    int item = 0;
    if (lane == 0) item = atomicAdd(p.queue, 1);
    item = __shfl_sync(0xffffffffu, item, 0);
    if (item >= p.total_items) break;
    const int b = item / p.items_per_request;
    const int rem = item - b * p.items_per_request;
    int below = 0;
    for (int i = lane; i < p.num_heads; i += 32) below += (p.head[i].part_off <= rem) ? 1 : 0;
    const int h = __reduce_add_sync(0xffffffffu, below) - 1;
    const HeadPlan& H = p.head[h];
    const int k = rem - H.part_off;
    const int len = p.b_seq_len[b];
    const int ntiles = tiles_of(len);
    const int t0 = k * H.chunk_tiles;
    const int t1 = min(ntiles, t0 + H.chunk_tiles);
    if (t0 >= t1) continue;
    if (!stream_item_ring<kHeadMajor>(p, H, b, h, rem, k, len, t0, t1, limb_scratch[warp], weight_limbs[warp],
                          ring_smem + warp * kRingBytesPerWarp, bars[warp], phases, lane))
      break;
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
  int32_t batch, num_heads, head_dim, items_per_request, acc_per_request;
  int32_t up_v_vec16;        // rows of up_v are 16-byte aligned: stage the head's block in shared memory
  int32_t v_off[LSVD_MAX_HEADS + 1];
  int32_t part_off[LSVD_MAX_HEADS];
  int32_t acc_off[LSVD_MAX_HEADS];
  int16_t chunk_tiles[LSVD_MAX_HEADS];
  int16_t parts[LSVD_MAX_HEADS];
};

constexpr int kMergeMaxParts = 512;     // part weights kept in shared memory; further parts are recomputed

__global__ void __launch_bounds__(128) merge_up_kernel(const __grid_constant__ MergeParams p) {
  extern __shared__ __align__(16) uint8_t merge_smem[];      // [rv][head_dim] fp16: this head's V up-factor
  __half* upv_s = reinterpret_cast<__half*>(merge_smem);
  __shared__ float olat[LSVD_MAX_RANK];
  const int h = blockIdx.x, b = blockIdx.y;
  const int v0_col = p.v_off[h], rv = p.v_off[h + 1] - v0_col;
  grid_dependency_release();
  // The up-factor does not depend on the partial results, nor on any kernel before this one: fetch it first,
  // with wide loads, so that its latency overlaps the end of the stream kernel and the merge.
  if (p.out != nullptr && p.up_v_vec16) {
    const int per_row = p.head_dim >> 3;
    for (int i = threadIdx.x; i < rv * per_row; i += blockDim.x) {
      const int r = i / per_row, c = i - r * per_row;
      reinterpret_cast<uint4*>(upv_s)[i] =
          __ldg(reinterpret_cast<const uint4*>(p.up_v + static_cast<int64_t>(v0_col + r) * p.up_v_row_stride) + c);
    }
  }
  grid_dependency_wait();
  // Items of (b, h) that held tokens: the same arithmetic as the stream kernel.
  const int ntiles = tiles_of(p.b_seq_len[b]);
  int nparts = (ntiles + p.chunk_tiles[h] - 1) / p.chunk_tiles[h];
  if (nparts > p.parts[h]) nparts = p.parts[h];
  const float* ml = p.part_ml + (static_cast<int64_t>(b) * p.items_per_request + p.part_off[h]) * 2;
  // weights of the parts: w_k = 2^(m_k - M) / sum_k l_k 2^(m_k - M), computed once by the block
  __shared__ float wpart[kMergeMaxParts];
  __shared__ float red_a[4], red_b[4];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float M = -INFINITY;
  for (int k = threadIdx.x; k < nparts; k += blockDim.x) M = fmaxf(M, ml[k * 2]);
  M = warp_max(M);
  if (lane == 0) red_a[warp] = M;
  __syncthreads();
  M = fmaxf(fmaxf(red_a[0], red_a[1]), fmaxf(red_a[2], red_a[3]));
  float denom = 0.f;
  for (int k = threadIdx.x; k < nparts; k += blockDim.x) {
    const float e = exp2f(ml[k * 2] - M);
    if (k < kMergeMaxParts) wpart[k] = e;
    denom += ml[k * 2 + 1] * e;
  }
  denom = warp_sum(denom);
  if (lane == 0) red_b[warp] = denom;
  __syncthreads();
  denom = red_b[0] + red_b[1] + red_b[2] + red_b[3];
  const int i = threadIdx.x;
  if (i < rv) {
    float num = 0.f;
    const float* pa = p.part_acc + static_cast<int64_t>(b) * p.acc_per_request + p.acc_off[h] + i;
    const int fast = min(nparts, kMergeMaxParts);
    int k = 0;
    for (; k + 8 <= fast; k += 8) {           // eight loads in flight
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = pa[static_cast<int64_t>(k + u) * rv];
#pragma unroll
      for (int u = 0; u < 8; ++u) num = fmaf(v[u], wpart[k + u], num);
    }
    for (; k < fast; ++k) num = fmaf(pa[static_cast<int64_t>(k) * rv], wpart[k], num);
    for (; k < nparts; ++k) num = fmaf(pa[static_cast<int64_t>(k) * rv], exp2f(ml[k * 2] - M), num);
    const float o = nparts > 0 ? num / denom : 0.f;
    olat[i] = o;
    if (p.out_latent != nullptr) p.out_latent[b * p.out_latent_stride_b + v0_col + i] = __float2half_rn(o);
  }
  __syncthreads();
  if (p.out != nullptr) {
    for (int d = threadIdx.x; d < p.head_dim; d += blockDim.x) {
      float acc = 0.f;
      if (p.up_v_vec16) {
#pragma unroll 8
        for (int r = 0; r < rv; ++r) acc = fmaf(olat[r], __half2float(upv_s[r * p.head_dim + d]), acc);
      } else {
        const __half* col = p.up_v + static_cast<int64_t>(v0_col) * p.up_v_row_stride + d;
#pragma unroll 8
        for (int r = 0; r < rv; ++r) acc = fmaf(olat[r], __half2float(col[static_cast<int64_t>(r) * p.up_v_row_stride]), acc);
      }
      p.out[b * p.out_stride_b + h * p.out_stride_h + d] = __float2half_rn(acc);
    }
  }
}

// ----------------------------------------------------------------------------------------------
// host: planning, validation, launch
// ----------------------------------------------------------------------------------------------

static int validate_offsets(const int32_t* off, int num_heads) {
  if (off == nullptr || off[0] != 0) return LSVD_ERR_INVALID_ARG;
  for (int h = 0; h < num_heads; ++h) {
    const int r = off[h + 1] - off[h];
    if (r <= 0 || r > LSVD_MAX_RANK || (r % 16) != 0) return LSVD_ERR_INVALID_ARG;
  }
  return LSVD_OK;
}

// Size of a work item in bytes: large enough to amortise an item's start-up (four dependent memory round trips), small
// enough that every warp of the grid gets at least two.  Measured on B200 at batch 16 x 4097 tokens, ragged ranks: items
// of 14 / 24 / 40 / 64 KB take 77.6 / 70.5 / 66.6 / 71.3 us.
static int choose_item_bytes(int batch, int sum_rk, int sum_rv, int max_len, int sms) {
  const int ntiles_max = (max_len + kTileTokens - 1) / kTileTokens;
  const int64_t total = static_cast<int64_t>(batch) * ntiles_max * kTileTokens * (sum_rk + sum_rv);
  const int64_t want = total / (static_cast<int64_t>(std::max(1, sms)) * kStreamWarps * 2);
  return static_cast<int>(std::max<int64_t>(1024, std::min<int64_t>(kItemBytes, want)));
}

static int make_plan(int batch, int num_heads, const int32_t* k_off, const int32_t* v_off, int max_len, HostPlan* hp) {
  if (batch <= 0 || num_heads <= 0 || num_heads > LSVD_MAX_HEADS || max_len < 0) return LSVD_ERR_INVALID_ARG;
  int rc = validate_offsets(k_off, num_heads);
  if (rc != LSVD_OK) return rc;
  rc = validate_offsets(v_off, num_heads);
  if (rc != LSVD_OK) return rc;
  const int sms = device_sm_count();
  if (sms <= 0) return LSVD_ERR_CUDA;
  const int ntiles_max = (max_len + kTileTokens - 1) / kTileTokens;
  hp->item_bytes = choose_item_bytes(batch, k_off[num_heads], v_off[num_heads], max_len, sms);
  for (int h = 0; h < num_heads; ++h) {
    HeadPlan& H = hp->head[h];
    const int rk = k_off[h + 1] - k_off[h], rv = v_off[h + 1] - v_off[h];
    H.k_col = k_off[h];
    H.v_col = v_off[h];
    H.nk = static_cast<int16_t>(rk / 16);
    H.nv = static_cast<int16_t>(rv / 16);
    const int ct = std::max(1, std::min(kMaxItemTiles, hp->item_bytes / (kTileTokens * (rk + rv))));
    H.chunk_tiles = static_cast<int16_t>(ct);
    const int parts = std::max(1, (ntiles_max + ct - 1) / ct);
    if (parts > 32767) return LSVD_ERR_UNSUPPORTED;
    H.parts = static_cast<int16_t>(parts);
  }
  int part_off = 0, acc_off = 0;
  for (int h = 0; h < num_heads; ++h) {
    HeadPlan& H = hp->head[h];
    H.part_off = part_off;
    H.acc_off = acc_off;
    part_off += H.parts;
    acc_off += H.parts * H.nv * 16;
  }
  hp->items_per_request = part_off;
  hp->acc_per_request = acc_off;
  hp->total_items = static_cast<int64_t>(batch) * part_off;
  if (hp->total_items > 0x7fffffffLL - 65536) return LSVD_ERR_UNSUPPORTED;
  hp->num_blocks = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(sms, (hp->total_items + kStreamWarps - 1) / kStreamWarps)));
  return LSVD_OK;
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }


static WorkspaceLayout workspace_layout(int batch, int num_heads, int sum_rk, int64_t items_per_request,
                                        int64_t acc_per_request) {
  WorkspaceLayout w{};
  size_t off = 0;
  w.qlimb = off; off = align_up(off + static_cast<size_t>(batch) * (sum_rk / 16) * 48, 256);
  w.qstep = off; off = align_up(off + static_cast<size_t>(batch) * num_heads * 4, 256);
  w.queue = off; off += 256;
  w.san = off; off = align_up(off + static_cast<size_t>(batch) * 8, 256);
  w.part_ml = off; off = align_up(off + static_cast<size_t>(batch) * items_per_request * 8, 256);
  w.part_acc = off; off = align_up(off + static_cast<size_t>(batch) * acc_per_request * 4, 256);
  w.total = off;
  return w;
}

}  // namespace lsvd

extern "C" size_t lsvd_attn_decode_workspace_bytes(int32_t batch, int32_t num_heads, int32_t sum_rank_k,
                                                   int32_t sum_rank_v, int32_t max_len_in_batch) {
  using namespace lsvd;
  if (batch <= 0 || num_heads <= 0 || sum_rank_k <= 0 || sum_rank_v <= 0 || max_len_in_batch < 0) return 0;
  // Upper bounds that hold for any split of the rank sums over the heads: a head's items hold at least
  // half the target size unless a single tile is larger, so there are at most twice the ideal number.
  const int sms = std::max(1, device_sm_count());
  const int64_t ntiles_max = (max_len_in_batch + kTileTokens - 1) / kTileTokens;
  const int item_bytes = choose_item_bytes(batch, sum_rank_k, sum_rank_v, max_len_in_batch, sms);
  const int64_t items = 2 * ntiles_max * kTileTokens * (sum_rank_k + sum_rank_v) / item_bytes + num_heads + 1 +
                        static_cast<int64_t>(num_heads) * (ntiles_max / kMaxItemTiles + 1);
  const int64_t items_b = std::min<int64_t>(items, ntiles_max * num_heads + num_heads);
  return workspace_layout(batch, num_heads, sum_rank_k, items_b, items_b * LSVD_MAX_RANK).total;
}

extern "C" int lsvd_attn_decode_plan(int32_t batch, int32_t num_heads, const int32_t* k_off, const int32_t* v_off,
                                     int32_t max_len_in_batch, int32_t* items_per_request, int32_t* item_bytes,
                                     int32_t* num_blocks) {
  lsvd::HostPlan hp;
  const int rc = lsvd::make_plan(batch, num_heads, k_off, v_off, max_len_in_batch, &hp);
  if (rc != LSVD_OK) return rc;
  if (items_per_request) *items_per_request = hp.items_per_request;
  if (item_bytes) *item_bytes = hp.item_bytes;
  if (num_blocks) *num_blocks = hp.num_blocks;
  return LSVD_OK;
}

namespace lsvd {

// Argument checks, the plan and the workspace layout of a call.
int attn_prepare(const lsvd_attn_decode_args* a, AttnLaunch* L) {
  if (a == nullptr) return LSVD_ERR_INVALID_ARG;
  if (a->batch <= 0 || a->head_dim <= 0 || a->head_dim > 256 || (a->head_dim % 8) != 0) return LSVD_ERR_INVALID_ARG;
  if (a->num_slots <= 0 || a->max_len_in_batch < 0) return LSVD_ERR_INVALID_ARG;
  if (!a->q || !a->cache_k || !a->cache_v || !a->scale_k || !a->scale_v || !a->up_k || !a->req_to_token ||
      !a->b_req_idx || !a->b_seq_len)
    return LSVD_ERR_INVALID_ARG;
  if (a->out == nullptr && a->out_latent == nullptr) return LSVD_ERR_INVALID_ARG;
  if (a->out != nullptr && a->up_v == nullptr) return LSVD_ERR_INVALID_ARG;
  if (a->cache_layout != LSVD_CACHE_SLOT_MAJOR && a->cache_layout != LSVD_CACHE_HEAD_MAJOR) return LSVD_ERR_INVALID_ARG;
  int rc = make_plan(a->batch, a->num_heads, a->k_off, a->v_off, a->max_len_in_batch, &L->hp);
  if (rc != LSVD_OK) return rc;
  const int sum_rk = a->k_off[a->num_heads], sum_rv = a->v_off[a->num_heads];
  if (!aligned(a->cache_k, 16) || !aligned(a->cache_v, 16)) return LSVD_ERR_INVALID_ARG;
  if (a->cache_layout == LSVD_CACHE_SLOT_MAJOR) {
    if ((a->cache_k_row_stride % 16) != 0 || (a->cache_v_row_stride % 16) != 0 || a->cache_k_row_stride < sum_rk ||
        a->cache_v_row_stride < sum_rv)
      return LSVD_ERR_INVALID_ARG;
    if (a->cache_k_row_stride > 0x7fffffffLL || a->cache_v_row_stride > 0x7fffffffLL) return LSVD_ERR_UNSUPPORTED;
    if (a->scale_k_row_stride < a->num_heads || a->scale_v_row_stride < a->num_heads) return LSVD_ERR_INVALID_ARG;
  }
  if (!aligned(a->q, 2) || !aligned(a->up_k, 2) || !aligned(a->scale_k, 2) || !aligned(a->scale_v, 2))
    return LSVD_ERR_INVALID_ARG;
  L->wl = workspace_layout(a->batch, a->num_heads, sum_rk, L->hp.items_per_request, L->hp.acc_per_request);
  if (a->workspace == nullptr || a->workspace_bytes < L->wl.total || !aligned(a->workspace, 256)) return LSVD_ERR_WORKSPACE;
  return LSVD_OK;
}

float attn_score_scale(const lsvd_attn_decode_args* a) {
  const float sm_scale = a->sm_scale > 0.f ? a->sm_scale : 1.0f / std::sqrt(static_cast<float>(a->head_dim));
  return sm_scale * kLog2e;
}

int attn_launch_absorb(const lsvd_attn_decode_args* a, const AttnLaunch& L, cudaStream_t st) {
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  AbsorbParams ap{};
  ap.q = static_cast<const __half*>(a->q);
  ap.q_stride_b = a->q_stride_b;
  ap.q_stride_h = a->q_stride_h;
  ap.up_k = static_cast<const __half*>(a->up_k);
  ap.up_k_row_stride = a->up_k_row_stride;
  ap.qlimb = reinterpret_cast<uint4*>(ws + L.wl.qlimb);
  ap.qstep = reinterpret_cast<float*>(ws + L.wl.qstep);
  ap.queue = reinterpret_cast<int32_t*>(ws + L.wl.queue);
  ap.score_scale = attn_score_scale(a);
  ap.num_heads = a->num_heads;
  ap.head_dim = a->head_dim;
  ap.sum_rk = a->k_off[a->num_heads];
  ap.up_k_vec16 = (aligned(a->up_k, 16) && (a->up_k_row_stride % 8) == 0) ? 1 : 0;
  ap.b_req_idx = a->b_req_idx;
  ap.b_seq_len = a->b_seq_len;
  ap.san_req = reinterpret_cast<int32_t*>(ws + L.wl.san);
  ap.san_len = ap.san_req + a->batch;
  ap.status_word = a->status_word;
  ap.max_len = a->max_len_in_batch;
  ap.r2t_rows = a->req_to_token_rows > 0 ? a->req_to_token_rows : 0;
  std::memcpy(ap.k_off, a->k_off, sizeof(int32_t) * (a->num_heads + 1));
  LSVD_CUDA_TRY(launch_chained(absorb_query_kernel, dim3(a->num_heads, a->batch), dim3(128), 0, st, 1, true, ap));
  return LSVD_OK;
}

int attn_launch_stream(const lsvd_attn_decode_args* a, const AttnLaunch& L, cudaStream_t st) {
  if (a->max_len_in_batch <= 0) return LSVD_OK;
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  const HostPlan& hp = L.hp;
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
  sp.b_req_idx = reinterpret_cast<const int32_t*>(ws + L.wl.san);      // the absorb kernel's checked copies
  sp.b_seq_len = sp.b_req_idx + a->batch;
  sp.qlimb = reinterpret_cast<uint4*>(ws + L.wl.qlimb);
  sp.qstep = reinterpret_cast<float*>(ws + L.wl.qstep);
  sp.part_ml = reinterpret_cast<float*>(ws + L.wl.part_ml);
  sp.part_acc = reinterpret_cast<float*>(ws + L.wl.part_acc);
  sp.queue = reinterpret_cast<int32_t*>(ws + L.wl.queue);
  sp.status_word = a->status_word;
  sp.batch = a->batch;
  sp.num_heads = a->num_heads;
  sp.num_slots = a->num_slots;
  sp.sum_rk = a->k_off[a->num_heads];
  sp.items_per_request = hp.items_per_request;
  sp.acc_per_request = hp.acc_per_request;
  sp.total_items = static_cast<int32_t>(hp.total_items);
  sp.head_major = a->cache_layout == LSVD_CACHE_HEAD_MAJOR ? 1 : 0;
  for (int h = 0; h < a->num_heads; ++h) sp.head[h] = hp.head[h];
  if (a->ev_stream_begin) LSVD_CUDA_TRY(cudaEventRecord(static_cast<cudaEvent_t>(a->ev_stream_begin), st));
  // head-major cache: the shared-memory ring form (same bits as the register-fed one, 61 against 67 us on config 3);
  // LSVD_STREAM_RING=0 selects the register-fed kernel, for measurements
  static const bool use_ring = [] {
    const char* e = std::getenv("LSVD_STREAM_RING");
    return e == nullptr || std::atoi(e) != 0;
  }();
  // The ring form pays off where a step's rows arrive as one bulk copy: on the head-major cache.  On the slot-major
  // cache every step is gathered piece by piece: 87 us against 80 us register-fed on config 3, so that layout keeps
  // the register-fed kernel unless LSVD_STREAM_RING=2 asks for the ring form (same bits).
  static const bool ring_slot_major = [] {
    const char* e = std::getenv("LSVD_STREAM_RING");
    return e != nullptr && std::atoi(e) == 2;
  }();
  const int ring_smem = kRingWarps * kRingBytesPerWarp;
  if (use_ring && sp.head_major) {
    LSVD_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(latent_stream_ring_kernel<true>), ring_smem));
    LSVD_CUDA_TRY(launch_chained(latent_stream_ring_kernel<true>, dim3(hp.num_blocks), dim3(kRingThreads), ring_smem, st, 1, true, sp));
  } else if (ring_slot_major && !sp.head_major) {
    LSVD_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(latent_stream_ring_kernel<false>), ring_smem));
    LSVD_CUDA_TRY(launch_chained(latent_stream_ring_kernel<false>, dim3(hp.num_blocks), dim3(kRingThreads), ring_smem, st, 1, true, sp));
  } else if (sp.head_major) LSVD_CUDA_TRY(launch_chained(latent_stream_kernel<true>, dim3(hp.num_blocks), dim3(kStreamThreads), 0, st, 1, true, sp));
  else LSVD_CUDA_TRY(launch_chained(latent_stream_kernel<false>, dim3(hp.num_blocks), dim3(kStreamThreads), 0, st, 1, true, sp));
  if (a->ev_stream_end) LSVD_CUDA_TRY(cudaEventRecord(static_cast<cudaEvent_t>(a->ev_stream_end), st));
  return LSVD_OK;
}

// The merge's view of the plan and the workspace, for the fused kernel that runs the merge as one of its stages.
void attn_fill_merge(const lsvd_attn_decode_args* a, const AttnLaunch& L, FMerge* mg) {
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  mg->part_ml = reinterpret_cast<const float*>(ws + L.wl.part_ml);
  mg->part_acc = reinterpret_cast<const float*>(ws + L.wl.part_acc);
  mg->b_seq_len = a->b_seq_len;
  mg->out_latent = static_cast<__half*>(a->out_latent);
  mg->out_latent_stride = a->out_latent_stride_b;
  mg->num_heads = a->num_heads;
  mg->items_per_request = L.hp.items_per_request;
  mg->acc_per_request = L.hp.acc_per_request;
  std::memcpy(mg->v_off, a->v_off, sizeof(int32_t) * (a->num_heads + 1));
  for (int h = 0; h < a->num_heads; ++h) {
    mg->part_off[h] = L.hp.head[h].part_off;
    mg->acc_off[h] = L.hp.head[h].acc_off;
    mg->chunk_tiles[h] = L.hp.head[h].chunk_tiles;
    mg->parts[h] = L.hp.head[h].parts;
  }
}

void attn_workspace_views(const lsvd_attn_decode_args* a, const AttnLaunch& L, uint4** qlimb, float** qstep, int32_t** queue) {
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  *qlimb = reinterpret_cast<uint4*>(ws + L.wl.qlimb);
  *qstep = reinterpret_cast<float*>(ws + L.wl.qstep);
  *queue = reinterpret_cast<int32_t*>(ws + L.wl.queue);
}

int attn_launch_merge(const lsvd_attn_decode_args* a, const AttnLaunch& L, cudaStream_t st) {
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  const HostPlan& hp = L.hp;
  MergeParams mp{};
  mp.part_ml = reinterpret_cast<const float*>(ws + L.wl.part_ml);
  mp.part_acc = reinterpret_cast<const float*>(ws + L.wl.part_acc);
  mp.b_seq_len = reinterpret_cast<const int32_t*>(ws + L.wl.san) + a->batch;
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
  mp.items_per_request = hp.items_per_request;
  mp.acc_per_request = hp.acc_per_request;
  std::memcpy(mp.v_off, a->v_off, sizeof(int32_t) * (a->num_heads + 1));
  for (int h = 0; h < a->num_heads; ++h) {
    mp.part_off[h] = hp.head[h].part_off;
    mp.acc_off[h] = hp.head[h].acc_off;
    mp.chunk_tiles[h] = hp.head[h].chunk_tiles;
    mp.parts[h] = hp.head[h].parts;
  }
  mp.up_v_vec16 = (a->up_v != nullptr && aligned(a->up_v, 16) && (a->up_v_row_stride % 8) == 0 && (a->head_dim % 8) == 0) ? 1 : 0;
  int max_rv = 0;
  for (int h = 0; h < a->num_heads; ++h) max_rv = std::max(max_rv, a->v_off[h + 1] - a->v_off[h]);
  const int merge_smem = (a->out != nullptr && mp.up_v_vec16) ? max_rv * a->head_dim * 2 : 0;
  if (merge_smem > 48 * 1024) LSVD_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(merge_up_kernel), merge_smem));
  LSVD_CUDA_TRY(launch_chained(merge_up_kernel, dim3(a->num_heads, a->batch), dim3(128), merge_smem, st, 1, true, mp));
  return LSVD_OK;
}

}  // namespace lsvd

extern "C" int lsvd_attn_decode(const lsvd_attn_decode_args* a, void* stream) {
  using namespace lsvd;
  AttnLaunch L;
  int rc = attn_prepare(a, &L);
  if (rc != LSVD_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rc = attn_launch_absorb(a, L, st);
  if (rc != LSVD_OK) return rc;
  rc = attn_launch_stream(a, L, st);
  if (rc != LSVD_OK) return rc;
  return attn_launch_merge(a, L, st);
}

// ----------------------------------------------------------------------------------------------
// Decode attention for callers that cannot allocate device memory
// ----------------------------------------------------------------------------------------------
// Some hosts of this library may not call cudaMalloc on the path that runs a decode step: an inference
// server that has handed all of its device memory to a paged KV-cache pool at start-up, a plugin that
// runs inside another runtime's memory budget, or a step that is being recorded into a CUDA graph, where
// allocation calls are not allowed.  lsvd_attn_decode leaves the workspace to the caller; this variant
// brings its own: a fixed array in the library's device image, present on every GPU that loads the
// library from load time until the process exits.
namespace lsvd {

static __device__ __align__(256) unsigned char g_static_scratch[LSVD_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static void* g_static_scratch_addr[kMaxDevices] = {nullptr};     // device address of the array, per device
static std::mutex g_static_scratch_mu;

// The array's name is only a host-side handle here; the device address has to be asked for, once per
// device, with that device current.  The address is kept for the life of the process: a cudaDeviceReset (or any
// other re-creation of the device's primary context) while the library is loaded is not supported.
static int static_scratch_address(void** out) {
  int dev = 0;
  LSVD_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return LSVD_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_static_scratch_mu);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    LSVD_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
    if (ptr == nullptr) return LSVD_ERR_CUDA;
    g_static_scratch_addr[dev] = ptr;
  }
  *out = g_static_scratch_addr[dev];
  return LSVD_OK;
}

}  // namespace lsvd

extern "C" size_t lsvd_attn_decode_static_scratch_bytes(void) { return LSVD_STATIC_SCRATCH_BYTES; }

extern "C" int lsvd_attn_decode_static(const lsvd_attn_decode_args* a, void* stream) {
  using namespace lsvd;
  if (a == nullptr || a->k_off == nullptr || a->v_off == nullptr || a->num_heads <= 0 || a->num_heads > LSVD_MAX_HEADS)
    return LSVD_ERR_INVALID_ARG;
  // Size check first, against the exact need of this problem: too large a batch or context is refused, not truncated.
  HostPlan hp;
  const int rc = make_plan(a->batch, a->num_heads, a->k_off, a->v_off, a->max_len_in_batch, &hp);
  if (rc != LSVD_OK) return rc;
  const WorkspaceLayout wl =
      workspace_layout(a->batch, a->num_heads, a->k_off[a->num_heads], hp.items_per_request, hp.acc_per_request);
  if (wl.total > LSVD_STATIC_SCRATCH_BYTES) return LSVD_ERR_WORKSPACE;
  void* scratch = nullptr;
  const int rc2 = static_scratch_address(&scratch);
  if (rc2 != LSVD_OK) return rc2;
  lsvd_attn_decode_args b = *a;
  b.workspace = scratch;
  b.workspace_bytes = LSVD_STATIC_SCRATCH_BYTES;
  return lsvd_attn_decode(&b, stream);
}
