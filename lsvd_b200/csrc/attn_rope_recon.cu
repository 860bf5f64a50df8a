// The reference's own decode attention ("rope_recon"): keys are rebuilt from the int8 latents with the int8 K
// up-factor, rotated at their logical position, and dotted with the rotated query; values stay in latent space.
//   K_t   = fp16((z_k[t] . W_uk) * s_k[t] * s_w)                  int8 x int8 -> int32 on mma.sync m16n8k32
//   K_rot = rope(K_t, t),  q_rot = fp16(rope(q, L - 1))           pairs (i, i + D/2), angle t / theta^(2i/D)
//   s_t   = (q_rot . K_rot) / sqrt(D),  p = softmax(s),  o = sum_t p_t * s_v[t] * z_v[t]        -> fp16 [B, H, R_v]
// Follows kernels/layer_bench/fd_kernel/flash_int8_latent_per_head_decoding_rope_stage1.py:55-194 (stage 1) and
// flash_latent_per_head_decoding_stage2.py:19-47 (merge), including grouped-query heads (kv head = h / group).
//
// Three kernels: a cos/sin table for the positions of the call (fp16, as the reference rounds them; shared by
// every request and head), the streaming kernel (one block per request, head and run of block_seq tokens), and
// the merge of the runs.  In the streaming kernel a warp handles 16 tokens at a time as one MMA row tile: the
// latents are the A operand straight from the cache rows, the head's slice of W_uk is staged transposed in
// shared memory once per block as the B operand, and a lane ends up with both members of every rotary pair of
// its columns, so rotation and the dot product with the query need no exchange beyond a reduction over the four
// lanes of a quad.  Rotation, dequantisation and the query are folded per rotary pair (columns i and i + D/2, integer
// sums a0, a1, column scales w0, w1, rotated query q0, q1, angle of the key's position (c, s)):
//   (k0 c - k1 s) q0 + (k1 c + k0 s) q1  with  k = a * s_k * w   =   s_k * [ c (a0 w0 q0 + a1 w1 q1) + s (a0 w0 q1 - a1 w1 q0) ]
// so a key costs four constants per pair (staged once per block) and six multiply-adds instead of a dequantised, rounded
// and rotated fp16 key; the fp16 roundings of the rebuilt key that the reference makes on the way are not reproduced
// (they move a score by about 1e-5 of its value).
#include <algorithm>
#include <cmath>

#include "common.cuh"
#include "gemv.cuh"

namespace lsvd {

constexpr int kRopeWarps = 4;
constexpr int kRopeMaxD = 128;        // largest head_dim (the rebuilt keys of a tile live in registers); 32, 64, 128 are built

struct RopeParams {
  const __half* q; int64_t q_stride_b, q_stride_h;
  const int8_t* cache_k; int64_t k_slot_stride, k_head_stride;
  const __half* scale_k; int64_t sk_slot_stride;
  const int8_t* cache_v; int64_t v_slot_stride, v_head_stride;
  const __half* scale_v; int64_t sv_slot_stride;
  const int8_t* wk; int64_t wk_row_stride;
  const __half* wk_scale;
  const int32_t* req_to_token; int64_t req_to_token_stride;
  const int32_t* b_req_idx;
  const int32_t* b_seq_len;
  __half2* table;            // [max_len][D/2] (cos, sin) rounded to fp16
  float* part;               // [B][H][nsplit][2 + rv]: running max (log2 domain), sum, unnormalised accumulators
  __half* out; int64_t out_stride_b, out_stride_h;
  int32_t* status_word;
  int32_t batch, heads, kv_heads, group, head_dim, rk, rv, num_slots, max_len, block_seq, nsplit;
  float score_scale;         // sm_scale * log2(e)
  float theta;
};

// inv[i] = theta^(2i/D); the angle of position t is t / inv[i] (the reference divides).
__device__ __forceinline__ float rope_divisor(float theta, int i, int D) {
  return powf(theta, static_cast<float>(2 * i) / static_cast<float>(D));
}

__global__ void rope_table_kernel(__half2* table, int max_len, int D, float theta) {
  grid_dependency_sync();
  const int D2 = D >> 1;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= max_len * D2) return;
  const int pos = idx / D2, i = idx - pos * D2;
  const float ang = static_cast<float>(pos) / rope_divisor(theta, i, D);
  table[idx] = __floats2half2_rn(cosf(ang), sinf(ang));
}

// RK, RV: the K and V ranks when known at compile time (0: read from the parameters).  With the ranks fixed the rank loop
// unrolls, its bounds checks fold away and the shared-memory offsets of the W_uk fragments become immediates.
template <int D, int RK, int RV>
__global__ void __launch_bounds__(kRopeWarps * 32, 4) rope_recon_kernel(const __grid_constant__ RopeParams p) {
  extern __shared__ __align__(16) uint8_t rope_smem[];
  constexpr int D2 = D >> 1;
  const int rk = RK ? RK : p.rk, rv = RV ? RV : p.rv;
  const int pitch = rk + 16;                                   // bytes per column of the transposed W_uk slice
  int8_t* wT = reinterpret_cast<int8_t*>(rope_smem);           // [D][pitch]: column c of the head, ranks contiguous
  float* sw = reinterpret_cast<float*>(rope_smem + ((D * pitch + 15) & ~15));     // [D] column scales
  float* qrot = sw + D;                                        // [D] rotated query (fp16 values)
  float4* cst = reinterpret_cast<float4*>(qrot + D);           // [D/2] (w0 q0, w1 q1, w0 q1, w1 q0) of every rotary pair
  float* wpart = reinterpret_cast<float*>(cst + D2);           // [kRopeWarps][2 + 128]
  grid_dependency_sync();

  const int sp = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / p.group;
  const int len = min(p.b_seq_len[b], p.max_len);
  const int start = sp * p.block_seq;
  if (start >= len) return;
  const int end = min(len, start + p.block_seq);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  // ---- stage W_uk[:, hk*D .. +D] transposed, the column scales and the rotated query ----
  {
    const int chunks = D >> 4;                                 // 16-column pieces of a rank's row
    for (int i = threadIdx.x; i < rk * chunks; i += blockDim.x) {
      const int r = i / chunks, c0 = (i - r * chunks) << 4;
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(p.wk + r * p.wk_row_stride + static_cast<int64_t>(hk) * D + c0));
      const int8_t* bytes = reinterpret_cast<const int8_t*>(&v);
#pragma unroll
      for (int e = 0; e < 16; ++e) wT[(c0 + e) * pitch + r] = bytes[e];
    }
    for (int c = threadIdx.x; c < D; c += blockDim.x) sw[c] = __half2float(p.wk_scale[static_cast<int64_t>(hk) * D + c]);
    const __half* qp = p.q + b * p.q_stride_b + h * p.q_stride_h;
    for (int i = threadIdx.x; i < D2; i += blockDim.x) {
      const float ang = static_cast<float>(len - 1) / rope_divisor(p.theta, i, D);
      const float qc = cosf(ang), qs = sinf(ang);
      const float q0 = __half2float(qp[i]), q1 = __half2float(qp[i + D2]);
      qrot[i] = __half2float(__float2half_rn(q0 * qc - q1 * qs));
      qrot[i + D2] = __half2float(__float2half_rn(q1 * qc + q0 * qs));
    }
  }
  __syncthreads();
  // pair c = 16 i + 4 t + m is stored at 16 i + 4 m + t: the four lanes of a quad then read one 64-byte run per load
  for (int i = threadIdx.x; i < D2; i += blockDim.x)
    cst[(i & ~15) | ((i & 3) << 2) | ((i >> 2) & 3)] = make_float4(sw[i] * qrot[i], sw[i + D2] * qrot[i + D2], sw[i] * qrot[i + D2], sw[i + D2] * qrot[i]);
  __syncthreads();

  const int32_t* r2t = p.req_to_token + static_cast<int64_t>(p.b_req_idx[b]) * p.req_to_token_stride;
  constexpr int ntile = D >> 3;        // 8-column MMA tiles of the head
  constexpr int npair = ntile >> 1;    // tile j pairs with tile j + npair (columns c and c + D/2)
  // Which columns of the head an MMA tile holds is free; they are chosen so that a lane's accumulators cover FOUR
  // consecutive rotary pairs per two tiles (one 16-byte piece of a cos/sin row, which then needs 2 * D / 32 loads per
  // tile and row instead of D / 8 eight-byte ones that each touched eight rows): column n of tile j = 2 i + u is head
  // column 16 i + u + 2 n, so lane (g, t) holds pairs 16 i + 4 t + u + 2 e in acc[j][e].  The stride of two columns
  // between lanes also spreads the W_uk fragment reads of a half-warp over all banks (pitch rk + 16).
  auto tile_col = [](int j) { return (j >= npair ? D2 : 0) + 16 * ((j % npair) >> 1) + (j & 1); };
  float m = -INFINITY, l = 0.f;
  // value latents: lane (tg = lane / 8, ch = lane % 8) adds tokens 4 i + tg of a tile into ranks 8 ch .. 8 ch + 7 and
  // 64 + 8 ch .. 64 + 8 ch + 7; the four token groups are summed once, after the loop
  float accv[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) accv[i] = 0.f;
  const int tg = lane >> 3, ch = lane & 7;
  int next_slot = r2t[min(start + warp * 16 + (lane & 15), end - 1)];

  for (int t0 = start + warp * 16; t0 < end; t0 += kRopeWarps * 16) {
    // slot of token t0 + (lane & 15), kept by every lane for the shuffles below; lanes past the end reuse the
    // tile's first token (a real row) and their scores are masked
    int my_slot = next_slot;
    next_slot = r2t[min(t0 + kRopeWarps * 16 + (lane & 15), end - 1)];      // the next tile's rows can then be requested at once
    if (my_slot < 0 || my_slot >= p.num_slots) {
      report_status(p.status_word, LSVD_ERR_BOUNDS);
      my_slot = 0;
    }
    const int slot_lo = __shfl_sync(0xffffffffu, my_slot, g), slot_hi = __shfl_sync(0xffffffffu, my_slot, g + 8);
    const bool ok_lo = t0 + g < end, ok_hi = t0 + g + 8 < end;
    const int8_t* klo = p.cache_k + slot_lo * p.k_slot_stride + hk * p.k_head_stride + 8 * t;
    const int8_t* khi = p.cache_k + slot_hi * p.k_slot_stride + hk * p.k_head_stride + 8 * t;

    // ---- K = Z W_uk: acc[j] holds columns tile_col(j) + 4t, + 4t + 2 of rows g (c = 0, 1) and g + 8 (c = 2, 3) ----
    int acc[ntile][4];
#pragma unroll
    for (int j = 0; j < ntile; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0;
#pragma unroll
    for (int ks = 0; ks < (RK ? RK : LSVD_MAX_RANK); ks += 32) {
      if (!RK && ks >= rk) break;
      // the MMA's k index is a permutation of the 32 ranks that both operands follow:
      // k 4t..4t+3 <-> ranks ks + 8t..8t+3, k 16+4t.. <-> ranks ks + 8t+4..8t+7
      uint2 alo = make_uint2(0u, 0u), ahi = alo;
      if (ks + 8 * t < rk) {
        alo = __ldg(reinterpret_cast<const uint2*>(klo + ks));
        ahi = __ldg(reinterpret_cast<const uint2*>(khi + ks));
      }
#pragma unroll
      for (int j = 0; j < ntile; ++j) {
        uint2 bw = make_uint2(0u, 0u);
        if (ks + 8 * t < rk) bw = *reinterpret_cast<const uint2*>(wT + (tile_col(j) + 2 * g) * pitch + ks + 8 * t);
        mma_s8(acc[j], alo.x, ahi.x, alo.y, ahi.y, bw.x, bw.y);
      }
    }

    // ---- rotation at the logical position and the dot product with the rotated query, folded (see the top) ----
    const float sk_lo = __half2float(p.scale_k[slot_lo * p.sk_slot_stride + hk]);
    const float sk_hi = __half2float(p.scale_k[slot_hi * p.sk_slot_stride + hk]);
    const __half2* tab_lo = p.table + static_cast<int64_t>(min(t0 + g, end - 1)) * D2;
    const __half2* tab_hi = p.table + static_cast<int64_t>(min(t0 + g + 8, end - 1)) * D2;
    float dot_lo = 0.f, dot_hi = 0.f;
#pragma unroll
    for (int i = 0; i < npair / 2; ++i) {
      // this lane's four rotary pairs 16 i + 4 t .. + 3 of both rows: (cos, sin) of all four in one 16-byte load
      const uint4 raw_lo = __ldg(reinterpret_cast<const uint4*>(tab_lo + 16 * i + 4 * t));
      const uint4 raw_hi = __ldg(reinterpret_cast<const uint4*>(tab_hi + 16 * i + 4 * t));
#pragma unroll
      for (int u = 0; u < 2; ++u) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = 2 * i + u;
          const float4 k4 = cst[16 * i + 4 * (u + 2 * e) + t];
          const uint32_t wl = e ? (u ? raw_lo.w : raw_lo.z) : (u ? raw_lo.y : raw_lo.x);
          const uint32_t wh = e ? (u ? raw_hi.w : raw_hi.z) : (u ? raw_hi.y : raw_hi.x);
          const float2 cs_lo = make_float2(__half2float(__ushort_as_half(static_cast<unsigned short>(wl & 0xffffu))),
                                           __half2float(__ushort_as_half(static_cast<unsigned short>(wl >> 16))));
          const float2 cs_hi = make_float2(__half2float(__ushort_as_half(static_cast<unsigned short>(wh & 0xffffu))),
                                           __half2float(__ushort_as_half(static_cast<unsigned short>(wh >> 16))));
          {
            const float a0 = static_cast<float>(acc[j][e]), a1 = static_cast<float>(acc[j + npair][e]);
            dot_lo = fmaf(cs_lo.x, fmaf(a1, k4.y, a0 * k4.x), dot_lo);
            dot_lo = fmaf(cs_lo.y, fmaf(-a1, k4.w, a0 * k4.z), dot_lo);
          }
          {
            const float a0 = static_cast<float>(acc[j][2 + e]), a1 = static_cast<float>(acc[j + npair][2 + e]);
            dot_hi = fmaf(cs_hi.x, fmaf(a1, k4.y, a0 * k4.x), dot_hi);
            dot_hi = fmaf(cs_hi.y, fmaf(-a1, k4.w, a0 * k4.z), dot_hi);
          }
        }
      }
    }
    dot_lo *= sk_lo;
    dot_hi *= sk_hi;
    dot_lo += __shfl_xor_sync(0xffffffffu, dot_lo, 1);
    dot_lo += __shfl_xor_sync(0xffffffffu, dot_lo, 2);
    dot_hi += __shfl_xor_sync(0xffffffffu, dot_hi, 1);
    dot_hi += __shfl_xor_sync(0xffffffffu, dot_hi, 2);
    const float s_lo = ok_lo ? dot_lo * p.score_scale : -INFINITY;      // log2 domain
    const float s_hi = ok_hi ? dot_hi * p.score_scale : -INFINITY;

    // ---- online softmax over the tile's 16 tokens ----
    float mx = fmaxf(s_lo, s_hi);
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
    mx = fmaxf(mx, m);
    const float corr = exp2f(m - mx);
    m = mx;
    const float p_lo = exp2f(s_lo - mx), p_hi = exp2f(s_hi - mx);
    float ps = (t == 0) ? p_lo + p_hi : 0.f;                            // one lane per quad counts its two tokens
    ps += __shfl_xor_sync(0xffffffffu, ps, 4);
    ps += __shfl_xor_sync(0xffffffffu, ps, 8);
    ps += __shfl_xor_sync(0xffffffffu, ps, 16);
    l = fmaf(l, corr, ps);
    const float w_lo = ok_lo ? p_lo * __half2float(p.scale_v[slot_lo * p.sv_slot_stride + hk]) : 0.f;
    const float w_hi = ok_hi ? p_hi * __half2float(p.scale_v[slot_hi * p.sv_slot_stride + hk]) : 0.f;

    // ---- values: 8-byte loads, four tokens of the tile at a time; token weights and slots come by shuffle ----
#pragma unroll
    for (int i = 0; i < 16; ++i) accv[i] *= corr;
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int r = 4 * it + tg;                       // this lane's token of the tile
      const float wa = __shfl_sync(0xffffffffu, w_lo, (r & 7) << 2), wb = __shfl_sync(0xffffffffu, w_hi, (r & 7) << 2);
      const float w = r < 8 ? wa : wb;
      const int slot = __shfl_sync(0xffffffffu, my_slot, r);
      const int8_t* vrow = p.cache_v + slot * p.v_slot_stride + hk * p.v_head_stride + 8 * ch;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        if (64 * half + 8 * ch < rv) {
          const uint2 v = __ldg(reinterpret_cast<const uint2*>(vrow + 64 * half));
          float* a = accv + 8 * half;
          a[0] = fmaf(w, s8_to_f32<0>(v.x), a[0]);
          a[1] = fmaf(w, s8_to_f32<1>(v.x), a[1]);
          a[2] = fmaf(w, s8_to_f32<2>(v.x), a[2]);
          a[3] = fmaf(w, s8_to_f32<3>(v.x), a[3]);
          a[4] = fmaf(w, s8_to_f32<0>(v.y), a[4]);
          a[5] = fmaf(w, s8_to_f32<1>(v.y), a[5]);
          a[6] = fmaf(w, s8_to_f32<2>(v.y), a[6]);
          a[7] = fmaf(w, s8_to_f32<3>(v.y), a[7]);
        }
      }
    }
  }

  // ---- the four token groups of a warp, then the block's warps (log-sum-exp); write the run's partial result ----
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    accv[i] += __shfl_xor_sync(0xffffffffu, accv[i], 8);
    accv[i] += __shfl_xor_sync(0xffffffffu, accv[i], 16);
  }
  float* mine = wpart + warp * (2 + 128);
  if (lane == 0) {
    mine[0] = m;
    mine[1] = l;
  }
  if (tg == 0) {
#pragma unroll
    for (int half = 0; half < 2; ++half)
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (64 * half + 8 * ch + e < rv) mine[2 + 64 * half + 8 * ch + e] = accv[8 * half + e];
  }
  __syncthreads();
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < kRopeWarps; ++w) M = fmaxf(M, wpart[w * (2 + 128)]);
  float* dst = p.part + ((static_cast<int64_t>(b) * p.heads + h) * p.nsplit + sp) * (2 + rv);
  for (int i = threadIdx.x; i < rv + 1; i += blockDim.x) {
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kRopeWarps; ++w) {
      const float mw = wpart[w * (2 + 128)];
      const float e = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      sum = fmaf(wpart[w * (2 + 128) + 1 + i], e, sum);       // i = 0: the sum, i >= 1: rank i - 1
    }
    dst[1 + i] = sum;
  }
  if (threadIdx.x == 0) dst[0] = M;
}

__global__ void __launch_bounds__(128) rope_merge_kernel(const __grid_constant__ RopeParams p) {
  grid_dependency_sync();
  const int h = blockIdx.x, b = blockIdx.y;
  const int len = min(p.b_seq_len[b], p.max_len);
  const int runs = (len + p.block_seq - 1) / p.block_seq;
  const int rv = p.rv;
  const float* part = p.part + (static_cast<int64_t>(b) * p.heads + h) * p.nsplit * (2 + rv);
  float M = -INFINITY;
  for (int k = 0; k < runs; ++k) M = fmaxf(M, part[k * (2 + rv)]);
  float denom = 0.f;
  for (int k = 0; k < runs; ++k) denom = fmaf(part[k * (2 + rv) + 1], exp2f(part[k * (2 + rv)] - M), denom);
  for (int i = threadIdx.x; i < rv; i += blockDim.x) {
    float num = 0.f;
    for (int k = 0; k < runs; ++k) num = fmaf(part[k * (2 + rv) + 2 + i], exp2f(part[k * (2 + rv)] - M), num);
    p.out[b * p.out_stride_b + h * p.out_stride_h + i] = __float2half_rn(runs > 0 ? num / denom : 0.f);
  }
}

static size_t rope_align(size_t x) { return (x + 255) / 256 * 256; }

static int rope_splits(int max_len, int block_seq) { return std::max(1, (max_len + block_seq - 1) / block_seq); }

}  // namespace lsvd

extern "C" size_t lsvd_attn_decode_rope_workspace_bytes(int32_t batch, int32_t num_q_heads, int32_t head_dim, int32_t rank_v,
                                                        int32_t max_len_in_batch, int32_t block_seq) {
  using namespace lsvd;
  if (batch <= 0 || num_q_heads <= 0 || head_dim <= 0 || rank_v <= 0 || max_len_in_batch < 0 || block_seq <= 0) return 0;
  const size_t table = rope_align(static_cast<size_t>(std::max(1, max_len_in_batch)) * (head_dim / 2) * 4);
  const size_t part = rope_align(static_cast<size_t>(batch) * num_q_heads * rope_splits(max_len_in_batch, block_seq) *
                                 (2 + rank_v) * 4);
  return table + part;
}

extern "C" int lsvd_attn_decode_rope(const lsvd_attn_rope_args* a, void* stream) {
  using namespace lsvd;
  if (a == nullptr || a->batch <= 0 || a->num_q_heads <= 0 || a->num_kv_heads <= 0 || (a->num_q_heads % a->num_kv_heads))
    return LSVD_ERR_INVALID_ARG;
  if (a->head_dim != 32 && a->head_dim != 64 && a->head_dim != 128) return LSVD_ERR_UNSUPPORTED;
  if (a->rank_k <= 0 || a->rank_k > LSVD_MAX_RANK || (a->rank_k % 16) || a->rank_v <= 0 || a->rank_v > LSVD_MAX_RANK ||
      (a->rank_v % 16))
    return LSVD_ERR_INVALID_ARG;
  if (!a->q || !a->cache_k || !a->cache_v || !a->scale_k || !a->scale_v || !a->wk || !a->wk_scale || !a->req_to_token ||
      !a->b_req_idx || !a->b_seq_len || !a->out)
    return LSVD_ERR_INVALID_ARG;
  if (a->num_slots <= 0 || a->max_len_in_batch < 0 || a->block_seq < 16 || (a->block_seq % 16)) return LSVD_ERR_INVALID_ARG;
  if (!aligned(a->cache_k, 8) || (a->cache_k_slot_stride % 8) || (a->cache_k_head_stride % 8)) return LSVD_ERR_INVALID_ARG;
  if (!aligned(a->cache_v, 8) || (a->cache_v_slot_stride % 8) || (a->cache_v_head_stride % 8)) return LSVD_ERR_INVALID_ARG;
  if (!aligned(a->wk, 16) || (a->wk_row_stride % 16)) return LSVD_ERR_INVALID_ARG;
  const size_t need = lsvd_attn_decode_rope_workspace_bytes(a->batch, a->num_q_heads, a->head_dim, a->rank_v,
                                                            a->max_len_in_batch, a->block_seq);
  if (a->workspace == nullptr || a->workspace_bytes < need || !aligned(a->workspace, 256)) return LSVD_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  RopeParams p{};
  p.q = static_cast<const __half*>(a->q); p.q_stride_b = a->q_stride_b; p.q_stride_h = a->q_stride_h;
  p.cache_k = a->cache_k; p.k_slot_stride = a->cache_k_slot_stride; p.k_head_stride = a->cache_k_head_stride;
  p.scale_k = static_cast<const __half*>(a->scale_k); p.sk_slot_stride = a->scale_k_slot_stride;
  p.cache_v = a->cache_v; p.v_slot_stride = a->cache_v_slot_stride; p.v_head_stride = a->cache_v_head_stride;
  p.scale_v = static_cast<const __half*>(a->scale_v); p.sv_slot_stride = a->scale_v_slot_stride;
  p.wk = a->wk; p.wk_row_stride = a->wk_row_stride;
  p.wk_scale = static_cast<const __half*>(a->wk_scale);
  p.req_to_token = a->req_to_token; p.req_to_token_stride = a->req_to_token_stride;
  p.b_req_idx = a->b_req_idx; p.b_seq_len = a->b_seq_len;
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  p.table = reinterpret_cast<__half2*>(ws);
  p.part = reinterpret_cast<float*>(ws + rope_align(static_cast<size_t>(std::max(1, a->max_len_in_batch)) * (a->head_dim / 2) * 4));
  p.out = static_cast<__half*>(a->out); p.out_stride_b = a->out_stride_b; p.out_stride_h = a->out_stride_h;
  p.status_word = a->status_word;
  p.batch = a->batch; p.heads = a->num_q_heads; p.kv_heads = a->num_kv_heads; p.group = a->num_q_heads / a->num_kv_heads;
  p.head_dim = a->head_dim; p.rk = a->rank_k; p.rv = a->rank_v; p.num_slots = a->num_slots;
  // Tokens per block: the caller's block_seq, doubled (up to 1024) while the grid still holds eight blocks per SM: every
  // block stages its head's slice of W_uk and the query constants first, which longer runs amortise.  The workspace was
  // sized for block_seq, so fewer, longer runs fit.
  int run = a->block_seq;
  while (run < 1024 && static_cast<int64_t>(rope_splits(a->max_len_in_batch, run * 2)) * a->num_q_heads * a->batch >= 148 * 8)
    run *= 2;
  p.max_len = a->max_len_in_batch; p.block_seq = run;
  p.nsplit = rope_splits(a->max_len_in_batch, run);
  const float sm_scale = a->sm_scale > 0.f ? a->sm_scale : 1.0f / std::sqrt(static_cast<float>(a->head_dim));
  p.score_scale = sm_scale * 1.4426950408889634f;
  p.theta = a->rope_theta > 0.f ? a->rope_theta : 10000.0f;
  if (a->max_len_in_batch > 0) {
    const int n = a->max_len_in_batch * (a->head_dim / 2);
    LSVD_CUDA_TRY(launch_chained(rope_table_kernel, dim3((n + 255) / 256), dim3(256), 0, st, 1, true, p.table,
                                 a->max_len_in_batch, a->head_dim, p.theta));
    const int pitch = a->rank_k + 16;
    const int smem = ((a->head_dim * pitch + 15) & ~15) + (2 * a->head_dim + 2 * a->head_dim + kRopeWarps * (2 + 128)) * 4;
    void (*kern)(RopeParams) = a->head_dim == 128 ? rope_recon_kernel<128, 0, 0>
                               : (a->head_dim == 64 ? rope_recon_kernel<64, 0, 0> : rope_recon_kernel<32, 0, 0>);
    if (a->head_dim == 128 && a->rank_k == 64 && a->rank_v == 64) kern = rope_recon_kernel<128, 64, 64>;
    if (a->head_dim == 128 && a->rank_k == 128 && a->rank_v == 128) kern = rope_recon_kernel<128, 128, 128>;
    if (smem > 48 * 1024) LSVD_CUDA_TRY(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem));
    LSVD_CUDA_TRY(launch_chained(kern, dim3(p.nsplit, a->num_q_heads, a->batch), dim3(kRopeWarps * 32), smem, st, 1, true, p));
  }
  LSVD_CUDA_TRY(launch_chained(rope_merge_kernel, dim3(a->num_q_heads, a->batch), dim3(128), 0, st, 1, true, p));
  return LSVD_OK;
}
