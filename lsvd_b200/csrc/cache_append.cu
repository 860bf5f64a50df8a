// Latent KV-cache append: per (token, head) absmax scale, int8 codes, scatter to the cache row
// dest_loc[token].  One launch covers K and V and every head.
//
// Arithmetic follows the reference exactly (bit-exact codes and scales):
//   scale = fp16(max(absmax/128, 1e-4))                 destindex_copy_quantize_latent.py:26,
//                                                       benchmark_triton_int8_layer.py:107-108
//   torch  rounding: q = clamp(rne(fp16(x / scale)))    benchmark_triton_int8_layer.py:109
//   triton rounding: q = clamp(trunc(x/scale +- 0.5))   destindex_copy_quantize_latent.py:27-29
//
// Mapping: one warp per (token, head, K|V).  A lane owns 4 consecutive latent entries (ranks are
// multiples of 16, at most 128), loads them with one 8-byte access and stores 4 codes with one
// 4-byte access, so a warp moves a head with one coalesced load and one coalesced store.
#include <algorithm>

#include "common.cuh"
#include "devfn.cuh"

namespace lsvd {

struct AppendSide {
  const __half* latent;
  int64_t token_stride;
  int8_t* cache;
  int64_t cache_row_stride;
  __half* scale;
  int64_t scale_row_stride;
  int64_t head_off[LSVD_MAX_HEADS];   // element offset of each head inside a token's latent
  int32_t rank_off[LSVD_MAX_HEADS + 1];
};

struct AppendParams {
  AppendSide side[2];
  const int32_t* dest_loc;
  int32_t* status_word;
  int32_t num_tokens, num_heads, num_slots, rounding;
  int32_t side_mask;                   // bit 0: K present, bit 1: V present
  int32_t head_major;                  // cache layout: 0 = [slot][sum r] (+ scales [slot][H]), 1 = [head][slot][r_h] (+ [H][slot])
};

// Where the codes of (slot, head) start and where its scale lives, in either layout.
__device__ __forceinline__ int8_t* cache_unit(const AppendParams& p, const AppendSide& s, int dest, int r0, int rank) {
  return p.head_major ? s.cache + static_cast<int64_t>(r0) * p.num_slots + static_cast<int64_t>(dest) * rank
                      : s.cache + static_cast<int64_t>(dest) * s.cache_row_stride + r0;
}
__device__ __forceinline__ __half* scale_unit(const AppendParams& p, const AppendSide& s, int dest, int h) {
  return p.head_major ? s.scale + static_cast<int64_t>(h) * p.num_slots + dest : s.scale + static_cast<int64_t>(dest) * s.scale_row_stride + h;
}

template <int kRounding>
__global__ void __launch_bounds__(128) cache_append_kernel(const __grid_constant__ AppendParams p) {
  grid_dependency_sync();
  const int lane = threadIdx.x & 31;
  const int64_t unit = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t per_side = static_cast<int64_t>(p.num_tokens) * p.num_heads;
  int side = 0;
  int64_t u = unit;
  if ((p.side_mask & 1) == 0) {
    side = 1;
  } else if (u >= per_side) {
    side = 1;
    u -= per_side;
  }
  if (u >= per_side || ((p.side_mask >> side) & 1) == 0) return;
  const int t = static_cast<int>(u / p.num_heads);
  const int h = static_cast<int>(u - static_cast<int64_t>(t) * p.num_heads);
  const AppendSide& s = p.side[side];

  const int r0 = s.rank_off[h];
  const int rank = s.rank_off[h + 1] - r0;
  const int i0 = lane * 4;
  const bool active = i0 < rank;

  float x[4] = {0.f, 0.f, 0.f, 0.f};
  if (active) {
    const __half* src = s.latent + static_cast<int64_t>(t) * s.token_stride + s.head_off[h] + i0;
    if ((reinterpret_cast<uintptr_t>(src) & 7) == 0) {
      const uint2 raw = *reinterpret_cast<const uint2*>(src);
      const __half2 a = *reinterpret_cast<const __half2*>(&raw.x);
      const __half2 b = *reinterpret_cast<const __half2*>(&raw.y);
      x[0] = __low2float(a); x[1] = __high2float(a); x[2] = __low2float(b); x[3] = __high2float(b);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) x[j] = __half2float(src[j]);
    }
  }
  float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
  amax = warp_max(amax);
  // absmax is an fp16 value; /128 in fp16 is one rounding of the exact quotient.
  __half s16 = __float2half_rn(amax * 0.0078125f);
  const __half floor16 = __float2half_rn(1e-4f);
  if (__half2float(s16) < __half2float(floor16)) s16 = floor16;
  const float sf = __half2float(s16);
  const float rsf = __frcp_rn(sf);

  const int dest = p.dest_loc[t];
  if (dest < 0 || dest >= p.num_slots) {
    if (lane == 0) report_status(p.status_word, LSVD_ERR_BOUNDS);
    return;
  }
  if (active) {
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int q = quantise_one<kRounding>(x[j], sf, rsf);
      packed |= (static_cast<uint32_t>(q) & 0xffu) << (8 * j);
    }
    int8_t* dst = cache_unit(p, s, dest, r0, rank) + i0;
    *reinterpret_cast<uint32_t*>(dst) = packed;
  }
  if (lane == 0) *scale_unit(p, s, dest, h) = s16;
}

// Prefill-sized calls.  Units are ordered head by head (all tokens of head 0 of K, then head 1, ...), so a warp works
// on ONE head and its lanes can be dealt by that head's rank: L = 2, 4, 8 or 16 lanes per (token, head) unit for ranks
// up to 16, 32, 64, 128, a lane owning 8 consecutive entries (16-byte load, 8-byte store), 32 / L tokens per warp.
// The one-unit-per-warp kernel above issues two to sixteen times as many warp instructions per byte, and at these
// sizes instruction issue, not memory, is what bounds it.  Same arithmetic, so the same bits.
struct WideTable {
  int32_t warp_begin[2 * LSVD_MAX_HEADS + 1];   // first warp of every (side, head) segment, in launch order
  int32_t seg_side_head[2 * LSVD_MAX_HEADS];    // side * LSVD_MAX_HEADS + head
  int32_t nseg;
};

template <int kRounding>
__global__ void __launch_bounds__(128) cache_append_wide_kernel(const __grid_constant__ AppendParams p,
                                                                const __grid_constant__ WideTable w) {
  grid_dependency_sync();
  const int lane = threadIdx.x & 31;
  const int warp_id = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (warp_id >= w.warp_begin[w.nseg]) return;
  int lo_seg = 0, hi_seg = w.nseg;                   // last segment whose first warp is <= warp_id
  while (hi_seg - lo_seg > 1) {
    const int mid = (lo_seg + hi_seg) >> 1;
    if (w.warp_begin[mid] <= warp_id) lo_seg = mid; else hi_seg = mid;
  }
  const int side = w.seg_side_head[lo_seg] / LSVD_MAX_HEADS, h = w.seg_side_head[lo_seg] % LSVD_MAX_HEADS;
  const AppendSide& s = p.side[side];
  const int r0 = s.rank_off[h];
  const int rank = s.rank_off[h + 1] - r0;
  const int lg = rank <= 16 ? 1 : (rank <= 32 ? 2 : (rank <= 64 ? 3 : 4));     // log2 of the lanes per unit
  const int sub = lane & ((1 << lg) - 1);
  const int t = (warp_id - w.warp_begin[lo_seg]) * (32 >> lg) + (lane >> lg);
  const bool live = t < p.num_tokens;
  const int i0 = sub * 8;
  const bool active = live && i0 < rank;

  float x[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) x[j] = 0.f;
  if (active) {
    const uint4 raw = *reinterpret_cast<const uint4*>(s.latent + static_cast<int64_t>(t) * s.token_stride + s.head_off[h] + i0);
    const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      x[2 * j] = __low2float(h2[j]);
      x[2 * j + 1] = __high2float(h2[j]);
    }
  }
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(x[j]));
#pragma unroll
  for (int o = 8; o > 0; o >>= 1)
    if (o < (1 << lg)) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));     // lg is uniform in the warp
  __half s16 = __float2half_rn(amax * 0.0078125f);
  const __half floor16 = __float2half_rn(1e-4f);
  if (__half2float(s16) < __half2float(floor16)) s16 = floor16;
  const float sf = __half2float(s16);
  const float rsf = __frcp_rn(sf);
  if (!live) return;
  const int dest = p.dest_loc[t];
  if (dest < 0 || dest >= p.num_slots) {
    if (sub == 0) report_status(p.status_word, LSVD_ERR_BOUNDS);
    return;
  }
  if (active) {
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      lo |= (static_cast<uint32_t>(quantise_one<kRounding>(x[j], sf, rsf)) & 0xffu) << (8 * j);
      hi |= (static_cast<uint32_t>(quantise_one<kRounding>(x[4 + j], sf, rsf)) & 0xffu) << (8 * j);
    }
    *reinterpret_cast<uint2*>(cache_unit(p, s, dest, r0, rank) + i0) = make_uint2(lo, hi);
  }
  if (sub == 0) *scale_unit(p, s, dest, h) = s16;
}

// The wide kernel's accesses: 16-byte loads of the latents, 8-byte stores of the codes.
static bool side_is_wide_ok(const lsvd_append_tensor& t, int num_heads, bool head_major) {
  if (!aligned(t.latent, 16) || (t.token_stride % 8) != 0 || !aligned(t.cache, 8) || (!head_major && (t.cache_row_stride % 8) != 0)) return false;
  for (int h = 0; h < num_heads; ++h) {
    const int64_t off = t.head_off ? t.head_off[h] : t.rank_off[h];
    if ((off % 8) != 0) return false;
  }
  return true;
}

static int fill_side(AppendSide& dst, const lsvd_append_tensor& src, int num_heads, bool head_major) {
  if (src.rank_off == nullptr || src.cache == nullptr || src.cache_scale == nullptr) return LSVD_ERR_INVALID_ARG;
  if (src.rank_off[0] != 0) return LSVD_ERR_INVALID_ARG;
  for (int h = 0; h < num_heads; ++h) {
    const int r = src.rank_off[h + 1] - src.rank_off[h];
    if (r <= 0 || r > LSVD_MAX_RANK || (r % 16) != 0) return LSVD_ERR_INVALID_ARG;
    dst.rank_off[h] = src.rank_off[h];
    dst.head_off[h] = src.head_off ? src.head_off[h] : src.rank_off[h];
  }
  dst.rank_off[num_heads] = src.rank_off[num_heads];
  if (!head_major && (src.cache_row_stride < src.rank_off[num_heads] || (src.cache_row_stride % 4) != 0)) return LSVD_ERR_INVALID_ARG;
  if (!aligned(src.cache, head_major ? 16 : 4) || !aligned(src.latent, 2) || !aligned(src.cache_scale, 2)) return LSVD_ERR_INVALID_ARG;
  if (!head_major && src.scale_row_stride < num_heads) return LSVD_ERR_INVALID_ARG;
  dst.latent = static_cast<const __half*>(src.latent);
  dst.token_stride = src.token_stride;
  dst.cache = src.cache;
  dst.cache_row_stride = src.cache_row_stride;
  dst.scale = static_cast<__half*>(src.cache_scale);
  dst.scale_row_stride = src.scale_row_stride;
  return LSVD_OK;
}

// One decode step further: every request is one token longer and its new token's slot is looked up.
__global__ void decode_advance_kernel(int32_t* b_seq_len, int32_t* mem_index, const int32_t* req_to_token, int64_t r2t_stride,
                                      const int32_t* b_req_idx, int32_t batch, int32_t base_len, int32_t period, int32_t max_len,
                                      int32_t* status_word) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  int len = b_seq_len[b] + 1;
  if (period > 0 && len >= base_len + period) len = base_len;       // start over (benchmarks that run longer than the context they reserved)
  if (len > max_len || len < 1) {
    report_status(status_word, LSVD_ERR_BOUNDS);
    return;
  }
  b_seq_len[b] = len;
  mem_index[b] = req_to_token[static_cast<int64_t>(b_req_idx[b]) * r2t_stride + len - 1];
}

}  // namespace lsvd

extern "C" int lsvd_decode_advance(int32_t* b_seq_len, int32_t* mem_index, const int32_t* req_to_token, int64_t req_to_token_stride,
                                   const int32_t* b_req_idx, int32_t batch, int32_t base_len, int32_t period, int32_t max_len,
                                   int32_t* status_word, void* stream) {
  if (b_seq_len == nullptr || mem_index == nullptr || req_to_token == nullptr || b_req_idx == nullptr || batch <= 0 || max_len < 1)
    return LSVD_ERR_INVALID_ARG;
  lsvd::decode_advance_kernel<<<(batch + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      b_seq_len, mem_index, req_to_token, req_to_token_stride, b_req_idx, batch, base_len, period, max_len, status_word);
  LSVD_CUDA_TRY(cudaGetLastError());
  return LSVD_OK;
}

extern "C" int lsvd_cache_append(const lsvd_append_args* a, void* stream) {
  using namespace lsvd;
  if (a == nullptr) return LSVD_ERR_INVALID_ARG;
  if (a->num_tokens < 0 || a->num_heads <= 0 || a->num_heads > LSVD_MAX_HEADS || a->num_slots <= 0)
    return LSVD_ERR_INVALID_ARG;
  if (a->rounding != LSVD_ROUND_TORCH && a->rounding != LSVD_ROUND_TRITON) return LSVD_ERR_INVALID_ARG;
  if (a->num_tokens == 0) return LSVD_OK;
  if (a->dest_loc == nullptr) return LSVD_ERR_INVALID_ARG;

  AppendParams p{};
  p.dest_loc = a->dest_loc;
  p.status_word = a->status_word;
  p.num_tokens = a->num_tokens;
  p.num_heads = a->num_heads;
  p.num_slots = a->num_slots;
  p.rounding = a->rounding;
  if (a->cache_layout != LSVD_CACHE_SLOT_MAJOR && a->cache_layout != LSVD_CACHE_HEAD_MAJOR) return LSVD_ERR_INVALID_ARG;
  p.head_major = a->cache_layout == LSVD_CACHE_HEAD_MAJOR ? 1 : 0;
  p.side_mask = 0;
  if (a->k.latent != nullptr) {
    int rc = fill_side(p.side[0], a->k, a->num_heads, p.head_major != 0);
    if (rc != LSVD_OK) return rc;
    p.side_mask |= 1;
  }
  if (a->v.latent != nullptr) {
    int rc = fill_side(p.side[1], a->v, a->num_heads, p.head_major != 0);
    if (rc != LSVD_OK) return rc;
    p.side_mask |= 2;
  }
  if (p.side_mask == 0) return LSVD_OK;

  const int sides = (p.side_mask == 3) ? 2 : 1;
  const int64_t units = static_cast<int64_t>(a->num_tokens) * a->num_heads * sides;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int warps_per_block = 4;
  bool wide = units >= 32768;
  for (int sd = 0; sd < 2 && wide; ++sd) {
    if (((p.side_mask >> sd) & 1) == 0) continue;
    wide = side_is_wide_ok(sd == 0 ? a->k : a->v, a->num_heads, p.head_major != 0);
  }
  if (wide) {
    WideTable wt{};
    int64_t warps = 0;
    for (int sd = 0; sd < 2; ++sd) {
      if (((p.side_mask >> sd) & 1) == 0) continue;
      const lsvd_append_tensor& t = sd == 0 ? a->k : a->v;
      for (int h = 0; h < a->num_heads; ++h) {
        const int rank = t.rank_off[h + 1] - t.rank_off[h];
        const int lanes = rank <= 16 ? 2 : (rank <= 32 ? 4 : (rank <= 64 ? 8 : 16));
        const int per_warp = 32 / lanes;
        wt.warp_begin[wt.nseg] = static_cast<int32_t>(warps);
        wt.seg_side_head[wt.nseg] = sd * LSVD_MAX_HEADS + h;
        ++wt.nseg;
        warps += (a->num_tokens + per_warp - 1) / per_warp;
      }
    }
    if (warps > 0x7fffffffLL - 8) return LSVD_ERR_UNSUPPORTED;
    wt.warp_begin[wt.nseg] = static_cast<int32_t>(warps);
    const int64_t blocks = (warps + warps_per_block - 1) / warps_per_block;
    auto kern = a->rounding == LSVD_ROUND_TORCH ? cache_append_wide_kernel<LSVD_ROUND_TORCH>
                                                : cache_append_wide_kernel<LSVD_ROUND_TRITON>;
    LSVD_CUDA_TRY(launch_chained(kern, dim3(static_cast<unsigned>(blocks)), dim3(warps_per_block * 32), 0, st, 1, true, p, wt));
    return LSVD_OK;
  }
  const int64_t blocks = (units + warps_per_block - 1) / warps_per_block;
  if (blocks > 0x7fffffffLL) return LSVD_ERR_UNSUPPORTED;
  const dim3 grid(static_cast<unsigned>(blocks)), block(warps_per_block * 32);
  if (a->rounding == LSVD_ROUND_TORCH)
    LSVD_CUDA_TRY(launch_chained(cache_append_kernel<LSVD_ROUND_TORCH>, grid, block, 0, st, 1, true, p));
  else
    LSVD_CUDA_TRY(launch_chained(cache_append_kernel<LSVD_ROUND_TRITON>, grid, block, 0, st, 1, true, p));
  return LSVD_OK;
}
