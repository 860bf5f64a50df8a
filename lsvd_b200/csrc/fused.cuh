// Parameter blocks of the fused decode kernel (fused_decode.cu), shared with the host code that fills them
// (ffn_chain.cu for the FFN alone, layer_decode.cu for the whole decoder layer).
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "devfn.cuh"

namespace lsvd {

constexpr int kFThreads = 256;                 // one block per SM, eight warps
constexpr int kFWarps = 8;
constexpr int kFStageBytes = 128 * 128;        // a ring stage: 128 weight rows x 128 bytes of K, one TMA box
constexpr int kFStages = 8;                    // 128 KB of weights in flight per SM
constexpr int kFRing = kFStages * kFStageBytes;
constexpr int kFPanelUnits = 32;               // 128-byte K blocks of the tokens' activations held in shared memory:
constexpr int kFPanel = kFPanelUnits * 2048;   // 16 rows x 128 bytes each (a whole row up to K = 4096, else a block's own run)
constexpr int kFScratch = 18 * 1024;           // quantiser rows, Hadamard tiles, query vectors
constexpr int kFSmem = kFRing + kFPanel + kFScratch + 1024 /* alignment slack */;
constexpr int kFMaxOps = 8;
constexpr int kFMaxPieces = 8;                 // runs of units inside one row tile, per product and block: 16 TMEM columns each
constexpr int kFSyncWords = 64;                // words of the sync block (256 bytes)
constexpr int kFMaxTokens = 16;
constexpr int kFProfSlots = 24;
constexpr int kFMaxZero = 4;

// One weight-streaming product: acc[tok, ch] += sum_k a[tok, k] * w[ch, k], exact int32, added into accumulators
// that a previous stage has set to zero (blocks split K, so several of them add to one element).
struct FOp {
  int32_t n, k;                 // channels (rows of w), reduction length in bytes (a multiple of 16)
  int32_t tiles, kblocks;       // ceil(n / 128), ceil(k / 128)
  // Activations.  Products that run as one group share one panel, described by the group's first product:
  //   act_kind 0: int8 codes [m, panel_k]; 1: fp16 values [m, panel_k] + one absmax word per token, quantised while
  //   the panel is written.  panel_tma: the codes are fetched by bulk tensor copies (act_kind 0), else by the threads.
  // panel_full: the panel holds K blocks 0 .. panel_k / 128 - 1 of the row, and a product reads from block a_kb0 on;
  // otherwise (a single product with K > 4096) it holds the block's own run of units.
  int32_t act_kind, panel_full, panel_k, a_kb0, panel_tma;
  const int8_t* a;  int64_t a_stride;
  const __half* a16; int64_t a16_stride; const uint32_t* a_amax; int32_t a_amax_stride;
  int32_t* acc; int64_t acc_stride;       // accumulator of (tok, ch) at acc[tok * acc_stride + ch]
};

struct alignas(64) FMaps {
  CUtensorMap w[kFMaxOps];      // weights of product i: [n, k] int8 row-major, boxes of 128 rows x 128 bytes, 128-byte swizzle
  // int8 activations of the group that starts at product i, seen as [K block][token][128 bytes]: boxes of 8 K blocks
  // (the whole-row panel) and of one K block (a block's own run), 128-byte swizzle, absent tokens read as zero
  CUtensorMap a8[kFMaxOps];
  CUtensorMap a1[kFMaxOps];
};

// Merge of the attention partials of a (request, head) into the value-latent output (stage 2 of the decode attention).
struct FMerge {
  const float* part_ml;
  const float* part_acc;
  const int32_t* b_seq_len;
  __half* out_latent; int64_t out_latent_stride;
  uint32_t* amax;               // one word per request: max |fp16 output|
  int32_t num_heads, items_per_request, acc_per_request;
  int32_t v_off[LSVD_MAX_HEADS + 1];
  int32_t part_off[LSVD_MAX_HEADS];
  int32_t acc_off[LSVD_MAX_HEADS];
  int16_t chunk_tiles[LSVD_MAX_HEADS];
  int16_t parts[LSVD_MAX_HEADS];
};

// Cache append + query absorption for the (request, head) units of one decode step; the latents come straight
// from the latent projection's accumulators: lat = fp16((acc * x_scale[tok]) * w_scale[col]).
struct FAppend {
  const int32_t* lat_acc; int64_t lat_stride;  // [m, Rq + sum r_k + sum r_v]: query latents, K latents, V latents
  const float* x_scale; const float* w_scale;
  __half* lat_out;                             // optional fp16 copy of the latents [m, lat_stride]
  int32_t q_col, k_col, v_col;                 // first column of each group
  int32_t rank_q;                              // query latent entries per head
  const int32_t* dest_loc;                     // slot of every request's new token
  int8_t* cache_k; int64_t cache_k_row_stride; __half* scale_k; int64_t scale_k_row_stride;
  int8_t* cache_v; int64_t cache_v_row_stride; __half* scale_v; int64_t scale_v_row_stride;
  int32_t head_major;                          // cache layout: 0 = [slot][sum r], 1 = [head][slot][r_h]
  int32_t num_slots, num_heads, rounding;
  const __half* up_k; int64_t up_k_row_stride; // [sum r_k, rank_q]
  uint4* qlimb; float* qstep; int32_t* queue;  // outputs for the streaming kernel
  float score_scale;
  int32_t sum_rk;
  int32_t k_off[LSVD_MAX_HEADS + 1];
  int32_t v_off[LSVD_MAX_HEADS + 1];
};

enum : int32_t {
  FST_MERGE = 1,        // merge attention partials -> o_lat (+ absmax); barrier
  FST_PROJ = 2,         // product: output projection; barrier; y1 = dequantised + residual; barrier
  FST_QIN = 4,          // per-token input quantiser (RMSNorm / rotation / plain); barrier
  FST_LATPROJ = 8,      // product: latent projection; barrier; cache append + query absorption
  FST_FFN = 16,         // products U, W_gate, W_up | latent quantiser | V_gate, V_up | SwiGLU | rotation + quantiser | W_down | output
};

struct FusedParams {
  uint32_t* sync;               // kFSyncWords words, zero before the first launch that uses them, then left to the kernel
  int32_t* status_word;
  int32_t m, nops, stages;
  ActQuantParams q_in;          // FST_QIN
  // ranges of 16-byte words set to zero by the first stage of the program (accumulators, absmax words)
  uint4* zero_ptr[kFMaxZero]; int32_t zero_count[kFMaxZero];
  uint32_t* clear_late; int32_t clear_late_count;   // words set to zero after FST_PROJ has read them
  FOp op[kFMaxOps];
  // FST_PROJ: y1[tok, ch] = fp16(fp16((acc * a_scale(tok)) * w_scale[ch]) + residual[tok, ch]); a_scale from the absmax word
  const float* proj_w_scale; const __half* proj_residual; int64_t proj_res_stride; __half* proj_out; int64_t proj_out_stride;
  // FST_FFN
  int32_t rank, n_svd, d_ffn, d_out;
  const float* x_scale;         // [m] scale of the quantised input
  const float* U_s; const float* Vg_s; const float* Vu_s; const float* Wg_s; const float* Wu_s; const float* Wd_s;
  int8_t* z_q; float* z_s;      // latents: codes [m, 2 r], scales [m, 2]
  __half* h16;                  // hidden vector [m, d_ffn]
  int32_t hq_kind;              // 0: per-token quantiser on h (act_quant_row: plain or power-of-two rotation); 1: H_K kron H_64
  ActQuantParams hq_plain;
  HadQuantParams hq;
  uint32_t* hq_amax;            // one word per token: absmax of the rotated hidden vector (zeroed with the ranges above)
  const float* h_scale;         // [m] scale of the quantised hidden vector
  const __half* out_residual; int64_t out_res_stride; __half* out; int64_t out_stride;
  unsigned long long* prof;     // optional [gridDim.x][kFProfSlots] %globaltimer stamps at the stage boundaries
};

int launch_fused(const FusedParams& p, const FMaps& maps, const FMerge* mg, const FAppend* ap, cudaStream_t st, bool chain);
// Geometry and tensor map of product `i`: false when the kernel has no form for it on this device.
bool fused_prepare_op(FusedParams& p, FMaps& maps, int i, const int8_t* w, int64_t w_stride);
bool fused_check_group(const FusedParams& p, int k0, int nk);
void fused_prepare_panel(FusedParams& p, FMaps& maps, int k0);
bool fused_enabled();
int ffn_fill_fused(const lsvd_ffn_decode_args* a, FusedParams& p, FMaps& maps, int first_op, int zero_slot);

}  // namespace lsvd
