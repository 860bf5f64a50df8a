/*
 * lsvd_b200 -- C ABI of the B200 (sm_100a) kernels for the LSVD decode hot paths.
 *
 * Every entry point takes plain device/host pointers, sizes and strides, returns an
 * int status (0 = success) and never throws.  Kernels are enqueued on the CUDA stream
 * passed as `stream` (a cudaStream_t cast to void*; NULL = legacy default stream); no
 * entry point synchronises the device.  Unless an entry point says otherwise the caller
 * owns every buffer, including the workspace, whose size comes from the matching
 * *_workspace_bytes query.
 *
 * Reference interfaces replaced (paths inside SAI-Lab-NYU/LSVD):
 *   lsvd_cache_append        kernels/layer_bench/fd_kernel/destindex_copy_quantize_latent.py:36-50
 *   lsvd_attn_decode         kernels/layer_bench/fd_kernel/flash_decoding.py:3-57
 *                            (stage 1: flash_int8_latent_per_head_decoding_rope_stage1.py:198-250,
 *                             stage 2: flash_latent_per_head_decoding_stage2.py:52-69)
 */
#ifndef LSVD_B200_H
#define LSVD_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LSVD_ABI_VERSION 3
#define LSVD_MAX_HEADS 128      /* heads per call (per GPU shard)                     */
#define LSVD_MAX_RANK 128       /* latent entries per head; ranks are multiples of 16 */

enum {
  LSVD_OK = 0,
  LSVD_ERR_INVALID_ARG = 1,   /* NULL pointer, negative size, misaligned buffer, bad rank table */
  LSVD_ERR_UNSUPPORTED = 2,   /* a valid request this build has no kernel for                   */
  LSVD_ERR_WORKSPACE = 3,     /* workspace missing or too small                                 */
  LSVD_ERR_CUDA = 4,          /* a CUDA runtime call failed; see lsvd_last_cuda_error()         */
  LSVD_ERR_TIMEOUT = 5,       /* device status word: a bounded wait inside a kernel gave up     */
  LSVD_ERR_BOUNDS = 6         /* device status word: an index was out of range and was skipped  */
};

int lsvd_abi_version(void);
const char* lsvd_status_string(int code);
/* cudaError_t of the most recent failing CUDA call made by this library on the calling thread. */
int lsvd_last_cuda_error(void);

/* Rounding used when fp16 latents become int8 cache entries.
 *   LSVD_ROUND_TORCH  : x/scale evaluated in fp16, round half to even -- the reference's PyTorch quantiser
 *                       (kernels/layer_bench/benchmark_triton_int8_layer.py:103-113), normative.
 *   LSVD_ROUND_TRITON : x/scale in fp32, round half away from zero -- the reference's Triton append kernel
 *                       (kernels/layer_bench/fd_kernel/destindex_copy_quantize_latent.py:26-29).        */
enum { LSVD_ROUND_TORCH = 0, LSVD_ROUND_TRITON = 1 };

/* Layout of the int8 latent cache (K and V alike) and of its fp16 scales.
 *   LSVD_CACHE_SLOT_MAJOR : cache [N_slots][sum r] (head h in bytes rank_off[h] .. rank_off[h+1]-1 of a row), scales
 *                           [N_slots][H] -- with a uniform rank the reference's [N_slots, H, R] / [N_slots, H] tensors
 *                           (kernels/layer_bench/benchmark_triton_int8_layer.py:116-149).
 *   LSVD_CACHE_HEAD_MAJOR : cache [H][N_slots][r_h] (head h starts at byte rank_off[h] * N_slots, slot s of it at
 *                           + s * r_h), scales [H][N_slots].  The rows a head reads for consecutive slots are then
 *                           contiguous, which is what the streaming kernel's loads want; same values either way.
 *                           Row strides of the argument blocks are ignored in this layout.                          */
enum { LSVD_CACHE_SLOT_MAJOR = 0, LSVD_CACHE_HEAD_MAJOR = 1 };

/* ---------------------------------------------------------------------------------------------
 * Latent KV-cache append / quantise.
 * Replaces destindex_copy_quantize_latent(latent, dest_loc, cache, cache_scale)
 * (kernels/layer_bench/fd_kernel/destindex_copy_quantize_latent.py:36-50); one call handles K and V.
 *
 * Cache layout: one row per slot; head h of a row occupies bytes rank_off[h] .. rank_off[h+1]-1, so a
 * uniform rank R gives the reference's [N_slots, H, R] tensor.  Scales: [N_slots, H] fp16.
 * ------------------------------------------------------------------------------------------- */
typedef struct lsvd_append_tensor {
  const void* latent;            /* device fp16; element (t, h, i) at latent[t*token_stride + head_off[h] + i]   */
  int64_t token_stride;          /* elements                                                                       */
  const int64_t* head_off;       /* HOST array [num_heads] of element offsets, or NULL for rank_off (packed rows) */
  const int32_t* rank_off;       /* HOST array [num_heads+1], multiples of 16, rank_off[0] = 0                    */
  int8_t* cache;                 /* device int8                                                                    */
  int64_t cache_row_stride;      /* bytes between consecutive slots                                                */
  void* cache_scale;             /* device fp16                                                                    */
  int64_t scale_row_stride;      /* elements between consecutive slots                                             */
} lsvd_append_tensor;

typedef struct lsvd_append_args {
  int32_t num_tokens;
  int32_t num_heads;
  int32_t rounding;              /* LSVD_ROUND_*                                                                   */
  int32_t num_slots;             /* rows in the cache; a dest_loc outside [0, num_slots) is skipped and reported   */
  const int32_t* dest_loc;       /* device int32 [num_tokens]                                                      */
  lsvd_append_tensor k;          /* k.latent == NULL skips K                                                       */
  lsvd_append_tensor v;          /* v.latent == NULL skips V                                                       */
  int32_t* status_word;          /* device int32 or NULL; receives LSVD_ERR_BOUNDS (never cleared by the library)  */
  int32_t cache_layout;          /* LSVD_CACHE_*                                                                   */
} lsvd_append_args;

int lsvd_cache_append(const lsvd_append_args* args, void* stream);

/* Advance the batch bookkeeping of a decode loop by one token, on the device (no host round trip between steps, so a
 * step can be replayed as a CUDA graph): b_seq_len[b] += 1 and mem_index[b] = req_to_token[b_req_idx[b], b_seq_len[b] - 1],
 * the slot the next step appends to.  The fields are those of the reference's MockInferState
 * (kernels/layer_bench/ffn_kernel/baseline_kernel.py:38-53), which the reference rebuilds on the host for every step.
 * A length that would pass max_len is left alone and reported as LSVD_ERR_BOUNDS in the status word.  With period > 0 a
 * request that reaches base_len + period starts over at base_len (benchmarks that replay more steps than the context
 * they reserved). */
int lsvd_decode_advance(int32_t* b_seq_len, int32_t* mem_index, const int32_t* req_to_token, int64_t req_to_token_stride,
                        const int32_t* b_req_idx, int32_t batch, int32_t base_len, int32_t period, int32_t max_len,
                        int32_t* status_word, void* stream);

/* ---------------------------------------------------------------------------------------------
 * int8 latent flash-decoding attention, one query token per request ("absorb" form).
 * Replaces token_decode_attention_flash_int8_latent_per_head_decoding_rope
 * (kernels/layer_bench/fd_kernel/flash_decoding.py:3-57) for the rotary-free configuration:
 *   q~   = B_k q                                   query folded into the per-head K up-factor
 *   s_t  = sm_scale * scale_k[t,h] * (z_k[t,h] . q~_h)
 *   p    = softmax_t(s)                            split over the sequence, merged by log-sum-exp
 *   o_lat= sum_t p_t * scale_v[t,h] * z_v[t,h]     (written to out_latent if not NULL)
 *   o    = B_v^T o_lat                             (written to out if not NULL)
 * Request b reads the cache rows req_to_token[b_req_idx[b], 0 .. b_seq_len[b]-1].  A request of
 * length 0 gets zeros (the reference leaves 0/0 there).  num_q_heads == num_kv_heads only.
 * up_k and up_v are weights: the kernels may read them before the work queued ahead of the call on `stream` has
 * finished (they start under programmatic stream serialisation), so they must not be produced by that work.
 * ------------------------------------------------------------------------------------------- */
typedef struct lsvd_attn_decode_args {
  int32_t batch;
  int32_t num_heads;
  int32_t head_dim;              /* multiple of 8, <= 256                                                          */
  int32_t max_len_in_batch;      /* upper bound of b_seq_len (sizes the grid, like the reference)                  */
  float sm_scale;                /* <= 0 selects 1/sqrt(head_dim)                                                  */
  int32_t num_slots;             /* rows in the cache, for the bounds guard                                        */
  const void* q;                 /* device fp16; (b, h, d) at q[b*q_stride_b + h*q_stride_h + d]                   */
  int64_t q_stride_b, q_stride_h;
  const int32_t* k_off;          /* HOST [num_heads+1] byte offsets of the heads inside a K cache row              */
  const int32_t* v_off;          /* HOST [num_heads+1]                                                             */
  const int8_t* cache_k;         /* device; 16-byte aligned, row stride a multiple of 16                           */
  int64_t cache_k_row_stride;
  const void* scale_k;           /* device fp16 [N_slots, H]                                                       */
  int64_t scale_k_row_stride;
  const int8_t* cache_v;
  int64_t cache_v_row_stride;
  const void* scale_v;
  int64_t scale_v_row_stride;
  const void* up_k;              /* device fp16 [sum r_k, head_dim]: row k_off[h]+i is latent entry i of head h    */
  int64_t up_k_row_stride;       /* elements                                                                       */
  const void* up_v;              /* device fp16 [sum r_v, head_dim]; may be NULL when out is NULL                  */
  int64_t up_v_row_stride;
  const int32_t* req_to_token;   /* device int32 [*, req_to_token_stride]                                          */
  int64_t req_to_token_stride;
  const int32_t* b_req_idx;      /* device int32 [batch]                                                           */
  const int32_t* b_seq_len;      /* device int32 [batch]                                                           */
  void* out;                     /* device fp16 (b, h, d) at out[b*out_stride_b + h*out_stride_h + d], or NULL     */
  int64_t out_stride_b, out_stride_h;
  void* out_latent;              /* device fp16 (b, v_off[h]+i) at out_latent[b*out_latent_stride_b + ...], or NULL */
  int64_t out_latent_stride_b;
  void* workspace;               /* device, 256-byte aligned                                                       */
  size_t workspace_bytes;
  int32_t* status_word;          /* device int32 or NULL                                                           */
  void* ev_stream_begin;         /* optional cudaEvent_t pair recorded around the streaming kernel alone (the      */
  void* ev_stream_end;           /* launch that reads the cache), for roofline measurements; NULL = not recorded   */
  int32_t cache_layout;          /* LSVD_CACHE_*                                                                   */
  int32_t req_to_token_rows;     /* rows of req_to_token: a b_req_idx outside [0, rows) is skipped and reported as     */
                                 /* LSVD_ERR_BOUNDS (0: not checked).  A b_seq_len above max_len_in_batch is treated   */
                                 /* as max_len_in_batch and reported the same way.                                      */
} lsvd_attn_decode_args;

/* Bytes of workspace lsvd_attn_decode needs for this problem on the current device. */
size_t lsvd_attn_decode_workspace_bytes(int32_t batch, int32_t num_heads, int32_t sum_rank_k,
                                        int32_t sum_rank_v, int32_t max_len_in_batch);
int lsvd_attn_decode(const lsvd_attn_decode_args* args, void* stream);

/* Launch geometry chosen for a problem (for reports and tests): work items per request, the byte size
 * an item aims for, thread blocks.  Returns a status. */
int lsvd_attn_decode_plan(int32_t batch, int32_t num_heads, const int32_t* k_off, const int32_t* v_off,
                          int32_t max_len_in_batch, int32_t* items_per_request, int32_t* item_bytes,
                          int32_t* num_blocks);

/* Decode attention without a caller workspace (no counterpart in the reference; added for hosts that cannot
 * allocate device memory on the decode path: servers whose memory pool owns the whole GPU, plugins inside another
 * runtime's budget, steps recorded while allocation is off limits).  Same arguments and results as
 * lsvd_attn_decode; `workspace` and `workspace_bytes` are ignored.  The scratch is a fixed array of
 * LSVD_STATIC_SCRATCH_BYTES inside the library's device image: every GPU that loads the library holds it until
 * the process exits, and every call on that GPU uses the same bytes.
 *   - A problem whose scratch need exceeds the array returns LSVD_ERR_WORKSPACE and launches nothing
 *     (the need grows with batch x (heads + context / item size); batch 16 x context 4096 at the 7B shape takes ~3 MB).
 *   - The call makes no cudaMalloc / cudaFree and uses no allocating library routine.  The first call on a
 *     device looks up the array's device address (cudaGetSymbolAddress); make that first call outside any
 *     stream capture.  The address is kept for the life of the process (no cudaDeviceReset while the library is loaded).
 *   - The array keeps what the last call left in it; the one word that must start at zero (the work counter)
 *     is cleared on the stream by the first kernel of each call.  Two calls that overlap on the GPU (different
 *     streams, no ordering) race on the scratch: order them, or give one of them lsvd_attn_decode with its own
 *     workspace. */
#define LSVD_STATIC_SCRATCH_BYTES (8u << 20)
size_t lsvd_attn_decode_static_scratch_bytes(void);
int lsvd_attn_decode_static(const lsvd_attn_decode_args* args, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Decode attention in the reference's own form ("rope_recon"): int8 K up-factor, keys rebuilt per token and
 * rotated at their logical position, uniform ranks, grouped-query heads.  Replaces
 * token_decode_attention_flash_int8_latent_per_head_decoding_rope (kernels/layer_bench/fd_kernel/flash_decoding.py:3-57),
 * i.e. stage 1 (flash_int8_latent_per_head_decoding_rope_stage1.py:32-250) + stage 2
 * (flash_latent_per_head_decoding_stage2.py:7-69):
 *   K_t = fp16((z_k[t] . wk) * scale_k[t] * wk_scale), rotated at position t; q rotated at position L - 1 (fp16);
 *   o[b, h, :] = sum_t softmax_t(q_rot . K_rot / sqrt(D)) * scale_v[t] * z_v[t]       fp16 [B, H, rank_v]
 * The kv head of query head h is h / (num_q_heads / num_kv_heads).  A request of length 0 gets zeros.
 * ------------------------------------------------------------------------------------------- */
typedef struct lsvd_attn_rope_args {
  int32_t batch, num_q_heads, num_kv_heads;
  int32_t head_dim;              /* 32, 64 or 128                                                                 */
  int32_t rank_k, rank_v;        /* multiples of 16, <= LSVD_MAX_RANK                                            */
  const void* q;                 /* device fp16 (b, h, d) at q[b*q_stride_b + h*q_stride_h + d]                  */
  int64_t q_stride_b, q_stride_h;
  const int8_t* cache_k;         /* device int8 (slot, kv head, rank) at slot*slot_stride + head*head_stride + r */
  int64_t cache_k_slot_stride, cache_k_head_stride;
  const void* scale_k;           /* device fp16 (slot, kv head) at slot*scale_k_slot_stride + head               */
  int64_t scale_k_slot_stride;
  const int8_t* cache_v;
  int64_t cache_v_slot_stride, cache_v_head_stride;
  const void* scale_v;
  int64_t scale_v_slot_stride;
  const int8_t* wk;              /* device int8 [rank_k, num_kv_heads*head_dim], rows 16-byte aligned            */
  int64_t wk_row_stride;
  const void* wk_scale;          /* device fp16 [num_kv_heads*head_dim]                                          */
  const int32_t* req_to_token;   /* device int32 [requests, >= max_len_in_batch]                                 */
  int64_t req_to_token_stride;
  const int32_t* b_req_idx;      /* device int32 [batch]                                                         */
  const int32_t* b_seq_len;      /* device int32 [batch]                                                         */
  int32_t num_slots;
  int32_t max_len_in_batch;
  int32_t block_seq;             /* tokens per run (the reference's BLOCK_SEQ, 256); multiple of 16              */
  float sm_scale;                /* <= 0: 1 / sqrt(head_dim)                                                     */
  float rope_theta;              /* <= 0: 10000                                                                  */
  void* out;                     /* device fp16 (b, h, rank_v) at out[b*out_stride_b + h*out_stride_h + i]       */
  int64_t out_stride_b, out_stride_h;
  void* workspace;               /* device, 256-byte aligned                                                     */
  size_t workspace_bytes;
  int32_t* status_word;          /* device int32 or NULL                                                         */
} lsvd_attn_rope_args;
size_t lsvd_attn_decode_rope_workspace_bytes(int32_t batch, int32_t num_q_heads, int32_t head_dim, int32_t rank_v,
                                             int32_t max_len_in_batch, int32_t block_seq);
int lsvd_attn_decode_rope(const lsvd_attn_rope_args* args, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Hybrid SVD/RTN FFN, decode (1..64 tokens): building blocks and the fused chain.
 * Semantics follow fake_quant/utils/hybrid_ffn_utils.py:956-984 (HybridSVDQuantFFN.forward) with real
 * int8 codes: activations are quantised per token (fake_quant/utils/quant_utils.py:201-212,30-33),
 * weights per output channel (quant_utils.py:436-498), every matrix product is an exact
 * int8 x int8 -> int32 contraction, and fp16 roundings sit where the reference's fp16 tensors are.
 * ------------------------------------------------------------------------------------------- */

/* Per-token symmetric int8 quantisation of fp16 rows, optionally after a Hadamard rotation of the row:
 *   sign != NULL : x <- FWHT(x * sign) / sqrt(cols)   (x @ random_hadamard_matrix, fake_quant/utils/hadamard_utils.py:99-104)
 *   fwht  != 0   : x <- FWHT(x) / sqrt(cols)          (matmul_hadU_cuda with K == 1, hadamard_utils.py:106-109)
 * then scale = absmax / 127 (1 for a zero row), q = clamp(rne(x / scale), -128, 127).  cols <= 16384; a
 * rotation needs cols to be a power of two.  Replaces ActQuantizer.find_params + quantize.
 * There is no separate entry for the rotation alone (matmul_hadU_cuda, fake_quant/utils/hadamard_utils.py:106-113): the
 * rotated fp16 row is the optional `x_rot` output here (K == 1), `y` of lsvd_hadamard_quant (K > 1) and `y` of
 * lsvd_heads_hadamard_quant (across heads); the codes and scales are written as well and may be ignored. */
typedef struct lsvd_act_quant_args {
  int32_t rows, cols;
  const void* x;                 /* device fp16 [rows, cols]                                        */
  int64_t x_row_stride;          /* elements                                                        */
  const void* sign;              /* device fp16 [cols] of +-1, or NULL                              */
  int32_t fwht;                  /* rotate without signs                                            */
  int8_t* q;                     /* device int8 [rows, cols]                                        */
  int64_t q_row_stride;
  float* scale;                  /* device fp32 [rows]                                              */
  void* x_rot;                   /* optional device fp16 [rows, cols] (contiguous): the row as quantised
                                    (after the rotation or the normalisation)                        */
  const void* norm_weight;       /* device fp16 [cols] or NULL: RMSNorm(x) * weight first, fp32 statistics and fp16
                                    products as kernels/layer_bench/ffn_kernel/utils.py:560-565 (not with `sign`) */
  float norm_eps;
  const float* x_f32;            /* optional device fp32 [rows, cols] (contiguous): the row is fp16(x_f32 + add) instead of
                                    x -- a partial sum that came back from an all-reduce plus its residual (tensor-parallel
                                    output projection); not with a rotation                                              */
  const void* add;               /* optional device fp16 [rows, cols] (contiguous), with x_f32                            */
  void* sum_out;                 /* optional device fp16 [rows, cols] (contiguous): receives fp16(x_f32 + add)            */
  void* fake;                    /* optional device fp16 [rows, cols] (contiguous): the fake-quantised row fp16(scale * code),
                                    what ActQuantizer.forward returns (fake_quant/utils/quant_utils.py:141-148)           */
} lsvd_act_quant_args;
int lsvd_act_quant(const lsvd_act_quant_args* args, void* stream);

/* Online Hadamard of the FFN hidden vector followed by per-token int8 quantisation:
 *   y = (H_K kron H_{cols/K}) x / sqrt(cols), rounded to fp16 after the power-of-two part and after the
 *   had_K product (matmul_hadU_cuda, fake_quant/utils/hadamard_utils.py:106-113), then quantised as above.
 * K > 1, K <= 256, cols / K a power of two in [8, 128]. */
typedef struct lsvd_hadamard_quant_args {
  int32_t rows, cols, K;
  const void* x;                 /* device fp16 [rows, cols]                                        */
  int64_t x_row_stride;
  const void* had_K_packed;      /* device buffer made by lsvd_hadamard_pack from had_K [K, K]      */
  int8_t* q;
  int64_t q_row_stride;
  float* scale;                  /* device fp32 [rows]                                              */
  void* y;                       /* optional device fp16 [rows, cols] (contiguous): the rotated row */
} lsvd_hadamard_quant_args;
int lsvd_hadamard_quant(const lsvd_hadamard_quant_args* args, void* stream);
/* One-time preparation of the K x K factor (device fp16, row-major, the `had_K` buffer of the reference's
 * modules, fake_quant/utils/hadamard_utils.py:7-69) into the tensor-core fragment order the kernel reads:
 * lsvd_hadamard_packed_bytes(K) bytes, 16-byte aligned. */
size_t lsvd_hadamard_packed_bytes(int32_t K);
int lsvd_hadamard_pack(const void* had_K, int32_t K, void* packed, void* stream);

/* Hadamard across heads followed by per-token int8 quantisation: a row [heads * head_dim] is seen as
 * [heads][head_dim] and every column is transformed over its `heads` entries (a power of two up to 64), scale
 * 1 / sqrt(heads), fp32 inside and fp16 out; then the row is quantised as in lsvd_act_quant.  The online
 * rotation in front of o_proj: ActQuantWrapper.forward with online_partial_had
 * (fake_quant/utils/quant_utils.py:302-322; K == 1 without had_K, K == heads with it).  head_dim even, <= 256. */
typedef struct lsvd_heads_hadamard_quant_args {
  int32_t rows, heads, head_dim;
  const void* x;                 /* device fp16 [rows, heads * head_dim]                            */
  int64_t x_row_stride;
  int8_t* q;                     /* device int8 [rows, heads * head_dim]                            */
  int64_t q_row_stride;
  float* scale;                  /* device fp32 [rows]                                              */
  void* y;                       /* optional device fp16 [rows, heads * head_dim] (contiguous): the rotated row */
  const void* had_K;             /* NULL, or device fp16 [heads, heads] (+-1): y = (had_K x) / sqrt(heads) with the     */
                                 /* reference's two fp16 roundings, for head counts that are not a power of two (<= 64) */
} lsvd_heads_hadamard_quant_args;
int lsvd_heads_hadamard_quant(const lsvd_heads_hadamard_quant_args* args, void* stream);

/* Row-wise gather of byte segments: for every row r < rows and segment s < nseg (at most 32),
 *   dst[r * dst_row_stride + dst_off[s] .. + len[s])  =  src[src_off[s] + r * src_row_stride[s] .. + len[s])
 * (all in bytes, multiples of 16; the four tables are HOST arrays).  The tensor-parallel FFN uses it to lay the
 * all-gathered [rank][token][svd slice | rtn slice] pieces of the hidden vector out in the global [SVD | RTN] channel
 * order in one pass.  No counterpart in the reference (it has no tensor parallelism). */
int lsvd_gather_segments(const void* src, void* dst, int64_t dst_row_stride_bytes, int32_t rows, int32_t nseg,
                         const int64_t* src_off_bytes, const int64_t* src_row_stride_bytes, const int64_t* dst_off_bytes,
                         const int32_t* len_bytes, void* stream);

/* The same rotation when the heads are sharded over tensor-parallel ranks.  x fp16 [rows, n_local * head_dim] holds the
 * heads head_ids[0 .. n_local) (HOST array of global head indices); out fp32 [rows, heads * head_dim] (contiguous) receives
 * this rank's terms of every output head, already scaled by 1 / sqrt(heads): out[h', d] = s * sum_j S[h', head_ids[j]] x[j, d]
 * with S the Sylvester signs (heads a power of two) or had_K (device fp16 [heads, heads] of +-1).  The sum of the ranks'
 * rows (one all-reduce) is the rotated row; lsvd_act_quant with x_f32 rounds it to fp16 and quantises it.  No
 * counterpart in the reference (it has no tensor parallelism); the single-GPU form is lsvd_heads_hadamard_quant. */
int lsvd_heads_hadamard_partial(const void* x, int64_t x_row_stride, const int32_t* head_ids, int32_t n_local,
                                int32_t heads, int32_t head_dim, const void* had_K, float* out, int32_t rows, void* stream);

/* Weight-streaming W8A8 product for 1..64 tokens: acc[m, n] = sum_k a[m, k] * w[n, k] (int32, exact),
 * optionally for a second weight matrix w2 (with its own activations a2, or the same ones) in the same pass.
 *   epilogue 0: out[m, out_col + n] = fp16((acc * a_scale[m]) * w_scale[n])              (a quantised Linear)
 *   epilogue 1: g = that for (w, a), u = that for (w2, a2); out = fp16(fp16(silu(g)) * u) (gate/up pair)
 *   epilogue 2: the same pair with g, u kept in fp32: out = fp16(u * (g * sigmoid(g))), the convention of
 *               kernels/layer_bench/ffn_kernel/mix_ffn_kernel.py:353-362,1885-1889 (forms 0 and 3 only)
 * With row_absmax the call also folds max |fp32 value before the fp16 rounding| of every token into a device
 * word per token (atomic maximum on the float's bit pattern; the caller zeroes it), which is what the reference's
 * tiled kernels hand to their next quantiser (mix_ffn_kernel.py:1229-1232, 1894-1895).
 * n and k multiples of 16, rows 16-byte aligned.  Replaces the reference's fp16 Linear on
 * fake-quantised tensors (ActQuantWrapper.forward, fake_quant/utils/quant_utils.py:319-333) and, on the kernel
 * side, the w8a8 matmul + dequant kernels of kernels/layer_bench/ffn_kernel/mix_ffn_kernel.py:968-1021,1292-1338. */
typedef struct lsvd_gemv_args {
  int32_t m, n, k;
  const int8_t* w;  int64_t w_row_stride;  const float* w_scale;
  const int8_t* w2; int64_t w2_row_stride; const float* w2_scale;     /* w2 == NULL: single product        */
  const int8_t* a;  int64_t a_row_stride;  const float* a_scale;  int64_t a_scale_stride;
  const int8_t* a2; int64_t a2_row_stride; const float* a2_scale; int64_t a2_scale_stride;   /* a2 == NULL: use a */
  int32_t epilogue;
  void* out;                     /* device fp16                                                      */
  int64_t out_row_stride;
  int32_t out_col;
  int32_t* acc_out;              /* optional device int32 [m, n] raw accumulators of (w, a)          */
  int32_t* acc2_out;             /* optional, of (w2, a2)                                            */
  const void* residual;          /* optional device fp16 [m, n] added to the fp16 result (fp16 add)  */
  int64_t residual_row_stride;
  int32_t* status_word;          /* device int32 or NULL: LSVD_ERR_TIMEOUT if a pipeline wait of the   */
                                 /* TMA-fed form ran out; the output is then incomplete               */
  int32_t form;                  /* 0: chosen by size (2 beyond 32 tokens on large matrices, else 3);    */
                                 /* 1: persistent TMA-fed kernel with K split over warps, m <= 16 only   */
                                 /*    (LSVD_ERR_UNSUPPORTED beyond); 2: TMA-fed kernel whose warps      */
                                 /*    share the token rows (built for 17..64 tokens, valid for any m);   */
                                 /* 3: register-fed kernel for any m.  Same values in every form.        */
  uint32_t* row_absmax;          /* optional device words [m * row_absmax_stride]: see above (forms 0, 3)  */
  int64_t row_absmax_stride;     /* words between two tokens                                              */
  int32_t absmax_split;          /* 0: one word per token; else channels >= absmax_split (a multiple of  */
                                 /* 16) go to the token's second word                                     */
  int32_t prefetch_weights;      /* register-fed form: every block asks for its weight rows (L2 prefetch) before */
                                 /* it waits for the kernel launched before it on the stream; pays when the       */
                                 /* call follows a short kernel (measured: 126 -> 120 us for the mixffn step)      */
  float* out_f32;                /* optional device fp32 [m, n] (single product, forms 0 and 3): (acc * a_scale) * w_scale  */
                                 /* with no fp16 rounding -- the partial sum a row-parallel rank sends to the all-reduce  */
} lsvd_gemv_args;
int lsvd_w8a8_gemv(const lsvd_gemv_args* args, void* stream);

/* out[m, n] = fp16(fp16((acc[m, n] * a_scale[m]) * w_scale[n]) + residual[m, n]): the epilogue of lsvd_w8a8_gemv applied to
 * accumulators that were summed over tensor-parallel ranks first (int32, exact).  acc contiguous; residual may be NULL. */
int lsvd_dequant_residual(const int32_t* acc, const float* a_scale, const float* w_scale, const void* residual,
                          int64_t residual_row_stride, void* out, int64_t out_row_stride, int32_t m, int32_t n, void* stream);

/* Ragged per-head up-projection of a latent, the arithmetic of SVDLinear.forward for per-head factors
 * (fake_quant/utils/svd_utils.py:1978-2027):
 *   y[t, h * cout + c] = fp16(sum_r A_h[c, r] * z[t, rank_off[h] + r]) (+ bias[h * cout + c], added in fp16)
 * z fp16 [tokens, >= rank_off[num_heads]]; factors fp16: A_0, A_1, ... one after the other, A_h [cout, r_h] row-major with
 * r_h = rank_off[h + 1] - rank_off[h] (rank_off: HOST array of num_heads + 1 ints, rank_off[0] = 0); y fp16
 * [tokens, >= num_heads * cout]; strides in elements.  Each head reads its own r_h columns: nothing is padded to the
 * largest rank.  fp32 accumulation. */
int lsvd_per_head_up(const void* z, int64_t z_row_stride, const void* factors, const int32_t* rank_off, const void* bias,
                     void* y, int64_t y_row_stride, int32_t tokens, int32_t num_heads, int32_t cout, void* stream);

/* ---------------------------------------------------------------------------------------------
 * The whole hybrid SVD/RTN FFN for a decode batch (1..64 tokens) in one call: the chain of lsvd_act_quant,
 * lsvd_w8a8_gemv and lsvd_hadamard_quant launches that replaces HybridSVDQuantFFN.forward
 * (fake_quant/utils/hybrid_ffn_utils.py:956-984):
 *   x_q = quant([rmsnorm | rotate](x));  z = quant(U x_q) (gate and up latents separately);
 *   h = [ silu(Vg z_g) * (Vu z_u) | silu(Wg x_q) * (Wu x_q) ];  out = Wd quant(hadamard(h)) [+ residual]
 * Weights are int8 [out, in] row-major with one fp32 scale per output channel; all of them contiguous.
 * With overlap != 0 the RTN pair runs on a second stream owned by the library (created on first use, one per
 * device) and rejoins `stream` before the Hadamard step, also inside a stream capture.  That stream and its two
 * events are shared by every call on the device: with overlap != 0 the entry point is for ONE calling thread and ONE
 * caller stream per device at a time (concurrent callers must pass overlap = 0 or serialise their calls).
 * ------------------------------------------------------------------------------------------- */
typedef struct lsvd_ffn_decode_args {
  int32_t m, d_in, d_ffn, d_out, rank, n_svd;   /* d_ffn = n_svd (SVD channels, first) + RTN channels            */
  int32_t K;                     /* order of the non-power-of-two Hadamard factor (1: none)                       */
  int32_t online_had;            /* rotate the hidden vector before quantising it                                 */
  int32_t overlap;               /* RTN gate/up pair on the library's second stream                               */
  const void* x;                 /* device fp16 [m, d_in]                                                         */
  int64_t x_row_stride;
  const void* had_sign;          /* device fp16 [d_in] of +-1 (input rotation), or NULL                           */
  const void* norm_weight;       /* device fp16 [d_in] or NULL (RMSNorm inside the first quantiser; not with had_sign) */
  float norm_eps;
  const int8_t* U_q;  const float* U_s;          /* [2 rank, d_in]: gate latent rows, then up latent rows         */
  const int8_t* Vg_q; const float* Vg_s;         /* [n_svd, rank]                                                 */
  const int8_t* Vu_q; const float* Vu_s;
  const int8_t* Wg_q; const float* Wg_s;         /* [d_ffn - n_svd, d_in]                                         */
  const int8_t* Wu_q; const float* Wu_s;
  const int8_t* Wd_q; const float* Wd_s;         /* [d_out, d_ffn], input columns [SVD | RTN]                     */
  const void* had_K_packed;      /* from lsvd_hadamard_pack, when K > 1                                           */
  const void* residual;          /* optional device fp16 [m, d_out]                                               */
  int64_t residual_row_stride;
  void* out;                     /* device fp16 [m, d_out]                                                        */
  int64_t out_row_stride;
  void* workspace;               /* device, 256-byte aligned, lsvd_ffn_decode_workspace_bytes(m, d_in, d_ffn, rank, d_out) */
  size_t workspace_bytes;
  int32_t* status_word;          /* device int32 or NULL                                                          */
  int32_t fused;                 /* non-zero: run the block as ONE persistent kernel (at most 16 tokens, rank a       */
                                 /* multiple of 128 and <= 1024, d_in <= 4096, Hadamard factor of 64-entry blocks):   */
                                 /* weights stream through a TMA ring into tcgen05.mma (weights as the 128-row        */
                                 /* operand, tokens as 16 columns), stages meet at grid barriers with bounded waits.   */
                                 /* Shapes outside its forms take the chain of launches.  The workspace must then     */
                                 /* have been set to zero once, before its first use (it holds the barrier counters,   */
                                 /* which the kernel maintains from call to call); calls that share a workspace must   */
                                 /* be ordered on a stream.  `overlap` is ignored.  Same values as the chain; slower   */
                                 /* than the chain on B200 at the 7B shape as measured (78 against 56 us), hence opt-in.   */
} lsvd_ffn_decode_args;
size_t lsvd_ffn_decode_workspace_bytes(int32_t m, int32_t d_in, int32_t d_ffn, int32_t rank, int32_t d_out);
int lsvd_ffn_decode(const lsvd_ffn_decode_args* args, void* stream);
/* 1 when lsvd_ffn_decode would run these arguments as the single persistent kernel, 0 when it would take the chain. */
int lsvd_ffn_decode_is_fused(const lsvd_ffn_decode_args* args);
/* Performance analysis of the persistent kernels: with a device buffer of [SM count][16] 64-bit words set here, every
 * block writes the GPU's global timer (ns) at each stage boundary of every later launch (last launch wins); NULL turns
 * it off.  Process-wide, not thread-safe: a tool for benchmarks, not for serving. */
void lsvd_fused_set_profile(void* device_buffer);

/* ---------------------------------------------------------------------------------------------
 * W8A8 GEMM for prefill / large batches on tcgen05 (kind::i8, accumulators in tensor memory, TMA-fed).
 * acc[m, n] = sum_k a[m, k] * w[n, k] (int32, exact); out[m, out_col + n] = fp16((acc * a_scale[m]) * w_scale[n]);
 * with w2: a gate/up pair sharing the activations, out = fp16(fp16(silu(gate)) * up).  Same values as
 * lsvd_w8a8_gemv for any m.  n and k multiples of 16, rows 16-byte aligned.  Replaces the int8 tl.dot kernels of
 * kernels/layer_bench/ffn_kernel/mix_ffn_kernel.py:410-500,903-1021,1152-1338 at prefill sizes.
 * ------------------------------------------------------------------------------------------- */
typedef struct lsvd_i8gemm_args {
  int32_t m, n, k;
  const int8_t* a;  int64_t a_row_stride;  const float* a_scale;     /* activations [m, k], scale per row      */
  const int8_t* w;  int64_t w_row_stride;  const float* w_scale;     /* weights [n, k], scale per row           */
  const int8_t* w2; int64_t w2_row_stride; const float* w2_scale;    /* NULL: single product                    */
  void* out;                     /* device fp16, or NULL when only accumulators are wanted            */
  int64_t out_row_stride;
  int32_t out_col;
  int32_t* acc_out;              /* optional device int32 [m, n] (single product only)                */
  int32_t* status_word;          /* device int32 or NULL: LSVD_ERR_TIMEOUT if a bounded wait gave up  */
  int64_t a_scale_stride;        /* elements between the scales of consecutive rows; 0 means 1        */
  const void* gate;              /* single product only, optional device fp16: the result becomes      */
  int64_t gate_row_stride;       /*   fp16(fp16(silu(gate[m, gate_col + n])) * value)  (an "up" product */
  int32_t gate_col;              /*   whose gate was computed before, with other activations)          */
  const void* residual;          /* single product only, optional device fp16 [m, n]: fp16 add         */
  int64_t residual_row_stride;
  const int8_t* a2;              /* gate/up pair only, optional: the up matrix' own activations [m, k]  */
  int64_t a2_row_stride;         /*   (the SVD branch: gate and up read different latents)              */
  const float* a2_scale;
  int64_t a2_scale_stride;
} lsvd_i8gemm_args;
int lsvd_i8gemm_prefill(const lsvd_i8gemm_args* args, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Quantisers of the reference's "mixffn" W8A8 pipeline (kernels/layer_bench/ffn_kernel/mix_ffn_kernel.py), whose
 * conventions differ from the fake_quant ones: scale = max(absmax / 127, 1e-8) with the absmax of the fp32 values,
 * codes = clamp(trunc(v / scale +- 0.5), -128, 127) (round half away from zero), divisions in fp32.
 * Together with lsvd_w8a8_gemv (epilogue 2, row_absmax) they replace its eleven Triton kernels:
 *   lsvd_mix_rmsnorm_quant   _rmsnorm_quant_kernel (:101-165)
 *   lsvd_w8a8_gemv           the tl.dot kernels and their dequantising / SwiGLU epilogues (:324-375, :1156-1342, :1822-1895)
 *   lsvd_mix_group_quant     _dual_quantize_with_scale_vec_kernel, _dual_quantize_with_shared_scale_vec_kernel (:1070-1150)
 *   lsvd_mix_acc_quant       _svd_rank_dequant_quant_down_kernel (:795-837)
 * ------------------------------------------------------------------------------------------- */
typedef struct lsvd_mix_rmsnorm_quant_args {
  int32_t rows, cols;
  const void* x;                 /* device fp16 [rows, cols]                                                     */
  int64_t x_row_stride;
  const void* norm_weight;       /* device fp16 [cols]                                                           */
  float eps;
  int8_t* q;                     /* codes of (x * rsqrt(mean x^2 + eps)) * weight, all in fp32                    */
  int64_t q_row_stride;
  float* scale;                  /* device fp32 [rows]: the scale after its rounding to fp16, which is the value  */
                                 /* the reference stores and later stages dequantise with (:34, :149-150)         */
  uint32_t* clear_words;         /* optional: clear_per_row words per row are set to zero (the row_absmax words   */
  int32_t clear_per_row;         /* of the products that follow)                                                  */
} lsvd_mix_rmsnorm_quant_args;
int lsvd_mix_rmsnorm_quant(const lsvd_mix_rmsnorm_quant_args* args, void* stream);

typedef struct lsvd_mix_group_quant_args {
  int32_t rows, cols;
  int32_t split;                 /* columns [0, split) use the token's first absmax word, [split, cols) the second */
                                 /* (split == cols: one group)                                                    */
  int32_t shared;                /* non-zero: both groups use the larger of the two maxima (:2075)                 */
  const void* x;                 /* device fp16 [rows, cols]                                                      */
  int64_t x_row_stride;
  const uint32_t* absmax;        /* device words written through lsvd_gemv_args.row_absmax                         */
  int64_t absmax_stride;         /* words between two tokens                                                      */
  int8_t* q;
  int64_t q_row_stride;
  float* scale;                  /* device fp32: scale[row * scale_stride + group] (group 0 only when shared)      */
  int64_t scale_stride;
} lsvd_mix_group_quant_args;
int lsvd_mix_group_quant(const lsvd_mix_group_quant_args* args, void* stream);

typedef struct lsvd_mix_acc_quant_args {
  int32_t rows, cols;
  const int32_t* acc;            /* device int32 [rows, cols] accumulators                                        */
  int64_t acc_row_stride;
  const float* row_scale;        /* value = (fp32(acc) * row_scale[row]) * col_scale[col], quantised from fp32     */
  int64_t row_scale_stride;
  const float* col_scale;
  int8_t* q;
  int64_t q_row_stride;
  float* scale;                  /* device fp32 [rows]                                                            */
} lsvd_mix_acc_quant_args;
int lsvd_mix_acc_quant(const lsvd_mix_acc_quant_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LSVD_B200_H */
