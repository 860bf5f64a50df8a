// The hybrid SVD/RTN FFN for a decode batch as ONE entry point: the seven launches of the block, with the RTN
// gate/up product on a second stream of the library beside the SVD branch.
//   x -> [rotate] quantise -> { U -> quantise latents -> V_gate, V_up (SwiGLU) }  ||  { W_gate, W_up (SwiGLU) }
//     -> Hadamard + quantise -> W_down (+ residual)
// Replaces HybridSVDQuantFFN.forward (fake_quant/utils/hybrid_ffn_utils.py:956-984) with real int8 weights and
// activations; each step is one of the library's own entry points, so the values are theirs.
#include <algorithm>
#include <cmath>
#include <mutex>

#include "common.cuh"
#include "fused.cuh"

namespace lsvd {

struct SideStream {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
};

constexpr int kMaxDev = 64;
static SideStream g_side[kMaxDev];
static std::mutex g_side_mu;

// The second stream and its two events, one set per device, made on first use and kept for the process.
static int side_stream(SideStream** out) {
  int dev = 0;
  LSVD_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDev) return LSVD_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_side_mu);
  SideStream& s = g_side[dev];
  if (s.stream == nullptr) {
    LSVD_CUDA_TRY(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking));
    LSVD_CUDA_TRY(cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming));
    LSVD_CUDA_TRY(cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming));
  }
  *out = &s;
  return LSVD_OK;
}

static size_t up256(size_t x) { return (x + 255) / 256 * 256; }

struct FfnWorkspace {
  size_t x_q, x_s, lat16, z_q, z_s, h16, h_q, h_s, sync, amax, acc, acc_end, total;
};

static FfnWorkspace ffn_layout(int m, int d_in, int d_ffn, int rank, int d_out) {
  FfnWorkspace w{};
  size_t off = 0;
  w.x_q = off; off = up256(off + static_cast<size_t>(m) * d_in);
  w.x_s = off; off = up256(off + static_cast<size_t>(m) * 4);
  w.lat16 = off; off = up256(off + static_cast<size_t>(m) * 2 * rank * 2);
  w.z_q = off; off = up256(off + static_cast<size_t>(m) * 2 * rank);
  w.z_s = off; off = up256(off + static_cast<size_t>(m) * 2 * 4);
  w.h16 = off; off = up256(off + static_cast<size_t>(m) * d_ffn * 2);
  w.h_q = off; off = up256(off + static_cast<size_t>(m) * d_ffn);
  w.h_s = off; off = up256(off + static_cast<size_t>(m) * 4);
  // the fused form: sync block; absmax words of the rotated hidden vector directly followed by the int32 accumulators
  // of the six products (U, gate, up, down), one range to clear per call
  w.sync = off; off = up256(off + kFSyncWords * 4);
  w.amax = off; off = up256(off + static_cast<size_t>(kFMaxTokens) * 4);
  w.acc = off;
  off = up256(off + static_cast<size_t>(kFMaxTokens) * (2 * static_cast<size_t>(rank) + 2 * static_cast<size_t>(d_ffn) + d_out) * 4);
  w.acc_end = off;
  w.total = off;
  return w;
}

}  // namespace lsvd

extern "C" size_t lsvd_ffn_decode_workspace_bytes(int32_t m, int32_t d_in, int32_t d_ffn, int32_t rank, int32_t d_out) {
  if (m <= 0 || d_in <= 0 || d_ffn <= 0 || rank <= 0 || d_out <= 0) return 0;
  return lsvd::ffn_layout(m, d_in, d_ffn, rank, d_out).total;
}


namespace lsvd {

// Fill the FFN part of a fused program: products first_op .. first_op + 5 (U, W_gate, W_up, V_gate, V_up, W_down), the
// buffers between them (all inside the FFN workspace) and the zero ranges.  The caller sets the stages, the input
// quantiser's source and the sync block.  LSVD_ERR_UNSUPPORTED when a shape falls outside the kernel's forms.
int ffn_fill_fused(const lsvd_ffn_decode_args* a, FusedParams& p, FMaps& maps, int first_op, int zero_slot) {
  const FfnWorkspace wl = ffn_layout(a->m, a->d_in, a->d_ffn, a->rank, a->d_out);
  const int m = a->m, r = a->rank, n_q = a->d_ffn - a->n_svd;
  if (m > kFMaxTokens) return LSVD_ERR_UNSUPPORTED;
  if ((a->d_in % 16) || (r % 16) || (a->d_ffn % 16) || (a->n_svd % 16) || (n_q % 16) || (a->d_out % 16)) return LSVD_ERR_UNSUPPORTED;
  if (r * 4 > kFScratch) return LSVD_ERR_UNSUPPORTED;
  if (a->had_sign != nullptr && a->norm_weight != nullptr) return LSVD_ERR_UNSUPPORTED;
  if (!aligned(a->x, 16) || (a->x_row_stride % 8) || !aligned(a->out, 2)) return LSVD_ERR_UNSUPPORTED;
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  p.status_word = a->status_word;
  p.m = m;
  p.rank = r; p.n_svd = a->n_svd; p.d_ffn = a->d_ffn; p.d_out = a->d_out;
  int8_t* x_q = reinterpret_cast<int8_t*>(ws + wl.x_q);
  float* x_s = reinterpret_cast<float*>(ws + wl.x_s);
  int8_t* z_q = reinterpret_cast<int8_t*>(ws + wl.z_q);
  float* z_s = reinterpret_cast<float*>(ws + wl.z_s);
  __half* h16 = reinterpret_cast<__half*>(ws + wl.h16);
  int8_t* h_q = reinterpret_cast<int8_t*>(ws + wl.h_q);
  float* h_s = reinterpret_cast<float*>(ws + wl.h_s);
  uint32_t* amax = reinterpret_cast<uint32_t*>(ws + wl.amax);
  int32_t* accU = reinterpret_cast<int32_t*>(ws + wl.acc);                       // [16][2 r]
  int32_t* accG = accU + static_cast<size_t>(kFMaxTokens) * 2 * r;               // [16][d_ffn] gate
  int32_t* accUp = accG + static_cast<size_t>(kFMaxTokens) * a->d_ffn;           // [16][d_ffn] up
  int32_t* accD = accUp + static_cast<size_t>(kFMaxTokens) * a->d_ffn;           // [16][d_out]
  p.zero_ptr[zero_slot] = reinterpret_cast<uint4*>(ws + wl.amax);                // the absmax words sit right in front of the accumulators
  p.zero_count[zero_slot] = static_cast<int32_t>((wl.acc_end - wl.amax) / 16);
  p.hq_amax = amax;

  // input quantiser
  ActQuantParams& q = p.q_in;
  q.x = static_cast<const __half*>(a->x); q.x_row_stride = a->x_row_stride;
  q.sign = static_cast<const __half*>(a->had_sign);
  q.norm_weight = static_cast<const __half*>(a->norm_weight); q.norm_eps = a->norm_eps;
  q.q = x_q; q.q_row_stride = a->d_in; q.scale = x_s; q.x_rot = nullptr;
  q.rows = m; q.cols = a->d_in; q.rotate = a->had_sign != nullptr ? 1 : 0;
  q.rot_scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(a->d_in)));
  q.vec8 = ((a->d_in % 8) == 0 && (a->had_sign == nullptr || aligned(a->had_sign, 16))) ? 1 : 0;
  if (q.rotate && (a->d_in & (a->d_in - 1)) != 0) return LSVD_ERR_UNSUPPORTED;
  if (!act_quant_rot4096_ok(q) && a->d_in * 4 > kFScratch) return LSVD_ERR_UNSUPPORTED;

  p.x_scale = x_s; p.U_s = a->U_s; p.Vg_s = a->Vg_s; p.Vu_s = a->Vu_s; p.Wg_s = a->Wg_s; p.Wu_s = a->Wu_s; p.Wd_s = a->Wd_s;
  p.z_q = z_q; p.z_s = z_s; p.h16 = h16; p.h_scale = h_s;
  p.out_residual = static_cast<const __half*>(a->residual); p.out_res_stride = a->residual_row_stride;
  p.out = static_cast<__half*>(a->out); p.out_stride = a->out_row_stride;

  struct Spec { const int8_t* w; int64_t ws; int n, k; const int8_t* act; int64_t as; int32_t* acc; int64_t accs; };
  const Spec spec[6] = {
      {a->U_q, a->d_in, 2 * r, a->d_in, x_q, a->d_in, accU, 2 * r},
      {a->Wg_q, a->d_in, n_q, a->d_in, x_q, a->d_in, accG + a->n_svd, a->d_ffn},
      {a->Wu_q, a->d_in, n_q, a->d_in, x_q, a->d_in, accUp + a->n_svd, a->d_ffn},
      {a->Vg_q, r, a->n_svd, r, z_q, 2 * r, accG, a->d_ffn},
      {a->Vu_q, r, a->n_svd, r, z_q + r, 2 * r, accUp, a->d_ffn},
      {a->Wd_q, a->d_ffn, a->d_out, a->d_ffn, h_q, a->d_ffn, accD, a->d_out},
  };
  if (first_op + 6 > kFMaxOps) return LSVD_ERR_UNSUPPORTED;
  if ((r % 128) != 0 || 2 * r > 2048) return LSVD_ERR_UNSUPPORTED;      // the up latents start at a K block of the latent panel
  for (int i = 0; i < 6; ++i) {
    FOp& o = p.op[first_op + i];
    o = FOp{};
    o.n = spec[i].n; o.k = spec[i].k; o.act_kind = 0; o.a = spec[i].act; o.a_stride = spec[i].as;
    o.acc = spec[i].acc; o.acc_stride = spec[i].accs;
    o.panel_full = 1; o.panel_k = spec[i].k;
    if (!fused_prepare_op(p, maps, first_op + i, spec[i].w, spec[i].ws)) return LSVD_ERR_UNSUPPORTED;
  }
  // V_gate / V_up read the two halves of one panel of latent codes [m, 2 r]
  p.op[first_op + 3].panel_k = 2 * r;
  p.op[first_op + 4].a = z_q; p.op[first_op + 4].panel_k = 2 * r; p.op[first_op + 4].a_kb0 = r / 128;
  // a down projection longer than the panel keeps only the block's own run of K blocks
  if (a->d_ffn > kFPanelUnits * 128) p.op[first_op + 5].panel_full = 0;
  p.nops = first_op + 6;
  if (!fused_check_group(p, first_op, 3) || !fused_check_group(p, first_op + 3, 2) || !fused_check_group(p, first_op + 5, 1))
    return LSVD_ERR_UNSUPPORTED;
  fused_prepare_panel(p, maps, first_op);
  fused_prepare_panel(p, maps, first_op + 3);
  fused_prepare_panel(p, maps, first_op + 5);

  // hidden-vector quantiser
  if (a->online_had && a->K > 1) {
    if (a->d_ffn % a->K || a->d_ffn / a->K != 64 || a->had_K_packed == nullptr) return LSVD_ERR_UNSUPPORTED;
    HadQuantParams& h = p.hq;
    h.x = h16; h.x_row_stride = a->d_ffn; h.packed = static_cast<const uint4*>(a->had_K_packed);
    h.q = h_q; h.q_row_stride = a->d_ffn; h.scale = h_s; h.y = nullptr;
    h.rows = m; h.cols = a->d_ffn; h.K = a->K; h.nb = 64; h.Kp = (a->K + 15) / 16 * 16; h.ld = h.Kp + 8;
    h.rot_scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(a->d_ffn)));
    if (h.Kp > 192 || device_sm_count() < m * 8) return LSVD_ERR_UNSUPPORTED;
    p.hq_kind = 1;
  } else {
    ActQuantParams& h = p.hq_plain;
    h = ActQuantParams{};
    h.x = h16; h.x_row_stride = a->d_ffn; h.q = h_q; h.q_row_stride = a->d_ffn; h.scale = h_s;
    h.rows = m; h.cols = a->d_ffn; h.rotate = a->online_had ? 1 : 0; h.vec8 = 1;
    h.rot_scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(a->d_ffn)));
    if (h.rotate && (a->d_ffn & (a->d_ffn - 1)) != 0) return LSVD_ERR_INVALID_ARG;
    if (a->d_ffn * 4 > kFScratch) return LSVD_ERR_UNSUPPORTED;
    p.hq_kind = 0;
  }
  return LSVD_OK;
}

// The hybrid FFN as one launch of the fused kernel; LSVD_ERR_UNSUPPORTED when a shape falls outside its forms
// (the caller then runs the chain of launches).
static int ffn_decode_fused(const lsvd_ffn_decode_args* a, const FfnWorkspace& wl, cudaStream_t st, bool dry_run) {
  FusedParams p{};
  FMaps maps{};
  p.sync = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(a->workspace) + wl.sync);
  p.stages = FST_QIN | FST_FFN;
  const int rc = ffn_fill_fused(a, p, maps, 0, 0);
  if (rc != LSVD_OK) return rc;
  if (dry_run) return LSVD_OK;
  return launch_fused(p, maps, nullptr, nullptr, st, false);
}

}  // namespace lsvd

extern "C" int lsvd_ffn_decode_is_fused(const lsvd_ffn_decode_args* a) {
  using namespace lsvd;
  if (a == nullptr || a->fused == 0 || !fused_enabled() || a->m <= 0 || a->workspace == nullptr) return 0;
  const FfnWorkspace wl = ffn_layout(a->m, a->d_in, a->d_ffn, a->rank, a->d_out);
  return ffn_decode_fused(a, wl, nullptr, true) == LSVD_OK ? 1 : 0;
}

#define LSVD_TRY(expr)            \
  do {                            \
    const int _rc = (expr);       \
    if (_rc != LSVD_OK) return _rc; \
  } while (0)

extern "C" int lsvd_ffn_decode(const lsvd_ffn_decode_args* a, void* stream) {
  using namespace lsvd;
  if (a == nullptr || a->m <= 0 || a->m > 64) return LSVD_ERR_INVALID_ARG;
  if (a->d_in <= 0 || a->d_ffn <= 0 || a->d_out <= 0 || a->rank <= 0 || a->n_svd <= 0 || a->n_svd >= a->d_ffn)
    return LSVD_ERR_INVALID_ARG;
  if (!a->x || !a->out || !a->U_q || !a->U_s || !a->Vg_q || !a->Vg_s || !a->Vu_q || !a->Vu_s || !a->Wg_q || !a->Wg_s ||
      !a->Wu_q || !a->Wu_s || !a->Wd_q || !a->Wd_s)
    return LSVD_ERR_INVALID_ARG;
  if (a->online_had && a->K > 1 && a->had_K_packed == nullptr) return LSVD_ERR_INVALID_ARG;
  const FfnWorkspace wl = ffn_layout(a->m, a->d_in, a->d_ffn, a->rank, a->d_out);
  if (a->workspace == nullptr || a->workspace_bytes < wl.total || !aligned(a->workspace, 256)) return LSVD_ERR_WORKSPACE;
  if (a->fused != 0 && fused_enabled()) {
    const int rc = ffn_decode_fused(a, wl, static_cast<cudaStream_t>(stream), false);
    if (rc != LSVD_ERR_UNSUPPORTED) return rc;
  }
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  int8_t* x_q = reinterpret_cast<int8_t*>(ws + wl.x_q);
  float* x_s = reinterpret_cast<float*>(ws + wl.x_s);
  void* lat16 = ws + wl.lat16;
  int8_t* z_q = reinterpret_cast<int8_t*>(ws + wl.z_q);
  float* z_s = reinterpret_cast<float*>(ws + wl.z_s);
  void* h16 = ws + wl.h16;
  int8_t* h_q = reinterpret_cast<int8_t*>(ws + wl.h_q);
  float* h_s = reinterpret_cast<float*>(ws + wl.h_s);
  const int m = a->m, r = a->rank, n_q = a->d_ffn - a->n_svd;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  // 1. input: [RMSNorm | sign-FWHT rotation] + per-token quantisation
  lsvd_act_quant_args q0{};
  q0.rows = m; q0.cols = a->d_in; q0.x = a->x; q0.x_row_stride = a->x_row_stride;
  q0.sign = a->had_sign; q0.fwht = 0; q0.q = x_q; q0.q_row_stride = a->d_in; q0.scale = x_s;
  q0.norm_weight = a->norm_weight; q0.norm_eps = a->norm_eps;
  LSVD_TRY(lsvd_act_quant(&q0, st));

  // 2. RTN gate/up pair: needs only x_q, runs beside the SVD branch
  lsvd_gemv_args gw{};
  gw.m = m; gw.n = n_q; gw.k = a->d_in;
  gw.w = a->Wg_q; gw.w_row_stride = a->d_in; gw.w_scale = a->Wg_s;
  gw.w2 = a->Wu_q; gw.w2_row_stride = a->d_in; gw.w2_scale = a->Wu_s;
  gw.a = x_q; gw.a_row_stride = a->d_in; gw.a_scale = x_s; gw.a_scale_stride = 1;
  gw.epilogue = 1; gw.out = h16; gw.out_row_stride = a->d_ffn; gw.out_col = a->n_svd;
  gw.status_word = a->status_word;
  SideStream* side = nullptr;
  if (a->overlap) {
    LSVD_TRY(side_stream(&side));
    LSVD_CUDA_TRY(cudaEventRecord(side->fork, st));
    LSVD_CUDA_TRY(cudaStreamWaitEvent(side->stream, side->fork, 0));
    LSVD_TRY(lsvd_w8a8_gemv(&gw, side->stream));
    LSVD_CUDA_TRY(cudaEventRecord(side->join, side->stream));
  }

  // 3. SVD branch: latents, their quantisation, gate/up from the latents
  lsvd_gemv_args gu{};
  gu.m = m; gu.n = 2 * r; gu.k = a->d_in;
  gu.w = a->U_q; gu.w_row_stride = a->d_in; gu.w_scale = a->U_s;
  gu.a = x_q; gu.a_row_stride = a->d_in; gu.a_scale = x_s; gu.a_scale_stride = 1;
  gu.out = lat16; gu.out_row_stride = 2 * r; gu.status_word = a->status_word;
  LSVD_TRY(lsvd_w8a8_gemv(&gu, st));
  lsvd_act_quant_args q1{};
  q1.rows = 2 * m; q1.cols = r; q1.x = lat16; q1.x_row_stride = r; q1.q = z_q; q1.q_row_stride = r; q1.scale = z_s;
  LSVD_TRY(lsvd_act_quant(&q1, st));
  lsvd_gemv_args gv{};
  gv.m = m; gv.n = a->n_svd; gv.k = r;
  gv.w = a->Vg_q; gv.w_row_stride = r; gv.w_scale = a->Vg_s;
  gv.w2 = a->Vu_q; gv.w2_row_stride = r; gv.w2_scale = a->Vu_s;
  gv.a = z_q; gv.a_row_stride = 2 * r; gv.a_scale = z_s; gv.a_scale_stride = 2;
  gv.a2 = z_q + r; gv.a2_row_stride = 2 * r; gv.a2_scale = z_s + 1; gv.a2_scale_stride = 2;
  gv.epilogue = 1; gv.out = h16; gv.out_row_stride = a->d_ffn; gv.out_col = 0; gv.status_word = a->status_word;
  LSVD_TRY(lsvd_w8a8_gemv(&gv, st));
  if (a->overlap) {
    LSVD_CUDA_TRY(cudaStreamWaitEvent(st, side->join, 0));
  } else {
    LSVD_TRY(lsvd_w8a8_gemv(&gw, st));
  }

  // 4. hidden vector: Hadamard (or plain) quantisation
  if (a->online_had && a->K > 1) {
    lsvd_hadamard_quant_args hq{};
    hq.rows = m; hq.cols = a->d_ffn; hq.K = a->K; hq.x = h16; hq.x_row_stride = a->d_ffn;
    hq.had_K_packed = a->had_K_packed; hq.q = h_q; hq.q_row_stride = a->d_ffn; hq.scale = h_s;
    LSVD_TRY(lsvd_hadamard_quant(&hq, st));
  } else {
    lsvd_act_quant_args q2{};
    q2.rows = m; q2.cols = a->d_ffn; q2.x = h16; q2.x_row_stride = a->d_ffn; q2.fwht = a->online_had ? 1 : 0;
    q2.q = h_q; q2.q_row_stride = a->d_ffn; q2.scale = h_s;
    LSVD_TRY(lsvd_act_quant(&q2, st));
  }

  // 5. down projection (+ residual)
  lsvd_gemv_args gd{};
  gd.m = m; gd.n = a->d_out; gd.k = a->d_ffn;
  gd.w = a->Wd_q; gd.w_row_stride = a->d_ffn; gd.w_scale = a->Wd_s;
  gd.a = h_q; gd.a_row_stride = a->d_ffn; gd.a_scale = h_s; gd.a_scale_stride = 1;
  gd.out = a->out; gd.out_row_stride = a->out_row_stride;
  gd.residual = a->residual; gd.residual_row_stride = a->residual_row_stride; gd.status_word = a->status_word;
  LSVD_TRY(lsvd_w8a8_gemv(&gd, st));
  return LSVD_OK;
}
