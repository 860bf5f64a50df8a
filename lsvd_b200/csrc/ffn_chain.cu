// The hybrid SVD/RTN FFN for a decode batch as ONE entry point: the seven launches of the block, with the RTN
// gate/up product on a second stream of the library beside the SVD branch.
//   x -> [rotate] quantise -> { U -> quantise latents -> V_gate, V_up (SwiGLU) }  ||  { W_gate, W_up (SwiGLU) }
//     -> Hadamard + quantise -> W_down (+ residual)
// Replaces HybridSVDQuantFFN.forward (fake_quant/utils/hybrid_ffn_utils.py:956-984) with real int8 weights and
// activations; each step is one of the library's own entry points, so the values are theirs.
#include <mutex>

#include "common.cuh"

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
  size_t x_q, x_s, lat16, z_q, z_s, h16, h_q, h_s, total;
};

static FfnWorkspace ffn_layout(int m, int d_in, int d_ffn, int rank) {
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
  w.total = off;
  return w;
}

}  // namespace lsvd

extern "C" size_t lsvd_ffn_decode_workspace_bytes(int32_t m, int32_t d_in, int32_t d_ffn, int32_t rank) {
  if (m <= 0 || d_in <= 0 || d_ffn <= 0 || rank <= 0) return 0;
  return lsvd::ffn_layout(m, d_in, d_ffn, rank).total;
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
  const FfnWorkspace wl = ffn_layout(a->m, a->d_in, a->d_ffn, a->rank);
  if (a->workspace == nullptr || a->workspace_bytes < wl.total || !aligned(a->workspace, 256)) return LSVD_ERR_WORKSPACE;
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
