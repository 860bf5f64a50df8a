"""Host side of the hybrid SVD/RTN FFN for decode batches.

Mirrors the reference's module interface for this path:

  * ``HybridFFN`` takes the place of ``HybridSVDQuantFFN``
    (fake_quant/utils/hybrid_ffn_utils.py:910-984): same forward contract
    (``x [..., d_in] -> [..., d_out]`` fp16), same channel order ``[SVD | RTN]`` of the
    down projection, the online Hadamard over d_ffn described by ``(had_K, K)``, and a
    ``forward_stages`` that exposes every intermediate the way the reference's kernel-side
    module does (kernels/layer_bench/ffn_kernel/mix_ffn_kernel.py:2066-2102).
  * ``quantize_weight_rtn`` is the per-output-channel RTN of ``WeightQuantizer``
    (fake_quant/utils/quant_utils.py:436-498), producing real int8 codes and fp32 scales.

The arithmetic of a forward pass runs in the CUDA kernels of ``liblsvd_b200.so``; weight
conversion is offline host code.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
from torch import nn

from . import _lib
from .attention import _require_cuda, _stream_ptr


@torch.no_grad()
def quantize_weight_rtn(w: torch.Tensor, mse: bool = False, norm: float = 2.4, grid: int = 100,
                        maxshrink: float = 0.8):
    """Symmetric int8 round-to-nearest per output channel: (codes int8 [out, in], scale fp32 [out]).

    scale = clamp(absmax, 1e-5) / 127 in fp32; with ``mse`` the reference's shrink search keeps, per
    channel, the factor p = 1 - i/grid (i < maxshrink * grid) that lowers sum |dequant - w| ** norm.
    """
    wf = w.flatten(1)
    zero = torch.zeros(wf.shape[0], device=w.device)
    amax = torch.maximum(torch.minimum(wf.min(1)[0], zero).abs(), torch.maximum(wf.max(1)[0], zero)).clamp(min=1e-5)
    scale = amax / 127
    if mse:
        best = torch.full([wf.shape[0]], float("inf"), device=w.device)
        for i in range(int(maxshrink * grid)):
            s1 = ((1 - i / grid) * amax) / 127
            err = (s1[:, None] * torch.round(wf / s1[:, None]).clamp(-128, 127) - wf).abs().pow(norm).sum(1)
            better = err < best
            best[better] = err[better]
            scale[better] = s1[better]
    q = torch.round(wf / scale[:, None]).clamp(-128, 127).to(torch.int8)
    return q.reshape(w.shape).contiguous(), scale.float().contiguous()


def _ptr(t):
    return t.data_ptr() if t is not None else None


def act_quant(x: torch.Tensor, sign: Optional[torch.Tensor] = None, fwht: bool = False, want_rotated: bool = False):
    """Per-token int8 quantisation of fp16 rows ``[rows, cols]`` (optionally after a Hadamard rotation).
    Returns (codes int8, scale fp32 [rows], rotated fp16 or None)."""
    _require_cuda(x)
    if x.dtype != torch.float16 or x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be a 2-D fp16 tensor with unit inner stride")
    rows, cols = x.shape
    q = torch.empty(rows, cols, dtype=torch.int8, device=x.device)
    scale = torch.empty(rows, dtype=torch.float32, device=x.device)
    rot = torch.empty(rows, cols, dtype=torch.float16, device=x.device) if want_rotated else None
    a = _lib.ActQuantArgs()
    a.rows, a.cols = rows, cols
    a.x, a.x_row_stride = x.data_ptr(), x.stride(0)
    a.sign = _ptr(sign)
    a.fwht = 1 if fwht else 0
    a.q, a.q_row_stride = q.data_ptr(), q.stride(0)
    a.scale = scale.data_ptr()
    a.x_rot = _ptr(rot)
    _lib.check(_lib.load().lsvd_act_quant(C.byref(a), _stream_ptr(x)))
    return q, scale, rot


def hadamard_quant(x: torch.Tensor, had_K: torch.Tensor, K: int, want_rotated: bool = False):
    """(H_K kron H_{cols/K}) rotation of fp16 rows followed by per-token int8 quantisation."""
    _require_cuda(x, had_K)
    if x.dtype != torch.float16 or had_K.dtype != torch.float16 or not had_K.is_contiguous():
        raise ValueError("x and had_K must be fp16 (had_K contiguous)")
    rows, cols = x.shape
    q = torch.empty(rows, cols, dtype=torch.int8, device=x.device)
    scale = torch.empty(rows, dtype=torch.float32, device=x.device)
    y = torch.empty(rows, cols, dtype=torch.float16, device=x.device) if want_rotated else None
    a = _lib.HadamardQuantArgs()
    a.rows, a.cols, a.K = rows, cols, K
    a.x, a.x_row_stride = x.data_ptr(), x.stride(0)
    a.had_K = had_K.data_ptr()
    a.q, a.q_row_stride = q.data_ptr(), q.stride(0)
    a.scale = scale.data_ptr()
    a.y = _ptr(y)
    _lib.check(_lib.load().lsvd_hadamard_quant(C.byref(a), _stream_ptr(x)))
    return q, scale, y


def w8a8_gemv(a_q, a_scale, w_q, w_scale, w2_q=None, w2_scale=None, a2_q=None, a2_scale=None, out=None, out_col=0,
              want_acc=False, want_out=True):
    """acc = a_q @ w_q^T (int32, exact) for 1..64 tokens, dequantised to fp16; with (w2, a2) a gate/up pair whose
    result is silu(gate) * up.  Returns (out fp16 [m, n] or the passed tensor, acc int32 or None, acc2 or None)."""
    _require_cuda(a_q, w_q)
    m, k = a_q.shape
    n = w_q.shape[0]
    dev = a_q.device
    dual = w2_q is not None
    if out is None and want_out:
        out = torch.empty(m, n, dtype=torch.float16, device=dev)
    acc = torch.empty(m, n, dtype=torch.int32, device=dev) if want_acc else None
    acc2 = torch.empty(m, n, dtype=torch.int32, device=dev) if (want_acc and dual) else None
    g = _lib.GemvArgs()
    g.m, g.n, g.k = m, n, k
    g.w, g.w_row_stride, g.w_scale = w_q.data_ptr(), w_q.stride(0), _ptr(w_scale)
    if dual:
        g.w2, g.w2_row_stride, g.w2_scale = w2_q.data_ptr(), w2_q.stride(0), _ptr(w2_scale)
    g.a, g.a_row_stride, g.a_scale = a_q.data_ptr(), a_q.stride(0), _ptr(a_scale)
    g.a_scale_stride = a_scale.stride(0) if a_scale is not None else 1
    if a2_q is not None:
        g.a2, g.a2_row_stride, g.a2_scale = a2_q.data_ptr(), a2_q.stride(0), _ptr(a2_scale)
        g.a2_scale_stride = a2_scale.stride(0) if a2_scale is not None else 1
    g.epilogue = 1 if dual else 0
    if out is not None:
        g.out, g.out_row_stride, g.out_col = out.data_ptr(), out.stride(0), out_col
    g.acc_out, g.acc2_out = _ptr(acc), _ptr(acc2)
    _lib.check(_lib.load().lsvd_w8a8_gemv(C.byref(g), _stream_ptr(a_q)))
    return out, acc, acc2


class HybridFFN(nn.Module):
    """Hybrid SVD/RTN gated FFN with real int8 weights and activations (decode batches of 1..64 tokens).

    Buffers (names follow the factorisation W ~ V U of the SVD channel group):
      had_sign [d_in] fp16 +-1 or None   input rotation x @ random_hadamard_matrix (QuaRot residual rotation)
      U_q [2r, d_in] int8, U_s [2r]      gate latent rows 0:r, up latent rows r:2r   (gate_svd / up_svd .BLinear)
      Vg_q, Vu_q [n_svd, r], Vg_s, Vu_s                                               (gate_svd / up_svd .ALinear)
      Wg_q, Wu_q [n_q, d_in], Wg_s, Wu_s                                              (gate_quant / up_quant)
      had_K [K, K] fp16 or None, K       online Hadamard over d_ffn before the down projection
      Wd_q [d_out, d_ffn], Wd_s          down projection, input columns ordered [SVD | RTN]
    """

    def __init__(self, weights: dict):
        super().__init__()
        self.K = int(weights.get("K", 1))
        self.online_had = bool(weights.get("online_had", True))
        for name in ("U_q", "U_s", "Vg_q", "Vg_s", "Vu_q", "Vu_s", "Wg_q", "Wg_s", "Wu_q", "Wu_s", "Wd_q", "Wd_s"):
            self.register_buffer(name, weights[name].contiguous())
        hs = weights.get("had_sign")
        self.register_buffer("had_sign", None if hs is None else hs.to(torch.float16).contiguous())
        hk = weights.get("had_K")
        self.register_buffer("had_K", None if hk is None else hk.to(torch.float16).contiguous())
        self.rank = self.U_q.shape[0] // 2
        self.n_svd = self.Vg_q.shape[0]
        self.n_q = self.Wg_q.shape[0]
        self.d_in = self.U_q.shape[1]
        self.d_ffn = self.n_svd + self.n_q
        self.d_out = self.Wd_q.shape[0]
        if self.n_svd % 16 or self.n_q % 16 or self.d_out % 16 or self.rank % 64 or self.d_in % 64 or self.d_ffn % 64:
            raise ValueError("channel groups must be multiples of 16 and reduction sizes multiples of 64")

    @classmethod
    def from_float(cls, U, Vg, Vu, Wg, Wu, Wd, had_sign=None, had_K=None, K=1, mse=False, online_had=True):
        """Quantise fp weights (RTN per output channel, like the reference's ``rtn_fwrd`` on these seven matrices)."""
        w = {"K": K, "had_K": had_K, "had_sign": had_sign, "online_had": online_had}
        for name, t in (("U", U), ("Vg", Vg), ("Vu", Vu), ("Wg", Wg), ("Wu", Wu), ("Wd", Wd)):
            w[name + "_q"], w[name + "_s"] = quantize_weight_rtn(t, mse)
        return cls(w)

    @torch.no_grad()
    def forward_stages(self, x: torch.Tensor, want_acc: bool = False) -> dict:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if x2.shape[0] > 64:
            raise ValueError("the decode FFN takes at most 64 tokens per call")
        st = {}
        r = self.rank
        x_q, x_s, x_rot = act_quant(x2, sign=self.had_sign, want_rotated=self.had_sign is not None)
        st.update(x_q=x_q, x_s=x_s, x_rot=x_rot if x_rot is not None else x2)
        lat16, lat_acc, _ = w8a8_gemv(x_q, x_s, self.U_q, self.U_s, want_acc=want_acc)
        st.update(lat16=lat16, lat_acc=lat_acc)
        # the two latents of a token are quantised separately: view them as 2 m rows of r columns
        z_q, z_s, _ = act_quant(lat16.view(-1, r))
        z_q = z_q.view(-1, 2 * r)
        z_s = z_s.view(-1, 2)
        st.update(latg_q=z_q[:, :r], latu_q=z_q[:, r:], latg_s=z_s[:, 0], latu_s=z_s[:, 1])
        h16 = torch.empty(x2.shape[0], self.d_ffn, dtype=torch.float16, device=x.device)
        _, g_svd_acc, u_svd_acc = w8a8_gemv(z_q[:, :r], z_s[:, 0], self.Vg_q, self.Vg_s, self.Vu_q, self.Vu_s,
                                            a2_q=z_q[:, r:], a2_scale=z_s[:, 1], out=h16, out_col=0, want_acc=want_acc)
        _, g_rtn_acc, u_rtn_acc = w8a8_gemv(x_q, x_s, self.Wg_q, self.Wg_s, self.Wu_q, self.Wu_s, out=h16,
                                            out_col=self.n_svd, want_acc=want_acc)
        st.update(h16=h16, g_svd_acc=g_svd_acc, u_svd_acc=u_svd_acc, g_rtn_acc=g_rtn_acc, u_rtn_acc=u_rtn_acc)
        if not self.online_had:
            h_q, h_s, h_rot = act_quant(h16)
            h_rot = h16
        elif self.K == 1:
            h_q, h_s, h_rot = act_quant(h16, fwht=True, want_rotated=True)
        else:
            h_q, h_s, h_rot = hadamard_quant(h16, self.had_K, self.K, want_rotated=True)
        st.update(h_q=h_q, h_s=h_s, h_rot=h_rot)
        out, out_acc, _ = w8a8_gemv(h_q, h_s, self.Wd_q, self.Wd_s, want_acc=want_acc)
        st.update(out_acc=out_acc, out=out.view(*shape[:-1], self.d_out))
        return st

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.forward_stages(x)["out"]
