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
import os
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


def act_quant(x: Optional[torch.Tensor], sign: Optional[torch.Tensor] = None, fwht: bool = False, want_rotated: bool = False,
              norm_weight: Optional[torch.Tensor] = None, norm_eps: float = 1e-5, x_f32: Optional[torch.Tensor] = None,
              add: Optional[torch.Tensor] = None, sum_out: Optional[torch.Tensor] = None, q: Optional[torch.Tensor] = None,
              scale: Optional[torch.Tensor] = None, rot: Optional[torch.Tensor] = None, fake: Optional[torch.Tensor] = None):
    """Per-token int8 quantisation of fp16 rows ``[rows, cols]`` (optionally after a Hadamard rotation or an RMSNorm).
    With ``x_f32`` (fp32, contiguous) the row is ``fp16(x_f32 + add)`` instead of ``x`` and ``sum_out`` receives it: the
    tensor-parallel output projection's reduced partial sums plus the residual.  ``q`` / ``scale`` / ``rot`` may be passed
    in (preallocated); ``fake`` (fp16 ``[rows, cols]``, contiguous) receives the fake-quantised rows ``fp16(scale * code)``.
    Returns (codes int8, scale fp32 [rows], rotated fp16 or None)."""
    src = x if x is not None else x_f32
    _require_cuda(src)
    if x is not None and (x.dtype != torch.float16 or x.dim() != 2 or x.stride(1) != 1):
        raise ValueError("x must be a 2-D fp16 tensor with unit inner stride")
    if x_f32 is not None and (x_f32.dtype != torch.float32 or not x_f32.is_contiguous() or
                              (add is not None and not add.is_contiguous()) or (sum_out is not None and not sum_out.is_contiguous())):
        raise ValueError("x_f32 must be contiguous fp32, add / sum_out contiguous fp16")
    rows, cols = src.shape
    if q is None:
        q = torch.empty(rows, cols, dtype=torch.int8, device=src.device)
    if scale is None:
        scale = torch.empty(rows, dtype=torch.float32, device=src.device)
    if rot is None and want_rotated:
        rot = torch.empty(rows, cols, dtype=torch.float16, device=src.device)
    a = _lib.ActQuantArgs()
    a.rows, a.cols = rows, cols
    if x is not None:
        a.x, a.x_row_stride = x.data_ptr(), x.stride(0)
    a.sign = _ptr(sign)
    a.fwht = 1 if fwht else 0
    a.q, a.q_row_stride = q.data_ptr(), q.stride(0)
    a.scale = scale.data_ptr()
    a.x_rot = _ptr(rot)
    a.norm_weight, a.norm_eps = _ptr(norm_weight), norm_eps
    a.x_f32, a.add, a.sum_out = _ptr(x_f32), _ptr(add), _ptr(sum_out)
    if fake is not None and (fake.dtype != torch.float16 or not fake.is_contiguous() or fake.shape != src.shape):
        raise ValueError("fake must be a contiguous fp16 tensor of the input's shape")
    a.fake = _ptr(fake)
    _lib.check(_lib.load().lsvd_act_quant(C.byref(a), _stream_ptr(src)))
    return q, scale, rot


def dequant_residual(acc: torch.Tensor, a_scale: torch.Tensor, w_scale: torch.Tensor, residual: Optional[torch.Tensor] = None,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``fp16(fp16((acc * a_scale[m]) * w_scale[n]) + residual)`` for int32 accumulators ``[m, n]`` (contiguous) that were
    summed over tensor-parallel ranks: the epilogue of ``w8a8_gemv`` applied after the all-reduce."""
    _require_cuda(acc)
    m, n = acc.shape
    if acc.dtype != torch.int32 or not acc.is_contiguous():
        raise ValueError("acc must be a contiguous int32 tensor")
    if out is None:
        out = torch.empty(m, n, dtype=torch.float16, device=acc.device)
    _lib.check(_lib.load().lsvd_dequant_residual(acc.data_ptr(), a_scale.data_ptr(), w_scale.data_ptr(), _ptr(residual),
                                                residual.stride(0) if residual is not None else 0, out.data_ptr(), out.stride(0),
                                                m, n, _stream_ptr(acc)))
    return out


def hadamard_pack(had_K: torch.Tensor) -> torch.Tensor:
    """One-time conversion of the K x K Hadamard factor into the layout ``hadamard_quant`` reads."""
    _require_cuda(had_K)
    had_K = had_K.to(torch.float16).contiguous()
    K = had_K.shape[0]
    lib = _lib.load()
    packed = torch.empty(int(lib.lsvd_hadamard_packed_bytes(K)), dtype=torch.uint8, device=had_K.device)
    _lib.check(lib.lsvd_hadamard_pack(had_K.data_ptr(), K, packed.data_ptr(), _stream_ptr(had_K)))
    return packed


def hadamard_quant(x: torch.Tensor, had_K_packed: torch.Tensor, K: int, want_rotated: bool = False, q=None, scale=None):
    """(H_K kron H_{cols/K}) rotation of fp16 rows followed by per-token int8 quantisation.
    ``had_K_packed`` comes from ``hadamard_pack(had_K)``."""
    _require_cuda(x, had_K_packed)
    if x.dtype != torch.float16 or had_K_packed.dtype != torch.uint8:
        raise ValueError("x must be fp16 and had_K_packed the buffer made by hadamard_pack")
    rows, cols = x.shape
    if q is None:
        q = torch.empty(rows, cols, dtype=torch.int8, device=x.device)
    if scale is None:
        scale = torch.empty(rows, dtype=torch.float32, device=x.device)
    y = torch.empty(rows, cols, dtype=torch.float16, device=x.device) if want_rotated else None
    a = _lib.HadamardQuantArgs()
    a.rows, a.cols, a.K = rows, cols, K
    a.x, a.x_row_stride = x.data_ptr(), x.stride(0)
    a.had_K_packed = had_K_packed.data_ptr()
    a.q, a.q_row_stride = q.data_ptr(), q.stride(0)
    a.scale = scale.data_ptr()
    a.y = _ptr(y)
    _lib.check(_lib.load().lsvd_hadamard_quant(C.byref(a), _stream_ptr(x)))
    return q, scale, y


def heads_hadamard_quant(x: torch.Tensor, heads: int, want_rotated: bool = False, had_K: Optional[torch.Tensor] = None):
    """Hadamard across heads (rows ``[rows, heads * head_dim]``) + per-token int8 quantisation: the online rotation in
    front of ``o_proj``.  ``heads`` a power of two, or any count up to 64 with its ``had_K [heads, heads]`` (+-1).
    Returns (codes, scale fp32 [rows], rotated fp16 or None)."""
    _require_cuda(x)
    if x.dtype != torch.float16 or x.dim() != 2 or x.stride(1) != 1 or x.shape[1] % heads:
        raise ValueError("x must be a 2-D fp16 tensor [rows, heads * head_dim] with unit inner stride")
    rows, cols = x.shape
    q = torch.empty(rows, cols, dtype=torch.int8, device=x.device)
    scale = torch.empty(rows, dtype=torch.float32, device=x.device)
    y = torch.empty(rows, cols, dtype=torch.float16, device=x.device) if want_rotated else None
    a = _lib.HeadsHadamardQuantArgs()
    a.rows, a.heads, a.head_dim = rows, heads, cols // heads
    a.x, a.x_row_stride, a.q, a.q_row_stride, a.scale, a.y = x.data_ptr(), x.stride(0), q.data_ptr(), q.stride(0), scale.data_ptr(), _ptr(y)
    if had_K is not None:
        had_K = had_K.to(device=x.device, dtype=torch.float16).contiguous()
        a.had_K = had_K.data_ptr()
    _lib.check(_lib.load().lsvd_heads_hadamard_quant(C.byref(a), _stream_ptr(x)))
    return q, scale, y


def w8a8_gemv(a_q, a_scale, w_q, w_scale, w2_q=None, w2_scale=None, a2_q=None, a2_scale=None, out=None, out_col=0,
              want_acc=False, want_out=True, residual=None, form=0, status_word=None, fp32_swiglu=False,
              row_absmax=None, absmax_split=0, prefetch_weights=False, out_f32=None, acc=None):
    """acc = a_q @ w_q^T (int32, exact) for 1..64 tokens, dequantised to fp16; with (w2, a2) a gate/up pair whose
    result is silu(gate) * up.  Returns (out fp16 [m, n] or the passed tensor, acc int32 or None, acc2 or None).
    ``form`` 0 is the register-fed kernel, 1 the persistent TMA-fed one (at most 16 tokens); ``status_word`` (int32
    device tensor) receives LSVD_ERR_TIMEOUT if a pipeline wait of form 1 gives up.  ``fp32_swiglu`` selects the
    all-fp32 gate/up epilogue ``up * (gate * sigmoid(gate))``; ``row_absmax`` (int32 view of the words, strided by
    token) collects max |fp32 value| per token, channels from ``absmax_split`` on in the token's second word."""
    _require_cuda(a_q, w_q)
    m, k = a_q.shape
    n = w_q.shape[0]
    dev = a_q.device
    dual = w2_q is not None
    if out is None and want_out:
        out = torch.empty(m, n, dtype=torch.float16, device=dev)
    if acc is None and want_acc:
        acc = torch.empty(m, n, dtype=torch.int32, device=dev)
    acc2 = torch.empty(m, n, dtype=torch.int32, device=dev) if (want_acc and dual) else None
    g = _lib.GemvArgs()
    g.out_f32 = _ptr(out_f32)          # fp32 [m, n], contiguous: the dequantised value before any fp16 rounding
    g.m, g.n, g.k = m, n, k
    g.w, g.w_row_stride, g.w_scale = w_q.data_ptr(), w_q.stride(0), _ptr(w_scale)
    if dual:
        g.w2, g.w2_row_stride, g.w2_scale = w2_q.data_ptr(), w2_q.stride(0), _ptr(w2_scale)
    g.a, g.a_row_stride, g.a_scale = a_q.data_ptr(), a_q.stride(0), _ptr(a_scale)
    g.a_scale_stride = a_scale.stride(0) if a_scale is not None else 1
    if a2_q is not None:
        g.a2, g.a2_row_stride, g.a2_scale = a2_q.data_ptr(), a2_q.stride(0), _ptr(a2_scale)
        g.a2_scale_stride = a2_scale.stride(0) if a2_scale is not None else 1
    g.epilogue = (2 if fp32_swiglu else 1) if dual else 0
    if row_absmax is not None:
        g.row_absmax, g.row_absmax_stride, g.absmax_split = row_absmax.data_ptr(), row_absmax.stride(0), absmax_split
    if out is not None:
        g.out, g.out_row_stride, g.out_col = out.data_ptr(), out.stride(0), out_col
    g.acc_out, g.acc2_out = _ptr(acc), _ptr(acc2)
    if residual is not None:
        g.residual, g.residual_row_stride = residual.data_ptr(), residual.stride(0)
    g.form, g.status_word = form, _ptr(status_word)
    g.prefetch_weights = 1 if prefetch_weights else 0
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
        self.register_buffer("had_K_packed", None if (hk is None or self.K == 1 or not hk.is_cuda)
                             else hadamard_pack(self.had_K))
        self._plans = {}
        self._chains = {}
        self.overlap_branches = True      # RTN gate/up on a second stream beside the SVD branch (chain of launches)
        # at most 16 tokens: the whole block as ONE persistent kernel (lsvd_ffn_decode with `fused`).  Off by default:
        # measured on B200 it is exact but slower than the chain (78 vs 56 us at the 7B shape: the device-wide barriers between its stages cost more than the launch gaps they replace)
        self.fused = os.environ.get("LSVD_FFN_FUSED", "0") == "1"
        self.rank = self.U_q.shape[0] // 2
        self.n_svd = self.Vg_q.shape[0]
        self.n_q = self.Wg_q.shape[0]
        self.d_in = self.U_q.shape[1]
        self.d_ffn = self.n_svd + self.n_q
        self.d_out = self.Wd_q.shape[0]
        if self.n_svd % 16 or self.n_q % 16 or self.d_out % 16 or self.rank % 16 or self.d_in % 16:
            raise ValueError("channel groups and reduction sizes must be multiples of 16")

    @classmethod
    def from_float(cls, U, Vg, Vu, Wg, Wu, Wd, had_sign=None, had_K=None, K=1, mse=False, online_had=True):
        """Quantise fp weights (RTN per output channel, like the reference's ``rtn_fwrd`` on these seven matrices)."""
        w = {"K": K, "had_K": had_K, "had_sign": had_sign, "online_had": online_had}
        for name, t in (("U", U), ("Vg", Vg), ("Vu", Vu), ("Wg", Wg), ("Wu", Wu), ("Wd", Wd)):
            w[name + "_q"], w[name + "_s"] = quantize_weight_rtn(t, mse)
        return cls(w)

    @classmethod
    def from_module(cls, mlp, mse: bool = False):
        """Build from a module laid out like the reference's ``HybridSVDQuantFFN``
        (fake_quant/utils/hybrid_ffn_utils.py:923-984): ``gate_svd`` / ``up_svd`` with ``BLinear`` (latent factor,
        possibly inside an ``ActQuantWrapper``: its Linear is then ``.module``) and ``ALinear``; ``gate_quant`` /
        ``up_quant`` / ``down_proj`` wrappers around Linears whose weights already follow the module's channel order
        ([SVD | RTN] input columns for ``down_proj``); ``had_K``, ``K``, ``online_had``.  The fp16
        weights of a module that went through ``rtn_fwrd`` are integer codes times a per-row scale with the largest
        code at +-127, so quantising them again reproduces the same codes and scales."""
        def weight(m):
            return getattr(m, "module", m).weight.data

        return cls.from_float(
            U=torch.cat([weight(mlp.gate_svd.BLinear), weight(mlp.up_svd.BLinear)]),
            Vg=weight(mlp.gate_svd.ALinear), Vu=weight(mlp.up_svd.ALinear),
            Wg=weight(mlp.gate_quant), Wu=weight(mlp.up_quant), Wd=weight(mlp.down_proj),
            had_K=getattr(mlp, "had_K", None), K=int(getattr(mlp, "K", 1)), mse=mse,
            online_had=bool(getattr(mlp, "online_had", getattr(mlp, "had_K", None) is not None)))

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
            if self.had_K_packed is None:
                self.had_K_packed = hadamard_pack(self.had_K)
            h_q, h_s, h_rot = hadamard_quant(h16, self.had_K_packed, self.K, want_rotated=True)
        st.update(h_q=h_q, h_s=h_s, h_rot=h_rot)
        out, out_acc, _ = w8a8_gemv(h_q, h_s, self.Wd_q, self.Wd_s, want_acc=want_acc)
        st.update(out_acc=out_acc, out=out.view(*shape[:-1], self.d_out))
        return st

    # ---- the decode path proper: preallocated buffers and argument blocks per batch size, seven launches ----
    def _plan(self, m: int, device):
        key = (m, str(device))
        plan = self._plans.get(key)
        if plan is not None:
            return plan
        r, dev = self.rank, device
        b = {
            "x_q": torch.empty(m, self.d_in, dtype=torch.int8, device=dev), "x_s": torch.empty(m, dtype=torch.float32, device=dev),
            "lat16": torch.empty(m, 2 * r, dtype=torch.float16, device=dev),
            "z_q": torch.empty(m, 2 * r, dtype=torch.int8, device=dev), "z_s": torch.empty(m, 2, dtype=torch.float32, device=dev),
            "h16": torch.empty(m, self.d_ffn, dtype=torch.float16, device=dev),
            "h_q": torch.empty(m, self.d_ffn, dtype=torch.int8, device=dev), "h_s": torch.empty(m, dtype=torch.float32, device=dev),
        }
        calls = []
        lib = _lib.load()

        def actq(x_ptr, x_stride, rows, cols, sign, fwht, q, scale):
            a = _lib.ActQuantArgs()
            a.rows, a.cols, a.x, a.x_row_stride = rows, cols, x_ptr, x_stride
            a.sign, a.fwht = _ptr(sign), 1 if fwht else 0
            a.q, a.q_row_stride, a.scale = q.data_ptr(), cols if q.dim() == 1 else q.stride(0), scale.data_ptr()
            return (lib.lsvd_act_quant, a)

        def gemv(a_q, a_stride, a_s, a_s_stride, k, w, ws, out, out_stride, out_col=0, w2=None, w2s=None,
                 a2=None, a2_s=None):
            g = _lib.GemvArgs()
            g.m, g.n, g.k = m, w.shape[0], k
            g.w, g.w_row_stride, g.w_scale = w.data_ptr(), w.stride(0), ws.data_ptr()
            if w2 is not None:
                g.w2, g.w2_row_stride, g.w2_scale, g.epilogue = w2.data_ptr(), w2.stride(0), w2s.data_ptr(), 1
            g.a, g.a_row_stride, g.a_scale, g.a_scale_stride = a_q, a_stride, a_s, a_s_stride
            if a2 is not None:
                g.a2, g.a2_row_stride, g.a2_scale, g.a2_scale_stride = a2, a_stride, a2_s, a_s_stride
            g.out, g.out_row_stride, g.out_col = out, out_stride, out_col
            return (lib.lsvd_w8a8_gemv, g)

        calls.append(actq(0, self.d_in, m, self.d_in, self.had_sign, False, b["x_q"], b["x_s"]))            # [0]: x set per call
        calls.append(gemv(b["x_q"].data_ptr(), self.d_in, b["x_s"].data_ptr(), 1, self.d_in, self.U_q, self.U_s,
                          b["lat16"].data_ptr(), 2 * r))
        calls.append(actq(b["lat16"].data_ptr(), r, 2 * m, r, None, False, b["z_q"].view(-1, r), b["z_s"].view(-1)))
        zq, zs = b["z_q"].data_ptr(), b["z_s"].data_ptr()
        calls.append(gemv(zq, 2 * r, zs, 2, r, self.Vg_q, self.Vg_s, b["h16"].data_ptr(), self.d_ffn, 0, self.Vu_q, self.Vu_s,
                          a2=zq + r, a2_s=zs + 4))
        calls.append(gemv(b["x_q"].data_ptr(), self.d_in, b["x_s"].data_ptr(), 1, self.d_in, self.Wg_q, self.Wg_s,
                          b["h16"].data_ptr(), self.d_ffn, self.n_svd, self.Wu_q, self.Wu_s))
        if self.online_had and self.K > 1:
            if self.had_K_packed is None:
                self.had_K_packed = hadamard_pack(self.had_K)
            h = _lib.HadamardQuantArgs()
            h.rows, h.cols, h.K = m, self.d_ffn, self.K
            h.x, h.x_row_stride, h.had_K_packed = b["h16"].data_ptr(), self.d_ffn, self.had_K_packed.data_ptr()
            h.q, h.q_row_stride, h.scale = b["h_q"].data_ptr(), self.d_ffn, b["h_s"].data_ptr()
            calls.append((lib.lsvd_hadamard_quant, h))
        else:
            calls.append(actq(b["h16"].data_ptr(), self.d_ffn, m, self.d_ffn, None, self.online_had, b["h_q"], b["h_s"]))
        calls.append(gemv(b["h_q"].data_ptr(), self.d_ffn, b["h_s"].data_ptr(), 1, self.d_ffn, self.Wd_q, self.Wd_s, 0, self.d_out))
        plan = (b, calls)
        self._plans[key] = plan
        return plan

    @torch.no_grad()
    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None,
                norm_eps: float = 1e-6, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x [..., d_in] fp16 -> [..., d_out] fp16.  Up to 64 tokens take the weight-streaming decode kernels, more
        take ``forward_prefill`` (same values).  In the decode form intermediate buffers are kept per batch size,
        so apart from the result (unless ``out`` is passed) a call allocates nothing and can be captured in a CUDA graph.
        ``norm_weight`` applies RMSNorm(x) * weight inside the first quantiser (for modules without an input rotation);
        ``residual [tokens, d_out]`` is added to the result in the down projection's epilogue."""
        _require_cuda(x)
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        m = x2.shape[0]
        if m < 1:
            raise ValueError("the FFN needs at least one token")
        if x2.dtype != torch.float16 or x2.stride(1) != 1 or shape[-1] != self.d_in:
            raise ValueError("x must be fp16 [..., d_in] with unit inner stride")
        if m > 64:
            y = self.forward_prefill(x2, out, norm_weight, norm_eps, residual)
            return y.view(*shape[:-1], self.d_out)
        if out is None:
            out = torch.empty(m, self.d_out, dtype=torch.float16, device=x.device)
        a, _ = self._chain(m, x.device)
        a.x, a.x_row_stride = x2.data_ptr(), x2.stride(0)
        a.norm_weight, a.norm_eps = _ptr(norm_weight), norm_eps
        a.out, a.out_row_stride = out.data_ptr(), out.stride(0)
        a.residual = _ptr(residual)
        a.residual_row_stride = residual.stride(0) if residual is not None else 0
        a.overlap = 1 if self.overlap_branches else 0
        a.fused = 1 if self.fused else 0
        _lib.check(_lib.load().lsvd_ffn_decode(C.byref(a), _stream_ptr(x)))
        return out.view(*shape[:-1], self.d_out)

    def _chain(self, m: int, device):
        """Argument block and workspace of ``lsvd_ffn_decode`` for m tokens (kept, so a call allocates nothing)."""
        key = (m, str(device))
        got = self._chains.get(key)
        if got is not None:
            return got
        lib = _lib.load()
        for t in (self.U_q, self.Vg_q, self.Vu_q, self.Wg_q, self.Wu_q, self.Wd_q):
            if not t.is_contiguous():
                raise ValueError("weights must be contiguous")
        a = _lib.FfnDecodeArgs()
        a.m, a.d_in, a.d_ffn, a.d_out, a.rank, a.n_svd = m, self.d_in, self.d_ffn, self.d_out, self.rank, self.n_svd
        a.K, a.online_had = self.K, 1 if self.online_had else 0
        a.had_sign = _ptr(self.had_sign)
        for name in ("U", "Vg", "Vu", "Wg", "Wu", "Wd"):
            setattr(a, name + "_q", getattr(self, name + "_q").data_ptr())
            setattr(a, name + "_s", getattr(self, name + "_s").data_ptr())
        if self.online_had and self.K > 1:
            if self.had_K_packed is None:
                self.had_K_packed = hadamard_pack(self.had_K)
            a.had_K_packed = self.had_K_packed.data_ptr()
        # zeroed once: the fused form keeps its barrier counters there from call to call
        ws = torch.zeros(int(lib.lsvd_ffn_decode_workspace_bytes(m, self.d_in, self.d_ffn, self.rank, self.d_out)),
                         dtype=torch.uint8, device=device)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        a.fused = 1 if self.fused else 0
        got = (a, ws)
        self._chains[key] = got
        return got

    @torch.no_grad()
    def forward_prefill(self, x2: torch.Tensor, out: Optional[torch.Tensor] = None, norm_weight=None, norm_eps: float = 1e-6,
                        residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The same block for prefill-sized batches ``x2 [m, d_in]``: the quantisers as in decode, every product on
        the tcgen05 GEMM (``i8gemm``); the SVD branch's gate and up products, which read different latents, are one
        launch with two activation tiles per stage.  Bit-identical to the decode form row by row."""
        m = x2.shape[0]
        r, dev = self.rank, x2.device
        x_q, x_s, _ = act_quant(x2, sign=self.had_sign, norm_weight=norm_weight, norm_eps=norm_eps)
        lat16, _ = i8gemm(x_q, x_s, self.U_q, self.U_s)
        z_q, z_s, _ = act_quant(lat16.view(2 * m, r))
        z_q, z_s = z_q.view(m, 2 * r), z_s.view(m, 2)
        h16 = torch.empty(m, self.d_ffn, dtype=torch.float16, device=dev)
        i8gemm(z_q[:, :r], z_s[:, 0], self.Vg_q, self.Vg_s, self.Vu_q, self.Vu_s, out=h16, out_col=0,
               a2_q=z_q[:, r:], a2_scale=z_s[:, 1])
        i8gemm(x_q, x_s, self.Wg_q, self.Wg_s, self.Wu_q, self.Wu_s, out=h16, out_col=self.n_svd)
        if self.online_had and self.K > 1:
            if self.had_K_packed is None:
                self.had_K_packed = hadamard_pack(self.had_K)
            h_q, h_s, _ = hadamard_quant(h16, self.had_K_packed, self.K)
        else:
            h_q, h_s, _ = act_quant(h16, fwht=self.online_had)
        if out is None:
            out = torch.empty(m, self.d_out, dtype=torch.float16, device=dev)
        i8gemm(h_q, h_s, self.Wd_q, self.Wd_s, out=out, residual=residual)
        return out


def i8gemm(a_q, a_scale, w_q, w_scale, w2_q=None, w2_scale=None, out=None, out_col=0, want_acc=False, want_out=True,
           status_word=None, gate=None, gate_col=0, residual=None, a2_q=None, a2_scale=None):
    """W8A8 product for any number of tokens on the tcgen05 tensor cores (prefill-sized batches): the same values
    as ``w8a8_gemv``.  ``gate`` (fp16, columns gate_col.. of it) turns a single product into the up half of a gate/up
    pair whose gate came from other activations; ``residual`` is added in fp16; ``a2_q`` / ``a2_scale`` give the up
    matrix of a pair its own activations.  Returns (out fp16 or None, acc int32 or None)."""
    _require_cuda(a_q, w_q)
    m, k = a_q.shape
    n = w_q.shape[0]
    dev = a_q.device
    if out is None and want_out:
        out = torch.empty(m, n, dtype=torch.float16, device=dev)
    acc = torch.empty(m, n, dtype=torch.int32, device=dev) if want_acc else None
    g = _lib.I8GemmArgs()
    g.m, g.n, g.k = m, n, k
    g.a, g.a_row_stride, g.a_scale, g.a_scale_stride = a_q.data_ptr(), a_q.stride(0), a_scale.data_ptr(), a_scale.stride(0)
    g.w, g.w_row_stride, g.w_scale = w_q.data_ptr(), w_q.stride(0), w_scale.data_ptr()
    if gate is not None:
        g.gate, g.gate_row_stride, g.gate_col = gate.data_ptr(), gate.stride(0), gate_col
    if residual is not None:
        g.residual, g.residual_row_stride = residual.data_ptr(), residual.stride(0)
    if w2_q is not None:
        g.w2, g.w2_row_stride, g.w2_scale = w2_q.data_ptr(), w2_q.stride(0), w2_scale.data_ptr()
    if a2_q is not None:
        g.a2, g.a2_row_stride = a2_q.data_ptr(), a2_q.stride(0)
        g.a2_scale, g.a2_scale_stride = a2_scale.data_ptr(), a2_scale.stride(0)
    if out is not None:
        g.out, g.out_row_stride, g.out_col = out.data_ptr(), out.stride(0), out_col
    g.acc_out = _ptr(acc)
    g.status_word = _ptr(status_word)
    _lib.check(_lib.load().lsvd_i8gemm_prefill(C.byref(g), _stream_ptr(a_q)))
    return out, acc
