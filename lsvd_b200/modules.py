"""Drop-in modules for the accuracy-side (fake_quant/) module tree of the reference.

The reference's quantisation flow addresses sub-modules by dotted name -- ``rtn_fwrd`` rewrites
``mlp.gate_svd.BLinear.weight`` etc. (fake_quant/utils/hybrid_ffn_utils.py:2870-2883), the quantiser set-up walks every
``ActQuantWrapper`` and configures ``.quantizer`` / ``.out_quantizer``
(fake_quant/main_llava_next_hybrid_ffn.py:380-420) -- so a replacement has to keep the attribute names.  This file has

  * ``ActQuantizer``     per-token activation quantiser (fake_quant/utils/quant_utils.py:122-221),
  * ``ActQuantWrapper``  a Linear with online rotation, input and output quantisers (``:225-340``),
  * ``SVDLinear``        low-rank Linear, in particular the ragged per-head form (fake_quant/utils/svd_utils.py:171-320,
                         1976-2040),
  * ``add_actquant``     the tree walk that wraps every ``nn.Linear`` (fake_quant/utils/quant_utils.py:550-577),

with the same constructor arguments, attributes and forward contracts.  Where the reference multiplies fake-quantised
fp16 tensors, these modules run the int8 kernels of ``liblsvd_b200.so`` on the real codes (exact int32 accumulation,
one dequantisation); a configuration the library has no kernel for raises ``ValueError`` when it is set or first used.
Plain fp16 Linears with 16-bit inputs stay ``torch.nn.functional.linear`` calls, as they are in the reference.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import List, Optional, Sequence

import torch
from torch import nn
import torch.nn.functional as F

from . import _lib
from .attention import _require_cuda, _stream_ptr
from .ffn import act_quant, hadamard_pack, hadamard_quant, heads_hadamard_quant, i8gemm, w8a8_gemv
from .formats import int8_from_fake_quant


def _ver(t: torch.Tensor) -> int:
    """Version counter of a tensor (0 for inference tensors, which have none): part of the keys of the cached conversions."""
    try:
        return t._version
    except RuntimeError:
        return 0


def _rows(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    return x2 if x2.stride(1) == 1 else x2.contiguous()


class ActQuantizer(nn.Module):
    """Per-token activation quantiser with the reference's interface: ``configure``, ``find_params``, ``forward`` (the
    fake-quantised tensor ``scale * code`` in the input dtype), ``quantize`` (codes and scales), ``free``.

    A kernel exists for the W8A8 setting of the reference's runs: 8 bits, symmetric, one scale per token, clip ratio 1;
    16 bits is the identity.  ``scale`` has shape ``[..., 1]`` (the reference repeats it to the input's shape)."""

    def __init__(self):
        super().__init__()
        self.register_buffer("maxq", torch.tensor(0))
        self.register_buffer("scale", torch.zeros(1))
        self.register_buffer("zero", torch.zeros(1))
        self.bits = 16
        self.groupsize = -1
        self.sym = False
        self.clip_ratio = 1.0
        self._cache = None

    def configure(self, bits, groupsize=-1, sym=False, clip_ratio=1.0):
        if not (0 < clip_ratio <= 1):
            raise AssertionError("Clip ratio should be in (0, 1]")
        if bits < 16 and not (bits == 8 and sym and groupsize <= 0 and clip_ratio == 1.0):
            raise ValueError("no kernel for this activation quantiser (bits=%s, groupsize=%s, sym=%s, clip_ratio=%s): "
                             "8-bit symmetric per-token with clip ratio 1 only" % (bits, groupsize, sym, clip_ratio))
        self.maxq = torch.tensor(2 ** (bits - 1) - 1 if sym else 2 ** bits - 1)
        self.bits, self.groupsize, self.sym, self.clip_ratio = bits, groupsize, sym, clip_ratio

    def free(self):
        self.zero = None
        self.scale = None
        self._cache = None

    def _run(self, x):
        key = (x.data_ptr(), _ver(x), tuple(x.shape))
        if self._cache is None or self._cache[0] != key:
            x2 = _rows(x)
            fake = torch.empty(x2.shape, dtype=torch.float16, device=x.device)
            q, s, _ = act_quant(x2, fake=fake)
            self._cache = (key, q.view(x.shape), s.view(*x.shape[:-1], 1), fake.view(x.shape))
        return self._cache

    def find_params(self, x):
        if self.bits == 16:
            return
        _, _, s, _ = self._run(x)
        self.scale = s
        self.zero = torch.zeros_like(s)

    def forward(self, x):
        if self.bits == 16:
            return x
        return self._run(x)[3].to(x.dtype)

    def quantize(self, x):
        """(codes int8 ``x.shape``, scale fp32 ``[..., 1]``)."""
        _, q, s, _ = self._run(x)
        return q, s


class ActQuantWrapper(nn.Module):
    """``y = out_quantizer(Linear(quantizer(rotate(x))))`` with the attributes of the reference's wrapper.

    Rotations (at most one, as in the reference's runs):
      online_full_had        (H_K kron H_{n/K}) / sqrt(n) over the input features (``had_K``, ``K`` from ``get_hadK``)
      online_partial_had     Hadamard across heads, ``had_dim`` = head size (the rotation in front of ``o_proj``)
      online_random_had      ``x @ had_K`` with ``had_K = diag(+-1) H / sqrt(n)`` (a QuaRot residual rotation applied
                             online); the signs are read off the matrix
    ``fp32_had`` is accepted where the result is the same (the kernels always butterfly in fp32 and round once): the
    power-of-two rotations.  ``fuse_bias`` / ``fuse_linear`` / ``online_full_hadnopow2`` have no kernel.

    When the wrapped Linear's weight is int8 fake-quantised per output row (after ``rtn_fwrd``) and the input quantiser is
    on, the product runs on the int8 codes; the codes are extracted once and again whenever the weight tensor changes."""

    def __init__(self, module: nn.Linear):
        super().__init__()
        assert isinstance(module, nn.Linear)
        self.module = module
        self.weight = module.weight
        self.in_features = module.in_features
        self.out_features = module.out_features
        self.bias = module.bias
        self.quantizer = ActQuantizer()
        self.out_quantizer = ActQuantizer()
        self.register_buffer("had_K", torch.tensor(0))
        self._buffers["had_K"] = None
        self.K = 1
        self.online_full_had = False
        self.online_full_hadnopow2 = False
        self.online_partial_had = False
        self.online_random_had = False
        self.had_dim = 0
        self.fp32_had = False
        self.fuse_bias = False
        self.fuse_linear = False
        self.bias_param = None
        self._w8 = None          # (key, codes, scales) or (key, None, None) when the weight is not int8-representable
        self._had = None         # (key, packed factor | sign vector)

    def extra_repr(self) -> str:
        s = "Input Quantizer Bits: %d" % self.quantizer.bits
        if self.quantizer.bits < 16:
            s += " (Symmetric Per-Token)" if self.quantizer.sym else " (Asymmetric Per-Token)"
        s += "\nOutput Quantizer Bits: %d" % self.out_quantizer.bits
        if self.out_quantizer.bits < 16:
            s += " (Symmetric Per-Token)" if self.out_quantizer.sym else " (Asymmetric Per-Token)"
        return s

    # ------------------------------------------------------------------ cached conversions
    def int8_weight(self):
        """(codes int8 [out, in], scales fp32 [out]) of the wrapped weight, or (None, None) if it is not an int8 code
        times a per-row scale."""
        w = self.module.weight
        key = (w.data_ptr(), _ver(w), tuple(w.shape))
        if self._w8 is None or self._w8[0] != key:
            try:
                q, s = int8_from_fake_quant(w.data)
            except ValueError:
                q = s = None
            self._w8 = (key, q, s)
        return self._w8[1], self._w8[2]

    def set_int8_weight(self, codes: torch.Tensor, scale: torch.Tensor):
        """Install codes and scales that are known from elsewhere (a checkpoint's quantisers); the fp16 weight of the
        wrapped Linear is set to their product so that both views agree."""
        w = self.module.weight
        w.data = (scale.float()[:, None].to(w.device) * codes.float().to(w.device)).to(w.dtype)
        self._w8 = ((w.data_ptr(), _ver(w), tuple(w.shape)), codes.to(w.device).contiguous(), scale.float().to(w.device).contiguous())

    def _rotation(self, dev):
        hk = self.had_K
        key = (None if hk is None else (hk.data_ptr(), _ver(hk)), self.K, str(dev))
        if self._had is None or self._had[0] != key:
            val = None
            if self.online_random_had:
                n = hk.shape[0]
                sign = torch.sign(hk[:, 0]).to(device=dev, dtype=torch.float16)      # column 0 of H is all ones
                if n <= 8192:
                    eye = torch.eye(n, dtype=torch.float16, device=dev)
                    _, _, rot = act_quant(eye, sign=sign, want_rotated=True)
                    if not torch.allclose(rot.float(), hk.to(dev).float(), atol=2e-3 / math.sqrt(n)):
                        raise ValueError("online_random_had: had_K is not diag(+-1) H / sqrt(n)")
                val = sign.contiguous()
            elif self.online_full_had and self.K > 1:
                val = hadamard_pack(hk.to(dev))
            self._had = (key, val)
        return self._had[1]

    # ------------------------------------------------------------------ forward
    def _rotate_quant(self, x2, need_q):
        """(codes, scale, rotated fp16 or None): the rotation and, if ``need_q``, the input quantiser in one launch."""
        dev = x2.device
        n = x2.shape[1]
        want_rot = not need_q
        if self.online_random_had:
            sign = self._rotation(dev)
            if sign.numel() != n:
                # had_K smaller than the row: the same rotation on every run of had_K.shape[0] features
                # (fake_quant/utils/quant_utils.py:275-281), then the quantiser over the whole row
                blk = sign.numel()
                _, _, rot = act_quant(x2.reshape(-1, blk), sign=sign, want_rotated=True)
                rot = rot.view(x2.shape)
                return (*act_quant(rot)[:2], rot) if need_q else (None, None, rot)
            return act_quant(x2, sign=sign, want_rotated=want_rot)
        if self.online_full_had:
            if self.K > 1:
                if self.fp32_had:
                    raise ValueError("fp32_had with a non-power-of-two Hadamard factor has no kernel")
                return hadamard_quant(x2, self._rotation(dev), self.K, want_rotated=want_rot)
            return act_quant(x2, fwht=True, want_rotated=want_rot)
        if self.online_partial_had:
            heads = n // self.had_dim
            if self.K == 1:
                return heads_hadamard_quant(x2, heads, want_rotated=want_rot)
            if self.fp32_had:
                raise ValueError("fp32_had with a non-power-of-two head count has no kernel")
            return heads_hadamard_quant(x2, heads, want_rotated=want_rot, had_K=self.had_K)
        q, s, _ = act_quant(x2) if need_q else (None, None, None)
        return q, s, None

    def forward(self, x):
        if self.fuse_linear or self.fuse_bias or self.online_full_hadnopow2:
            raise ValueError("fuse_linear / fuse_bias / online_full_hadnopow2 have no kernel in this library")
        _require_cuda(x)
        x_dtype = x.dtype
        if x_dtype != torch.float16:
            raise ValueError("fp16 activations expected")
        rotating = self.online_full_had or self.online_partial_had or self.online_random_had
        quant_in = self.quantizer.bits < 16
        lead = x.shape[:-1]
        x2 = _rows(x)
        m = x2.shape[0]
        wq, ws = self.int8_weight() if quant_in else (None, None)
        bias = self.module.bias
        if quant_in and wq is not None:
            q, s, _ = self._rotate_quant(x2, True)
            res = bias.to(torch.float16).view(1, -1).expand(m, -1) if bias is not None else None   # row stride 0
            if m <= 64:
                y, _, _ = w8a8_gemv(q, s, wq, ws, residual=res)
            else:
                y, _ = i8gemm(q, s, wq, ws, residual=res)
        else:
            if quant_in:
                # 8-bit activations into a weight that is not int8: fake-quantised values through the library GEMM
                q, s, rot = self._rotate_quant(x2, True)
                xin = torch.empty(x2.shape, dtype=torch.float16, device=x.device)
                act_quant_fake_from_codes(q, s, xin)
            elif rotating:
                xin = self._rotate_quant(x2, False)[2]
            else:
                xin = x2
            y = F.linear(xin.to(self.module.weight.dtype), self.module.weight, bias).to(x_dtype)
        if self.out_quantizer.bits < 16:
            self.out_quantizer.find_params(y)
            y = self.out_quantizer(y).to(x_dtype)
            self.out_quantizer.free()
        return y.view(*lead, -1)


def act_quant_fake_from_codes(q: torch.Tensor, s: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out = fp16(s[row] * q)`` for codes that an earlier launch produced (one elementwise pass)."""
    torch.mul(q, s[:, None], out=out)
    return out


class SVDLinear(nn.Module):
    """Low-rank Linear ``y = A (B x)`` with the reference's constructor and attribute names.

    Per-head form with a rank split (the one the latent attention uses): ``ALinear`` is a ``ParameterList`` of H factors
    ``[cout, r_h]``, ``BLinear`` a Linear ``C_in -> sum r_h`` (it may later be wrapped by ``ActQuantWrapper``: its output
    quantiser is then the latent quantiser), ``rank_split`` the list of r_h, ``head_num`` = H.  Forward: ``z = BLinear(x)``,
    then every head multiplies its own r_h latents -- one launch of the ragged kernel instead of the reference's padding
    to the largest rank plus einsum.  The uniform per-head form (``ALinear [H, cout, r]``) takes the same kernel; the plain
    form is two Linears.  ``is_ma_hack`` / ``topk`` (an accuracy experiment that re-runs the dense Linear) are not built."""

    def __init__(self, U, S, V, bias=None, sigma_fuse="UV", had_K=None, K=-1, had_mode="hadamard", is_ma_hack=False,
                 original_linear=None, topk=1, is_per_head_svd=False, rank_split=None) -> None:
        super().__init__()
        if is_ma_hack:
            raise ValueError("is_ma_hack is not built")
        self.rank_split = rank_split
        if sigma_fuse == "local_ft" and S is not None:
            raise ValueError("local_ft SVDLinear expects already fused A/B weights with S=None")
        if is_per_head_svd:
            if bias is not None:
                self.bias = nn.Parameter(bias.contiguous())
            else:
                self.register_parameter("bias", None)
            if rank_split is not None:
                self.head_num = len(V)
                self.ALinear = nn.ParameterList()
                rows = []
                for i in range(self.head_num):
                    if sigma_fuse == "UV":
                        a, b = U[i].mul(S[i].sqrt()), V[i].t().mul(S[i].sqrt().view(-1, 1))
                    elif sigma_fuse == "U":
                        a, b = U[i].mul(S[i]), V[i].t()
                    elif sigma_fuse == "V":
                        a, b = U[i], V[i].t().mul(S[i].view(-1, 1))
                    elif sigma_fuse == "local_ft":
                        a, b = U[i], V[i]
                        if b.shape[0] != a.shape[-1]:
                            raise ValueError("local_ft per-head V/BLinear must have shape (rank, hidden); got %s for rank %d"
                                             % (tuple(b.shape), a.shape[-1]))
                    else:
                        raise ValueError(f"Unsupported sigma_fuse in per head SVD: {sigma_fuse}")
                    self.ALinear.append(nn.Parameter(a.contiguous()))
                    rows.append(b.contiguous())
                Bw = torch.cat(rows, dim=0)                        # [sum r_h, C_in]
            else:
                # U [H, cout, r], S [H, r], V [H, C_in, r]  (local_ft: V [H, r, C_in])
                self.head_num = V.size(0)
                if sigma_fuse == "local_ft":
                    if V.size(1) != U.size(-1):
                        raise ValueError("local_ft per-head V/BLinear must have shape (heads, rank, hidden)")
                    self.head_rank = V.size(1)
                    a, Bw = U, V.reshape(-1, V.size(2))
                else:
                    self.head_rank = V.size(2)
                    if sigma_fuse == "UV":
                        a, b = U.mul(S.sqrt().unsqueeze(1)), V.mul(S.sqrt().unsqueeze(1))
                    elif sigma_fuse == "U":
                        a, b = U.mul(S.unsqueeze(1)), V
                    elif sigma_fuse == "V":
                        a, b = U, V.mul(S.unsqueeze(1))
                    else:
                        raise ValueError(f"Unsupported sigma_fuse in per head SVD: {sigma_fuse}")
                    Bw = b.transpose(1, 2).reshape(-1, V.size(1))
                self.ALinear = nn.Parameter(a.contiguous())
            self.BLinear = nn.Linear(Bw.size(1), Bw.size(0), bias=False)
            self.BLinear.weight.data = Bw.contiguous()
        else:
            self.ALinear = nn.Linear(U.size(1), U.size(0), bias=bias is not None)
            if bias is not None:
                self.ALinear.bias.data = bias
            if sigma_fuse == "UV":
                a, b = U.mul(S.sqrt()), V.t().mul(S.sqrt().view(-1, 1))
            elif sigma_fuse in ("U", "profile"):
                a, b = U.mul(S), V.t()
            elif sigma_fuse == "V":
                a, b = U, V.t().mul(S.view(-1, 1))
            elif sigma_fuse == "local_ft":
                a, b = U, V
            else:
                f = float(sigma_fuse)
                if not 0.0 <= f <= 1.0:
                    raise RuntimeError(f"Error: unsupported sigma mode {sigma_fuse}")
                a, b = U.mul(S ** (1 - f)), V.t().mul((S ** f).view(-1, 1))
            self.BLinear = nn.Linear(b.size(1), b.size(0), bias=False)
            self.ALinear.weight.data = a.contiguous()
            self.BLinear.weight.data = b.contiguous()
        self.had_K = had_K
        self.K = K
        self.had_mode = had_mode
        self.is_ma_hack = False
        self.original_linear = None
        self.topk = topk
        self.is_per_head_svd = is_per_head_svd
        self._packed = None

    # ------------------------------------------------------------------
    def _factors(self, dev):
        """(packed factors fp16, rank offsets int32 host array, cout) for the ragged kernel; rebuilt when a factor changes."""
        plist = list(self.ALinear) if self.rank_split is not None else [self.ALinear]
        key = tuple((p.data_ptr(), _ver(p)) for p in plist) + (str(dev),)
        if self._packed is None or self._packed[0] != key:
            if self.rank_split is not None:
                ranks = [int(r) for r in self.rank_split]
                got = [p.shape[1] for p in plist]
                if len(ranks) != self.head_num:
                    raise AssertionError(f"len(rank_split)={len(ranks)} != head_num={self.head_num}")
                if got != ranks:
                    raise ValueError(f"Per-head rank mismatch: weight {got} vs split {ranks}")
                cout = plist[0].shape[0]
                flat = torch.cat([p.data.to(device=dev, dtype=torch.float16).reshape(-1) for p in plist])
            else:
                ranks = [self.head_rank] * self.head_num
                cout = self.ALinear.shape[1]
                flat = self.ALinear.data.to(device=dev, dtype=torch.float16).reshape(-1)
            off = (C.c_int32 * (self.head_num + 1))()
            for h, r in enumerate(ranks):
                off[h + 1] = off[h] + r
            self._packed = (key, flat.contiguous(), off, cout)
        return self._packed[1:]

    def forward(self, inp):
        if not self.is_per_head_svd:
            return self.ALinear(self.BLinear(inp))
        z = self.BLinear(inp)
        _require_cuda(z)
        if z.dtype != torch.float16:
            raise ValueError("fp16 activations expected")
        flat, off, cout = self._factors(z.device)
        z2 = _rows(z)
        tokens = z2.shape[0]
        y = torch.empty(tokens, self.head_num * cout, dtype=torch.float16, device=z.device)
        bias = None if self.bias is None else self.bias.data.to(torch.float16).contiguous()
        _lib.check(_lib.load().lsvd_per_head_up(z2.data_ptr(), z2.stride(0), flat.data_ptr(), off,
                                               None if bias is None else bias.data_ptr(), y.data_ptr(), y.stride(0),
                                               tokens, self.head_num, cout, _stream_ptr(z)))
        if self.rank_split is None:
            # the reference's uniform form returns [1, tokens, H * cout] whatever the input's leading shape
            return y.unsqueeze(0)
        return y.view(*z.shape[:-1], self.head_num * cout)


def add_actquant(module: nn.Module, name: str = "", layers: Sequence[type] = (nn.Linear,)) -> None:
    """Wrap every ``nn.Linear`` below ``module`` (attributes, ``Sequential`` and ``ModuleList`` members) in an
    ``ActQuantWrapper``, in place, like the reference's walk (fake_quant/utils/quant_utils.py:550-577)."""
    if isinstance(module, ActQuantWrapper):
        return
    layers = tuple(layers)
    for attr, child in list(module.named_children()):
        if type(child) in layers:
            setattr(module, attr, ActQuantWrapper(child))
        elif type(child) is nn.Sequential:
            setattr(module, attr, nn.Sequential(*[ActQuantWrapper(c) if type(c) in layers else c for c in child.children()]))
        elif type(child) is nn.ModuleList:
            setattr(module, attr, nn.ModuleList([ActQuantWrapper(c) if type(c) in layers else c for c in child.children()]))
    for cname, child in module.named_children():
        add_actquant(child, name + "." + cname if name else cname, layers)


def find_qlayers(module: nn.Module, layers: Sequence[type] = (ActQuantWrapper,), name: str = "") -> dict:
    """{dotted name: module} of every sub-module whose type is in ``layers``
    (fake_quant/utils/quant_utils.py ``find_qlayers``)."""
    if type(module) in tuple(layers):
        return {name: module}
    res = {}
    for cname, child in module.named_children():
        res.update(find_qlayers(child, layers, name + "." + cname if name else cname))
    return res
