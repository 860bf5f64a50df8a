"""The reference's ``mixffn`` W8A8 FFN on this library's kernels.

``MixedFFNGateUpDenseLatentFused`` stands where the class of that name does in
kernels/layer_bench/ffn_kernel/mix_ffn_kernel.py:1978-2123: RMSNorm + quantiser, for gate/up a low-rank branch on the
first ``svd_out`` output channels and a dense int8 branch on the rest, SwiGLU, one shared quantiser of the hidden
vector, and a down projection split the same way over its output channels, plus the residual.  Every intermediate
follows that file's all-fp32 conventions (see ``oracle/`` for the statement the tests check against), so the integer
stages agree with the reference's bit for bit.

A decode step (1..64 tokens) is ten launches where the reference has eleven plus two concatenations:

    lsvd_mix_rmsnorm_quant                       x -> x_q, x_scale          (also clears the row-maximum words)
    lsvd_w8a8_gemv   [up_a ; gate_a]             -> fp16 latents + their fp32 row maxima
    lsvd_mix_group_quant                         -> int8 latents, one scale each
    lsvd_w8a8_gemv   (gate_b, up_b) fp32 SwiGLU  -> hidden[:, :svd_out] + row maximum
    lsvd_w8a8_gemv   (gate, up dense) fp32 SwiGLU-> hidden[:, svd_out:] + row maximum
    lsvd_mix_group_quant  shared scale           -> mid_q, mid_scale
    lsvd_w8a8_gemv   down_a                      -> int32 latent accumulators
    lsvd_mix_acc_quant                           -> int8 latent, scale
    lsvd_w8a8_gemv   down_b   + residual         -> out[:, :svd_out_down]
    lsvd_w8a8_gemv   down dense + residual       -> out[:, svd_out_down:]

``b200_mixffn(x, module)`` is the provider in the reference's ``fn(x, module: SwiGLUFFN)`` convention
(mix_ffn_kernel.py:2223-2246), with the conversion cached per source module like ``get_mixed_gateup_v8_ffn``.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict

import torch
from torch import nn

from . import _lib
from .ffn import w8a8_gemv, _stream_ptr, _require_cuda

_PROJ = ("up", "gate", "down")
_KEYS = ("a_q", "a_scale", "b_q", "b_scale", "q", "scale")


def rounded_rank(in_features: int, out_features: int, rank_ratio: float, round_to: int = 64) -> int:
    """Rank of the low-rank branch: floor(in * out * ratio / (in + out)), rounded down to a multiple of ``round_to``
    once it reaches it (mix_ffn_kernel.py:536-543)."""
    if rank_ratio <= 0.0:
        return 0
    rank = max(1, min(int(in_features * out_features * rank_ratio / (in_features + out_features)), in_features, out_features))
    if round_to > 1 and rank >= round_to:
        rank = max(round_to, rank // round_to * round_to)
    return max(1, min(rank, in_features, out_features))


def svd_out_from_ratio(out_dim: int, svd_ratio: float, round_to: int = 64) -> int:
    """Output channels served by the low-rank branch (mix_ffn_kernel.py:889-897)."""
    if svd_ratio <= 0.0:
        return 0
    if svd_ratio >= 1.0:
        return out_dim
    s = int(out_dim * svd_ratio)
    return max(0, min(out_dim, s // round_to * round_to if round_to > 1 else s))


def quantize_weights_per_channel(w: torch.Tensor):
    """Per-output-channel int8 codes and scales ``max(absmax / 127, 1e-8)`` evaluated in the weight's dtype, the scale
    kept as the fp32 copy of its fp16 value (mix_ffn_kernel.py:200-210, 1500-1502).  Offline host/device torch code."""
    scale = torch.maximum(w.abs().amax(dim=1) / 127, torch.tensor(1e-8, device=w.device, dtype=w.dtype))
    q = torch.clamp(torch.round(w / scale.unsqueeze(-1)), -128, 127).to(torch.int8)
    return q.contiguous(), scale.to(torch.float16).to(torch.float32).contiguous()


def mix_rmsnorm_quant(x, norm_weight, eps, clear_words=None):
    """x [rows, cols] fp16 -> (codes int8, scale fp32 holding the fp16-rounded value)."""
    _require_cuda(x, norm_weight)
    rows, cols = x.shape
    q = torch.empty(rows, cols, dtype=torch.int8, device=x.device)
    scale = torch.empty(rows, dtype=torch.float32, device=x.device)
    a = _lib.MixRmsnormQuantArgs()
    a.rows, a.cols, a.x, a.x_row_stride = rows, cols, x.data_ptr(), x.stride(0)
    a.norm_weight, a.eps = norm_weight.data_ptr(), eps
    a.q, a.q_row_stride, a.scale = q.data_ptr(), q.stride(0), scale.data_ptr()
    if clear_words is not None:
        a.clear_words, a.clear_per_row = clear_words.data_ptr(), clear_words.shape[1]
    _lib.check(_lib.load().lsvd_mix_rmsnorm_quant(C.byref(a), _stream_ptr(x)))
    return q, scale


def mix_group_quant(x, absmax, split, shared):
    """x [rows, cols] fp16 with row maxima ``absmax [rows, >=2]`` (int32 view of float bits) -> (codes, scales)."""
    rows, cols = x.shape
    q = torch.empty(rows, cols, dtype=torch.int8, device=x.device)
    scale = torch.empty(rows, 1 if (shared or split == cols) else 2, dtype=torch.float32, device=x.device)
    a = _lib.MixGroupQuantArgs()
    a.rows, a.cols, a.split, a.shared = rows, cols, split, 1 if shared else 0
    a.x, a.x_row_stride, a.absmax, a.absmax_stride = x.data_ptr(), x.stride(0), absmax.data_ptr(), absmax.stride(0)
    a.q, a.q_row_stride, a.scale, a.scale_stride = q.data_ptr(), q.stride(0), scale.data_ptr(), scale.stride(0)
    _lib.check(_lib.load().lsvd_mix_group_quant(C.byref(a), _stream_ptr(x)))
    return q, scale


def mix_acc_quant(acc, row_scale, col_scale):
    """int32 accumulators -> codes of ``(acc * row_scale) * col_scale`` quantised from fp32, and their scales."""
    rows, cols = acc.shape
    q = torch.empty(rows, cols, dtype=torch.int8, device=acc.device)
    scale = torch.empty(rows, dtype=torch.float32, device=acc.device)
    a = _lib.MixAccQuantArgs()
    a.rows, a.cols, a.acc, a.acc_row_stride = rows, cols, acc.data_ptr(), acc.stride(0)
    a.row_scale, a.row_scale_stride, a.col_scale = row_scale.data_ptr(), row_scale.stride(0), col_scale.data_ptr()
    a.q, a.q_row_stride, a.scale = q.data_ptr(), q.stride(0), scale.data_ptr()
    _lib.check(_lib.load().lsvd_mix_acc_quant(C.byref(a), _stream_ptr(acc)))
    return q, scale


class MixedFFNGateUpDenseLatentFused(nn.Module):
    """Buffers, for p in up / gate / down: ``{p}_a_q [r, in]``, ``{p}_b_q [svd_out, r]`` int8 with fp32 ``{p}_a_scale``,
    ``{p}_b_scale`` (low-rank branch), ``{p}_q [out - svd_out, in]`` int8 with ``{p}_scale`` (dense branch);
    ``norm_weight [hidden]`` fp16."""

    def __init__(self, weights: Dict[str, torch.Tensor], eps: float = 1e-6):
        super().__init__()
        self.eps, self.bits = float(eps), 8
        self.register_buffer("norm_weight", weights["norm_weight"].to(torch.float16).contiguous())
        for p in _PROJ:
            for k in _KEYS:
                self.register_buffer(f"{p}_{k}", weights[f"{p}_{k}"].contiguous())
        self.hidden_size = self.up_a_q.shape[1]
        self.svd_out, self.rank = self.up_b_q.shape
        self.intermediate_size = self.svd_out + self.up_q.shape[0]
        self.down_svd_out, self.down_rank = self.down_b_q.shape
        if self.gate_a_q.shape != self.up_a_q.shape or self.gate_b_q.shape != self.up_b_q.shape:
            raise ValueError("up/gate svd branch layouts must match")
        for v in (self.hidden_size, self.intermediate_size, self.svd_out, self.rank, self.down_svd_out, self.down_rank):
            if v % 16:
                raise ValueError("every extent (hidden, intermediate, low-rank channels, ranks) must be a multiple of 16")
        # both "A" factors in one matrix: rows [0, r) give the up latent, [r, 2r) the gate latent
        self.register_buffer("ab_a_q", torch.cat([self.up_a_q, self.gate_a_q]).contiguous(), persistent=False)
        self.register_buffer("ab_a_scale", torch.cat([self.up_a_scale, self.gate_a_scale]).contiguous(), persistent=False)

    # ---- construction -------------------------------------------------------------------------------------------
    @classmethod
    def from_float(cls, module, svd_ratio: float, rank_ratio: float, round_to: int, seed: int = 0):
        """From a module with the reference's ``SwiGLUFFN`` layout (``norm.weight``, ``norm.variance_epsilon``,
        ``up_proj`` / ``gate_proj`` / ``down_proj`` Linear weights), as the reference's ``from_float`` (:1993-2000):
        the dense branch is the RTN of the trailing output rows; the low-rank branch gets *random* factors of the
        reference's rank, as there (:545-554 -- it is a kernel benchmark and does not decompose the weight)."""
        dev = module.up_proj.weight.device
        gen = torch.Generator(device=dev).manual_seed(seed)
        w = {"norm_weight": module.norm.weight.detach()}
        for p in _PROJ:
            wt = getattr(module, p + "_proj").weight.detach()
            out_f, in_f = wt.shape
            s = svd_out_from_ratio(out_f, svd_ratio, round_to)
            r = rounded_rank(in_f, s, rank_ratio, round_to)
            if s == 0 or s == out_f:
                raise ValueError("both branches are needed: 0 < svd_ratio < 1")
            a = (torch.randn(r, in_f, device=dev, generator=gen) / in_f ** 0.5).to(wt.dtype)
            b = (torch.randn(s, r, device=dev, generator=gen) / r ** 0.5).to(wt.dtype)
            w[p + "_a_q"], w[p + "_a_scale"] = quantize_weights_per_channel(a)
            w[p + "_b_q"], w[p + "_b_scale"] = quantize_weights_per_channel(b)
            w[p + "_q"], w[p + "_scale"] = quantize_weights_per_channel(wt[s:].contiguous())
        return cls(w, eps=module.norm.variance_epsilon)

    @classmethod
    def from_module(cls, mixed):
        """Take over the buffers of a converted reference module (``{up,gate,down}_proj.svd_branch.{a_q,b_q,a_scale,
        b_scale}``, ``.dense_branch.{q,scale}``, ``norm_weight``, ``eps``; mix_ffn_kernel.py:1489-1565)."""
        w = {"norm_weight": mixed.norm_weight.detach()}
        for p in _PROJ:
            proj = getattr(mixed, p + "_proj")
            if proj.svd_branch is None or proj.dense_branch is None:
                raise ValueError("both branches are needed")
            for k in ("a_q", "a_scale", "b_q", "b_scale"):
                w[f"{p}_{k}"] = getattr(proj.svd_branch, k).detach()
            w[p + "_q"], w[p + "_scale"] = proj.dense_branch.q.detach(), proj.dense_branch.scale.detach()
        return cls(w, eps=mixed.eps)

    # ---- the step -----------------------------------------------------------------------------------------------
    @torch.no_grad()
    def _run(self, x2, want: bool, out=None):
        m, hid = x2.shape
        if x2.dtype != torch.float16 or x2.stride(1) != 1 or hid != self.hidden_size:
            raise ValueError("x must be fp16 [..., hidden] with unit inner stride")
        if m > 64:
            # Any number of tokens, like the reference's kernels (mix_ffn_kernel.py:1157-1232 are tiled over M): every
            # quantity of this block is per token, so 64 tokens at a time through the decode kernels give the same values.
            # (The weights are streamed once per 64 tokens: correct, not the fast way to run a prefill; the fp32-SwiGLU /
            # row-maximum epilogues this structure needs are built into the weight-streaming product only.)
            if out is None:
                out = torch.empty(m, hid, dtype=torch.float16, device=x2.device)
            parts = []
            for r0 in range(0, m, 64):
                _, st_c = self._run(x2[r0:r0 + 64], want, out=out[r0:r0 + 64])
                parts.append(st_c)
            st_all = {}
            if want:
                for key in parts[0]:
                    vals = [pc[key] for pc in parts]
                    st_all[key] = None if vals[0] is None else torch.cat(vals, dim=0)
            return out, st_all
        dev, r, s, d = x2.device, self.rank, self.svd_out, self.intermediate_size
        st = {}
        amax = torch.empty(m, 4, dtype=torch.int32, device=dev)          # float bits: up latent, gate latent, low-rank mid, dense mid
        x_q, x_scale = mix_rmsnorm_quant(x2, self.norm_weight, self.eps, clear_words=amax)
        lat, _, _ = w8a8_gemv(x_q, x_scale, self.ab_a_q, self.ab_a_scale, row_absmax=amax, absmax_split=r, form=3, prefetch_weights=True)
        lat_q, lat_s = mix_group_quant(lat, amax, split=r, shared=False)
        mid = torch.empty(m, d, dtype=torch.float16, device=dev)
        w8a8_gemv(lat_q[:, r:], lat_s[:, 1], self.gate_b_q, self.gate_b_scale, self.up_b_q, self.up_b_scale,
                  a2_q=lat_q[:, :r], a2_scale=lat_s[:, 0], out=mid, out_col=0, fp32_swiglu=True, row_absmax=amax[:, 2:], form=3, prefetch_weights=True)
        _, gacc, uacc = w8a8_gemv(x_q, x_scale, self.gate_q, self.gate_scale, self.up_q, self.up_scale, out=mid, out_col=s,
                                  fp32_swiglu=True, row_absmax=amax[:, 3:], want_acc=want, form=3, prefetch_weights=True)
        mid_q, mid_s = mix_group_quant(mid, amax[:, 2:], split=s, shared=True)
        mid_s = mid_s.view(m)
        _, racc, _ = w8a8_gemv(mid_q, None, self.down_a_q, None, want_acc=True, want_out=False, form=3, prefetch_weights=True)
        r_q, r_s = mix_acc_quant(racc, mid_s, self.down_a_scale)
        if out is None:
            out = torch.empty(m, hid, dtype=torch.float16, device=dev)
        so = self.down_svd_out
        res = None if want else x2
        tgt = torch.empty_like(out) if want else out                       # stage dump: the projection before the residual
        w8a8_gemv(r_q, r_s, self.down_b_q, self.down_b_scale, out=tgt, out_col=0, residual=res, form=3, prefetch_weights=True)
        w8a8_gemv(mid_q, mid_s, self.down_q, self.down_scale, out=tgt, out_col=so, residual=None if want else x2[:, so:], form=3, prefetch_weights=True)
        if want:
            torch.add(tgt, x2, out=out)
            maxq = torch.full((m,), 127.0, dtype=torch.float32, device=dev)       # a tensor divisor: true division
            to_scale = lambda bits: (bits.contiguous().view(torch.float32) / maxq).clamp_min(1e-8)
            st.update({"x_q": x_q, "x_scale": x_scale.half(), "mid_fp": None, "mid_q": mid_q, "mid_scale": mid_s,
                       "down_fp": tgt, "svd_mid_fp": mid[:, :s], "dense_mid_fp": mid[:, s:],
                       "svd_mid_scale": to_scale(amax[:, 2]), "dense_mid_scale": to_scale(amax[:, 3]),
                       "up_svd_rank_fp": lat[:, :r], "gate_svd_rank_fp": lat[:, r:], "up_svd_rank_q": lat_q[:, :r],
                       "gate_svd_rank_q": lat_q[:, r:], "up_svd_rank_scale": lat_s[:, 0], "gate_svd_rank_scale": lat_s[:, 1],
                       "up_dense_out_acc": uacc, "gate_dense_out_acc": gacc, "down_svd_rank_acc": racc,
                       "down_svd_rank_q": r_q, "down_svd_rank_scale": r_s, "down_svd_out_fp": tgt[:, :so],
                       "down_dense_out_fp": tgt[:, so:]})
        return out, st

    def forward_stages(self, x: torch.Tensor) -> Dict[str, torch.Tensor]:
        """Every intermediate under the reference's names (mix_ffn_kernel.py:2087-2102)."""
        out, st = self._run(x.reshape(-1, x.shape[-1]), want=True)
        st["out"] = out.reshape_as(x)
        return st

    def forward(self, x: torch.Tensor, out=None) -> torch.Tensor:
        y, _ = self._run(x.reshape(-1, x.shape[-1]), want=False, out=None if out is None else out.view(-1, x.shape[-1]))
        return y.reshape_as(x)


_CACHE: Dict[tuple, MixedFFNGateUpDenseLatentFused] = {}


def get_b200_mixffn(module, svd_ratio=None, rank_ratio=None, round_to=None):
    """Converted module of a ``SwiGLUFFN``, cached by the module's identity, weight pointers and ratios
    (mix_ffn_kernel.py:2125-2143); defaults from the attributes ``make_ffn_inputs`` sets, else 0.5 / 0.5 / 64."""
    svd_ratio = float(svd_ratio if svd_ratio is not None else getattr(module, "svd_ratio", 0.5))
    rank_ratio = float(rank_ratio if rank_ratio is not None else getattr(module, "rank_ratio", 0.5))
    round_to = int(round_to if round_to is not None else getattr(module, "round_to", 64))
    key = (id(module), module.norm.weight.data_ptr(), module.up_proj.weight.data_ptr(), module.gate_proj.weight.data_ptr(),
           module.down_proj.weight.data_ptr(), svd_ratio, rank_ratio, round_to)
    hit = _CACHE.get(key)
    if hit is None:
        hit = _CACHE[key] = MixedFFNGateUpDenseLatentFused.from_float(module, svd_ratio, rank_ratio, round_to)
    return hit


def b200_mixffn(x: torch.Tensor, module) -> torch.Tensor:
    return get_b200_mixffn(module)(x)
