"""The reference's ``mixffn`` W8A8 FFN pipeline on the CPU (test infrastructure; never imported by lsvd_b200/).

Restates ``MixedFFNGateUpDenseLatentFused.forward_stages`` (kernels/layer_bench/ffn_kernel/mix_ffn_kernel.py:2066-2102)
and the eleven Triton kernels behind it.  Conventions of that file, which differ from the fake_quant FFN:

  * every dequantisation is ``(fp32(acc) * row_scale) * column_scale`` in fp32, rounded to fp16 only where a tensor is
    stored as fp16;
  * activation scales are ``max(absmax / 127, 1e-8)`` with the absmax taken over the fp32 values *before* they are
    rounded to fp16 (:365-366, :1229-1232, :1894-1895), and codes are round-half-away-from-zero of ``v / scale``
    clamped to [-128, 127] (:163-165);
  * the first quantiser's scale is computed in fp32, used in fp32 for its own codes and then *stored as fp16* (:34,
    :149-150, :220-221), so later stages dequantise with the rounded value;
  * weight scales are ``max(absmax / 127, 1e-8)`` in the weight dtype, codes round-half-even (:200-210);
  * SwiGLU is ``up * (gate * sigmoid(gate))`` in fp32 (:362, :1889).

The RMSNorm statistic (a sum of 4096 squares) is evaluated exactly here (float64) and then rounded to fp32; the Triton
kernel adds in fp32 in block order, which can differ in the last bit.
"""
from __future__ import annotations

import torch

MAXQ = 127.0


def rounded_rank(in_features: int, out_features: int, rank_ratio: float, round_to: int = 64) -> int:
    """mix_ffn_kernel.py:536-543."""
    if rank_ratio <= 0.0:
        return 0
    rank = int(in_features * out_features * rank_ratio / (in_features + out_features))
    rank = max(1, min(rank, in_features, out_features))
    if round_to > 1 and rank >= round_to:
        rank = max(round_to, (rank // round_to) * round_to)
    return max(1, min(rank, in_features, out_features))


def svd_out_from_ratio(out_dim: int, svd_ratio: float, round_to: int = 64) -> int:
    """mix_ffn_kernel.py:889-897."""
    if svd_ratio <= 0.0:
        return 0
    if svd_ratio >= 1.0:
        return out_dim
    s = int(out_dim * svd_ratio)
    if round_to > 1:
        s = (s // round_to) * round_to
    return max(0, min(out_dim, s))


def quantize_weights_per_channel(w: torch.Tensor):
    """int8 codes and fp32 copies of the fp16 scales of ``w [out, in]`` (mix_ffn_kernel.py:200-210, :1500-1502).
    Evaluated in the weight's dtype like the reference (fp16 weights give fp16 quotients)."""
    scale = torch.maximum(w.abs().amax(dim=1) / MAXQ, torch.tensor(1e-8, dtype=w.dtype))
    q = torch.clamp(torch.round(w / scale.unsqueeze(-1)), -128, 127).to(torch.int8)
    return q.contiguous(), scale.to(torch.float16).to(torch.float32).contiguous()


def rha_codes(v32: torch.Tensor, scale32: torch.Tensor) -> torch.Tensor:
    """clamp(trunc(v/scale +- 0.5), -128, 127): the Triton kernels' rounding (:162-165)."""
    s = v32 / scale32
    r = torch.where(s >= 0, s + 0.5, s - 0.5).to(torch.int32)       # float -> int conversion truncates
    return r.clamp_(-128, 127).to(torch.int8)


def scale_from_absmax(absmax32: torch.Tensor) -> torch.Tensor:
    return torch.clamp(absmax32 / MAXQ, min=1e-8)


def rmsnorm_quantize_per_token(x16: torch.Tensor, w16: torch.Tensor, eps: float):
    """K4 (:101-165): returns int8 codes and the scale as stored (fp16)."""
    x = x16.float()
    sumsq = x.double().pow(2).sum(-1).float()
    inv = 1.0 / torch.sqrt(sumsq / x.shape[-1] + eps)
    normed = (x * inv[:, None]) * w16.float()[None, :]
    scale = torch.clamp(normed.abs().amax(-1) / MAXQ, min=1e-8)
    return rha_codes(normed, scale[:, None]), scale.to(torch.float16)


def i32_matmul(a_q: torch.Tensor, w_q: torch.Tensor) -> torch.Tensor:
    """``a_q [M, K] int8`` times ``w_q [N, K]^T`` with exact integer accumulation."""
    return (a_q.double() @ w_q.double().t()).to(torch.int64).to(torch.int32)


def dequant(acc: torch.Tensor, row_scale: torch.Tensor, col_scale: torch.Tensor) -> torch.Tensor:
    return (acc.float() * row_scale.float()[:, None]) * col_scale.float()[None, :]


def swiglu32(up: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    return up * (gate * torch.sigmoid(gate))


def forward_stages(x16: torch.Tensor, w: dict, eps: float = 1e-6, given: dict | None = None) -> dict:
    """``x16 [M, hidden]`` fp16.  ``w``: ``norm_weight`` fp16 and, for p in up/gate/down, ``{p}_a_q``, ``{p}_a_scale``,
    ``{p}_b_q``, ``{p}_b_scale`` (the low-rank branch of the first ``svd_out`` output columns) and ``{p}_q``,
    ``{p}_scale`` (the dense branch of the remaining ones).  Returns the stage tensors under the reference's names.
    ``given`` may supply ``svd_mid_fp``, ``svd_mid_scale``, ``dense_mid_fp``, ``dense_mid_scale`` (the outputs of the two
    SwiGLU stages, the only ones that depend on a transcendental function): the stages after them then start from those
    values, which lets a test check everything downstream of another implementation's SwiGLU bit for bit."""
    st = {}
    given = given or {}
    x_q, x_scale = rmsnorm_quantize_per_token(x16, w["norm_weight"], eps)
    st["x_q"], st["x_scale"] = x_q, x_scale
    # K5: both low-rank "A" products, dequantised; scales from the fp32 values (:1156-1232, :1689-1692)
    for p in ("up", "gate"):
        val = dequant(i32_matmul(x_q, w[p + "_a_q"]), x_scale, w[p + "_a_scale"])
        st[p + "_svd_rank_fp"] = val.half()
        st[p + "_svd_rank_scale"] = scale_from_absmax(val.abs().amax(-1))
        # K6 (:1070-1108): codes of the fp16 latent with that scale
        st[p + "_svd_rank_q"] = rha_codes(st[p + "_svd_rank_fp"].float(), st[p + "_svd_rank_scale"][:, None])
    # K7 (:1822-1895): "B" products of both latents, SwiGLU in fp32
    up = dequant(i32_matmul(st["up_svd_rank_q"], w["up_b_q"]), st["up_svd_rank_scale"], w["up_b_scale"])
    gate = dequant(i32_matmul(st["gate_svd_rank_q"], w["gate_b_q"]), st["gate_svd_rank_scale"], w["gate_b_scale"])
    sw = swiglu32(up, gate)
    st["svd_mid_fp"], st["svd_mid_scale"] = sw.half(), scale_from_absmax(sw.abs().amax(-1))
    st["svd_mid_fp32"] = sw
    # K8 + K9 (:967-1021, :324-375): dense gate/up, SwiGLU in fp32
    st["up_dense_out_acc"] = i32_matmul(x_q, w["up_q"])
    st["gate_dense_out_acc"] = i32_matmul(x_q, w["gate_q"])
    sw = swiglu32(dequant(st["up_dense_out_acc"], x_scale, w["up_scale"]),
                  dequant(st["gate_dense_out_acc"], x_scale, w["gate_scale"]))
    st["dense_mid_fp"], st["dense_mid_scale"] = sw.half(), scale_from_absmax(sw.abs().amax(-1))
    st["dense_mid_fp32"] = sw
    for k in ("svd_mid_fp", "svd_mid_scale", "dense_mid_fp", "dense_mid_scale"):
        if k in given:
            st[k] = given[k]
    # K10 (:1114-1150): one scale for both halves (:2075)
    st["mid_scale"] = torch.maximum(st["svd_mid_scale"], st["dense_mid_scale"])
    st["mid_q"] = torch.cat([rha_codes(st["svd_mid_fp"].float(), st["mid_scale"][:, None]),
                             rha_codes(st["dense_mid_fp"].float(), st["mid_scale"][:, None])], dim=1)
    # K11 + K12 (:676-711, :795-837): the down projection's latent, quantised from its fp32 value
    st["down_svd_rank_acc"] = i32_matmul(st["mid_q"], w["down_a_q"])
    val = dequant(st["down_svd_rank_acc"], st["mid_scale"], w["down_a_scale"])
    st["down_svd_rank_scale"] = scale_from_absmax(val.abs().amax(-1))
    st["down_svd_rank_q"] = rha_codes(val, st["down_svd_rank_scale"][:, None])
    # K13, K14 (:1238-1342): the two groups of output columns
    st["down_svd_out_fp"] = dequant(i32_matmul(st["down_svd_rank_q"], w["down_b_q"]), st["down_svd_rank_scale"],
                                    w["down_b_scale"]).half()
    st["down_dense_out_fp"] = dequant(i32_matmul(st["mid_q"], w["down_q"]), st["mid_scale"], w["down_scale"]).half()
    st["down_fp"] = torch.cat([st["down_svd_out_fp"], st["down_dense_out_fp"]], dim=1)
    st["out"] = (st["down_fp"].float() + x16.float()).half()                  # fp16 add (:2085)
    return st


def convert_swiglu(up_w, gate_w, down_w, norm_w, svd_ratio, rank_ratio, round_to, gen):
    """The weights ``forward_stages`` takes, built as ``from_float`` does (:1993-2000, :1541-1557): dense branch =
    per-channel RTN of the trailing output rows; low-rank branch = *random* factors of the reference's rank
    (:545-554: it does not decompose the weight), drawn here from ``gen``."""
    w = {"norm_weight": norm_w.half()}
    for name, wt in (("up", up_w), ("gate", gate_w), ("down", down_w)):
        out_f, in_f = wt.shape
        s = svd_out_from_ratio(out_f, svd_ratio, round_to)
        r = rounded_rank(in_f, s, rank_ratio, round_to)
        a = (torch.randn(r, in_f, generator=gen) / in_f ** 0.5).to(wt.dtype)
        b = (torch.randn(s, r, generator=gen) / r ** 0.5).to(wt.dtype)
        w[name + "_a_q"], w[name + "_a_scale"] = quantize_weights_per_channel(a)
        w[name + "_b_q"], w[name + "_b_scale"] = quantize_weights_per_channel(b)
        w[name + "_q"], w[name + "_scale"] = quantize_weights_per_channel(wt[s:].contiguous())
    return w
