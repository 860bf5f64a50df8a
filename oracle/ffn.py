"""Hybrid SVD/RTN FFN in integer form on the CPU (test infrastructure).

The reference's ``HybridSVDQuantFFN`` (fake_quant/utils/hybrid_ffn_utils.py:910-984)
keeps integer-valued numbers in fp16 tensors ("fake" quantisation).  This file
computes the same network with real int8 codes and int32 accumulators and states
where each fp16 rounding of the reference happens, so that every stage is a
well-defined bit pattern the CUDA kernels can be compared with.

Weight container (plain dict of CPU tensors)
    had_sign  [d_in]  +-1 float or None   input random-Hadamard signs
    U_q [2r, d_in] int8, U_s [2r] fp32    rows 0:r gate latent, r:2r up latent  (BLinear of gate_svd / up_svd)
    Vg_q, Vu_q [n_svd, r] int8, Vg_s, Vu_s [n_svd] fp32                          (ALinear of gate_svd / up_svd)
    Wg_q, Wu_q [n_q, d_in] int8, Wg_s, Wu_s [n_q] fp32                           (gate_quant / up_quant)
    had_K [K, K] +-1 or None, K int       non-power-of-two Hadamard factor of d_ffn
    Wd_q [d_out, d_ffn] int8, Wd_s [d_out] fp32                                  (down_proj, columns [SVD | RTN])
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import quant


def fwht(x: torch.Tensor) -> torch.Tensor:
    """Unnormalised Sylvester Walsh-Hadamard transform over the last axis (power of two), in x's dtype.

    Same matrix as the reference's butterflies (fake_quant/utils/hadamard_utils.py:72-93,
    fake_quant/utils/hybrid_ffn_utils.py:483-498) and as the external
    ``fast_hadamard_transform`` extension (pinned at e7706faf, not vendored) that
    the reference calls on the GPU.
    """
    n = x.shape[-1]
    assert n & (n - 1) == 0
    y = x.reshape(-1, n).clone()
    h = 1
    while h < n:
        y = y.view(-1, n // (2 * h), 2, h)
        y = torch.stack((y[:, :, 0] + y[:, :, 1], y[:, :, 0] - y[:, :, 1]), dim=2).reshape(-1, n)
        h *= 2
    return y.reshape(x.shape)


def partial_hadamard_heads_hadk(x16: torch.Tensor, head_dim: int, had_K: torch.Tensor) -> torch.Tensor:
    """Hadamard across heads for a head count H that is not a power of two (H = K, e.g. 28):
    ``(had_K @ x.reshape(-1, H, head_dim)) / sqrt(H)`` as fp16 tensor operations, i.e. an fp16 matmul (fp32
    accumulation, one rounding) followed by the division of an fp16 tensor by a Python scalar (evaluated in fp32,
    rounded to fp16) (fake_quant/utils/quant_utils.py:312-313)."""
    n = x16.shape[-1]
    H = n // head_dim
    x = x16.reshape(-1, H, head_dim)
    y = (had_K.float() @ x.float()).to(x16.dtype)
    y = (y.float() / torch.tensor(math.sqrt(H), dtype=torch.float32)).to(x16.dtype)
    return y.reshape(x16.shape)


def partial_hadamard_heads(x16: torch.Tensor, head_dim: int) -> torch.Tensor:
    """Hadamard across heads: rows ``[..., H * head_dim]`` seen as ``[H, head_dim]``, each of the head_dim columns
    transformed over its H entries (H a power of two), scale 1/sqrt(H), fp32 inside and fp16 out.

    fake_quant/utils/quant_utils.py:302-317 with K == 1 (the ``fast_hadamard_transform`` call on the transposed
    view): the online rotation in front of ``o_proj``.
    """
    n = x16.shape[-1]
    H = n // head_dim
    x = x16.float().reshape(-1, H, head_dim).transpose(1, 2)          # [.., head_dim, H]
    y = (fwht(x.contiguous()) * (1.0 / math.sqrt(H))).to(x16.dtype)
    return y.transpose(1, 2).reshape(x16.shape)


def partial_hadamard_heads_terms(x_local16: torch.Tensor, head_ids, num_heads: int, had_K=None) -> torch.Tensor:
    """One tensor-parallel rank's terms of the Hadamard across heads (lsvd_b200.parallel.tp_heads_hadamard_quant): the rank
    holds heads ``head_ids`` of the ``num_heads``; returns fp32 ``[rows, num_heads * head_dim]`` with
    ``out[h', d] = sum_j S[h', head_ids[j]] x[j, d] / sqrt(num_heads)``.  The sum of all ranks' terms, rounded to fp16, is
    ``partial_hadamard_heads`` of the whole row (the transform is linear; Sylvester signs are (-1)^popcount(h' & h))."""
    n_local = len(head_ids)
    rows, cols = x_local16.shape
    hd = cols // n_local
    if had_K is None:
        hp = torch.arange(num_heads)
        S = torch.tensor([[(-1.0) ** bin(int(a) & int(b)).count("1") for b in head_ids] for a in hp])
    else:
        S = had_K.float()[:, list(head_ids)]
    x = x_local16.float().reshape(rows, n_local, hd)
    return (torch.einsum("oj,rjd->rod", S, x) * (1.0 / math.sqrt(num_heads))).reshape(rows, num_heads * hd)


def hadamard_full(x16: torch.Tensor, had_K, K: int) -> torch.Tensor:
    """(H_K kron H_{n/K}) x / sqrt(n) on the last axis, with the reference's two fp16 roundings.

    fake_quant/utils/hadamard_utils.py:106-113: view (.., K, n/K); transform the
    n/K axis with scale 1/sqrt(n) (fp32 inside, fp16 out); then had_K @ (.) as an
    fp16 matmul (fp32 accumulation, fp16 out).
    """
    n = x16.shape[-1]
    if K == 1:
        return (fwht(x16.float()) * (1.0 / math.sqrt(n))).to(torch.float16)
    t = x16.reshape(-1, K, n // K).float()
    t = (fwht(t) * (1.0 / math.sqrt(n))).to(torch.float16)
    y = had_K.float() @ t.float()
    return y.to(torch.float16).reshape(x16.shape)


def input_rotation(x16: torch.Tensor, had_sign) -> torch.Tensor:
    """x @ Q for Q = random_hadamard_matrix(n) (fake_quant/utils/hadamard_utils.py:99-104).

    Q[i, :] = sign[i] * H[i, :] / sqrt(n), hence x @ Q = FWHT(x * sign) / sqrt(n); fp32 inside, fp16 out.
    """
    n = x16.shape[-1]
    return (fwht(x16.float() * had_sign.float()) * (1.0 / math.sqrt(n))).to(torch.float16)


def _i32_matmul(a_q: torch.Tensor, w_q: torch.Tensor) -> torch.Tensor:
    """Exact int8 x int8 -> int32 product a_q [M, K] @ w_q [N, K]^T.

    float64 holds every partial sum exactly (|sum| <= K * 2**14 < 2**53).
    """
    return (a_q.double() @ w_q.double().t()).to(torch.int32)


def _dequant16(acc: torch.Tensor, s_row: torch.Tensor, s_col: torch.Tensor) -> torch.Tensor:
    """fp16((fp32(acc) * s_row[m]) * s_col[n]) -- the Linear output the reference rounds to fp16."""
    return ((acc.float() * s_row.float()[:, None]) * s_col.float()[None, :]).to(torch.float16)


def silu_mul16(g16: torch.Tensor, u16: torch.Tensor) -> torch.Tensor:
    """F.silu(g) * u on fp16 tensors as PyTorch evaluates it: silu in fp32 rounded to fp16, then an fp16 product."""
    s = F.silu(g16.float()).to(torch.float16)
    return (s.float() * u16.float()).to(torch.float16)


def hybrid_ffn_stages(x16: torch.Tensor, w: dict) -> dict:
    """All stages of the hybrid FFN for ``x16 [M, d_in]`` fp16.  Returns a dict of tensors.

    Stage list (reference line numbers are for fake_quant/utils/hybrid_ffn_utils.py
    unless stated):
      x_rot            optional input rotation
      x_q, x_s         A8 per-token quantisation of the FFN input; the reference
                       quantises the same x once per wrapped Linear (four times)
                       with identical results (quant_utils.py:319-322)
      lat_acc          int32 [M, 2r]  x_q . U_q^T                         (:962-963, BLinear)
      lat16            fp16  BLinear output
      latg_q/latu_q    A8 codes of each latent (BLinear.out_quantizer, quant_utils.py:335-338)
      g_svd_acc, u_svd_acc  int32 [M, n_svd]  latent . V^T               (ALinear)
      g_rtn_acc, u_rtn_acc  int32 [M, n_q]    x_q . W^T                  (:967-968)
      h16              fp16 [M, d_ffn] = cat(silu(g)*u)                   (:964-972)
      h_rot            fp16  online Hadamard                              (:976-981)
      h_q, h_s         A8 per-token                                       (down_proj wrapper)
      out_acc          int32 [M, d_out]
      out              fp16                                               (:984)
    """
    st = {}
    x = x16
    if w.get("had_sign") is not None:
        x = input_rotation(x16, w["had_sign"])
    st["x_rot"] = x
    x_q, x_s = quant.act_quant(x)
    st["x_q"], st["x_s"] = x_q, x_s

    r = w["U_q"].shape[0] // 2
    lat_acc = _i32_matmul(x_q, w["U_q"])
    lat16 = _dequant16(lat_acc, x_s, w["U_s"])
    st["lat_acc"], st["lat16"] = lat_acc, lat16
    latg_q, latg_s = quant.act_quant(lat16[:, :r])
    latu_q, latu_s = quant.act_quant(lat16[:, r:])
    st.update(latg_q=latg_q, latg_s=latg_s, latu_q=latu_q, latu_s=latu_s)

    g_svd_acc = _i32_matmul(latg_q, w["Vg_q"])
    u_svd_acc = _i32_matmul(latu_q, w["Vu_q"])
    g_rtn_acc = _i32_matmul(x_q, w["Wg_q"])
    u_rtn_acc = _i32_matmul(x_q, w["Wu_q"])
    st.update(g_svd_acc=g_svd_acc, u_svd_acc=u_svd_acc, g_rtn_acc=g_rtn_acc, u_rtn_acc=u_rtn_acc)
    g16 = torch.cat((_dequant16(g_svd_acc, latg_s, w["Vg_s"]), _dequant16(g_rtn_acc, x_s, w["Wg_s"])), dim=1)
    u16 = torch.cat((_dequant16(u_svd_acc, latu_s, w["Vu_s"]), _dequant16(u_rtn_acc, x_s, w["Wu_s"])), dim=1)
    st["g16"], st["u16"] = g16, u16
    h16 = silu_mul16(g16, u16)
    st["h16"] = h16

    if w.get("online_had", True):
        h_rot = hadamard_full(h16, w.get("had_K"), w["K"])
    else:
        h_rot = h16
    st["h_rot"] = h_rot
    h_q, h_s = quant.act_quant(h_rot)
    st["h_q"], st["h_s"] = h_q, h_s
    out_acc = _i32_matmul(h_q, w["Wd_q"])
    st["out_acc"] = out_acc
    st["out"] = _dequant16(out_acc, h_s, w["Wd_s"])
    return st


def stage_from(stage: str, w: dict, **given) -> dict:
    """Recompute one stage from oracle-supplied inputs (isolated comparison, the way the
    reference isolates stage errors in kernels/layer_bench/ffn_kernel/utils.py:877-914)."""
    if stage == "act_quant":
        q, s = quant.act_quant(given["x"])
        return {"q": q, "s": s}
    if stage == "i32":
        return {"acc": _i32_matmul(given["a_q"], given["w_q"])}
    if stage == "hadamard":
        return {"y": hadamard_full(given["x"], w.get("had_K"), w["K"])}
    raise ValueError(stage)
