"""Quantiser conventions of the reference, restated step by step (test infrastructure).

Every function spells out the floating-point type of each intermediate, because
the int8 codes depend on it.  ``rne`` = round half to even, ``rha`` = round half
away from zero.
"""
from __future__ import annotations

import torch

F16_TINY_SCALE = torch.tensor(1e-4, dtype=torch.float16)  # the 1e-4 floor as fp16 sees it


def _f16_div(a16: torch.Tensor, b16: torch.Tensor) -> torch.Tensor:
    """fp16 / fp16 as PyTorch evaluates it: exact quotient rounded once to fp16.

    An fp32 quotient of two fp16 numbers carries enough bits that rounding it
    again to fp16 equals a single rounding of the exact quotient.
    """
    return (a16.float() / b16.float()).to(torch.float16)


def latent_scale(x16: torch.Tensor) -> torch.Tensor:
    """Per-(token, head) scale of the latent cache: fp16(max(absmax/128, 1e-4)).

    Follows kernels/layer_bench/benchmark_triton_int8_layer.py:107-108 and
    kernels/layer_bench/fd_kernel/destindex_copy_quantize_latent.py:26.
    ``x16`` is fp16 with the rank on the last axis.  absmax/128 is exact in fp16
    (power-of-two division) unless it underflows, and then the floor wins anyway.
    """
    assert x16.dtype == torch.float16
    amax = x16.abs().amax(dim=-1)
    return torch.maximum(amax / 128, F16_TINY_SCALE.to(amax.device))


def latent_quant(x16: torch.Tensor, rounding: str = "torch"):
    """int8 codes and fp16 scales of a latent tensor ``[..., R]``.

    rounding="torch": the reference's PyTorch quantiser (normative) divides in
      fp16 and rounds half to even
      (kernels/layer_bench/benchmark_triton_int8_layer.py:109).
    rounding="triton": the reference's Triton append kernel divides in fp32 and
      rounds half away from zero
      (kernels/layer_bench/fd_kernel/destindex_copy_quantize_latent.py:27-29).
    """
    s16 = latent_scale(x16)
    if rounding == "torch":
        y = _f16_div(x16, s16[..., None]).float()
        r = torch.round(y)
    elif rounding == "triton":
        y = x16.float() / s16.float()[..., None]
        r = torch.where(y >= 0, y + 0.5, y - 0.5).to(torch.int32).float()  # truncation toward zero
    else:
        raise ValueError(rounding)
    q = r.clamp(-128, 127).to(torch.int8)
    return q, s16


def latent_quant_ragged(x16: torch.Tensor, offsets, rounding: str = "torch"):
    """Ragged variant: ``x16`` is ``[T, sum(r_h)]``, head h owns columns offsets[h]:offsets[h+1].

    Returns codes ``[T, sum(r_h)]`` int8 and scales ``[T, H]`` fp16.  Each head is
    quantised on its own, exactly like one slice of the uniform tensor.
    """
    T = x16.shape[0]
    H = len(offsets) - 1
    q = torch.empty(x16.shape, dtype=torch.int8)
    s = torch.empty((T, H), dtype=torch.float16)
    for h in range(H):
        qh, sh = latent_quant(x16[:, offsets[h]:offsets[h + 1]], rounding)
        q[:, offsets[h]:offsets[h + 1]] = qh
        s[:, h] = sh
    return q, s


def wuk_quant(wuk16: torch.Tensor):
    """K up-factor ``[R, H*D]`` to int8 with one fp16 scale per output column.

    Follows kernels/layer_bench/ffn_kernel/baseline_kernel.py:101-105: the same
    fp16 arithmetic as the latent cache, with the absmax taken over the rank axis.
    """
    q, s = latent_quant(wuk16.t().contiguous(), "torch")  # columns become rows
    return q.t().contiguous(), s[None, :].contiguous()


def act_scale(x: torch.Tensor, clip_ratio: float = 1.0) -> torch.Tensor:
    """Per-token symmetric activation scale of the fake-quant code, fp32.

    fake_quant/utils/quant_utils.py:201-210: row min/max are promoted to fp32 by
    a float32 zero vector, so scale = fp32(absmax) * clip / 127 whatever the dtype
    of ``x``; a zero row gets scale 1.
    """
    rows = x.reshape(-1, x.shape[-1]).float()
    amax = rows.abs().amax(dim=1) * clip_ratio
    s = amax / 127
    s[amax == 0] = 1.0
    return s.reshape(x.shape[:-1])


def act_quant(x: torch.Tensor, clip_ratio: float = 1.0):
    """int8 codes ``clamp(rne(x / s), -128, 127)`` (fp32 division) and fp32 scales.

    fake_quant/utils/quant_utils.py:30-33,41-46 (``sym_quant`` / ``STEQuantize``).
    """
    s = act_scale(x, clip_ratio)
    q = torch.round(x.float() / s[..., None]).clamp(-128, 127).to(torch.int8)
    return q, s


def weight_quant_rtn(w: torch.Tensor, mse: bool = False, norm: float = 2.4,
                     grid: int = 100, maxshrink: float = 0.8):
    """Per-output-channel symmetric int8 RTN of a weight ``[out, in]``.

    fake_quant/utils/quant_utils.py:436-498: scale = clamp(absmax, 1e-5) / 127 in
    fp32; with ``mse`` a shrink factor p = 1 - i/grid (i < maxshrink*grid) is kept
    per channel when it lowers sum(|dequant - w| ** norm).  Codes are
    clamp(rne(w / scale), -128, 127) (quant_utils.py:511-516).
    Returns (codes int8 [out, in], scale fp32 [out]).
    """
    wf = w.flatten(1)
    zero = torch.zeros(wf.shape[0])
    xmin = torch.minimum(wf.min(1)[0], zero)   # promoted to fp32 like the reference
    xmax = torch.maximum(wf.max(1)[0], zero)
    amax = torch.maximum(xmin.abs(), xmax).clamp(min=1e-5)
    scale = amax / 127
    if mse:
        best = torch.full([wf.shape[0]], float("inf"))
        for i in range(int(maxshrink * grid)):
            p = 1 - i / grid
            s1 = (p * amax) / 127
            deq = s1[:, None] * torch.round(wf / s1[:, None]).clamp(-128, 127)
            err = (deq - wf).abs().pow(norm).sum(1)
            better = err < best
            best[better] = err[better]
            scale[better] = s1[better]
    q = torch.round(wf / scale[:, None]).clamp(-128, 127).to(torch.int8)
    return q.reshape(w.shape), scale.float()
