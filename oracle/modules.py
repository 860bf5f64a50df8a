"""CPU restatement of the reference's accuracy-side modules ``SVDLinear`` (per-head form) and ``ActQuantWrapper``
(test infrastructure: used by tests/ only, never by the product path).

Pinned by tests/test_oracle_golden.py against outputs of the reference's own modules run on the CPU
(tests/golden/svd_linear.npz, act_quant_wrapper.npz, made by tests/golden/make_golden.py).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

from . import ffn as offn
from . import quant


def linear16(x16: torch.Tensor, w16: torch.Tensor, bias16: Optional[torch.Tensor] = None) -> torch.Tensor:
    """An fp16 ``nn.Linear``: products accumulated in fp32, bias added before the single rounding to fp16."""
    y = x16.float() @ w16.float().t()
    if bias16 is not None:
        y = y + bias16.float()
    return y.half()


def svd_linear_per_head(x16: torch.Tensor, B16: torch.Tensor, A16: Sequence[torch.Tensor],
                        bias16: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``SVDLinear.forward`` for per-head factors (fake_quant/utils/svd_utils.py:1978-2027): ``z = BLinear(x)`` in fp16,
    head h multiplies its own slice of z by ``A_h [cout, r_h]`` (the reference pads slices and factors with zeros to the
    largest rank, which adds exact zeros), one rounding to fp16, then ``y + bias`` as an fp16 addition (``:2029-2031``)."""
    z = linear16(x16, B16)
    outs, c = [], 0
    for a in A16:
        r = a.shape[1]
        outs.append((z[..., c:c + r].float() @ a.float().t()).half())
        c += r
    y = torch.cat(outs, dim=-1)
    if bias16 is not None:
        y = (y.float() + bias16.float()).half()
    return y


def fake_quant16(x16: torch.Tensor) -> torch.Tensor:
    """``ActQuantizer.forward`` for 8 bits, symmetric, per token (fake_quant/utils/quant_utils.py:141-148, 201-212)."""
    q, s = quant.act_quant(x16)
    return (s[..., None] * q.float()).half()


def act_quant_wrapper(x16: torch.Tensor, w16: torch.Tensor, bias16: Optional[torch.Tensor] = None, *, rotation: str = "none",
                      had_K: Optional[torch.Tensor] = None, K: int = 1, had_dim: int = 0, in_bits: int = 8,
                      out_bits: int = 16) -> torch.Tensor:
    """``ActQuantWrapper.forward`` (fake_quant/utils/quant_utils.py:267-340): rotation, input quantiser, fp16 Linear,
    output quantiser.  ``rotation``: "none" | "full" (matmul_hadU_cuda with (had_K, K)) | "partial" (across heads of
    size ``had_dim``) | "random" (``x @ had_K``, an fp16 product)."""
    lead = x16.shape[:-1]
    x = x16.reshape(-1, x16.shape[-1])
    if rotation == "full":
        x = offn.hadamard_full(x, had_K, K)
    elif rotation == "partial":
        x = offn.partial_hadamard_heads(x, had_dim) if K == 1 else offn.partial_hadamard_heads_hadk(x, had_dim, had_K)
    elif rotation == "random":
        x = (x.float() @ had_K.float()).half()
    elif rotation != "none":
        raise ValueError(rotation)
    if in_bits < 16:
        x = fake_quant16(x)
    y = linear16(x, w16, bias16)
    if out_bits < 16:
        y = fake_quant16(y)
    return y.reshape(*lead, -1)
