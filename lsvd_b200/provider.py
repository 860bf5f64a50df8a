"""The hybrid FFN as a provider for the reference's layer benchmark.

The reference looks FFN implementations up by name and calls them as ``fn(x, module)`` with ``module`` its fp16
``SwiGLUFFN`` (norm + up_proj / gate_proj / down_proj + residual)
(kernels/layer_bench/ffn_kernel/mix_ffn_kernel.py:2223-2246, kernels/layer_bench/benchmark_triton_int8_layer.py:819);
the conversion of a source module is cached like ``get_mixed_gateup_v8_ffn`` does (:2125-2143).  Registering this
provider there is one line: ``NAME["b200"] = lsvd_b200.provider.b200_ffn``.

Conversion (offline, host code): the first ``svd_out`` intermediate channels (a multiple of 64, as
``svd_out_from_ratio``, :889-897) form the SVD group, whose gate/up rows are replaced by seeded synthetic low-rank
factors exactly as the reference's kernel experiments do (:545-554: no decomposition is computed there either); the
other channels keep their dense rows; everything is quantised per output channel to int8.  The module's RMSNorm
runs inside the first quantiser and its residual in the last epilogue.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .ffn import HybridFFN

_CACHE = {}


def rounded_rank(in_features: int, out_features: int, rank_ratio: float, round_to: int = 64) -> int:
    """Rank of a low-rank branch holding ``rank_ratio`` of the dense parameters, rounded down to ``round_to``
    (the reference's formula, mix_ffn_kernel.py:536-543)."""
    if rank_ratio <= 0.0:
        return 0
    rank = int(in_features * out_features * rank_ratio / (in_features + out_features))
    rank = max(1, min(rank, in_features, out_features))
    if round_to > 1 and rank >= round_to:
        rank = max(round_to, (rank // round_to) * round_to)
    return max(1, min(rank, in_features, out_features))


def convert_swiglu(module, svd_ratio: float = 0.5, rank_ratio: float = 0.25, round_to: int = 64, seed: int = 0,
                   had: Optional[Tuple[torch.Tensor, int]] = None) -> HybridFFN:
    """HybridFFN from a SwiGLUFFN-like module (``norm.weight``, ``up_proj``, ``gate_proj``, ``down_proj``).
    ``had = (had_K, K)`` enables the online Hadamard of the hidden vector for an intermediate size K * 2^n."""
    wg, wu, wd = module.gate_proj.weight.data, module.up_proj.weight.data, module.down_proj.weight.data
    d_ffn, d_in = wg.shape
    n_svd = int(d_ffn * svd_ratio) // round_to * round_to
    if n_svd <= 0 or n_svd >= d_ffn:
        raise ValueError("svd_ratio must leave channels on both branches")
    r = max(16, rounded_rank(d_in, n_svd, rank_ratio, round_to) // 16 * 16)
    g = torch.Generator().manual_seed(seed)
    dev = wg.device

    def factors():
        a = torch.randn(r, d_in, generator=g) / d_in ** 0.5
        b = torch.randn(n_svd, r, generator=g) / r ** 0.5
        return a.to(dev), b.to(dev)

    ug, vg = factors()
    uu, vu = factors()
    had_K, K = had if had is not None else (None, 1)
    return HybridFFN.from_float(U=torch.cat([ug, uu]), Vg=vg, Vu=vu, Wg=wg[n_svd:].float(), Wu=wu[n_svd:].float(),
                                Wd=wd.float(), had_K=had_K, K=K, online_had=had is not None)


def get_b200_ffn(module, **kw):
    """Converted FFN of a source module, cached per module object and conversion arguments."""
    key = (id(module), tuple(sorted((k, v) for k, v in kw.items() if k != "had")))
    got = _CACHE.get(key)
    if got is None:
        ffn = convert_swiglu(module, **kw).to(module.down_proj.weight.device)
        got = (ffn, module.norm.weight.data.to(torch.float16).contiguous(), float(getattr(module.norm, "variance_epsilon", 1e-6)))
        _CACHE[key] = got
    return got


@torch.no_grad()
def b200_ffn(x: torch.Tensor, module) -> torch.Tensor:
    """``x [batch, q_len, hidden]`` fp16 -> same shape: RMSNorm, hybrid FFN, residual, as ``mixffn_ffn`` is called."""
    ffn, norm_w, eps = get_b200_ffn(module)
    x2 = x.reshape(-1, x.shape[-1])
    return ffn(x2, norm_weight=norm_w, norm_eps=eps, residual=x2).view_as(x)


from .mixffn import b200_mixffn  # noqa: E402  (the mixffn-structure provider lives beside its module)

# "b200": the hybrid SVD/RTN FFN of fake_quant (Hadamard in front of the down projection);
# "b200_mixffn": the reference's own mixffn structure and arithmetic, for a head-to-head with its "mixffn" provider
NAME = {"b200": b200_ffn, "b200_mixffn": b200_mixffn}
