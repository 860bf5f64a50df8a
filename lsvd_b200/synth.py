"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

No dataset or checkpoint is involved on this path: the reference's own latency benchmark draws its
latents, weights and activations from normal distributions
(kernels/layer_bench/benchmark_triton_int8_layer.py:116-149,
kernels/layer_bench/ffn_kernel/mix_ffn_kernel.py:294-318).  Everything is drawn from a CPU
``torch.Generator`` so the CPU checker and the GPU see identical bits.
"""
from __future__ import annotations

import torch


def ragged_ranks(num_heads: int, mean: int = 64, lo: int = 16, hi: int = 128, seed: int = 0):
    """Per-head ranks: multiples of 16 in [lo, hi] whose sum is num_heads * mean (a seeded draw)."""
    g = torch.Generator().manual_seed(seed)
    steps = torch.randint(lo // 16, hi // 16 + 1, (num_heads,), generator=g).tolist()
    target = num_heads * mean // 16
    order = torch.randperm(num_heads, generator=g).tolist()
    i = 0
    while sum(steps) != target:
        h = order[i % num_heads]
        if sum(steps) > target and steps[h] > lo // 16:
            steps[h] -= 1
        elif sum(steps) < target and steps[h] < hi // 16:
            steps[h] += 1
        i += 1
    return [s * 16 for s in steps]


def attention_inputs(batch: int, num_heads: int, head_dim: int, k_ranks, v_ranks, seq_lens, seed: int = 0,
                     shuffle_slots: bool = False, extra_slots: int = 0):
    """fp16 latents for every cached token, per-head up-factors N(0, 1/64) and a query N(0, 1), on the CPU.

    Returns a dict: latent_k/v ``[N_slots, sum r]`` fp16 (to be quantised into the cache), up_k/up_v
    ``[sum r, D]`` fp16, q ``[B, H, D]`` fp16, req_to_token ``[B, max_len]`` int32, b_req_idx, b_seq_len.
    """
    g = torch.Generator().manual_seed(seed)
    max_len = max(max(seq_lens), 1)
    n_slots = batch * max_len + extra_slots
    sum_k, sum_v = sum(k_ranks), sum(v_ranks)
    lat_k = torch.randn(n_slots, sum_k, generator=g, dtype=torch.float32).to(torch.float16)
    lat_v = torch.randn(n_slots, sum_v, generator=g, dtype=torch.float32).to(torch.float16)
    up_k = (torch.randn(sum_k, head_dim, generator=g) / 8).to(torch.float16)
    up_v = (torch.randn(sum_v, head_dim, generator=g) / 8).to(torch.float16)
    q = torch.randn(batch, num_heads, head_dim, generator=g).to(torch.float16)
    if shuffle_slots:
        r2t = torch.randperm(n_slots, generator=g)[: batch * max_len].to(torch.int32).view(batch, max_len)
        b_req = torch.randperm(batch, generator=g).to(torch.int32)
    else:
        r2t = torch.arange(batch * max_len, dtype=torch.int32).view(batch, max_len)
        b_req = torch.arange(batch, dtype=torch.int32)
    return dict(latent_k=lat_k, latent_v=lat_v, up_k=up_k, up_v=up_v, q=q, req_to_token=r2t, b_req_idx=b_req,
                b_seq_len=torch.tensor(list(seq_lens), dtype=torch.int32), max_len=max_len, n_slots=n_slots)


def sign_matrix(K: int, seed: int = 0):
    """A seeded +-1 matrix [K, K] standing in for the non-power-of-two Hadamard factor of d_ffn when the
    reference's literal matrices are not at hand.  The kernels treat ``had_K`` as an arbitrary input matrix, so
    timings and parity against the CPU checker do not depend on it being orthogonal."""
    g = torch.Generator().manual_seed(seed)
    return (torch.randint(0, 2, (K, K), generator=g) * 2 - 1).to(torch.float16)


def ffn_weights(d_in: int, d_ffn: int, rank: int, n_svd: int, seed: int = 0, std: float = 0.02, had_K=None,
                K: int = 1, input_had: bool = True, mse: bool = False, device=None) -> dict:
    """Seeded hybrid-FFN weights on the CPU: N(0, std) draws, int8 RTN per output channel.

    A seeded ``randperm(d_ffn)[:n_svd]`` picks the SVD channel group; the weights being random, the permutation
    only fixes the input-column order [SVD | RTN] of the down projection, which is the order they are drawn in.
    Returns the dict ``HybridFFN`` and the CPU checker both take.
    """
    from .ffn import quantize_weight_rtn
    # `device`: draw on that device (benchmarks of whole stacks, where a CPU draw of every layer would take minutes);
    # the default CPU generator is what the parity tests and the CPU checker share
    g = (torch.Generator() if device is None else torch.Generator(device=device)).manual_seed(seed)
    dv = dict(device=device) if device is not None else {}
    n_q = d_ffn - n_svd
    w = {"K": K, "had_K": had_K, "online_had": True}
    for name, shape in (("U", (2 * rank, d_in)), ("Vg", (n_svd, rank)), ("Vu", (n_svd, rank)),
                        ("Wg", (n_q, d_in)), ("Wu", (n_q, d_in)), ("Wd", (d_in, d_ffn))):
        w[name + "_q"], w[name + "_s"] = quantize_weight_rtn(torch.randn(*shape, generator=g, **dv) * std, mse)
    w["perm"] = torch.randperm(d_ffn, generator=g, **dv)
    w["had_sign"] = (torch.randint(0, 2, (d_in,), generator=g, **dv).float() * 2 - 1).to(torch.float16) if input_had else None
    return w
