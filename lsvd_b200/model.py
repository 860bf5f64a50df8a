"""Stacks of LSVD W8A8 decoder layers: the layer-loop drivers of BASELINE configs 4 and 5.

The reference benchmarks one layer (kernels/layer_bench/benchmark_triton_int8_layer.py:541-566, 769-780) and evaluates
whole checkpoints through HuggingFace models; it has no serving loop of its own.  These classes are the thin loop over
``LSVDDecoderLayer`` / ``TPDecoderLayer`` with per-layer weights (seeded random init, one seed per layer) and per-layer
latent caches: decode steps for a batch (config 4: 40 layers of the 13B shape, tensor-parallel), and prefill followed by
decode steps (config 5: 32 layers of the 7B shape).
"""
from __future__ import annotations

from typing import List, Optional

import torch
from torch import nn

from . import synth
from .attention import InferState, LatentCacheLayout, decode_advance
from .ffn import HybridFFN
from .layer import LSVDDecoderLayer, TPDecoderLayer, make_layer_weights
from .parallel import shard_layer


class LSVDModel(nn.Module):
    """``n_layers`` decoder layers on one GPU with their int8 latent caches.

    ``prefill(x, dest_slots)`` runs ``x [T, hidden]`` through every layer's prefill form (cache rows written at
    ``dest_slots``); ``decode_step(x, state)`` runs one token per request through every layer (each layer appends to its
    own cache at ``state.mem_index`` and attends over ``state.b_seq_len`` tokens) and returns the last hidden state.
    """

    def __init__(self, n_layers: int, hidden: int, num_heads: int, head_dim: int, d_ffn: int, rank_q: int, k_ranks, v_ranks,
                 ffn_rank: int, n_svd: int, had_K: Optional[torch.Tensor], K: int, num_slots: int, device="cuda", seed: int = 0,
                 head_major: bool = False, weights: Optional[List[tuple]] = None):
        """``weights``: optional list of (layer dict, ffn dict) per layer (parity tests); otherwise drawn on ``device``."""
        super().__init__()
        self.layout = LatentCacheLayout(k_ranks, v_ranks, head_major=head_major)
        self.hidden, self.n_layers = hidden, n_layers
        layers, self.caches = [], []
        for i in range(n_layers):
            if weights is not None:
                lw, fw = weights[i]
            else:
                lw = make_layer_weights(hidden, num_heads, head_dim, rank_q, k_ranks, v_ranks, seed=seed + 2 * i, device=device)
                fw = synth.ffn_weights(hidden, d_ffn, ffn_rank, n_svd, seed=seed + 2 * i + 1, had_K=had_K, K=K, input_had=False,
                                       device=device)
            to = lambda d: {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
            layers.append(LSVDDecoderLayer(self.layout, head_dim, rank_q, to(lw), HybridFFN(to(fw))))
            self.caches.append(self.layout.alloc(num_slots, device))
        self.layers = nn.ModuleList(layers)

    @torch.no_grad()
    def prefill(self, x: torch.Tensor, dest_slots: torch.Tensor) -> torch.Tensor:
        for layer, (ck, sk, cv, sv) in zip(self.layers, self.caches):
            x = layer.forward_prefill(x, ck, sk, cv, sv, dest_slots)
        return x

    @torch.no_grad()
    def decode_step(self, x: torch.Tensor, state: InferState, after_last_attention=None) -> torch.Tensor:
        """One token per request through every layer.  ``after_last_attention`` (a callable) runs on a side stream once
        the last layer's attention has read ``state``, beside that layer's output projection and FFN."""
        last = len(self.layers) - 1
        for i, (layer, (ck, sk, cv, sv)) in enumerate(zip(self.layers, self.caches)):
            x = layer(x, ck, sk, cv, sv, state, after_attention=after_last_attention if i == last else None)
        return x

    @torch.no_grad()
    def capture_decode(self, x: torch.Tensor, state: InferState, advance: Optional[dict] = None):
        """One decode step of the whole stack as a CUDA graph: ``(graph, out)``.  The graph reads ``x`` and the device
        tensors of ``state`` in place (lengths and slots are read on the device, so the same graph serves a growing
        context up to ``state.max_len_in_batch``) and writes ``out``; with ``advance`` (keyword arguments of
        ``decode_advance``) the step also moves ``state`` to the next token on the device, so a decode loop is
        ``x.copy_(...); graph.replay()`` with no other host work -- the way the reference's harness replays its layer
        (kernels/layer_bench/ffn_kernel/utils.py:687-706).  One eager step runs first (it sizes the workspaces); it
        writes the cache rows that the first replay rewrites."""
        side = torch.cuda.Stream(device=x.device)
        side.wait_stream(torch.cuda.current_stream(x.device))
        with torch.cuda.stream(side):
            self.decode_step(x, state)
        torch.cuda.current_stream(x.device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = self.decode_step(x, state, after_last_attention=(
                None if advance is None else (lambda: decode_advance(state, **advance))))
        return graph, out


class TPModel(nn.Module):
    """One tensor-parallel rank of a stack: ``n_layers`` ``TPDecoderLayer``s with the rank's share of every cache."""

    def __init__(self, n_layers: int, hidden: int, num_heads: int, head_dim: int, d_ffn: int, rank_q: int, k_ranks, v_ranks,
                 ffn_rank: int, n_svd: int, had_K, K: int, num_slots: int, world: int, rank: int, device="cuda", seed: int = 0,
                 head_major: bool = False, group=None, fill_cache: bool = False):
        super().__init__()
        layers, self.caches = [], []
        for i in range(n_layers):
            # the same seeds on every rank: every rank draws the whole layer and keeps its shard
            lw_full = make_layer_weights(hidden, num_heads, head_dim, rank_q, k_ranks, v_ranks, seed=seed + 2 * i, device=device)
            fw_full = synth.ffn_weights(hidden, d_ffn, ffn_rank, n_svd, seed=seed + 2 * i + 1, had_K=had_K, K=K, input_had=False,
                                        device=device)
            lw, fw, info = shard_layer(lw_full, fw_full, k_ranks, v_ranks, rank_q, world, rank)
            del lw_full, fw_full
            to = lambda d: {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
            layer = TPDecoderLayer(to(lw), to(fw), info, head_dim, rank_q, world, group=group, head_major=head_major)
            layers.append(layer)
            cache = layer.layout.alloc(num_slots, device)
            if fill_cache:
                fill_random_cache(cache, seed=seed + 1000 * rank + i, device=device)
            self.caches.append(cache)
        self.layers = nn.ModuleList(layers)
        self.layout = layers[0].layout
        self.weight_bytes = sum(b.numel() for b in self.buffers() if b.dtype == torch.int8)

    @torch.no_grad()
    def decode_step(self, x: torch.Tensor, state: InferState, timing_events=None) -> torch.Tensor:
        for i, (layer, (ck, sk, cv, sv)) in enumerate(zip(self.layers, self.caches)):
            x = layer(x, ck, sk, cv, sv, state, timing_events=timing_events if i == 0 else None)
        return x


def fill_random_cache(cache, seed: int = 0, device="cuda") -> None:
    """Random int8 codes and plausible scales for benchmark caches (what a long context would have left there)."""
    ck, sk, cv, sv = cache
    g = torch.Generator(device=device).manual_seed(seed)
    for t in (ck, cv):
        flat = t.view(-1)
        for o in range(0, flat.numel(), 1 << 28):
            n = min(1 << 28, flat.numel() - o)
            flat[o:o + n] = torch.randint(-128, 128, (n,), dtype=torch.int8, device=device, generator=g)
    for t in (sk, sv):
        t.copy_((torch.rand(t.shape, device=device, generator=g) * 0.02 + 0.01).half())
