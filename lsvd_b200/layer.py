"""One LSVD W8A8 decoder layer for decode steps, composed of the library's kernels.

Structure (the kernel-side attention block of the reference,
kernels/layer_bench/ffn_kernel/baseline_kernel.py:107-145, with its fp16 projections replaced by int8
products, followed by the hybrid FFN of fake_quant/utils/hybrid_ffn_utils.py:956-984):

    xn   = RMSNorm(x) * w1                  (eps 1e-5; the residual of the attention block is xn, as in the reference)
    lat  = A8(xn) . W_lat^T                 [q latents | K latents | V latents], int8 product, fp16 out
    cache <- quantise(K, V latents) at mem_index
    o    = latent decode attention(q latents, C = B_k A_q^T per head, cache)     in V-latent space
    y1   = A8(o) . W_uvo^T + xn             W_uvo = the V up-factor composed with the output projection
    out  = hybrid FFN(RMSNorm(y1) * w2) + y1            (eps 1e-6; the residual of the FFN is its raw input)

The per-head query up-projection A_q and the K up-factor B_k are composed offline into C_h = B_k,h A_q,h^T
(r_k x r_q), so the attention kernel's query absorption takes the query latent directly.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import nn

from .attention import LatentCacheLayout, cache_append, token_decode_attention_int8_latent_absorb, attn_decode_workspace_bytes
from .ffn import HybridFFN, act_quant, w8a8_gemv, quantize_weight_rtn


class LSVDDecoderLayer(nn.Module):
    def __init__(self, layout: LatentCacheLayout, head_dim: int, rank_q: int, w: dict, ffn: HybridFFN):
        """``w``: ln1 [hidden] fp16, ln2 [hidden] fp16, W_lat_q int8 [H*rank_q + sum r_k + sum r_v, hidden] + W_lat_s,
        C fp16 [sum r_k, rank_q] (per-head blocks), W_uvo_q int8 [hidden, sum r_v] + W_uvo_s."""
        super().__init__()
        self.layout, self.head_dim, self.rank_q, self.ffn = layout, head_dim, rank_q, ffn
        for name in ("ln1", "ln2", "W_lat_q", "W_lat_s", "C", "W_uvo_q", "W_uvo_s"):
            self.register_buffer(name, w[name].contiguous())
        self.hidden = self.ln1.shape[0]
        self.Rq = layout.num_heads * rank_q
        self._ws = None

    @torch.no_grad()
    def forward(self, x, cache_k, scale_k, cache_v, scale_v, infer_state, stages: Optional[dict] = None):
        """x [B, hidden] fp16 (one token per request).  Mutates the cache rows ``infer_state.mem_index`` in place."""
        lay, H, B = self.layout, self.layout.num_heads, x.shape[0]
        xq, xs, xn = act_quant(x, want_rotated=True, norm_weight=self.ln1, norm_eps=1e-5)
        lat, _, _ = w8a8_gemv(xq, xs, self.W_lat_q, self.W_lat_s)
        lk = lat[:, self.Rq:self.Rq + lay.sum_k]
        lv = lat[:, self.Rq + lay.sum_k:]
        cache_append(lay, lk, lv, infer_state.mem_index, cache_k, scale_k, cache_v, scale_v)
        need = attn_decode_workspace_bytes(B, lay, infer_state.max_len_in_batch)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=x.device)
        o_lat = torch.empty(B, lay.sum_v, dtype=torch.float16, device=x.device)
        q = lat[:, :self.Rq].unflatten(1, (H, self.rank_q))
        token_decode_attention_int8_latent_absorb(q, infer_state, H, self.rank_q, cache_k, scale_k, cache_v, scale_v,
                                                  self.C, None, layout=lay, out_latent=o_lat, workspace=self._ws,
                                                  sm_scale=1.0 / math.sqrt(self.head_dim))
        oq, os_, _ = act_quant(o_lat)
        y1, _, _ = w8a8_gemv(oq, os_, self.W_uvo_q, self.W_uvo_s, residual=xn)
        out = self.ffn(y1, norm_weight=self.ln2, norm_eps=1e-6, residual=y1)
        if stages is not None:
            stages.update(xn=xn, lat=lat, o_lat=o_lat, y1=y1, out=out)
        return out


def make_layer_weights(hidden: int, num_heads: int, head_dim: int, rank_q: int, k_ranks, v_ranks, seed: int = 0):
    """Seeded random layer weights on the CPU (xavier-like scales as the reference's block,
    kernels/layer_bench/ffn_kernel/baseline_kernel.py:86-91); returns the dict ``LSVDDecoderLayer`` takes."""
    g = torch.Generator().manual_seed(seed)
    Rq, Rk, Rv = num_heads * rank_q, sum(k_ranks), sum(v_ranks)

    def rnd(*shape, std):
        return torch.randn(*shape, generator=g) * std

    W_lat = rnd(Rq + Rk + Rv, hidden, std=1.0 / math.sqrt(hidden))
    A_q = rnd(num_heads, head_dim, rank_q, std=1.0 / math.sqrt(rank_q))          # query up-factor per head
    B_k = rnd(Rk, head_dim, std=1.0 / 8)                                           # K up-factor rows per head
    C = torch.empty(Rk, rank_q)
    off = 0
    for h, r in enumerate(k_ranks):
        C[off:off + r] = B_k[off:off + r] @ A_q[h]
        off += r
    W_uvo = rnd(hidden, Rv, std=1.0 / math.sqrt(Rv))
    w = {"ln1": (1 + 0.1 * rnd(hidden, std=1.0)).half(), "ln2": (1 + 0.1 * rnd(hidden, std=1.0)).half(), "C": C.half()}
    w["W_lat_q"], w["W_lat_s"] = quantize_weight_rtn(W_lat)
    w["W_uvo_q"], w["W_uvo_s"] = quantize_weight_rtn(W_uvo)
    return w
