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
    def forward(self, x, cache_k, scale_k, cache_v, scale_v, infer_state, stages: Optional[dict] = None, out=None,
                timing_events=None):
        """x [B, hidden] fp16 (one token per request).  Mutates the cache rows ``infer_state.mem_index`` in place.
        ``out`` receives the result if given; ``timing_events`` (a CUDA event pair) is recorded around the attention's
        streaming kernel."""
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
                                                  sm_scale=1.0 / math.sqrt(self.head_dim), timing_events=timing_events)
        oq, os_, _ = act_quant(o_lat)
        y1, _, _ = w8a8_gemv(oq, os_, self.W_uvo_q, self.W_uvo_s, residual=xn)
        out = self.ffn(y1, out=out, norm_weight=self.ln2, norm_eps=1e-6, residual=y1)
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


class TPDecoderLayer(nn.Module):
    """The decoder layer of one tensor-parallel rank (see lsvd_b200/parallel.py for the sharding).

    Built from that rank's local weights; ``forward`` takes the replicated hidden state and the rank's own cache
    columns, and issues one all-reduce in the attention block, one all-gather and one all-reduce in the FFN block.
    """

    def __init__(self, lw: dict, fw: dict, info: dict, head_dim: int, rank_q: int, world: int, group=None):
        super().__init__()
        self.info, self.head_dim, self.rank_q, self.world, self.group = info, head_dim, rank_q, world, group
        self.layout = LatentCacheLayout(info["k_ranks"], info["v_ranks"])
        for name in ("ln1", "ln2", "W_lat_q", "W_lat_s", "C", "W_uvo_q", "W_uvo_s"):
            self.register_buffer(name, lw[name].contiguous())
        for name in ("U_q", "U_s", "Vg_q", "Vg_s", "Vu_q", "Vu_s", "Wg_q", "Wg_s", "Wu_q", "Wu_s", "Wd_svd_q", "Wd_rtn_q", "Wd_s"):
            self.register_buffer("f_" + name, fw[name].contiguous())
        self.K = int(fw.get("K", 1))
        hk = fw.get("had_K")
        self.register_buffer("had_K", None if hk is None else hk.to(torch.float16).contiguous())
        self.had_K_packed = None
        self.Rq = self.layout.num_heads * rank_q
        self._ws = None

    @torch.no_grad()
    def forward(self, x, cache_k, scale_k, cache_v, scale_v, infer_state, stages=None):
        import torch.distributed as dist
        from .ffn import hadamard_pack, hadamard_quant
        from .parallel import gather_hidden
        lay, Hl, B, dev = self.layout, self.layout.num_heads, x.shape[0], x.device
        xq, xs, xn = act_quant(x, want_rotated=True, norm_weight=self.ln1, norm_eps=1e-5)
        lat, _, _ = w8a8_gemv(xq, xs, self.W_lat_q, self.W_lat_s)
        cache_append(lay, lat[:, self.Rq:self.Rq + lay.sum_k], lat[:, self.Rq + lay.sum_k:], infer_state.mem_index,
                     cache_k, scale_k, cache_v, scale_v)
        need = attn_decode_workspace_bytes(B, lay, infer_state.max_len_in_batch)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=dev)
        o_lat = torch.empty(B, lay.sum_v, dtype=torch.float16, device=dev)
        token_decode_attention_int8_latent_absorb(lat[:, :self.Rq].unflatten(1, (Hl, self.rank_q)), infer_state, Hl,
                                                  self.rank_q, cache_k, scale_k, cache_v, scale_v, self.C, None,
                                                  layout=lay, out_latent=o_lat, workspace=self._ws,
                                                  sm_scale=1.0 / math.sqrt(self.head_dim))
        # row-parallel output projection: dequantised partial sums in fp32, ONE all-reduce, then the residual
        oq, os_, _ = act_quant(o_lat)
        _, acc, _ = w8a8_gemv(oq, os_, self.W_uvo_q, None, want_acc=True, want_out=False)
        part = (acc.float() * os_[:, None]) * self.W_uvo_s[None, :]
        dist.all_reduce(part, group=self.group)
        y1 = (part + xn.float()).half()
        # FFN: replicated latents, column-parallel gate/up, gathered hidden vector, row-parallel int32 down projection
        r = self.f_U_q.shape[0] // 2
        x2q, x2s, _ = act_quant(y1, norm_weight=self.ln2, norm_eps=1e-6)
        lat2, _, _ = w8a8_gemv(x2q, x2s, self.f_U_q, self.f_U_s)
        zq, zs, _ = act_quant(lat2.view(-1, r))
        zq, zs = zq.view(-1, 2 * r), zs.view(-1, 2)
        ns, nq = self.f_Vg_q.shape[0], self.f_Wg_q.shape[0]
        h_local = torch.empty(B, ns + nq, dtype=torch.float16, device=dev)
        w8a8_gemv(zq[:, :r], zs[:, 0], self.f_Vg_q, self.f_Vg_s, self.f_Vu_q, self.f_Vu_s, a2_q=zq[:, r:], a2_scale=zs[:, 1],
                  out=h_local, out_col=0)
        w8a8_gemv(x2q, x2s, self.f_Wg_q, self.f_Wg_s, self.f_Wu_q, self.f_Wu_s, out=h_local, out_col=ns)
        h = gather_hidden(h_local, self.info, self.world, self.group)
        if self.had_K_packed is None:
            self.had_K_packed = hadamard_pack(self.had_K)
        hq, hs, _ = hadamard_quant(h, self.had_K_packed, self.K)
        s0, s1 = self.info["svd"]
        q0, q1 = self.info["rtn"]
        n_svd = self.info["n_svd"]
        _, a1, _ = w8a8_gemv(hq[:, s0:s1], hs, self.f_Wd_svd_q, None, want_acc=True, want_out=False)
        _, a2, _ = w8a8_gemv(hq[:, n_svd + q0:n_svd + q1], hs, self.f_Wd_rtn_q, None, want_acc=True, want_out=False)
        acc = a1 + a2
        dist.all_reduce(acc, group=self.group)
        down = ((acc.float() * hs[:, None]) * self.f_Wd_s[None, :]).half()
        out = (down.float() + y1.float()).half()
        if stages is not None:
            stages.update(xn=xn, o_lat=o_lat, y1=y1, h_q=hq, down_acc=acc, out=out)
        return out
