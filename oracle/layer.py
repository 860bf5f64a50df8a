"""The W8A8 decoder layer composed from the oracle's stage functions (test infrastructure).

Mirrors lsvd_b200/layer.py stage by stage; every stage is one of the pinned oracle functions, plus the
reference's RMSNorm (kernels/layer_bench/ffn_kernel/utils.py:560-565).
"""
import math

import torch

from . import quant, attention, ffn


def rms_norm(x16, w16, eps):
    """fp32 statistics, normalised value rounded to fp16, fp16 product with the weight."""
    xf = x16.float()
    xn = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).half()
    return (xn.float() * w16.float()).half()


def linear_a8w8(x16, w_q, w_s, residual=None):
    q, s = quant.act_quant(x16)
    y = ffn._dequant16(ffn._i32_matmul(q, w_q), s, w_s)
    if residual is not None:
        y = (y.float() + residual.float()).half()
    return y


def decoder_layer(x16, w, ffn_w, k_off, v_off, num_heads, head_dim, rank_q, cache_k, scale_k, cache_v, scale_v,
                  req_to_token, b_req_idx, b_seq_len, mem_index, xn=None, y1=None):
    """Returns (out fp16, stages).  Mutates the cache like the reference block does.  ``xn`` / ``y1`` replace the
    normalised input / the attention block's output by values computed elsewhere, so that the stages behind them can be
    compared bit for bit (an fp32 mean of 4096 squares depends on the order of the additions)."""
    Rq = num_heads * rank_q
    xn_own = rms_norm(x16, w["ln1"], 1e-5)
    xn = xn_own if xn is None else xn
    lat = linear_a8w8(xn, w["W_lat_q"], w["W_lat_s"])
    attention.cache_append(lat[:, Rq:Rq + k_off[-1]].contiguous(), mem_index, k_off, cache_k, scale_k)
    if cache_v is not cache_k:                  # a shared K/V latent is cached once (svd_utils.py:1505-1507)
        attention.cache_append(lat[:, Rq + k_off[-1]:].contiguous(), mem_index, v_off, cache_v, scale_v)
    q = lat[:, :Rq].reshape(-1, num_heads, rank_q)
    ident = torch.zeros(v_off[-1], 1, dtype=torch.float16)          # the V up-projection is folded into W_uvo
    _, o_lat = attention.decode_absorb(q, cache_k, scale_k, cache_v, scale_v, w["C"], ident, k_off, v_off,
                                       req_to_token, b_req_idx, b_seq_len, sm_scale=1.0 / math.sqrt(head_dim),
                                       dtype=torch.float32)
    o16 = o_lat.half()
    y1_own = linear_a8w8(o16, w["W_uvo_q"], w["W_uvo_s"], residual=xn)
    y1 = y1_own if y1 is None else y1
    x2 = rms_norm(y1, w["ln2"], 1e-6)
    st = ffn.hybrid_ffn_stages(x2, ffn_w)
    out = (st["out"].float() + y1.float()).half()
    return out, dict(xn=xn_own, lat=lat, o_lat=o16, y1=y1_own, out=out)


def prefill_layer(x16, w, ffn_w, k_off, v_off, num_heads, rank_q, cache_k, scale_k, cache_v, scale_v, dest_slots):
    """The prefill form of the layer (lsvd_b200/layer.py, forward_prefill): the same stages as a decode step with the
    attention output replaced by the token's own V latent (the reference has no prefill attention; see that docstring)."""
    Rq = num_heads * rank_q
    xn = rms_norm(x16, w["ln1"], 1e-5)
    lat = linear_a8w8(xn, w["W_lat_q"], w["W_lat_s"])
    attention.cache_append(lat[:, Rq:Rq + k_off[-1]].contiguous(), dest_slots, k_off, cache_k, scale_k)
    attention.cache_append(lat[:, Rq + k_off[-1]:].contiguous(), dest_slots, v_off, cache_v, scale_v)
    o16 = lat[:, Rq + k_off[-1]:].contiguous()
    y1 = linear_a8w8(o16, w["W_uvo_q"], w["W_uvo_s"], residual=xn)
    x2 = rms_norm(y1, w["ln2"], 1e-6)
    st = ffn.hybrid_ffn_stages(x2, ffn_w)
    out = (st["out"].float() + y1.float()).half()
    return out, dict(xn=xn, lat=lat, y1=y1, out=out)


def decoder_layer_tp_rank(x16, lw, fw, info, head_dim, rank_q, world, cache_k, scale_k, cache_v, scale_v,
                          req_to_token, b_req_idx, b_seq_len, mem_index, group=None):
    """One tensor-parallel rank of the layer on the CPU (gloo collectives): the same algebra as
    lsvd_b200.layer.TPDecoderLayer with the oracle's stage functions.  ``cache_*`` hold this rank's columns."""
    import torch.distributed as dist
    from lsvd_b200.parallel import gather_hidden
    kr, vr = info["k_ranks"], info["v_ranks"]
    k_off, v_off = [0], [0]
    for a, b in zip(kr, vr):
        k_off.append(k_off[-1] + a)
        v_off.append(v_off[-1] + b)
    Hl = len(kr)
    Rq = Hl * rank_q
    xn = rms_norm(x16, lw["ln1"], 1e-5)
    lat = linear_a8w8(xn, lw["W_lat_q"], lw["W_lat_s"])
    attention.cache_append(lat[:, Rq:Rq + k_off[-1]].contiguous(), mem_index, k_off, cache_k, scale_k)
    attention.cache_append(lat[:, Rq + k_off[-1]:].contiguous(), mem_index, v_off, cache_v, scale_v)
    ident = torch.zeros(v_off[-1], 1, dtype=torch.float16)
    _, o_lat = attention.decode_absorb(lat[:, :Rq].reshape(-1, Hl, rank_q), cache_k, scale_k, cache_v, scale_v, lw["C"],
                                       ident, k_off, v_off, req_to_token, b_req_idx, b_seq_len,
                                       sm_scale=1.0 / math.sqrt(head_dim), dtype=torch.float32)
    oq, os_ = quant.act_quant(o_lat.half())
    part = (ffn._i32_matmul(oq, lw["W_uvo_q"]).float() * os_[:, None]) * lw["W_uvo_s"][None, :]
    dist.all_reduce(part, group=group)
    y1 = (part + xn.float()).half()
    x2 = rms_norm(y1, lw["ln2"], 1e-6)
    x2q, x2s = quant.act_quant(x2)
    r = fw["U_q"].shape[0] // 2
    lat2 = ffn._dequant16(ffn._i32_matmul(x2q, fw["U_q"]), x2s, fw["U_s"])
    gq, gs = quant.act_quant(lat2[:, :r])
    uq, us = quant.act_quant(lat2[:, r:])
    g16 = torch.cat((ffn._dequant16(ffn._i32_matmul(gq, fw["Vg_q"]), gs, fw["Vg_s"]),
                     ffn._dequant16(ffn._i32_matmul(x2q, fw["Wg_q"]), x2s, fw["Wg_s"])), 1)
    u16 = torch.cat((ffn._dequant16(ffn._i32_matmul(uq, fw["Vu_q"]), us, fw["Vu_s"]),
                     ffn._dequant16(ffn._i32_matmul(x2q, fw["Wu_q"]), x2s, fw["Wu_s"])), 1)
    h_local = ffn.silu_mul16(g16, u16)
    h = gather_hidden(h_local, info, world, group)
    h_rot = ffn.hadamard_full(h, fw["had_K"], fw["K"])
    hq, hs = quant.act_quant(h_rot)
    s0, s1 = info["svd"]
    q0, q1 = info["rtn"]
    n_svd = info["n_svd"]
    acc = ffn._i32_matmul(torch.cat((hq[:, s0:s1], hq[:, n_svd + q0:n_svd + q1]), dim=1), fw["Wd_loc_q"])
    dist.all_reduce(acc, group=group)
    down = ((acc.float() * hs[:, None]) * fw["Wd_s"][None, :]).half()
    out = (down.float() + y1.float()).half()
    return out, dict(y1=y1, h_q=hq, down_acc=acc, out=out)


def int8_attention_block(x16, w, cache_k, scale_k, cache_v, scale_v, req_to_token, b_req_idx, b_seq_len, mem_index,
                         num_heads, head_dim, theta=10000.0):
    """One decode step of the reference's Int8AttentionBlock (kernels/layer_bench/ffn_kernel/baseline_kernel.py:107-145).

    ``w`` holds its parameters by name plus ``wuk_q``, ``wuk_scale`` and ``wuvout``.  fp16 GEMMs are computed in fp32
    and rounded once, as a library GEMM with fp32 accumulation does; the append uses the Triton kernel's rounding
    (the block imports fd_kernel/destindex_copy_quantize_latent.py).  Mutates the caches like the block; returns
    ``[B, 1, hidden]`` fp16.
    """
    B = x16.shape[0]
    H, D = num_heads, head_dim
    xn = rms_norm(x16.view(B, -1), w["input_layernorm_weight"], 1e-5)                       # :119-120
    R = w["up_proj_q"].shape[0]
    lat_q = (xn.float() @ w["down_proj_q"].float().t()).half().view(B, H, R)                # :122
    wuq = w["up_proj_q"].view(H, R, D)                                                      # :123 (a plain reshape)
    q = torch.einsum("bhr,hrd->bhd", lat_q.float(), wuq.float()).half()                     # :124
    lat_kv = (xn.float() @ w["down_proj_kv"].float().t()).half().view(B, 2, H * R)          # :128
    offs = [h * R for h in range(H + 1)]
    attention.cache_append(lat_kv[:, 0], mem_index, offs, cache_k.view(cache_k.shape[0], -1), scale_k, "triton")   # :129
    attention.cache_append(lat_kv[:, 1], mem_index, offs, cache_v.view(cache_v.shape[0], -1), scale_v, "triton")   # :130
    o = attention.decode_rope_recon(q, cache_k, scale_k, cache_v, scale_v, w["wuk_q"], w["wuk_scale"],
                                    req_to_token, b_req_idx, b_seq_len, theta=theta)        # :132-143
    y = (o.reshape(B, H * R).float() @ w["wuvout"].float()).half()                          # :145
    return (y.float() + xn.float()).half().view(B, 1, -1)
