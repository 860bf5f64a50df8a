"""Latent KV-cache append and int8 latent decode attention on the CPU (test infrastructure).

Cache layout (shared with the CUDA path): one row per cache slot,
``cache_k [N_slots, sum(r_k)] int8`` with head h in columns k_off[h]:k_off[h+1],
``scale_k [N_slots, H] fp16``; the same for V.  With a uniform rank this is the
reference's ``[N_slots, H, R]`` tensor viewed as two-dimensional.
"""
from __future__ import annotations

import math

import torch

from . import quant


def cache_append(latent16, dest_loc, offsets, cache, cache_scale, rounding="torch"):
    """Quantise ``latent16 [T, sum(r)]`` per (token, head) and scatter to rows ``dest_loc``.

    kernels/layer_bench/fd_kernel/destindex_copy_quantize_latent.py:7-50 (one
    program per (token, head): scale, int8 codes, store at Cache[dest_loc[t]]).
    Mutates ``cache`` and ``cache_scale`` in place like the reference.
    """
    q, s = quant.latent_quant_ragged(latent16, offsets, rounding)
    rows = dest_loc.long()
    cache[rows] = q
    cache_scale[rows] = s
    return q, s


def absorb_query(q16, up_k16, k_off):
    """q~[b, k_off[h]+i] = sum_d up_k[k_off[h]+i, d] * q[b, h, d], in fp32.

    ``up_k16 [sum(r_k), D]`` holds the per-head K up-factors (rank rows, head-dim
    columns).  Folding the query into the up-factor turns the per-token score
    q . (B_k^T z_t) into q~ . z_t over the r_k latent entries; the reference
    instead rebuilds each key
    (kernels/layer_bench/fd_kernel/flash_int8_latent_per_head_decoding_rope_stage1.py:138-166).
    """
    B, H, D = q16.shape
    out = torch.zeros(B, k_off[-1], dtype=torch.float32)
    for h in range(H):
        blk = up_k16[k_off[h]:k_off[h + 1]].float()          # [r, D]
        out[:, k_off[h]:k_off[h + 1]] = q16[:, h].float() @ blk.t()
    return out


def _rows(req_to_token, b_req_idx, b_seq_len, b):
    L = int(b_seq_len[b])
    return req_to_token[int(b_req_idx[b]), :L].long()


def decode_absorb(q16, cache_k, scale_k, cache_v, scale_v, up_k16, up_v16, k_off, v_off,
                  req_to_token, b_req_idx, b_seq_len, sm_scale=None, dtype=torch.float64):
    """Rotary-free latent decode attention with an absorbed query and a fused V up-projection.

    score_t = sm_scale * s_k[t] * (z_k[t] . q~),  p = softmax(score),
    o_lat   = sum_t p_t * s_v[t] * z_v[t]          (r_v values per head)
    o       = B_v^T o_lat                           (head_dim values per head)
    Equal, term by term, to reconstructing K = s_k * (z_k B_k) and V = s_v * (z_v B_v)
    and running ordinary attention: the split-sequence / log-sum-exp structure of
    the reference (stage 1 + stage 2) only changes the summation order.
    Returns (o fp16 [B, H, D], o_lat fp32 [B, sum(r_v)]).
    """
    B, H, D = q16.shape
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    qt = absorb_query(q16, up_k16, k_off).to(dtype)
    o = torch.zeros(B, H, D, dtype=dtype)
    o_lat = torch.zeros(B, v_off[-1], dtype=dtype)
    for b in range(B):
        rows = _rows(req_to_token, b_req_idx, b_seq_len, b)
        if rows.numel() == 0:
            continue
        zk = cache_k[rows].to(dtype)
        zv = cache_v[rows].to(dtype)
        sk = scale_k[rows].to(dtype)
        sv = scale_v[rows].to(dtype)
        for h in range(H):
            s = (zk[:, k_off[h]:k_off[h + 1]] @ qt[b, k_off[h]:k_off[h + 1]]) * sk[:, h] * sm_scale
            p = torch.softmax(s, 0)
            ol = (p * sv[:, h]) @ zv[:, v_off[h]:v_off[h + 1]]
            o_lat[b, v_off[h]:v_off[h + 1]] = ol
            o[b, h] = ol @ up_v16[v_off[h]:v_off[h + 1]].to(dtype)
    return o.to(torch.float16), o_lat.float()


def decode_reconstruct(q16, cache_k, scale_k, cache_v, scale_v, up_k16, k_off, v_off,
                       req_to_token, b_req_idx, b_seq_len, sm_scale=None):
    """The same attention written the long way round (keys rebuilt, no absorption, no rotary).

    Used only to check ``decode_absorb``: K_t = s_k[t] * (z_k[t] B_k), score = q . K_t.
    Returns o_lat fp32 [B, sum(r_v)].
    """
    B, H, D = q16.shape
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    o_lat = torch.zeros(B, v_off[-1], dtype=torch.float64)
    for b in range(B):
        rows = _rows(req_to_token, b_req_idx, b_seq_len, b)
        if rows.numel() == 0:
            continue
        for h in range(H):
            K = (cache_k[rows, k_off[h]:k_off[h + 1]].double() @ up_k16[k_off[h]:k_off[h + 1]].double())
            K = K * scale_k[rows, h].double()[:, None]
            p = torch.softmax((K @ q16[b, h].double()) * sm_scale, 0)
            V = cache_v[rows, v_off[h]:v_off[h + 1]].double() * scale_v[rows, h].double()[:, None]
            o_lat[b, v_off[h]:v_off[h + 1]] = p @ V
    return o_lat.float()


def decode_rope_recon(q16, cache_k, scale_k, cache_v, scale_v, wk_q, wk_scale16,
                      req_to_token, b_req_idx, b_seq_len, theta=10000.0, gqa_group=1):
    """The reference's decode attention: int8 K up-factor, keys rebuilt and rotated per token.

    Follows kernels/layer_bench/fd_kernel/flash_int8_latent_per_head_decoding_rope_stage1.py:55-194
    and flash_latent_per_head_decoding_stage2.py:19-47 with uniform ranks:
      * the query is rotated at position L-1 in fp32 and rounded to fp16 (:78-85);
      * K_t = fp16((z_k[t] . W_uk int8) * s_k[t] * s_w) per output column (:138-150);
      * cos / sin at the logical position t are rounded to fp16 (:153-156), pairs
        are (i, i + D/2) and the angle is t / theta**(2i/D) (:9-14);
      * score = (q_rot . K_rot) / sqrt(D) (:162-166); softmax; o_lat = sum p * s_v * z_v.
    fp16 roundings are applied where the kernel casts; products in between are
    kept in fp32.  The split into sequence blocks and their merge only reorder the
    sum and are not reproduced.
    Shapes: cache_* ``[N, H_kv, R]`` int8, scale_* ``[N, H_kv]`` fp16, wk_q
    ``[R_k, H_kv*D]`` int8, wk_scale16 ``[1, H_kv*D]`` fp16.  Returns fp16 ``[B, H, R_v]``.
    """
    B, H, D = q16.shape
    D2 = D // 2
    Rv = cache_v.shape[-1]
    inv = theta ** (torch.arange(0, D2, dtype=torch.float32) * 2 / D)      # "inv_freq" of the kernel: a divisor
    sm_scale = 1.0 / math.sqrt(D)
    out = torch.zeros(B, H, Rv, dtype=torch.float32)
    for b in range(B):
        rows = _rows(req_to_token, b_req_idx, b_seq_len, b)
        L = rows.numel()
        if L == 0:
            continue
        pos = torch.arange(L, dtype=torch.float32)
        ang = pos[:, None] / inv[None, :]
        cos = ang.cos().half().float()
        sin = ang.sin().half().float()
        qang = float(L - 1) / inv
        qc, qs = qang.cos(), qang.sin()
        for h in range(H):
            hk = h // gqa_group
            q0, q1 = q16[b, h, :D2].float(), q16[b, h, D2:].float()
            q0r = (q0 * qc - q1 * qs).half().float()
            q1r = (q1 * qc + q0 * qs).half().float()
            acc = cache_k[rows, hk].float() @ wk_q[:, hk * D:(hk + 1) * D].float()       # exact: |acc| < 2**24
            k = (acc * scale_k[rows, hk].float()[:, None] * wk_scale16[0, hk * D:(hk + 1) * D].float()[None, :])
            k = k.half().float()
            k0, k1 = k[:, :D2], k[:, D2:]
            k0r = k0 * cos - k1 * sin
            k1r = k1 * cos + k0 * sin
            s = (k0r @ q0r + k1r @ q1r) * sm_scale
            p = torch.softmax(s, 0)
            v = cache_v[rows, hk].float() * scale_v[rows, hk].float()[:, None]
            out[b, h] = p @ v
    return out.half()
