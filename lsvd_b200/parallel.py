"""Tensor-parallel sharding of the W8A8 decoder layer across the GPUs of one node (one process per GPU).

The reference has no tensor parallelism.  The layer shards by independent units with one sum per block:

  attention block   heads are dealt to the ranks by latent bytes (largest first, each to the lightest rank); a rank
                    owns its heads' rows of the latent projection, their K/V cache columns, their query/K factors and
                    the matching input columns of the fused output projection, which makes that projection
                    row-parallel: ONE all-reduce (sum, fp32 [B, hidden]) per block.
  FFN block         the intermediate channels of both branches are split over the ranks (column-parallel
                    gate/up; the small latent factors U are replicated so that every rank quantises the same
                    latents).  The d_ffn Hadamard and the per-token absmax couple all channels, so the fp16
                    hidden vector is all-gathered ([B, d_ffn] fp16), rotated and quantised identically on every
                    rank, and the down projection runs row-parallel on the rank's channel columns with an
                    all-reduce of the int32 accumulators: integer sums are exact, so the FFN output does not
                    depend on the number of GPUs.

Collectives go through ``torch.distributed`` (NCCL over NVLink on GPUs, gloo in the CPU tests) on whole
buffers in the GPU's own memory; no kernel here reads a peer's memory.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch


def partition_heads(k_ranks: Sequence[int], v_ranks: Sequence[int], world: int) -> List[List[int]]:
    """Heads of every rank (ascending), balanced by latent bytes r_k + r_v: the heaviest head first, each to the rank
    that is lightest so far (ties: fewer heads, then the lower rank).  Every rank gets at least one head."""
    H = len(k_ranks)
    if world < 1 or world > H:
        raise ValueError("need 1 <= world <= number of heads")
    cost = [a + b for a, b in zip(k_ranks, v_ranks)]
    order = sorted(range(H), key=lambda h: (-cost[h], h))
    load, heads = [0] * world, [[] for _ in range(world)]
    for h in order:
        r = min(range(world), key=lambda i: (load[i], len(heads[i]), i))
        heads[r].append(h)
        load[r] += cost[h]
    return [sorted(hs) for hs in heads]


def channel_slices(n: int, world: int) -> List[Tuple[int, int]]:
    """Split n channels (a multiple of 16) into `world` contiguous slices whose sizes are multiples of 16."""
    if n % 16:
        raise ValueError("channel count must be a multiple of 16")
    units = n // 16
    out, start = [], 0
    for r in range(world):
        size = (units // world + (1 if r < units % world else 0)) * 16
        out.append((start, start + size))
        start += size
    return out


def _off(ranks):
    o = [0]
    for r in ranks:
        o.append(o[-1] + r)
    return o


def _cols(off, heads):
    return torch.cat([torch.arange(off[h], off[h + 1]) for h in heads])


def shard_layer(w: dict, ffn_w: dict, k_ranks, v_ranks, rank_q: int, world: int, rank: int):
    """Local weights of `rank`.  Returns (layer dict, ffn dict, info) with info = the rank's heads, their local rank
    lists, the columns of the unsharded K / V cache rows they occupy (index tensors) and the rank's channel slices.
    The down projection's local input columns are one matrix ``Wd_loc_q [d_out, svd slice | rtn slice]``."""
    H = len(k_ranks)
    heads = partition_heads(k_ranks, v_ranks, world)[rank]
    ko, vo = _off(k_ranks), _off(v_ranks)
    Rq, Rk = H * rank_q, ko[-1]
    k_cols, v_cols = _cols(ko, heads), _cols(vo, heads)
    q_rows = torch.cat([torch.arange(h * rank_q, (h + 1) * rank_q) for h in heads])
    rows = torch.cat([q_rows, Rq + k_cols, Rq + Rk + v_cols])
    lw = {"ln1": w["ln1"], "ln2": w["ln2"], "W_lat_q": w["W_lat_q"][rows].contiguous(), "W_lat_s": w["W_lat_s"][rows].contiguous(),
          "C": w["C"][k_cols].contiguous(), "W_uvo_q": w["W_uvo_q"][:, v_cols].contiguous(), "W_uvo_s": w["W_uvo_s"]}
    n_svd, n_q = ffn_w["Vg_q"].shape[0], ffn_w["Wg_q"].shape[0]
    s0, s1 = channel_slices(n_svd, world)[rank]
    q0, q1 = channel_slices(n_q, world)[rank]
    fw = dict(ffn_w)
    for name in ("Vg", "Vu"):
        fw[name + "_q"], fw[name + "_s"] = ffn_w[name + "_q"][s0:s1].contiguous(), ffn_w[name + "_s"][s0:s1].contiguous()
    for name in ("Wg", "Wu"):
        fw[name + "_q"], fw[name + "_s"] = ffn_w[name + "_q"][q0:q1].contiguous(), ffn_w[name + "_s"][q0:q1].contiguous()
    fw["Wd_loc_q"] = torch.cat([ffn_w["Wd_q"][:, s0:s1], ffn_w["Wd_q"][:, n_svd + q0:n_svd + q1]], dim=1).contiguous()
    fw.pop("Wd_q", None)
    info = dict(heads=heads, k_ranks=[k_ranks[h] for h in heads], v_ranks=[v_ranks[h] for h in heads], k_cols=k_cols,
                v_cols=v_cols, svd=(s0, s1), rtn=(q0, q1), n_svd=n_svd, n_q=n_q)
    return lw, fw, info


def gather_plan(info: dict, world: int, device=None):
    """(widest, index): every rank sends ``[B, widest]`` (its SVD slice, then its RTN slice, zero padded); the gathered
    ``[world, B, widest]`` buffer seen as ``[B, world * widest]`` gives the hidden vector in the global [SVD | RTN] order
    through ``index`` (one index_select)."""
    n_svd, n_q = info["n_svd"], info["n_q"]
    svd_sl, rtn_sl = channel_slices(n_svd, world), channel_slices(n_q, world)
    widest = max((a[1] - a[0]) + (b[1] - b[0]) for a, b in zip(svd_sl, rtn_sl))
    idx = torch.empty(n_svd + n_q, dtype=torch.int64)
    for r in range(world):
        ns = svd_sl[r][1] - svd_sl[r][0]
        nr = rtn_sl[r][1] - rtn_sl[r][0]
        idx[svd_sl[r][0]:svd_sl[r][1]] = r * widest + torch.arange(ns)
        idx[n_svd + rtn_sl[r][0]:n_svd + rtn_sl[r][1]] = r * widest + ns + torch.arange(nr)
    return widest, (idx if device is None else idx.to(device))


def gather_hidden(h_local: torch.Tensor, info: dict, world: int, group=None, plan=None, send=None, recv=None) -> torch.Tensor:
    """All-gather the ranks' [B, svd slice | rtn slice] pieces and lay them out in the global [SVD | RTN] order:
    one collective into a preallocated buffer, one index_select.  ``send [B, widest]`` must have its padding columns zero."""
    import torch.distributed as dist
    B = h_local.shape[0]
    widest, idx = plan if plan is not None else gather_plan(info, world, h_local.device)
    if send is None:
        send = h_local.new_zeros(B, widest)
    if send.data_ptr() != h_local.data_ptr():
        send[:, :h_local.shape[1]].copy_(h_local)
    if recv is None:
        recv = h_local.new_empty(world * B, widest)            # rank r's rows at r * B ..
    dist.all_gather_into_tensor(recv, send, group=group)
    return recv.view(world, B, widest).permute(1, 0, 2).reshape(B, world * widest).index_select(1, idx)


def tp_heads_hadamard_quant(x_local: torch.Tensor, head_ids, num_heads: int, group=None, had_K: Optional[torch.Tensor] = None,
                            partial: Optional[torch.Tensor] = None):
    """The Hadamard across heads + per-token int8 quantisation in front of ``o_proj`` (``ActQuantWrapper`` with
    ``online_partial_had``, fake_quant/utils/quant_utils.py:302-322) when the heads are sharded: ``x_local
    [rows, len(head_ids) * head_dim]`` fp16 holds this rank's heads (global indices ``head_ids``).  Every rank adds its heads'
    terms of all ``num_heads`` output heads into an fp32 row (``lsvd_heads_hadamard_partial``), ONE all-reduce sums the
    rows, and the quantiser rounds the sum to fp16 once.  Returns (codes int8 [rows, num_heads * head_dim], scale fp32
    [rows], rotated fp16): the same on every rank; a row-parallel ``o_proj`` then multiplies its own columns of the codes."""
    import ctypes as C
    import torch.distributed as dist
    from . import _lib
    from .attention import _require_cuda, _stream_ptr
    from .ffn import act_quant
    _require_cuda(x_local)
    n_local = len(head_ids)
    rows, cols = x_local.shape
    if x_local.dtype != torch.float16 or x_local.stride(1) != 1 or n_local == 0 or cols % n_local:
        raise ValueError("x_local must be fp16 [rows, len(head_ids) * head_dim] with unit inner stride")
    head_dim = cols // n_local
    if partial is None:
        partial = torch.empty(rows, num_heads * head_dim, dtype=torch.float32, device=x_local.device)
    hk = None if had_K is None else had_K.to(device=x_local.device, dtype=torch.float16).contiguous()
    ids = (C.c_int32 * n_local)(*[int(h) for h in head_ids])
    _lib.check(_lib.load().lsvd_heads_hadamard_partial(x_local.data_ptr(), x_local.stride(0), ids, n_local, num_heads, head_dim,
                                                      None if hk is None else hk.data_ptr(), partial.data_ptr(), rows,
                                                      _stream_ptr(x_local)))
    dist.all_reduce(partial, group=group)
    rot = torch.empty(rows, num_heads * head_dim, dtype=torch.float16, device=x_local.device)
    q, s, _ = act_quant(None, x_f32=partial, sum_out=rot)
    return q, s, rot
