"""Tensor-parallel sharding of the W8A8 decoder layer across the GPUs of one node (one process per GPU).

The reference has no tensor parallelism.  The layer shards by independent units with one sum per block:

  attention block   heads are split over the ranks (contiguous runs balanced by latent bytes); a rank owns its
                    heads' rows of the latent projection, their K/V cache columns, their query/K factors and
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

from typing import List, Sequence, Tuple

import torch


def partition_heads(k_ranks: Sequence[int], v_ranks: Sequence[int], world: int) -> List[Tuple[int, int]]:
    """Contiguous head ranges [h0, h1) per rank, balanced by latent bytes (r_k + r_v), every rank non-empty."""
    H = len(k_ranks)
    if world < 1 or world > H:
        raise ValueError("need 1 <= world <= number of heads")
    cost = [a + b for a, b in zip(k_ranks, v_ranks)]
    total = sum(cost)
    bounds, acc, h = [0], 0, 0
    for r in range(1, world):
        target = total * r / world
        while h < H - (world - r) and acc + cost[h] / 2 < target:
            acc += cost[h]
            h += 1
        h = max(h, bounds[-1] + 1)
        bounds.append(h)
        acc = sum(cost[:h])
    bounds.append(H)
    return [(bounds[i], bounds[i + 1]) for i in range(world)]


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


def shard_layer(w: dict, ffn_w: dict, k_ranks, v_ranks, rank_q: int, world: int, rank: int):
    """Local weights of `rank`.  Returns (layer dict, ffn dict, info) with info = head range, local rank lists,
    cache column ranges and the rank's channel slices."""
    H = len(k_ranks)
    h0, h1 = partition_heads(k_ranks, v_ranks, world)[rank]
    ko, vo = _off(k_ranks), _off(v_ranks)
    Rq, Rk = H * rank_q, ko[-1]
    rows = torch.cat([torch.arange(h0 * rank_q, h1 * rank_q), Rq + torch.arange(ko[h0], ko[h1]),
                      Rq + Rk + torch.arange(vo[h0], vo[h1])])
    lw = {"ln1": w["ln1"], "ln2": w["ln2"], "W_lat_q": w["W_lat_q"][rows].contiguous(), "W_lat_s": w["W_lat_s"][rows].contiguous(),
          "C": w["C"][ko[h0]:ko[h1]].contiguous(), "W_uvo_q": w["W_uvo_q"][:, vo[h0]:vo[h1]].contiguous(), "W_uvo_s": w["W_uvo_s"]}
    n_svd, n_q = ffn_w["Vg_q"].shape[0], ffn_w["Wg_q"].shape[0]
    s0, s1 = channel_slices(n_svd, world)[rank]
    q0, q1 = channel_slices(n_q, world)[rank]
    fw = dict(ffn_w)
    for name in ("Vg", "Vu"):
        fw[name + "_q"], fw[name + "_s"] = ffn_w[name + "_q"][s0:s1].contiguous(), ffn_w[name + "_s"][s0:s1].contiguous()
    for name in ("Wg", "Wu"):
        fw[name + "_q"], fw[name + "_s"] = ffn_w[name + "_q"][q0:q1].contiguous(), ffn_w[name + "_s"][q0:q1].contiguous()
    fw["Wd_svd_q"] = ffn_w["Wd_q"][:, s0:s1].contiguous()
    fw["Wd_rtn_q"] = ffn_w["Wd_q"][:, n_svd + q0:n_svd + q1].contiguous()
    info = dict(heads=(h0, h1), k_ranks=list(k_ranks[h0:h1]), v_ranks=list(v_ranks[h0:h1]), k_cols=(ko[h0], ko[h1]),
                v_cols=(vo[h0], vo[h1]), svd=(s0, s1), rtn=(q0, q1), n_svd=n_svd, n_q=n_q)
    return lw, fw, info


def gather_hidden(h_local: torch.Tensor, info: dict, world: int, group=None) -> torch.Tensor:
    """All-gather the ranks' [B, svd slice | rtn slice] pieces and lay them out in the global [SVD | RTN] order."""
    import torch.distributed as dist
    B = h_local.shape[0]
    n_svd, n_q = info["n_svd"], info["n_q"]
    svd_sl, rtn_sl = channel_slices(n_svd, world), channel_slices(n_q, world)
    widest = max((a[1] - a[0]) + (b[1] - b[0]) for a, b in zip(svd_sl, rtn_sl))
    send = h_local.new_zeros(B, widest)
    send[:, :h_local.shape[1]] = h_local
    parts = [torch.empty_like(send) for _ in range(world)]
    dist.all_gather(parts, send, group=group)
    full = h_local.new_empty(B, n_svd + n_q)
    for r in range(world):
        ns = svd_sl[r][1] - svd_sl[r][0]
        nr = rtn_sl[r][1] - rtn_sl[r][0]
        full[:, svd_sl[r][0]:svd_sl[r][1]] = parts[r][:, :ns]
        full[:, n_svd + rtn_sl[r][0]:n_svd + rtn_sl[r][1]] = parts[r][:, ns:ns + nr]
    return full
