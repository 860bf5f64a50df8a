"""Tensor-parallel sharding on the CPU: gloo ranks run the oracle's sharded layer and must agree with the
unsharded oracle layer (host-side sharding logic and collectives; no GPU involved)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import load_golden, unpack_had, rel_to_norm
from lsvd_b200 import synth
from lsvd_b200.layer import make_layer_weights
from lsvd_b200.parallel import partition_heads, channel_slices, shard_layer, gather_plan
from oracle import layer as olayer, quant


def test_partitions_are_balanced_and_cover_everything():
    for H in (32, 40):
        kr, vr = synth.ragged_ranks(H, 64, seed=0), synth.ragged_ranks(H, 64, seed=1)
        for world in (1, 2, 4, 8):
            parts = partition_heads(kr, vr, world)
            assert sorted(h for p in parts for h in p) == list(range(H)) and all(p == sorted(p) and p for p in parts)
            loads = [sum(kr[h] + vr[h] for h in p) for p in parts]
            assert max(loads) <= 1.10 * sum(loads) / world, (H, world, loads)      # by bytes, not by count
            sl = channel_slices(5504, world)
            assert sl[0][0] == 0 and sl[-1][1] == 5504 and all((b - a) % 16 == 0 for a, b in sl)
    with pytest.raises(ValueError):
        partition_heads([16], [16], 2)


def test_gather_plan_restores_the_global_channel_order():
    info = dict(n_svd=96, n_q=160)
    for world in (2, 4):
        widest, idx = gather_plan(info, world)
        svd, rtn = channel_slices(96, world), channel_slices(160, world)
        full = torch.arange(256.0)[None]
        recv = torch.zeros(world, 1, widest)
        for r in range(world):
            piece = torch.cat((full[:, svd[r][0]:svd[r][1]], full[:, 96 + rtn[r][0]:96 + rtn[r][1]]), dim=1)
            recv[r, :, :piece.shape[1]] = piece
        assert torch.equal(recv.permute(1, 0, 2).reshape(1, world * widest).index_select(1, idx), full)


def _case(H=8):
    """H = 8: the smallest case; H = 40: the head count of BASELINE config 4 (13B shape) at reduced widths."""
    D, rq = 64, 32
    hidden = 256 if H == 8 else 320
    kr, vr = synth.ragged_ranks(H, 32, lo=16, hi=64, seed=5), synth.ragged_ranks(H, 32, lo=16, hi=64, seed=6)
    w = make_layer_weights(hidden, H, D, rq, kr, vr, seed=1)
    hk = unpack_had(load_golden("hadamard")["had172_bits"], 172)
    fw = synth.ffn_weights(hidden, 172 * 8, 64, 688, seed=2, had_K=hk, K=172, input_had=False, std=0.05)
    B, lens = 2, [40, 17]
    c = synth.attention_inputs(B, H, D, kr, vr, lens, seed=9)
    ko, vo = [0], [0]
    for a, b in zip(kr, vr):
        ko.append(ko[-1] + a)
        vo.append(vo[-1] + b)
    c["cache_k"], c["scale_k"] = quant.latent_quant_ragged(c["latent_k"], ko)
    c["cache_v"], c["scale_v"] = quant.latent_quant_ragged(c["latent_v"], vo)
    x = torch.randn(B, hidden, generator=torch.Generator().manual_seed(3)).half()
    mem_index = c["req_to_token"][torch.arange(B), torch.tensor(lens) - 1]
    return dict(H=H, D=D, rq=rq, kr=kr, vr=vr, w=w, fw=fw, c=c, x=x, ko=ko, vo=vo, mem_index=mem_index)


def local_cache(c, info):
    """The rank's columns of the unsharded cache rows and its heads' scales."""
    heads = torch.tensor(info["heads"])
    return (c["cache_k"][:, info["k_cols"]].contiguous(), c["scale_k"][:, heads].contiguous(),
            c["cache_v"][:, info["v_cols"]].contiguous(), c["scale_v"][:, heads].contiguous())


def _rank_main(rank, world, port, out, H):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        t = _case(H)
        c = t["c"]
        lw, fw, info = shard_layer(t["w"], t["fw"], t["kr"], t["vr"], t["rq"], world, rank)
        ck, sk, cv, sv = local_cache(c, info)
        res, st = olayer.decoder_layer_tp_rank(t["x"], lw, fw, info, t["D"], t["rq"], world, ck, sk, cv, sv, c["req_to_token"],
                                               c["b_req_idx"], c["b_seq_len"], t["mem_index"])
        out[rank] = (res, st["down_acc"], st["h_q"])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,H", [(2, 8), (4, 40), (8, 40)])
def test_sharded_layer_matches_the_unsharded_oracle(world, H):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_rank_main, args=(world, port, out, H), nprocs=world, join=True)
    t = _case(H)
    c = t["c"]
    ref, rst = olayer.decoder_layer(t["x"], t["w"], t["fw"], t["ko"], t["vo"], t["H"], t["D"], t["rq"], c["cache_k"].clone(),
                                    c["scale_k"].clone(), c["cache_v"].clone(), c["scale_v"].clone(), c["req_to_token"],
                                    c["b_req_idx"], c["b_seq_len"], t["mem_index"])
    for r in range(1, world):        # ranks agree bit for bit: output, int32 accumulators, quantised hidden vector
        assert torch.equal(out[0][0], out[r][0]) and torch.equal(out[0][1], out[r][1]) and torch.equal(out[0][2], out[r][2])
    assert rel_to_norm(out[0][0].float(), ref.float()) < 2e-3


def _had_rank_main(rank, world, port, out, H, with_hadk):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import ffn as offn
        from lsvd_b200.parallel import partition_heads
        D = 16
        x = torch.randn(5, H * D, generator=torch.Generator().manual_seed(4)).half()
        heads = partition_heads([64] * H, [64] * H, world)[rank]
        x_local = torch.cat([x[:, h * D:(h + 1) * D] for h in heads], dim=1)
        hk = load_golden("partial_hadamard")["had28"].float() if with_hadk else None
        terms = offn.partial_hadamard_heads_terms(x_local, heads, H, hk)
        dist.all_reduce(terms)
        out[rank] = terms.half()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,H,with_hadk", [(2, 32, False), (4, 32, False), (2, 28, True)])
def test_heads_hadamard_under_head_sharding(world, H, with_hadk):
    """The across-heads Hadamard in front of o_proj when every rank holds only its own heads: each rank's terms summed by
    one all-reduce give the single-process rotation (fake_quant/utils/quant_utils.py:302-317)."""
    from oracle import ffn as offn
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_had_rank_main, args=(world, port, out, H, with_hadk), nprocs=world, join=True)
    x = torch.randn(5, H * 16, generator=torch.Generator().manual_seed(4)).half()
    if with_hadk:
        ref = offn.partial_hadamard_heads_hadk(x, 16, load_golden("partial_hadamard")["had28"].float())
    else:
        ref = offn.partial_hadamard_heads(x, 16)
    for r in range(world):
        assert torch.equal(out[r], out[0])
        d = (out[r].float() - ref.float()).abs()
        assert (d <= ref.float().abs() * 2.0 ** -10 + 1e-6).all()      # one fp16 rounding (the reference rounds twice with had_K)
        assert (d == 0).float().mean() > (0.6 if with_hadk else 0.9)
