"""Tensor-parallel sharding on the CPU: two gloo ranks run the oracle's sharded layer and must agree with the
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
from lsvd_b200.parallel import partition_heads, channel_slices, shard_layer
from oracle import layer as olayer, quant


def test_partitions_are_balanced_and_cover_everything():
    kr, vr = synth.ragged_ranks(32, 64, seed=0), synth.ragged_ranks(32, 64, seed=1)
    for world in (1, 2, 4, 8):
        parts = partition_heads(kr, vr, world)
        assert parts[0][0] == 0 and parts[-1][1] == 32 and all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
        loads = [sum(kr[h] + vr[h] for h in range(a, b)) for a, b in parts]
        assert max(loads) <= 1.35 * sum(loads) / world
        sl = channel_slices(5504, world)
        assert sl[0][0] == 0 and sl[-1][1] == 5504 and all((b - a) % 16 == 0 for a, b in sl)
    with pytest.raises(ValueError):
        partition_heads([16], [16], 2)


def _case():
    H, D, rq, hidden = 8, 64, 32, 256
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


def _rank_main(rank, world, port, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        t = _case()
        c = t["c"]
        lw, fw, info = shard_layer(t["w"], t["fw"], t["kr"], t["vr"], t["rq"], world, rank)
        h0, h1 = info["heads"]
        kc, vc = info["k_cols"], info["v_cols"]
        res, st = olayer.decoder_layer_tp_rank(
            t["x"], lw, fw, info, t["D"], t["rq"], world, c["cache_k"][:, kc[0]:kc[1]].contiguous(),
            c["scale_k"][:, h0:h1].contiguous(), c["cache_v"][:, vc[0]:vc[1]].contiguous(),
            c["scale_v"][:, h0:h1].contiguous(), c["req_to_token"], c["b_req_idx"], c["b_seq_len"], t["mem_index"])
        out[rank] = (res, st["down_acc"], st["h_q"])
    finally:
        dist.destroy_process_group()


def test_two_rank_layer_matches_the_unsharded_oracle():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_rank_main, args=(2, port, out), nprocs=2, join=True)
    t = _case()
    c = t["c"]
    ref, rst = olayer.decoder_layer(t["x"], t["w"], t["fw"], t["ko"], t["vo"], t["H"], t["D"], t["rq"], c["cache_k"].clone(),
                                    c["scale_k"].clone(), c["cache_v"].clone(), c["scale_v"].clone(), c["req_to_token"],
                                    c["b_req_idx"], c["b_seq_len"], t["mem_index"])
    r0, r1 = out[0], out[1]
    assert torch.equal(r0[0], r1[0]) and torch.equal(r0[1], r1[1]) and torch.equal(r0[2], r1[2])     # ranks agree bit for bit
    assert rel_to_norm(r0[0].float(), ref.float()) < 2e-3
