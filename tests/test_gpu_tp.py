"""Tensor-parallel decoder layer on two GPUs (NCCL) against the single-GPU layer.  Skipped with fewer than two GPUs."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from conftest import rel_to_norm

pytestmark = pytest.mark.gpu


def _rank_main(rank, world, port, out):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from test_tp_cpu import _case, local_cache
        from lsvd_b200.attention import InferState
        from lsvd_b200.layer import TPDecoderLayer
        from lsvd_b200.parallel import shard_layer
        t = _case()
        c = t["c"]
        lw, fw, info = shard_layer(t["w"], t["fw"], t["kr"], t["vr"], t["rq"], world, rank)
        dev = lambda d: {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
        layer = TPDecoderLayer(dev(lw), dev(fw), info, t["D"], t["rq"], world)
        ck, sk, cv, sv = (x.cuda() for x in local_cache(c, info))
        st = InferState(2, c["max_len"], c["b_seq_len"], device="cuda")
        stages = {}
        res = layer(t["x"].cuda(), ck, sk, cv, sv, st, stages=stages)
        torch.cuda.synchronize()
        out[rank] = (res.cpu(), stages["down_acc"].cpu(), stages["h_q"].cpu())
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_layer_matches_oracle_and_ranks_agree():
    from test_tp_cpu import _case
    from oracle import layer as olayer
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_rank_main, args=(2, port, out), nprocs=2, join=True)
    t = _case()
    c = t["c"]
    ref, _ = olayer.decoder_layer(t["x"], t["w"], t["fw"], t["ko"], t["vo"], t["H"], t["D"], t["rq"], c["cache_k"].clone(),
                                  c["scale_k"].clone(), c["cache_v"].clone(), c["scale_v"].clone(), c["req_to_token"],
                                  c["b_req_idx"], c["b_seq_len"], t["mem_index"])
    r0, r1 = out[0], out[1]
    assert torch.equal(r0[0], r1[0]) and torch.equal(r0[1], r1[1]) and torch.equal(r0[2], r1[2])
    assert rel_to_norm(r0[0].float(), ref.float()) < 2e-3
