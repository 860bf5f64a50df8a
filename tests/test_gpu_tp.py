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
        x = t["x"].cuda()
        res = layer(x, ck, sk, cv, sv, st, stages=stages).clone()
        torch.cuda.synchronize()
        # the same step again on the same tensors: eager, then captured (four graphs between the collectives), then replayed;
        # the step rewrites the same cache rows from the same input, so every repetition must give the same bits
        assert layer.use_graphs
        same = True
        for _ in range(4):
            same = same and torch.equal(layer(x, ck, sk, cv, sv, st), res)
        torch.cuda.synchronize()
        assert len(layer._graphs) == 1
        # the across-heads Hadamard in front of o_proj under head sharding, against the single-GPU kernel on the whole row
        from conftest import load_golden
        from lsvd_b200.ffn import heads_hadamard_quant
        from lsvd_b200.parallel import partition_heads, tp_heads_hadamard_quant
        had_ok = True
        for Hh, hk in ((32, None), (28, load_golden("partial_hadamard")["had28"].float())):
            D = 16
            xf = torch.randn(6, Hh * D, generator=torch.Generator().manual_seed(8)).half().cuda()
            heads = partition_heads([64] * Hh, [64] * Hh, world)[rank]
            x_loc = torch.cat([xf[:, h * D:(h + 1) * D] for h in heads], dim=1).contiguous()
            q, s, rot = tp_heads_hadamard_quant(x_loc, heads, Hh, had_K=hk)
            q1, s1, rot1 = heads_hadamard_quant(xf, Hh, want_rotated=True, had_K=hk)
            d = (rot.float() - rot1.float()).abs()
            had_ok = had_ok and bool((d <= rot1.float().abs() * 2.0 ** -10 + 1e-6).all())
            had_ok = had_ok and bool(((q.int() - q1.int()).abs() <= 1).all()) and bool(((s - s1).abs() <= 1e-3 * s1).all())
            if hk is None:
                had_ok = had_ok and float((d == 0).float().mean()) > 0.99
        out[rank] = (res.cpu(), stages["down_acc"].cpu(), stages["h_q"].cpu(), same, had_ok)
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
    assert r0[3] and r1[3]
    assert r0[4] and r1[4]
    assert rel_to_norm(r0[0].float(), ref.float()) < 2e-3


def test_gather_segments_lays_out_the_gathered_hidden_vector():
    """lsvd_gather_segments on one GPU: the [rank][token][svd slice | rtn slice] pieces of a 4-way split into rows in the
    global [SVD | RTN] order, against the index table of ``gather_plan``; and its argument checks."""
    import ctypes as C
    from lsvd_b200 import _lib
    from lsvd_b200.parallel import channel_slices, gather_plan
    world, B, n_svd, n_q = 4, 5, 6912, 6912
    info = dict(n_svd=n_svd, n_q=n_q)
    widest, idx = gather_plan(info, world)
    recv = torch.randn(world * B, widest, generator=torch.Generator().manual_seed(1)).half().cuda()
    want = recv.view(world, B, widest).permute(1, 0, 2).reshape(B, world * widest).index_select(1, idx.cuda())
    src_off, src_stride, dst_off, length = [], [], [], []
    for rk, (sv, rt) in enumerate(zip(channel_slices(n_svd, world), channel_slices(n_q, world))):
        for first, (c0, c1), base in ((0, sv, 0), (sv[1] - sv[0], rt, n_svd)):
            src_off.append((rk * B * widest + first) * 2)
            src_stride.append(widest * 2)
            dst_off.append((base + c0) * 2)
            length.append((c1 - c0) * 2)
    n = len(length)
    out = torch.zeros(B, n_svd + n_q, dtype=torch.float16, device="cuda")
    tabs = ((C.c_int64 * n)(*src_off), (C.c_int64 * n)(*src_stride), (C.c_int64 * n)(*dst_off), (C.c_int32 * n)(*length))
    lib = _lib.load()
    rc = lib.lsvd_gather_segments(recv.data_ptr(), out.data_ptr(), out.stride(0) * 2, B, n, *tabs, None)
    torch.cuda.synchronize()
    assert rc == 0 and torch.equal(out, want)
    bad = (C.c_int32 * n)(*([length[0] + 2] + length[1:]))           # not a multiple of 16 bytes
    assert lib.lsvd_gather_segments(recv.data_ptr(), out.data_ptr(), out.stride(0) * 2, B, n, tabs[0], tabs[1], tabs[2], bad, None) == 1
    assert lib.lsvd_gather_segments(recv.data_ptr(), out.data_ptr(), out.stride(0) * 2, B, 33, *tabs, None) == 1
