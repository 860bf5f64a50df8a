"""GPU parity of lsvd_b200.block.Int8AttentionBlock (the module that takes the place of the reference's class of that
name): against one decode step of the reference's own module, and against the oracle on a larger seeded case."""
import pytest
import torch

from conftest import load_golden, rel_to_norm
from oracle import layer as olayer, quant
from lsvd_b200.attention import InferState
from lsvd_b200.block import Int8AttentionBlock

pytestmark = pytest.mark.gpu

TOL = 2e-3       # max-abs error of the fp16 output over the 2-norm of the reference output


def load_block(w, H, D, R):
    blk = Int8AttentionBlock(H * D, H, D, (R + 0.5) / D, device="cuda")
    with torch.no_grad():
        for name in ("up_proj_q", "up_proj_k", "up_proj_v", "input_layernorm_weight"):
            getattr(blk, name).copy_(w[name])
        for name in ("down_proj_q", "down_proj_kv", "o_proj"):
            getattr(blk, name).weight.copy_(w[name])
    blk.refresh()
    return blk


def codes_close(a, b, max_off_by_one=0.02):
    """int8 cache rows equal up to a small share of one-step differences (an fp16 latent that a library GEMM rounds
    the other way can move a code by one)."""
    d = (a.int() - b.int()).abs()
    return int(d.max()) <= 1 and float((d > 0).float().mean()) <= max_off_by_one


def test_one_decode_step_of_the_reference_module():
    g = load_golden("attention_block")
    H, D, R = g["num_heads"], g["head_dim"], g["rank_head"]
    blk = load_block(g, H, D, R)
    assert torch.equal(blk.wuk_q.cpu(), g["wuk_q"]) and torch.equal(blk.wuk_scale.cpu(), g["wuk_scale"])
    B = g["x"].shape[0]
    st = InferState(B, g["req_to_token"].shape[1], g["b_seq_len"], req_to_token=g["req_to_token"], b_req_idx=g["b_req_idx"])
    assert torch.equal(st.mem_index.cpu(), g["mem_index"])
    ck, sk, cv, sv = (g[k].cuda() for k in ("cache_k", "scale_k", "cache_v", "scale_v"))
    y = blk(g["x"].cuda(), ck, sk, cv, sv, st)
    torch.cuda.synchronize()
    assert y.shape == g["y"].shape
    assert rel_to_norm(y.cpu().float(), g["y"].float()) < TOL
    rows = g["mem_index"].long()
    rest = torch.ones(ck.shape[0], dtype=torch.bool)
    rest[rows] = False
    for got, want, before in ((ck, "cache_k_after", "cache_k"), (cv, "cache_v_after", "cache_v")):
        assert torch.equal(got.cpu()[rest], g[before][rest])            # only the step's rows are written
        assert codes_close(got.cpu()[rows], g[want][rows])
    assert (sk.cpu()[rows].float() - g["scale_k_after"][rows].float()).abs().max() <= 2e-3 * g["scale_k_after"][rows].float().abs().max()
    assert (sv.cpu()[rows].float() - g["scale_v_after"][rows].float()).abs().max() <= 2e-3 * g["scale_v_after"][rows].float().abs().max()


def test_7b_head_shape_against_the_oracle():
    """hidden 1024 = 8 heads x 128, rank 64, ragged batch, shuffled slots; two consecutive steps on the same cache."""
    torch.manual_seed(3)
    H, D = 8, 128
    blk = Int8AttentionBlock(H * D, H, D, 0.5, device="cuda")
    with torch.no_grad():
        blk.input_layernorm_weight.copy_(1 + 0.1 * torch.randn(H * D))
    R = blk.rank_head
    gen = torch.Generator().manual_seed(4)
    lens = [300, 1, 77, 256]
    B, S = len(lens), max(lens) + 1
    N = B * S + 11
    ck, sk = quant.latent_quant(torch.randn(N, H, R, generator=gen).half())
    cv, sv = quant.latent_quant(torch.randn(N, H, R, generator=gen).half())
    r2t = torch.randperm(N, generator=gen)[:B * S].to(torch.int32).view(B, S)
    w = {k: v.detach().cpu() for k, v in blk.named_parameters()}
    w = {"down_proj_q": w["down_proj_q.weight"], "down_proj_kv": w["down_proj_kv.weight"], "up_proj_q": w["up_proj_q"],
         "input_layernorm_weight": w["input_layernorm_weight"], "wuk_q": blk.wuk_q.cpu(), "wuk_scale": blk.wuk_scale.cpu(),
         "wuvout": blk.wuvout.cpu()}
    gck, gsk, gcv, gsv = ck.cuda(), sk.cuda(), cv.cuda(), sv.cuda()
    for step in range(2):
        cur = [L + step for L in lens]
        x = torch.randn(B, 1, H * D, generator=gen).half()
        st = InferState(B, S, cur, req_to_token=r2t)
        y = blk(x.cuda(), gck, gsk, gcv, gsv, st)
        torch.cuda.synchronize()
        ref = olayer.int8_attention_block(x, w, ck, sk, cv, sv, r2t, st.b_req_idx.cpu(), st.b_seq_len.cpu(),
                                          st.mem_index.cpu(), H, D)
        assert rel_to_norm(y.cpu().float(), ref.float()) < TOL
        assert codes_close(gck.cpu(), ck) and codes_close(gcv.cpu(), cv)
        # carry the oracle's cache forward so that a one-step code difference does not compound
        gck.copy_(ck); gsk.copy_(sk); gcv.copy_(cv); gsv.copy_(sv)


def test_query_length_above_one_is_refused():
    blk = Int8AttentionBlock(128, 4, 32, 0.5, device="cuda")
    x = torch.zeros(2, 2, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        blk(x, None, None, None, None, None)
