"""The W8A8 decoder layer on the GPU against the oracle's composition of the same stages."""
import pytest
import torch

from conftest import load_golden, unpack_had, rel_to_norm
import gpu_util as U
from oracle import layer as olayer, quant
from lsvd_b200 import synth
from lsvd_b200.attention import LatentCacheLayout, InferState, cache_append, decode_advance
from lsvd_b200.ffn import HybridFFN
from lsvd_b200.layer import LSVDDecoderLayer, make_layer_weights

pytestmark = pytest.mark.gpu


def test_decoder_layer_against_oracle_composition():
    H, D, rq, hidden = 8, 128, 64, 1024
    kr, vr = synth.ragged_ranks(H, 64, seed=5), synth.ragged_ranks(H, 64, seed=6)
    lay = LatentCacheLayout(kr, vr)
    w = make_layer_weights(hidden, H, D, rq, kr, vr, seed=1)
    hk = unpack_had(load_golden("hadamard")["had172_bits"], 172)
    fw = synth.ffn_weights(hidden, 172 * 16, 128, 1376, seed=2, had_K=hk, K=172, input_had=False, std=0.05)
    B, lens = 3, [200, 33, 77]
    c = U.build_case(B, H, D, kr, vr, lens, seed=9)
    st = InferState(B, c["max_len"], lens, device="cuda")
    x = torch.randn(B, hidden, generator=torch.Generator().manual_seed(3)).half()
    dev = lambda d: {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
    layer = LSVDDecoderLayer(lay, D, rq, dev(w), HybridFFN(dev(fw)))
    ck, sk, cv, sv = (c[k].cuda() for k in ("cache_k", "scale_k", "cache_v", "scale_v"))
    stages = {}
    out = layer(x.cuda(), ck, sk, cv, sv, st, stages=stages).cpu()
    ck_ref, sk_ref, cv_ref, sv_ref = (c[k].clone() for k in ("cache_k", "scale_k", "cache_v", "scale_v"))
    ref, rst = olayer.decoder_layer(x, w, fw, lay.k_off, lay.v_off, H, D, rq, ck_ref, sk_ref, cv_ref, sv_ref,
                                    c["req_to_token"], c["b_req_idx"], c["b_seq_len"], st.mem_index.cpu())
    # stages with bit-identical inputs: normalised input, int8 projections, the appended cache rows
    assert torch.equal(stages["xn"].cpu(), rst["xn"])
    assert torch.equal(stages["lat"].cpu(), rst["lat"])
    assert torch.equal(ck.cpu(), ck_ref) and torch.equal(sk.cpu(), sk_ref) and torch.equal(cv.cpu(), cv_ref)
    # attention output and everything after it: fp16 tolerance of the specification
    assert rel_to_norm(stages["o_lat"].cpu().float(), rst["o_lat"].float()) < 2e-3
    assert rel_to_norm(stages["y1"].cpu().float(), rst["y1"].float()) < 2e-3
    assert rel_to_norm(out.float(), ref.float()) < 2e-3


def test_config3_full_size_layer_stage_by_stage():
    """BASELINE config 3 at its real size: hidden 4096, 32 heads x 128, ragged K/V ranks (mean 64), query latents of rank
    64, hybrid FFN 4096 / 11008 (rank 512, half of the channels on the SVD branch, Hadamard 64 x 172), batch 16, context
    4096 + the decoding token.  The integer stages fed identical inputs (normalised input, int8 latent projection, the
    appended cache rows) are bit-exact; what follows the attention is held to 2e-3 * ||ref||_2.  The oracle runs the
    whole layer for a sample of requests (its attention loops over every cached token on the CPU)."""
    H, D, rq, hidden = 32, 128, 64, 4096
    kr, vr = synth.ragged_ranks(H, 64, seed=0), synth.ragged_ranks(H, 64, seed=1)
    w = make_layer_weights(hidden, H, D, rq, kr, vr, seed=70)
    hk = unpack_had(load_golden("hadamard")["had172_bits"], 172)
    fw = synth.ffn_weights(hidden, 11008, 512, 5504, seed=50, had_K=hk, K=172, input_had=False)
    B, L = 16, 4097
    for head_major in (False, True):
        lay = LatentCacheLayout(kr, vr, head_major=head_major)
        c = U.build_case(B, H, D, kr, vr, [L] * B, seed=33)
        st = InferState(B, c["max_len"], [L] * B, device="cuda")
        x = torch.randn(B, hidden, generator=torch.Generator().manual_seed(4)).half()
        dev = lambda d: {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
        layer = LSVDDecoderLayer(lay, D, rq, dev(w), HybridFFN(dev(fw)))
        ck, sk, cv, sv = c["cache_k"], c["scale_k"], c["cache_v"], c["scale_v"]
        if head_major:
            ck, sk = lay.to_head_major(ck, sk, "k")
            cv, sv = lay.to_head_major(cv, sv, "v")
        ck, sk, cv, sv = ck.cuda(), sk.cuda(), cv.cuda(), sv.cuda()
        stages = {}
        out = layer(x.cuda(), ck, sk, cv, sv, st, stages=stages).cpu()
        if head_major:
            ck, sk = lay.from_head_major(ck, sk, "k")
            cv, sv = lay.from_head_major(cv, sv, "v")
        # the oracle on requests 0, 7 and 15: a batch of three with the same slots
        sample = [0, 7, 15]
        ck_ref, sk_ref, cv_ref, sv_ref = (c[k].clone() for k in ("cache_k", "scale_k", "cache_v", "scale_v"))
        # The normalised input: an fp32 mean of 4096 squares depends on the order of the additions, so a few values sit
        # one fp16 step away from the oracle's; the stages behind it are compared from the GPU's own normalised input.
        xn_gpu = stages["xn"].cpu()[sample]
        ref, rst = olayer.decoder_layer(x[sample], w, fw, lay.k_off, lay.v_off, H, D, rq, ck_ref, sk_ref, cv_ref, sv_ref,
                                        c["req_to_token"], c["b_req_idx"][sample], c["b_seq_len"][sample],
                                        st.mem_index.cpu()[sample], xn=xn_gpu)
        diff = (xn_gpu.float() - rst["xn"].float()).abs()
        assert (diff > 0).float().mean() < 2e-3 and (diff <= rst["xn"].float().abs() * 2 ** -10 + 1e-7).all()
        assert torch.equal(stages["lat"].cpu()[sample], rst["lat"])
        rows = st.mem_index.cpu()[sample].long()
        assert torch.equal(ck.cpu()[rows], ck_ref[rows]) and torch.equal(sk.cpu()[rows], sk_ref[rows])
        assert torch.equal(cv.cpu()[rows], cv_ref[rows]) and torch.equal(sv.cpu()[rows], sv_ref[rows])
        assert rel_to_norm(stages["o_lat"].cpu()[sample].float(), rst["o_lat"].float()) < 2e-3
        assert rel_to_norm(stages["y1"].cpu()[sample].float(), rst["y1"].float()) < 2e-3
        assert rel_to_norm(out[sample].float(), ref.float()) < 2e-3


@pytest.mark.parametrize("head_major", [False, True])
def test_multi_step_decode_cache_rows_and_last_output(head_major):
    """Ten consecutive decode steps: the lengths and the slot of the new token advance ON THE DEVICE
    (lsvd_decode_advance), a row appended at step t is attended from step t on.  After the last step every appended
    cache row equals the oracle's bit for bit and the last output is inside the tolerance."""
    H, D, rq, hidden, steps = 8, 128, 64, 1024, 10
    kr, vr = synth.ragged_ranks(H, 64, seed=5), synth.ragged_ranks(H, 64, seed=6)
    lay = LatentCacheLayout(kr, vr, head_major=head_major)
    w = make_layer_weights(hidden, H, D, rq, kr, vr, seed=1)
    hk = unpack_had(load_golden("hadamard")["had172_bits"], 172)
    fw = synth.ffn_weights(hidden, 172 * 16, 128, 1376, seed=2, had_K=hk, K=172, input_had=False, std=0.05)
    B, lens = 3, [200, 33, 77]
    cap = max(lens) + steps                         # slots reserved per request
    c = U.build_case(B, H, D, kr, vr, [cap] * B, seed=9)          # latents for every reserved slot; only `lens` are "cached"
    c["b_seq_len"] = torch.tensor(lens, dtype=torch.int32)
    st = InferState(B, cap, lens, device="cuda", req_to_token=c["req_to_token"])
    gen = torch.Generator().manual_seed(3)
    xs = [torch.randn(B, hidden, generator=gen).half() for _ in range(steps)]
    dev = lambda d: {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
    layer = LSVDDecoderLayer(lay, D, rq, dev(w), HybridFFN(dev(fw)))
    ck, sk, cv, sv = c["cache_k"], c["scale_k"], c["cache_v"], c["scale_v"]
    if head_major:
        ck, sk = lay.to_head_major(ck, sk, "k")
        cv, sv = lay.to_head_major(cv, sv, "v")
    ck, sk, cv, sv = ck.cuda(), sk.cuda(), cv.cuda(), sv.cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = None
    for t in range(steps):
        out = layer(xs[t].cuda(), ck, sk, cv, sv, st)
        if t + 1 < steps:
            decode_advance(st, status_word=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert st.b_seq_len.cpu().tolist() == [n + steps - 1 for n in lens]
    if head_major:
        ck, sk = lay.from_head_major(ck, sk, "k")
        cv, sv = lay.from_head_major(cv, sv, "v")
    # the oracle's loop, host bookkeeping
    ck_ref, sk_ref, cv_ref, sv_ref = (c[k].clone() for k in ("cache_k", "scale_k", "cache_v", "scale_v"))
    ref = None
    for t in range(steps):
        cur = torch.tensor([n + t for n in lens], dtype=torch.int32)
        mem = c["req_to_token"][torch.arange(B), cur.long() - 1]
        ref, _ = olayer.decoder_layer(xs[t], w, fw, lay.k_off, lay.v_off, H, D, rq, ck_ref, sk_ref, cv_ref, sv_ref,
                                      c["req_to_token"], c["b_req_idx"], cur, mem)
    assert torch.equal(ck.cpu(), ck_ref) and torch.equal(sk.cpu(), sk_ref)
    assert torch.equal(cv.cpu(), cv_ref) and torch.equal(sv.cpu(), sv_ref)
    assert rel_to_norm(out.cpu().float(), ref.float()) < 2e-3


@pytest.mark.parametrize("head_major", [False, True])
def test_prefill_append_then_decode_attention(head_major):
    """Prefill to decode hand-off: the cache is written by the prefill-sized form of the append kernel (2 requests x 2304
    tokens x 8 heads x K and V = 73 728 units) and then attended by the decode kernel; rows equal the oracle's quantiser
    bit for bit, the attention output is inside the tolerance."""
    from oracle import attention as oattn
    H, D = 8, 128
    kr, vr = synth.ragged_ranks(H, 64, seed=2), synth.ragged_ranks(H, 64, seed=3)
    B, L = 2, 2304
    c = U.build_case(B, H, D, kr, vr, [L, L - 100], seed=17, shuffle=True, extra_slots=64)
    lay = LatentCacheLayout(kr, vr, head_major=head_major)
    n_slots = c["n_slots"]
    ck, sk, cv, sv = [t.zero_() for t in lay.alloc(n_slots)]
    # every token of both requests in one call: latents in token order, destination slots from the request table
    slots = torch.cat([c["req_to_token"][c["b_req_idx"][b].item(), :L] for b in range(B)]).to(torch.int32)
    lk, lv = c["latent_k"][slots.long()].contiguous(), c["latent_v"][slots.long()].contiguous()
    assert slots.numel() * H * 2 >= 32768
    cache_append(lay, lk.cuda(), lv.cuda(), slots.cuda(), ck, sk, cv, sv)
    torch.cuda.synchronize()
    k2, sk2 = (lay.from_head_major(ck, sk, "k") if head_major else (ck, sk))
    v2, sv2 = (lay.from_head_major(cv, sv, "v") if head_major else (cv, sv))
    rows = slots.long()
    assert torch.equal(k2.cpu()[rows], c["cache_k"][rows]) and torch.equal(sk2.cpu()[rows], c["scale_k"][rows])
    assert torch.equal(v2.cpu()[rows], c["cache_v"][rows]) and torch.equal(sv2.cpu()[rows], c["scale_v"][rows])
    # decode over the cache the GPU wrote
    from lsvd_b200.attention import token_decode_attention_int8_latent_absorb as attend
    st = InferState(B, c["max_len"], c["b_seq_len"], device="cuda", req_to_token=c["req_to_token"], b_req_idx=c["b_req_idx"])
    o = attend(c["q"].cuda(), st, H, D, ck, sk, cv, sv, c["up_k"].cuda(), c["up_v"].cuda(), layout=lay).cpu()
    o_ref, _ = U.run_oracle(c)
    assert rel_to_norm(o.float(), o_ref.float()) < 2e-4


@pytest.mark.parametrize("head_major", [False, True])
def test_shared_kv_latent_layer(head_major):
    """One cached latent per head serving as K and as V latent (the reference's shared-``BLinear`` factors,
    fake_quant/utils/svd_utils.py:1505-1507): the cache holds half the bytes, the append writes it once, the attention
    reads scores and values from the same rows.  Against the oracle run with the same tensor on both sides."""
    H, D, rq, hidden = 8, 128, 64, 1024
    kr = synth.ragged_ranks(H, 64, seed=5)
    lay = LatentCacheLayout(kr, shared_kv=True, head_major=head_major)
    w = make_layer_weights(hidden, H, D, rq, kr, kr, seed=4, shared_kv=True)
    assert w["W_lat_q"].shape[0] == H * rq + sum(kr)
    fw = synth.ffn_weights(hidden, 12 * 64, 128, 384, seed=2, had_K=synth.sign_matrix(12, seed=1).float(), K=12, input_had=False, std=0.05)
    B, lens = 3, [150, 33, 64]
    c = U.build_case(B, H, D, kr, kr, lens, seed=11)
    st = InferState(B, c["max_len"], lens, device="cuda")
    x = torch.randn(B, hidden, generator=torch.Generator().manual_seed(3)).half()
    dev = lambda d: {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
    layer = LSVDDecoderLayer(lay, D, rq, dev(w), HybridFFN(dev(fw)))
    ck, sk, cv, sv = lay.alloc(c["cache_k"].shape[0])
    assert cv is ck and sv is sk
    if head_major:
        a, b = lay.to_head_major(c["cache_k"], c["scale_k"], "k")
        ck.copy_(a.cuda()); sk.copy_(b.cuda())
    else:
        ck.copy_(c["cache_k"].cuda()); sk.copy_(c["scale_k"].cuda())
    stages = {}
    out = layer(x.cuda(), ck, sk, cv, sv, st, stages=stages).cpu()
    ck_ref, sk_ref = c["cache_k"].clone(), c["scale_k"].clone()
    ref, rst = olayer.decoder_layer(x, w, fw, lay.k_off, lay.v_off, H, D, rq, ck_ref, sk_ref, ck_ref, sk_ref,
                                    c["req_to_token"], c["b_req_idx"], c["b_seq_len"], st.mem_index.cpu())
    got_k, got_s = (lay.from_head_major(ck, sk, "k") if head_major else (ck, sk))
    assert torch.equal(stages["lat"].cpu(), rst["lat"])
    assert torch.equal(got_k.cpu(), ck_ref) and torch.equal(got_s.cpu(), sk_ref)
    assert rel_to_norm(stages["o_lat"].cpu().float(), rst["o_lat"].float()) < 2e-3
    assert rel_to_norm(out.float(), ref.float()) < 2e-3
