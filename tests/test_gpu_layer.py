"""The W8A8 decoder layer on the GPU against the oracle's composition of the same stages."""
import pytest
import torch

from conftest import load_golden, unpack_had, rel_to_norm
import gpu_util as U
from oracle import layer as olayer, quant
from lsvd_b200 import synth
from lsvd_b200.attention import LatentCacheLayout, InferState
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
