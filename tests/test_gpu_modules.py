"""The drop-in modules (``SVDLinear``, ``ActQuantWrapper``, ``ActQuantizer``) and the checkpoint loader on the GPU, against
outputs of the reference's own modules (tests/golden/svd_linear.npz, act_quant_wrapper.npz, qmodel_ffn_io.npz) and the CPU
oracle.  fp16 outputs: 2e-3 * ||ref||_2 (BASELINE tolerance); quantiser codes: bit-exact."""
import ctypes as C
import os

import pytest
import torch
from torch import nn

from conftest import GOLDEN, load_golden, rel_to_norm
from oracle import modules as omod, quant as oquant, ffn as offn
from lsvd_b200 import _lib, formats
from lsvd_b200.modules import ActQuantWrapper, ActQuantizer, SVDLinear

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _lists(g):
    ranks = [int(r) for r in g["ranks"]]
    cout, cin = g["cout"], g["cin"]
    U, S, V, cu, cs, cv = [], [], [], 0, 0, 0
    for r in ranks:
        U.append(g["U"][cu:cu + cout * r].reshape(cout, r)); cu += cout * r
        S.append(g["S"][cs:cs + r]); cs += r
        V.append(g["V"][cv:cv + cin * r].reshape(cin, r)); cv += cin * r
    return ranks, U, S, V


@pytest.mark.parametrize("fuse", ["UV", "U", "V"])
def test_svd_linear_ragged_matches_reference(fuse):
    g = load_golden("svd_linear")
    ranks, U, S, V = _lists(g)
    m = SVDLinear(U, S, V, bias=g["bias"] if fuse == "UV" else None, sigma_fuse=fuse, is_per_head_svd=True, rank_split=ranks).cuda()
    y = m(g[f"ragged_{fuse}_x"].cuda())
    ref = g[f"ragged_{fuse}_y"]
    assert y.shape == ref.shape and y.dtype == torch.float16
    assert rel_to_norm(y.cpu().float(), ref.float()) < TOL
    # a factor changed in place (fine-tuning, rtn): the packed copy follows
    with torch.no_grad():
        m.ALinear[1].mul_(2)
    y2 = m(g[f"ragged_{fuse}_x"].cuda())
    A = [a.data.cpu() for a in m.ALinear]
    want = omod.svd_linear_per_head(g[f"ragged_{fuse}_x"], m.BLinear.weight.data.cpu(), A, None if m.bias is None else m.bias.data.cpu())
    assert rel_to_norm(y2.cpu().float(), want.float()) < TOL


def test_svd_linear_uniform_matches_reference():
    g = load_golden("svd_linear")
    m = SVDLinear(g["uni_U"], g["uni_S"], g["uni_V"], sigma_fuse="UV", is_per_head_svd=True).cuda()
    y = m(g["uni_x"].cuda())
    assert y.shape == g["uni_y"].shape
    assert rel_to_norm(y.cpu().float(), g["uni_y"].float()) < TOL


def test_per_head_up_large_ragged_against_oracle():
    """Llama-7B-like geometry: 32 heads of 128 channels, ranks 16..128, 70 tokens (tiles of 8 with a ragged last one)."""
    gen = torch.Generator().manual_seed(4)
    H, cout, cin, T = 32, 128, 256, 70
    ranks = [16 * int(v) for v in torch.randint(1, 9, (H,), generator=gen)]
    A = [(torch.randn(cout, r, generator=gen) * 0.1).half() for r in ranks]
    B = (torch.randn(sum(ranks), cin, generator=gen) * 0.05).half()
    m = SVDLinear([a for a in A], None, [B[sum(ranks[:h]):sum(ranks[:h + 1])] for h in range(H)], sigma_fuse="local_ft",
                  is_per_head_svd=True, rank_split=ranks).cuda()
    x = torch.randn(T, cin, generator=gen).half()
    y = m(x.cuda())
    want = omod.svd_linear_per_head(x, B, A)
    assert rel_to_norm(y.cpu().float(), want.float()) < TOL
    # the C entry checks its rank table
    off = (C.c_int32 * (H + 1))(*([0] + [5] * H))
    off[2] = 1
    z = torch.zeros(T, sum(ranks), dtype=torch.float16, device="cuda")
    rc = _lib.load().lsvd_per_head_up(z.data_ptr(), z.stride(0), z.data_ptr(), off, None, y.data_ptr(), y.stride(0), T, H, cout, None)
    assert rc == 1


def test_act_quantizer_matches_reference_fixture():
    g = load_golden("fq_quantizers")
    aq = ActQuantizer()
    aq.configure(bits=8, groupsize=-1, sym=True, clip_ratio=1.0)
    x = g["x"].cuda()
    aq.find_params(x)
    assert aq.scale.shape == (9, 1) and torch.equal(aq.scale.flatten().cpu(), g["a_scale"])
    q, s = aq.quantize(x)
    assert torch.equal(q.cpu().float(), g["a_codes"])
    assert torch.equal(aq(x).cpu(), g["a_fake"])
    aq.free()
    assert aq.scale is None
    aq.configure(bits=16)
    assert aq(x) is x


def _wrapper(g, tag, setup=None, out_bits=16, bias=False):
    W = g[tag + "_W"]
    lin = nn.Linear(W.shape[1], W.shape[0], bias=bias).half()
    lin.weight.data = W.clone()
    if bias:
        lin.bias.data = g[tag + "_b"].clone()
    w = ActQuantWrapper(lin)
    if setup is not None:
        setup(w)
    w.quantizer.configure(bits=8, groupsize=-1, sym=True, clip_ratio=1.0)
    if out_bits < 16:
        w.out_quantizer.configure(bits=out_bits, groupsize=-1, sym=True, clip_ratio=1.0)
    return w.cuda()


def test_wrapper_plain_int8_with_bias_and_output_quantiser():
    g = load_golden("act_quant_wrapper")
    w = _wrapper(g, "plain", out_bits=8, bias=True)
    y = w(g["plain_x"].cuda()).cpu().float()
    assert w.int8_weight()[0] is not None            # the product ran on int8 codes
    ref = g["plain_y"].float()
    step = ref.abs().amax(-1, keepdim=True) / 127
    assert ((y - ref).abs() <= 1.01 * step + 1e-6).all()
    assert ((y - ref).abs() > 0.5 * step).float().mean() < 0.1


def test_wrapper_more_than_64_tokens_takes_the_tensor_core_product():
    g = load_golden("act_quant_wrapper")
    w = _wrapper(g, "many", bias=True)
    y = w(g["many_x"].cuda())
    assert y.shape == g["many_y"].shape
    assert rel_to_norm(y.cpu().float(), g["many_y"].float()) < TOL


def test_wrapper_fp16_weight_keeps_the_library_product():
    g = load_golden("act_quant_wrapper")
    w = _wrapper(g, "w16")
    y = w(g["w16_x"].cuda())
    assert w.int8_weight() == (None, None)
    assert rel_to_norm(y.cpu().float(), g["w16_y"].float()) < TOL


@pytest.mark.parametrize("tag", ["full64", "full64_fp32", "full768", "partial", "random"])
def test_wrapper_online_rotations(tag):
    g = load_golden("act_quant_wrapper")

    def setup(w):
        if tag.startswith("full"):
            w.online_full_had = True
            w.fp32_had = tag.endswith("fp32")
            if tag == "full768":
                w.had_K, w.K = g["had12"].float(), 12
        elif tag == "partial":
            w.online_partial_had, w.had_dim, w.K = True, 16, 1
        else:
            w.online_random_had, w.had_K = True, g["random_Q"]

    w = _wrapper(g, tag, setup)
    y = w(g[tag + "_x"].cuda())
    assert rel_to_norm(y.cpu().float(), g[tag + "_y"].float()) < TOL
    # 16-bit input: the rotation alone, then the fp16 product
    w.quantizer.configure(bits=16)
    y16 = w(g[tag + "_x"].cuda())
    kw = {"full64": dict(rotation="full"), "full64_fp32": dict(rotation="full"),
          "full768": dict(rotation="full", K=12, had_K=g["had12"].float()), "partial": dict(rotation="partial", had_dim=16),
          "random": dict(rotation="random", had_K=g["random_Q"])}[tag]
    want = omod.act_quant_wrapper(g[tag + "_x"], g[tag + "_W"], None, in_bits=16, **kw)
    assert rel_to_norm(y16.cpu().float(), want.float()) < TOL


def test_wrapper_rejects_what_has_no_kernel():
    g = load_golden("act_quant_wrapper")
    w = _wrapper(g, "plain", bias=True)
    w.fuse_bias = True
    with pytest.raises(ValueError):
        w(g["plain_x"].cuda())
    w.fuse_bias = False
    with pytest.raises(ValueError):
        w(g["plain_x"].cuda().float())
    w.online_random_had, w.had_K = True, torch.randn(96, 96).half()     # not a signed Hadamard matrix
    with pytest.raises(ValueError):
        w(g["plain_x"].cuda())


def test_checkpoint_to_hybrid_ffn_matches_reference_output():
    """--save_qmodel_path checkpoint -> int8 buffers -> HybridFFN: the output the reference's module gave on the same x."""
    io = load_golden("qmodel_ffn_io")
    ffn = formats.load_hybrid_ffn(os.path.join(GOLDEN, "qmodel_ffn.pt"), "model.layers.0.mlp")
    y = ffn(io["x"].cuda())
    assert rel_to_norm(y.cpu().float(), io["y"].float()) < TOL
    sd, scales = formats.load_qmodel(os.path.join(GOLDEN, "qmodel_ffn.pt"))
    w = formats.hybrid_ffn_weights(sd, "model.layers.0.mlp", scales)
    w.pop("perm")
    w["had_sign"] = None
    ref = offn.hybrid_ffn_stages(io["x"], w)["out"]
    assert rel_to_norm(y.cpu().float(), ref.float()) < TOL
