"""GPU parity of the hybrid FFN kernels, through the C ABI, against the CPU oracle.

Integer stages (int8 codes, int32 accumulators) are bit-exact when fed the same inputs.  fp16 stage outputs
can differ in the last bit where a sum is formed in another order; the end-to-end output is held to
2e-3 * ||y_ref||_2 (specification) and to a tighter bound the kernels actually meet.
"""
import pytest
import torch

from conftest import load_golden, unpack_had, rel_to_norm
from oracle import ffn as offn, quant
from lsvd_b200 import synth
from lsvd_b200.ffn import (HybridFFN, act_quant, hadamard_quant, hadamard_pack, w8a8_gemv, quantize_weight_rtn,
                           heads_hadamard_quant)

pytestmark = pytest.mark.gpu
TOL = 2e-3


def to_dev(w):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in w.items()}


def test_weight_rtn_matches_oracle_and_reference_fixture():
    g = load_golden("fq_quantizers")
    for tag, mse in (("rtn", False), ("mse", True)):
        q, s = quantize_weight_rtn(g["W"], mse=mse)
        assert torch.equal(s, g["w_scale_" + tag].flatten()) and torch.equal(q.float(), g["w_codes_" + tag])


@pytest.mark.parametrize("cols", [64, 512, 4096, 11008])
def test_act_quant_bit_exact(cols):
    gen = torch.Generator().manual_seed(cols)
    x = (torch.randn(9, cols, generator=gen) * 3).half()
    x[0] = 0
    x[1, 5] = 1000.0
    q, s, _ = act_quant(x.cuda())
    q_ref, s_ref = quant.act_quant(x)
    assert torch.equal(s.cpu(), s_ref) and torch.equal(q.cpu(), q_ref)


def test_act_quant_reference_fixture():
    g = load_golden("fq_quantizers")
    q, s, _ = act_quant(g["x"].cuda())
    assert torch.equal(s.cpu(), g["a_scale"]) and torch.equal(q.cpu().float(), g["a_codes"])


def test_input_rotation_bit_exact():
    gen = torch.Generator().manual_seed(1)
    x = torch.randn(5, 4096, generator=gen).half()
    sign = (torch.randint(0, 2, (4096,), generator=gen).float() * 2 - 1).half()
    q, s, rot = act_quant(x.cuda(), sign=sign.cuda(), want_rotated=True)
    rot_ref = offn.input_rotation(x, sign)
    assert torch.equal(rot.cpu(), rot_ref)
    q_ref, s_ref = quant.act_quant(rot_ref)
    assert torch.equal(s.cpu(), s_ref) and torch.equal(q.cpu(), q_ref)
    # power-of-two rotation without signs (K == 1 form of the d_ffn Hadamard)
    q2, s2, rot2 = act_quant(x.cuda(), fwht=True, want_rotated=True)
    assert torch.equal(rot2.cpu(), offn.hadamard_full(x, None, 1))


@pytest.mark.parametrize("K,nb", [(172, 64), (108, 128), (172, 8), (172, 16)])
def test_hadamard_quant_against_oracle(K, nb):
    g = load_golden("hadamard")
    hk = unpack_had(g[f"had{K}_bits"], K)
    gen = torch.Generator().manual_seed(K + nb)
    x = torch.randn(4, K * nb, generator=gen).half()
    q, s, y = hadamard_quant(x.cuda(), hadamard_pack(hk.half().cuda()), K, want_rotated=True)
    y_ref = offn.hadamard_full(x, hk, K)
    d = (y.cpu().float() - y_ref.float()).abs()
    assert d.max() <= 2 ** -10 * y_ref.float().abs().max()          # at most one fp16 ulp of the largest entry
    assert (d == 0).float().mean() > 0.97
    # isolated: the quantiser applied to the kernel's own rotated row is bit-exact
    q_ref, s_ref = quant.act_quant(y.cpu())
    assert torch.equal(s.cpu(), s_ref) and torch.equal(q.cpu(), q_ref)


def test_hadamard_quant_reference_fixture():
    g = load_golden("hadamard")
    hk = unpack_had(g["had172_bits"], 172)
    x = g["x_688"]                                   # 172 x 4: below the kernel's smallest block, so embed:
    # (H_172 kron H_8) on [x, 0] interleaved is not the same transform; use the 1376-wide FFN fixture instead
    f = load_golden("hybrid_ffn")
    st = offn.hybrid_ffn_stages(f["x"], _golden_weights(f))
    q, s, y = hadamard_quant(st["h16"].cuda(), hadamard_pack(hk.half().cuda()), 172, want_rotated=True)
    assert rel_to_norm(y.cpu().float(), f["h"].float()) < 2e-3      # the reference module's rotated hidden vector
    assert x.shape[1] == 688


@pytest.mark.parametrize("m", [1, 5, 8, 33, 64])
def test_gemv_int32_exact_and_dequant(m):
    gen = torch.Generator().manual_seed(m)
    n, k = 1024, 4096
    a = torch.randint(-128, 128, (m, k), generator=gen, dtype=torch.int8)
    w = torch.randint(-128, 128, (n, k), generator=gen, dtype=torch.int8)
    sa = torch.rand(m, generator=gen) * 0.05 + 1e-3
    sw = torch.rand(n, generator=gen) * 0.01 + 1e-4
    out, acc, _ = w8a8_gemv(a.cuda(), sa.cuda(), w.cuda(), sw.cuda(), want_acc=True)
    acc_ref = offn._i32_matmul(a, w)
    assert torch.equal(acc.cpu(), acc_ref)
    assert torch.equal(out.cpu(), offn._dequant16(acc_ref, sa, sw))


@pytest.mark.parametrize("m,n,k,split", [(2, 64, 688, False), (9, 32, 48, None), (4, 48, 1376 + 16, True), (1, 5504, 512, True), (64, 1024, 512, True), (8, 688, 4096, False), (64, 512, 4096, False),
                                          (3, 4096, 11008, None)])
def test_gemv_shapes_dual_and_down(m, n, k, split):
    gen = torch.Generator().manual_seed(m * 7 + n)
    a = torch.randint(-128, 128, (m, k), generator=gen, dtype=torch.int8)
    w = torch.randint(-20, 21, (n, k), generator=gen, dtype=torch.int8)
    sa = torch.rand(m, generator=gen) * 0.02 + 1e-3
    sw = torch.rand(n, generator=gen) * 0.002 + 1e-4
    if split is None:
        out, acc, _ = w8a8_gemv(a.cuda(), sa.cuda(), w.cuda(), sw.cuda(), want_acc=True)
        acc_ref = offn._i32_matmul(a, w)
        assert torch.equal(acc.cpu(), acc_ref) and torch.equal(out.cpu(), offn._dequant16(acc_ref, sa, sw))
        return
    w2 = torch.randint(-20, 21, (n, k), generator=gen, dtype=torch.int8)
    sw2 = torch.rand(n, generator=gen) * 0.002 + 1e-4
    a2 = torch.randint(-128, 128, (m, k), generator=gen, dtype=torch.int8) if split else None
    sa2 = torch.rand(m, generator=gen) * 0.02 + 1e-3 if split else None
    out, acc, acc2 = w8a8_gemv(a.cuda(), sa.cuda(), w.cuda(), sw.cuda(), w2.cuda(), sw2.cuda(),
                               a2_q=a2.cuda() if split else None, a2_scale=sa2.cuda() if split else None, want_acc=True)
    g_ref = offn._i32_matmul(a, w)
    u_ref = offn._i32_matmul(a2 if split else a, w2)
    assert torch.equal(acc.cpu(), g_ref) and torch.equal(acc2.cpu(), u_ref)
    h_ref = offn.silu_mul16(offn._dequant16(g_ref, sa, sw), offn._dequant16(u_ref, sa2 if split else sa, sw2))
    d = (out.cpu().float() - h_ref.float()).abs()
    assert (d == 0).float().mean() > 0.999 and d.max() <= 2 ** -10 * h_ref.float().abs().max()


@pytest.mark.parametrize("m,n,k,kind", [(1, 1024, 4096, "single"), (16, 4096, 11008, "single"), (5, 48, 1376 + 16, "single"),
                                        (16, 5504, 4096, "dual"), (9, 688, 4096, "dual"), (16, 5504, 512, "split"),
                                        (3, 64, 48, "split")])
def test_gemv_tma_form_equals_register_form(m, n, k, kind):
    """form 1 (persistent, TMA-fed, at most 16 tokens) against form 0 and the oracle: same integers, same fp16."""
    gen = torch.Generator().manual_seed(m * 11 + n + k)
    a = torch.randint(-128, 128, (m, k), generator=gen, dtype=torch.int8).cuda()
    w = torch.randint(-128, 128, (n, k), generator=gen, dtype=torch.int8).cuda()
    sa = (torch.rand(m, generator=gen) * 0.02 + 1e-3).cuda()
    sw = (torch.rand(n, generator=gen) * 0.002 + 1e-4).cuda()
    kw = {}
    if kind != "single":
        kw["w2_q"] = torch.randint(-128, 128, (n, k), generator=gen, dtype=torch.int8).cuda()
        kw["w2_scale"] = (torch.rand(n, generator=gen) * 0.002 + 1e-4).cuda()
    if kind == "split":
        kw["a2_q"] = torch.randint(-128, 128, (m, k), generator=gen, dtype=torch.int8).cuda()
        kw["a2_scale"] = (torch.rand(m, generator=gen) * 0.02 + 1e-3).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    o0, acc0, acc0b = w8a8_gemv(a, sa, w, sw, want_acc=True, form=0, **kw)
    o1, acc1, acc1b = w8a8_gemv(a, sa, w, sw, want_acc=True, form=1, status_word=status, **kw)
    assert int(status.item()) == 0
    assert torch.equal(acc1.cpu(), offn._i32_matmul(a.cpu(), w.cpu()))
    assert torch.equal(acc0, acc1) and torch.equal(o0, o1)
    if kind != "single":
        assert torch.equal(acc0b, acc1b)


def test_gemv_tma_form_rejects_large_batches():
    a = torch.zeros(17, 64, dtype=torch.int8, device="cuda")
    w = torch.zeros(16, 64, dtype=torch.int8, device="cuda")
    s = torch.ones(17, device="cuda")
    with pytest.raises(ValueError):
        w8a8_gemv(a, s, w, s[:16].contiguous(), form=1)


def _golden_weights(g):
    K = g["K"]
    return {"had_sign": None, "K": K, "had_K": unpack_had(g["had_bits"], K),
            "U_q": torch.cat([g["Ug_q"], g["Uu_q"]]), "U_s": torch.cat([g["Ug_s"], g["Uu_s"]]),
            "Vg_q": g["Vg_q"], "Vg_s": g["Vg_s"], "Vu_q": g["Vu_q"], "Vu_s": g["Vu_s"],
            "Wg_q": g["Wg_q"], "Wg_s": g["Wg_s"], "Wu_q": g["Wu_q"], "Wu_s": g["Wu_s"],
            "Wd_q": g["Wd_q"], "Wd_s": g["Wd_s"]}


def test_full_ffn_against_reference_module_fixture():
    """The reference's HybridSVDQuantFFN (fp16, run on the CPU when the fixture was made) vs the int8 kernels."""
    g = load_golden("hybrid_ffn")
    ffn = HybridFFN(to_dev(_golden_weights(g)))
    y = ffn(g["x"].cuda()).cpu()
    assert rel_to_norm(y.float(), g["y"].float()) < TOL


@pytest.mark.parametrize("m", [1, 8, 64])
def test_config2_chain_stage_by_stage(m):
    """BASELINE config 2: hidden 4096, intermediate 11008, rank 512, 50 % SVD channels, Hadamard 64 x 172."""
    g = load_golden("hadamard")
    hk = unpack_had(g["had172_bits"], 172)
    w = synth.ffn_weights(4096, 11008, 512, 5504, seed=0, had_K=hk, K=172)
    gen = torch.Generator().manual_seed(100 + m)
    x = torch.randn(m, 4096, generator=gen).half()
    ffn = HybridFFN(to_dev(w))
    st = ffn.forward_stages(x.cuda(), want_acc=True)
    st = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in st.items()}
    ref = offn.hybrid_ffn_stages(x, w)
    # stages whose inputs are bit-identical by construction
    assert torch.equal(st["x_rot"], ref["x_rot"]) and torch.equal(st["x_q"], ref["x_q"]) and torch.equal(st["x_s"], ref["x_s"])
    assert torch.equal(st["lat_acc"], ref["lat_acc"]) and torch.equal(st["lat16"], ref["lat16"])
    assert torch.equal(st["latg_q"], ref["latg_q"]) and torch.equal(st["latu_q"], ref["latu_q"])
    assert torch.equal(st["g_svd_acc"], ref["g_svd_acc"]) and torch.equal(st["u_rtn_acc"], ref["u_rtn_acc"])
    # isolated downstream stages: the oracle recomputes each from the kernel's own inputs
    y_ref = offn.hadamard_full(st["h16"], hk, 172)
    assert (st["h_rot"].float() - y_ref.float()).abs().max() <= 2 ** -10 * y_ref.float().abs().max()
    hq_ref, hs_ref = quant.act_quant(st["h_rot"])
    assert torch.equal(st["h_q"], hq_ref) and torch.equal(st["h_s"], hs_ref)
    acc_ref = offn._i32_matmul(st["h_q"], w["Wd_q"])
    assert torch.equal(st["out_acc"], acc_ref)
    assert torch.equal(st["out"], offn._dequant16(acc_ref, st["h_s"], w["Wd_s"]))
    # the allocation-free decode path runs the same kernels
    assert torch.equal(ffn(x.cuda()).cpu(), st["out"])
    # end to end
    err = rel_to_norm(st["out"].float(), ref["out"].float())
    assert err < TOL, err


@pytest.mark.parametrize("m", [65, 300])
def test_prefill_form_equals_decode_form_row_by_row(m):
    """More than 64 tokens go through the tcgen05 GEMMs (forward_prefill): same bits as the decode kernels fed
    the same rows 64 at a time, with and without a residual; the golden-fixture module likewise."""
    g = load_golden("hadamard")
    hk = unpack_had(g["had172_bits"], 172)
    w = synth.ffn_weights(4096, 11008, 512, 5504, seed=3, had_K=hk, K=172)
    gen = torch.Generator().manual_seed(200 + m)
    x = torch.randn(m, 4096, generator=gen).half().cuda()
    res = torch.randn(m, 4096, generator=gen).half().cuda()
    ffn = HybridFFN(to_dev(w))
    y = ffn(x)
    y_res = ffn(x, residual=res)
    for r0 in range(0, m, 64):
        assert torch.equal(y[r0:r0 + 64], ffn(x[r0:r0 + 64]))
        assert torch.equal(y_res[r0:r0 + 64], ffn(x[r0:r0 + 64], residual=res[r0:r0 + 64]))
    gf = load_golden("hybrid_ffn")
    small = HybridFFN(to_dev(_golden_weights(gf)))
    xs = gf["x"].cuda()
    reps = (70 + xs.shape[0] - 1) // xs.shape[0]
    xb = xs.repeat(reps, 1)
    yb = small(xb)
    assert torch.equal(yb[:xs.shape[0]], small(xs))


def test_13b_shape_chain_hadamard_108_x_128():
    """BASELINE config 4's FFN shape: hidden 5120, intermediate 13824 = 108 x 128 (had_K of order 108), rank 640, half
    of the channels on the SVD branch, no input rotation (5120 is not a power of two: the model's residual rotation is
    folded into the weights offline)."""
    g = load_golden("hadamard")
    hk = unpack_had(g["had108_bits"], 108)
    w = synth.ffn_weights(5120, 13824, 640, 6912, seed=4, had_K=hk, K=108, input_had=False)
    gen = torch.Generator().manual_seed(13)
    x = torch.randn(8, 5120, generator=gen).half()
    ffn = HybridFFN(to_dev(w))
    st = ffn.forward_stages(x.cuda(), want_acc=True)
    st = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in st.items()}
    ref = offn.hybrid_ffn_stages(x, w)
    assert torch.equal(st["x_q"], ref["x_q"]) and torch.equal(st["lat_acc"], ref["lat_acc"])
    assert torch.equal(st["g_svd_acc"], ref["g_svd_acc"]) and torch.equal(st["u_rtn_acc"], ref["u_rtn_acc"])
    y_ref = offn.hadamard_full(st["h16"], hk, 108)
    assert (st["h_rot"].float() - y_ref.float()).abs().max() <= 2 ** -10 * y_ref.float().abs().max()
    hq_ref, hs_ref = quant.act_quant(st["h_rot"])
    assert torch.equal(st["h_q"], hq_ref) and torch.equal(st["h_s"], hs_ref)
    assert torch.equal(st["out_acc"], offn._i32_matmul(st["h_q"], w["Wd_q"]))
    y = ffn(x.cuda()).cpu()
    assert torch.equal(y, st["out"])
    assert rel_to_norm(y.float(), ref["out"].float()) < TOL
    # prefill form of the same module (tokens beyond 64)
    xb = torch.randn(80, 5120, generator=gen).half().cuda()
    yb = ffn(xb)
    assert torch.equal(yb[:64], ffn(xb[:64])) and torch.equal(yb[64:], ffn(xb[64:]))


def test_hadamard_across_heads_reference_fixture_and_7b_shape():
    g = load_golden("partial_hadamard")
    q, s, y = heads_hadamard_quant(g["x"].cuda(), g["heads"], want_rotated=True)
    assert (y.cpu().float() - g["rotated"].float()).abs().max() <= 2 ** -10 * g["rotated"].float().abs().max()
    q_ref, s_ref = quant.act_quant(y.cpu())
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)
    gen = torch.Generator().manual_seed(77)
    x = torch.randn(16, 32 * 128, generator=gen).half()
    q, s, y = heads_hadamard_quant(x.cuda(), 32, want_rotated=True)
    y_ref = offn.partial_hadamard_heads(x, 128)
    assert torch.equal(y.cpu(), y_ref)
    q_ref, s_ref = quant.act_quant(y_ref)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)
    # 28 heads (not a power of two): the had_K @ x form
    q, s, y = heads_hadamard_quant(g["x28"].cuda(), 28, want_rotated=True, had_K=g["had28"].float())
    assert torch.equal(y.cpu(), g["rotated28"])
    q_ref, s_ref = quant.act_quant(g["rotated28"])
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)
    x28 = torch.randn(9, 28 * 128, generator=gen).half()
    q, s, y = heads_hadamard_quant(x28.cuda(), 28, want_rotated=True, had_K=g["had28"].float())
    y_ref = offn.partial_hadamard_heads_hadk(x28, 128, g["had28"].float())
    assert (y.cpu().float() - y_ref.float()).abs().max() <= 2 ** -10 * y_ref.float().abs().max()


@pytest.mark.parametrize("m,n,k,kind", [(17, 1024, 4096, "single"), (64, 4096, 11008, "single"), (33, 48, 1376 + 16, "single"),
                                        (64, 5504, 4096, "dual"), (40, 688, 4096, "dual"), (64, 5504, 512, "split"),
                                        (20, 80, 48, "split"), (5, 4096, 512, "single"),
                                        # a tensor-parallel rank's column slices at the 13B shape: few channels, so the
                                        # block's warps split K (four warps on one 16-channel tile / two on each of two)
                                        (64, 1728, 5120, "dual"), (64, 3456, 5120, "dual"), (64, 1920, 5120, "single"),
                                        (64, 1280, 5120, "single"), (48, 2400, 2048 + 64, "split")])
def test_gemv_wide_form_equals_register_form(m, n, k, kind):
    """form 2 (token rows shared through shared memory, the default beyond 32 tokens) against form 3 (register-fed)
    and the oracle: same integers, same fp16."""
    gen = torch.Generator().manual_seed(m * 13 + n + k)
    a = torch.randint(-128, 128, (m, k), generator=gen, dtype=torch.int8).cuda()
    w = torch.randint(-128, 128, (n, k), generator=gen, dtype=torch.int8).cuda()
    sa = (torch.rand(m, generator=gen) * 0.02 + 1e-3).cuda()
    sw = (torch.rand(n, generator=gen) * 0.002 + 1e-4).cuda()
    kw = {}
    if kind != "single":
        kw["w2_q"] = torch.randint(-128, 128, (n, k), generator=gen, dtype=torch.int8).cuda()
        kw["w2_scale"] = (torch.rand(n, generator=gen) * 0.002 + 1e-4).cuda()
    if kind == "split":
        kw["a2_q"] = torch.randint(-128, 128, (m, k), generator=gen, dtype=torch.int8).cuda()
        kw["a2_scale"] = (torch.rand(m, generator=gen) * 0.02 + 1e-3).cuda()
    res = (torch.randn(m, n, generator=gen).half().cuda()) if kind == "single" else None
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    o3, acc3, acc3b = w8a8_gemv(a, sa, w, sw, want_acc=True, form=3, residual=res, **kw)
    o2, acc2, acc2b = w8a8_gemv(a, sa, w, sw, want_acc=True, form=2, residual=res, status_word=status, **kw)
    assert int(status.item()) == 0
    assert torch.equal(acc2.cpu(), offn._i32_matmul(a.cpu(), w.cpu()))
    assert torch.equal(acc3, acc2) and torch.equal(o3, o2)
    if kind != "single":
        assert torch.equal(acc3b, acc2b)


def test_provider_converts_a_swiglu_module_and_matches_the_oracle():
    """The "b200" FFN provider on a stand-in for the reference's SwiGLUFFN (norm + three Linears + residual)."""
    import types
    from torch import nn
    from oracle import layer as olayer
    from lsvd_b200.provider import b200_ffn, get_b200_ffn
    gen = torch.Generator().manual_seed(9)
    hidden, inter = 256, 512
    mod = types.SimpleNamespace(
        norm=types.SimpleNamespace(weight=nn.Parameter(torch.randn(hidden, generator=gen).half().cuda()), variance_epsilon=1e-6),
        up_proj=nn.Linear(hidden, inter, bias=False).half().cuda(), gate_proj=nn.Linear(hidden, inter, bias=False).half().cuda(),
        down_proj=nn.Linear(inter, hidden, bias=False).half().cuda())
    x = torch.randn(2, 3, hidden, generator=gen).half().cuda()
    y = b200_ffn(x, mod)
    assert y.shape == x.shape
    ffn, norm_w, eps = get_b200_ffn(mod)
    assert get_b200_ffn(mod)[0] is ffn                      # cached
    w = {k: v.cpu() for k, v in ffn.state_dict().items() if v is not None}
    w.update(K=1, had_K=None, had_sign=None, online_had=False)
    x2 = x.reshape(-1, hidden).cpu()
    xn = olayer.rms_norm(x2, norm_w.cpu(), eps)
    ref = offn.hybrid_ffn_stages(xn, w)["out"]
    ref = (ref.float() + x2.float()).half()
    assert rel_to_norm(y.reshape(-1, hidden).cpu().float(), ref.float()) < TOL
