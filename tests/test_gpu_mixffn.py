"""GPU parity of the mixffn-structure FFN (lsvd_b200.mixffn) through the C ABI: against the stage tensors of the
reference's own pipeline (fixture: its eleven Triton kernels run in the interpreter) and against the oracle."""
import pytest
import torch

from conftest import load_golden, rel_to_norm
from oracle import mixffn as omix
from lsvd_b200.mixffn import (MixedFFNGateUpDenseLatentFused, b200_mixffn, get_b200_mixffn, mix_rmsnorm_quant,
                              mix_acc_quant, rounded_rank, svd_out_from_ratio)

pytestmark = pytest.mark.gpu

TOL = 2e-3
EXACT_BEFORE_SWIGLU = ["x_q", "x_scale", "up_svd_rank_fp", "gate_svd_rank_fp", "up_svd_rank_scale", "gate_svd_rank_scale",
                       "up_svd_rank_q", "gate_svd_rank_q", "up_dense_out_acc", "gate_dense_out_acc"]
EXACT_AFTER = ["mid_scale", "mid_q", "down_svd_rank_acc", "down_svd_rank_scale", "down_svd_rank_q", "down_svd_out_fp",
               "down_dense_out_fp", "down_fp", "out"]


def weights_of(g):
    return {k: v for k, v in g.items() if not k.startswith(("st_", "fp16_")) and k not in ("x", "eps")}


def check_stages(st, ref_before, x2, w, eps):
    """Integer stages in front of the SwiGLUs equal ``ref_before``; the SwiGLU outputs within one fp16 step and their
    maxima within 2 ulp of fp32; everything after them equal to the oracle continued from the GPU's SwiGLU outputs."""
    cpu = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in st.items()}
    for name in EXACT_BEFORE_SWIGLU:
        assert torch.equal(cpu[name], ref_before[name]), name
    for name in ("svd_mid_fp", "dense_mid_fp"):
        a, b = cpu[name].float(), ref_before[name].float()
        assert ((a - b).abs() <= 1e-3 * b.abs() + 1e-7).all(), name
    for name in ("svd_mid_scale", "dense_mid_scale"):
        a, b = cpu[name], ref_before[name]
        assert ((a - b).abs() <= 3e-7 * b.abs()).all(), name
    cont = omix.forward_stages(x2, w, eps, given={k: cpu[k] for k in ("svd_mid_fp", "svd_mid_scale", "dense_mid_fp", "dense_mid_scale")})
    for name in EXACT_AFTER:
        assert torch.equal(cpu[name].reshape(cont[name].shape), cont[name]), name
    return cpu


def test_reference_pipeline_fixture_stage_by_stage():
    g = load_golden("mixffn")
    w = weights_of(g)
    mod = MixedFFNGateUpDenseLatentFused({k: v.cuda() for k, v in w.items()}, eps=g["eps"])
    st = mod.forward_stages(g["x"].cuda())
    torch.cuda.synchronize()
    ref = {k[3:]: v for k, v in g.items() if k.startswith("st_")}
    x2 = g["x"].reshape(-1, g["x"].shape[-1])
    cpu = check_stages(st, ref, x2, w, g["eps"])
    assert cpu["out"].shape == g["st_out"].shape
    assert rel_to_norm(cpu["out"].float(), g["st_out"].float()) < TOL
    # codes of the hidden vector against the reference's own: equal but for rare one-step differences next to a
    # rounding boundary of the SwiGLU value
    d = (cpu["mid_q"].int() - g["st_mid_q"].int()).abs()
    assert int(d.max()) <= 1 and float((d > 0).float().mean()) < 0.01
    # forward() (residual inside the last two products) gives the same bits as the staged run
    y = mod(g["x"].cuda())
    assert torch.equal(y.cpu(), cpu["out"])


@pytest.mark.parametrize("tokens", [1, 8, 33, 64, 150])
def test_seeded_module_against_the_oracle(tokens):
    """hidden 1024, intermediate 2816 (low-rank channels 1408, rank 256; down: 512 channels, rank 192).  150 tokens: more
    than one pass of the 64-token kernels (the module takes any number of tokens, like the reference's tiled kernels)."""
    gen = torch.Generator().manual_seed(100 + tokens)
    hid, d = 1024, 2816
    up = (torch.randn(d, hid, generator=gen) / hid ** 0.5).half()
    gate = (torch.randn(d, hid, generator=gen) / hid ** 0.5).half()
    down = (torch.randn(hid, d, generator=gen) / d ** 0.5).half()
    norm = torch.randn(hid, generator=gen).half()
    w = omix.convert_swiglu(up, gate, down, norm, 0.5, 0.5, 64, gen)
    assert w["up_b_q"].shape == (svd_out_from_ratio(d, 0.5, 64), rounded_rank(hid, 1408, 0.5, 64))
    x = torch.randn(tokens, hid, generator=gen).half()
    if tokens > 2:
        x[2] = 0
        x[1] *= 30
    mod = MixedFFNGateUpDenseLatentFused({k: v.cuda() for k, v in w.items()}, eps=1e-6)
    st = mod.forward_stages(x.cuda())
    torch.cuda.synchronize()
    ref = omix.forward_stages(x, w, 1e-6)
    cpu = check_stages(st, ref, x, w, 1e-6)
    assert rel_to_norm(cpu["out"].float(), ref["out"].float()) < TOL
    assert torch.equal(mod(x.cuda()).cpu(), cpu["out"])


def test_quantisers_alone_edge_rows():
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(6, 272, generator=gen).half()              # a width that is not a multiple of the block size
    x[0] = 0
    x[1] = 65504.0
    x[2] *= 1e-4
    wn = torch.randn(272, generator=gen).half()
    q, s = mix_rmsnorm_quant(x.cuda(), wn.cuda(), 1e-6)
    q_ref, s_ref = omix.rmsnorm_quantize_per_token(x, wn, 1e-6)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu().half(), s_ref)
    acc = torch.randint(-2 ** 20, 2 ** 20, (6, 80), generator=gen, dtype=torch.int32)
    acc[3] = 0
    rs, cs = torch.rand(6, generator=gen) * 1e-2, torch.rand(80, generator=gen) * 1e-2
    q2, s2 = mix_acc_quant(acc.cuda(), rs.cuda(), cs.cuda())
    val = omix.dequant(acc, rs, cs)
    sc = omix.scale_from_absmax(val.abs().amax(-1))
    assert torch.equal(s2.cpu(), sc) and torch.equal(q2.cpu(), omix.rha_codes(val, sc[:, None]))


def test_provider_converts_and_caches():
    from types import SimpleNamespace
    gen = torch.Generator(device="cuda").manual_seed(1)
    hid, d = 512, 1024
    lin = lambda o, i: SimpleNamespace(weight=(torch.randn(o, i, device="cuda", generator=gen) / i ** 0.5).half())
    module = SimpleNamespace(norm=SimpleNamespace(weight=torch.randn(hid, device="cuda", generator=gen).half(), variance_epsilon=1e-6),
                             up_proj=lin(d, hid), gate_proj=lin(d, hid), down_proj=lin(hid, d), hidden_size=hid,
                             intermediate_size=d)
    x = torch.randn(2, 3, hid, device="cuda", generator=gen).half()
    y = b200_mixffn(x, module)
    conv = get_b200_mixffn(module)
    assert conv is get_b200_mixffn(module) and y.shape == x.shape
    w = {k: v.cpu() for k, v in conv.state_dict().items()}
    ref = omix.forward_stages(x.cpu().reshape(-1, hid), w, 1e-6)["out"]
    assert rel_to_norm(y.cpu().reshape(-1, hid).float(), ref.float()) < TOL
    # more than 64 tokens: passes of 64 through the same kernels, the same rows
    xl = torch.randn(130, hid, device="cuda", generator=gen).half()
    yl = conv(xl)
    assert torch.equal(yl[:64], conv(xl[:64])) and torch.equal(yl[128:], conv(xl[128:]))
    with pytest.raises(ValueError):
        conv(torch.zeros(3, hid + 16, dtype=torch.float16, device="cuda"))
