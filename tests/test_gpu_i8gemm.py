"""The tcgen05 W8A8 GEMM against the oracle: int32 accumulators bit-exact, fp16 epilogues as the decode kernels."""
import pytest
import torch

from oracle import ffn as offn
from lsvd_b200.ffn import i8gemm, w8a8_gemv

pytestmark = pytest.mark.gpu


def _rand(m, n, k, seed):
    gen = torch.Generator().manual_seed(seed)
    a = torch.randint(-128, 128, (m, k), generator=gen, dtype=torch.int8)
    w = torch.randint(-128, 128, (n, k), generator=gen, dtype=torch.int8)
    sa = torch.rand(m, generator=gen) * 0.05 + 1e-3
    sw = torch.rand(n, generator=gen) * 0.01 + 1e-4
    return a, w, sa, sw


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (128, 256, 512), (300, 528, 400), (1000, 1024, 4096), (64, 48, 1376)])
def test_accumulators_exact_and_dequant(m, n, k):
    a, w, sa, sw = _rand(m, n, k, m + n + k)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, acc = i8gemm(a.cuda(), sa.cuda(), w.cuda(), sw.cuda(), want_acc=True, status_word=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    acc_ref = offn._i32_matmul(a, w)
    assert torch.equal(acc.cpu(), acc_ref)
    assert torch.equal(out.cpu(), offn._dequant16(acc_ref, sa, sw))


def test_gate_up_pair_and_agreement_with_decode_kernel():
    m, n, k = 200, 688, 512
    a, wg, sa, sg = _rand(m, n, k, 1)
    _, wu, _, su = _rand(m, n, k, 2)
    wg = (wg.float() / 6).round().to(torch.int8)
    wu = (wu.float() / 6).round().to(torch.int8)
    sg, su = sg * 0.2, su * 0.2
    out, _ = i8gemm(a.cuda(), sa.cuda(), wg.cuda(), sg.cuda(), wu.cuda(), su.cuda())
    g = offn._dequant16(offn._i32_matmul(a, wg), sa, sg)
    u = offn._dequant16(offn._i32_matmul(a, wu), sa, su)
    ref = offn.silu_mul16(g, u)
    d = (out.cpu().float() - ref.float()).abs()
    assert (d == 0).float().mean() > 0.999 and d.max() <= 2 ** -10 * ref.float().abs().max()
    # the first 64 tokens through the decode kernel give the same bits
    out64, _, _ = w8a8_gemv(a[:64].cuda(), sa[:64].cuda(), wg.cuda(), sg.cuda(), wu.cuda(), su.cuda())
    assert torch.equal(out64.cpu(), out[:64].cpu())


def test_many_tiles_per_block_both_accumulators():
    """More tiles than SMs: every block walks several tiles, alternating between the two TMEM accumulators."""
    m, n, k = 5000, 2048, 272
    a, w, sa, sw = _rand(m, n, k, 7)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, acc = i8gemm(a.cuda(), sa.cuda(), w.cuda(), sw.cuda(), want_acc=True, status_word=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    acc_ref = offn._i32_matmul(a, w)
    assert torch.equal(acc.cpu(), acc_ref)
    assert torch.equal(out.cpu(), offn._dequant16(acc_ref, sa, sw))


def test_gated_up_product_and_residual():
    """A lone "up" product gated by a gate computed from other activations, and a product with a residual."""
    m, n, k = 300, 528, 256
    a, wu, sa, su = _rand(m, n, k, 11)
    wu = (wu.float() / 6).round().to(torch.int8)
    su = su * 0.2
    gen = torch.Generator().manual_seed(12)
    gate = (torch.randn(m, n + 16, generator=gen) * 2).half()
    out, _ = i8gemm(a.cuda(), sa.cuda(), wu.cuda(), su.cuda(), gate=gate.cuda(), gate_col=16)
    u = offn._dequant16(offn._i32_matmul(a, wu), sa, su)
    ref = offn.silu_mul16(gate[:, 16:], u)
    d = (out.cpu().float() - ref.float()).abs()
    assert (d == 0).float().mean() > 0.999 and d.max() <= 2 ** -10 * ref.float().abs().max()
    res = torch.randn(m, n, generator=gen).half()
    out2, _ = i8gemm(a.cuda(), sa.cuda(), wu.cuda(), su.cuda(), residual=res.cuda())
    assert torch.equal(out2.cpu(), (u.float() + res.float()).half())
    # scales with a stride (one column of a [m, 2] array)
    s2 = torch.stack([sa, sa * 3], 1).contiguous().cuda()
    out3, _ = i8gemm(a.cuda(), s2[:, 1], wu.cuda(), su.cuda())
    assert torch.equal(out3.cpu(), offn._dequant16(offn._i32_matmul(a, wu), sa * 3, su))


def test_gate_up_pair_with_separate_activations():
    """The SVD branch's form: the up matrix reads its own activations (and row scales with a stride)."""
    m, n, k = 300, 688, 512
    a, wg, sa, sg = _rand(m, n, k, 21)
    a2, wu, sa2, su = _rand(m, n, k, 22)
    wg = (wg.float() / 6).round().to(torch.int8)
    wu = (wu.float() / 6).round().to(torch.int8)
    sg, su = sg * 0.2, su * 0.2
    z = torch.cat([a, a2], 1).contiguous().cuda()                       # [m, 2k]: the two latents side by side
    zs = torch.stack([sa, sa2], 1).contiguous().cuda()                  # [m, 2]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, _ = i8gemm(z[:, :k], zs[:, 0], wg.cuda(), sg.cuda(), wu.cuda(), su.cuda(), a2_q=z[:, k:], a2_scale=zs[:, 1],
                    status_word=status)
    assert status.item() == 0
    g = offn._dequant16(offn._i32_matmul(a, wg), sa, sg)
    u = offn._dequant16(offn._i32_matmul(a2, wu), sa2, su)
    ref = offn.silu_mul16(g, u)
    d = (out.cpu().float() - ref.float()).abs()
    assert (d == 0).float().mean() > 0.999 and d.max() <= 2 ** -10 * ref.float().abs().max()
    out64, _, _ = w8a8_gemv(z[:64, :k], zs[:64, 0], wg.cuda(), sg.cuda(), wu.cuda(), su.cuda(), a2_q=z[:64, k:], a2_scale=zs[:64, 1])
    assert torch.equal(out64.cpu(), out[:64].cpu())
