"""The hybrid FFN as ONE persistent kernel (lsvd_ffn_decode with `fused`) against the chain of launches and the
CPU oracle: the two forms run the same device functions, so every output must be bit-identical; the oracle bounds
the end-to-end error (2e-3 * ||y_ref||_2, BASELINE tolerance for fp16 outputs).
"""
import ctypes as C

import pytest
import torch

from conftest import load_golden, unpack_had, rel_to_norm
from oracle import ffn as offn
from lsvd_b200 import _lib, synth
from lsvd_b200.ffn import HybridFFN

pytestmark = pytest.mark.gpu
TOL = 2e-3


def to_dev(w):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in w.items()}


def both_forms(w, x, **kw):
    """Output of the fused kernel and of the chain for the same module and input."""
    ffn = HybridFFN(to_dev(w))
    ffn.fused = True
    y_fused = ffn(x, **kw).clone()
    a, _ = ffn._chain(x.shape[0], x.device)
    assert _lib.load().lsvd_ffn_decode_is_fused(C.byref(a)) == 1, "this shape was expected to take the fused kernel"
    ffn2 = HybridFFN(to_dev(w))
    ffn2.fused = False
    y_chain = ffn2(x, **kw).clone()
    torch.cuda.synchronize()
    return ffn, y_fused, y_chain


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
def test_config2_fused_equals_chain_and_oracle(m):
    """BASELINE config 2 (4096 / 11008, rank 512, 50 % SVD channels, input rotation, Hadamard 64 x 172)."""
    g = load_golden("hadamard")
    hk = unpack_had(g["had172_bits"], 172)
    w = synth.ffn_weights(4096, 11008, 512, 5504, seed=m, had_K=hk, K=172)
    x = torch.randn(m, 4096, generator=torch.Generator().manual_seed(300 + m)).half()
    ffn, y_fused, y_chain = both_forms(w, x.cuda())
    assert torch.equal(y_fused, y_chain)
    # the counters of the sync block carry over from call to call: the same answer every time
    for _ in range(3):
        assert torch.equal(ffn(x.cuda()), y_fused)
    if m in (1, 16):
        ref = offn.hybrid_ffn_stages(x, w)["out"]
        assert rel_to_norm(y_fused.cpu().float(), ref.float()) < TOL


def test_fused_with_rmsnorm_prologue_and_residual():
    """The form the decoder layer uses: RMSNorm inside the first quantiser, residual added by the down projection."""
    w = synth.ffn_weights(4096, 11008, 512, 5504, seed=7, had_K=synth.sign_matrix(172, seed=1).float(), K=172, input_had=False)
    gen = torch.Generator().manual_seed(8)
    x = torch.randn(16, 4096, generator=gen).half().cuda()
    nw = (1 + 0.1 * torch.randn(4096, generator=gen)).half().cuda()
    _, y_fused, y_chain = both_forms(w, x, norm_weight=nw, norm_eps=1e-6, residual=x)
    assert torch.equal(y_fused, y_chain)


@pytest.mark.parametrize("shape", [
    dict(d_in=512, d_ffn=1024, rank=128, n_svd=512, K=1, online=True),     # power-of-two rotation of the hidden vector
    dict(d_in=512, d_ffn=1024, rank=128, n_svd=256, K=1, online=False),    # no rotation
    dict(d_in=1024, d_ffn=768, rank=128, n_svd=384, K=12, online=True),    # Hadamard 64 x 12, short K everywhere
    dict(d_in=272, d_ffn=768, rank=128, n_svd=400, K=12, online=True),     # K and channel counts that are not multiples of 128
])
def test_small_shapes_fused_equals_chain(shape):
    hk = synth.sign_matrix(shape["K"], seed=2).float() if shape["K"] > 1 else None
    pow2 = shape["d_in"] & (shape["d_in"] - 1) == 0          # the input rotation needs a power of two
    w = synth.ffn_weights(shape["d_in"], shape["d_ffn"], shape["rank"], shape["n_svd"], seed=11, had_K=hk, K=shape["K"],
                          input_had=pow2)
    w["online_had"] = shape["online"]
    for m in (2, 13):
        x = torch.randn(m, shape["d_in"], generator=torch.Generator().manual_seed(m)).half()
        _, y_fused, y_chain = both_forms(w, x.cuda())
        assert torch.equal(y_fused, y_chain)
        ref = offn.hybrid_ffn_stages(x, w)["out"]
        assert rel_to_norm(y_fused.cpu().float(), ref.float()) < TOL


def test_shapes_outside_the_fused_forms_take_the_chain():
    """rank 32 (the up latents do not start at a 128-byte block of the latent panel): lsvd_ffn_decode falls back, the
    result is the chain's."""
    hk = synth.sign_matrix(12, seed=0).float()
    w = synth.ffn_weights(256, 12 * 16, 32, 96, seed=0, had_K=hk, K=12)
    x = torch.randn(4, 256, generator=torch.Generator().manual_seed(2)).half().cuda()
    ffn = HybridFFN(to_dev(w))
    y = ffn(x)
    a, _ = ffn._chain(4, x.device)
    assert _lib.load().lsvd_ffn_decode_is_fused(C.byref(a)) == 0
    ref = offn.hybrid_ffn_stages(x.cpu(), w)["out"]
    assert rel_to_norm(y.cpu().float(), ref.float()) < TOL
