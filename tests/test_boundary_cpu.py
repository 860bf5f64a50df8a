"""CPU-side checks of the C-ABI boundary: the library loads, exports what the header declares, and
rejects bad arguments before touching the device."""
import ctypes as C
import os
import re

import pytest
import torch

from conftest import ROOT
from lsvd_b200 import _lib, build
from lsvd_b200.attention import LatentCacheLayout
from lsvd_b200 import synth


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def test_header_symbols_are_exported_and_bound(lib):
    hdr = open(os.path.join(ROOT, "include", "lsvd_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = set(re.findall(r"\b(lsvd_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations parsed"
    assert declared == set(_lib.SIGNATURES), (declared ^ set(_lib.SIGNATURES))
    for name in declared:
        assert hasattr(lib, name)
    assert lib.lsvd_abi_version() == 3
    assert lib.lsvd_status_string(_lib.ERR_TIMEOUT) == b"a bounded device-side wait gave up"


def test_null_and_bad_arguments_are_rejected_without_a_device(lib):
    assert lib.lsvd_cache_append(None, None) == _lib.ERR_INVALID_ARG
    assert lib.lsvd_attn_decode(None, None) == _lib.ERR_INVALID_ARG
    a = _lib.AppendArgs()
    a.num_tokens, a.num_heads, a.num_slots, a.rounding = 1, 0, 4, 0
    assert lib.lsvd_cache_append(C.byref(a), None) == _lib.ERR_INVALID_ARG
    a.num_heads, a.rounding = 2, 7
    assert lib.lsvd_cache_append(C.byref(a), None) == _lib.ERR_INVALID_ARG
    a.rounding, a.num_tokens = 0, 0
    assert lib.lsvd_cache_append(C.byref(a), None) == _lib.OK          # nothing to do
    # rank table that is not a multiple of 16
    a.num_tokens = 1
    a.dest_loc = 16
    side = _lib.AppendTensor()
    side.latent, side.cache, side.cache_scale = 16, 16, 16
    side.rank_off = _lib.i32_array([0, 24, 48])
    a.k = side
    assert lib.lsvd_cache_append(C.byref(a), None) == _lib.ERR_INVALID_ARG
    with pytest.raises(ValueError):
        _lib.check(_lib.ERR_INVALID_ARG)
    with pytest.raises(_lib.LsvdError):
        _lib.check(_lib.ERR_TIMEOUT)


def test_layout_validation():
    lay = LatentCacheLayout([16, 48, 128], [32, 16, 64])
    assert lay.k_off == [0, 16, 64, 192] and lay.v_off == [0, 32, 48, 112]
    for bad in ([0], [24], [144], []):
        with pytest.raises(ValueError):
            LatentCacheLayout(bad)
    with pytest.raises(ValueError):
        LatentCacheLayout([16, 16], [16])


def test_cpu_tensors_are_refused():
    from lsvd_b200 import destindex_copy_quantize_latent
    with pytest.raises(ValueError):
        destindex_copy_quantize_latent(torch.zeros(1, 2, 16, dtype=torch.float16), torch.zeros(1, dtype=torch.int32),
                                       torch.zeros(4, 2, 16, dtype=torch.int8), torch.zeros(4, 2, dtype=torch.float16))


def test_ragged_ranks_meet_the_budget():
    for H in (32, 40):
        r = synth.ragged_ranks(H, 64, seed=H)
        assert len(r) == H and sum(r) == 64 * H and all(16 <= x <= 128 and x % 16 == 0 for x in r)
        assert len(set(r)) > 3


def test_hybrid_ffn_from_module_reads_the_reference_layout():
    """HybridFFN.from_module on a stand-in with HybridSVDQuantFFN's attribute names: fake-quantised fp16 weights
    (codes x scale, as rtn_fwrd leaves them) come back as the same int8 codes and scales."""
    import types
    import torch
    from torch import nn
    from lsvd_b200.ffn import HybridFFN, quantize_weight_rtn
    g = torch.Generator().manual_seed(0)
    d_in, r, n_svd, n_q = 64, 16, 32, 48

    def fake(out_f, in_f):
        w = torch.randn(out_f, in_f, generator=g) * 0.05
        q, s = quantize_weight_rtn(w)
        lin = nn.Linear(in_f, out_f, bias=False)
        lin.weight.data = (q.float() * s[:, None]).half()
        return lin, q, s

    wrap = lambda lin: types.SimpleNamespace(module=lin)             # ActQuantWrapper keeps its Linear in .module
    parts = {k: fake(*shape) for k, shape in dict(Ug=(r, d_in), Uu=(r, d_in), Vg=(n_svd, r), Vu=(n_svd, r), Wg=(n_q, d_in),
                                                   Wu=(n_q, d_in), Wd=(d_in, n_svd + n_q)).items()}
    mlp = types.SimpleNamespace(
        gate_svd=types.SimpleNamespace(BLinear=wrap(parts["Ug"][0]), ALinear=parts["Vg"][0]),
        up_svd=types.SimpleNamespace(BLinear=wrap(parts["Uu"][0]), ALinear=parts["Vu"][0]),
        gate_quant=wrap(parts["Wg"][0]), up_quant=wrap(parts["Wu"][0]), down_proj=wrap(parts["Wd"][0]),
        had_K=None, K=1, online_had=False, n_svd=n_svd)
    ffn = HybridFFN.from_module(mlp)
    assert torch.equal(ffn.U_q, torch.cat([parts["Ug"][1], parts["Uu"][1]]))
    for name in ("Vg", "Vu", "Wg", "Wu", "Wd"):
        assert torch.equal(getattr(ffn, name + "_q"), parts[name][1])
        # fp16 storage of code x scale moves the recovered scale by at most one fp16 rounding
        assert torch.allclose(getattr(ffn, name + "_s"), parts[name][2], rtol=2e-3)
    assert ffn.n_svd == n_svd and ffn.rank == r and ffn.online_had is False
