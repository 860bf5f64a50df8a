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
    assert lib.lsvd_abi_version() == 1
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
