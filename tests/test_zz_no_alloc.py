"""Decode attention through the entry point that brings its own scratch memory.

Some callers of the library cannot allocate device memory where a decode step runs -- a serving process
whose KV-cache pool already owns the GPU, a plugin living inside another runtime's memory budget -- so
`lsvd_attn_decode_static` uses a fixed array inside the library instead of a caller workspace.  This test
calls it through the C ABI, twice in a row (the array keeps the previous call's contents), and compares it
with the ordinary entry point; it also checks that a problem too large for the array is refused.
It is collected last so that a failure here cannot hide the results of the other tests.
"""
import ctypes as C

import pytest
import torch

from conftest import rel_to_norm
import gpu_util as U
from lsvd_b200 import _lib, synth
from lsvd_b200.attention import InferState

pytestmark = pytest.mark.gpu
TIGHT = 2e-4     # the bound the other attention tests hold the kernel to


def _args(c, st, out, dev_tensors):
    """Fill the C argument block by hand: this test goes through the C ABI, not the Python helpers."""
    lay = c["layout"]
    a = _lib.AttnDecodeArgs()
    a.batch, a.num_heads, a.head_dim = c["batch"], c["num_heads"], c["head_dim"]
    a.max_len_in_batch = c["max_len"]
    a.sm_scale = 0.0
    q, ck, sk, cv, sv, up_k, up_v = dev_tensors
    a.num_slots = ck.shape[0]
    a.q, a.q_stride_b, a.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    a.k_off, a.v_off = lay.off_c("k"), lay.off_c("v")
    a.cache_k, a.cache_k_row_stride = ck.data_ptr(), ck.stride(0)
    a.scale_k, a.scale_k_row_stride = sk.data_ptr(), sk.stride(0)
    a.cache_v, a.cache_v_row_stride = cv.data_ptr(), cv.stride(0)
    a.scale_v, a.scale_v_row_stride = sv.data_ptr(), sv.stride(0)
    a.up_k, a.up_k_row_stride = up_k.data_ptr(), up_k.stride(0)
    a.up_v, a.up_v_row_stride = up_v.data_ptr(), up_v.stride(0)
    r2t = st.req_manager.req_to_token_indexs
    a.req_to_token, a.req_to_token_stride = r2t.data_ptr(), r2t.stride(0)
    a.b_req_idx, a.b_seq_len = st.b_req_idx.data_ptr(), st.b_seq_len.data_ptr()
    a.out, a.out_stride_b, a.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
    return a


def _run_static(c):
    lib = _lib.load()
    dev = "cuda"
    st = InferState(c["batch"], c["max_len"], c["b_seq_len"], device=dev, req_to_token=c["req_to_token"],
                    b_req_idx=c["b_req_idx"])
    tens = [c[k].to(dev) for k in ("q", "cache_k", "scale_k", "cache_v", "scale_v", "up_k", "up_v")]
    out = torch.full((c["batch"], c["num_heads"], c["head_dim"]), float("nan"), dtype=torch.float16, device=dev)
    a = _args(c, st, out, tens)
    code = lib.lsvd_attn_decode_static(C.byref(a), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return code, out.cpu()


def test_static_scratch_entry_matches_the_ordinary_one_twice_in_a_row():
    assert _lib.load().lsvd_attn_decode_static_scratch_bytes() == 8 << 20
    kr, vr = synth.ragged_ranks(32, 64, seed=3), synth.ragged_ranks(32, 64, seed=4)
    first = U.build_case(3, 32, 128, kr, vr, [900, 17, 400], seed=21, shuffle=True, extra_slots=7)
    second = U.build_case(2, 8, 128, [64] * 8, [32] * 8, [65, 300], seed=22)     # another shape over the same bytes
    for c in (first, second, first):
        ref = U.run_gpu(c)                       # ordinary entry point, caller-owned workspace
        code, out = _run_static(c)
        assert code == _lib.OK
        assert torch.isfinite(out.float()).all()
        assert rel_to_norm(out.float(), ref.float()) < TIGHT
        assert torch.equal(out, ref)             # the two entry points run the same kernels on the same items
        o_ref, _ = U.run_oracle(c)               # and both stand against the CPU oracle
        assert rel_to_norm(out.float(), o_ref.float()) < TIGHT


def test_static_scratch_entry_refuses_a_problem_that_does_not_fit():
    # 64 requests x 32768 tokens would need far more than the 8 MiB array; nothing is launched
    lay_ranks = [64] * 32
    c = U.build_case(1, 32, 128, lay_ranks, lay_ranks, [8], seed=23)
    c["batch"], c["max_len"] = 64, 32768          # only the declared sizes matter: the call must stop before any launch
    lib = _lib.load()
    st = InferState(1, 8, [8], device="cuda")
    tens = [c[k].cuda() for k in ("q", "cache_k", "scale_k", "cache_v", "scale_v", "up_k", "up_v")]
    out = torch.zeros(64, 32, 128, dtype=torch.float16, device="cuda")
    a = _args(c, st, out, tens)
    assert lib.lsvd_attn_decode_static(C.byref(a), torch.cuda.current_stream().cuda_stream) == _lib.ERR_WORKSPACE
    torch.cuda.synchronize()
    assert (out == 0).all()
