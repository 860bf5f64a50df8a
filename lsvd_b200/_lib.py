"""ctypes binding of ``liblsvd_b200.so`` (the C ABI declared in ``include/lsvd_b200.h``).

There is no fallback: if the shared library is missing or does not load, importing
the kernels raises.  Tensors cross the boundary as raw device pointers, strides
and the current CUDA stream handle.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liblsvd_b200.so")

LSVD_MAX_HEADS = 128
LSVD_MAX_RANK = 128
ROUND_TORCH, ROUND_TRITON = 0, 1
CACHE_SLOT_MAJOR, CACHE_HEAD_MAJOR = 0, 1
OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_CUDA, ERR_TIMEOUT, ERR_BOUNDS = range(7)


class LsvdError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"lsvd_b200: {what} (status {code})")
        self.code = code


class AppendTensor(C.Structure):
    _fields_ = [
        ("latent", C.c_void_p), ("token_stride", C.c_int64), ("head_off", C.POINTER(C.c_int64)),
        ("rank_off", C.POINTER(C.c_int32)), ("cache", C.c_void_p), ("cache_row_stride", C.c_int64),
        ("cache_scale", C.c_void_p), ("scale_row_stride", C.c_int64),
    ]


class AppendArgs(C.Structure):
    _fields_ = [
        ("num_tokens", C.c_int32), ("num_heads", C.c_int32), ("rounding", C.c_int32), ("num_slots", C.c_int32),
        ("dest_loc", C.c_void_p), ("k", AppendTensor), ("v", AppendTensor), ("status_word", C.c_void_p),
        ("cache_layout", C.c_int32),
    ]


class AttnDecodeArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("num_heads", C.c_int32), ("head_dim", C.c_int32), ("max_len_in_batch", C.c_int32),
        ("sm_scale", C.c_float), ("num_slots", C.c_int32),
        ("q", C.c_void_p), ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64),
        ("k_off", C.POINTER(C.c_int32)), ("v_off", C.POINTER(C.c_int32)),
        ("cache_k", C.c_void_p), ("cache_k_row_stride", C.c_int64),
        ("scale_k", C.c_void_p), ("scale_k_row_stride", C.c_int64),
        ("cache_v", C.c_void_p), ("cache_v_row_stride", C.c_int64),
        ("scale_v", C.c_void_p), ("scale_v_row_stride", C.c_int64),
        ("up_k", C.c_void_p), ("up_k_row_stride", C.c_int64),
        ("up_v", C.c_void_p), ("up_v_row_stride", C.c_int64),
        ("req_to_token", C.c_void_p), ("req_to_token_stride", C.c_int64),
        ("b_req_idx", C.c_void_p), ("b_seq_len", C.c_void_p),
        ("out", C.c_void_p), ("out_stride_b", C.c_int64), ("out_stride_h", C.c_int64),
        ("out_latent", C.c_void_p), ("out_latent_stride_b", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("status_word", C.c_void_p), ("ev_stream_begin", C.c_void_p), ("ev_stream_end", C.c_void_p),
        ("cache_layout", C.c_int32), ("req_to_token_rows", C.c_int32),
    ]


class AttnRopeArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("num_q_heads", C.c_int32), ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32),
        ("rank_k", C.c_int32), ("rank_v", C.c_int32),
        ("q", C.c_void_p), ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64),
        ("cache_k", C.c_void_p), ("cache_k_slot_stride", C.c_int64), ("cache_k_head_stride", C.c_int64),
        ("scale_k", C.c_void_p), ("scale_k_slot_stride", C.c_int64),
        ("cache_v", C.c_void_p), ("cache_v_slot_stride", C.c_int64), ("cache_v_head_stride", C.c_int64),
        ("scale_v", C.c_void_p), ("scale_v_slot_stride", C.c_int64),
        ("wk", C.c_void_p), ("wk_row_stride", C.c_int64), ("wk_scale", C.c_void_p),
        ("req_to_token", C.c_void_p), ("req_to_token_stride", C.c_int64),
        ("b_req_idx", C.c_void_p), ("b_seq_len", C.c_void_p),
        ("num_slots", C.c_int32), ("max_len_in_batch", C.c_int32), ("block_seq", C.c_int32),
        ("sm_scale", C.c_float), ("rope_theta", C.c_float),
        ("out", C.c_void_p), ("out_stride_b", C.c_int64), ("out_stride_h", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("status_word", C.c_void_p),
    ]


class ActQuantArgs(C.Structure):
    _fields_ = [
        ("rows", C.c_int32), ("cols", C.c_int32), ("x", C.c_void_p), ("x_row_stride", C.c_int64),
        ("sign", C.c_void_p), ("fwht", C.c_int32), ("q", C.c_void_p), ("q_row_stride", C.c_int64),
        ("scale", C.c_void_p), ("x_rot", C.c_void_p), ("norm_weight", C.c_void_p), ("norm_eps", C.c_float),
        ("x_f32", C.c_void_p), ("add", C.c_void_p), ("sum_out", C.c_void_p), ("fake", C.c_void_p),
    ]


class HadamardQuantArgs(C.Structure):
    _fields_ = [
        ("rows", C.c_int32), ("cols", C.c_int32), ("K", C.c_int32), ("x", C.c_void_p), ("x_row_stride", C.c_int64),
        ("had_K_packed", C.c_void_p), ("q", C.c_void_p), ("q_row_stride", C.c_int64), ("scale", C.c_void_p), ("y", C.c_void_p),
    ]


class HeadsHadamardQuantArgs(C.Structure):
    _fields_ = [
        ("rows", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
        ("x", C.c_void_p), ("x_row_stride", C.c_int64), ("q", C.c_void_p), ("q_row_stride", C.c_int64),
        ("scale", C.c_void_p), ("y", C.c_void_p), ("had_K", C.c_void_p),
    ]


class GemvArgs(C.Structure):
    _fields_ = [
        ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
        ("w", C.c_void_p), ("w_row_stride", C.c_int64), ("w_scale", C.c_void_p),
        ("w2", C.c_void_p), ("w2_row_stride", C.c_int64), ("w2_scale", C.c_void_p),
        ("a", C.c_void_p), ("a_row_stride", C.c_int64), ("a_scale", C.c_void_p), ("a_scale_stride", C.c_int64),
        ("a2", C.c_void_p), ("a2_row_stride", C.c_int64), ("a2_scale", C.c_void_p), ("a2_scale_stride", C.c_int64),
        ("epilogue", C.c_int32), ("out", C.c_void_p), ("out_row_stride", C.c_int64), ("out_col", C.c_int32),
        ("acc_out", C.c_void_p), ("acc2_out", C.c_void_p), ("residual", C.c_void_p), ("residual_row_stride", C.c_int64),
        ("status_word", C.c_void_p), ("form", C.c_int32),
        ("row_absmax", C.c_void_p), ("row_absmax_stride", C.c_int64), ("absmax_split", C.c_int32),
        ("prefetch_weights", C.c_int32), ("out_f32", C.c_void_p),
    ]


class MixRmsnormQuantArgs(C.Structure):
    _fields_ = [
        ("rows", C.c_int32), ("cols", C.c_int32), ("x", C.c_void_p), ("x_row_stride", C.c_int64),
        ("norm_weight", C.c_void_p), ("eps", C.c_float), ("q", C.c_void_p), ("q_row_stride", C.c_int64),
        ("scale", C.c_void_p), ("clear_words", C.c_void_p), ("clear_per_row", C.c_int32),
    ]


class MixGroupQuantArgs(C.Structure):
    _fields_ = [
        ("rows", C.c_int32), ("cols", C.c_int32), ("split", C.c_int32), ("shared", C.c_int32),
        ("x", C.c_void_p), ("x_row_stride", C.c_int64), ("absmax", C.c_void_p), ("absmax_stride", C.c_int64),
        ("q", C.c_void_p), ("q_row_stride", C.c_int64), ("scale", C.c_void_p), ("scale_stride", C.c_int64),
    ]


class MixAccQuantArgs(C.Structure):
    _fields_ = [
        ("rows", C.c_int32), ("cols", C.c_int32), ("acc", C.c_void_p), ("acc_row_stride", C.c_int64),
        ("row_scale", C.c_void_p), ("row_scale_stride", C.c_int64), ("col_scale", C.c_void_p),
        ("q", C.c_void_p), ("q_row_stride", C.c_int64), ("scale", C.c_void_p),
    ]


class FfnDecodeArgs(C.Structure):
    _fields_ = [
        ("m", C.c_int32), ("d_in", C.c_int32), ("d_ffn", C.c_int32), ("d_out", C.c_int32), ("rank", C.c_int32),
        ("n_svd", C.c_int32), ("K", C.c_int32), ("online_had", C.c_int32), ("overlap", C.c_int32),
        ("x", C.c_void_p), ("x_row_stride", C.c_int64), ("had_sign", C.c_void_p), ("norm_weight", C.c_void_p),
        ("norm_eps", C.c_float),
        ("U_q", C.c_void_p), ("U_s", C.c_void_p), ("Vg_q", C.c_void_p), ("Vg_s", C.c_void_p),
        ("Vu_q", C.c_void_p), ("Vu_s", C.c_void_p), ("Wg_q", C.c_void_p), ("Wg_s", C.c_void_p),
        ("Wu_q", C.c_void_p), ("Wu_s", C.c_void_p), ("Wd_q", C.c_void_p), ("Wd_s", C.c_void_p),
        ("had_K_packed", C.c_void_p), ("residual", C.c_void_p), ("residual_row_stride", C.c_int64),
        ("out", C.c_void_p), ("out_row_stride", C.c_int64), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("status_word", C.c_void_p), ("fused", C.c_int32),
    ]


class I8GemmArgs(C.Structure):
    _fields_ = [
        ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
        ("a", C.c_void_p), ("a_row_stride", C.c_int64), ("a_scale", C.c_void_p),
        ("w", C.c_void_p), ("w_row_stride", C.c_int64), ("w_scale", C.c_void_p),
        ("w2", C.c_void_p), ("w2_row_stride", C.c_int64), ("w2_scale", C.c_void_p),
        ("out", C.c_void_p), ("out_row_stride", C.c_int64), ("out_col", C.c_int32),
        ("acc_out", C.c_void_p), ("status_word", C.c_void_p),
        ("a_scale_stride", C.c_int64), ("gate", C.c_void_p), ("gate_row_stride", C.c_int64), ("gate_col", C.c_int32),
        ("residual", C.c_void_p), ("residual_row_stride", C.c_int64),
        ("a2", C.c_void_p), ("a2_row_stride", C.c_int64), ("a2_scale", C.c_void_p), ("a2_scale_stride", C.c_int64),
    ]


# Every symbol include/lsvd_b200.h declares, with its ctypes signature.
SIGNATURES = {
    "lsvd_abi_version": (C.c_int, []),
    "lsvd_status_string": (C.c_char_p, [C.c_int]),
    "lsvd_last_cuda_error": (C.c_int, []),
    "lsvd_cache_append": (C.c_int, [C.POINTER(AppendArgs), C.c_void_p]),
    "lsvd_decode_advance": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                      C.c_int32, C.c_void_p, C.c_void_p]),
    "lsvd_attn_decode_workspace_bytes": (C.c_size_t, [C.c_int32] * 5),
    "lsvd_attn_decode": (C.c_int, [C.POINTER(AttnDecodeArgs), C.c_void_p]),
    "lsvd_attn_decode_static_scratch_bytes": (C.c_size_t, []),
    "lsvd_attn_decode_static": (C.c_int, [C.POINTER(AttnDecodeArgs), C.c_void_p]),
    "lsvd_heads_hadamard_quant": (C.c_int, [C.POINTER(HeadsHadamardQuantArgs), C.c_void_p]),
    "lsvd_ffn_decode_workspace_bytes": (C.c_size_t, [C.c_int32] * 5),
    "lsvd_ffn_decode_is_fused": (C.c_int, [C.POINTER(FfnDecodeArgs)]),
    "lsvd_fused_set_profile": (None, [C.c_void_p]),
    "lsvd_ffn_decode": (C.c_int, [C.POINTER(FfnDecodeArgs), C.c_void_p]),
    "lsvd_attn_decode_rope_workspace_bytes": (C.c_size_t, [C.c_int32] * 6),
    "lsvd_attn_decode_rope": (C.c_int, [C.POINTER(AttnRopeArgs), C.c_void_p]),
    "lsvd_act_quant": (C.c_int, [C.POINTER(ActQuantArgs), C.c_void_p]),
    "lsvd_hadamard_quant": (C.c_int, [C.POINTER(HadamardQuantArgs), C.c_void_p]),
    "lsvd_hadamard_packed_bytes": (C.c_size_t, [C.c_int32]),
    "lsvd_hadamard_pack": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "lsvd_w8a8_gemv": (C.c_int, [C.POINTER(GemvArgs), C.c_void_p]),
    "lsvd_dequant_residual": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int32,
                                        C.c_int32, C.c_void_p]),
    "lsvd_heads_hadamard_partial": (C.c_int, [C.c_void_p, C.c_int64, C.POINTER(C.c_int32), C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                              C.c_void_p, C.c_int32, C.c_void_p]),
    "lsvd_gather_segments": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.POINTER(C.c_int64),
                                       C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int32), C.c_void_p]),
    "lsvd_per_head_up": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.POINTER(C.c_int32), C.c_void_p, C.c_void_p, C.c_int64,
                                   C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "lsvd_i8gemm_prefill": (C.c_int, [C.POINTER(I8GemmArgs), C.c_void_p]),
    "lsvd_mix_rmsnorm_quant": (C.c_int, [C.POINTER(MixRmsnormQuantArgs), C.c_void_p]),
    "lsvd_mix_group_quant": (C.c_int, [C.POINTER(MixGroupQuantArgs), C.c_void_p]),
    "lsvd_mix_acc_quant": (C.c_int, [C.POINTER(MixAccQuantArgs), C.c_void_p]),
    "lsvd_attn_decode_plan": (C.c_int, [C.c_int32, C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.c_int32,
                                        C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library once; raise if it is absent (there is no CPU path behind it)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise LsvdError(-1, f"{LIB_PATH} not found: build it with `python -m lsvd_b200.build`")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code: int) -> None:
    """Turn a non-zero status into the exception type the reference raises for the same mistake."""
    if code == OK:
        return
    lib = load()
    what = lib.lsvd_status_string(code).decode()
    if code == ERR_CUDA:
        what += f" (cudaError {lib.lsvd_last_cuda_error()})"
    if code in (ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_WORKSPACE):
        raise ValueError(f"lsvd_b200: {what} (status {code})")
    raise LsvdError(code, what)


def i32_array(values):
    arr = (C.c_int32 * len(values))(*[int(v) for v in values])
    return arr


def i64_array(values):
    arr = (C.c_int64 * len(values))(*[int(v) for v in values])
    return arr
