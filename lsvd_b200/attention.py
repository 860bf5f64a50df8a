"""Host side of the latent KV cache and the int8 latent decode attention.

Mirrors the reference's Python interface for this path so that it drops into the
same call sites:

  * ``destindex_copy_quantize_latent(latent, dest_loc, cache, cache_scale)``
    -- kernels/layer_bench/fd_kernel/destindex_copy_quantize_latent.py:36-50
  * ``token_decode_attention_int8_latent_absorb(q, infer_state, ...)``
    -- kernels/layer_bench/fd_kernel/flash_decoding.py:3-57 (same ``infer_state``
    contract: batch_size, max_len_in_batch, b_seq_len, b_req_idx,
    req_manager.req_to_token_indexs)
  * ``InferState`` -- kernels/layer_bench/ffn_kernel/baseline_kernel.py:38-53

Everything here is argument checking and pointer plumbing; the arithmetic runs in
the CUDA kernels of ``liblsvd_b200.so``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch
from torch import nn

from . import _lib


def _stream_ptr(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("lsvd_b200 kernels need CUDA tensors; there is no CPU path")


class LatentCacheLayout:
    """Per-head latent ranks of a K/V cache row (multiples of 16, at most 128) and their offsets.

    The reference keeps per-head ranks as ragged ``ParameterList``s
    (fake_quant/utils/svd_utils.py:185-233); the kernel benchmark uses one rank
    for every head.  A cache row stores the heads back to back, so a uniform rank
    R gives exactly the reference's ``[N_slots, H, R]`` tensor.
    """

    def __init__(self, k_ranks: Sequence[int], v_ranks: Optional[Sequence[int]] = None, head_major: bool = False,
                 shared_kv: bool = False):
        """``shared_kv``: K and V of a head are up-projections of ONE cached latent, as when the reference builds the
        Q, K and V factors over a shared ``BLinear`` (fake_quant/utils/svd_utils.py:1505-1507): the cache holds that latent
        once (half the bytes); ``alloc`` returns the same tensors for the K and the V side, ``cache_append`` writes them
        once, and the attention reads its score and value operands from the same rows.
        ``head_major``: the cache is stored head by head -- ``cache [H][N_slots][r_h]`` as one flat int8 buffer of
        ``N_slots * sum(r)`` bytes and scales ``[H, N_slots]`` -- instead of one row per slot (``[N_slots, sum r]``,
        scales ``[N_slots, H]``, the reference's layout).  Same values; the rows a head reads for consecutive slots are
        then contiguous in memory, which the streaming kernel's loads prefer."""
        self.head_major = bool(head_major)
        self.shared_kv = bool(shared_kv)
        v_ranks = list(k_ranks if v_ranks is None else v_ranks)
        k_ranks = list(k_ranks)
        if self.shared_kv and k_ranks != v_ranks:
            raise ValueError("a shared K/V latent has one rank per head")
        if len(k_ranks) != len(v_ranks) or not k_ranks:
            raise ValueError("k_ranks and v_ranks must list the same, non-zero number of heads")
        if len(k_ranks) > _lib.LSVD_MAX_HEADS:
            raise ValueError(f"at most {_lib.LSVD_MAX_HEADS} heads per call")
        for r in k_ranks + v_ranks:
            if r <= 0 or r % 16 or r > _lib.LSVD_MAX_RANK:
                raise ValueError(f"latent ranks must be multiples of 16 in [16, {_lib.LSVD_MAX_RANK}], got {r}")
        self.num_heads = len(k_ranks)
        self.k_ranks, self.v_ranks = k_ranks, v_ranks
        self.k_off = [0]
        self.v_off = [0]
        for a, b in zip(k_ranks, v_ranks):
            self.k_off.append(self.k_off[-1] + a)
            self.v_off.append(self.v_off[-1] + b)
        self.sum_k, self.sum_v = self.k_off[-1], self.v_off[-1]
        self._k_off_c = _lib.i32_array(self.k_off)
        self._v_off_c = _lib.i32_array(self.v_off)

    @classmethod
    def uniform(cls, num_heads: int, rank_k: int, rank_v: Optional[int] = None):
        return cls([rank_k] * num_heads, [rank_v if rank_v is not None else rank_k] * num_heads)

    def as_head_major(self):
        return LatentCacheLayout(self.k_ranks, self.v_ranks, head_major=True, shared_kv=self.shared_kv)

    def alloc(self, num_slots: int, device="cuda"):
        """Empty (cache_k, scale_k, cache_v, scale_v) for ``num_slots`` slots in this layout."""
        if self.shared_kv:
            one = LatentCacheLayout(self.k_ranks, None, head_major=self.head_major)
            ck, sk, _, _ = one._alloc_sides(num_slots, device, ("k",))
            return ck, sk, ck, sk
        return self._alloc_sides(num_slots, device, ("k", "v"))

    def _alloc_sides(self, num_slots: int, device, sides):
        if sides == ("k",):
            total = self.sum_k
            if self.head_major:
                return (torch.empty(num_slots * total, dtype=torch.int8, device=device),
                        torch.empty(self.num_heads, num_slots, dtype=torch.float16, device=device), None, None)
            return (torch.empty(num_slots, total, dtype=torch.int8, device=device),
                    torch.empty(num_slots, self.num_heads, dtype=torch.float16, device=device), None, None)
        if self.head_major:
            return (torch.empty(num_slots * self.sum_k, dtype=torch.int8, device=device),
                    torch.empty(self.num_heads, num_slots, dtype=torch.float16, device=device),
                    torch.empty(num_slots * self.sum_v, dtype=torch.int8, device=device),
                    torch.empty(self.num_heads, num_slots, dtype=torch.float16, device=device))
        return (torch.empty(num_slots, self.sum_k, dtype=torch.int8, device=device),
                torch.empty(num_slots, self.num_heads, dtype=torch.float16, device=device),
                torch.empty(num_slots, self.sum_v, dtype=torch.int8, device=device),
                torch.empty(num_slots, self.num_heads, dtype=torch.float16, device=device))

    def num_slots_of(self, cache: torch.Tensor, which: str = "k") -> int:
        total = self.sum_k if which == "k" else self.sum_v
        return cache.numel() // total if self.head_major else cache.shape[0]

    def to_head_major(self, cache: torch.Tensor, scale: torch.Tensor, which: str = "k"):
        """Slot-major ``cache [N, sum r]`` / ``scale [N, H]`` -> the head-major buffers (a copy)."""
        off = self.k_off if which == "k" else self.v_off
        flat = torch.cat([cache[:, off[h]:off[h + 1]].contiguous().flatten() for h in range(self.num_heads)])
        return flat, scale.t().contiguous()

    def from_head_major(self, flat: torch.Tensor, scale_hn: torch.Tensor, which: str = "k"):
        """The inverse of ``to_head_major``."""
        off = self.k_off if which == "k" else self.v_off
        n = scale_hn.shape[1]
        cols = [flat[off[h] * n:off[h + 1] * n].view(n, off[h + 1] - off[h]) for h in range(self.num_heads)]
        return torch.cat(cols, dim=1).contiguous(), scale_hn.t().contiguous()

    def off_c(self, which: str):
        return self._k_off_c if which == "k" else self._v_off_c


def _rounding_code(rounding: str) -> int:
    try:
        return {"torch": _lib.ROUND_TORCH, "triton": _lib.ROUND_TRITON}[rounding]
    except KeyError:
        raise ValueError(f"rounding must be 'torch' or 'triton', got {rounding!r}")


def _append_side(latent, off_c, offs, cache, scale, keep, head_major=False):
    """Fill one AppendTensor from 2-D views: latent [T, sum r] (unit inner stride), cache [N, >= sum r] int8 (or the flat
    head-major buffer)."""
    side = _lib.AppendTensor()
    if latent is None:
        return side
    if latent.dtype != torch.float16 or cache.dtype != torch.int8 or scale.dtype != torch.float16:
        raise ValueError("latent and cache_scale must be fp16 and cache int8")
    if latent.stride(-1) != 1 or cache.stride(-1) != 1 or scale.stride(-1) != 1:
        raise ValueError("innermost strides must be 1")
    if head_major and (not cache.is_contiguous() or not scale.is_contiguous()):
        raise ValueError("head-major caches and scales must be contiguous")
    side.latent = latent.data_ptr()
    side.token_stride = latent.stride(0)
    side.head_off = None
    side.rank_off = off_c
    side.cache = cache.data_ptr()
    side.cache_row_stride = 0 if head_major else cache.stride(0)
    side.cache_scale = scale.data_ptr()
    side.scale_row_stride = 0 if head_major else scale.stride(0)
    keep.extend((latent, cache, scale))
    return side


def cache_append(layout: LatentCacheLayout, latent_k, latent_v, dest_loc, cache_k, scale_k, cache_v, scale_v,
                 rounding: str = "torch", status_word: Optional[torch.Tensor] = None) -> None:
    """Quantise this step's K and V latents and write them to cache rows ``dest_loc`` in one launch.

    ``latent_* [T, sum(r)]`` fp16 (head h in columns off[h]:off[h+1]); ``cache_* [N_slots, sum(r)]`` int8;
    ``scale_* [N_slots, H]`` fp16; ``dest_loc [T]`` int32.  Either side may be None.  With a shared K/V latent
    (``layout.shared_kv``) the one latent is ``latent_k`` and ``latent_v`` must be None or the same tensor.
    """
    if layout.shared_kv:
        if latent_v is not None and latent_v.data_ptr() != latent_k.data_ptr():
            raise ValueError("shared K/V latent: pass the latent once (latent_v None)")
        latent_v = None
    _require_cuda(latent_k, latent_v, dest_loc, cache_k, cache_v)
    lib = _lib.load()
    if dest_loc.dtype != torch.int32 or not dest_loc.is_contiguous():
        raise ValueError("dest_loc must be a contiguous int32 tensor")
    T = dest_loc.numel()
    keep = []
    args = _lib.AppendArgs()
    args.num_tokens = T
    args.num_heads = layout.num_heads
    args.rounding = _rounding_code(rounding)
    hm = layout.head_major
    args.cache_layout = _lib.CACHE_HEAD_MAJOR if hm else _lib.CACHE_SLOT_MAJOR
    args.num_slots = layout.num_slots_of(cache_k, "k") if latent_k is not None else layout.num_slots_of(cache_v, "v")
    args.dest_loc = dest_loc.data_ptr()
    for name, lat, cache, scale, total in (("k", latent_k, cache_k, scale_k, layout.sum_k),
                                            ("v", latent_v, cache_v, scale_v, layout.sum_v)):
        if lat is None:
            continue
        if lat.dim() != 2 or lat.shape[0] != T or lat.shape[1] != total:
            raise ValueError(f"latent_{name} must be [{T}, {total}], got {tuple(lat.shape)}")
        if hm:
            if cache.numel() != args.num_slots * total or tuple(scale.shape) != (layout.num_heads, args.num_slots):
                raise ValueError(f"cache_{name} / scale_{name} do not match the head-major layout")
        else:
            if cache.dim() != 2 or cache.shape[1] != total or scale.shape[1] != layout.num_heads:
                raise ValueError(f"cache_{name} / scale_{name} do not match the layout")
            if cache.shape[0] != args.num_slots or scale.shape[0] != args.num_slots:
                raise ValueError("K and V caches must have the same number of slots")
        setattr(args, name, _append_side(lat, layout.off_c(name), None, cache, scale, keep, hm))
    args.status_word = status_word.data_ptr() if status_word is not None else None
    _lib.check(lib.lsvd_cache_append(C.byref(args), _stream_ptr(dest_loc)))


@torch.no_grad()
def destindex_copy_quantize_latent(latent, dest_loc, cache, cache_scale, rounding: str = "torch") -> None:
    """Drop-in for the reference's cache-append function (uniform rank, one tensor per call).

    latent ``[T, H, R]`` fp16 (any token / head strides), cache ``[N, H, R]`` int8, cache_scale ``[N, H]``
    fp16.  Same shape checks as kernels/layer_bench/fd_kernel/destindex_copy_quantize_latent.py:40-41.
    ``rounding='torch'`` reproduces the reference's PyTorch quantiser bit for bit, ``'triton'`` its Triton kernel.
    """
    token_num, head_num, rank = latent.shape
    assert cache.shape[1:] == (head_num, rank)
    assert cache_scale.shape[1] == head_num
    _require_cuda(latent, dest_loc, cache, cache_scale)
    lib = _lib.load()
    if latent.stride(2) != 1:
        latent = latent.contiguous()
    if not cache.is_contiguous() or cache_scale.stride(1) != 1:
        raise ValueError("cache must be contiguous and cache_scale have unit head stride")
    if rank % 16 or rank > _lib.LSVD_MAX_RANK:
        raise ValueError(f"rank must be a multiple of 16 and at most {_lib.LSVD_MAX_RANK}")
    if dest_loc.dtype != torch.int32:
        dest_loc = dest_loc.to(torch.int32)
    dest_loc = dest_loc.contiguous()
    side = _lib.AppendTensor()
    side.latent = latent.data_ptr()
    side.token_stride = latent.stride(0)
    head_off = _lib.i64_array([h * latent.stride(1) for h in range(head_num)])
    rank_off = _lib.i32_array([h * rank for h in range(head_num + 1)])
    side.head_off = head_off
    side.rank_off = rank_off
    side.cache = cache.data_ptr()
    side.cache_row_stride = cache.stride(0)
    side.cache_scale = cache_scale.data_ptr()
    side.scale_row_stride = cache_scale.stride(0)
    args = _lib.AppendArgs()
    args.num_tokens = token_num
    args.num_heads = head_num
    args.rounding = _rounding_code(rounding)
    args.num_slots = cache.shape[0]
    args.dest_loc = dest_loc.data_ptr()
    args.k = side
    _lib.check(lib.lsvd_cache_append(C.byref(args), _stream_ptr(latent)))


class InferState:
    """Batch bookkeeping of a decode step, with the reference's field names
    (kernels/layer_bench/ffn_kernel/baseline_kernel.py:38-53): request b reads cache rows
    ``req_manager.req_to_token_indexs[b_req_idx[b], :b_seq_len[b]]`` and its current token lives in row
    ``mem_index[b]``.  ``req_to_token`` defaults to the identity map of the reference's benchmark."""

    class _ReqManager:
        def __init__(self, table):
            self.req_to_token_indexs = table

    def __init__(self, batch_size: int, max_len_in_batch: int, seq_lens, device="cuda",
                 req_to_token: Optional[torch.Tensor] = None, b_req_idx: Optional[torch.Tensor] = None):
        self.batch_size = batch_size
        self.max_len_in_batch = max_len_in_batch
        self.b_seq_len = torch.as_tensor(seq_lens, dtype=torch.int32).to(device)
        self.b_req_idx = (torch.arange(batch_size, dtype=torch.int32) if b_req_idx is None
                          else b_req_idx.to(torch.int32)).to(device)
        if req_to_token is None:
            req_to_token = torch.arange(batch_size * max_len_in_batch, dtype=torch.int32).view(batch_size, max_len_in_batch)
        self.req_manager = InferState._ReqManager(req_to_token.to(torch.int32).to(device).contiguous())
        last = (self.b_seq_len.long() - 1).clamp_min(0)
        self.mem_index = self.req_manager.req_to_token_indexs[self.b_req_idx.long(), last].contiguous()


def decode_advance(infer_state: "InferState", base_len: int = 0, period: int = 0, status_word=None) -> None:
    """One token further, on the device: ``b_seq_len += 1`` and ``mem_index`` = the slot of the new last position (read
    from ``req_to_token``).  ``max_len_in_batch`` of the state is the bound the lengths may reach.  With ``period`` a
    request that reaches ``base_len + period`` starts over at ``base_len``."""
    r2t = infer_state.req_manager.req_to_token_indexs
    _lib.check(_lib.load().lsvd_decode_advance(
        infer_state.b_seq_len.data_ptr(), infer_state.mem_index.data_ptr(), r2t.data_ptr(), r2t.stride(0),
        infer_state.b_req_idx.data_ptr(), infer_state.batch_size, base_len, period, int(infer_state.max_len_in_batch),
        status_word.data_ptr() if status_word is not None else None, torch.cuda.current_stream(r2t.device).cuda_stream))


def attn_decode_workspace_bytes(batch: int, layout: LatentCacheLayout, max_len_in_batch: int) -> int:
    return int(_lib.load().lsvd_attn_decode_workspace_bytes(batch, layout.num_heads, layout.sum_k, layout.sum_v,
                                                            max_len_in_batch))


@torch.no_grad()
def token_decode_attention_int8_latent_absorb(
        q, infer_state, q_head_num: int, head_dim: int,
        cache_latent_k, cache_latent_k_scale, cache_latent_v, cache_latent_v_scale,
        up_k, up_v=None, layout: Optional[LatentCacheLayout] = None,
        out=None, out_latent=None, alloc_tensor_func=torch.empty, workspace=None,
        sm_scale: Optional[float] = None, status_word=None, timing_events=None):
    """Decode attention over the int8 latent cache, one query token per request.

    Same call shape as the reference's ``token_decode_attention_flash_int8_latent_per_head_decoding_rope``
    (kernels/layer_bench/fd_kernel/flash_decoding.py:3-17), with the int8 K up-factor and its column scales
    replaced by the fp16 per-head up-factors ``up_k [sum r_k, D]`` / ``up_v [sum r_v, D]`` of the rotary-free
    configuration.  ``cache_latent_*`` may be ``[N, H, R]`` (uniform rank) or ``[N, sum r]``.  Returns
    ``out [B, H, D]`` fp16 when ``up_v`` is given, otherwise the latent-space result ``[B, sum r_v]`` fp16
    like the reference.  Workspace and outputs come from ``alloc_tensor_func`` unless passed in.
    """
    _require_cuda(q, cache_latent_k, cache_latent_v, up_k)
    lib = _lib.load()
    B = infer_state.batch_size
    if q.dtype != torch.float16 or up_k.dtype != torch.float16:
        raise ValueError("q and up-factors must be fp16")
    q = q.view(B, q_head_num, head_dim)
    if q.stride(2) != 1:
        q = q.contiguous()
    if cache_latent_k.dim() == 3:
        if layout is None:
            layout = LatentCacheLayout.uniform(q_head_num, cache_latent_k.shape[-1], cache_latent_v.shape[-1])
        if not cache_latent_k.is_contiguous() or not cache_latent_v.is_contiguous():
            raise ValueError("3-D latent caches must be contiguous")
        cache_latent_k = cache_latent_k.view(cache_latent_k.shape[0], -1)
        cache_latent_v = cache_latent_v.view(cache_latent_v.shape[0], -1)
    if layout is None:
        raise ValueError("a LatentCacheLayout is needed for 2-D (ragged) caches")
    if layout.num_heads != q_head_num:
        raise ValueError("only num_q_heads == num_kv_heads is supported")
    hm = layout.head_major
    if hm:
        n_slots = layout.num_slots_of(cache_latent_k, "k")
        if (cache_latent_k.numel() != n_slots * layout.sum_k or cache_latent_v.numel() != n_slots * layout.sum_v or
                tuple(cache_latent_k_scale.shape) != (layout.num_heads, n_slots) or
                tuple(cache_latent_v_scale.shape) != (layout.num_heads, n_slots)):
            raise ValueError("caches / scales do not match the head-major layout")
        if not (cache_latent_k.is_contiguous() and cache_latent_v.is_contiguous() and cache_latent_k_scale.is_contiguous()
                and cache_latent_v_scale.is_contiguous()):
            raise ValueError("head-major caches and scales must be contiguous")
    elif cache_latent_k.shape[1] != layout.sum_k or cache_latent_v.shape[1] != layout.sum_v:
        raise ValueError("cache row width does not match the layout")
    if up_k.shape != (layout.sum_k, head_dim) or (up_v is not None and up_v.shape != (layout.sum_v, head_dim)):
        raise ValueError("up-factors must be [sum r, head_dim]")
    dev = q.device
    if out is None and up_v is not None:
        out = alloc_tensor_func((B, q_head_num, head_dim), dtype=torch.float16, device=dev)
    if out_latent is None and up_v is None:
        out_latent = alloc_tensor_func((B, layout.sum_v), dtype=torch.float16, device=dev)
    need = attn_decode_workspace_bytes(B, layout, infer_state.max_len_in_batch)
    if workspace is None:
        workspace = alloc_tensor_func((need,), dtype=torch.uint8, device=dev)
    r2t = infer_state.req_manager.req_to_token_indexs
    a = _lib.AttnDecodeArgs()
    a.batch, a.num_heads, a.head_dim = B, q_head_num, head_dim
    a.max_len_in_batch = int(infer_state.max_len_in_batch)
    a.sm_scale = float(sm_scale) if sm_scale is not None else 0.0
    a.num_slots = layout.num_slots_of(cache_latent_k, "k")
    a.cache_layout = _lib.CACHE_HEAD_MAJOR if hm else _lib.CACHE_SLOT_MAJOR
    a.q, a.q_stride_b, a.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    a.k_off, a.v_off = layout.off_c("k"), layout.off_c("v")
    a.cache_k, a.cache_k_row_stride = cache_latent_k.data_ptr(), 0 if hm else cache_latent_k.stride(0)
    a.scale_k, a.scale_k_row_stride = cache_latent_k_scale.data_ptr(), 0 if hm else cache_latent_k_scale.stride(0)
    a.cache_v, a.cache_v_row_stride = cache_latent_v.data_ptr(), 0 if hm else cache_latent_v.stride(0)
    a.scale_v, a.scale_v_row_stride = cache_latent_v_scale.data_ptr(), 0 if hm else cache_latent_v_scale.stride(0)
    a.up_k, a.up_k_row_stride = up_k.data_ptr(), up_k.stride(0)
    if up_v is not None:
        a.up_v, a.up_v_row_stride = up_v.data_ptr(), up_v.stride(0)
    a.req_to_token, a.req_to_token_stride = r2t.data_ptr(), r2t.stride(0)
    a.req_to_token_rows = r2t.shape[0]
    a.b_req_idx, a.b_seq_len = infer_state.b_req_idx.data_ptr(), infer_state.b_seq_len.data_ptr()
    if out is not None:
        a.out, a.out_stride_b, a.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
    if out_latent is not None:
        a.out_latent, a.out_latent_stride_b = out_latent.data_ptr(), out_latent.stride(0)
    a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    a.status_word = status_word.data_ptr() if status_word is not None else None
    if timing_events is not None:        # (begin, end) torch.cuda.Event pair around the cache-streaming kernel
        a.ev_stream_begin, a.ev_stream_end = timing_events[0].cuda_event, timing_events[1].cuda_event
    _lib.check(lib.lsvd_attn_decode(C.byref(a), _stream_ptr(q)))
    return out if out is not None else out_latent


class LatentDecodeAttention(nn.Module):
    """Decode attention over an int8 latent KV cache with per-head fp16 up-factors (``absorb`` form).

    Holds ``up_k [sum r_k, D]`` and ``up_v [sum r_v, D]`` (the per-head ``B_k`` / ``B_v`` of the latent
    factorisation stacked by head) and a persistent workspace, so a decode step allocates nothing.
    ``forward`` appends the step's K/V latents to the cache (in place, like the reference's
    ``Int8AttentionBlock`` does at kernels/layer_bench/ffn_kernel/baseline_kernel.py:129-130) when they
    are given, then attends.
    """

    def __init__(self, layout: LatentCacheLayout, head_dim: int, up_k: torch.Tensor, up_v: torch.Tensor,
                 rounding: str = "torch"):
        super().__init__()
        self.layout = layout
        self.head_dim = head_dim
        self.rounding = rounding
        self.register_buffer("up_k", up_k.to(torch.float16).contiguous())
        self.register_buffer("up_v", up_v.to(torch.float16).contiguous())
        self._workspace = None

    def _ws(self, batch, max_len, device):
        need = attn_decode_workspace_bytes(batch, self.layout, max_len)
        if self._workspace is None or self._workspace.numel() < need or self._workspace.device != device:
            self._workspace = torch.empty(need, dtype=torch.uint8, device=device)
        return self._workspace

    @torch.no_grad()
    def forward(self, q, cache_k, scale_k, cache_v, scale_v, infer_state, latent_k=None, latent_v=None, out=None):
        if q.dim() == 4:
            if q.shape[1] != 1:
                raise ValueError(f"latent decode attention only supports query_len=1, got {q.shape[1]}")
            q = q[:, 0]
        if latent_k is not None or latent_v is not None:
            hm = self.layout.head_major
            cache_append(self.layout, latent_k, latent_v, infer_state.mem_index,
                         cache_k if hm else cache_k.view(cache_k.shape[0], -1), scale_k,
                         cache_v if hm else cache_v.view(cache_v.shape[0], -1), scale_v, rounding=self.rounding)
        ws = self._ws(infer_state.batch_size, infer_state.max_len_in_batch, q.device)
        return token_decode_attention_int8_latent_absorb(
            q, infer_state, self.layout.num_heads, self.head_dim, cache_k, scale_k, cache_v, scale_v,
            self.up_k, self.up_v, layout=self.layout, out=out, workspace=ws)


@torch.no_grad()
def token_decode_attention_flash_int8_latent_per_head_decoding_rope(
        q, infer_state, q_head_num: int, head_dim: int,
        cache_latent_k, cache_latent_k_scale, cache_latent_v, cache_latent_v_scale, wk, wk_scale,
        out=None, alloc_tensor_func=torch.empty, block_seq: int = 256, rope_theta: float = 10000.0,
        sm_scale: Optional[float] = None, workspace=None, status_word=None):
    """The reference's decode attention under its own name and argument list
    (kernels/layer_bench/fd_kernel/flash_decoding.py:3-17): int8 K up-factor ``wk [R_k, H_kv*D]`` with fp16 column
    scales ``wk_scale [1, H_kv*D]``, keys rebuilt and rotated per token, caches ``[N, H_kv, R]`` int8 with scales
    ``[N, H_kv]`` fp16, grouped-query heads when ``H_kv < q_head_num``.  Returns ``o [B, H, R_v]`` fp16 in the value
    latent space, as the reference does.  ``alloc_tensor_func`` provides the output and the workspace."""
    _require_cuda(q, cache_latent_k, cache_latent_v, wk)
    lib = _lib.load()
    B = infer_state.batch_size
    if cache_latent_k.dim() != 3 or cache_latent_v.dim() != 3:
        raise ValueError("latent caches must be [N, H_kv, R]")
    if q.dtype != torch.float16 or wk.dtype != torch.int8 or wk_scale.dtype != torch.float16:
        raise ValueError("q fp16, wk int8 and wk_scale fp16 are expected")
    N, Hkv, Rk = cache_latent_k.shape
    Rv = cache_latent_v.shape[-1]
    if q_head_num % Hkv:
        raise ValueError("q_head_num must be a multiple of the number of kv heads")
    if tuple(wk.shape) != (Rk, Hkv * head_dim) or wk_scale.numel() != Hkv * head_dim:
        raise ValueError("wk must be [R_k, H_kv*D] and wk_scale [1, H_kv*D]")
    q = q.view(B, q_head_num, head_dim)
    if q.stride(2) != 1:
        q = q.contiguous()
    for t in (cache_latent_k, cache_latent_v):
        if t.stride(2) != 1:
            raise ValueError("the rank dimension of the caches must be contiguous")
    if cache_latent_k_scale.stride(-1) != 1 or cache_latent_v_scale.stride(-1) != 1 or wk.stride(1) != 1:
        raise ValueError("scales and wk must have unit inner stride")
    dev = q.device
    if out is None:
        out = alloc_tensor_func((B, q_head_num, Rv), dtype=torch.float16, device=dev)
    max_len = int(infer_state.max_len_in_batch)
    need = lib.lsvd_attn_decode_rope_workspace_bytes(B, q_head_num, head_dim, Rv, max_len, block_seq)
    if workspace is None:
        workspace = alloc_tensor_func((max(need, 256),), dtype=torch.uint8, device=dev)
    r2t = infer_state.req_manager.req_to_token_indexs
    wk_scale = wk_scale.reshape(-1)
    a = _lib.AttnRopeArgs()
    a.batch, a.num_q_heads, a.num_kv_heads, a.head_dim, a.rank_k, a.rank_v = B, q_head_num, Hkv, head_dim, Rk, Rv
    a.q, a.q_stride_b, a.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    a.cache_k, a.cache_k_slot_stride, a.cache_k_head_stride = cache_latent_k.data_ptr(), cache_latent_k.stride(0), cache_latent_k.stride(1)
    a.scale_k, a.scale_k_slot_stride = cache_latent_k_scale.data_ptr(), cache_latent_k_scale.stride(0)
    a.cache_v, a.cache_v_slot_stride, a.cache_v_head_stride = cache_latent_v.data_ptr(), cache_latent_v.stride(0), cache_latent_v.stride(1)
    a.scale_v, a.scale_v_slot_stride = cache_latent_v_scale.data_ptr(), cache_latent_v_scale.stride(0)
    a.wk, a.wk_row_stride, a.wk_scale = wk.data_ptr(), wk.stride(0), wk_scale.data_ptr()
    a.req_to_token, a.req_to_token_stride = r2t.data_ptr(), r2t.stride(0)
    a.b_req_idx, a.b_seq_len = infer_state.b_req_idx.data_ptr(), infer_state.b_seq_len.data_ptr()
    a.num_slots, a.max_len_in_batch, a.block_seq = N, max_len, block_seq
    a.sm_scale = float(sm_scale) if sm_scale is not None else 0.0
    a.rope_theta = float(rope_theta)
    a.out, a.out_stride_b, a.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
    a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    a.status_word = status_word.data_ptr() if status_word is not None else None
    _lib.check(lib.lsvd_attn_decode_rope(C.byref(a), _stream_ptr(q)))
    return out
