"""The reference's int8 latent attention block as a module over this library's kernels.

``Int8AttentionBlock`` takes the place of the class of the same name in
kernels/layer_bench/ffn_kernel/baseline_kernel.py:56-145: the same parameters (``down_proj_q``, ``down_proj_kv``,
``up_proj_q``, ``up_proj_k``, ``up_proj_v``, ``o_proj``, ``input_layernorm_weight``), the same derived buffers
(``wuk_q``, ``wuk_scale``, ``wuvout``), the same ``forward`` arguments and the same in-place cache update.  Its
decode step is

    RMSNorm (library kernel)  ->  one fp16 GEMM for [q | K | V] latents  ->  per-head query up-projection
    ->  quantise + append of the K and V latents (one library launch for both sides)
    ->  int8 latent decode attention with rebuilt, rotated keys (library kernels)
    ->  fp16 GEMM with the composed V-up/output factor, plus the normalised input as residual

The three dense fp16 products stay library GEMMs, as they are in the reference; everything that touches the int8
cache runs in this library's CUDA kernels.  For the all-int8 layer see ``lsvd_b200.layer.LSVDDecoderLayer``.
"""
from __future__ import annotations

import torch
from torch import nn

from .attention import (LatentCacheLayout, cache_append,
                        token_decode_attention_flash_int8_latent_per_head_decoding_rope as _rope_attention)
from .ffn import act_quant


def quantize_wuk(wuk: torch.Tensor):
    """int8 codes and fp16 column scales of the K up-factor ``[R, H*D]``: scale = max|column| / 128 floored at 1e-4,
    codes = round(w / scale) clamped to [-128, 127]  (baseline_kernel.py:102-106)."""
    scale = (wuk.abs().amax(dim=0, keepdim=True) / 128).clamp_min(1e-4).to(torch.float16)
    codes = torch.round(wuk / scale).clamp_(-128, 127).to(torch.int8)
    return codes.contiguous(), scale.contiguous()


class Int8AttentionBlock(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rank_ratio: float, device="cuda",
                 dtype: torch.dtype = torch.float16, rope_theta: float = 10000.0, block_seq: int = 256):
        super().__init__()
        if hidden_size != num_heads * head_dim:
            raise ValueError("hidden_size must equal num_heads * head_dim")
        if dtype != torch.float16:
            raise ValueError("the block computes in fp16")
        self.hidden_size, self.num_heads, self.head_dim = hidden_size, num_heads, head_dim
        self.rank_head = max(1, int(rank_ratio * head_dim))
        self.rope_theta, self.block_seq = rope_theta, block_seq
        lat = num_heads * self.rank_head
        kw = dict(bias=False, device=device, dtype=dtype)
        self.down_proj_q = nn.Linear(hidden_size, lat, **kw)
        self.down_proj_kv = nn.Linear(hidden_size, 2 * lat, **kw)          # [K latents of all heads | V latents]
        self.o_proj = nn.Linear(hidden_size, hidden_size, **kw)
        for name in ("up_proj_q", "up_proj_k", "up_proj_v"):
            p = nn.Parameter(torch.empty(self.rank_head, hidden_size, device=device, dtype=dtype))
            nn.init.xavier_uniform_(p)
            setattr(self, name, p)
        for lin in (self.down_proj_q, self.down_proj_kv, self.o_proj):
            nn.init.xavier_uniform_(lin.weight)
        self.input_layernorm_weight = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        self.refresh()

    @classmethod
    def from_module(cls, block, rope_theta: float = 10000.0, block_seq: int = 256):
        """Take over the parameters of a reference ``Int8AttentionBlock`` (or any module with its attribute names)."""
        w = block.down_proj_q.weight
        rank_ratio = (block.rank_head + 0.5) / block.head_dim
        new = cls(block.hidden_size, block.num_heads, block.head_dim, rank_ratio, device=w.device, dtype=w.dtype,
                  rope_theta=rope_theta, block_seq=block_seq)
        with torch.no_grad():
            for name in ("up_proj_q", "up_proj_k", "up_proj_v", "input_layernorm_weight"):
                getattr(new, name).copy_(getattr(block, name))
            for name in ("down_proj_q", "down_proj_kv", "o_proj"):
                getattr(new, name).weight.copy_(getattr(block, name).weight)
        new.refresh()
        return new

    @torch.no_grad()
    def refresh(self):
        """Rebuild what is derived from the parameters: the int8 K up-factor, the composed V-up/output factor
        (per head ``W_uv,h @ W_o,h``, baseline_kernel.py:97-100) and the stacked latent projection."""
        H, R, D, hid = self.num_heads, self.rank_head, self.head_dim, self.hidden_size
        wuk_q, wuk_scale = quantize_wuk(self.up_proj_k.detach())
        wuv = self.up_proj_v.detach().view(H, R, D)
        wout = self.o_proj.weight.detach().t().contiguous().view(H, D, hid)
        self.register_buffer("wuk_q", wuk_q, persistent=False)
        self.register_buffer("wuk_scale", wuk_scale, persistent=False)
        self.register_buffer("wuvout", (wuv @ wout).reshape(H * R, hid).contiguous(), persistent=False)
        self.register_buffer("w_latent", torch.cat([self.down_proj_q.weight.detach(), self.down_proj_kv.weight.detach()])
                             .contiguous(), persistent=False)
        self.layout = LatentCacheLayout.uniform(H, R, R)
        self._workspace = None

    @torch.no_grad()
    def forward(self, x, cache_latent_k, cache_latent_k_scale, cache_latent_v, cache_latent_v_scale, infer_state):
        """x [B, 1, hidden] fp16; caches ``[N, H, R]`` int8 with scales ``[N, H]`` fp16.  Writes the step's K and V
        latents into rows ``infer_state.mem_index`` and returns ``[B, 1, hidden]``."""
        bsz, q_len, hid = x.shape
        if q_len != 1:
            raise ValueError(f"Int8 latent attention only supports decode query_len=1, got {q_len}")
        H, R, D = self.num_heads, self.rank_head, self.head_dim
        _, _, xn = act_quant(x.view(bsz, hid), want_rotated=True, norm_weight=self.input_layernorm_weight, norm_eps=1e-5)
        lat = xn @ self.w_latent.t()                                   # [B, 3*H*R]: q | K | V latents
        HR = H * R
        # the reference reads the [R, H*D] query up-factor as [H, R, D] (baseline_kernel.py:123), and so does this
        q = torch.bmm(lat[:, :HR].view(bsz, H, R).transpose(0, 1), self.up_proj_q.view(H, R, D)).transpose(0, 1)
        cache_append(self.layout, lat[:, HR:2 * HR], lat[:, 2 * HR:], infer_state.mem_index,
                     cache_latent_k.view(cache_latent_k.shape[0], -1), cache_latent_k_scale,
                     cache_latent_v.view(cache_latent_v.shape[0], -1), cache_latent_v_scale, rounding="triton")
        lib_need = self._workspace_bytes(bsz, int(infer_state.max_len_in_batch))
        if self._workspace is None or self._workspace.numel() < lib_need or self._workspace.device != x.device:
            self._workspace = torch.empty(lib_need, dtype=torch.uint8, device=x.device)
        o = _rope_attention(q, infer_state, H, D, cache_latent_k, cache_latent_k_scale, cache_latent_v,
                            cache_latent_v_scale, self.wuk_q, self.wuk_scale, block_seq=self.block_seq,
                            rope_theta=self.rope_theta, workspace=self._workspace)
        return (o.view(bsz, HR) @ self.wuvout + xn).view(bsz, 1, hid)

    def _workspace_bytes(self, batch: int, max_len: int) -> int:
        from . import _lib
        need = _lib.load().lsvd_attn_decode_rope_workspace_bytes(batch, self.num_heads, self.head_dim, self.rank_head,
                                                                 max_len, self.block_seq)
        return max(int(need), 256)
