"""lsvd_b200: B200 (sm_100a) kernels for the LSVD decode hot paths behind the reference's PyTorch API.

Python here is host plumbing only (argument checks, pointers, streams); the work
is done by hand-written CUDA kernels in ``liblsvd_b200.so``, reached through a
plain C ABI (``include/lsvd_b200.h``).  There is no CPU or PyTorch fallback.
"""
from . import _lib
from ._lib import LsvdError
from .attention import (LatentCacheLayout, destindex_copy_quantize_latent, cache_append,
                        token_decode_attention_int8_latent_absorb,
                        token_decode_attention_flash_int8_latent_per_head_decoding_rope, LatentDecodeAttention, InferState)
from .block import Int8AttentionBlock
from .mixffn import MixedFFNGateUpDenseLatentFused, b200_mixffn
from .ffn import (HybridFFN, quantize_weight_rtn, act_quant, hadamard_pack, hadamard_quant, heads_hadamard_quant, w8a8_gemv,
                  i8gemm)

from .modules import ActQuantizer, ActQuantWrapper, SVDLinear, add_actquant, find_qlayers
from .formats import load_channel_groups, resolve_channel_group, load_qmodel, hybrid_ffn_weights, load_hybrid_ffn, int8_from_fake_quant

__all__ = ["ActQuantizer", "ActQuantWrapper", "SVDLinear", "add_actquant", "find_qlayers", "load_channel_groups",
           "resolve_channel_group", "load_qmodel", "hybrid_ffn_weights", "load_hybrid_ffn", "int8_from_fake_quant",
           "LsvdError", "LatentCacheLayout", "destindex_copy_quantize_latent", "cache_append",
           "token_decode_attention_int8_latent_absorb", "token_decode_attention_flash_int8_latent_per_head_decoding_rope",
           "LatentDecodeAttention", "InferState", "Int8AttentionBlock", "MixedFFNGateUpDenseLatentFused", "b200_mixffn", "HybridFFN", "quantize_weight_rtn", "act_quant", "hadamard_pack",
           "hadamard_quant", "heads_hadamard_quant", "w8a8_gemv", "i8gemm"]
