"""Helpers shared by the GPU parity tests: build a cache with the CPU oracle, upload, run, compare."""
import torch

from oracle import quant, attention as oattn
from lsvd_b200 import synth
from lsvd_b200.attention import LatentCacheLayout, InferState, token_decode_attention_int8_latent_absorb


def offsets(ranks):
    off = [0]
    for r in ranks:
        off.append(off[-1] + r)
    return off


def build_case(batch, num_heads, head_dim, k_ranks, v_ranks, seq_lens, seed=0, shuffle=False, extra_slots=0):
    """Synthetic inputs + the cache quantised on the CPU by the oracle (the reference's PyTorch quantiser)."""
    c = synth.attention_inputs(batch, num_heads, head_dim, k_ranks, v_ranks, seq_lens, seed, shuffle, extra_slots)
    c["k_off"], c["v_off"] = offsets(k_ranks), offsets(v_ranks)
    c["cache_k"], c["scale_k"] = quant.latent_quant_ragged(c["latent_k"], c["k_off"])
    c["cache_v"], c["scale_v"] = quant.latent_quant_ragged(c["latent_v"], c["v_off"])
    c["layout"] = LatentCacheLayout(k_ranks, v_ranks)
    c["batch"], c["num_heads"], c["head_dim"] = batch, num_heads, head_dim
    return c


def run_gpu(c, want="out", status=None, head_major=False):
    """The kernels on the case's cache; ``head_major`` re-stores the cache head by head first (same values)."""
    dev = "cuda"
    st = InferState(c["batch"], c["max_len"], c["b_seq_len"], device=dev, req_to_token=c["req_to_token"],
                    b_req_idx=c["b_req_idx"])
    lay = c["layout"]
    ck, sk, cv, sv = c["cache_k"], c["scale_k"], c["cache_v"], c["scale_v"]
    if head_major:
        lay = lay.as_head_major()
        ck, sk = lay.to_head_major(ck, sk, "k")
        cv, sv = lay.to_head_major(cv, sv, "v")
    args = [c["q"].to(dev), st, c["num_heads"], c["head_dim"], ck.to(dev), sk.to(dev), cv.to(dev), sv.to(dev), c["up_k"].to(dev)]
    if want == "out":
        o = token_decode_attention_int8_latent_absorb(*args, c["up_v"].to(dev), layout=lay, status_word=status)
    else:
        o = token_decode_attention_int8_latent_absorb(*args, None, layout=lay, status_word=status)
    torch.cuda.synchronize()
    return o.cpu()


def run_oracle(c):
    return oattn.decode_absorb(c["q"], c["cache_k"], c["scale_k"], c["cache_v"], c["scale_v"], c["up_k"], c["up_v"],
                               c["k_off"], c["v_off"], c["req_to_token"], c["b_req_idx"], c["b_seq_len"])
