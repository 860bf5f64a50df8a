"""The CPU oracle against outputs of the reference's own code (fixtures made by tests/golden/make_golden.py)."""
import torch

from conftest import load_golden, unpack_had, rel_to_norm
from oracle import quant, attention, ffn


def test_latent_quant_matches_reference_pytorch_quantiser():
    g = load_golden("latent_quant")
    q, s = quant.latent_quant(g["x"], "torch")
    assert torch.equal(s, g["s_torch"])
    assert torch.equal(q, g["q_torch"])


def test_latent_append_matches_reference_triton_kernel():
    g = load_golden("latent_quant")
    T, H, R = g["x"].shape
    offs = [h * R for h in range(H + 1)]
    cache = torch.zeros(64, H * R, dtype=torch.int8)
    scale = torch.zeros(64, H, dtype=torch.float16)
    attention.cache_append(g["x"].reshape(T, H * R), g["dest_loc"], offs, cache, scale, rounding="triton")
    assert torch.equal(scale, g["scale_triton"])
    assert torch.equal(cache.view(64, H, R), g["cache_triton"])
    # the two roundings do differ on this input, so the test above can tell them apart
    q_t, _ = quant.latent_quant(g["x"], "torch")
    q_r, _ = quant.latent_quant(g["x"], "triton")
    assert (q_t != q_r).any()


def test_wuk_quant_matches_reference():
    g = load_golden("wuk_quant")
    q, s = quant.wuk_quant(g["wuk"])
    assert torch.equal(s, g["wuk_scale"])
    assert torch.equal(q, g["wuk_q"])


def test_act_and_weight_quantisers_match_reference():
    g = load_golden("fq_quantizers")
    q, s = quant.act_quant(g["x"])
    assert torch.equal(s, g["a_scale"])
    assert torch.equal(q.float(), g["a_codes"])
    assert torch.equal((s[:, None] * q.float()).half(), g["a_fake"])
    for tag, mse in (("rtn", False), ("mse", True)):
        wq, ws = quant.weight_quant_rtn(g["W"], mse=mse)
        assert torch.equal(ws, g["w_scale_" + tag].flatten())
        assert torch.equal(wq.float(), g["w_codes_" + tag])


def test_hadamard_matches_reference():
    g = load_golden("hadamard")
    for n, K in ((64, 1), (688, 172), (864, 108)):
        assert g[f"K_{n}"] == K
        hk = unpack_had(g[f"had{K}_bits"], K) if K > 1 else None
        y = ffn.hadamard_full(g[f"x_{n}"], hk, K)
        # the two implementations add the same fp16 numbers in a different order: allow one fp16 ulp
        d = (y.float() - g[f"y_{n}"].float()).abs()
        assert d.max() <= 2 ** -10 * g[f"y_{n}"].float().abs().max()
        assert (d == 0).float().mean() > 0.9
    for K in (172, 108):
        hk = unpack_had(g[f"had{K}_bits"], K)
        assert torch.equal(hk @ hk.t(), K * torch.eye(K))
    y = ffn.input_rotation(g["rot_x"], g["rot_sign"])
    assert (y.float() - g["rot_y"].float()).abs().max() <= 2 ** -10 * g["rot_y"].float().abs().max()


def test_rope_recon_attention_matches_reference_triton_kernels():
    g = load_golden("attn_rope_recon")
    o = attention.decode_rope_recon(g["q"], g["cache_k"], g["scale_k"], g["cache_v"], g["scale_v"], g["wk_q"],
                                    g["wk_scale"], g["req_to_token"], g["b_req_idx"], g["b_seq_len"], gqa_group=2)
    for tag in ("o_a", "o_b"):
        assert rel_to_norm(o.float(), g[tag].float()) < 5e-4
    # the kernel's own two block configurations agree with each other no better than that
    assert rel_to_norm(g["o_a"].float(), g["o_b"].float()) < 5e-4


def test_absorb_equals_reconstruct_form():
    gen = torch.Generator().manual_seed(3)
    B, H, D, N = 3, 4, 32, 200
    rk = [16, 48, 32, 16]
    rv = [32, 16, 16, 64]
    k_off = [0]
    v_off = [0]
    for a, b in zip(rk, rv):
        k_off.append(k_off[-1] + a)
        v_off.append(v_off[-1] + b)
    lk = torch.randn(N, k_off[-1], generator=gen).half()
    lv = torch.randn(N, v_off[-1], generator=gen).half()
    ck, sk = quant.latent_quant_ragged(lk, k_off)
    cv, sv = quant.latent_quant_ragged(lv, v_off)
    up_k = (torch.randn(k_off[-1], D, generator=gen) / 8).half()
    up_v = (torch.randn(v_off[-1], D, generator=gen) / 8).half()
    q = torch.randn(B, H, D, generator=gen).half()
    r2t = torch.randperm(N, generator=gen).to(torch.int32).view(2, 100)
    r2t = torch.cat([r2t, r2t[:1]], 0)
    breq = torch.tensor([1, 0, 2], dtype=torch.int32)
    blen = torch.tensor([100, 63, 1], dtype=torch.int32)
    o, o_lat = attention.decode_absorb(q, ck, sk, cv, sv, up_k, up_v, k_off, v_off, r2t, breq, blen)
    o_lat2 = attention.decode_reconstruct(q, ck, sk, cv, sv, up_k, k_off, v_off, r2t, breq, blen)
    assert rel_to_norm(o_lat, o_lat2) < 1e-6
    assert o.shape == (B, H, D) and torch.isfinite(o.float()).all()


def _ffn_weights_from_golden(g):
    K = g["K"]
    return {
        "had_sign": None, "K": K, "had_K": unpack_had(g["had_bits"], K),
        "U_q": torch.cat([g["Ug_q"], g["Uu_q"]]), "U_s": torch.cat([g["Ug_s"], g["Uu_s"]]),
        "Vg_q": g["Vg_q"], "Vg_s": g["Vg_s"], "Vu_q": g["Vu_q"], "Vu_s": g["Vu_s"],
        "Wg_q": g["Wg_q"], "Wg_s": g["Wg_s"], "Wu_q": g["Wu_q"], "Wu_s": g["Wu_s"],
        "Wd_q": g["Wd_q"], "Wd_s": g["Wd_s"],
    }


def test_hybrid_ffn_integer_form_matches_reference_module():
    """Integer-form FFN vs the reference's fake-quant HybridSVDQuantFFN run in fp16 on the CPU.

    The reference multiplies fp16-rounded dequantised numbers; the integer form multiplies the codes and
    scales once at the end.  Stage outputs therefore agree to fp16 rounding, and the final output within
    the 2e-3 * ||y|| tolerance of the specification (observed: far below).
    """
    g = load_golden("hybrid_ffn")
    w = _ffn_weights_from_golden(g)
    st = ffn.hybrid_ffn_stages(g["x"], w)
    r = g["Ug_q"].shape[0]
    n_svd = g["Vg_q"].shape[0]
    # latents after the output quantiser: dequantised codes vs the reference's fake-quantised latent
    latg = (st["latg_q"].float() * st["latg_s"][:, None]).half()
    latu = (st["latu_q"].float() * st["latu_s"][:, None]).half()
    assert rel_to_norm(latg.float(), g["latg"].float()) < 2e-3
    assert rel_to_norm(latu.float(), g["latu"].float()) < 2e-3
    assert rel_to_norm(st["g16"][:, :n_svd].float(), g["g_svd"].float()) < 2e-3
    assert rel_to_norm(st["u16"][:, n_svd:].float(), g["u_rtn"].float()) < 2e-3
    assert rel_to_norm(st["h_rot"].float(), g["h"].float()) < 2e-3   # the hook sees h after the Hadamard
    hq = (st["h_q"].float() * st["h_s"][:, None]).half()
    assert rel_to_norm(hq.float(), g["h_fakeq"].float()) < 2e-3
    assert rel_to_norm(st["out"].float(), g["y"].float()) < 2e-3
    assert r == 64


def test_hybrid_ffn_stage_isolation_is_exact():
    """Fed the reference's own stage inputs, the integer stages reproduce the reference's next stage."""
    g = load_golden("hybrid_ffn")
    w = _ffn_weights_from_golden(g)
    # (a) A8 quantiser of the reference's rotated h: dequantised codes are bit-equal to its fake-quantised tensor
    q, s = quant.act_quant(g["h"])
    assert torch.equal((s[:, None] * q.float()).half(), g["h_fakeq"])
    # (b) int32 down projection of those codes, dequantised, vs the reference's fp16 Linear on the fake-quantised h
    acc = ffn.stage_from("i32", w, a_q=q, w_q=w["Wd_q"])["acc"]
    y = ((acc.float() * s[:, None]) * w["Wd_s"][None, :]).half()
    assert rel_to_norm(y.float(), g["y"].float()) < 1e-3


def test_partial_hadamard_across_heads_matches_reference_wrapper():
    g = load_golden("partial_hadamard")
    y = ffn.partial_hadamard_heads(g["x"], g["head_dim"])
    assert (y.float() - g["rotated"].float()).abs().max() <= 2 ** -10 * g["rotated"].float().abs().max()
    q, s = quant.act_quant(g["rotated"])
    assert torch.equal((q.float() * s[:, None]).half(), g["fake_quant"])
    y28 = ffn.partial_hadamard_heads_hadk(g["x28"], g["head_dim"], g["had28"].float())
    assert (y28.float() - g["rotated28"].float()).abs().max() <= 2 ** -10 * g["rotated28"].float().abs().max()


def test_int8_attention_block_against_the_reference_module():
    """The oracle's restatement of the whole attention block against one decode step of the reference's module
    (projections by PyTorch on the CPU, append and attention kernels in the Triton interpreter)."""
    from oracle import layer as olayer
    g = load_golden("attention_block")
    ck, sk, cv, sv = (g[k].clone() for k in ("cache_k", "scale_k", "cache_v", "scale_v"))
    y = olayer.int8_attention_block(g["x"], g, ck, sk, cv, sv, g["req_to_token"], g["b_req_idx"], g["b_seq_len"],
                                    g["mem_index"], int(g["num_heads"]), int(g["head_dim"]))
    # the appended rows: bit-exact codes and scales; every other row untouched
    assert torch.equal(ck, g["cache_k_after"]) and torch.equal(cv, g["cache_v_after"])
    assert torch.equal(sk, g["scale_k_after"]) and torch.equal(sv, g["scale_v_after"])
    rows = g["mem_index"].long()
    assert not torch.equal(g["cache_k"][rows], g["cache_k_after"][rows])
    assert rel_to_norm(y.float(), g["y"].float()) < 5e-4


def test_attention_block_derived_buffers_match_the_reference():
    """lsvd_b200.block.Int8AttentionBlock derives wuk_q / wuk_scale / wuvout from the parameters as the reference does."""
    from lsvd_b200.block import Int8AttentionBlock
    g = load_golden("attention_block")
    H, D, R = int(g["num_heads"]), int(g["head_dim"]), int(g["rank_head"])
    blk = Int8AttentionBlock(H * D, H, D, (R + 0.5) / D, device="cpu")
    assert blk.rank_head == R
    with torch.no_grad():
        for name in ("up_proj_q", "up_proj_k", "up_proj_v", "input_layernorm_weight"):
            getattr(blk, name).copy_(g[name])
        for name in ("down_proj_q", "down_proj_kv", "o_proj"):
            getattr(blk, name).weight.copy_(g[name])
    blk.refresh()
    assert torch.equal(blk.wuk_q, g["wuk_q"]) and torch.equal(blk.wuk_scale, g["wuk_scale"])
    assert rel_to_norm(blk.wuvout.float(), g["wuvout"].float()) < 1e-3
    same = Int8AttentionBlock.from_module(blk)
    assert torch.equal(same.wuk_q, blk.wuk_q) and torch.equal(same.w_latent, blk.w_latent)


def _mix_weights(g):
    return {k: v for k, v in g.items() if not k.startswith(("st_", "fp16_")) and k not in ("x", "eps")}


def test_mixffn_pipeline_against_the_reference_stage_by_stage():
    """oracle.mixffn.forward_stages against the reference's forward_stages (its eleven Triton kernels, interpreter)."""
    from oracle import mixffn
    g = load_golden("mixffn")
    x = g["x"].reshape(-1, g["x"].shape[-1])
    st = mixffn.forward_stages(x, _mix_weights(g), eps=float(g["eps"]))
    exact = ["x_q", "x_scale", "up_svd_rank_fp", "gate_svd_rank_fp", "up_svd_rank_scale", "gate_svd_rank_scale",
             "up_svd_rank_q", "gate_svd_rank_q", "up_dense_out_acc", "gate_dense_out_acc", "svd_mid_scale",
             "dense_mid_scale", "mid_scale", "mid_q", "down_svd_rank_acc", "down_svd_rank_scale", "down_svd_rank_q",
             "down_svd_out_fp", "down_dense_out_fp", "down_fp"]
    for name in exact:
        assert torch.equal(st[name], g["st_" + name]), name
    # SwiGLU outputs: sigmoid implementations may differ in the last bit of fp32, visible as one fp16 ulp at most
    for name in ("svd_mid_fp", "dense_mid_fp"):
        a, b = st[name].float(), g["st_" + name].float()
        assert ((a - b).abs() <= 1e-3 * b.abs() + 1e-7).all(), name
    assert torch.equal(st["out"], g["st_out"].reshape(st["out"].shape))
    # the token of zeros: scales at their floor, the residual passes through
    assert st["x_scale"][3] == 0 and (st["out"][3] == 0).all()


def test_mixffn_weight_conversion_matches_the_reference():
    from oracle import mixffn
    g = load_golden("mixffn")
    for name, key in (("up", "fp16_up_w"), ("gate", "fp16_gate_w"), ("down", "fp16_down_w")):
        w = g[key]
        s = mixffn.svd_out_from_ratio(w.shape[0], 0.5, 64)
        assert s == g[name + "_b_q"].shape[0]
        assert mixffn.rounded_rank(w.shape[1], s, 0.5, 64) == g[name + "_a_q"].shape[0]
        q, sc = mixffn.quantize_weights_per_channel(w[s:].contiguous())
        assert torch.equal(q, g[name + "_q"]) and torch.equal(sc, g[name + "_scale"])
