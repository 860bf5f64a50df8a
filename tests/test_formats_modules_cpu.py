"""On-disk formats and the attribute surface of the drop-in modules, on the CPU.

Fixtures (tests/golden/make_golden.py ``modules``) were written by the reference's own code: ``channel_groups.json`` in the
layout of the analysis pass and accepted by the reference's ``load_channel_groups``; ``qmodel_ffn.pt`` by ``torch.save`` of
``{"model": state_dict, "w_quantizers": ...}`` after the reference's RTN loop with the MSE clip search;
``svd_linear.npz`` / ``act_quant_wrapper.npz`` are inputs and outputs of the reference's modules.
"""
import os

import pytest
import torch
from torch import nn

from conftest import GOLDEN, load_golden, rel_to_norm
from oracle import modules as omod
from lsvd_b200 import formats
from lsvd_b200.modules import ActQuantWrapper, ActQuantizer, SVDLinear, add_actquant, find_qlayers


# ------------------------------------------------------------------------------------------ oracle pins
def _ragged(g, fuse):
    ranks = [int(r) for r in g["ranks"]]
    cout = g["cout"]
    A, c = [], 0
    for r in ranks:
        A.append(g[f"ragged_{fuse}_A"][c:c + cout * r].reshape(cout, r))
        c += cout * r
    return ranks, A


def test_oracle_svd_linear_matches_reference():
    g = load_golden("svd_linear")
    for fuse in ("UV", "U", "V"):
        _, A = _ragged(g, fuse)
        y = omod.svd_linear_per_head(g[f"ragged_{fuse}_x"], g[f"ragged_{fuse}_B"], A, g["bias"] if fuse == "UV" else None)
        assert rel_to_norm(y.float(), g[f"ragged_{fuse}_y"].float()) < 1e-3
    y = omod.svd_linear_per_head(g["uni_x"], g["uni_B"], list(g["uni_A"]))
    assert rel_to_norm(y.float(), g["uni_y"].float()) < 1e-3


def test_oracle_act_quant_wrapper_matches_reference():
    g = load_golden("act_quant_wrapper")
    cases = {
        "plain": dict(bias=g["plain_b"], out_bits=8), "w16": {}, "many": dict(bias=g["many_b"]),
        "full64": dict(rotation="full", K=1), "full64_fp32": dict(rotation="full", K=1),
        "partial": dict(rotation="partial", had_dim=16),
        "full768": dict(rotation="full", K=12, had_K=g["had12"].float()),
        "random": dict(rotation="random", had_K=g["random_Q"]),
    }
    for tag, kw in cases.items():
        kw = dict(kw)
        y = omod.act_quant_wrapper(g[tag + "_x"], g[tag + "_W"], kw.pop("bias", None), **kw)
        ref = g[tag + "_y"].float()
        if tag == "plain":
            # 8-bit output: the codes may differ by one where the fp16 product sits on a rounding boundary
            step = ref.abs().amax(-1, keepdim=True) / 127
            assert ((y.float() - ref).abs() <= 1.01 * step + 1e-6).all()
            assert ((y.float() - ref).abs() > 0.5 * step).float().mean() < 0.05
        else:
            assert rel_to_norm(y.float(), ref) < 2e-3, tag


# ------------------------------------------------------------------------------------------ channel groups
def test_channel_groups_round_trip_and_reslice():
    groups = formats.load_channel_groups(os.path.join(GOLDEN, "channel_groups.json"))
    assert sorted(groups["layers"]) == ["0", "1"]
    l0 = groups["layers"]["0"]
    d_ffn = l0["d_ffn"]
    svd, quant, perm, rank = formats.resolve_channel_group(l0, d_ffn)
    assert rank == 32 and len(svd) == l0["n_svd"] == 96 and perm == svd + quant and sorted(perm) == list(range(d_ffn))
    assert svd == sorted(svd) and quant == sorted(quant)
    # no accept order stored: another ratio cannot be derived, the stored groups come back
    assert formats.resolve_channel_group(l0, d_ffn, n_svd=64)[0] == svd
    l1 = groups["layers"]["1"]
    order = l1["greedy_accept_order"]
    # more RTN channels than stored, fewer than the accept order holds: its first d_ffn - n_svd entries, in that order
    svd2, quant2, perm2, rank2 = formats.resolve_channel_group(l1, d_ffn, n_svd=64)
    assert rank2 is None and quant2 == order[:128] and svd2 == [c for c in range(d_ffn) if c not in set(quant2)]
    assert perm2 == svd2 + quant2
    # more than the accept order holds (150): padded with never-accepted channels in index order
    svd3, quant3, _, _ = formats.resolve_channel_group(l1, d_ffn, n_svd=16)
    rest = [c for c in range(d_ffn) if c not in set(order)]
    assert quant3 == order + rest[:176 - len(order)] and len(svd3) == 16
    # the stored ratio: untouched
    assert formats.resolve_channel_group(l1, d_ffn, n_svd=96)[3] == 32


def test_channel_groups_malformed(tmp_path):
    p = tmp_path / "bad.json"
    p.write_text('{"layerz": {}}')
    with pytest.raises(KeyError):
        formats.load_channel_groups(str(p))
    groups = formats.load_channel_groups(os.path.join(GOLDEN, "channel_groups.json"))
    bad = dict(groups["layers"]["0"])
    bad["perm"] = bad["perm"][:-1] + [bad["perm"][0]]
    with pytest.raises(ValueError):
        formats.resolve_channel_group(bad, bad["d_ffn"])


# ------------------------------------------------------------------------------------------ checkpoints
def test_qmodel_checkpoint_to_int8_buffers():
    """The reference's quantiser classes are not importable here: the loader reads their scales all the same, and the int8
    codes times those scales give back the stored fp16 weights exactly."""
    sd, scales = formats.load_qmodel(os.path.join(GOLDEN, "qmodel_ffn.pt"))
    io = load_golden("qmodel_ffn_io")
    assert len(scales) == 7
    for name, s in scales.items():
        assert torch.equal(s, io[name.replace(".", "__")])
    w = formats.hybrid_ffn_weights(sd, "model.layers.0.mlp", scales)
    assert w["K"] == 12 and w["online_had"] and tuple(w["had_K"].shape) == (12, 12)
    assert w["U_q"].dtype == torch.int8 and tuple(w["U_q"].shape) == (64, 64) and tuple(w["Wd_q"].shape) == (64, 192)
    groups = formats.load_channel_groups(os.path.join(GOLDEN, "channel_groups.json"))
    assert w["perm"].tolist() == groups["layers"]["0"]["perm"]
    pairs = {"Vg": "gate_svd.ALinear", "Vu": "up_svd.ALinear", "Wg": "gate_quant.module", "Wu": "up_quant.module",
             "Wd": "down_proj.module"}
    for short, target in pairs.items():
        stored = sd["model.layers.0.mlp.%s.weight" % target]
        assert torch.equal((w[short + "_s"][:, None] * w[short + "_q"].float()).half(), stored)
    stored = torch.cat([sd["model.layers.0.mlp.gate_svd.BLinear.module.weight"], sd["model.layers.0.mlp.up_svd.BLinear.module.weight"]])
    assert torch.equal((w["U_s"][:, None] * w["U_q"].float()).half(), stored)
    # the clip search shrank some scales: absmax / 127 would not reproduce those rows
    wd = sd["model.layers.0.mlp.down_proj.module.weight"].float()
    assert (w["Wd_s"] < wd.abs().amax(1) / 127 * 0.999).any()


def test_int8_from_fake_quant_without_scales():
    g = load_golden("fq_quantizers")
    q, s = formats.int8_from_fake_quant(g["w_fake_rtn"])
    assert torch.equal(q.float(), g["w_codes_rtn"])
    nz = g["w_codes_rtn"].abs().amax(1) > 0
    assert ((s[nz] - g["w_scale_rtn"].flatten()[nz]).abs() <= 2e-4 * s[nz]).all()
    with pytest.raises(ValueError):
        formats.int8_from_fake_quant((torch.randn(8, 64, generator=torch.Generator().manual_seed(0)) * 0.1).half())
    with pytest.raises(ValueError):
        formats.int8_from_fake_quant(g["w_fake_rtn"], torch.ones(3))


# ------------------------------------------------------------------------------------------ module surfaces
def test_svd_linear_constructor_matches_reference_factors():
    g = load_golden("svd_linear")
    ranks = [int(r) for r in g["ranks"]]
    cout, cin = g["cout"], g["cin"]
    U, S, V, cu, cs, cv = [], [], [], 0, 0, 0
    for r in ranks:
        U.append(g["U"][cu:cu + cout * r].reshape(cout, r)); cu += cout * r
        S.append(g["S"][cs:cs + r]); cs += r
        V.append(g["V"][cv:cv + cin * r].reshape(cin, r)); cv += cin * r
    for fuse in ("UV", "U", "V"):
        m = SVDLinear(U, S, V, bias=g["bias"] if fuse == "UV" else None, sigma_fuse=fuse, is_per_head_svd=True, rank_split=ranks)
        assert isinstance(m.ALinear, nn.ParameterList) and len(m.ALinear) == m.head_num == 4 and m.rank_split == ranks
        assert isinstance(m.BLinear, nn.Linear) and m.is_per_head_svd
        assert torch.equal(m.BLinear.weight.data, g[f"ragged_{fuse}_B"])
        assert torch.equal(torch.cat([a.data.reshape(-1) for a in m.ALinear]), g[f"ragged_{fuse}_A"])
        assert (m.bias is None) == (fuse != "UV")
        names = dict(m.named_parameters())
        assert "ALinear.0" in names and "BLinear.weight" in names
    m = SVDLinear(g["uni_U"], g["uni_S"], g["uni_V"], sigma_fuse="UV", is_per_head_svd=True)
    assert m.head_num == 4 and m.head_rank == 32 and torch.equal(m.ALinear.data, g["uni_A"]) and torch.equal(m.BLinear.weight.data, g["uni_B"])
    with pytest.raises(ValueError):
        SVDLinear(U, S, V, sigma_fuse="nope", is_per_head_svd=True, rank_split=ranks)
    with pytest.raises(ValueError):
        SVDLinear(U, S, V, sigma_fuse="local_ft", is_per_head_svd=True, rank_split=ranks)   # S given with local_ft
    plain = SVDLinear(torch.randn(24, 8), torch.rand(8) + 0.5, torch.randn(16, 8), sigma_fuse="UV")
    assert isinstance(plain.ALinear, nn.Linear) and plain.ALinear.weight.shape == (24, 8) and plain.BLinear.weight.shape == (8, 16)
    x = torch.randn(3, 16)
    assert torch.allclose(plain(x), x @ plain.BLinear.weight.t() @ plain.ALinear.weight.t(), atol=1e-5)


def test_act_quant_wrapper_surface_and_tree_walk():
    lin = nn.Linear(32, 16, bias=True)
    w = ActQuantWrapper(lin)
    for name, val in (("K", 1), ("online_full_had", False), ("online_full_hadnopow2", False), ("online_partial_had", False),
                      ("online_random_had", False), ("had_dim", 0), ("fp32_had", False), ("fuse_bias", False),
                      ("fuse_linear", False), ("bias_param", None), ("in_features", 32), ("out_features", 16)):
        assert getattr(w, name) == val, name
    assert w.module is lin and w.weight is lin.weight and w.bias is lin.bias and w.had_K is None
    assert isinstance(w.quantizer, ActQuantizer) and isinstance(w.out_quantizer, ActQuantizer)
    assert w.quantizer.bits == 16 and w.out_quantizer.bits == 16
    assert "module.weight" in w.state_dict() and "weight" in w.state_dict()
    w.quantizer.configure(bits=8, groupsize=-1, sym=True, clip_ratio=1.0)
    assert w.quantizer.bits == 8 and int(w.quantizer.maxq) == 127 and "Symmetric Per-Token" in w.extra_repr()
    for kw in (dict(bits=4, sym=True), dict(bits=8, sym=False), dict(bits=8, sym=True, groupsize=32),
               dict(bits=8, sym=True, clip_ratio=0.9)):
        with pytest.raises(ValueError):
            ActQuantizer().configure(**kw)
    with pytest.raises(AssertionError):
        ActQuantizer().configure(bits=8, sym=True, clip_ratio=1.5)

    class Mlp(nn.Module):
        def __init__(self):
            super().__init__()
            self.up = nn.Linear(8, 16)
            self.seq = nn.Sequential(nn.Linear(16, 16), nn.ReLU())
            self.lst = nn.ModuleList([nn.Linear(16, 8)])

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.mlp = Mlp()
            self.norm = nn.LayerNorm(8)

    blk = Block()
    add_actquant(blk)
    q = find_qlayers(blk)
    assert sorted(q) == ["mlp.lst.0", "mlp.seq.0", "mlp.up"]
    assert isinstance(blk.norm, nn.LayerNorm) and isinstance(blk.mlp.seq[1], nn.ReLU)
    add_actquant(blk)                                   # a second walk wraps nothing twice
    assert isinstance(blk.mlp.up.module, nn.Linear)


def test_wrapper_int8_weight_cache():
    g = load_golden("act_quant_wrapper")
    lin = nn.Linear(96, 48, bias=False).half()
    lin.weight.data = g["plain_W"].clone()
    w = ActQuantWrapper(lin)
    q, s = w.int8_weight()
    # the scale is recovered from the weight (no quantiser at hand): code * scale is the stored weight to one fp16 rounding
    def same(a, b):
        return bool(((a.float() - b.float()).abs() <= b.float().abs() * 2.0 ** -10 + 1e-7).all())

    assert q.dtype == torch.int8 and same((s[:, None] * q.float()).half(), g["plain_W"])
    assert w.int8_weight()[0] is q                       # cached
    lin.weight.data = g["w16_W"].clone()                 # a weight that is not int8 fake-quantised
    assert w.int8_weight() == (None, None)
    w.set_int8_weight(q, s)
    assert same(lin.weight.data, g["plain_W"]) and w.int8_weight()[0] is q
