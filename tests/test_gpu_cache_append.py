"""GPU parity of the latent cache append kernel, through the C ABI: bit-exact int8 codes and fp16 scales."""
import pytest
import torch

from conftest import load_golden
from oracle import quant, attention as oattn
from lsvd_b200 import destindex_copy_quantize_latent, cache_append, LatentCacheLayout
from lsvd_b200 import synth

pytestmark = pytest.mark.gpu


def test_append_matches_reference_fixture_both_roundings():
    g = load_golden("latent_quant")
    x = g["x"].cuda()
    T, H, R = x.shape
    # R = 24 is not a multiple of 16: the kernel wants 16-aligned ranks, so embed into R = 32 with zero padding,
    # which changes neither the absmax nor the codes of the first 24 entries.
    xp = torch.zeros(T, H, 32, dtype=torch.float16, device="cuda")
    xp[:, :, :R] = x
    for rounding, cache_ref, scale_ref in (("triton", g["cache_triton"], g["scale_triton"]), ("torch", None, None)):
        cache = torch.zeros(64, H, 32, dtype=torch.int8, device="cuda")
        scale = torch.zeros(64, H, dtype=torch.float16, device="cuda")
        destindex_copy_quantize_latent(xp, g["dest_loc"].cuda(), cache, scale, rounding=rounding)
        torch.cuda.synchronize()
        if rounding == "triton":
            assert torch.equal(scale.cpu(), scale_ref)
            assert torch.equal(cache.cpu()[:, :, :R], cache_ref)
        else:
            rows = g["dest_loc"].long()
            assert torch.equal(scale.cpu()[rows], g["s_torch"])
            assert torch.equal(cache.cpu()[rows][:, :, :R], g["q_torch"])
        assert (cache.cpu()[:, :, R:] == 0).all()


@pytest.mark.parametrize("rounding", ["torch", "triton"])
def test_append_ragged_k_and_v_one_launch(rounding):
    gen = torch.Generator().manual_seed(5)
    k_ranks, v_ranks = [16, 128, 48, 64, 32], [64, 16, 16, 112, 128]
    lay = LatentCacheLayout(k_ranks, v_ranks)
    T, N = 37, 101
    lk = (torch.randn(T, lay.sum_k, generator=gen) * 2).half()
    lv = (torch.randn(T, lay.sum_v, generator=gen) * 0.01).half()
    lk[0] = 0
    lv[1] = 60000.0
    dest = torch.randperm(N, generator=gen)[:T].to(torch.int32)
    ck = torch.full((N, lay.sum_k), 7, dtype=torch.int8)
    cv = torch.full((N, lay.sum_v), 7, dtype=torch.int8)
    sk = torch.full((N, 5), 3.0, dtype=torch.float16)
    sv = torch.full((N, 5), 3.0, dtype=torch.float16)
    ck_ref, sk_ref, cv_ref, sv_ref = ck.clone(), sk.clone(), cv.clone(), sv.clone()
    oattn.cache_append(lk, dest, lay.k_off, ck_ref, sk_ref, rounding)
    oattn.cache_append(lv, dest, lay.v_off, cv_ref, sv_ref, rounding)
    d = [t.cuda() for t in (lk, lv, dest, ck, sk, cv, sv)]
    cache_append(lay, d[0], d[1], d[2], d[3], d[4], d[5], d[6], rounding=rounding)
    torch.cuda.synchronize()
    assert torch.equal(d[3].cpu(), ck_ref) and torch.equal(d[4].cpu(), sk_ref)      # untouched rows stay untouched
    assert torch.equal(d[5].cpu(), cv_ref) and torch.equal(d[6].cpu(), sv_ref)


def test_append_strided_latent_view_like_the_reference_block():
    # the reference appends latent_kv[:, 0] and latent_kv[:, 1] of one [T, 2, H, R] projection output
    gen = torch.Generator().manual_seed(6)
    T, H, R, N = 16, 32, 64, 64
    kv = torch.randn(T, 2, H, R, generator=gen).half()
    dest = torch.arange(T, dtype=torch.int32) * 3
    for side in (0, 1):
        cache = torch.zeros(N, H, R, dtype=torch.int8, device="cuda")
        scale = torch.zeros(N, H, dtype=torch.float16, device="cuda")
        destindex_copy_quantize_latent(kv.cuda()[:, side], dest.cuda(), cache, scale)
        q, s = quant.latent_quant(kv[:, side])
        assert torch.equal(cache.cpu()[dest.long()], q) and torch.equal(scale.cpu()[dest.long()], s)


def test_append_out_of_range_slot_is_skipped_and_reported():
    lay = LatentCacheLayout.uniform(2, 16)
    lat = torch.ones(3, 32, dtype=torch.float16, device="cuda")
    dest = torch.tensor([1, 99, -4], dtype=torch.int32, device="cuda")
    ck = torch.zeros(8, 32, dtype=torch.int8, device="cuda")
    sk = torch.zeros(8, 2, dtype=torch.float16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cache_append(lay, lat, None, dest, ck, sk, None, None, status_word=status)
    torch.cuda.synchronize()
    assert status.item() == 6
    assert (ck.cpu()[1] == 127).all() and (ck.cpu()[[0, 2, 3, 4, 5, 6, 7]] == 0).all()


def test_append_prefill_sized_batch_checksum():
    """Full prefill-sized append (32768 tokens x 32 heads x 64): compared with the oracle through a checksum."""
    T, H, R = 32768, 32, 64
    gen = torch.Generator().manual_seed(9)
    lat = torch.randn(T, H * R, generator=gen).half()
    dest = torch.randperm(T, generator=gen).to(torch.int32)
    lay = LatentCacheLayout.uniform(H, R)
    ck = torch.zeros(T, H * R, dtype=torch.int8, device="cuda")
    sk = torch.zeros(T, H, dtype=torch.float16, device="cuda")
    cache_append(lay, lat.cuda(), None, dest.cuda(), ck, sk, None, None)
    q, s = quant.latent_quant(lat.view(T, H, R))
    ck_ref = torch.empty(T, H * R, dtype=torch.int8)
    ck_ref[dest.long()] = q.view(T, -1)
    assert torch.equal(ck.cpu(), ck_ref)
    sk_ref = torch.empty(T, H, dtype=torch.float16)
    sk_ref[dest.long()] = s
    assert torch.equal(sk.cpu(), sk_ref)


@pytest.mark.parametrize("rounding", ["torch", "triton"])
def test_append_many_tokens_ragged_both_sides(rounding):
    """Thousands of tokens with ragged ranks, K and V in one launch, strided latents (views of one wider tensor) and
    slots scattered over a larger cache."""
    gen = torch.Generator().manual_seed(21)
    k_ranks, v_ranks = [16, 128, 48, 64, 32], [64, 16, 16, 112, 128]
    lay = LatentCacheLayout(k_ranks, v_ranks)
    T, N = 4001, 4100
    both = torch.randn(T, lay.sum_k + lay.sum_v, generator=gen).half()
    both[7] = 0
    lk, lv = both[:, :lay.sum_k], both[:, lay.sum_k:]                # views with a row stride of both widths
    dest = torch.randperm(N, generator=gen)[:T].to(torch.int32)
    ck = torch.zeros(N, lay.sum_k, dtype=torch.int8, device="cuda")
    cv = torch.zeros(N, lay.sum_v, dtype=torch.int8, device="cuda")
    sk = torch.zeros(N, 5, dtype=torch.float16, device="cuda")
    sv = torch.zeros(N, 5, dtype=torch.float16, device="cuda")
    gb = both.cuda()
    cache_append(lay, gb[:, :lay.sum_k], gb[:, lay.sum_k:], dest.cuda(), ck, sk, cv, sv, rounding=rounding)
    torch.cuda.synchronize()
    for lat, offs, cache, scale in ((lk, lay.k_off, ck, sk), (lv, lay.v_off, cv, sv)):
        c_ref = torch.zeros(N, lat.shape[1], dtype=torch.int8)
        s_ref = torch.zeros(N, 5, dtype=torch.float16)
        oattn.cache_append(lat.contiguous(), dest, list(offs), c_ref, s_ref, rounding=rounding)
        assert torch.equal(cache.cpu(), c_ref) and torch.equal(scale.cpu(), s_ref)


def test_append_many_tokens_out_of_range_slots_are_skipped_and_reported():
    """The same guard in the form used for thousands of tokens: bad slots are skipped, every other row is written."""
    lay = LatentCacheLayout([16, 64, 128], [32, 48, 16])
    T, N = 6000, 6000
    gen = torch.Generator().manual_seed(33)
    lk = torch.randn(T, lay.sum_k, generator=gen).half()
    lv = torch.randn(T, lay.sum_v, generator=gen).half()
    dest = torch.arange(T, dtype=torch.int32)
    dest[17], dest[4242] = N + 5, -1
    ck = torch.zeros(N, lay.sum_k, dtype=torch.int8, device="cuda")
    cv = torch.zeros(N, lay.sum_v, dtype=torch.int8, device="cuda")
    sk = torch.zeros(N, 3, dtype=torch.float16, device="cuda")
    sv = torch.zeros(N, 3, dtype=torch.float16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cache_append(lay, lk.cuda(), lv.cuda(), dest.cuda(), ck, sk, cv, sv, status_word=status)
    torch.cuda.synchronize()
    assert status.item() == 6
    good = torch.ones(T, dtype=torch.bool)
    good[17] = good[4242] = False
    for lat, offs, cache, scale in ((lk, lay.k_off, ck, sk), (lv, lay.v_off, cv, sv)):
        q, s = quant.latent_quant_ragged(lat, list(offs))
        assert torch.equal(cache.cpu()[good], q[good]) and torch.equal(scale.cpu()[good], s[good])
        assert (cache.cpu()[~good] == 0).all() and (scale.cpu()[~good] == 0).all()


@pytest.mark.parametrize("tokens", [37, 2100])
def test_head_major_layout_holds_the_same_codes(tokens):
    """LSVD_CACHE_HEAD_MAJOR ([H][N_slots][r_h] + scales [H][N_slots]): the same codes and scales as the slot-major
    cache, in both the decode-sized and the prefill-sized kernel (2100 tokens x 5 heads x 2 sides = 21 000 units < 32 768
    stays on the first; the second size is reached with 16 heads below)."""
    gen = torch.Generator().manual_seed(tokens)
    heads = 5 if tokens < 100 else 16
    k_ranks = synth.ragged_ranks(heads, 64, seed=1) if heads == 16 else [16, 128, 48, 64, 32]
    v_ranks = synth.ragged_ranks(heads, 64, seed=2) if heads == 16 else [64, 16, 16, 112, 128]
    lay = LatentCacheLayout(k_ranks, v_ranks)
    hm = lay.as_head_major()
    N = tokens + 64
    lk = (torch.randn(tokens, lay.sum_k, generator=gen) * 2).half().cuda()
    lv = (torch.randn(tokens, lay.sum_v, generator=gen) * 0.5).half().cuda()
    dest = torch.randperm(N, generator=gen)[:tokens].to(torch.int32).cuda()
    ck, sk, cv, sv = [t.zero_() for t in lay.alloc(N)]
    hk, hsk, hv, hsv = [t.zero_() for t in hm.alloc(N)]
    cache_append(lay, lk, lv, dest, ck, sk, cv, sv)
    cache_append(hm, lk, lv, dest, hk, hsk, hv, hsv)
    torch.cuda.synchronize()
    k2, sk2 = hm.from_head_major(hk, hsk, "k")
    v2, sv2 = hm.from_head_major(hv, hsv, "v")
    assert torch.equal(k2, ck) and torch.equal(sk2, sk) and torch.equal(v2, cv) and torch.equal(sv2, sv)
    # and the conversion helpers are inverses of each other
    fk, fsk = hm.to_head_major(ck, sk, "k")
    assert torch.equal(fk, hk) and torch.equal(fsk, hsk)
