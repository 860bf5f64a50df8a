"""Stacks of decoder layers (lsvd_b200/model.py) against the oracle's layer loop: decode steps through two layers, and a
prefill followed by decode steps (the prefill-to-decode flow of BASELINE config 5 at a small shape)."""
import pytest
import torch

from conftest import load_golden, unpack_had, rel_to_norm
from oracle import layer as olayer
from lsvd_b200 import synth
from lsvd_b200.attention import InferState, decode_advance
from lsvd_b200.layer import make_layer_weights
from lsvd_b200.model import LSVDModel

pytestmark = pytest.mark.gpu


def _weights(n_layers, hidden, H, D, rq, kr, vr, d_ffn, rank, n_svd, hk, K):
    return [(make_layer_weights(hidden, H, D, rq, kr, vr, seed=10 + 2 * i),
             synth.ffn_weights(hidden, d_ffn, rank, n_svd, seed=11 + 2 * i, had_K=hk, K=K, input_had=False, std=0.05))
            for i in range(n_layers)]


@pytest.mark.parametrize("head_major", [False, True])
def test_two_layer_stack_prefill_then_decode(head_major):
    H, D, rq, hidden, n_layers = 8, 128, 64, 1024, 2
    kr, vr = synth.ragged_ranks(H, 64, seed=5), synth.ragged_ranks(H, 64, seed=6)
    hk = unpack_had(load_golden("hadamard")["had172_bits"], 172)
    d_ffn, rank, n_svd, K = 172 * 16, 128, 1376, 172
    ws = _weights(n_layers, hidden, H, D, rq, kr, vr, d_ffn, rank, n_svd, hk, K)
    B, L, steps = 2, 40, 3                       # 80 prefill tokens: more than 64, so the FFN takes its tcgen05 form
    cap = L + steps
    n_slots = B * cap
    model = LSVDModel(n_layers, hidden, H, D, d_ffn, rq, kr, vr, rank, n_svd, hk, K, n_slots, weights=ws, head_major=head_major)
    lay = model.layout
    gen = torch.Generator().manual_seed(1)
    x_pre = torch.randn(B * L, hidden, generator=gen).half()
    r2t = torch.arange(n_slots, dtype=torch.int32).view(B, cap)
    dest = torch.cat([r2t[b, :L] for b in range(B)]).contiguous()
    xs = [torch.randn(B, hidden, generator=gen).half() for _ in range(steps)]
    for c in model.caches:
        for t in c:
            t.zero_()
    # ---- GPU: prefill, then decode steps with the state advanced on the device ----
    model.prefill(x_pre.cuda(), dest.cuda())
    st = InferState(B, cap, [L + 1] * B, device="cuda", req_to_token=r2t)
    out = None
    for t in range(steps):
        out = model.decode_step(xs[t].cuda(), st)
        if t + 1 < steps:
            decode_advance(st)
    torch.cuda.synchronize()
    # ---- oracle: the same loop on the CPU ----
    ref_caches = [(torch.zeros(n_slots, lay.sum_k, dtype=torch.int8), torch.zeros(n_slots, H, dtype=torch.float16),
                   torch.zeros(n_slots, lay.sum_v, dtype=torch.int8), torch.zeros(n_slots, H, dtype=torch.float16))
                  for _ in range(n_layers)]
    x = x_pre
    for (lw, fw), (ck, sk, cv, sv) in zip(ws, ref_caches):
        x, _ = olayer.prefill_layer(x, lw, fw, lay.k_off, lay.v_off, H, rq, ck, sk, cv, sv, dest)
    ref = None
    b_req = torch.arange(B, dtype=torch.int32)
    for t in range(steps):
        cur = torch.tensor([L + 1 + t] * B, dtype=torch.int32)
        mem = r2t[torch.arange(B), cur.long() - 1]
        x = xs[t]
        for (lw, fw), (ck, sk, cv, sv) in zip(ws, ref_caches):
            x, _ = olayer.decoder_layer(x, lw, fw, lay.k_off, lay.v_off, H, D, rq, ck, sk, cv, sv, r2t, b_req, cur, mem)
        ref = x
    # Cache rows.  First layer: integer stages behind an fp32 mean of squares whose addition order differs between the GPU
    # and the CPU, so a code may sit one step away here and there.  Deeper layers quantise latents of inputs that agree
    # only to the fp16 tolerance (and a moved row maximum moves every code of the row a little): there the dequantised
    # rows are compared.  (Appended rows from identical inputs are compared bit for bit in test_gpu_layer.py.)
    for li in range(n_layers):
        ck, sk, cv, sv = model.caches[li]
        if head_major:
            ck, sk = lay.from_head_major(ck, sk, "k")
            cv, sv = lay.from_head_major(cv, sv, "v")
        for got, gs, want, wsc, off in ((ck, sk, ref_caches[li][0], ref_caches[li][1], lay.k_off),
                                        (cv, sv, ref_caches[li][2], ref_caches[li][3], lay.v_off)):
            d = (got.cpu().int() - want.int()).abs()
            if li == 0:
                assert d.max() <= 2 and (d > 0).float().mean() < 2e-3, (li, d.max(), (d > 0).float().mean())
                continue
            rep = torch.tensor([off[h + 1] - off[h] for h in range(H)])
            deq_got = got.cpu().float() * torch.repeat_interleave(gs.cpu().float(), rep, dim=1)
            deq_want = want.float() * torch.repeat_interleave(wsc.float(), rep, dim=1)
            used = want.abs().sum(1) > 0
            err = (deq_got - deq_want)[used].abs().amax(1) / deq_want[used].norm(dim=1)
            assert err.max() < 1e-2, (li, err.max())
            assert (d > 0).float().mean() < 5e-2
    assert rel_to_norm(out.cpu().float(), ref.float()) < 2e-3


def test_stack_decode_graph_replays_the_eager_loop():
    """``capture_decode``: the decode loop as graph replays (state advanced on the device inside the graph) gives the same
    outputs and cache rows, bit for bit, as eager steps with ``decode_advance`` between them."""
    H, D, rq, hidden, n_layers = 8, 128, 64, 1024, 2
    kr, vr = synth.ragged_ranks(H, 64, seed=5), synth.ragged_ranks(H, 64, seed=6)
    hk = synth.sign_matrix(12, seed=3).float()
    d_ffn, rank, n_svd, K = 12 * 64, 128, 384, 12
    ws = _weights(n_layers, hidden, H, D, rq, kr, vr, d_ffn, rank, n_svd, hk, K)
    B, L, steps = 3, 70, 4
    cap = L + steps + 1                          # the state is advanced after the last step too
    n_slots = B * cap
    gen = torch.Generator().manual_seed(2)
    x_pre = torch.randn(B * L, hidden, generator=gen).half().cuda()
    r2t = torch.arange(n_slots, dtype=torch.int32).view(B, cap)
    dest = torch.cat([r2t[b, :L] for b in range(B)]).contiguous().cuda()
    xs = [torch.randn(B, hidden, generator=gen).half().cuda() for _ in range(steps)]

    def fresh():
        m = LSVDModel(n_layers, hidden, H, D, d_ffn, rq, kr, vr, rank, n_svd, hk, K, n_slots, weights=ws)
        for c in m.caches:
            for t in c:
                t.zero_()
        m.prefill(x_pre, dest)
        return m, InferState(B, cap, [L + 1] * B, device="cuda", req_to_token=r2t)

    eager, st = fresh()
    outs = []
    for t in range(steps):
        outs.append(eager.decode_step(xs[t], st).clone())
        decode_advance(st)
    graphed, st2 = fresh()
    x_in = torch.empty_like(xs[0])
    x_in.copy_(xs[0])
    graph, y = graphed.capture_decode(x_in, st2, advance={})
    for t in range(steps):
        x_in.copy_(xs[t])
        graph.replay()
        assert torch.equal(y, outs[t]), t
    torch.cuda.synchronize()
    assert torch.equal(st2.b_seq_len, st.b_seq_len) and torch.equal(st2.mem_index, st.mem_index)
    for ce, cg in zip(eager.caches, graphed.caches):
        for a, b in zip(ce, cg):
            assert torch.equal(a, b)
