"""One LSVD W8A8 decoder layer for decode steps, composed of the library's kernels.

Structure (the kernel-side attention block of the reference,
kernels/layer_bench/ffn_kernel/baseline_kernel.py:107-145, with its fp16 projections replaced by int8
products, followed by the hybrid FFN of fake_quant/utils/hybrid_ffn_utils.py:956-984):

    xn   = RMSNorm(x) * w1                  (eps 1e-5; the residual of the attention block is xn, as in the reference)
    lat  = A8(xn) . W_lat^T                 [q latents | K latents | V latents], int8 product, fp16 out
    cache <- quantise(K, V latents) at mem_index
    o    = latent decode attention(q latents, C = B_k A_q^T per head, cache)     in V-latent space
    y1   = A8(o) . W_uvo^T + xn             W_uvo = the V up-factor composed with the output projection
    out  = hybrid FFN(RMSNorm(y1) * w2) + y1            (eps 1e-6; the residual of the FFN is its raw input)

The per-head query up-projection A_q and the K up-factor B_k are composed offline into C_h = B_k,h A_q,h^T
(r_k x r_q), so the attention kernel's query absorption takes the query latent directly.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch
from torch import nn

from . import _lib
from .attention import LatentCacheLayout, cache_append, token_decode_attention_int8_latent_absorb, attn_decode_workspace_bytes
from .ffn import HybridFFN, act_quant, w8a8_gemv, quantize_weight_rtn, i8gemm


class LSVDDecoderLayer(nn.Module):
    def __init__(self, layout: LatentCacheLayout, head_dim: int, rank_q: int, w: dict, ffn: HybridFFN):
        """``w``: ln1 [hidden] fp16, ln2 [hidden] fp16, W_lat_q int8 [H*rank_q + sum r_k + sum r_v, hidden] + W_lat_s,
        C fp16 [sum r_k, rank_q] (per-head blocks), W_uvo_q int8 [hidden, sum r_v] + W_uvo_s."""
        super().__init__()
        self.layout, self.head_dim, self.rank_q, self.ffn = layout, head_dim, rank_q, ffn
        for name in ("ln1", "ln2", "W_lat_q", "W_lat_s", "C", "W_uvo_q", "W_uvo_s"):
            self.register_buffer(name, w[name].contiguous())
        self.hidden = self.ln1.shape[0]
        self.Rq = layout.num_heads * rank_q
        self._ws = None
        self._side = None

    @torch.no_grad()
    def forward(self, x, cache_k, scale_k, cache_v, scale_v, infer_state, stages: Optional[dict] = None, out=None,
                timing_events=None, after_attention=None):
        """x [B, hidden] fp16 (one token per request).  Mutates the cache rows ``infer_state.mem_index`` in place.
        ``out`` receives the result if given; ``timing_events`` (a CUDA event pair) is recorded around the attention's
        streaming kernel.  ``after_attention`` (a callable) is run on a side stream as soon as the attention has read
        ``infer_state`` for the last time, beside the output projection and the FFN, and joined before the step ends:
        the place for the device-side move to the next token (``decode_advance``) of a decode loop."""
        lay, H, B = self.layout, self.layout.num_heads, x.shape[0]
        xq, xs, xn = act_quant(x, want_rotated=True, norm_weight=self.ln1, norm_eps=1e-5)
        lat, _, _ = w8a8_gemv(xq, xs, self.W_lat_q, self.W_lat_s)
        lk = lat[:, self.Rq:self.Rq + lay.sum_k]
        lv = None if lay.shared_kv else lat[:, self.Rq + lay.sum_k:]       # shared: one latent per head serves K and V
        cache_append(lay, lk, lv, infer_state.mem_index, cache_k, scale_k, cache_v, scale_v)
        need = attn_decode_workspace_bytes(B, lay, infer_state.max_len_in_batch)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=x.device)
        o_lat = torch.empty(B, lay.sum_v, dtype=torch.float16, device=x.device)
        q = lat[:, :self.Rq].unflatten(1, (H, self.rank_q))
        token_decode_attention_int8_latent_absorb(q, infer_state, H, self.rank_q, cache_k, scale_k, cache_v, scale_v,
                                                  self.C, None, layout=lay, out_latent=o_lat, workspace=self._ws,
                                                  sm_scale=1.0 / math.sqrt(self.head_dim), timing_events=timing_events)
        side = None
        if after_attention is not None:
            if self._side is None:
                self._side = torch.cuda.Stream(device=x.device)
            side, cur = self._side, torch.cuda.current_stream(x.device)
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                after_attention()
        oq, os_, _ = act_quant(o_lat)
        y1, _, _ = w8a8_gemv(oq, os_, self.W_uvo_q, self.W_uvo_s, residual=xn)
        out = self.ffn(y1, out=out, norm_weight=self.ln2, norm_eps=1e-6, residual=y1)
        if side is not None:
            torch.cuda.current_stream(x.device).wait_stream(side)
        if stages is not None:
            stages.update(xn=xn, lat=lat, o_lat=o_lat, y1=y1, out=out)
        return out


def _layer_prefill(self, x, cache_k, scale_k, cache_v, scale_v, dest_slots, stages=None, out=None):
    """The layer for a prefill-sized batch of tokens ``x [T, hidden]`` whose cache slots are ``dest_slots [T]``: the same
    stages as a decode step with every product on the tcgen05 GEMM (lsvd_i8gemm_prefill) and the cache written by the
    prefill-sized form of the append kernel.  The reference has no prefill attention (its kernels are decode-only,
    kernels/layer_bench/fd_kernel/): between the cache write and the output projection this step lets every token attend
    to ITSELF only, i.e. the attention output is the token's own (fp16) V latent.  Everything BASELINE config 5 names for
    the prefill -- the latent-projection, gate / up / down GEMMs and the cache write -- runs as in a real prefill; the
    values that reach the decode steps differ from a causal-attention prefill, which this library does not have."""
    lay = self.layout
    xq, xs, xn = act_quant(x, want_rotated=True, norm_weight=self.ln1, norm_eps=1e-5)
    lat, _ = i8gemm(xq, xs, self.W_lat_q, self.W_lat_s)
    lk = lat[:, self.Rq:self.Rq + lay.sum_k]
    lv = lat[:, self.Rq + lay.sum_k:]
    cache_append(lay, lk, lv, dest_slots, cache_k, scale_k, cache_v, scale_v)
    o_lat = lv.contiguous()
    oq, os_, _ = act_quant(o_lat)
    y1, _ = i8gemm(oq, os_, self.W_uvo_q, self.W_uvo_s, residual=xn)
    out = self.ffn(y1, out=out, norm_weight=self.ln2, norm_eps=1e-6, residual=y1)
    if stages is not None:
        stages.update(xn=xn, lat=lat, o_lat=o_lat, y1=y1, out=out)
    return out


LSVDDecoderLayer.forward_prefill = torch.no_grad()(_layer_prefill)


def make_layer_weights(hidden: int, num_heads: int, head_dim: int, rank_q: int, k_ranks, v_ranks, seed: int = 0, device=None,
                       shared_kv: bool = False):
    """Seeded random layer weights (xavier-like scales as the reference's block,
    kernels/layer_bench/ffn_kernel/baseline_kernel.py:86-91); returns the dict ``LSVDDecoderLayer`` takes.  Drawn on the
    CPU unless ``device`` is given (whole stacks in benchmarks)."""
    g = (torch.Generator() if device is None else torch.Generator(device=device)).manual_seed(seed)
    dv = dict(device=device) if device is not None else {}
    Rq, Rk, Rv = num_heads * rank_q, sum(k_ranks), sum(v_ranks)
    lat_rows = Rq + Rk + (0 if shared_kv else Rv)      # shared: the V latent IS the K latent, no rows of its own

    def rnd(*shape, std):
        return torch.randn(*shape, generator=g, **dv) * std

    W_lat = rnd(lat_rows, hidden, std=1.0 / math.sqrt(hidden))
    A_q = rnd(num_heads, head_dim, rank_q, std=1.0 / math.sqrt(rank_q))          # query up-factor per head
    B_k = rnd(Rk, head_dim, std=1.0 / 8)                                           # K up-factor rows per head
    C = torch.empty(Rk, rank_q, **dv)
    off = 0
    for h, r in enumerate(k_ranks):
        C[off:off + r] = B_k[off:off + r] @ A_q[h]
        off += r
    W_uvo = rnd(hidden, Rv, std=1.0 / math.sqrt(Rv))
    w = {"ln1": (1 + 0.1 * rnd(hidden, std=1.0)).half(), "ln2": (1 + 0.1 * rnd(hidden, std=1.0)).half(), "C": C.half()}
    w["W_lat_q"], w["W_lat_s"] = quantize_weight_rtn(W_lat)
    w["W_uvo_q"], w["W_uvo_s"] = quantize_weight_rtn(W_uvo)
    return w


def _recorded_event():
    ev = torch.cuda.Event(enable_timing=True)
    ev.record()
    return ev


class TPDecoderLayer(nn.Module):
    """The decoder layer of one tensor-parallel rank (see lsvd_b200/parallel.py for the sharding).

    Built from that rank's local weights; ``forward`` takes the replicated hidden state and the rank's own cache
    columns, and issues one all-reduce in the attention block, one all-gather and one all-reduce in the FFN block.
    Everything between the collectives runs in the library's kernels (the dequantising steps around a collective are
    epilogues: an fp32 partial-sum output of the product before the first all-reduce, the residual + RMSNorm + A8
    quantiser after it, a dequantise + residual kernel after the second); buffers are kept per batch size, so a step
    allocates nothing: about twenty host calls when launched eagerly, seven once the runs between the collectives are
    replayed as CUDA graphs (``use_graphs``, on unless ``LSVD_TP_GRAPHS=0``).
    """

    def __init__(self, lw: dict, fw: dict, info: dict, head_dim: int, rank_q: int, world: int, group=None, head_major: bool = False):
        super().__init__()
        self.info, self.head_dim, self.rank_q, self.world, self.group = info, head_dim, rank_q, world, group
        self.layout = LatentCacheLayout(info["k_ranks"], info["v_ranks"], head_major=head_major)
        for name in ("ln1", "ln2", "W_lat_q", "W_lat_s", "C", "W_uvo_q", "W_uvo_s"):
            self.register_buffer(name, lw[name].contiguous())
        for name in ("U_q", "U_s", "Vg_q", "Vg_s", "Vu_q", "Vu_s", "Wg_q", "Wg_s", "Wu_q", "Wu_s", "Wd_loc_q", "Wd_s"):
            self.register_buffer("f_" + name, fw[name].contiguous())
        self.K = int(fw.get("K", 1))
        hk = fw.get("had_K")
        self.register_buffer("had_K", None if hk is None else hk.to(torch.float16).contiguous())
        self.had_K_packed = None
        self.Rq = self.layout.num_heads * rank_q
        self._bufs = {}
        self.use_graphs = os.environ.get("LSVD_TP_GRAPHS", "1") == "1"
        self._graphs, self._seen = {}, {}
        # profiling aid: one rank's launches of an N-way split on a single GPU, the three collectives left out (the
        # results are then not those of the layer)
        self.skip_collectives = False

    def _step_buffers(self, B: int, max_len: int, dev):
        key = (B, max_len, str(dev))
        b = self._bufs.get(key)
        if b is not None:
            return b
        from .parallel import gather_plan
        lay, hidden = self.layout, self.ln1.shape[0]
        r = self.f_U_q.shape[0] // 2
        ns, nq = self.f_Vg_q.shape[0], self.f_Wg_q.shape[0]
        d_ffn = self.info["n_svd"] + self.info["n_q"]
        widest, idx = gather_plan(self.info, self.world, dev)
        e = lambda *shape, dt=torch.float16: torch.empty(*shape, dtype=dt, device=dev)
        b = dict(
            ws=torch.empty(attn_decode_workspace_bytes(B, lay, max_len), dtype=torch.uint8, device=dev),
            xq=e(B, hidden, dt=torch.int8), xs=e(B, dt=torch.float32), xn=e(B, hidden),
            lat=e(B, self.W_lat_q.shape[0]), o_lat=e(B, lay.sum_v), oq=e(B, lay.sum_v, dt=torch.int8), os=e(B, dt=torch.float32),
            part=e(B, hidden, dt=torch.float32), y1=e(B, hidden), x2q=e(B, hidden, dt=torch.int8), x2s=e(B, dt=torch.float32),
            lat2=e(B, 2 * r), zq=e(2 * B, r, dt=torch.int8), zs=e(2 * B, dt=torch.float32),
            send=torch.zeros(B, widest, dtype=torch.float16, device=dev), recv=e(self.world * B, widest),
            h=e(B, d_ffn), hq=e(B, d_ffn, dt=torch.int8), hs=e(B, dt=torch.float32), hloc=e(B, ns + nq, dt=torch.int8),
            acc=e(B, hidden, dt=torch.int32), out=e(B, hidden), plan=(widest, idx))
        # the gathered pieces [rank][token][svd slice | rtn slice] -> rows in the global [SVD | RTN] order: two byte
        # segments per rank (lsvd_gather_segments)
        from .parallel import channel_slices
        n_svd, n_q = self.info["n_svd"], self.info["n_q"]
        src_off, src_stride, dst_off, length = [], [], [], []
        for rk, (sv, rt) in enumerate(zip(channel_slices(n_svd, self.world), channel_slices(n_q, self.world))):
            for first, (c0, c1), base in ((0, sv, 0), (sv[1] - sv[0], rt, n_svd)):
                src_off.append((rk * B * widest + first) * 2)
                src_stride.append(widest * 2)
                dst_off.append((base + c0) * 2)
                length.append((c1 - c0) * 2)
        import ctypes as C
        n = len(length)
        b["segments"] = (n, (C.c_int64 * n)(*src_off), (C.c_int64 * n)(*src_stride), (C.c_int64 * n)(*dst_off), (C.c_int32 * n)(*length))
        self._bufs[key] = b
        return b

    def _segments(self, b, x, cache_k, scale_k, cache_v, scale_v, infer_state, timing_events=None):
        """The four runs of kernel launches between the step's collectives, as callables over the step buffers ``b``."""
        from .ffn import hadamard_pack, hadamard_quant, dequant_residual
        lay, Hl, B = self.layout, self.layout.num_heads, x.shape[0]
        r = self.f_U_q.shape[0] // 2
        ns = self.f_Vg_q.shape[0]
        widest, idx = b["plan"]
        if self.had_K_packed is None:
            self.had_K_packed = hadamard_pack(self.had_K)

        def attention_block():
            # RMSNorm + A8, latent projection, append, attention, row-parallel output projection (fp32 partial sums)
            act_quant(x, norm_weight=self.ln1, norm_eps=1e-5, q=b["xq"], scale=b["xs"], rot=b["xn"])
            w8a8_gemv(b["xq"], b["xs"], self.W_lat_q, self.W_lat_s, out=b["lat"])
            lat = b["lat"]
            cache_append(lay, lat[:, self.Rq:self.Rq + lay.sum_k], lat[:, self.Rq + lay.sum_k:], infer_state.mem_index,
                         cache_k, scale_k, cache_v, scale_v)
            token_decode_attention_int8_latent_absorb(lat[:, :self.Rq].unflatten(1, (Hl, self.rank_q)), infer_state, Hl,
                                                      self.rank_q, cache_k, scale_k, cache_v, scale_v, self.C, None,
                                                      layout=lay, out_latent=b["o_lat"], workspace=b["ws"],
                                                      sm_scale=1.0 / math.sqrt(self.head_dim), timing_events=timing_events)
            act_quant(b["o_lat"], q=b["oq"], scale=b["os"])
            w8a8_gemv(b["oq"], b["os"], self.W_uvo_q, self.W_uvo_s, want_out=False, out_f32=b["part"])

        def gate_up():
            # y1 = fp16(sum + xn); x2 = A8(RMSNorm(y1)): one launch; replicated latents; column-parallel gate / up
            act_quant(None, x_f32=b["part"], add=b["xn"], sum_out=b["y1"], norm_weight=self.ln2, norm_eps=1e-6, q=b["x2q"],
                      scale=b["x2s"])
            w8a8_gemv(b["x2q"], b["x2s"], self.f_U_q, self.f_U_s, out=b["lat2"])
            act_quant(b["lat2"].view(-1, r), q=b["zq"], scale=b["zs"])
            zq, zs = b["zq"].view(B, 2 * r), b["zs"].view(B, 2)
            # the rank's [SVD slice | RTN slice] straight into the send buffer; its padding columns stay zero
            w8a8_gemv(zq[:, :r], zs[:, 0], self.f_Vg_q, self.f_Vg_s, self.f_Vu_q, self.f_Vu_s, a2_q=zq[:, r:], a2_scale=zs[:, 1],
                      out=b["send"], out_col=0)
            w8a8_gemv(b["x2q"], b["x2s"], self.f_Wg_q, self.f_Wg_s, self.f_Wu_q, self.f_Wu_s, out=b["send"], out_col=ns)

        def down():
            # gathered pieces -> global [SVD | RTN] order, Hadamard + A8, the rank's columns, row-parallel int32 product
            seg = b["segments"]
            _lib.check(_lib.load().lsvd_gather_segments(b["recv"].data_ptr(), b["h"].data_ptr(), b["h"].stride(0) * 2, B, seg[0],
                                                       seg[1], seg[2], seg[3], seg[4],
                                                       torch.cuda.current_stream(b["h"].device).cuda_stream))
            hadamard_quant(b["h"], self.had_K_packed, self.K, q=b["hq"], scale=b["hs"])
            s0, s1 = self.info["svd"]
            q0, q1 = self.info["rtn"]
            n_svd = self.info["n_svd"]
            torch.cat((b["hq"][:, s0:s1], b["hq"][:, n_svd + q0:n_svd + q1]), dim=1, out=b["hloc"])
            w8a8_gemv(b["hloc"], b["hs"], self.f_Wd_loc_q, None, want_out=False, acc=b["acc"])

        def finish():
            dequant_residual(b["acc"], b["hs"], self.f_Wd_s, residual=b["y1"], out=b["out"])

        return attention_block, gate_up, down, finish

    @torch.no_grad()
    def forward(self, x, cache_k, scale_k, cache_v, scale_v, infer_state, stages=None, timing_events=None, segment_events=None):
        """One step.  ``segment_events`` (a list) receives eight CUDA events recorded around the four runs of launches and
        the three collectives: attention block | all-reduce | gate/up | all-gather | down | all-reduce | finish.
        With ``use_graphs`` the four runs of launches between the collectives are captured as CUDA graphs
        the second time a step sees the same tensors (``x``, caches, state: callers that reuse their buffers, as a decode
        loop does) and replayed from then on: seven host calls per step (four replays, three collectives; the
        collectives themselves are never captured)."""
        import torch.distributed as dist
        B, dev = x.shape[0], x.device
        b = self._step_buffers(B, int(infer_state.max_len_in_batch), dev)
        r2t = infer_state.req_manager.req_to_token_indexs
        key = (x.data_ptr(), cache_k.data_ptr(), scale_k.data_ptr(), cache_v.data_ptr(), scale_v.data_ptr(),
               infer_state.b_seq_len.data_ptr(), infer_state.b_req_idx.data_ptr(), infer_state.mem_index.data_ptr(), r2t.data_ptr(),
               B, int(infer_state.max_len_in_batch))
        graphs = None
        if self.use_graphs and x.is_cuda and stages is None and timing_events is None:
            graphs = self._graphs.get(key)
            if graphs is None and self._seen.get(key, 0) >= 1:
                pool = torch.cuda.graph_pool_handle()
                graphs = []
                for seg in self._segments(b, x, cache_k, scale_k, cache_v, scale_v, infer_state):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, pool=pool):
                        seg()
                    graphs.append(g)
                self._graphs[key] = graphs
            self._seen[key] = self._seen.get(key, 0) + 1
        if graphs is not None:
            run = [g.replay for g in graphs]
        else:
            run = self._segments(b, x, cache_k, scale_k, cache_v, scale_v, infer_state, timing_events)
        mark = (lambda: None) if segment_events is None else (lambda: segment_events.append(_recorded_event()))
        mark()
        run[0]()
        mark()
        if not self.skip_collectives:
            dist.all_reduce(b["part"], group=self.group)
        mark()
        run[1]()
        mark()
        if not self.skip_collectives:
            dist.all_gather_into_tensor(b["recv"], b["send"], group=self.group)
        mark()
        run[2]()
        mark()
        if not self.skip_collectives:
            dist.all_reduce(b["acc"], group=self.group)
        mark()
        run[3]()
        mark()
        if stages is not None:
            stages.update(xn=b["xn"], o_lat=b["o_lat"], y1=b["y1"], h_q=b["hq"], down_acc=b["acc"], out=b["out"])
        return b["out"]
