#!/usr/bin/env python
"""Benchmark of the LSVD decode hot path on B200: one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A "step" is one decode step of one decoder layer over one batch of synthetic requests.

N = 1, default workload `c3_layer` (BASELINE config 3): the full LSVD W8A8 decoder layer at the LLaVA-Next-7B shape
(RMSNorm + A8, int8 latent projection, cache append, int8 latent flash-decoding attention over the whole context --
batch 16, context 4096 growing by one token per step for 128 steps, ragged per-head ranks mean 64 -- fused output
projection, hybrid SVD/RTN FFN 4096/11008).  Metric: decode tokens/s of that layer step.

N > 1 (launched by torch.distributed.run), default workload `c4_layer_tp` (BASELINE config 4): one decoder layer of the
13B shape (hidden 5120, 40 heads, intermediate 13824, batch 64, context 8192) TENSOR-PARALLEL over the N ranks -- heads
and FFN channels sharded, one NCCL all-reduce per block plus the all-gather of the FFN hidden vector -- strong scaling:
the same total work at every N.  `--replicas` runs N independent copies of the 1-GPU workload instead.

Other workloads: `c2_ffn` (--tokens 1/8/64), `c3_attention`, `c1_attention`, `c5_prefill_ffn`, ... (see WORKLOADS).
Every timed leg is repeated (each repeat = exactly --steps steps between a barrier + synchronize on both sides, maximum
over ranks); `ms_per_step` is the median repeat, the spread is reported in `parts`.

--impl reference times the CPU restatement of the reference's algorithm (the oracle, a port: the reference has no CPU
implementation of latent attention) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch

WORKLOADS = {
    "c3_layer": dict(batch=16, heads=32, head_dim=128, context=4096, ragged=True, ffn=True, full=True,
                     desc="BASELINE config 3: the full LSVD W8A8 decoder layer at the LLaVA-Next-7B shape (hidden 4096, "
                          "32 heads x 128, intermediate 11008), batch 16, context 4096, ragged per-head K/V ranks "
                          "(multiples of 16 in [16,128], mean 64), query latents of rank 64 per head; hybrid FFN rank 512, "
                          "50 % SVD channels, Hadamard 64 x 172"),
    "c3_attention_ffn": dict(batch=16, heads=32, head_dim=128, context=4096, ragged=True, ffn=True,
                             desc="BASELINE config 3 without the projections: cache append + attention (absorb, V "
                                  "up-projection) + hybrid FFN on the attention output"),
    "c2_ffn": dict(batch=8, heads=0, head_dim=0, context=0, ragged=False, ffn=True, ffn_only=True,
                   desc="BASELINE config 2: hybrid FFN decode block 4096/11008, rank 512, 50 % SVD channels, input "
                        "rotation + Hadamard 64 x 172, batch of --tokens tokens (1/8/64)"),
    # name: batch, heads, head_dim, context, ragged?
    "c3_attention": dict(batch=16, heads=32, head_dim=128, context=4096, ragged=True,
                         desc="BASELINE config 3 attention block: LLaVA-Next-7B layer shape, batch 16, "
                              "context 4096, ragged per-head K/V ranks (multiples of 16 in [16,128], mean 64)"),
    "c1_attention": dict(batch=1, heads=32, head_dim=128, context=2048, ragged=False,
                         desc="BASELINE config 1: batch 1, context 2048, uniform rank 64"),
    "c1_attention_rope": dict(batch=1, heads=32, head_dim=128, context=2048, aux="rope",
                              desc="BASELINE config 1 shape in the reference's own attention form: int8 K up-factor, "
                                   "keys rebuilt and rotated per token (lsvd_attn_decode_rope)"),
    "c3_attention_rope": dict(batch=16, heads=32, head_dim=128, context=4096, aux="rope",
                              desc="BASELINE config 3 batch/context with uniform rank 64 in the reference's own attention "
                                   "form (int8 K up-factor, rotary keys)"),
    "c1_attention_block": dict(batch=1, heads=32, head_dim=128, context=2048, aux="block",
                               desc="BASELINE config 1 through the module that takes the place of the reference's "
                                    "Int8AttentionBlock: RMSNorm, fp16 latent projections (library GEMMs, as in the "
                                    "reference), append, rotary int8 latent attention, composed output projection"),
    "c4_layer_tp": dict(batch=64, heads=40, head_dim=128, context=8192, aux="tp", hidden=5120, d_ffn=13824,
                        desc="BASELINE config 4, one decoder layer of the 13B shape (hidden 5120, 40 heads x 128, "
                             "intermediate 13824 = 108 x 128) tensor-parallel over the ranks: batch 64, context 8192, "
                             "ragged K/V ranks (mean 64); heads and FFN channels sharded, NCCL all-reduce per block and "
                             "an all-gather of the FFN hidden vector; needs --gpus >= 2"),
    "c4_stack": dict(batch=64, heads=40, head_dim=128, context=8192, aux="stack_tp", hidden=5120, d_ffn=13824, layers=40,
                     desc="BASELINE config 4: the LLaVA-Next-13B-shape LSVD layer stack (hidden 5120, 40 heads x 128, "
                          "intermediate 13824, 40 layers), random init with ragged K/V ranks (mean 64), batch 64, context 8192, "
                          "int8 latent cache; heads and FFN channels tensor-parallel over the ranks with an NCCL all-reduce per "
                          "block; one decode step of the whole stack per step; needs --gpus >= 2 (the cache alone is 107 GB)"),
    "c5_e2e": dict(batch=8, heads=32, head_dim=128, context=4096, aux="stack_e2e", hidden=4096, d_ffn=11008, layers=32,
                   decode_steps=256,
                   desc="BASELINE config 5: a 32-layer LLaVA-Next-7B-shape LSVD W8A8 language-model stack, random init: prefill "
                        "of 8 x 4096 tokens (latent-projection, gate / up / down GEMMs on tcgen05 kind::i8, latent cache written "
                        "by the prefill), then 256 decode steps; one step = one whole prefill + decode run"),
    "fig5_mixffn": dict(batch=32, context=0, aux="mixffn", hidden=4096, d_ffn=14336,
                        desc="the reference's mixffn W8A8 FFN (its own structure and fp32 conventions) at the shape of "
                             "its layer benchmark: hidden 4096, intermediate 14336, 32 tokens, svd_ratio 0.5, "
                             "rank_ratio 0.5, round_to 64"),
    "c5_prefill_append": dict(batch=8, context=4096, heads=32, aux="append",
                              desc="BASELINE config 5 prefill, cache append of one layer: K and V latents of 8 x 4096 "
                                   "tokens (32 heads, ragged ranks mean 64) quantised and scattered into the int8 cache"),
    "c5_prefill_ffn": dict(batch=8, context=4096, aux="prefill_ffn",
                           desc="BASELINE config 5 prefill, FFN block of one layer: 8 x 4096 tokens through the hybrid "
                                "SVD/RTN FFN 4096/11008 (rank 512, 50 % SVD channels) on the tcgen05 int8 GEMM"),
}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._pump, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def timed_repeats(loop, steps, barrier, world, dev, min_seconds=0.5, min_repeats=5, max_repeats=400):
    """Milliseconds of repeated runs of exactly `steps` steps (`loop(steps)` enqueues them): every repeat sits between a
    barrier + synchronize on both sides and is timed by CUDA events; with several ranks a repeat counts as its slowest
    rank.  Repeats go on until they add up to `min_seconds` (the ranks decide on the reduced times, hence together)."""
    times = []
    while True:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        loop(steps)
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(t.item())
        if (len(times) >= min_repeats and sum(times) >= min_seconds * 1e3) or len(times) >= max_repeats:
            return times


def spread(times, steps):
    """p50 / p20 / p80 of the repeats, per step, in microseconds (the reference's harness reports the same three,
    kernels/layer_bench/ffn_kernel/utils.py:709-712)."""
    s = sorted(times)
    pick = lambda q: s[min(len(s) - 1, int(q * len(s)))] / steps * 1e3
    return {"repeats": len(s), "p50_us": pick(0.5), "p20_us": pick(0.2), "p80_us": pick(0.8)}


def make_workload(w, device, seed):
    """Synthetic cache, weights and per-step inputs, resident on `device`; the cache is built by the library's
    own append kernel from fp16 N(0,1) latents (bit-identical to the reference's PyTorch quantiser)."""
    from lsvd_b200 import synth, cache_append, LatentCacheLayout, InferState
    B, H, D, L = w["batch"], w["heads"], w["head_dim"], w["context"]
    kr = synth.ragged_ranks(H, 64, seed=0) if w["ragged"] else [64] * H
    vr = synth.ragged_ranks(H, 64, seed=1) if w["ragged"] else [64] * H
    shared = bool(w.get("shared_kv"))          # one cached latent per head serves as K and as V latent
    if shared:
        vr = kr
    lay = LatentCacheLayout(kr, vr, head_major=w.get("cache_layout", "slot") == "head", shared_kv=shared)
    seq = L + 1                      # context plus the slot of the decoding token, as the reference's benchmark
    grow = DECODE_TOKENS if w.get("full") else 0     # slots reserved for the tokens the decode loop appends
    n_slots = B * (seq + grow)
    g = torch.Generator(device=device).manual_seed(seed)
    ck, sk, cv, sv = lay.alloc(n_slots, device)
    chunk = 8192
    for s0 in range(0, n_slots, chunk):
        n = min(chunk, n_slots - s0)
        lk = torch.randn(n, lay.sum_k, generator=g, device=device, dtype=torch.float32).half()
        lv = None if shared else torch.randn(n, lay.sum_v, generator=g, device=device, dtype=torch.float32).half()
        dest = torch.arange(s0, s0 + n, dtype=torch.int32, device=device)
        cache_append(lay, lk, lv, dest, ck, sk, cv, sv)
    up_k = (torch.randn(lay.sum_k, D, generator=g, device=device) / 8).half()
    up_v = (torch.randn(lay.sum_v, D, generator=g, device=device) / 8).half()
    st = InferState(B, seq + grow, [seq] * B, device=device)
    return dict(layout=lay, ck=ck, cv=cv, sk=sk, sv=sv, up_k=up_k, up_v=up_v, state=st, B=B, H=H, D=D, L=L, seq=seq,
                n_slots=n_slots, grow=grow)


DECODE_TOKENS = int(os.environ.get("LSVD_BENCH_DECODE_TOKENS", "128"))          # BASELINE config 3: "decode 128 tokens"


def algorithmic_bytes(wl):
    """Bytes one launch of the streaming kernel must move: the int8 K and V latents of every cached token, their
    fp16 scales and the slot indices.  With a growing context: the mean over the decode loop's lengths."""
    lay, B, H = wl["layout"], wl["B"], wl["H"]
    tokens = B * (wl["seq"] + (wl["grow"] - 1) / 2.0) if wl.get("grow") else B * wl["seq"]
    sides = 1 if lay.shared_kv else 2          # a shared latent and its scale are stored, and must be read, once
    cache = tokens * (lay.sum_k + (0 if lay.shared_kv else lay.sum_v))
    scales = tokens * H * 2 * sides
    slots = tokens * 4
    return int(cache + scales + slots)


FFN_SHAPE = dict(d_in=4096, d_ffn=11008, rank=512, n_svd=5504, K=172)
FFN_BYTES = 2 * 4096 * 512 + 2 * 512 * 5504 + 2 * 5504 * 4096 + 11008 * 4096      # int8 weights of one FFN
FFN_RTN_PAIR_BYTES = 2 * 5504 * 4096                                               # its largest launch


def make_ffn(device, seed, copies, input_had=True):
    """`copies` hybrid FFNs with different seeded weights (cycled so that weights never sit in L2 between steps)."""
    from lsvd_b200 import synth
    from lsvd_b200.ffn import HybridFFN
    hk = synth.sign_matrix(FFN_SHAPE["K"], seed=0)
    out = []
    for c in range(copies):
        w = synth.ffn_weights(FFN_SHAPE["d_in"], FFN_SHAPE["d_ffn"], FFN_SHAPE["rank"], FFN_SHAPE["n_svd"],
                              seed=seed + c, had_K=hk, K=FFN_SHAPE["K"], input_had=input_had)
        out.append(HybridFFN({k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in w.items()}))
    return out


def run_ours(args, rank, world, local):
    from lsvd_b200 import _lib, cache_append, token_decode_attention_int8_latent_absorb
    from lsvd_b200.attention import attn_decode_workspace_bytes, decode_advance
    _lib.load()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    w = dict(WORKLOADS[args.workload])
    w["cache_layout"] = args.cache_layout
    w["shared_kv"] = args.shared_kv
    has_attn = not w.get("ffn_only", False)
    has_ffn = w.get("ffn", False)
    if w.get("ffn_only"):
        w["batch"] = args.tokens
    B = w["batch"]
    g = torch.Generator().manual_seed(7 + rank)
    n_in = 8
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    host_in, dev_in, stage_in = [], [], []
    launches = 0

    full = w.get("full", False)
    if has_attn:
        wl = make_workload(w, dev, seed=1000 + rank)
        lay, st, H, D = wl["layout"], wl["state"], wl["H"], wl["D"]
        ws = torch.empty(attn_decode_workspace_bytes(B, lay, wl["seq"]), dtype=torch.uint8, device=dev)
        attn_out = torch.empty(B, H, D, dtype=torch.float16, device=dev)
        shapes = [(B, H * D)] if full else [(B, H, D), (B, lay.sum_k), (B, lay.sum_v)]
        launches += 9 if full else 4
    else:
        shapes = [(B, FFN_SHAPE["d_in"])]
    if has_ffn:
        ffns = make_ffn(dev, seed=50 + rank, copies=1 if has_attn else 3, input_had=not full)
        ffn_out = torch.empty(B, FFN_SHAPE["d_in"], dtype=torch.float16, device=dev)
        launches += 7
    layer = None
    if full:
        # the whole decoder layer: RMSNorm + A8 quantiser, int8 latent projection (query, K and V latents), cache
        # append, attention with the query up-factor folded into the K factor, fused W_uv W_o int8 projection +
        # residual, hybrid FFN with its RMSNorm prologue + residual
        from lsvd_b200.layer import LSVDDecoderLayer, make_layer_weights
        RANK_Q = 64
        lw = make_layer_weights(H * D, H, D, RANK_Q, lay.k_ranks, lay.v_ranks, seed=70 + rank, shared_kv=lay.shared_kv)
        layer = LSVDDecoderLayer(lay, D, RANK_Q, {k: v.to(dev) for k, v in lw.items()}, ffns[0])
        proj_bytes = lw["W_lat_q"].numel() + lw["W_uvo_q"].numel()
    # per-step inputs; host copies live in pinned memory for the end-to-end leg
    # A step's inputs (query + the new token's K and V latents) sit in ONE buffer, so a step costs one copy:
    # n_in such buffers in pinned host memory, their copies in HBM, and the staging buffer the graph reads.
    sizes = [int(torch.tensor(shp).prod().item()) for shp in shapes]
    total = sum(-(-n // 8) * 8 for n in sizes)                     # 16-byte aligned pieces
    host_pack = [torch.empty(total, dtype=torch.float16).pin_memory() for _ in range(n_in)]
    for hp in host_pack:
        hp.copy_(torch.randn(total, generator=g).half())
    dev_pack = [t.to(dev) for t in host_pack]
    stage_pack = torch.empty_like(dev_pack[0])

    def views(buf):
        out, off = [], 0
        for shp, n in zip(shapes, sizes):
            out.append(buf[off:off + n].view(*shp))
            off += -(-n // 8) * 8
        return out
    host_in = [[views(hp)[i] for hp in host_pack] for i in range(len(shapes))]
    dev_in = [[views(dp)[i] for dp in dev_pack] for i in range(len(shapes))]
    stage_in = views(stage_pack)
    result = ffn_out if has_ffn else attn_out
    host_out = torch.empty(result.shape, dtype=torch.float16).pin_memory()

    def step(inputs, i, ev=None):
        """One decode step of the layer's hot path.  The FFN takes the attention output's heads flattened
        (hidden = heads x head_dim) as its input: the data dependency of the layer without the projections."""
        if full:
            # the layer step, then one token further on the device: lengths + 1, the new token's slot looked up; after
            # DECODE_TOKENS steps the requests start over at the initial context (the slots reserved for them are reused)
            # (the move runs beside the output projection and the FFN, which no longer read the state)
            layer(inputs[0], wl["ck"], wl["sk"], wl["cv"], wl["sv"], st, out=ffn_out, timing_events=ev,
                  after_attention=lambda: decode_advance(st, base_len=wl["seq"], period=DECODE_TOKENS, status_word=status))
            return
        if has_attn:
            q, lk, lv = inputs
            cache_append(lay, lk, None if lay.shared_kv else lv, st.mem_index, wl["ck"], wl["sk"], wl["cv"], wl["sv"])
            token_decode_attention_int8_latent_absorb(q, st, H, D, wl["ck"], wl["sk"], wl["cv"], wl["sv"], wl["up_k"],
                                                      wl["up_v"], layout=lay, out=attn_out, workspace=ws,
                                                      status_word=status, timing_events=ev)
            x = attn_out.view(B, H * D)
        else:
            x = inputs[0]
        if has_ffn:
            ffns[i % len(ffns)](x, out=ffn_out)

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    pick = lambda pool, i: [p[i % n_in] for p in pool]
    for i in range(max(args.warmup, 3)):
        step(pick(dev_in, i), i)
    torch.cuda.synchronize()

    # CUDA graphs of the step, as the reference's harness replays its layer (kernels/layer_bench/ffn_kernel/utils.py:687-706):
    # one graph per FFN weight copy, all reading the staging inputs.
    graphs = []
    side = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(side):
        for c in range(len(ffns) if has_ffn else 1):
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=side):
                step(stage_in, c)
            graphs.append(gr)
    torch.cuda.synchronize()

    def load_inputs(i, from_host):
        stage_pack.copy_((host_pack if from_host else dev_pack)[i % n_in], non_blocking=True)

    # End-to-end form of a step: the copy of THIS step's inputs out of pinned host memory, the step, and the copy of its
    # result back into pinned host memory, as one graph per host input buffer (the copies are graph nodes, so a step is
    # one host call; nothing is overlapped across steps: the nodes of a graph run in order, and so do the replays).
    graphs_e2e = []
    with torch.cuda.stream(side):
        for j in range(n_in):
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=side):
                stage_pack.copy_(host_pack[j], non_blocking=True)
                step(stage_in, j % len(graphs))
                host_out.copy_(result, non_blocking=True)
            graphs_e2e.append(gr)
    torch.cuda.synchronize()

    for i in range(3):
        load_inputs(i, False)
        graphs[i % len(graphs)].replay()
    torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    # ---- device-resident leg (value): inputs already in HBM, graph replays ----
    def loop_dev(n):
        for i in range(n):
            load_inputs(i, False)                   # device-to-device refresh of this step's inputs (a few hundred KB)
            graphs[i % len(graphs)].replay()

    # ---- end-to-end leg: this step's inputs from pinned host memory, the result read back, every step ----
    def loop_e2e(n):
        for i in range(n):
            graphs_e2e[i % n_in].replay()

    t_dev = timed_repeats(loop_dev, args.steps, barrier, world, dev)
    t_e2e = timed_repeats(loop_e2e, args.steps, barrier, world, dev)
    ms_total, ms_e2e = statistics.median(t_dev), statistics.median(t_e2e)
    # ---- the dominant kernel on its own, timed by event pairs on the launching stream (eager steps) ----
    kernel_ms = []
    if has_attn:
        kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for a, b in kev:
            a.record()
            b.record()
        torch.cuda.synchronize()
        for i in range(args.steps):
            step(pick(dev_in, i), i, kev[i])
        torch.cuda.synchronize()
        kernel_ms = [a.elapsed_time(b) for a, b in kev]
    else:
        # the RTN gate/up pair (45 MB of weights) of the FFN: the plan's fifth launch, other copies' weights in between
        x = dev_in[0][0]
        for f in ffns:
            f(x, out=ffn_out)
        kev = []
        for i in range(args.steps):
            f = ffns[i % len(ffns)]
            _, calls = f._plan(B, dev)
            fn, a = calls[4]
            import ctypes
            s_ptr = torch.cuda.current_stream().cuda_stream
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            fn(ctypes.byref(a), s_ptr)
            a1.record()
            kev.append((a0, a1))
        torch.cuda.synchronize()
        kernel_ms = [a.elapsed_time(b) for a, b in kev]
    clocks = sampler.stop() if rank == 0 else None
    if status.item() != 0:
        raise RuntimeError(f"device status word = {status.item()}")

    if rank != 0:
        return None
    ms_step = ms_total / args.steps
    tokens = B * world
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    k_ms = statistics.mean(kernel_ms)
    if has_attn:
        abytes = algorithmic_bytes(wl)
        kname = "latent_stream_ring_kernel" if args.cache_layout == "head" else "latent_stream_kernel"
    else:
        abytes, kname = FFN_RTN_PAIR_BYTES + B * 4096 + 2 * 5504 * 4, "w8a8_gemv_kernel (RTN gate/up pair)"
    achieved = abytes / (k_ms * 1e-3) / 1e9
    step_bytes = (algorithmic_bytes(wl) if has_attn else 0) + (FFN_BYTES if has_ffn else 0) + (proj_bytes if full else 0)
    h2d = stage_pack.numel() * stage_pack.element_size()
    d2h = host_out.numel() * host_out.element_size()
    what = []
    if full:
        what.append("RMSNorm + A8 quantiser + int8 latent projection (Q, K, V latents) + cache append (K+V) + int8 latent "
                    "decode attention (absorb, query up-factor folded into K) + fused W_uv W_o int8 projection + residual")
    elif has_attn:
        what.append("cache append (K+V) + int8 latent decode attention (absorb) + V up-projection")
    if has_ffn:
        what.append("hybrid SVD/RTN FFN (input rotation, A8 quantisers, SVD and RTN gate/up, Hadamard 64x172, down)")
    line = {
        "metric": "decode_tokens_per_s", "value": tokens / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 (int32 accumulate), fp32 softmax, fp16 out",
        "data": "synthetic",
        "config": bench_config(args, w, B, world),
        "config_detail": {"step": " + ".join(what), "launch": "CUDA graph replay of the step",
                          "e2e": "one graph per step: copy of the step's inputs from pinned host memory, the step, copy of the "
                                 "result to pinned host memory; steps strictly one after the other",
                          "cache_layout": args.cache_layout if has_attn else None, "shared_kv_latent": bool(args.shared_kv) if has_attn else None,
                          "l2": "inputs larger than L2: every step streams %.0f MB of cache/weights%s"
                                % (step_bytes / 1e6, "" if has_attn else " (three weight copies cycled, 300 MB)")},
        "e2e": {"value": tokens / (ms_e2e / args.steps * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches * args.steps,
        "roofline": {"kernel": kname, "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "of": "measured" if "hbm_gbs" in peaks else "fallback",
                     # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this workload, from the
                     # ncu captures summarised under profiles/ (context 4097: 278.4 MB + 4.8 MB for the ring kernel on the
                     # head-major cache, 277.8 MB + 7.2 MB for the register-fed kernel on the slot-major one); other
                     # workloads were not captured
                     "traffic": ((283184384 if args.cache_layout == "head" else 284975872)
                                 if (has_attn and w["batch"] == 16 and w["context"] == 4096 and w["ragged"] and not args.shared_kv)
                                 else None),
                     "algorithmic_bytes_per_launch": abytes, "kernel_us": k_ms * 1e3, "frac_of_8TBs": achieved / 8000.0},
        "parts": {"step_us": ms_step * 1e3, "step_hbm_gbs": step_bytes / (ms_step * 1e-3) / 1e9,
                  "step_algorithmic_bytes": step_bytes, "dominant_kernel_us": k_ms * 1e3,
                  "value_leg": spread(t_dev, args.steps), "e2e_leg": spread(t_e2e, args.steps)},
        "clocks": clocks,
    }
    return line


def run_aux(args, rank, world, local):
    """Auxiliary workloads with their own step: the rotary attention form and the prefill FFN.  Same timing rules
    and JSON keys as the decode workloads; ranks run replicas (no collective on these paths)."""
    from lsvd_b200 import _lib
    _lib.load()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    w = WORKLOADS[args.workload]
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    g = torch.Generator(device=dev).manual_seed(11 + rank)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    if w["aux"] == "rope":
        from lsvd_b200.attention import InferState, token_decode_attention_flash_int8_latent_per_head_decoding_rope as rope
        B, H, D, L, R = w["batch"], w["heads"], w["head_dim"], w["context"], 64
        n_slots = B * L
        ck = torch.randint(-128, 128, (n_slots, H, R), dtype=torch.int8, device=dev, generator=g)
        cv = torch.randint(-128, 128, (n_slots, H, R), dtype=torch.int8, device=dev, generator=g)
        sk = (torch.rand(n_slots, H, device=dev, generator=g) * 0.02 + 0.01).half()
        sv = (torch.rand(n_slots, H, device=dev, generator=g) * 0.02 + 0.01).half()
        wk = torch.randint(-128, 128, (R, H * D), dtype=torch.int8, device=dev, generator=g)
        wks = (torch.rand(1, H * D, device=dev, generator=g) * 0.002 + 0.001).half()
        st = InferState(B, L, [L] * B, device=dev)
        qs_host = [torch.randn(B, H, D).half().pin_memory() for _ in range(8)]
        qs = [t.to(dev) for t in qs_host]
        q_in = torch.empty_like(qs[0])
        out = torch.empty(B, H, R, dtype=torch.float16, device=dev)
        need = _lib.load().lsvd_attn_decode_rope_workspace_bytes(B, H, D, R, L, 256)
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        host_out = torch.empty(out.shape, dtype=torch.float16).pin_memory()
        step = lambda: rope(q_in, st, H, D, ck, sk, cv, sv, wk, wks, out=out, workspace=ws, status_word=status)
        feed = lambda i, host: q_in.copy_((qs_host if host else qs)[i % 8], non_blocking=True)
        units, metric, launches = B, "decode_tokens_per_s", 3
        abytes = n_slots * H * R * 2 + n_slots * H * 4 + n_slots * 4
        roof = dict(kernel="rope_recon_kernel", bound="hbm", peak=float(peaks.get("hbm_gbs", 6650.0)), unit="GB/s", work=abytes)
        h2d, d2h = q_in.numel() * 2, out.numel() * 2
        l2 = "the cache (%.0f MB) %s L2" % (abytes / 1e6, "exceeds" if abytes > 126e6 else "fits in")
        what = "cos/sin table + rotary reconstruct attention + merge"
    elif w["aux"] == "block":
        from lsvd_b200.attention import InferState
        from lsvd_b200.block import Int8AttentionBlock
        B, H, D, L = w["batch"], w["heads"], w["head_dim"], w["context"]
        torch.manual_seed(21 + rank)
        blk = Int8AttentionBlock(H * D, H, D, 0.5, device=dev)
        R = blk.rank_head
        n_slots = B * L
        ck = torch.randint(-128, 128, (n_slots, H, R), dtype=torch.int8, device=dev, generator=g)
        cv = torch.randint(-128, 128, (n_slots, H, R), dtype=torch.int8, device=dev, generator=g)
        sk = (torch.rand(n_slots, H, device=dev, generator=g) * 0.02 + 0.01).half()
        sv = (torch.rand(n_slots, H, device=dev, generator=g) * 0.02 + 0.01).half()
        st = InferState(B, L, [L] * B, device=dev)
        xs_host = [torch.randn(B, 1, H * D).half().pin_memory() for _ in range(8)]
        xs = [t.to(dev) for t in xs_host]
        x_in = torch.empty_like(xs[0])
        box = {}
        host_out = torch.empty(B, 1, H * D, dtype=torch.float16).pin_memory()
        out = torch.empty(B, 1, H * D, dtype=torch.float16, device=dev)

        def eager_step():
            out.copy_(blk(x_in, ck, sk, cv, sv, st))
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                eager_step()
        torch.cuda.current_stream().wait_stream(side)
        block_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(block_graph):
            eager_step()
        step = block_graph.replay
        feed = lambda i, host: x_in.copy_((xs_host if host else xs)[i % 8], non_blocking=True)
        units, metric, launches = B, "decode_tokens_per_s", 5
        wbytes = (3 * H * R * H * D + R * H * D + H * R * H * D) * 2 + R * H * D
        abytes = n_slots * H * R * 2 + n_slots * H * 4 + n_slots * 4 + wbytes
        roof = dict(kernel="whole block step (5 library launches of this package + 4 of the fp16 GEMM / elementwise library)",
                    bound="hbm", peak=float(peaks.get("hbm_gbs", 6650.0)), unit="GB/s", work=abytes)
        h2d, d2h = x_in.numel() * 2, out.numel() * 2
        l2 = "cache + weights (%.0f MB) fit in L2: the figure is a warm-L2 one" % (abytes / 1e6)
        what = "RMSNorm + fp16 latent GEMM + query up-projection + append + rotary attention (3 launches) + fp16 output GEMM + residual"
    elif w["aux"] == "append":
        from lsvd_b200 import synth
        from lsvd_b200.attention import LatentCacheLayout, cache_append
        T, H = w["batch"] * w["context"], w["heads"]
        lay = LatentCacheLayout(synth.ragged_ranks(H, 64, seed=0), synth.ragged_ranks(H, 64, seed=1))
        lats_host = None
        lk = [torch.randn(T, lay.sum_k, device=dev, generator=g).half() for _ in range(2)]
        lv = [torch.randn(T, lay.sum_v, device=dev, generator=g).half() for _ in range(2)]
        dest = torch.randperm(T, device=dev, generator=g).to(torch.int32)
        ck = torch.empty(T, lay.sum_k, dtype=torch.int8, device=dev)
        cv = torch.empty(T, lay.sum_v, dtype=torch.int8, device=dev)
        sk = torch.empty(T, H, dtype=torch.float16, device=dev)
        sv = torch.empty(T, H, dtype=torch.float16, device=dev)
        out = sk
        host_out = torch.empty(sk.shape, dtype=torch.float16).pin_memory()
        hk = lk[0].cpu().pin_memory()
        hv = lv[0].cpu().pin_memory()
        turn = [0]

        def step():
            i = turn[0] % 2
            turn[0] += 1
            cache_append(lay, lk[i], lv[i], dest, ck, sk, cv, sv, status_word=status)

        def feed(i, host):
            if host:                      # the latents of the step come from pinned host memory
                lk[turn[0] % 2].copy_(hk, non_blocking=True)
                lv[turn[0] % 2].copy_(hv, non_blocking=True)
        units, metric, launches = T, "prefill_tokens_per_s", 1
        abytes = T * (lay.sum_k + lay.sum_v) * 3 + T * H * 4 + T * 4
        roof = dict(kernel="cache_append_kernel", bound="hbm", peak=float(peaks.get("hbm_gbs", 6650.0)), unit="GB/s", work=abytes)
        h2d, d2h = (hk.numel() + hv.numel()) * 2, host_out.numel() * 2
        l2 = "%.0f MB per step (fp16 latents in, int8 rows and fp16 scales out): larger than L2" % (abytes / 1e6)
        what = "one launch: per (token, head) absmax, scale, int8 codes, scatter to the slot rows (K and V)"
    elif w["aux"] == "mixffn":
        from types import SimpleNamespace
        from lsvd_b200.mixffn import MixedFFNGateUpDenseLatentFused
        M, hid, dff = w["batch"], w["hidden"], w["d_ffn"]
        lin = lambda o, i: SimpleNamespace(weight=(torch.randn(o, i, device=dev, generator=g) / i ** 0.5).half())
        src = SimpleNamespace(norm=SimpleNamespace(weight=torch.randn(hid, device=dev, generator=g).half(), variance_epsilon=1e-6),
                              up_proj=lin(dff, hid), gate_proj=lin(dff, hid), down_proj=lin(hid, dff))
        mods = [MixedFFNGateUpDenseLatentFused.from_float(src, 0.5, 0.5, 64, seed=s) for s in range(2)]   # 2 x 131 MB > L2
        del src
        xs_host = [torch.randn(M, hid).half().pin_memory() for _ in range(8)]
        xs = [t.to(dev) for t in xs_host]
        x_in = torch.empty_like(xs[0])
        out = torch.empty(M, hid, dtype=torch.float16, device=dev)
        host_out = torch.empty(out.shape, dtype=torch.float16).pin_memory()
        graphs = []
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for mod in mods:
                for _ in range(2):
                    mod(x_in, out=out)
        torch.cuda.current_stream().wait_stream(side)
        for mod in mods:
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                mod(x_in, out=out)
            graphs.append(gr)
        turn = [0]

        def step():
            graphs[turn[0] % 2].replay()
            turn[0] += 1
        feed = lambda i, host: x_in.copy_((xs_host if host else xs)[i % 8], non_blocking=True)
        units, metric, launches = M, "decode_tokens_per_s", 10
        m0 = mods[0]
        wbytes = sum(getattr(m0, n).numel() for n in ("ab_a_q", "up_b_q", "gate_b_q", "up_q", "gate_q", "down_a_q", "down_b_q", "down_q"))
        abytes = wbytes + M * hid * 4
        roof = dict(kernel="whole mixffn step (10 launches: 7 weight-streaming products, 3 quantisers)", bound="hbm",
                    peak=float(peaks.get("hbm_gbs", 6650.0)), unit="GB/s", work=abytes)
        h2d, d2h = x_in.numel() * 2, out.numel() * 2
        l2 = "two weight sets of %.0f MB alternate, so every step streams its weights from HBM" % (wbytes / 1e6)
        what = "RMSNorm quantiser + low-rank and dense gate/up (fp32 SwiGLU) + shared quantiser + low-rank and dense down + residual; CUDA graph replay"
    else:
        M = w["batch"] * w["context"]
        ffn = make_ffn(dev, seed=50 + rank, copies=1)[0]
        xs_host = [torch.randn(M, FFN_SHAPE["d_in"]).half().pin_memory() for _ in range(2)]
        xs = [t.to(dev) for t in xs_host]
        x_in = torch.empty_like(xs[0])
        out = torch.empty(M, FFN_SHAPE["d_in"], dtype=torch.float16, device=dev)
        host_out = torch.empty(out.shape, dtype=torch.float16).pin_memory()
        step = lambda: ffn(x_in, out=out)
        feed = lambda i, host: x_in.copy_((xs_host if host else xs)[i % 2], non_blocking=True)
        units, metric, launches = M, "prefill_tokens_per_s", 9
        ops = 2.0 * M * FFN_BYTES
        int8_peak = 2.0 * float(peaks.get("bf16_tflops", 1590.0))
        roof = dict(kernel="i8gemm_tcgen05_kernel (whole FFN step: six GEMM launches + three quantiser launches)",
                    bound="tensor", peak=int8_peak, unit="TOP/s", work=ops,
                    peak_note="int8 dense rate taken as twice the measured bf16 GEMM figure; nominal 4500")
        h2d, d2h = x_in.numel() * 2, out.numel() * 2
        l2 = "activations of %.0f MB per stage exceed L2" % (M * FFN_SHAPE["d_ffn"] * 2 / 1e6)
        what = "input rotation + A8 quantisers + SVD and RTN gate/up GEMMs + Hadamard 64x172 + down GEMM"

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        feed(i, False)
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    def loop_dev(n):
        for i in range(n):
            feed(i, False)
            step()

    def loop_e2e(n):
        for i in range(n):
            feed(i, True)
            step()
            host_out.copy_(out, non_blocking=True)

    t_dev = timed_repeats(loop_dev, args.steps, barrier, world, dev)
    t_e2e = timed_repeats(loop_e2e, args.steps, barrier, world, dev)
    ms_total, ms_e2e = statistics.median(t_dev), statistics.median(t_e2e)
    # the step alone (no input refresh), for the roofline figure
    k0, k1 = ev(), ev()
    torch.cuda.synchronize()
    k0.record()
    for i in range(args.steps):
        step()
    k1.record()
    torch.cuda.synchronize()
    k_ms = k0.elapsed_time(k1) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    if status.item() != 0:
        raise RuntimeError(f"device status word = {status.item()}")
    if rank != 0:
        return None
    ms_step = ms_total / args.steps
    achieved = roof["work"] / (k_ms * 1e-3) / (1e9 if roof["bound"] == "hbm" else 1e12)
    line = {
        "metric": metric, "value": units * world / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 (int32 accumulate), fp16 out", "data": "synthetic",
        "config": bench_config(args, w, w["batch"], world),
        "config_detail": {"step": what, "launch": "CUDA graph replay of the step" if w["aux"] in ("mixffn", "block") else "eager launches on one stream", "l2": l2},
        "e2e": {"value": units * world / (ms_e2e / args.steps * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches * args.steps,
        "roofline": {"kernel": roof["kernel"], "bound": roof["bound"], "achieved": achieved, "peak": roof["peak"],
                     "unit": roof["unit"], "frac": achieved / roof["peak"], "of": "measured" if peaks else "fallback",
                     "traffic": None, "work_per_step": roof["work"], "step_us": k_ms * 1e3,
                     **({"peak_note": roof["peak_note"]} if "peak_note" in roof else {})},
        "parts": {"value_leg": spread(t_dev, args.steps), "e2e_leg": spread(t_e2e, args.steps)},
        "clocks": clocks,
    }
    return line


def run_tp(args, rank, world, local):
    """One tensor-parallel decoder layer step (TPDecoderLayer): total work fixed, sharded over the ranks."""
    import torch.distributed as dist
    from lsvd_b200 import _lib, synth
    from lsvd_b200.attention import InferState
    from lsvd_b200.layer import TPDecoderLayer, make_layer_weights
    from lsvd_b200.parallel import shard_layer
    _lib.load()
    w = WORKLOADS[args.workload]
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world == 1 and "RANK" not in os.environ:
        # the unsharded layer on one GPU (the first point of the strong-scaling curve): a process group of one
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(29500 + os.getpid() % 2000))
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    else:
        dist.init_process_group("nccl", device_id=dev)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    B, H, D, L, hid, dff, rq = w["batch"], w["heads"], w["head_dim"], w["context"], w["hidden"], w["d_ffn"], 64
    kr, vr = synth.ragged_ranks(H, 64, seed=0), synth.ragged_ranks(H, 64, seed=1)
    lw_full = make_layer_weights(hid, H, D, rq, kr, vr, seed=1)                       # same seed: same weights on every rank
    fw_full = synth.ffn_weights(hid, dff, 640, dff // 2, seed=2, had_K=synth.sign_matrix(108, seed=0).float(), K=108, input_had=False)
    ew = args.emulate_world if (args.emulate_world > 1 and world == 1) else world
    lw, fw, info = shard_layer(lw_full, fw_full, kr, vr, rq, ew, rank)
    del lw_full, fw_full
    to = lambda d: {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
    head_major = args.cache_layout == "head"
    layer = TPDecoderLayer(to(lw), to(fw), info, D, rq, ew, head_major=head_major)
    layer.skip_collectives = ew != world
    lay = layer.layout
    g = torch.Generator(device=dev).manual_seed(5 + rank)
    n_slots = B * (L + 1)
    h_loc = lay.num_heads
    ck, sk, cv, sv = lay.alloc(n_slots, dev)
    for t in (ck, cv):                                  # random codes, chunked: torch's RNG makes int64 on the way
        flat = t.view(-1)
        for o in range(0, flat.numel(), 1 << 28):
            n = min(1 << 28, flat.numel() - o)
            flat[o:o + n] = torch.randint(-128, 128, (n,), dtype=torch.int8, device=dev, generator=g)
    sk.copy_((torch.rand(sk.shape, device=dev, generator=g) * 0.02 + 0.01).half())
    sv.copy_((torch.rand(sv.shape, device=dev, generator=g) * 0.02 + 0.01).half())
    st = InferState(B, L + 1, [L + 1] * B, device=dev)
    gx = torch.Generator().manual_seed(9)                                              # replicated hidden states
    xs_host = [torch.randn(B, hid, generator=gx).half().pin_memory() for _ in range(4)]
    xs = [t.to(dev) for t in xs_host]
    x_in = torch.empty_like(xs[0])
    host_out = torch.empty(B, hid, dtype=torch.float16).pin_memory()

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def loop(n, host, evs=None):
        for i in range(n):
            x_in.copy_((xs_host if host else xs)[i % 4], non_blocking=True)
            y = layer(x_in, ck, sk, cv, sv, st, timing_events=None if evs is None else evs[i])
            if host:
                host_out.copy_(y, non_blocking=True)
    loop(max(args.warmup, 3), False)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    t_dev = timed_repeats(lambda n: loop(n, False), args.steps, barrier, world, dev)
    t_e2e = timed_repeats(lambda n: loop(n, True), args.steps, barrier, world, dev)
    ms_total, ms_e2e = statistics.median(t_dev), statistics.median(t_e2e)
    # the dominant kernel of every rank (its share of the cache stream), by event pairs around that launch
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for a0, a1 in kev:
        a0.record()
        a1.record()
    barrier()
    loop(args.steps, False, kev)
    barrier()
    k_ms = statistics.mean(a0.elapsed_time(a1) for a0, a1 in kev)
    kt = torch.tensor([k_ms], dtype=torch.float64, device=dev)
    dist.all_reduce(kt, op=dist.ReduceOp.MAX)
    k_ms = kt.item()
    # where the step's time goes on rank 0: events around the runs of launches and the collectives
    seg_names = ("attention_block", "all_reduce_attn", "gate_up", "all_gather_h", "hadamard_down", "all_reduce_ffn", "finish")
    seg_sum = [0.0] * len(seg_names)
    barrier()
    all_evs = []
    for i in range(args.steps):              # back to back, as in the timed loop: a rank that runs ahead waits in a collective
        evs = []
        x_in.copy_(xs[i % 4], non_blocking=True)
        layer(x_in, ck, sk, cv, sv, st, segment_events=evs)
        all_evs.append(evs)
    barrier()
    for evs in all_evs[args.steps // 2:]:    # the second half: the ranks have settled into their steady offsets
        for j in range(len(seg_names)):
            seg_sum[j] += evs[j].elapsed_time(evs[j + 1]) * 1e3 / (args.steps - args.steps // 2)
    clocks = sampler.stop() if rank == 0 else None
    local_bytes = ck.numel() + cv.numel() + (sk.numel() + sv.numel()) * 2 + sum(
        v.numel() for v in list(lw.values()) + list(fw.values()) if isinstance(v, torch.Tensor) and v.dtype == torch.int8)
    stream_bytes = n_slots * (lay.sum_k + lay.sum_v + 4 * h_loc + 4)
    dist.destroy_process_group()
    if rank != 0:
        return None
    ms_step = ms_total / args.steps
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = stream_bytes / (k_ms * 1e-3) / 1e9
    return {
        "metric": "decode_tokens_per_s", "value": B / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8 (int32 accumulate), fp32 softmax, fp16 out", "data": "synthetic",
        "config": bench_config(args, w, B, world),
        **({"emulated": "rank 0 of a %d-way split on one GPU, collectives left out: a profiling aid, not a result" % ew} if ew != world else {}),
        "config_detail": {"step": "RMSNorm + A8, int8 latent projection, cache append, int8 latent decode attention on the rank's "
                                  "heads, row-parallel output projection + all-reduce, column-parallel hybrid FFN gate/up, "
                                  "all-gather of the hidden vector, Hadamard 128 x 108 + A8, row-parallel int32 down projection + "
                                  "all-reduce",
                          "launch": ("four CUDA-graph replays per step (the launches between the collectives) + three NCCL collectives, one stream"
                                     if layer.use_graphs else "eager launches (about 20 host calls per step), NCCL collectives on the same stream"),
                          "cache_layout": args.cache_layout,
                          "l2": "each rank streams %.0f MB of cache and weights per step" % (local_bytes / 1e6)},
        "e2e": {"value": B / (ms_e2e / args.steps * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": x_in.numel() * 2,
                "d2h_bytes_per_step": host_out.numel() * 2},
        "gpu_launches": 19 * args.steps,
        "roofline": {"kernel": "latent_stream_ring_kernel (slowest rank's share of the cache)", "bound": "hbm", "achieved": achieved,
                     "peak": peak, "unit": "GB/s", "frac": achieved / peak, "of": "measured" if peaks else "fallback",
                     "traffic": None, "algorithmic_bytes_per_launch": stream_bytes, "kernel_us": k_ms * 1e3},
        "parts": {"step_us": ms_step * 1e3, "bytes_per_gpu_per_step": local_bytes,
                  "step_hbm_gbs_per_gpu": local_bytes / (ms_step * 1e-3) / 1e9,
                  "segments_us_rank0": dict(zip(seg_names, seg_sum)),
                  "value_leg": spread(t_dev, args.steps), "e2e_leg": spread(t_e2e, args.steps)},
        "clocks": clocks,
    }


def bench_config(args, w, batch, world):
    """The `config` object of a line: the same object from both arms (ours / reference) of a workload at a given N."""
    tp = w.get("aux") in ("tp", "stack_tp")
    return {"workload": args.workload, "what": w["desc"], "layers": w.get("layers", 1),
            ("global_batch" if tp else "batch_per_gpu"): batch,
            "parallelism": f"tp{world}" if tp else ("single GPU" if world == 1 else f"{world} independent replicas")}


def run_stack(args, rank, world, local):
    """Whole layer stacks: config 4 (40 tensor-parallel layers, one decode step of the stack per step) and config 5
    (32 layers on one GPU: prefill of 8 x 4096 tokens, then 256 decode steps; one run per step)."""
    from lsvd_b200 import _lib, synth
    from lsvd_b200.attention import InferState, decode_advance
    from lsvd_b200.model import LSVDModel, TPModel, fill_random_cache
    _lib.load()
    w = WORKLOADS[args.workload]
    tp = w["aux"] == "stack_tp"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 or tp:
        import torch.distributed as dist
        if tp and world < 2:
            raise SystemExit("c4_stack needs --gpus 2, 4 or 8 under torchrun: its cache does not fit one GPU")
        dist.init_process_group("nccl", device_id=dev)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    B, H, D, L, hid, dff, nl, rq = w["batch"], w["heads"], w["head_dim"], w["context"], w["hidden"], w["d_ffn"], w["layers"], 64
    if args.layers > 0:
        nl = args.layers
    kr, vr = synth.ragged_ranks(H, 64, seed=0), synth.ragged_ranks(H, 64, seed=1)
    head_major = args.cache_layout == "head"

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if tp:
        K = 108
        n_slots = B * (L + 1)
        model = TPModel(nl, hid, H, D, dff, rq, kr, vr, 640, dff // 2, synth.sign_matrix(K, seed=0).float(), K, n_slots, world, rank,
                        device=dev, seed=100, head_major=head_major, fill_cache=True)
        st = InferState(B, L + 1, [L + 1] * B, device=dev)
        gx = torch.Generator().manual_seed(9)
        xs_host = [torch.randn(B, hid, generator=gx).half().pin_memory() for _ in range(4)]
        xs = [t.to(dev) for t in xs_host]
        x_in = torch.empty_like(xs[0])
        host_out = torch.empty(B, hid, dtype=torch.float16).pin_memory()

        def loop(n, host):
            for i in range(n):
                x_in.copy_((xs_host if host else xs)[i % 4], non_blocking=True)
                y = model.decode_step(x_in, st)
                if host:
                    host_out.copy_(y, non_blocking=True)
        loop(max(args.warmup, 3), False)
        if rank == 0:
            sampler.start()
            time.sleep(0.3)
        t_dev = timed_repeats(lambda n: loop(n, False), args.steps, barrier, world, dev, min_repeats=3)
        t_e2e = timed_repeats(lambda n: loop(n, True), args.steps, barrier, world, dev, min_repeats=3)
        ms_total, ms_e2e = statistics.median(t_dev), statistics.median(t_e2e)
        lay = model.layout
        per_layer_cache = n_slots * (lay.sum_k + lay.sum_v + 4 * lay.num_heads + 4)
        local_bytes = nl * per_layer_cache + model.weight_bytes
        units, metric = B, "decode_tokens_per_s"
        h2d, d2h = x_in.numel() * 2, host_out.numel() * 2
        what = "one decode step of %d tensor-parallel layers (each: about 20 host calls, 2 all-reduces, 1 all-gather)" % nl
        roof = dict(kernel="whole stack step, per GPU", bound="hbm", peak=float(peaks.get("hbm_gbs", 6650.0)), unit="GB/s",
                    work=local_bytes)
        launches = 19 * nl
        parts_extra = {"bytes_per_gpu_per_step": local_bytes}
    else:
        K = 172
        steps_dec = w["decode_steps"]
        n_slots = B * (L + steps_dec)
        model = LSVDModel(nl, hid, H, D, dff, rq, kr, vr, 512, dff // 2, synth.sign_matrix(K, seed=0).float(), K, n_slots, device=dev,
                          seed=200 + rank, head_major=head_major)
        r2t = torch.arange(n_slots, dtype=torch.int32).view(B, L + steps_dec)
        dest = torch.cat([r2t[b, :L] for b in range(B)]).contiguous().to(dev)
        gx = torch.Generator().manual_seed(9 + rank)
        x_host = torch.randn(B * L, hid, generator=gx).half().pin_memory()
        x_pre_dev = x_host.to(dev)
        x_pre = torch.empty_like(x_pre_dev)
        xd_host = [torch.randn(B, hid, generator=gx).half().pin_memory() for _ in range(4)]
        xd = [t.to(dev) for t in xd_host]
        x_in = torch.empty_like(xd[0])
        host_out = torch.empty(B, hid, dtype=torch.float16).pin_memory()
        st = InferState(B, L + steps_dec, [L + 1] * B, device=dev, req_to_token=r2t)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        pre_ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        split = {"prefill_ms": [], "decode_ms": []}

        def one_run(host, record=False):
            x_pre.copy_(x_host if host else x_pre_dev, non_blocking=True)
            if record:
                pre_ev[0].record()
            model.prefill(x_pre, dest)
            if record:
                pre_ev[1].record()
            # the decode loop restarts at the prefilled length: period = decode_steps brings the state back for the next run
            for t in range(steps_dec):
                x_in.copy_((xd_host if host else xd)[t % 4], non_blocking=True)
                dec_graph.replay()
                if host:
                    host_out.copy_(y_dec, non_blocking=True)
            if record:
                pre_ev[2].record()

        def loop(n, host):
            for _ in range(n):
                one_run(host)
        # a decode step of the whole stack (all layers + the device-side state advance) is one CUDA graph
        model.prefill(x_pre_dev, dest)
        dec_graph, y_dec = model.capture_decode(x_in, st, advance=dict(base_len=L + 1, period=steps_dec, status_word=status))
        one_run(False)
        if rank == 0:
            sampler.start()
            time.sleep(0.3)
        t_dev = timed_repeats(lambda n: loop(n, False), args.steps, barrier, world, dev, min_repeats=2, min_seconds=0.1)
        t_e2e = timed_repeats(lambda n: loop(n, True), args.steps, barrier, world, dev, min_repeats=2, min_seconds=0.1)
        ms_total, ms_e2e = statistics.median(t_dev), statistics.median(t_e2e)
        torch.cuda.synchronize()
        one_run(False, record=True)
        torch.cuda.synchronize()
        pre_ms, dec_ms = pre_ev[0].elapsed_time(pre_ev[1]), pre_ev[1].elapsed_time(pre_ev[2])
        if status.item() != 0:
            raise RuntimeError(f"device status word = {status.item()}")
        units, metric = (B * L + B * steps_dec) * world, "tokens_per_s"
        h2d, d2h = x_pre.numel() * 2 + steps_dec * x_in.numel() * 2, steps_dec * host_out.numel() * 2
        what = "%d layers: prefill of %d x %d tokens (tcgen05 GEMMs, cache written), then %d decode steps" % (nl, B, L, steps_dec)
        # tensor-core work of the prefill: the int8 GEMMs of every layer (latent projection, fused output projection, FFN)
        lat_rows = H * rq + sum(kr) + sum(vr)
        ops = 2.0 * B * L * nl * (lat_rows * hid + hid * sum(vr) + FFN_BYTES)
        int8_peak = 2.0 * float(peaks.get("bf16_tflops", 1590.0))
        roof = dict(kernel="the prefill's int8 GEMMs (i8gemm_tcgen05_kernel), all layers, over the prefill's whole time", bound="tensor",
                    peak=int8_peak, unit="TOP/s", work=ops, time_ms=pre_ms,
                    peak_note="int8 dense rate taken as twice the measured bf16 GEMM figure (nominal: 4500 TOP/s)")
        launches = nl * (9 + 15 * steps_dec)
        parts_extra = {"prefill_ms": pre_ms, "decode_ms": dec_ms, "prefill_tokens_per_s": B * L / (pre_ms * 1e-3),
                       "decode_tokens_per_s": B * steps_dec / (dec_ms * 1e-3), "decode_step_us": dec_ms / steps_dec * 1e3,
                       "prefill_int8_frac_of_nominal_4500": ops / (pre_ms * 1e-3) / 1e12 / 4500.0}
    clocks = sampler.stop() if rank == 0 else None
    if world > 1 or tp:
        import torch.distributed as dist
        dist.destroy_process_group()
    if rank != 0:
        return None
    ms_step = ms_total / args.steps
    t_roof = roof.get("time_ms", ms_step)
    achieved = roof["work"] / (t_roof * 1e-3) / (1e9 if roof["bound"] == "hbm" else 1e12)
    line = {
        "metric": metric, "value": units / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3) if tp else 1, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong" if tp else "weak", "vs_baseline": None, "dtype": "int8 (int32 accumulate), fp32 softmax, fp16 out",
        "data": "synthetic", "config": bench_config(args, w, B, world),
        "config_detail": {"step": what, "layers": nl,
                          "launch": "eager launches" if tp else "prefill: eager launches; decode: one CUDA graph per step of the stack",
                          "cache_layout": args.cache_layout,
                          "prefill_attention": None if tp else "none in the reference: every prefill token attends to itself only "
                                                                  "(its own V latent); the GEMMs and the cache write are those of a real prefill"},
        "e2e": {"value": units / (ms_e2e / args.steps * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches * args.steps,
        "roofline": {"kernel": roof["kernel"], "bound": roof["bound"], "achieved": achieved, "peak": roof["peak"], "unit": roof["unit"],
                     "frac": achieved / roof["peak"], "of": "measured" if peaks else "fallback", "traffic": None,
                     **({"peak_note": roof["peak_note"]} if "peak_note" in roof else {})},
        "parts": {"step_us": ms_step * 1e3, **parts_extra, "value_leg": spread(t_dev, args.steps), "e2e_leg": spread(t_e2e, args.steps)},
        "clocks": clocks,
    }
    return line


def cpu_baseline(workload, tokens, seconds_hint=15.0, threads=None):
    """The oracle (a CPU port of the reference's algorithm: the reference has no CPU implementation of latent
    attention, and its FFN module is fake-quant fp16 GPU code) timed on the host cores on a bounded sample of
    the same workload: a slice of the batch for attention, the full FFN on its tokens."""
    from oracle import attention as oattn, ffn as offn, quant
    from lsvd_b200 import synth
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    w = dict(WORKLOADS[workload])
    if w.get("aux"):
        return cpu_baseline_aux(w, seconds_hint, threads)
    if w.get("ffn_only"):
        w["batch"] = tokens
    B = w["batch"]
    has_attn, has_ffn = not w.get("ffn_only", False), w.get("ffn", False)
    bs = min(B, 4)
    fns = []
    if has_attn:
        H, D, L = w["heads"], w["head_dim"], w["context"]
        kr = synth.ragged_ranks(H, 64, seed=0) if w["ragged"] else [64] * H
        vr = synth.ragged_ranks(H, 64, seed=1) if w["ragged"] else [64] * H
        c = synth.attention_inputs(bs, H, D, kr, vr, [L + 1] * bs, seed=0)
        ko, vo = [0], [0]
        for a, b in zip(kr, vr):
            ko.append(ko[-1] + a)
            vo.append(vo[-1] + b)
        ck, sk = quant.latent_quant_ragged(c["latent_k"], ko)
        cv, sv = quant.latent_quant_ragged(c["latent_v"], vo)
        fns.append(lambda: oattn.decode_absorb(c["q"], ck, sk, cv, sv, c["up_k"], c["up_v"], ko, vo, c["req_to_token"],
                                               c["b_req_idx"], c["b_seq_len"], dtype=torch.float32))
    if has_ffn:
        fw = synth.ffn_weights(FFN_SHAPE["d_in"], FFN_SHAPE["d_ffn"], FFN_SHAPE["rank"], FFN_SHAPE["n_svd"], seed=0,
                               had_K=synth.sign_matrix(FFN_SHAPE["K"]).float(), K=FFN_SHAPE["K"])
        x = torch.randn(bs, FFN_SHAPE["d_in"], generator=torch.Generator().manual_seed(1)).half()
        fns.append(lambda: offn.hybrid_ffn_stages(x, fw))
    if w.get("full"):
        # the two int8 projections of the full layer (latent projection, fused output projection) on the same sample
        from oracle import layer as olayer
        from lsvd_b200.layer import make_layer_weights
        lw = make_layer_weights(H * D, H, D, 64, kr, vr, seed=70)
        xl = torch.randn(bs, H * D, generator=torch.Generator().manual_seed(2)).half()
        ol = torch.randn(bs, sum(vr), generator=torch.Generator().manual_seed(3)).half()
        fns.append(lambda: (olayer.linear_a8w8(olayer.rms_norm(xl, lw["ln1"], 1e-5), lw["W_lat_q"], lw["W_lat_s"]),
                            olayer.linear_a8w8(ol, lw["W_uvo_q"], lw["W_uvo_s"], residual=xl)))

    def once():
        for f in fns:
            f()
    once()
    n, t0 = 0, time.perf_counter()
    while True:
        once()
        n += 1
        dt = time.perf_counter() - t0
        if dt > seconds_hint or n >= 20:
            break
    return {"value": bs * n / dt, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"{bs} of {B} requests/tokens of the same workload, {n} steps, torch on {threads} threads "
                      f"(int8 products evaluated in float64 for exactness, attention in fp32; the cache is pre-quantised; "
                      f"left out of the sample: the cache append of the step's token, the RMSNorm in front of the FFN, the "
                      f"bookkeeping between steps; the context stays at its initial length)"}


def cpu_baseline_aux(w, seconds_hint, threads):
    """CPU port timings of the auxiliary workloads on a bounded sample."""
    import math
    from oracle import attention as oattn, ffn as offn, quant
    from lsvd_b200 import synth
    gen = torch.Generator().manual_seed(0)
    if w["aux"] in ("rope", "block"):
        H, D, L, R, hs = w["heads"], w["head_dim"], w["context"], 64, 4
        ck, sk = quant.latent_quant(torch.randn(L, hs, R, generator=gen).half())
        cv, sv = quant.latent_quant(torch.randn(L, hs, R, generator=gen).half())
        wk, wks = quant.wuk_quant((torch.randn(R, hs * D, generator=gen) / math.sqrt(R)).half())
        q = torch.randn(1, hs, D, generator=gen).half()
        r2t = torch.arange(L, dtype=torch.int32)[None]
        one = torch.tensor([0], dtype=torch.int32)
        fn = lambda: oattn.decode_rope_recon(q, ck, sk, cv, sv, wk, wks, r2t, one, torch.tensor([L], dtype=torch.int32))
        per_call = hs / H                      # requests' worth of work per call
        sample = f"1 request, {hs} of {H} heads, context {L}" + (" (attention only, projections left out)" if w["aux"] == "block" else "")
    elif w["aux"] == "append":
        H, T = w["heads"], 4096
        kr, vr = synth.ragged_ranks(H, 64, seed=0), synth.ragged_ranks(H, 64, seed=1)
        offs = lambda r: [sum(r[:i]) for i in range(len(r) + 1)]
        ko, vo = offs(kr), offs(vr)
        zk, zv = torch.randn(T, ko[-1], generator=gen).half(), torch.randn(T, vo[-1], generator=gen).half()
        dest = torch.randperm(T, generator=gen).to(torch.int32)
        ck, cv = torch.zeros(T, ko[-1], dtype=torch.int8), torch.zeros(T, vo[-1], dtype=torch.int8)
        sk, sv = torch.zeros(T, H, dtype=torch.float16), torch.zeros(T, H, dtype=torch.float16)

        def fn():
            oattn.cache_append(zk, dest, ko, ck, sk)
            oattn.cache_append(zv, dest, vo, cv, sv)
        per_call = T
        sample = f"{T} of {w['batch'] * w['context']} tokens"
    elif w["aux"] in ("tp", "stack_tp", "stack_e2e"):
        # the attention of the layer (its dominant part) for one request and a few heads; the projections and the FFN,
        # a few per cent of the CPU time at this context length, are left out
        H, D, L, R, hs = w["heads"], w["head_dim"], w["context"] + 1, 64, 4
        ck, sk = quant.latent_quant(torch.randn(L, hs, R, generator=gen).half())
        cv, sv = quant.latent_quant(torch.randn(L, hs, R, generator=gen).half())
        upk = (torch.randn(hs * R, D, generator=gen) / 8).half()
        q = torch.randn(1, hs, D, generator=gen).half()
        offs = [i * R for i in range(hs + 1)]
        r2t = torch.arange(L, dtype=torch.int32)[None]
        one = torch.tensor([0], dtype=torch.int32)
        fn = lambda: oattn.decode_absorb(q, ck.view(L, -1), sk, cv.view(L, -1), sv, upk, upk, offs, offs, r2t, one,
                                         torch.tensor([L], dtype=torch.int32), dtype=torch.float32)
        per_call = hs / H / w.get("layers", 1)
        sample = (f"attention only: 1 of {w['batch']} requests, {hs} of {H} heads, context {L}, one layer"
                  + (f" (scaled by the {w['layers']} layers of the stack; decode steps only)" if w.get("layers") else ""))
    elif w["aux"] == "mixffn":
        from oracle import mixffn as omix
        hid, dff, M = w["hidden"], w["d_ffn"], w["batch"]
        mk = lambda o, i: (torch.randn(o, i, generator=gen) / i ** 0.5).half()
        mw = omix.convert_swiglu(mk(dff, hid), mk(dff, hid), mk(hid, dff), torch.randn(hid, generator=gen).half(), 0.5, 0.5, 64, gen)
        x = torch.randn(M, hid, generator=gen).half()
        fn = lambda: omix.forward_stages(x, mw, 1e-6)
        per_call = M
        sample = f"all {M} tokens of a step"
    else:
        fw = synth.ffn_weights(FFN_SHAPE["d_in"], FFN_SHAPE["d_ffn"], FFN_SHAPE["rank"], FFN_SHAPE["n_svd"], seed=0,
                               had_K=synth.sign_matrix(FFN_SHAPE["K"]).float(), K=FFN_SHAPE["K"])
        x = torch.randn(64, FFN_SHAPE["d_in"], generator=gen).half()
        fn = lambda: offn.hybrid_ffn_stages(x, fw)
        per_call = 64
        sample = f"64 of {w['batch'] * w['context']} tokens"
    fn()
    n, t0 = 0, time.perf_counter()
    while True:
        fn()
        n += 1
        dt = time.perf_counter() - t0
        if dt > seconds_hint or n >= 20:
            break
    return {"value": per_call * n / dt, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"{sample}, {n} calls of the oracle, torch on {threads} threads"}


def run_reference(args, rank, world):
    if rank != 0:
        return None
    w = WORKLOADS[args.workload]
    B = args.tokens if w.get("ffn_only") else w["batch"]
    if w.get("aux") in ("prefill_ffn", "append"):
        B = w["batch"] * w["context"]
    B_cfg = args.tokens if w.get("ffn_only") else w["batch"]            # what the other arm prints as its batch
    cb = cpu_baseline(args.workload, args.tokens, seconds_hint=max(5.0, 3.0 * args.steps))
    return {"impl": "reference", "metric": "prefill_tokens_per_s" if w.get("aux") in ("prefill_ffn", "append") else "decode_tokens_per_s", "value": cb["value"], "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * B / cb["value"],
            "higher_is_better": True, "scaling": "strong" if w.get("aux") == "tp" else "weak", "vs_baseline": None,
            "dtype": "fp32/fp64 (CPU)", "data": "synthetic",
            "config": bench_config(args, w, B_cfg, world), "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="default: c3_layer on one GPU, c4_layer_tp (the tensor-parallel layer) on several")
    ap.add_argument("--layers", type=int, default=0, help="stack workloads: run this many layers instead of the configuration's")
    ap.add_argument("--replicas", action="store_true",
                    help="with several GPUs: N independent copies of the 1-GPU workload instead of the tensor-parallel layer")
    ap.add_argument("--tokens", type=int, default=8, help="tokens per step of the c2_ffn workload (1..64)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cache-layout", default="head", choices=["head", "slot"],
                    help="latent cache stored head by head ([H][slots][r_h] with scales [H][slots]: the layout of the library's "
                         "own layer and stack, whose streaming kernel then reads a step's 32 token scales as one 64-byte run) or "
                         "slot by slot ([slots][sum r], the reference's tensors, which the drop-in functions take)")
    ap.add_argument("--emulate-world", type=int, default=0,
                    help="c4_layer_tp on one GPU: run rank 0's shard of an N-way split without the collectives (for profilers, "
                         "which take one process); the line is marked `emulated`")
    ap.add_argument("--shared-kv", action="store_true",
                    help="attention / layer workloads: one cached latent per head serving as K and V latent (half the cache)")
    args = ap.parse_args()
    rank, world, local = dist_env()
    if args.workload is None:
        args.workload = "c3_layer" if (world == 1 or args.replicas) else "c4_layer_tp"
    if args.impl == "reference":
        line = run_reference(args, rank, world)
        if line is not None:
            print(json.dumps(line))
        return
    aux = WORKLOADS[args.workload].get("aux")
    if aux == "tp":
        line = run_tp(args, rank, world, local)
        if line is not None:
            print(json.dumps(line))
        return
    if aux in ("stack_tp", "stack_e2e"):
        line = run_stack(args, rank, world, local)
        if line is not None:
            if world == 1 and not args.no_cpu_baseline:
                line["cpu_baseline"] = cpu_baseline(args.workload, args.tokens)
            print(json.dumps(line))
        return
    line = run_aux(args, rank, world, local) if aux else run_ours(args, rank, world, local)
    if line is not None:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args.workload, args.tokens)
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
