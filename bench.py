#!/usr/bin/env python
"""Benchmark of the LSVD decode hot path on B200: one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A "step" is one decode step of one decoder-layer's hot path over one batch of synthetic
requests: append this step's K/V latents to the int8 latent cache, then int8 latent
flash-decoding attention over the whole context.  The default workload is the attention
block of BASELINE config 3 (LLaVA-Next-7B layer shape, batch 16, context 4096, ragged
per-head ranks with mean 64); the metric is decode tokens/s for that layer step.

N > 1 (launched by torch.distributed.run): requests are independent, so each rank serves
its own batch of the same size with no data-path collective (weak scaling).

--impl reference times the CPU restatement of the reference's algorithm (the oracle, a
port: the reference has no CPU implementation of latent attention) on the host cores.
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
    # name: batch, heads, head_dim, context, ragged?
    "c3_attention": dict(batch=16, heads=32, head_dim=128, context=4096, ragged=True,
                         desc="BASELINE config 3 attention block: LLaVA-Next-7B layer shape, batch 16, "
                              "context 4096, ragged per-head K/V ranks (multiples of 16 in [16,128], mean 64)"),
    "c1_attention": dict(batch=1, heads=32, head_dim=128, context=2048, ragged=False,
                         desc="BASELINE config 1: batch 1, context 2048, uniform rank 64"),
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


def make_workload(w, device, seed):
    """Synthetic cache, weights and per-step inputs, resident on `device`; the cache is built by the library's
    own append kernel from fp16 N(0,1) latents (bit-identical to the reference's PyTorch quantiser)."""
    from lsvd_b200 import synth, cache_append, LatentCacheLayout, InferState
    B, H, D, L = w["batch"], w["heads"], w["head_dim"], w["context"]
    kr = synth.ragged_ranks(H, 64, seed=0) if w["ragged"] else [64] * H
    vr = synth.ragged_ranks(H, 64, seed=1) if w["ragged"] else [64] * H
    lay = LatentCacheLayout(kr, vr)
    seq = L + 1                      # context plus the slot of the decoding token, as the reference's benchmark
    n_slots = B * seq
    g = torch.Generator(device=device).manual_seed(seed)
    ck = torch.empty(n_slots, lay.sum_k, dtype=torch.int8, device=device)
    cv = torch.empty(n_slots, lay.sum_v, dtype=torch.int8, device=device)
    sk = torch.empty(n_slots, H, dtype=torch.float16, device=device)
    sv = torch.empty(n_slots, H, dtype=torch.float16, device=device)
    chunk = 8192
    for s0 in range(0, n_slots, chunk):
        n = min(chunk, n_slots - s0)
        lk = torch.randn(n, lay.sum_k, generator=g, device=device, dtype=torch.float32).half()
        lv = torch.randn(n, lay.sum_v, generator=g, device=device, dtype=torch.float32).half()
        dest = torch.arange(s0, s0 + n, dtype=torch.int32, device=device)
        cache_append(lay, lk, lv, dest, ck, sk, cv, sv)
    up_k = (torch.randn(lay.sum_k, D, generator=g, device=device) / 8).half()
    up_v = (torch.randn(lay.sum_v, D, generator=g, device=device) / 8).half()
    st = InferState(B, seq, [seq] * B, device=device)
    return dict(layout=lay, ck=ck, cv=cv, sk=sk, sv=sv, up_k=up_k, up_v=up_v, state=st, B=B, H=H, D=D, L=L, seq=seq,
                n_slots=n_slots)


def algorithmic_bytes(wl):
    """Bytes one launch of the streaming kernel must move: the int8 K and V latents of every cached token, their
    fp16 scales, the slot indices, the absorbed query limbs and the partial results."""
    lay, B, H = wl["layout"], wl["B"], wl["H"]
    tokens = B * wl["seq"]
    cache = tokens * (lay.sum_k + lay.sum_v)
    scales = tokens * H * 2 * 2
    slots = tokens * 4
    return cache + scales + slots


def run_ours(args, rank, world, local):
    from lsvd_b200 import _lib, cache_append, token_decode_attention_int8_latent_absorb
    from lsvd_b200.attention import attn_decode_workspace_bytes
    _lib.load()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    w = WORKLOADS[args.workload]
    wl = make_workload(w, dev, seed=1000 + rank)
    lay, st, B, H, D = wl["layout"], wl["state"], wl["B"], wl["H"], wl["D"]
    ws = torch.empty(attn_decode_workspace_bytes(B, lay, wl["seq"]), dtype=torch.uint8, device=dev)
    out = torch.empty(B, H, D, dtype=torch.float16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    # per-step inputs: this step's query and K/V latents.  Host copies live in pinned memory for the e2e leg.
    g = torch.Generator().manual_seed(7 + rank)
    n_in = 8
    host_q = [torch.randn(B, H, D, generator=g).half().pin_memory() for _ in range(n_in)]
    host_lk = [torch.randn(B, lay.sum_k, generator=g).half().pin_memory() for _ in range(n_in)]
    host_lv = [torch.randn(B, lay.sum_v, generator=g).half().pin_memory() for _ in range(n_in)]
    dev_q = [t.to(dev) for t in host_q]
    dev_lk = [t.to(dev) for t in host_lk]
    dev_lv = [t.to(dev) for t in host_lv]
    q_in = torch.empty_like(dev_q[0])
    lk_in = torch.empty_like(dev_lk[0])
    lv_in = torch.empty_like(dev_lv[0])
    host_out = torch.empty(B, H, D, dtype=torch.float16).pin_memory()

    def step(q, lk, lv, ev=None):
        cache_append(lay, lk, lv, st.mem_index, wl["ck"], wl["sk"], wl["cv"], wl["sv"])
        token_decode_attention_int8_latent_absorb(q, st, H, D, wl["ck"], wl["sk"], wl["cv"], wl["sv"], wl["up_k"],
                                                  wl["up_v"], layout=lay, out=out, workspace=ws, status_word=status,
                                                  timing_events=ev)

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(dev_q[i % n_in], dev_lk[i % n_in], dev_lv[i % n_in])
    torch.cuda.synchronize()

    # ---- device-resident leg (value) with the streaming kernel timed on its own by event pairs ----
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for a, b in kev:
        a.record()
        b.record()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        step(dev_q[i % n_in], dev_lk[i % n_in], dev_lv[i % n_in], kev[i])
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    kernel_ms = [a.elapsed_time(b) for a, b in kev]

    # ---- end-to-end leg: host inputs from pinned memory, result read back, every step ----
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    f0.record()
    for i in range(args.steps):
        q_in.copy_(host_q[i % n_in], non_blocking=True)
        lk_in.copy_(host_lk[i % n_in], non_blocking=True)
        lv_in.copy_(host_lv[i % n_in], non_blocking=True)
        step(q_in, lk_in, lv_in)
        host_out.copy_(out, non_blocking=True)
    f1.record()
    barrier()
    ms_e2e = f0.elapsed_time(f1)
    clocks = sampler.stop() if rank == 0 else None
    if status.item() != 0:
        raise RuntimeError(f"device status word = {status.item()}")

    t = torch.tensor([ms_total, ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e = t.tolist()
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
    abytes = algorithmic_bytes(wl)
    k_ms = statistics.mean(kernel_ms)
    achieved = abytes / (k_ms * 1e-3) / 1e9
    h2d = sum(t.numel() * t.element_size() for t in (host_q[0], host_lk[0], host_lv[0]))
    d2h = host_out.numel() * host_out.element_size()
    line = {
        "metric": "decode_tokens_per_s", "value": tokens / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 latents, fp32 softmax/accumulate, fp16 out",
        "data": "synthetic",
        "config": {"workload": args.workload, "what": w["desc"], "batch_per_gpu": B, "context": wl["L"],
                   "layers": 1, "step": "cache append (K+V) + int8 latent decode attention (absorb) + V up-projection",
                   "l2": "inputs larger than L2: the cache read by every step is %.0f MB" % (abytes / 1e6)},
        "e2e": {"value": tokens / (ms_e2e / args.steps * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": 4 * args.steps,
        "roofline": {"kernel": "latent_stream_kernel", "bound": "hbm", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "of": "measured" if "hbm_gbs" in peaks else "fallback",
                     "traffic": None, "algorithmic_bytes_per_launch": abytes, "kernel_us": k_ms * 1e3,
                     "frac_of_8TBs": achieved / 8000.0},
        "parts": {"latent_decode_us_per_step": k_ms * 1e3, "latent_decode_hbm_gbs": achieved,
                  "step_us": ms_step * 1e3},
        "clocks": clocks,
    }
    return line


def cpu_baseline(w, seconds_hint=15.0, threads=None):
    """The oracle (a CPU port of the reference's algorithm) timed on the host cores on a bounded sample:
    a slice of the batch of the same workload."""
    from oracle import attention as oattn, quant
    from lsvd_b200 import synth
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    B, H, D, L = w["batch"], w["heads"], w["head_dim"], w["context"]
    kr = synth.ragged_ranks(H, 64, seed=0) if w["ragged"] else [64] * H
    vr = synth.ragged_ranks(H, 64, seed=1) if w["ragged"] else [64] * H
    bs = min(B, 4)
    c = synth.attention_inputs(bs, H, D, kr, vr, [L + 1] * bs, seed=0)
    ko, vo = [0], [0]
    for a, b in zip(kr, vr):
        ko.append(ko[-1] + a)
        vo.append(vo[-1] + b)
    ck, sk = quant.latent_quant_ragged(c["latent_k"], ko)
    cv, sv = quant.latent_quant_ragged(c["latent_v"], vo)

    def once():
        return oattn.decode_absorb(c["q"], ck, sk, cv, sv, c["up_k"], c["up_v"], ko, vo, c["req_to_token"],
                                   c["b_req_idx"], c["b_seq_len"], dtype=torch.float32)
    once()
    n, t0 = 0, time.perf_counter()
    while True:
        once()
        n += 1
        dt = time.perf_counter() - t0
        if dt > seconds_hint or n >= 20:
            break
    return {"value": bs * n / dt, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"{bs} of {B} requests of the same workload, {n} steps, fp32 torch on {threads} threads "
                      f"(attention only; the cache is pre-quantised)"}


def run_reference(args, rank, world):
    if rank != 0:
        return None
    w = WORKLOADS[args.workload]
    cb = cpu_baseline(w, seconds_hint=max(5.0, 3.0 * args.steps))
    return {"impl": "reference", "metric": "decode_tokens_per_s", "value": cb["value"], "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * w["batch"] / cb["value"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32 (CPU)", "data": "synthetic",
            "config": {"workload": args.workload, "what": w["desc"]}, "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3_attention", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank, world, local = dist_env()
    if args.impl == "reference":
        line = run_reference(args, rank, world)
        if line is not None:
            print(json.dumps(line))
        return
    line = run_ours(args, rank, world, local)
    if line is not None:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(WORKLOADS[args.workload])
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
