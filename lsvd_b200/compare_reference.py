"""Head-to-head with the reference's own GPU kernels, on the GPU this runs on.

    python -m lsvd_b200.compare_reference /path/to/LSVD [--batch 32] [--context 4096] [--max-configs 6] [--out cmp.json]

Needs a checkout of SAI-Lab-NYU/LSVD (it is not part of this repository).  The reference's Triton layer -- its
``Int8AttentionBlock`` (kernels/layer_bench/ffn_kernel/baseline_kernel.py:56-145) and the ``mixffn`` provider
(kernels/layer_bench/ffn_kernel/mix_ffn_kernel.py:2223-2246) -- and this library's drop-ins for the same two modules
(``lsvd_b200.Int8AttentionBlock.from_module``, ``MixedFFNGateUpDenseLatentFused.from_module``) are built from the SAME parameters, fed the SAME synthetic
cache and hidden states (the reference's generators, kernels/layer_bench/benchmark_triton_int8_layer.py:103-149), compared
value by value, and timed by the reference's own harness function ``bench_ms`` (CUDA-graph replay + ``triton.testing.do_bench``,
kernels/layer_bench/ffn_kernel/utils.py:687-712) in one process.  One JSON line is printed (and written to ``--out``).

``--max-configs N`` thins every Triton autotune space of the reference to N evenly spaced configurations (its full spaces
hold 45 to 324 per kernel and take hours to search); 0 keeps them whole.  Which configurations won is not recorded here.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import sys
import time

import torch


def _thin_autotune(max_configs: int) -> None:
    import triton
    original = triton.autotune

    def autotune(configs, key, **kw):
        if max_configs > 0 and len(configs) > max_configs:
            stride = len(configs) / max_configs
            configs = [configs[int(i * stride)] for i in range(max_configs)]
        return original(configs=configs, key=key, **kw)

    triton.autotune = autotune


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("reference", help="path to a checkout of SAI-Lab-NYU/LSVD")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--intermediate", type=int, default=14336)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--attention-rank-ratio", type=float, default=0.5)
    ap.add_argument("--ffn-rank-ratio", type=float, default=0.9)
    ap.add_argument("--ffn-svd-ratio", type=float, default=0.5)
    ap.add_argument("--repeat-ms", type=int, default=300, help="the harness's --repeat-time")
    ap.add_argument("--max-configs", type=int, default=6)
    ap.add_argument("--skip-reference-timing", action="store_true", help="values only (no autotune search of the timed shapes)")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    bench_dir = os.path.join(args.reference, "kernels", "layer_bench")
    if not os.path.isdir(bench_dir):
        sys.exit("no kernels/layer_bench under %s" % args.reference)
    sys.path.insert(0, bench_dir)
    _thin_autotune(args.max_configs)
    harness = importlib.import_module("benchmark_triton_int8_layer")
    utils = importlib.import_module("ffn_kernel.utils")
    mix = importlib.import_module("ffn_kernel.mix_ffn_kernel")
    base = importlib.import_module("ffn_kernel.baseline_kernel")
    import lsvd_b200
    from lsvd_b200.mixffn import MixedFFNGateUpDenseLatentFused

    dev = "cuda"
    gen = torch.Generator(device=dev).manual_seed(0)
    B, L = args.batch, args.context
    x = torch.randn(B, 1, args.hidden, device=dev, dtype=torch.float16, generator=gen)
    ck, sk, cv, sv, state = harness.make_latent_kv_cache(B, args.heads, L, args.head_dim, args.attention_rank_ratio, dev, gen)
    torch.manual_seed(0)
    ref_block = base.Int8AttentionBlock(args.hidden, args.heads, args.head_dim, args.attention_rank_ratio, dev, torch.float16).eval()
    _, ffn_module = mix.make_ffn_inputs(1, 1, args.hidden, args.intermediate, seed=0, dtype=torch.float16, device=dev,
                                        svd_ratio=args.ffn_svd_ratio, rank_ratio=args.ffn_rank_ratio, round_to=64)
    ffn_module = ffn_module.eval()
    our_block = lsvd_b200.Int8AttentionBlock.from_module(ref_block)
    ref_ffn = utils.FFN_NAME_MAP["mixffn"]

    def rel(a, b):
        return float((a.float() - b.float()).abs().max() / b.float().norm().clamp_min(1e-12))

    res = {"gpu": torch.cuda.get_device_name(0), "batch": B, "context": L, "hidden": args.hidden, "intermediate": args.intermediate,
           "heads": args.heads, "head_dim": args.head_dim, "attention_rank_ratio": args.attention_rank_ratio,
           "ffn_rank_ratio": args.ffn_rank_ratio, "ffn_svd_ratio": args.ffn_svd_ratio, "max_configs": args.max_configs,
           "timer": "the reference's bench_ms: CUDA-graph replay, triton.testing.do_bench, rep=%d ms, median" % args.repeat_ms}
    with torch.inference_mode():
        # ---- values: both blocks append to their own copy of the cache, then attend ----
        caches_ref = [t.clone() for t in (ck, sk, cv, sv)]
        caches_our = [t.clone() for t in (ck, sk, cv, sv)]
        t0 = time.time()
        a_ref = ref_block(x, *caches_ref, state)
        torch.cuda.synchronize()
        res["reference_first_call_s"] = time.time() - t0          # compile + autotune of the attention kernels
        a_our = our_block(x, *caches_our, state)
        slot = state.mem_index.long()
        res["attention_rel_err"] = rel(a_our, a_ref)
        res["appended_rows_equal"] = bool(all(torch.equal(r[slot], o[slot]) for r, o in zip(caches_ref, caches_our)))
        t0 = time.time()
        f_ref = ref_ffn(a_ref, ffn_module)
        torch.cuda.synchronize()
        res["reference_ffn_first_call_s"] = time.time() - t0
        # this library's module takes over the int8 weights the reference derived from the fp16 module (its own SVD and
        # quantisation), so both sides multiply the same integers
        ref_mixed = mix.get_mixed_gateup_v8_ffn(ffn_module)
        our_mixed = MixedFFNGateUpDenseLatentFused.from_module(ref_mixed)
        b200_mixffn = lambda t, _module=None: our_mixed(t)
        f_our = b200_mixffn(a_ref, ffn_module)
        res["ffn_rel_err"] = rel(f_our, f_ref)
        # stage by stage, each side on its own intermediates (integers: fraction of entries that differ and the largest
        # difference; floating point: max difference over the reference's norm)
        st_ref, st_our = ref_mixed.forward_stages(a_ref), our_mixed.forward_stages(a_ref)
        stages = {}
        for name, tr in st_ref.items():
            to = st_our.get(name)
            if not isinstance(tr, torch.Tensor) or not isinstance(to, torch.Tensor) or tr.numel() != to.numel():
                continue
            to = to.reshape(tr.shape)
            if tr.dtype in (torch.int8, torch.int32, torch.int16, torch.int64):
                d = (tr.long() - to.long()).abs()
                stages[name] = {"differ": float((d > 0).float().mean()), "max": int(d.max())}
            else:
                stages[name] = {"rel": rel(to, tr)}
        res["ffn_stages"] = stages
        res["tolerance"] = "max|ours - reference| / ||reference||_2 (2e-3 is the fp16 output bound)"
        # ---- time: the same callables the reference's harness times ----
        def timed(fn):
            p50, p20, p80 = utils.bench_ms(fn, repeat_time=args.repeat_ms, bench_mode="cuda_graph")
            return {"p50_us": p50 * 1e3, "p20_us": p20 * 1e3, "p80_us": p80 * 1e3}

        ours = {"attention": timed(lambda: our_block(x, *caches_our, state)),
                "ffn": timed(lambda: b200_mixffn(a_ref, ffn_module)),
                "layer": timed(lambda: b200_mixffn(our_block(x, *caches_our, state), ffn_module))}
        res["ours"] = ours
        if not args.skip_reference_timing:
            res["reference"] = {"attention": timed(lambda: ref_block(x, *caches_ref, state)),
                                "ffn": timed(lambda: ref_ffn(a_ref, ffn_module)),
                                "layer": timed(lambda: ref_ffn(ref_block(x, *caches_ref, state), ffn_module))}
            res["speedup"] = {k: res["reference"][k]["p50_us"] / ours[k]["p50_us"] for k in ours}
    line = json.dumps(res)
    print(line)
    if args.out:
        with open(args.out, "w") as f:
            f.write(line + "\n")


if __name__ == "__main__":
    main()
