"""Qwen3.5 benchmark with roofline and profiler hooks (scripts/qwen35_benchmark.py:78-491).

Prints, per module and for the whole model, FLOPs, bytes, arithmetic intensity and the bound
(compute / HBM) against the rates measured on the B200 pool, then times prefill and decode.
``--profile`` (or $PROFILE_DIR) writes a torch.profiler trace. Config fields can be overridden
(--n-layers, --n-experts, --chunk-size). ``--sharding A|B --devices N`` runs tensor parallel over N processes
(launch with torchrun --nproc-per-node N): every rank keeps its shard of the parameters and of the recurrent
caches and all ranks feed the same tokens (models/qwen35/sharding.py, parallel/tp_ops.py).
"""
from __future__ import annotations

import argparse
import json
import statistics
import time

from utils import init_distributed, qwen_config

import torch


def main(argv=None):
    from jax_gpt_b200.models.qwen35 import forward, init_cache, init_params
    from jax_gpt_b200.models.qwen35.sharding import (AXIS_RULES_A, AXIS_RULES_B, make_mesh, shard_cache, shard_params,
                                                     tree_map)
    from jax_gpt_b200.utils import roofline as R
    from jax_gpt_b200.utils.profiling import profiler_trace
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--config", default="mini")
    ap.add_argument("--sharding", default="none", choices=["none", "A", "B"])
    ap.add_argument("--devices", type=int, default=1)
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--decode-steps", type=int, default=16)
    ap.add_argument("--max-seq-len", type=int, default=0)
    ap.add_argument("--n-runs", type=int, default=3)
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--skip-prefill", action="store_true")
    ap.add_argument("--skip-decode", action="store_true")
    ap.add_argument("--dtype", default="bfloat16", choices=["float32", "bfloat16", "fp8"])
    ap.add_argument("--chunk-size", type=int, default=0)
    ap.add_argument("--n-layers", type=int, default=0)
    ap.add_argument("--n-experts", type=int, default=0)
    ap.add_argument("--roofline", action="store_true")
    args = ap.parse_args(argv)
    rank, world, device = init_distributed()
    cfg = qwen_config(args.config)
    over = {}
    if args.chunk_size:
        over["delta_chunk_size"] = args.chunk_size
    if args.n_layers:
        over["n_layers"] = args.n_layers
    if args.n_experts:
        over["n_routed_experts"] = args.n_experts
    cfg = cfg.replace(**over)
    B, T = args.batch_size, args.prompt_len
    if args.roofline and rank == 0:
        peaks = R.load_peaks()
        print(f"roofline denominators ({peaks['source']}): {peaks['bf16_tflops']:.0f} TFLOP/s bf16, {peaks['hbm_gbs']:.0f} GB/s HBM")
        for decode in (False, True):
            mods = R.qwen35_modules(cfg, B, 1 if decode else T, decode)
            print(f"--- {'decode step' if decode else 'prefill'} (B={B}, T={1 if decode else T}) per layer ---")
            for m in mods:
                b = m.bound(peaks)
                print(f"{b['name']:24s} {b['flops'] / 1e9:12.3f} GFLOP {b['hbm_bytes'] / 1e6:12.3f} MB  AI {b['intensity']:8.1f}  "
                      f"{b['bound']:8s} {b['seconds'] * 1e6:10.2f} us")
    dtype = torch.float32 if (args.dtype == "float32" or device.type == "cpu") else torch.bfloat16
    t0 = time.perf_counter()
    params = init_params(cfg, 0, dtype=dtype, fp8=args.dtype == "fp8")
    tp_group, mesh, rules = None, None, None
    if args.sharding != "none" and args.devices > 1:
        if world != args.devices:
            raise SystemExit(f"--devices {args.devices} needs {args.devices} processes: launch with torchrun "
                             f"--nproc-per-node {args.devices} (found {world})")
        rules = AXIS_RULES_A if args.sharding == "A" else AXIS_RULES_B
        mesh = make_mesh(args.devices)
        tp_group = mesh.group
        params = shard_params(params, mesh, cfg, rules, rank=rank)
    params = tree_map(lambda t: t.to(device), params)

    def new_cache():
        cache = init_cache(cfg, B, max_len, dtype=dtype, device=device)
        return shard_cache(cache, mesh, cfg, rules, rank=rank) if mesh is not None else cache
    if rank == 0:
        print(f"init + placement: {(time.perf_counter() - t0) * 1e3:.0f} ms")
    max_len = args.max_seq_len or (T + args.decode_steps)
    tok = torch.randint(0, cfg.vocab_size, (B, T), generator=torch.Generator().manual_seed(0)).to(device)
    sync = (lambda: torch.cuda.synchronize()) if device.type == "cuda" else (lambda: None)
    res = {}
    with torch.no_grad(), profiler_trace("profile_out" if args.profile else ""):
        if not args.skip_prefill:
            times = []
            for _ in range(args.n_runs + 1):
                cache = new_cache()
                sync(); t = time.perf_counter()
                logits, cache = forward(params, tok, cfg, cache=cache, tp_group=tp_group)
                sync(); times.append((time.perf_counter() - t) * 1e3)
            res["first_call_ms"] = times[0]
            res["prefill_ms"] = statistics.mean(times[1:])
            res["prefill_toks_per_sec"] = B * T / (res["prefill_ms"] / 1e3)
        if not args.skip_decode:
            cache = new_cache()
            logits, cache = forward(params, tok, cfg, cache=cache, tp_group=tp_group)
            nxt = logits[:, -1].argmax(-1)
            steps = []
            for _ in range(args.decode_steps):
                sync(); t = time.perf_counter()
                logits, cache = forward(params, nxt[:, None], cfg, cache=cache, is_decode=True, tp_group=tp_group)
                nxt = logits[:, -1].argmax(-1)
                sync(); steps.append((time.perf_counter() - t) * 1e3)
            res["decode_ms_p50"] = statistics.median(steps)
            res["decode_toks_per_sec"] = B / (statistics.mean(steps) / 1e3)
    if rank == 0:
        print(json.dumps(res, indent=1))
    return res


if __name__ == "__main__":
    main()
