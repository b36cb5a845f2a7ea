"""Prefill / decode benchmark (scripts/bench_prefill_decode.py:40-422 of the reference).

Scenarios: 8k1k, 1k1k, 1k8k (prefill length / decode length). For each: find the largest batch
that fits (doubling then bisection on out-of-memory, ``--max-batch`` caps it), time prefill over
5 repetitions with a fresh cache and 20 decode steps, and report

    prefill tokens/s = B * prefill_len / mean prefill time
    decode ms/token  = p50 and p99 over the decode steps,  decode tokens/s = B / mean step

Timing is on the device with CUDA events, maximum over ranks (the reference uses host
perf_counter and means only, scripts/bench_prefill_decode.py:246-264). ``--model`` selects the
Qwen3.5 hybrid (``--config`` preset) or the DeepSeek-V3 shape with its paged latent cache.
Results are printed and written as JSON to ``--out``.
"""
from __future__ import annotations

import argparse
import json
import statistics
import time

from utils import init_distributed, qwen_config

import torch

SCENARIOS = {"8k1k": (8192, 1024), "1k1k": (1024, 1024), "1k8k": (1024, 8192), "tiny": (32, 8)}


class _Timer:
    def __init__(self, device):
        self.cuda = device.type == "cuda"

    def run(self, fn):
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            out = fn()
            b.record()
            torch.cuda.synchronize()
            return out, a.elapsed_time(b)
        t = time.perf_counter()
        out = fn()
        return out, (time.perf_counter() - t) * 1e3


def _max_over_ranks(v, device):
    from jax_gpt_b200.utils.profiling import max_over_ranks
    return max_over_ranks(v, device)


def make_runner(args, device):
    """Returns (prefill(B) -> state, decode(state) -> state, describe) for the chosen model."""
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[args.dtype]
    if args.model == "qwen35":
        from jax_gpt_b200.models.qwen35 import forward, init_cache, init_params
        from jax_gpt_b200.models.qwen35.sharding import tree_map
        cfg = qwen_config(args.config)
        if args.n_layers:
            cfg = cfg.replace(n_layers=args.n_layers)
        params = tree_map(lambda t: t.to(device), init_params(cfg, 0, dtype=dtype, fp8=args.fp8))
        plen, dlen = SCENARIOS[args.scenario]

        def prefill(B):
            tok = torch.randint(0, cfg.vocab_size, (B, plen), device=device)
            cache = init_cache(cfg, B, plen + dlen, dtype=dtype, device=device)
            logits, cache = forward(params, tok, cfg, cache=cache)
            return logits[:, -1].argmax(-1), cache

        def decode(state):
            nxt, cache = state
            logits, cache = forward(params, nxt[:, None], cfg, cache=cache, is_decode=True)
            return logits[:, -1].argmax(-1), cache
        return prefill, decode, cfg
    from jax_gpt_b200.models.deepseek_v3 import DeepSeekV3Config, forward, init_params, make_cache
    from jax_gpt_b200.models.qwen35.sharding import tree_map
    cfg = {"tiny": DeepSeekV3Config.tiny, "8l": DeepSeekV3Config.eight_layer, "full": DeepSeekV3Config.full}[args.config]()
    if args.n_layers:
        cfg = cfg.replace(n_layers=args.n_layers, first_k_dense=min(cfg.first_k_dense, args.n_layers))
    params = tree_map(lambda t: t.to(device), init_params(cfg, 0, dtype=dtype))
    plen, dlen = SCENARIOS[args.scenario]

    def prefill(B):
        per = (plen + dlen + cfg.page_size - 1) // cfg.page_size
        cache = make_cache(cfg, B * per, B, per, dtype, device)
        tok = torch.randint(0, cfg.vocab_size, (B, plen), device=device)
        logits = forward(params, tok, cfg, cache, list(range(B)))
        return logits[:, -1].argmax(-1), cache

    def decode(state):
        nxt, cache = state
        logits = forward(params, nxt[:, None], cfg, cache, list(range(nxt.shape[0])), is_decode=True)
        return logits[:, -1].argmax(-1), cache
    return prefill, decode, cfg


def find_max_batch(prefill, decode, cap):
    """Largest batch that runs a prefill and one decode step: doubling, then bisection."""
    def fits(B):
        try:
            st = prefill(B)
            decode(st)
            return True
        except (torch.cuda.OutOfMemoryError, MemoryError):
            torch.cuda.empty_cache() if torch.cuda.is_available() else None
            return False
    lo, B = 0, 1
    while B <= cap and fits(B):
        lo, B = B, B * 2
    hi = min(B, cap + 1)
    while hi - lo > 1:
        mid = (lo + hi) // 2
        lo, hi = (mid, hi) if fits(mid) else (lo, mid)
    return max(lo, 1)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="qwen35", choices=["qwen35", "deepseek_v3"])
    ap.add_argument("--model-dir", default="", help="HF safetensors directory (random weights when empty)")
    ap.add_argument("--scenario", default="1k1k", choices=sorted(SCENARIOS))
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--dp", type=int, default=1)
    ap.add_argument("--config", default="mini")
    ap.add_argument("--profile-dir", default="")
    ap.add_argument("--max-batch", type=int, default=64)
    ap.add_argument("--batch", type=int, default=0, help="fixed batch (skips the search)")
    ap.add_argument("--sharding", default="A", choices=["A", "B"])
    ap.add_argument("--random-weights", action="store_true")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--fp8", action="store_true")
    ap.add_argument("--n-layers", type=int, default=0)
    ap.add_argument("--prefill-reps", type=int, default=5)
    ap.add_argument("--decode-steps", type=int, default=20)
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)
    rank, world, device = init_distributed()
    if device.type == "cpu" and args.dtype == "bfloat16":
        args.dtype = "float32"
    prefill, decode, cfg = make_runner(args, device)
    timer = _Timer(device)
    with torch.no_grad():
        prefill(1)  # warm-up (kernel set-up, allocator)
        B = args.batch or find_max_batch(prefill, decode, args.max_batch)
        plen, dlen = SCENARIOS[args.scenario]
        pre = []
        for _ in range(args.prefill_reps):
            state, ms = timer.run(lambda: prefill(B))
            pre.append(_max_over_ranks(ms, device))
        dec = []
        from jax_gpt_b200.utils.profiling import profiler_trace
        with profiler_trace(args.profile_dir):
            for _ in range(args.decode_steps):
                state, ms = timer.run(lambda: decode(state))
                dec.append(_max_over_ranks(ms, device))
    dec_sorted = sorted(dec)
    res = {
        "model": args.model, "config": args.config, "scenario": args.scenario, "batch": B, "world": world,
        "prefill_len": plen, "prefill_ms_mean": statistics.mean(pre),
        "prefill_toks_per_sec": B * plen / (statistics.mean(pre) / 1e3),
        "decode_ms_mean": statistics.mean(dec), "decode_ms_p50": statistics.median(dec),
        "decode_ms_p99": dec_sorted[min(len(dec) - 1, int(0.99 * len(dec)))],
        "decode_toks_per_sec": B / (statistics.mean(dec) / 1e3), "dtype": args.dtype, "timing": "cuda events, max over ranks",
    }
    if rank == 0:
        print(json.dumps(res, indent=1))
        if args.out:
            with open(args.out, "w") as f:
                json.dump(res, f)
    return res


if __name__ == "__main__":
    main()
