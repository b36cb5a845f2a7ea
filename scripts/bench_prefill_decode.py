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

from utils import fake_quant_w8a8, init_distributed, load_hf_dir, make_tp_dp_groups, qwen_config

import torch

SCENARIOS = {"8k1k": (8192, 1024), "1k1k": (1024, 1024), "1k8k": (1024, 8192), "2k256": (2048, 256), "tiny": (32, 8)}


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
        if args.model_dir and not args.random_weights:
            from jax_gpt_b200.models.qwen35.weight_loader import load_from_hf_state_dict
            params = load_from_hf_state_dict(load_hf_dir(args.model_dir), cfg, dtype=dtype)
        else:
            params = init_params(cfg, 0, dtype=dtype, fp8=args.fp8)
        if args.w8a8:
            params = fake_quant_w8a8(params)
        ep = None
        tp_group, tp_rank, _ = make_tp_dp_groups(args.tp, args.dp)
        if args.tp > 1:
            # tensor parallel: this rank keeps its shard (rules A: heads, experts, vocabulary; B: experts, vocabulary)
            from jax_gpt_b200.models.qwen35.sharding import AXIS_RULES_A, AXIS_RULES_B, make_mesh, shard_cache, shard_params
            rules = AXIS_RULES_A if args.sharding == "A" else AXIS_RULES_B
            mesh = make_mesh(args.tp, group=tp_group)
            params = shard_params(params, mesh, cfg, rules, rank=tp_rank)
        elif device.type == "cuda" and not args.fp8 and cfg.d_model % 256 == 0 and cfg.moe_intermediate_size % 128 == 0 \
                and args.dp == 1:
            # routed experts through the fused dispatch / grouped-GEMM / combine kernel, expert-parallel over the
            # ranks (with one rank: one kernel per MoE layer instead of a launch per expert)
            import os
            import torch.distributed as dist
            from jax_gpt_b200.comm.symm import Communicator
            from jax_gpt_b200.parallel.expert_parallel import EPMoEInferenceRuntime, shard_experts
            if not dist.is_initialized():
                os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
                os.environ.setdefault("MASTER_PORT", "29534")
                dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
            if dist.get_world_size() > 1:
                params = shard_experts(params, dist.get_rank(), dist.get_world_size())
            ep = EPMoEInferenceRuntime(Communicator(device=device, wait_seconds=30.0), cfg.d_model,
                                       cfg.moe_intermediate_size, cfg.n_routed_experts, cfg.n_experts_per_token)
        params = tree_map(lambda t: t.to(device), params)
        plen, dlen = SCENARIOS[args.scenario]

        def prefill(B):
            gen = torch.Generator(device="cpu").manual_seed(1234 + (0 if args.tp > 1 else 0))
            tok = torch.randint(0, cfg.vocab_size, (B, plen), generator=gen).to(device)   # same tokens within a TP group
            cache = init_cache(cfg, B, plen + dlen, dtype=dtype, device=device)
            if args.tp > 1:
                cache = shard_cache(cache, mesh, cfg, rules, rank=tp_rank)
            logits, cache = forward(params, tok, cfg, cache=cache, ep_group=ep, tp_group=tp_group)
            return logits[:, -1].argmax(-1), cache

        engines = {}

        def decode(state):
            nxt, cache = state
            if args.engine:
                # in-place decode engine: device-side position, one CUDA-graph replay per token
                from jax_gpt_b200.models.qwen35.decode_engine import Qwen35DecodeEngine
                eng = engines.get(id(cache))
                if eng is None:
                    engines.clear()
                    eng = engines[id(cache)] = Qwen35DecodeEngine(params, cfg, cache, ep=ep,
                                                                  use_cuda_graph=not args.no_graph,
                                                                  paged_kv=args.paged_kv)
                return eng.step(nxt), cache
            logits, cache = forward(params, nxt[:, None], cfg, cache=cache, is_decode=True, ep_group=ep, tp_group=tp_group)
            return logits[:, -1].argmax(-1), cache
        return prefill, decode, cfg
    if args.tp > 1 or args.dp > 1 or args.model_dir or args.w8a8:
        raise SystemExit("--tp / --dp / --sharding / --model-dir / --w8a8 apply to --model qwen35; the DeepSeek-V3 shape "
                         "runs data-parallel attention with expert-parallel MoE over all ranks of the launch")
    from jax_gpt_b200.models.deepseek_v3 import DeepSeekV3Config, forward, init_params, make_cache
    from jax_gpt_b200.models.qwen35.sharding import tree_map
    cfg = {"tiny": DeepSeekV3Config.tiny, "8l": DeepSeekV3Config.eight_layer, "full": DeepSeekV3Config.full}[args.config]()
    if args.n_layers:
        cfg = cfg.replace(n_layers=args.n_layers, first_k_dense=min(cfg.first_k_dense, max(args.n_layers - 1, 0)))
    if args.experts:
        cfg = cfg.replace(n_routed_experts=args.experts)
    params = init_params(cfg, 0, dtype=dtype)
    ep = None
    import torch.distributed as dist
    world = dist.get_world_size() if dist.is_initialized() else 1
    if world > 1 and device.type == "cuda" and cfg.n_moe_layers > 0:
        # data-parallel attention (every rank serves its own sequences), expert-parallel MoE over all ranks
        from jax_gpt_b200.comm.symm import Communicator
        from jax_gpt_b200.parallel.expert_parallel import (EPMoEInferenceRuntime, quantize_stacked_experts_fp8,
                                                           shard_experts)
        params = shard_experts(params, dist.get_rank(), world)
        params = tree_map(lambda t: t.to(device), params)
        if args.fp8:
            params["moe_layers"]["moe"] = quantize_stacked_experts_fp8(params["moe_layers"]["moe"])
        ep = EPMoEInferenceRuntime(Communicator(device=device, wait_seconds=30.0), cfg.d_model, cfg.moe_intermediate_size,
                                   cfg.n_routed_experts, cfg.n_experts_per_token, fp8=args.fp8)
    else:
        params = tree_map(lambda t: t.to(device), params)
    plen, dlen = SCENARIOS[args.scenario]

    def prefill(B):
        per = (plen + dlen + cfg.page_size - 1) // cfg.page_size
        cache = make_cache(cfg, B * per, B, per, dtype, device)
        tok = torch.randint(0, cfg.vocab_size, (B, plen), device=device)
        logits = forward(params, tok, cfg, cache, list(range(B)), ep=ep)
        return logits[:, -1].argmax(-1), cache

    engines = {}

    def decode(state):
        nxt, cache = state
        B = nxt.shape[0]
        if args.engine and device.type == "cuda" and cfg.kv_lora_rank == 512 and cfg.qk_rope_head_dim == 64:
            # graph-captured token step (one replay per token); the engine is built once per cache
            from jax_gpt_b200.models.deepseek_v3.decode_engine import DeepSeekV3DecodeEngine
            eng = engines.get(id(cache))
            if eng is None:
                engines.clear()
                eng = engines[id(cache)] = DeepSeekV3DecodeEngine(params, cfg, cache, list(range(B)), ep=ep,
                                                                  use_cuda_graph=not args.no_graph, max_len=plen + dlen)
            return eng.step(nxt).clone(), cache
        logits = forward(params, nxt[:, None], cfg, cache, list(range(B)), is_decode=True, ep=ep)
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
    ap.add_argument("--random-weights", action="store_true", help="ignore --model-dir and use random weights")
    ap.add_argument("--w8a8", action="store_true", help="per-tensor fp8 fake quantisation of the weights (reference mode)")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--fp8", action="store_true")
    ap.add_argument("--n-layers", type=int, default=0)
    ap.add_argument("--experts", type=int, default=0, help="deepseek_v3: override the routed expert count")
    ap.add_argument("--engine", action="store_true", help="decode through the model family's CUDA-graph decode engine")
    ap.add_argument("--no-graph", action="store_true", help="with --engine: run the engine's step eagerly")
    ap.add_argument("--paged-kv", action="store_true",
                    help="qwen35 with --engine: gated-attention keys / values in a paged cache (64-token pages)")
    ap.add_argument("--prefill-reps", type=int, default=5)
    ap.add_argument("--decode-steps", type=int, default=256, help="timed decode steps (capped by the scenario)")
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)
    rank, world, device = init_distributed()
    if device.type == "cpu" and args.dtype == "bfloat16":
        args.dtype = "float32"
    if args.engine and args.tp > 1:
        raise SystemExit("--engine (the in-place decode engine) serves unsharded or expert-parallel parameters; use the "
                         "function-style decode with --tp")
    prefill, decode, cfg = make_runner(args, device)
    args.decode_steps = max(1, min(args.decode_steps, SCENARIOS[args.scenario][1] - 1))
    timer = _Timer(device)
    with torch.no_grad():
        prefill(1)  # warm-up (kernel set-up, allocator)
        B = args.batch or find_max_batch(prefill, decode, args.max_batch)
        plen, dlen = SCENARIOS[args.scenario]
        pre = []
        for _ in range(args.prefill_reps):
            state, ms = timer.run(lambda: prefill(B))
            pre.append(_max_over_ranks(ms, device))
        state = decode(state)   # untimed: first decode step (buffer set-up, graph capture)
        dec = []
        from jax_gpt_b200.utils.profiling import profiler_trace
        with profiler_trace(args.profile_dir):
            for _ in range(args.decode_steps):
                state, ms = timer.run(lambda: decode(state))
                dec.append(_max_over_ranks(ms, device))
    dec_sorted = sorted(dec)
    res = {
        "model": args.model, "config": args.config, "scenario": args.scenario, "batch_per_rank": B,
        "global_batch": B * world if args.model == "deepseek_v3" else B * args.dp, "world": world, "fp8_moe": bool(args.fp8),
        "prefill_len": plen, "prefill_ms_mean": statistics.mean(pre),
        "prefill_toks_per_sec": B * plen * (world if args.model == "deepseek_v3" else args.dp) / (statistics.mean(pre) / 1e3),
        "decode_ms_mean": statistics.mean(dec), "decode_ms_p50": statistics.median(dec),
        "decode_ms_p99": (dec_sorted[-(-99 * len(dec) // 100) - 1] if len(dec) >= 100 else None),
        "decode_ms_max": dec_sorted[-1], "decode_steps": len(dec), "tp": args.tp, "dp": args.dp,
        "sharding": args.sharding if args.tp > 1 else "none",
        "decode_toks_per_sec": B * (world if args.model == "deepseek_v3" else args.dp) / (statistics.mean(dec) / 1e3),
        "dtype": args.dtype, "timing": "cuda events, max over ranks",
    }
    if rank == 0:
        print(json.dumps(res, indent=1))
        if args.out:
            with open(args.out, "w") as f:
                json.dump(res, f)
    return res


if __name__ == "__main__":
    main()
