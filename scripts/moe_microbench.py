"""Expert-parallel MoE layer micro-benchmark (DeepSeek-V3 layer shape by default).

    torchrun --nproc-per-node N --master-addr 127.0.0.1 scripts/moe_microbench.py \
        --tokens 4096 --router normal|zipf [--d-model 7168 --inter 2048 --experts 256 --top-k 8]

Every rank owns ``--tokens`` bf16 activations ~N(0,1); router logits are N(0,1) or Zipf(s=1.2)
skewed over the experts; routing is the group-limited sigmoid top-k (8 groups, top-4 groups).
Times the fused one-kernel path (dispatch + grouped SwiGLU GEMMs + weighted combine over NVLink)
against the library baseline (NCCL all_to_all + per-expert GEMMs + all_to_all), with CUDA events,
max over ranks, and prints one JSON line with the roofline fraction
``max(FLOPs / measured GEMM rate, NVLink bytes / measured link rate) / time``.
"""
from __future__ import annotations

import argparse
import json

from utils import init_distributed

import torch
import torch.distributed as dist


def make_logits(tokens, experts, mode, device, gen):
    logits = torch.randn(tokens, experts, device=device, generator=gen)
    if mode == "zipf":
        ranks = torch.arange(1, experts + 1, device=device, dtype=torch.float32)
        prior = torch.log(ranks.pow(-1.2) / ranks.pow(-1.2).sum())
        perm = torch.randperm(experts, device=device, generator=torch.Generator(device=device).manual_seed(7))
        logits = logits + prior[perm] - prior.mean()
    return logits


def timed(fn, warmup, iters, device):
    from jax_gpt_b200.utils.profiling import max_over_ranks
    for _ in range(warmup):
        fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return max_over_ranks(a.elapsed_time(b) / iters, device)


def main(argv=None):
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.comm.symm import Communicator
    from jax_gpt_b200.ops.router import deepseek_router_from_logits
    from jax_gpt_b200.parallel.expert_parallel import FusedEPMoE, NcclEPMoE
    from jax_gpt_b200.utils import roofline as R
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--d-model", type=int, default=7168)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--n-group", type=int, default=8)
    ap.add_argument("--topk-group", type=int, default=4)
    ap.add_argument("--router", default="normal", choices=["normal", "zipf"])
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--skip-baseline", action="store_true")
    ap.add_argument("--check", action="store_true", help="compare fused and baseline outputs")
    ap.add_argument("--backward", action="store_true", help="also time the fused backward kernel")
    ap.add_argument("--fp8", action="store_true", help="also time the FP8 (block-scaled tensor-core) fused forward")
    args = ap.parse_args(argv)
    rank, world, device = init_distributed()
    if world == 1:
        # one rank holding all experts: the same kernels with every "peer" being this GPU (the only form in
        # which the fused kernel can be profiled: a profiler is never wrapped around a multi-rank command)
        import os
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
        args.skip_baseline = True
    E, D, I, k, T = args.experts, args.d_model, args.inter, args.top_k, args.tokens
    el = E // world
    gen = torch.Generator(device=device).manual_seed(11 + rank)
    wgen = torch.Generator(device=device).manual_seed(5)
    local = {n: (torch.randn(el, a, b, device=device, generator=wgen) * 0.02).to(torch.bfloat16)
             for n, (a, b) in (("gate_proj", (D, I)), ("up_proj", (D, I)), ("down_proj", (I, D)))}
    x = torch.randn(T, D, device=device, generator=gen).to(torch.bfloat16)
    logits = make_logits(T, E, args.router, device, gen)
    w, idx = deepseek_router_from_logits(logits, torch.zeros(E, device=device), k, args.n_group, args.topk_group, 2.5)
    comm = Communicator(device=device, wait_seconds=20.0)
    fused = FusedEPMoE(comm, T, D, I, E, k, training=args.backward)
    ms_fused = timed(lambda: fused.forward(x, w, idx, local), args.warmup, args.iters, device)
    _ext.check_status(device)
    rows = fused.rows_out.sum().item()
    res = {"world": world, "tokens_per_rank": T, "router": args.router, "d_model": D, "inter": I, "experts": E,
           "top_k": k, "dtype": "bf16", "fused_fwd_ms": ms_fused, "rows_this_rank": rows}
    if args.backward:
        dout = torch.randn(T, D, device=device, generator=gen).to(torch.bfloat16)
        grads = {n: torch.zeros_like(t, dtype=torch.float32) for n, t in local.items()}
        fused.forward(x, w, idx, local)
        ms_bwd = timed(lambda: fused.backward(x, dout, w, idx, local, grads), args.warmup, args.iters, device)
        _ext.check_status(device)
        res["fused_bwd_ms"] = ms_bwd
        res["bwd_tflops_this_rank"] = 2.0 * rows * 6 * D * I / ms_bwd / 1e9
    if args.fp8:
        from jax_gpt_b200.parallel.expert_parallel import FusedEPMoEFp8, quantize_expert_weights_fp8
        qw = quantize_expert_weights_fp8(local)
        f8 = FusedEPMoEFp8(comm, T, D, I, E, k)
        ms8 = timed(lambda: f8.forward(x, w, idx, qw), args.warmup, args.iters, device)
        _ext.check_status(device)
        res["fused_fp8_fwd_ms"] = ms8
        res["fp8_tflops_this_rank"] = 2.0 * rows * 3 * D * I / ms8 / 1e9
        if args.check:
            a8 = f8.forward(x, w, idx, qw).float().clone()
            b16 = fused.forward(x, w, idx, local).float()
            res["fp8_vs_bf16_rel"] = ((a8 - b16).norm() / b16.norm()).item()
    if not args.skip_baseline:
        base = NcclEPMoE(dist.group.WORLD, E)
        res["nccl_fwd_ms"] = timed(lambda: base.forward(x, w, idx, local), 1, max(1, args.iters // 2), device)
        res["speedup"] = res["nccl_fwd_ms"] / ms_fused
        if args.check:
            a = fused.forward(x, w, idx, local).float()
            b = base.forward(x, w, idx, local).float()
            res["fused_vs_nccl_rel"] = ((a - b).norm() / b.norm()).item()
    # roofline of the busiest rank: FLOPs of the rows it received, NVLink bytes it sent / received
    t = torch.tensor([float(rows)], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    max_rows = t.item()
    flops = 2.0 * max_rows * 3 * D * I
    remote = (world - 1) / world
    nv_bytes = max(max_rows, T * k) * remote * (D * 2 + D * 4)   # bf16 row in, fp32 reduction out
    peaks = R.load_peaks()
    bound = max(flops / (peaks["bf16_tflops"] * 1e12), nv_bytes / (R.NVLINK_GBS_MEASURED * 1e9))
    res.update(max_rows_any_rank=max_rows, tflops_busiest_rank=flops / ms_fused / 1e9,
               roofline_ms=bound * 1e3, roofline_fraction=bound * 1e3 / ms_fused, denominators=peaks["source"],
               tokens_per_s=T * world / (ms_fused / 1e3))
    if rank == 0:
        print(json.dumps(res))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
