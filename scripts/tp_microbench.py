"""Fused tensor-parallel / FSDP GEMM kernels against their NCCL + GEMM baselines, with roofline fractions.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 scripts/tp_microbench.py --rows 4096 --K 7168 --N 16384
    python scripts/tp_microbench.py --rows 2048 --K 2048 --N 4096        # one rank: same kernels, for profiling

Three fused paths, each timed with CUDA events (max over ranks) next to the same math done with a library
collective followed (or preceded) by the plain GEMM:

* all-gather -> GEMM   ``concat_ranks(x_local) @ W``   (column-parallel projection under sequence parallelism):
  ``x_local`` has ``--rows`` rows per rank, ``W`` is (K, N / world);
* GEMM -> reduce-scatter   rows of ``sum_ranks(x @ W_r)``   (row-parallel projection): ``x`` is (rows * world, K / world);
* sharded-weight GEMM   ``x @ W`` with W column-sharded over the ranks (FSDP parameter all-gather fused into the GEMM).

Roofline per path: the slower of (FLOPs of this rank / measured bf16 GEMM rate) and (bytes this rank must move
over NVLink / link bandwidth per direction); the JSON line reports time, the two bounds and achieved / bound.
"""
from __future__ import annotations

import argparse
import json
import os

from utils import init_distributed

import torch
import torch.distributed as dist


def timed(fn, warmup, iters, device, world):
    for _ in range(warmup):
        fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main(argv=None):
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.parallel.fsdp import ShardedWeight
    from jax_gpt_b200.parallel.tensor_parallel import (TPContext, all_gather_matmul_nccl, matmul_reduce_scatter_nccl)
    from jax_gpt_b200.utils import roofline as R
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", type=int, default=4096, help="token rows per rank")
    ap.add_argument("--K", type=int, default=7168)
    ap.add_argument("--N", type=int, default=16384, help="full output width (all-gather -> GEMM computes N / world per rank)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--link-gbs", type=float, default=770.0, help="NVLink bandwidth per direction per GPU for the bound")
    args = ap.parse_args(argv)
    rank, world, device = init_distributed()
    if world == 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29541")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
    peaks = R.load_peaks()
    peak = peaks["bf16_tflops"] * 1e12
    link = args.link_gbs * 1e9
    rows, K, N = args.rows, args.K, args.N
    assert K % (world * 64) == 0 and N % (world * 128) == 0 and rows % 128 == 0
    ctx = TPContext(device=device)
    g = torch.Generator(device=device).manual_seed(1 + rank)
    res = {"world": world, "rows_per_rank": rows, "K": K, "N": N, "denominators": peaks["source"], "link_gbs": args.link_gbs}

    def report(name, ms, ms_base, flops, nvlink_bytes):
        t_c, t_l = flops / peak * 1e3, nvlink_bytes / link * 1e3
        bound = max(t_c, t_l)
        res[name] = {"fused_ms": ms, "nccl_plus_gemm_ms": ms_base, "speedup": ms_base / ms, "compute_bound_ms": t_c,
                     "nvlink_bound_ms": t_l, "roofline_fraction": bound / ms, "tflops": flops / ms / 1e9}

    # all-gather -> GEMM
    x_local = torch.randn(rows, K, device=device, generator=g).to(torch.bfloat16)
    w_col = (torch.randn(K, N // world, device=device, generator=g) * 0.02).to(torch.bfloat16)
    ms = timed(lambda: ctx.all_gather_matmul(x_local, w_col), args.warmup, args.iters, device, world)
    mb = timed(lambda: all_gather_matmul_nccl(x_local, w_col), args.warmup, args.iters, device, world)
    report("all_gather_gemm", ms, mb, 2.0 * rows * world * K * (N // world), 2.0 * rows * (world - 1) * K)
    # GEMM -> reduce-scatter
    x_full = torch.randn(rows * world, K // world, device=device, generator=g).to(torch.bfloat16)
    w_row = (torch.randn(K // world, N, device=device, generator=g) * 0.02).to(torch.bfloat16)
    ms = timed(lambda: ctx.matmul_reduce_scatter(x_full, w_row), args.warmup, args.iters, device, world)
    mb = timed(lambda: matmul_reduce_scatter_nccl(x_full, w_row), args.warmup, args.iters, device, world)
    report("gemm_reduce_scatter", ms, mb, 2.0 * rows * world * (K // world) * N, 2.0 * rows * (world - 1) * N)   # bf16 partials
    # sharded-weight GEMM (FSDP)
    wg = torch.Generator(device=device).manual_seed(7)
    w_full = (torch.randn(K, N, device=device, generator=wg) * 0.02).to(torch.bfloat16)
    sw = ShardedWeight(ctx.comm, w_full)
    from jax_gpt_b200.ops.gemm import gemm

    def base():
        parts = torch.empty(world, K, N // world, device=device, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(parts, sw.shard)
        out = torch.empty(rows, N, device=device, dtype=torch.bfloat16)
        for s_ in range(world):
            gemm(x_local, parts[s_], b_mn_major=True, out=out[:, s_ * (N // world):(s_ + 1) * (N // world)])
        return out
    ms = timed(lambda: sw.matmul(x_local), args.warmup, args.iters, device, world)
    mb = timed(base, args.warmup, args.iters, device, world)
    report("sharded_weight_gemm", ms, mb, 2.0 * rows * K * N, 2.0 * K * N * (world - 1) / world)
    torch.cuda.synchronize()
    _ext.check_status(device)
    if rank == 0:
        print(json.dumps(res))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
