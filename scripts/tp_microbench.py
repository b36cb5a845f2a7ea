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


def main(argv=None):
    from jax_gpt_b200.utils.bench_extras import tp_fused_gemm_bench
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
    res = tp_fused_gemm_bench(device, rank, world, rows=args.rows, K=args.K, N=args.N, warmup=args.warmup, iters=args.iters,
                              link_gbs=args.link_gbs)
    if rank == 0:
        print(json.dumps(res))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
