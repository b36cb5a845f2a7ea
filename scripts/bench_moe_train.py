"""Training-throughput benchmark of the MoE model families at a chosen (reduced) depth / expert count.

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 scripts/bench_moe_train.py --model qwen35 \
        --layers 8 --experts 64 --seq 4096 --batch 1 --steps 5 --warmup 2
    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 scripts/bench_moe_train.py --model deepseek_v3 \
        --layers 3 --experts 32 --seq 2048

The widths are the benchmark shapes (Qwen3.5: d_model 2048, 16/32 Gated-DeltaNet heads of 128, 16/2
attention heads of 256, experts of inter 512, top-10; DeepSeek-V3: d_model 7168, 128 MLA heads, experts of
inter 2048, top-8 group-limited); ``--layers`` / ``--experts`` shrink depth and expert count so that the
run fits the GPUs at hand. Experts are sharded over the ranks (fused dispatch / grouped GEMM / combine
kernels forward and backward), dense weights go through the fused sharded optimizer; uniform-random
token ids, random-init weights, bf16 compute with fp32 master weights. Prints one JSON line: tokens/s
over all ranks, CUDA-event time per step (max over ranks), loss of the last step.
"""
from __future__ import annotations

import argparse
import json

from utils import init_distributed

import torch
import torch.distributed as dist


def main(argv=None):
    from jax_gpt_b200.utils.bench_extras import moe_train_bench
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="qwen35", choices=["qwen35", "deepseek_v3"])
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=1, help="sequences per rank and micro-batch")
    ap.add_argument("--accum", type=int, default=1, help="micro-batches per optimizer step")
    ap.add_argument("--vocab", type=int, default=0, help="override the vocabulary size (0 = the family's)")
    ap.add_argument("--moe-buffer-sets", type=int, default=4,
                    help="buffer sets of the fused expert kernels used in rotation (as many as MoE layers: no "
                         "forward launch is repeated in the backward pass)")
    ap.add_argument("--fp8", action="store_true", help="dense projections in block-scaled FP8 (forward, dgrad, wgrad)")
    ap.add_argument("--lowmem", action="store_true",
                    help="expert weights without an fp32 master, bf16 moments (the full-size shapes need it)")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    args = ap.parse_args(argv)
    rank, world, device = init_distributed()
    if world == 1:
        import os
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29535")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
    res = moe_train_bench(device, rank, world, model=args.model, layers=args.layers, experts=args.experts, seq=args.seq,
                          batch=args.batch, accum=args.accum, vocab=args.vocab, buffer_sets=args.moe_buffer_sets,
                          fp8=args.fp8, lowmem=args.lowmem, steps=args.steps, warmup=args.warmup)
    if rank == 0:
        print(json.dumps(res))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
