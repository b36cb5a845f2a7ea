"""Expert-parallel MoE layer micro-benchmark (DeepSeek-V3 layer shape by default).

    torchrun --nproc-per-node N --master-addr 127.0.0.1 scripts/moe_microbench.py \
        --tokens 4096 --router normal|zipf [--d-model 7168 --inter 2048 --experts 256 --top-k 8]

Every rank owns ``--tokens`` bf16 activations ~N(0,1); router logits are N(0,1) or Zipf(s=1.2)
skewed over the experts; routing is the group-limited sigmoid top-k (8 groups, top-4 groups).
Times the fused one-kernel path (dispatch + grouped SwiGLU GEMMs + weighted combine over NVLink)
against the library baseline (NCCL all_to_all + per-expert GEMMs + all_to_all), with CUDA events,
max over ranks, and prints one JSON line with the roofline fraction
``max(FLOPs / measured GEMM rate, NVLink bytes / measured link rate) / time`` (``roofline_fraction``) and the same with
the HBM floor of the launch added (``hbm_floor_*_ms``, ``roofline_fraction_*_with_hbm``). With ``B200_MOE_PROFILE=1``
in the environment the line also carries the kernels' per-CTA phase timeline (``fwd_timeline_us``, ``bwd_timeline_us``:
dispatch, tile phase, time the load warp waited for dependencies and the MMA warp for operands / accumulators).
"""
from __future__ import annotations

import argparse
import json

from utils import init_distributed

import torch
import torch.distributed as dist


def main(argv=None):
    from jax_gpt_b200.utils.bench_extras import ep_moe_layer_bench
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
    res = ep_moe_layer_bench(device, rank, world, tokens=args.tokens, d_model=args.d_model, inter=args.inter,
                             experts=args.experts, top_k=args.top_k, n_group=args.n_group, topk_group=args.topk_group,
                             router=args.router, warmup=args.warmup, iters=args.iters, backward=args.backward,
                             fp8=args.fp8, baseline=not args.skip_baseline and world > 1, check=args.check)
    if rank == 0:
        print(json.dumps(res))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
