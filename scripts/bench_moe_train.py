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
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.trainer.lm_loss import deepseek_v3_loss_fn, deepseek_v3_unstack, qwen35_loss_fn, qwen35_unstack
    from jax_gpt_b200.trainer.tree_engine import TreeTrainEngine
    from jax_gpt_b200.utils.profiling import max_over_ranks
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="qwen35", choices=["qwen35", "deepseek_v3"])
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=1, help="sequences per rank")
    ap.add_argument("--vocab", type=int, default=0, help="override the vocabulary size (0 = the family's)")
    ap.add_argument("--moe-buffer-sets", type=int, default=4,
                    help="buffer sets of the fused expert kernels used in rotation (as many as MoE layers: no "
                         "forward launch is repeated in the backward pass)")
    ap.add_argument("--fp8", action="store_true", help="dense projections in block-scaled FP8 (forward, dgrad, wgrad)")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    args = ap.parse_args(argv)
    rank, world, device = init_distributed()
    if args.model == "qwen35":
        from jax_gpt_b200.models.qwen35.config import Qwen35Config
        from jax_gpt_b200.models.qwen35.model import init_params
        cfg = Qwen35Config.ns().replace(n_layers=args.layers, n_routed_experts=args.experts,
                                        max_position_embeddings=args.seq)
        make_loss, unstack = qwen35_loss_fn, qwen35_unstack
    else:
        from jax_gpt_b200.models.deepseek_v3.config import DeepSeekV3Config
        from jax_gpt_b200.models.deepseek_v3.model import init_params
        cfg = DeepSeekV3Config.full().replace(n_layers=args.layers, first_k_dense=1, n_routed_experts=args.experts,
                                              max_position_embeddings=args.seq)
        make_loss, unstack = deepseek_v3_loss_fn, deepseek_v3_unstack
    if args.vocab:
        cfg = cfg.replace(vocab_size=args.vocab)
    params = init_params(cfg, 0, torch.bfloat16)
    ep = dist_opt = local = None
    n_moe = cfg.n_layers if args.model == "qwen35" else cfg.n_layers - cfg.first_k_dense
    n_sets = max(1, min(args.moe_buffer_sets, n_moe))
    if world == 1 and device.type == "cuda" and cfg.n_routed_experts <= 512:
        # one GPU: the same fused expert kernels with all experts local (one launch per MoE layer and direction)
        import os
        from jax_gpt_b200.comm.symm import Communicator
        from jax_gpt_b200.parallel.expert_parallel import EPMoERuntime, FusedEPMoE, is_expert_leaf
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29535")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
        comm = Communicator(device=device)
        layers = [FusedEPMoE(comm, args.batch * args.seq, cfg.d_model, cfg.moe_intermediate_size, cfg.n_routed_experts,
                             cfg.n_experts_per_token, training=True) for _ in range(n_sets)]
        ep, local = EPMoERuntime(layers), is_expert_leaf
    if world > 1:
        from jax_gpt_b200.parallel.expert_parallel import EPMoERuntime, FusedEPMoE, is_expert_leaf, shard_experts
        from jax_gpt_b200.parallel.fsdp import FusedShardedAdamW
        dist_opt = FusedShardedAdamW(device=device)
        layers = [FusedEPMoE(dist_opt.comm, args.batch * args.seq, cfg.d_model, cfg.moe_intermediate_size,
                             cfg.n_routed_experts, cfg.n_experts_per_token, training=True) for _ in range(n_sets)]
        ep, local = EPMoERuntime(layers), is_expert_leaf
        params = shard_experts(params, rank, world)
    eng = TreeTrainEngine(params, make_loss(cfg, ep, fp8=args.fp8), device=device, local=local, lr=1e-4, min_lr=1e-4, warmup_steps=0,
                          dist_optimizer=dist_opt, unstack=unstack)
    del params
    g = torch.Generator().manual_seed(1 + rank)
    tok = torch.randint(0, cfg.vocab_size, (args.batch, args.seq + 1), generator=g).to(device)
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    for _ in range(args.warmup):
        out = eng.train_step(x, y)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a.record()
    for _ in range(args.steps):
        out = eng.train_step(x, y)
    b.record()
    torch.cuda.synchronize()
    _ext.check_status(device)
    ms = max_over_ranks(a.elapsed_time(b) / args.steps, device) if world > 1 else a.elapsed_time(b) / args.steps
    res = {"model": args.model, "layers": args.layers, "experts": args.experts, "seq_len": args.seq,
           "global_batch": args.batch * world, "n_gpus": world, "params_this_rank_M": eng.n_params() / 1e6,
           "ms_per_step": ms, "tokens_per_s": args.batch * args.seq * world / (ms / 1e3), "loss": float(out["loss"]),
           "dtype": "bf16 + fp8 dense GEMMs" if args.fp8 else "bf16", "expert_parallel": ep is not None, "peak_mem_GB": torch.cuda.max_memory_allocated() / 2 ** 30}
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
