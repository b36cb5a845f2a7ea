"""Training entry point: the loop the reference sketches but leaves as a stub
(scripts/train.py:1-17, phase2_plan.md:514-552).

    python scripts/train.py --preset gpt2 --synthetic --max_steps=50 --micro_batch_size=16 --seq_len=1024
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 scripts/train.py --preset gpt2 --synthetic ...

Every TrainConfig field is a ``--name=value`` flag. Flow: process group -> model -> optimizer and
state (fused engine on CUDA; sharded fused AdamW across ranks) -> resume from the latest
checkpoint -> data pipelines positioned at the restored step -> loop with gradient
accumulation, periodic evaluation, logging and asynchronous checkpoints.
"""
from __future__ import annotations

import argparse
import sys

from utils import get_tokenizer, gpt_config, init_distributed  # noqa: F401  (also fixes sys.path)

import torch


def main(argv=None):
    from jax_gpt_b200.data.pipeline import DataPipeline
    from jax_gpt_b200.data.tokenize import write_synthetic
    from jax_gpt_b200.models.gpt2 import GPT
    from jax_gpt_b200.trainer import (MetricsLogger, TrainConfig, apply_overrides, create_optimizer, create_train_state,
                                      eval_step, train_step_with_accumulation)
    from jax_gpt_b200.trainer.checkpointing import CheckpointManager

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="gpt2", help="gpt2 | gpt2-medium | gpt2-large | gpt2-xl | gpt2-tiny")
    ap.add_argument("--synthetic", action="store_true", help="train on uniform-random token ids written to local_data_path")
    ap.add_argument("--synthetic_tokens", type=int, default=8_000_000)
    ap.add_argument("--nccl_optimizer", action="store_true", help="multi-GPU: NCCL reduce-scatter/all-gather baseline")
    ap.add_argument("--jsonl", default="", help="also append metrics to this JSONL file")
    args, rest = ap.parse_known_args(argv)
    tc, rest = apply_overrides(TrainConfig(), rest)
    if rest:
        ap.error(f"unknown arguments: {rest}")

    rank, world, device = init_distributed()
    cfg = gpt_config(args.preset)
    tc = tc.replace(dp=world)
    if args.synthetic and rank == 0:
        import os
        if not os.path.exists(os.path.join(tc.local_data_path, "train.bin")):
            write_synthetic(tc.local_data_path, args.synthetic_tokens, cfg.vocab_size, tc.seed)
    if world > 1:
        torch.distributed.barrier()

    model = GPT(cfg, seed=tc.seed)
    tx = create_optimizer(model, tc)
    dist_opt = None
    if world > 1 and device.type == "cuda":
        from jax_gpt_b200.parallel.fsdp import FusedShardedAdamW, NcclShardedAdamW
        dist_opt = NcclShardedAdamW(device=device) if args.nccl_optimizer else FusedShardedAdamW(device=device)
    state = create_train_state(model, tx, train_config=tc, device=device, dist_optimizer=dist_opt)

    ckpt = CheckpointManager(tc, cfg)
    if tc.resume_from:
        step = None if tc.resume_from == "latest" else int(tc.resume_from)
        state = ckpt.restore(step, state)
        if rank == 0:
            print(f"resumed at step {state.step}")
    train_data = DataPipeline(tc, "train")
    val_data = DataPipeline(tc, "val")
    train_data.skip_to_step(state.step, tc.grad_accum_steps)
    logger = MetricsLogger(tc, cfg, jsonl_path=args.jsonl if rank == 0 else "")
    tokens_per_step = tc.micro_batch_size * tc.seq_len * tc.grad_accum_steps * world
    metrics = {}
    tokens_since_log = 0
    while state.step < tc.max_steps:
        micro = [train_data.get_batch() for _ in range(tc.grad_accum_steps)]
        state, metrics = train_step_with_accumulation(state, micro)
        tokens_since_log += tokens_per_step
        if state.step % tc.log_interval == 0:
            logger.log(state.step, metrics, tokens_since_log)
            tokens_since_log = 0
        if tc.eval_interval > 0 and state.step % tc.eval_interval == 0:
            losses = [float(eval_step(model, val_data.get_batch(), engine=state.engine)) for _ in range(tc.eval_steps)]
            logger.log_val(state.step, sum(losses) / len(losses))
        if ckpt.should_save(state.step) and rank == 0 and dist_opt is None:
            ckpt.save(state.step, state, data_state=train_data.state())
    ckpt.wait_until_finished()
    if rank == 0 and metrics:
        print(f"done: step {state.step} loss {float(metrics['loss']):.4f}")
    train_data.close()
    val_data.close()
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
