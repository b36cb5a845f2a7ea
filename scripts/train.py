"""Training entry point: the loop the reference sketches but leaves as a stub
(scripts/train.py:1-17, phase2_plan.md:514-552).

    python scripts/train.py --preset gpt2 --synthetic --max_steps=50 --micro_batch_size=16 --seq_len=1024
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 scripts/train.py --preset gpt2 --synthetic ...
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 scripts/train.py --preset qwen35-mini --synthetic ...
    python scripts/train.py --preset deepseek-v3-tiny --synthetic --max_steps=20 --micro_batch_size=2 --seq_len=64

``--preset qwen35-<tiny|mini|mid|ns>`` / ``deepseek-v3-<tiny|train8>`` train the MoE families: experts
are sharded over the ranks (fused dispatch / grouped GEMM / combine kernels, forward and backward),
dense weights go through the fused sharded optimizer.

``--tp=N`` (GPT-2 presets, N = number of processes) trains tensor parallel on the shards of
``trainer/sharding.py`` through the autograd model (add ``--sequence_parallel=true`` on GPUs to shard the token
rows between the blocks and run the projections on the fused all-gather -> GEMM / GEMM -> reduce-scatter kernels);
``--pp=N`` trains in N pipeline stages (1F1B over
point-to-point sends, the ``--grad_accum_steps`` micro-batches fill the pipeline); with several ranks a watchdog over the rendezvous store turns a
rank that stops beating into a ``PeerFailure`` on the others before their next step. The MoE families checkpoint
periodically too (``--save_interval``, ``--resume_from=latest``): dense state gathered to rank 0, every rank writes
its experts, and a checkpoint restores at another expert-parallel degree (ckpt/tree_ckpt.py).

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


def moe_config(preset: str):
    """(family, config) of a ``qwen35-*`` / ``deepseek-v3-*`` preset."""
    if preset.startswith("qwen35-"):
        from utils import qwen_config
        return "qwen35", qwen_config(preset.split("-", 1)[1])
    from jax_gpt_b200.models.deepseek_v3.config import DeepSeekV3Config
    name = preset.split("-", 2)[2]
    return "deepseek_v3", {"tiny": DeepSeekV3Config.tiny, "train8": DeepSeekV3Config.eight_layer,
                           "full": DeepSeekV3Config.full}[name]()


def start_watchdog(rank, world):
    """Heartbeats over the job's rendezvous store (utils/watchdog.py); None for a single process."""
    if world <= 1 or not torch.distributed.is_initialized():
        return None
    from jax_gpt_b200.utils.watchdog import Watchdog
    try:
        store = torch.distributed.distributed_c10d._get_default_store()
    except Exception:
        return None
    return Watchdog(store, rank, world, interval=2.0, timeout=120.0, startup_grace=900.0).start()


def train_moe(args, tc, rank, world, device):
    """Loop for the function-style MoE models on ``TreeTrainEngine``."""
    import os

    from jax_gpt_b200.data.pipeline import DataPipeline
    from jax_gpt_b200.data.tokenize import write_synthetic
    from jax_gpt_b200.trainer import MetricsLogger
    from jax_gpt_b200.trainer.lm_loss import deepseek_v3_loss_fn, deepseek_v3_unstack, qwen35_loss_fn, qwen35_unstack
    from jax_gpt_b200.trainer.tree_engine import TreeTrainEngine
    family, cfg = moe_config(args.preset)
    if family == "qwen35":
        from jax_gpt_b200.models.qwen35.model import init_params
        make_loss, unstack = qwen35_loss_fn, qwen35_unstack
    else:
        from jax_gpt_b200.models.deepseek_v3.model import init_params
        make_loss, unstack = deepseek_v3_loss_fn, deepseek_v3_unstack
    if args.synthetic and rank == 0 and not os.path.exists(os.path.join(tc.local_data_path, "train.bin")):
        write_synthetic(tc.local_data_path, args.synthetic_tokens, cfg.vocab_size, tc.seed)
    if world > 1:
        torch.distributed.barrier()
    params = init_params(cfg, tc.seed, torch.float32)
    ep = dist_opt = local = None
    on_gpu = device.type == "cuda"
    fusable = cfg.d_model % 256 == 0 and cfg.moe_intermediate_size % 256 == 0 and cfg.n_routed_experts <= 512
    if world == 1 and on_gpu and fusable:
        # one GPU: the fused expert kernels with all experts local (one launch per MoE layer and direction)
        import torch.distributed as dist
        from jax_gpt_b200.comm.symm import Communicator
        from jax_gpt_b200.parallel.expert_parallel import EPMoERuntime, FusedEPMoE, is_expert_leaf
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29536")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
        layer = FusedEPMoE(Communicator(device=device), tc.micro_batch_size * tc.seq_len, cfg.d_model,
                           cfg.moe_intermediate_size, cfg.n_routed_experts, cfg.n_experts_per_token, training=True)
        ep, local = EPMoERuntime(layer), is_expert_leaf
    if world > 1 and on_gpu:
        from jax_gpt_b200.parallel.expert_parallel import EPMoERuntime, FusedEPMoE, is_expert_leaf, shard_experts
        from jax_gpt_b200.parallel.fsdp import FusedShardedAdamW, NcclShardedAdamW
        dist_opt = NcclShardedAdamW(device=device) if args.nccl_optimizer else FusedShardedAdamW(device=device)
        if not args.nccl_optimizer and cfg.d_model % 256 == 0 and cfg.moe_intermediate_size % 256 == 0:
            layer = FusedEPMoE(dist_opt.comm, tc.micro_batch_size * tc.seq_len, cfg.d_model, cfg.moe_intermediate_size,
                               cfg.n_routed_experts, cfg.n_experts_per_token, training=True)
            ep, local = EPMoERuntime(layer), is_expert_leaf
            params = shard_experts(params, rank, world)
    eng = TreeTrainEngine(params, make_loss(cfg, ep), device=device, local=local, unstack=unstack,
                          compute_dtype=torch.bfloat16 if on_gpu else torch.float32, lr=tc.learning_rate,
                          min_lr=tc.min_lr, warmup_steps=tc.warmup_steps, lr_decay_steps=tc.lr_decay_steps,
                          weight_decay=tc.weight_decay, beta1=tc.beta1, beta2=tc.beta2, grad_clip=tc.grad_clip,
                          dist_optimizer=dist_opt)
    del params
    from jax_gpt_b200.ckpt.tree_ckpt import TreeCheckpointer
    ckpt = None
    if tc.checkpoint_dir and tc.save_interval > 0:
        ckpt = TreeCheckpointer(os.path.join(tc.checkpoint_dir, args.preset), tc.max_checkpoints_to_keep, rank, world,
                                barrier=(torch.distributed.barrier if world > 1 else None))
        if tc.resume_from:
            man = ckpt.load(eng, None if tc.resume_from == "latest" else int(tc.resume_from))
            if man is not None and rank == 0:
                print(f"resumed at step {eng.step_count}")
    data = DataPipeline(tc, "train")
    data.skip_to_step(eng.step_count, tc.grad_accum_steps)
    wd = start_watchdog(rank, world)
    logger = MetricsLogger(tc, cfg, jsonl_path=args.jsonl if rank == 0 else "")
    tokens_per_step = tc.micro_batch_size * tc.seq_len * tc.grad_accum_steps * world
    if rank == 0:
        print(f"{args.preset}: {eng.n_params() / 1e6:.1f}M parameters on this rank, expert parallel: {ep is not None}")
    out, since = {}, 0
    while eng.step_count < tc.max_steps:
        if wd is not None:
            wd.check()          # a peer that stopped beating: PeerFailure here, before the next collective
        for _ in range(tc.grad_accum_steps):
            x, y = data.get_batch()
            eng.micro_step(x.to(device, non_blocking=True), y.to(device, non_blocking=True))
        out = eng.apply_gradients()
        since += tokens_per_step
        if eng.step_count % tc.log_interval == 0:
            logger.log(eng.step_count, {"loss": out["loss"], "grad_norm": out["grad_norm_sq"].sqrt() * out["grad_scale"],
                                        "lr": out["lr"]}, since)
            since = 0
        if ckpt is not None and eng.step_count % tc.save_interval == 0:
            ckpt.save(eng.step_count, eng, extra={"data_state": data.state()})      # collective: every rank
    if rank == 0 and out:
        print(f"done: step {eng.step_count} loss {float(out['loss']):.4f}")
    if ckpt is not None and eng.step_count % tc.save_interval != 0:
        ckpt.save(eng.step_count, eng, extra={"data_state": data.state()})
    if wd is not None:
        wd.stop()
    data.close()
    if torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()


def train_gpt2_tp(args, tc, cfg, rank, world, device):
    """GPT-2 tensor parallel over all processes (``--tp=N``): every rank holds its shard of the attention heads,
    the MLP and the vocabulary (trainer/sharding.py), feeds the SAME batch, and the autograd model runs the
    Megatron-style forward / backward of parallel/tp_ops.py. Replicated parameters see the full gradient on every
    rank, so each rank updates its own shard with the plain optimizer and no gradient exchange."""
    import os

    from jax_gpt_b200.data.pipeline import DataPipeline
    from jax_gpt_b200.data.tokenize import write_synthetic
    from jax_gpt_b200.models.gpt2 import GPT
    from jax_gpt_b200.trainer import MetricsLogger, create_optimizer, create_train_state, train_step_with_accumulation
    from jax_gpt_b200.trainer.sharding import make_mesh, shard_train_state
    if tc.tp != world:
        raise SystemExit(f"--tp={tc.tp} needs {tc.tp} processes (found {world}); combine with data parallelism by "
                         f"launching tp x dp processes is not wired into this loop")
    if args.synthetic and rank == 0 and not os.path.exists(os.path.join(tc.local_data_path, "train.bin")):
        write_synthetic(tc.local_data_path, args.synthetic_tokens, cfg.vocab_size, tc.seed)
    torch.distributed.barrier()
    mesh = make_mesh(tc)
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    model = GPT(cfg, seed=tc.seed, device=device, dtype=torch.float32)
    state = create_train_state(model, create_optimizer(model, tc))
    state = shard_train_state(state, mesh, cfg)
    state.mesh = mesh
    data = DataPipeline(tc, "train", _shard_index=0, _shard_count=1)       # the ranks of a TP group read the same windows
    logger = MetricsLogger(tc, cfg, jsonl_path=args.jsonl if rank == 0 else "")
    wd = start_watchdog(rank, world)
    metrics, since = {}, 0
    while state.step < tc.max_steps:
        if wd is not None:
            wd.check()
        micro = [tuple(t.to(device) for t in data.get_batch()) for _ in range(tc.grad_accum_steps)]
        state, metrics = train_step_with_accumulation(state, micro, mesh=mesh)
        since += tc.micro_batch_size * tc.seq_len * tc.grad_accum_steps
        if state.step % tc.log_interval == 0:
            logger.log(state.step, metrics, since)
            since = 0
    if rank == 0 and metrics:
        print(f"done: step {state.step} loss {float(metrics['loss']):.4f} (tensor parallel x{tc.tp}, {dtype})")
    if wd is not None:
        wd.stop()
    data.close()
    torch.distributed.destroy_process_group()


def train_gpt2_sp(args, tc, cfg, rank, world, device):
    """GPT-2 with ``--tp=N --sequence_parallel=true`` on GPUs: heads and MLP columns sharded, token rows sharded
    between the blocks, the four projections of every block on the fused all-gather -> GEMM and GEMM ->
    reduce-scatter kernels, forward and backward (parallel/sequence_parallel.py). bf16 compute copies, fp32 master
    weights and AdamW per shard; every rank feeds the same batch and works on its own rows of it."""
    import os

    import torch.distributed as dist

    from jax_gpt_b200.data.pipeline import DataPipeline
    from jax_gpt_b200.data.tokenize import write_synthetic
    from jax_gpt_b200.models.gpt2 import GPT
    from jax_gpt_b200.parallel.sequence_parallel import (SHARDED, gpt2_sequence_parallel_loss,
                                                         shard_gpt2_for_sequence_parallel, sync_replicated_grads)
    from jax_gpt_b200.parallel.tensor_parallel import TPContext
    from jax_gpt_b200.trainer import MetricsLogger, create_optimizer
    if device.type != "cuda" or tc.tp != world:
        raise SystemExit("--sequence_parallel needs GPUs and --tp equal to the number of processes")
    if args.synthetic and rank == 0 and not os.path.exists(os.path.join(tc.local_data_path, "train.bin")):
        write_synthetic(tc.local_data_path, args.synthetic_tokens, cfg.vocab_size, tc.seed)
    dist.barrier()
    full = GPT(cfg, seed=tc.seed, device=device, dtype=torch.float32)
    master = shard_gpt2_for_sequence_parallel(full.params, cfg, world, rank)       # fp32, this rank's shard
    del full
    shard_model = type("Shard", (), {"params": master, "config": cfg})()
    tx = create_optimizer(shard_model, tc)
    opt_state = tx.init(master)
    compute = {k: v.to(torch.bfloat16).requires_grad_(True) for k, v in master.items()}
    tp = TPContext(device=device)
    data = DataPipeline(tc, "train", _shard_index=0, _shard_count=1)            # the ranks read the same windows
    logger = MetricsLogger(tc, cfg, jsonl_path=args.jsonl if rank == 0 else "")
    wd = start_watchdog(rank, world)
    n_micro = tc.grad_accum_steps
    step, since, loss_v = 0, 0, float("nan")
    while step < tc.max_steps:
        if wd is not None:
            wd.check()
        tot = torch.zeros((), device=device)
        for _ in range(n_micro):
            x, y = [t.to(device) for t in data.get_batch()]
            part = gpt2_sequence_parallel_loss(compute, cfg, x, y, tp) / n_micro
            part.backward()
            tot += part.detach()
        sync_replicated_grads(compute)
        grads = {k: (v.grad.float() if v.grad is not None else torch.zeros_like(master[k])) for k, v in compute.items()}
        sq_sh = sum((g ** 2).sum() for k, g in grads.items() if k in SHARDED)
        dist.all_reduce(sq_sh)
        sq = sq_sh + sum((g ** 2).sum() for k, g in grads.items() if k not in SHARDED)
        gnorm, lr = tx.update(grads, opt_state, master, global_sq=sq)
        with torch.no_grad():
            for k, v in compute.items():
                v.copy_(master[k])
                v.grad = None
        dist.all_reduce(tot)
        loss_v = float(tot)
        step += 1
        since += tc.micro_batch_size * tc.seq_len * n_micro
        if step % tc.log_interval == 0:
            logger.log(step, {"loss": loss_v, "grad_norm": gnorm, "lr": lr}, since)
            since = 0
    if rank == 0:
        print(f"done: step {step} loss {loss_v:.4f} (tensor + sequence parallel x{tc.tp}, fused collective GEMMs)")
    if wd is not None:
        wd.stop()
    data.close()
    dist.destroy_process_group()


def train_gpt2_pp(args, tc, cfg, rank, world, device):
    """GPT-2 in ``--pp=N`` pipeline stages, one per process (parallel/pipeline.py): stage r runs its contiguous
    range of blocks, activations and their gradients travel over point-to-point sends in the 1F1B order, the
    ``grad_accum_steps`` micro-batches of a step are the pipeline's micro-batches. The first stage reads the
    tokens and the last the targets of the same data windows; the tied embedding's gradient is summed between
    them; the clipping norm is summed over the stages (the tied embedding counted once)."""
    import os

    import torch.distributed as dist

    from jax_gpt_b200.data.pipeline import DataPipeline
    from jax_gpt_b200.data.tokenize import write_synthetic
    from jax_gpt_b200.models.gpt2 import GPT
    from jax_gpt_b200.parallel.pipeline import gpt2_stage, sync_tied_embedding_grad
    from jax_gpt_b200.trainer import MetricsLogger, create_optimizer
    if tc.pp != world or world < 2:
        raise SystemExit(f"--pp={tc.pp} needs exactly {tc.pp} processes (found {world})")
    if cfg.n_layers < world:
        raise SystemExit(f"{cfg.n_layers} layers cannot fill {world} pipeline stages")
    if args.synthetic and rank == 0 and not os.path.exists(os.path.join(tc.local_data_path, "train.bin")):
        write_synthetic(tc.local_data_path, args.synthetic_tokens, cfg.vocab_size, tc.seed)
    dist.barrier()
    model = GPT(cfg, seed=tc.seed, device=device, dtype=torch.float32)
    model.requires_grad_(True)
    tx = create_optimizer(model, tc)
    opt_state = tx.init(model.params)
    stage = gpt2_stage(model, rank, world, tc.micro_batch_size, tc.seq_len, device=device)
    data = DataPipeline(tc, "train", _shard_index=0, _shard_count=1)       # every stage walks the same windows
    logger = MetricsLogger(tc, cfg, jsonl_path=args.jsonl if rank == 0 else "")
    wd = start_watchdog(rank, world)
    n_micro = tc.grad_accum_steps
    step, since, last_loss = 0, 0, float("nan")
    while step < tc.max_steps:
        if wd is not None:
            wd.check()
        micro = [data.get_batch() for _ in range(n_micro)]
        if rank == 0:
            inputs = [x.to(device) for x, _ in micro]
        elif rank == world - 1:
            inputs = [y.to(device) for _, y in micro]
        else:
            inputs = [None] * n_micro
        loss = stage.run(inputs)
        sync_tied_embedding_grad(model)
        grads = {k: (p.grad if p.grad is not None else torch.zeros_like(p)) for k, p in model.params.items()}
        sq = torch.zeros((), device=device)
        for k, g in grads.items():
            if k == "wte.embedding" and rank != 0:
                continue                        # summed over the stages above: count it on the first stage only
            sq = sq + (g.float() ** 2).sum()
        dist.all_reduce(sq)
        with torch.no_grad():
            gnorm, lr = tx.update(grads, opt_state, model.params, global_sq=sq)
        for p in model.params.values():
            p.grad = None
        lt = torch.tensor([float(loss) if loss is not None else 0.0], device=device)
        dist.broadcast(lt, src=world - 1)
        last_loss = float(lt)
        step += 1
        since += tc.micro_batch_size * tc.seq_len * n_micro
        if step % tc.log_interval == 0:
            logger.log(step, {"loss": last_loss, "grad_norm": gnorm, "lr": lr}, since)
            since = 0
    if rank == 0:
        print(f"done: step {step} loss {last_loss:.4f} (pipeline parallel x{tc.pp})")
    if wd is not None:
        wd.stop()
    data.close()
    dist.destroy_process_group()


def main(argv=None):
    from jax_gpt_b200.data.pipeline import DataPipeline
    from jax_gpt_b200.data.tokenize import write_synthetic
    from jax_gpt_b200.models.gpt2 import GPT
    from jax_gpt_b200.trainer import (MetricsLogger, TrainConfig, apply_overrides, create_optimizer, create_train_state,
                                      eval_step, train_step_with_accumulation)
    from jax_gpt_b200.trainer.checkpointing import CheckpointManager

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="gpt2", help="gpt2 | gpt2-medium | gpt2-large | gpt2-xl | gpt2-tiny | qwen35-<tiny|mini|mid|ns> | "
                    "deepseek-v3-<tiny|train8>")
    ap.add_argument("--synthetic", action="store_true", help="train on uniform-random token ids written to local_data_path")
    ap.add_argument("--synthetic_tokens", type=int, default=8_000_000)
    ap.add_argument("--nccl_optimizer", action="store_true", help="multi-GPU: NCCL reduce-scatter/all-gather baseline")
    ap.add_argument("--jsonl", default="", help="also append metrics to this JSONL file")
    args, rest = ap.parse_known_args(argv)
    tc, rest = apply_overrides(TrainConfig(), rest)
    if rest:
        ap.error(f"unknown arguments: {rest}")

    rank, world, device = init_distributed()
    if args.preset.startswith(("qwen35-", "deepseek-v3-")):
        return train_moe(args, tc.replace(dp=world), rank, world, device)
    cfg = gpt_config(args.preset)
    if tc.tp > 1 and tc.sequence_parallel:
        return train_gpt2_sp(args, tc, cfg, rank, world, device)
    if tc.tp > 1:
        return train_gpt2_tp(args, tc, cfg, rank, world, device)
    if tc.pp > 1:
        return train_gpt2_pp(args, tc, cfg, rank, world, device)
    if tc.fsdp > 1 and tc.fsdp != world:
        raise SystemExit(f"--fsdp={tc.fsdp} must equal the number of processes ({world}): the data-parallel ranks ARE the "
                         f"shards (gradients reduce-scattered, fp32 master weights and moments kept as shards)")
    # several GPUs, no --tp / --pp: data parallel with sharded state (--fsdp=N spells it out): every rank keeps 1 / N of
    # the fp32 master weights and Adam moments, one fused kernel does reduce-scatter + AdamW + all-gather
    tc = tc.replace(dp=world if tc.fsdp == 1 else 1)
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
    wd = start_watchdog(rank, world)
    logger = MetricsLogger(tc, cfg, jsonl_path=args.jsonl if rank == 0 else "")
    tokens_per_step = tc.micro_batch_size * tc.seq_len * tc.grad_accum_steps * world
    metrics = {}
    tokens_since_log = 0
    while state.step < tc.max_steps:
        if wd is not None:
            wd.check()
        micro = [train_data.get_batch() for _ in range(tc.grad_accum_steps)]
        state, metrics = train_step_with_accumulation(state, micro)
        tokens_since_log += tokens_per_step
        if state.step % tc.log_interval == 0:
            logger.log(state.step, metrics, tokens_since_log)
            tokens_since_log = 0
        if tc.eval_interval > 0 and state.step % tc.eval_interval == 0:
            losses = [float(eval_step(model, val_data.get_batch(), engine=state.engine)) for _ in range(tc.eval_steps)]
            logger.log_val(state.step, sum(losses) / len(losses))
        if ckpt.should_save(state.step):
            # with the sharded optimizer, save() gathers master weights and moments collectively: every rank
            # calls it and rank 0 writes; the saved tree does not depend on the number of ranks
            if dist_opt is not None or rank == 0:
                ckpt.save(state.step, state, data_state=train_data.state())
    ckpt.wait_until_finished()
    if wd is not None:
        wd.stop()
    if rank == 0 and metrics:
        print(f"done: step {state.step} loss {float(metrics['loss']):.4f}")
    train_data.close()
    val_data.close()
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
