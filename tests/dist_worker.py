"""Worker run under torchrun by the multi-GPU tests (one process per GPU, NCCL)."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def small_cfg():
    from jax_gpt_b200.models.gpt2 import GPTConfig
    return GPTConfig(d_model=128, d_head=64, d_ff=512, d_context=256, n_head=2, n_kv_head=2, n_layers=2, vocab_size=1003)


def batch(rank, step, cfg, device):
    g = torch.Generator().manual_seed(1000 * step + rank)
    tok = torch.randint(0, cfg.vocab_size, (2, 257), generator=g, dtype=torch.int32)
    return tok[:, :-1].contiguous().to(device), tok[:, 1:].contiguous().to(device)


def run_fsdp(rank, world, device, use_multimem):
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.models.gpt2.engine import GPT2TrainEngine
    from jax_gpt_b200.parallel.fsdp import FusedShardedAdamW, NcclShardedAdamW
    cfg = small_cfg()
    kw = dict(lr=1e-3, warmup_steps=0, lr_decay_steps=1000, use_cuda_graph=False, seed=5)
    fused = GPT2TrainEngine(cfg, 2, 256, device=device,
                            dist_optimizer=FusedShardedAdamW(device=device, use_multimem=use_multimem, wait_seconds=5.0), **kw)
    nccl = GPT2TrainEngine(cfg, 2, 256, device=device, dist_optimizer=NcclShardedAdamW(device=device), **kw)
    # the same fused optimizer with every layer's gradient reduce-scatter launched during backward; once eager,
    # once through CUDA graphs (side-stream fork / join inside the capture)
    overlap = GPT2TrainEngine(cfg, 2, 256, device=device, overlap_grad_reduce=True,
                              dist_optimizer=FusedShardedAdamW(device=device, wait_seconds=5.0), **kw)
    kwg = dict(kw, use_cuda_graph=True)
    overlap_g = GPT2TrainEngine(cfg, 2, 256, device=device, overlap_grad_reduce=True,
                                dist_optimizer=FusedShardedAdamW(device=device, wait_seconds=5.0), **kwg)
    single = GPT2TrainEngine(cfg, 2, 256, device=device, **kw)
    res = {}
    for step in range(3):
        x, y = batch(rank, step, cfg, device)
        of = fused.train_step(x, y)
        on = nccl.train_step(x, y)
        overlap.train_step(x, y)
        overlap_g.train_step(x, y)
        for r in range(world):  # the single-GPU engine sees every rank's batch as a micro-batch
            xs, ys = batch(r, step, cfg, device)
            single.micro_step(xs, ys)
        single.apply_gradients()
        torch.cuda.synchronize()
        _ext.check_status(device)
        res[f"step{step}_fused_vs_nccl"] = rel(fused.flat.compute, nccl.flat.compute)
        res[f"step{step}_fused_vs_single"] = rel(fused.flat.compute, single.flat.compute)
        res[f"step{step}_overlap_fused_vs_nccl"] = rel(overlap.flat.compute, fused.flat.compute)
        res[f"step{step}_overlapgraph_fused_vs_nccl"] = rel(overlap_g.flat.compute, fused.flat.compute)
        res[f"step{step}_gnorm_rel"] = abs(float(of["grad_norm_sq"]) - float(on["grad_norm_sq"])) / float(on["grad_norm_sq"])
    # checkpoint state of the sharded optimizer: gathered trees match the single-GPU engine, and a fresh
    # sharded engine loaded from them continues identically
    p_tree = {k: v.clone() for k, v in fused.params().items()}
    st = fused.opt_state()
    st = {"count": st["count"], "mu": {k: v.clone() for k, v in st["mu"].items()}, "nu": {k: v.clone() for k, v in st["nu"].items()}}
    ss = single.opt_state()
    res["ckpt_mu_vs_single"] = max(rel(st["mu"][k], ss["mu"][k]) for k in list(ss["mu"])[:6])
    res["ckpt_nu_vs_single"] = max(rel(st["nu"][k], ss["nu"][k]) for k in list(ss["nu"])[:6])
    fused2 = GPT2TrainEngine(cfg, 2, 256, device=device,
                             dist_optimizer=FusedShardedAdamW(device=device, use_multimem=use_multimem, wait_seconds=5.0), **kw)
    fused2.load(p_tree, st, fused.step_count)
    x, y = batch(rank, 7, cfg, device)
    fused.train_step(x, y)
    fused2.train_step(x, y)
    torch.cuda.synchronize()
    _ext.check_status(device)
    res["ckpt_resume_fused_vs_nccl"] = rel(fused2.flat.compute, fused.flat.compute)
    # identical weights on every rank
    mine = fused.flat.compute.float().sum().reshape(1).clone()
    lst = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(lst, mine)
    res["rank_checksum_spread"] = float(max(lst).item() - min(lst).item())
    dist.barrier()
    return res


def run_ckpt_manager(rank, world, device, tmp_dir):
    """The trainer API with the fused sharded optimizer: a few steps, then CheckpointManager.save called on every
    rank; the file must hold the TRAINED weights and moments (equal to a single-GPU run over the same batches)."""
    from jax_gpt_b200.ckpt.manager import CheckpointManager
    from jax_gpt_b200.models.gpt2.engine import GPT2TrainEngine
    from jax_gpt_b200.models.gpt2.model import GPT
    from jax_gpt_b200.parallel.fsdp import FusedShardedAdamW
    from jax_gpt_b200.trainer.config import TrainConfig
    from jax_gpt_b200.trainer.optimizer import create_optimizer
    from jax_gpt_b200.trainer.train_state import create_train_state
    from jax_gpt_b200.trainer.train_step import train_step
    cfg = small_cfg()
    tc = TrainConfig(micro_batch_size=2, seq_len=256, learning_rate=1e-3, warmup_steps=0, lr_decay_steps=1000,
                     checkpoint_dir=tmp_dir, max_checkpoints_to_keep=2, save_interval=1, cuda_graph=False)
    model = GPT(cfg, rngs=5)
    state = create_train_state(model, create_optimizer(model, tc), train_config=tc, device=device,
                               dist_optimizer=FusedShardedAdamW(device=device, wait_seconds=5.0))
    single = GPT2TrainEngine(cfg, 2, 256, device=device, lr=1e-3, warmup_steps=0, lr_decay_steps=1000,
                             use_cuda_graph=False, init={k: v.detach().cpu() for k, v in GPT(cfg, rngs=5).params.items()})
    for step in range(3):
        state, _ = train_step(state, batch(rank, step, cfg, device))
        for r in range(world):
            xs, ys = batch(r, step, cfg, device)
            single.micro_step(xs, ys)
        single.apply_gradients()
    mgr = CheckpointManager(tc, cfg)
    mgr.save(3, state)                 # collective: every rank
    res = {}
    if rank == 0:
        mgr.wait_until_finished()
        from safetensors.torch import load_file
        flat = load_file(os.path.join(tmp_dir, "3", "params.safetensors"))
        opt = load_file(os.path.join(tmp_dir, "3", "opt_state.safetensors"))
        sp, so = single.params(), single.opt_state()
        keys = list(sp)[:8]
        res["ckpt_params_vs_single"] = max(rel(flat[k].to(device), sp[k]) for k in keys)
        res["ckpt_mu_vs_single"] = max(rel(opt["mu." + k].to(device), so["mu"][k]) for k in keys)
        init = GPT(cfg, rngs=5).params
        res["moved_from_init"] = min(rel(flat[k], init[k].float()) for k in keys if flat[k].dim() > 1)
    dist.barrier()
    return res


def run_pp(rank, world, device):
    """GPT-2 in pipeline stages over NCCL point-to-point (1F1B, four micro-batches): the loss and the gradients of
    every stage's layers against one process running the same micro-batches."""
    from jax_gpt_b200.models.gpt2 import GPT, GPTConfig
    from jax_gpt_b200.parallel.pipeline import gpt2_stage, split_layers
    cfg = GPTConfig(d_model=128, d_head=64, d_ff=512, d_context=128, n_head=2, n_kv_head=2, n_layers=4, vocab_size=512)
    B, T, n_micro = 2, 128, 4
    model = GPT(cfg, seed=9, device=device, dtype=torch.bfloat16)
    ref = GPT(cfg, seed=9, device=device, dtype=torch.bfloat16)
    for m in (model, ref):
        m.requires_grad_(True)
    g = torch.Generator().manual_seed(3)
    toks = [torch.randint(0, cfg.vocab_size, (B, T + 1), generator=g).to(device) for _ in range(n_micro)]
    stage = gpt2_stage(model, rank, world, B, T, device=device)
    inputs = [t[:, :-1] for t in toks] if rank == 0 else ([t[:, 1:] for t in toks] if rank == world - 1 else [None] * n_micro)
    loss = stage.run(inputs)
    torch.cuda.synchronize()
    tot = 0.0
    for t in toks:
        logits, _ = ref(t[:, :-1])
        l = torch.nn.functional.cross_entropy(logits.float().reshape(-1, cfg.vocab_size), t[:, 1:].reshape(-1)) / n_micro
        l.backward()
        tot += float(l)
    mine = split_layers(cfg.n_layers, world)[rank]
    worst = 0.0
    for k, v in model.params.items():
        if not k.startswith("h.") or v.grad is None:
            continue
        worst = max(worst, rel(v.grad[mine.start:mine.stop], ref.params[k].grad[mine.start:mine.stop]))
    res = {"stage_grad_rel": worst}
    t = torch.tensor([worst], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res["stage_grad_rel"] = float(t)
    lt = torch.tensor([float(loss) if loss is not None else 0.0], device=device)
    dist.all_reduce(lt, op=dist.ReduceOp.MAX)
    res["loss_abs_err"] = abs(float(lt) - tot)
    if rank == 0:
        e = model.params["wte.embedding"].grad
        res["first_stage_embed_grad"] = float(e.abs().sum()) if e is not None else 0.0
    return res


def run_tp(rank, world, device):
    """all-gather -> GEMM and GEMM -> reduce-scatter (copier CTAs / pushed partials inside the GEMM kernel) against
    their unfused definitions; several calls back to back with fresh data, so that the alternating staging buffers,
    the epochs of the ready flags and the cumulative arrival counters are all exercised."""
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.parallel.tensor_parallel import TPContext
    torch.manual_seed(7)
    ctx = TPContext(device=device, wait_seconds=5.0)
    res = {}
    for (rows, K, N) in [(256, 512, 384), (1024, 1024, 2048)]:
        w = (torch.randn(K, N, device=device, generator=torch.Generator(device=device).manual_seed(11)) * 0.05).to(torch.bfloat16)
        worst_ag = worst_rs = 0.0
        for call in range(4):
            g = torch.Generator(device=device).manual_seed(1000 * call + rank)
            x_local = (torch.randn(rows, K, device=device, generator=g) * (rank + 1)).to(torch.bfloat16)
            y = ctx.all_gather_matmul(x_local, w)
            parts = [torch.empty_like(x_local) for _ in range(world)]
            dist.all_gather(parts, x_local)
            worst_ag = max(worst_ag, rel(y, torch.cat(parts).float() @ w.float()))
            # row-parallel: each rank holds a K-slice; result rows are scattered
            xr = torch.randn(rows * world, K, device=device, generator=g).to(torch.bfloat16)
            z = ctx.matmul_reduce_scatter(xr, w)
            full = xr.float() @ w.float()
            dist.all_reduce(full)
            worst_rs = max(worst_rs, rel(z, full[rank * rows:(rank + 1) * rows]))
        res[f"ag_gemm_{rows}x{K}x{N}"] = worst_ag
        res[f"gemm_rs_{rows}x{K}x{N}"] = worst_rs
    # a column-parallel + row-parallel pair (the shape of an MLP or attention block under sequence parallelism),
    # differentiated through the fused kernels, against the same pair on gathered tensors with library collectives
    from jax_gpt_b200.parallel.tensor_parallel import column_parallel_linear, row_parallel_linear
    rows, K, H = 256, 512, 1024
    gen = torch.Generator(device=device).manual_seed(50 + rank)
    x_local = torch.randn(rows, K, device=device, generator=gen).to(torch.bfloat16).requires_grad_()
    w1 = (torch.randn(K, H // world, device=device, generator=gen) * 0.05).to(torch.bfloat16).requires_grad_()
    w2 = (torch.randn(H // world, K, device=device, generator=gen) * 0.05).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(rows, K, device=device, generator=gen).to(torch.bfloat16)
    y = row_parallel_linear(torch.nn.functional.gelu(column_parallel_linear(x_local, w1, ctx).float()).to(torch.bfloat16), w2, ctx)
    y.backward(dy)
    xs = [torch.empty_like(x_local) for _ in range(world)]
    dist.all_gather(xs, x_local.detach())
    xf = torch.cat(xs).float().requires_grad_()
    w1f, w2f = w1.detach().float().requires_grad_(), w2.detach().float().requires_grad_()
    part = torch.nn.functional.gelu(xf @ w1f).to(torch.bfloat16).float() @ w2f
    full = part.detach().clone()
    dist.all_reduce(full)
    dys = [torch.empty_like(dy) for _ in range(world)]
    dist.all_gather(dys, dy)
    part.backward(torch.cat(dys).float())
    gx = xf.grad.clone()
    dist.all_reduce(gx)
    res["tp_pair_out"] = rel(y, full[rank * rows:(rank + 1) * rows])
    res["tp_pair_dx"] = rel(x_local.grad, gx[rank * rows:(rank + 1) * rows])
    res["tp_pair_dw1"] = rel(w1.grad, w1f.grad)
    res["tp_pair_dw2"] = rel(w2.grad, w2f.grad)
    torch.cuda.synchronize()
    _ext.check_status(device)
    dist.barrier()
    return res


def run_cp(rank, world, device):
    """Context-parallel causal attention on the flash kernels (block by block, merged with log-sum-exps) against
    dense attention in fp32; head widths 64 (GPT-2) and 256 with grouped kv heads (gated attention)."""
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.ops.attention import attention_ref
    from jax_gpt_b200.parallel.context_parallel import context_parallel_attention, zigzag_split
    res = {}
    for (H, Hkv, D) in [(4, 4, 64), (4, 2, 256)]:
        g = torch.Generator(device=device).manual_seed(17)
        B, T = 2, 256 * 2 * world
        q = torch.randn(B, T, H, D, device=device, generator=g).to(torch.bfloat16)
        k = torch.randn(B, T, Hkv, D, device=device, generator=g).to(torch.bfloat16)
        v = torch.randn(B, T, Hkv, D, device=device, generator=g).to(torch.bfloat16)
        w = torch.randn(B, T, H, D, device=device, generator=g).to(torch.bfloat16)
        qr, kr, vr = [t.float().requires_grad_() for t in (q, k, v)]
        ref = attention_ref(qr, kr, vr, causal=True)
        (ref * w.float()).sum().backward()
        ql, kl, vl = [zigzag_split(t, world, rank).contiguous().requires_grad_() for t in (q, k, v)]
        out = context_parallel_attention(ql, kl, vl)
        (out.float() * zigzag_split(w, world, rank).float()).sum().backward()
        torch.cuda.synchronize()
        _ext.check_status(device)
        res[f"cp_out_d{D}"] = rel(out, zigzag_split(ref, world, rank))
        res[f"cp_dq_d{D}"] = rel(ql.grad, zigzag_split(qr.grad, world, rank))
        res[f"cp_dk_d{D}"] = rel(kl.grad, zigzag_split(kr.grad, world, rank))
        res[f"cp_dv_d{D}"] = rel(vl.grad, zigzag_split(vr.grad, world, rank))
    return res


def run_sp(rank, world, device):
    """GPT-2 with tensor + sequence parallelism on the fused all-gather -> GEMM / GEMM -> reduce-scatter kernels:
    loss and every gradient against the unsharded bf16 model run on the same batch."""
    from types import SimpleNamespace
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.models.gpt2 import GPT, GPTConfig
    from jax_gpt_b200.parallel.sequence_parallel import (SHARDED, gpt2_sequence_parallel_loss,
                                                         shard_gpt2_for_sequence_parallel, sync_replicated_grads)
    from jax_gpt_b200.parallel.tensor_parallel import TPContext
    from jax_gpt_b200.trainer.sharding import shard_gpt2_tensor
    cfg = GPTConfig(d_model=256, d_head=64, d_ff=1024, d_context=256, n_head=4, n_kv_head=4, n_layers=2, vocab_size=512)
    ref = GPT(cfg, seed=21, device=device, dtype=torch.bfloat16)
    ref.requires_grad_(True)
    g = torch.Generator().manual_seed(4)
    tok = torch.randint(0, cfg.vocab_size, (2 * world, 257), generator=g).to(device)
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    logits, _ = ref(x)
    loss_ref = torch.nn.functional.cross_entropy(logits.float().reshape(-1, cfg.vocab_size), y.reshape(-1))
    loss_ref.backward()
    tp = TPContext(device=device, wait_seconds=5.0)
    params = shard_gpt2_for_sequence_parallel(ref.params, cfg, world, rank)
    for v in params.values():
        v.requires_grad_(True)
    part = gpt2_sequence_parallel_loss(params, cfg, x, y, tp)
    part.backward()
    sync_replicated_grads(params)
    torch.cuda.synchronize()
    _ext.check_status(device)
    tot = part.detach().clone()
    dist.all_reduce(tot)
    res = {"sp_loss_abs": abs(float(tot) - float(loss_ref))}
    mesh = SimpleNamespace(size=lambda ax: world if ax == "tp" else 1, rank=lambda ax: rank if ax == "tp" else 0)
    worst_sh = worst_rep = 0.0
    for k, v in params.items():
        rg = ref.params[k].grad
        if rg is None or v.grad is None or k == "lm_head.kernel":
            continue
        if k in SHARDED:
            worst_sh = max(worst_sh, rel(v.grad, shard_gpt2_tensor(k, rg, cfg, mesh)))
        else:
            worst_rep = max(worst_rep, rel(v.grad, rg))
    res["sp_sharded_grad_rel"] = worst_sh
    res["sp_replicated_grad_rel"] = worst_rep
    dist.barrier()
    return res


def run_fsdp_ag(rank, world, device):
    """Column-sharded weight gathered inside the consuming GEMM (pushed by copier CTAs) vs the plain product."""
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.comm.symm import Communicator
    from jax_gpt_b200.parallel.fsdp import ShardedWeight
    comm = Communicator(device=device, wait_seconds=5.0)
    res = {}
    for (M, K, N) in [(512, 1024, 1024), (300, 512, 512)]:
        g = torch.Generator(device=device).manual_seed(21)
        w = (torch.randn(K, N, device=device, generator=g) * 0.05).to(torch.bfloat16)
        x = torch.randn(M, K, device=device, generator=torch.Generator(device=device).manual_seed(rank)).to(torch.bfloat16)
        sw = ShardedWeight(comm, w)
        w2 = (w.float() * 0.5 + 0.01).to(torch.bfloat16)        # a second weight of the same shape shares the scratch buffer
        sw2 = ShardedWeight(comm, w2)
        worst = 0.0
        for call in range(3):
            y, y2 = sw.matmul(x), sw2.matmul(x)
            worst = max(worst, rel(y, x.float() @ w.float()), rel(y2, x.float() @ w2.float()))
        torch.cuda.synchronize()
        _ext.check_status(device)
        res[f"ag_gemm_{M}x{K}x{N}"] = worst
        comm.barrier()
    dist.barrier()
    return res


def run_ep(rank, world, device):
    """Fused expert-parallel MoE forward vs a dense evaluation with all experts and vs the NCCL path."""
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.comm.symm import Communicator
    from jax_gpt_b200.models.qwen35.moe import expert_forward_single
    from jax_gpt_b200.parallel.expert_parallel import FusedEPMoE, NcclEPMoE
    tokens, D, I, E, k = 384, 512, 256, 16, 4
    g = torch.Generator(device=device).manual_seed(3)  # same weights on every rank
    full = {"gate_proj": (torch.randn(E, D, I, device=device, generator=g) * 0.05).to(torch.bfloat16),
            "up_proj": (torch.randn(E, D, I, device=device, generator=g) * 0.05).to(torch.bfloat16),
            "down_proj": (torch.randn(E, I, D, device=device, generator=g) * 0.05).to(torch.bfloat16)}
    el = E // world
    local = {n: t[rank * el:(rank + 1) * el].contiguous() for n, t in full.items()}
    comm = Communicator(device=device, wait_seconds=5.0)
    fused = FusedEPMoE(comm, tokens, D, I, E, k)
    nccl = NcclEPMoE(dist.group.WORLD, E)
    res = {}
    for step, mode in enumerate(["uniform", "skewed", "uniform"]):
        gs = torch.Generator(device=device).manual_seed(100 * step + rank)
        x = torch.randn(tokens, D, device=device, generator=gs).to(torch.bfloat16)
        logits = torch.randn(tokens, E, device=device, generator=gs)
        if mode == "skewed":
            logits[:, :3] += 6.0     # almost everything goes to three experts of rank 0; several experts stay empty
            logits[:, 5] = -1e9
        w, idx = torch.softmax(logits, -1).topk(k, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        out = fused.forward(x, w, idx, local).clone()
        torch.cuda.synchronize()
        _ext.check_status(device)
        ref = expert_forward_single(x.float(), w, idx, {n: t.float() for n, t in full.items()})
        base = nccl.forward(x, w, idx, local)
        res[f"{mode}{step}_fused_vs_dense"] = rel(out, ref)
        res[f"{mode}{step}_nccl_vs_dense"] = rel(base, ref)
        dist.barrier()
    res["rows_last"] = fused.rows_out.tolist()
    return res


def run_ep_bwd(rank, world, device):
    """Fused expert-parallel MoE backward vs autograd of the dense evaluation with all experts."""
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.comm.symm import Communicator
    from jax_gpt_b200.models.qwen35.moe import expert_forward_single
    from jax_gpt_b200.parallel.expert_parallel import FusedEPMoE
    tokens, D, I, E, k = 384, 512, 256, 16, 4
    g = torch.Generator(device=device).manual_seed(3)
    full = {"gate_proj": (torch.randn(E, D, I, device=device, generator=g) * 0.05).to(torch.bfloat16),
            "up_proj": (torch.randn(E, D, I, device=device, generator=g) * 0.05).to(torch.bfloat16),
            "down_proj": (torch.randn(E, I, D, device=device, generator=g) * 0.05).to(torch.bfloat16)}
    el = E // world
    local = {n: t[rank * el:(rank + 1) * el].contiguous() for n, t in full.items()}
    comm = Communicator(device=device, wait_seconds=5.0)
    fused = FusedEPMoE(comm, tokens, D, I, E, k, training=True)
    res = {}
    for step, mode in enumerate(["uniform", "skewed", "uniform"]):
        gs = torch.Generator(device=device).manual_seed(100 * step + rank)
        x = torch.randn(tokens, D, device=device, generator=gs).to(torch.bfloat16)
        dout = torch.randn(tokens, D, device=device, generator=gs).to(torch.bfloat16)
        logits = torch.randn(tokens, E, device=device, generator=gs)
        if mode == "skewed":
            logits[:, :3] += 6.0
            logits[:, 5] = -1e9
        w, idx = torch.softmax(logits, -1).topk(k, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        grads = {n: torch.zeros_like(t, dtype=torch.float32) for n, t in local.items()}
        out = fused.forward(x, w, idx, local).clone()
        dx, dw = fused.backward(x, dout, w, idx, local, grads)
        dx, dw = dx.clone(), dw.clone()
        torch.cuda.synchronize()
        _ext.check_status(device)
        xr = x.float().requires_grad_(True)
        wr = w.float().requires_grad_(True)
        pr = {n: t.float().requires_grad_(True) for n, t in full.items()}
        ref = expert_forward_single(xr, wr, idx, pr)
        (ref * dout.float()).sum().backward()
        res[f"{mode}{step}_out"] = rel(out, ref.detach())
        res[f"{mode}{step}_dx"] = rel(dx, xr.grad)
        res[f"{mode}{step}_dw"] = rel(dw, wr.grad)
        for n in full:
            gfull = pr[n].grad.clone()
            dist.all_reduce(gfull)
            res[f"{mode}{step}_d{n}"] = rel(grads[n], gfull[rank * el:(rank + 1) * el])
        dist.barrier()
    return res


def run_ep_fp8(rank, world, device):
    """FP8 fused expert-parallel forward vs the fp32 restatement of its quantised arithmetic and vs bf16 math."""
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.comm.symm import Communicator
    from jax_gpt_b200.models.qwen35.moe import expert_forward_single
    from jax_gpt_b200.parallel.expert_parallel import FusedEPMoEFp8, fp8_moe_reference, quantize_expert_weights_fp8
    tokens, D, I, E, k = 384, 512, 256, 16, 4
    g = torch.Generator(device=device).manual_seed(3)
    full = {"gate_proj": (torch.randn(E, D, I, device=device, generator=g) * 0.05).to(torch.bfloat16),
            "up_proj": (torch.randn(E, D, I, device=device, generator=g) * 0.05).to(torch.bfloat16),
            "down_proj": (torch.randn(E, I, D, device=device, generator=g) * 0.05).to(torch.bfloat16)}
    el = E // world
    qw_full = quantize_expert_weights_fp8(full)
    qw = {n: t[rank * el:(rank + 1) * el].contiguous() for n, t in qw_full.items()}
    comm = Communicator(device=device, wait_seconds=5.0)
    fused = FusedEPMoEFp8(comm, tokens, D, I, E, k)
    res = {}
    for step, mode in enumerate(["uniform", "skewed", "uniform"]):
        gs = torch.Generator(device=device).manual_seed(100 * step + rank)
        x = (torch.randn(tokens, D, device=device, generator=gs) * (1 + 3 * torch.rand(tokens, 1, device=device, generator=gs))).to(torch.bfloat16)
        logits = torch.randn(tokens, E, device=device, generator=gs)
        if mode == "skewed":
            logits[:, :3] += 6.0
            logits[:, 5] = -1e9
        w, idx = torch.softmax(logits, -1).topk(k, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        out = fused.forward(x, w, idx, qw).clone()
        torch.cuda.synchronize()
        _ext.check_status(device)
        ref_q = fp8_moe_reference(x, w, idx, qw_full)
        ref = expert_forward_single(x.float(), w, idx, {n: t.float() for n, t in full.items()})
        res[f"{mode}{step}_fused_vs_quantised_ref"] = rel(out, ref_q)
        res[f"{mode}{step}_fused_vs_bf16_math"] = rel(out, ref)
        dist.barrier()
    return res


def run_tp_attention(rank, world, device):
    """MLA and gated attention with heads split over the ranks and tokens sharded between layers (fused
    all-gather -> GEMM in, GEMM -> reduce-scatter out) vs the single-GPU layers."""
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.models.deepseek_v3.config import DeepSeekV3Config
    from jax_gpt_b200.models.deepseek_v3.model import _attn_params, mla_prefill
    from jax_gpt_b200.models.qwen35.gqa import gqa_attention
    from jax_gpt_b200.models.qwen35.primitives import precompute_rope_freqs
    from jax_gpt_b200.parallel.tensor_parallel import TPContext
    from jax_gpt_b200.parallel.tp_attention import gqa_attention_tp, mla_prefill_tp, shard_gqa_params, shard_mla_params
    ctx = TPContext(device=device, wait_seconds=5.0)
    g = torch.Generator().manual_seed(5)
    bf = torch.bfloat16
    res = {}
    # ---- MLA ----
    c = DeepSeekV3Config.tiny().replace(d_model=512, n_heads=8, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                                        q_lora_rank=256, kv_lora_rank=512, max_position_embeddings=512)
    n = lambda *s: (torch.randn(*s, generator=g) * 0.05).to(device=device, dtype=bf)
    ones = lambda *s: torch.ones(*s, device=device, dtype=bf)
    ap = _attn_params(c, (), n, ones)
    B, T = 2, 256
    x = torch.randn(B, T, c.d_model, generator=g).to(device=device, dtype=bf)
    rope = precompute_rope_freqs(c.qk_rope_head_dim, 512, c.rope_theta, device=device)
    with torch.no_grad():
        ref, _ = mla_prefill(x, ap, c, rope)
        rows = B * T // world
        xl = x.reshape(B * T, -1)[rank * rows:(rank + 1) * rows].contiguous()
        out = mla_prefill_tp(ctx, xl, shard_mla_params(ap, c, rank, world), c, rope, B, T)
    res["mla_tp"] = rel(out, ref.reshape(B * T, -1)[rank * rows:(rank + 1) * rows])
    # ---- gated attention ----
    D, Hq, Hkv, dh = 512, 8, 2, 128
    gp = {"q_proj": n(D, 2 * Hq * dh), "k_proj": n(D, Hkv * dh), "v_proj": n(D, Hkv * dh), "o_proj": n(Hq * dh, D),
          "q_norm": torch.zeros(dh, device=device, dtype=bf), "k_norm": torch.zeros(dh, device=device, dtype=bf)}
    x2 = torch.randn(B, T, D, generator=g).to(device=device, dtype=bf)
    fr = precompute_rope_freqs(32, 512, 1e7, device=device)
    with torch.no_grad():
        ref2, _, _ = gqa_attention(x2, gp, Hq, Hkv, dh, fr, 32)
        xl2 = x2.reshape(B * T, -1)[rank * rows:(rank + 1) * rows].contiguous()
        out2 = gqa_attention_tp(ctx, xl2, shard_gqa_params(gp, Hq, Hkv, dh, rank, world), Hkv, dh, fr, 32, B, T)
    res["gqa_tp"] = rel(out2, ref2.reshape(B * T, -1)[rank * rows:(rank + 1) * rows])
    torch.cuda.synchronize()
    _ext.check_status(device)
    dist.barrier()
    return res


def run_vocab_ce(rank, world, device):
    """Vocabulary-parallel cross-entropy (one kernel, statistics exchanged over peer memory) vs the full softmax."""
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.comm.symm import Communicator
    from jax_gpt_b200.parallel.tensor_parallel import VocabParallelCE, vocab_parallel_ce_reference
    M, V, D = 777, 50304, 256
    g = torch.Generator(device=device).manual_seed(11)
    h = torch.randn(M, D, device=device, generator=g).to(torch.bfloat16)
    w = (torch.randn(D, V, device=device, generator=g) * 0.2).to(torch.bfloat16)
    targets = torch.randint(0, V, (M,), device=device, generator=g)
    targets[5] = -1
    comm = Communicator(device=device, wait_seconds=5.0)
    vp = VocabParallelCE(comm, V)
    res = {}
    for step in range(3):
        w_local = w[:, vp.v0:vp.v0 + vp.v_local].contiguous().requires_grad_(True)
        logits_local = (h @ w_local)
        keep = logits_local.detach().clone()
        loss = vp(logits_local, targets)
        loss.backward()
        torch.cuda.synchronize()
        _ext.check_status(device)
        wf = w.float().requires_grad_(True)
        full = torch.nn.functional.cross_entropy(h.float() @ wf, targets.long(), ignore_index=-1)
        full.backward()
        res[f"loss_err{step}"] = abs(loss.item() - full.item()) / full.item()
        res[f"dw_rel{step}"] = rel(w_local.grad, wf.grad[:, vp.v0:vp.v0 + vp.v_local])
        l2, g2 = vocab_parallel_ce_reference(keep, targets, vp.v0)
        res[f"ref_loss_err{step}"] = abs((l2.sum() / (targets >= 0).sum()).item() - full.item()) / full.item()
        dist.barrier()
    return res


def run_moe_train(rank, world, device):
    """Qwen3.5-style training with expert parallelism (fused MoE forward/backward kernels) and the fused
    sharded optimizer for the dense weights, against one process that holds all experts and sees every
    rank's batch as micro-batches."""
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.models.qwen35.config import Qwen35Config
    from jax_gpt_b200.models.qwen35.model import init_params
    from jax_gpt_b200.parallel.expert_parallel import EPMoERuntime, FusedEPMoE, is_expert_leaf, shard_experts
    from jax_gpt_b200.parallel.fsdp import FusedShardedAdamW
    from jax_gpt_b200.trainer.lm_loss import qwen35_loss_fn
    from jax_gpt_b200.trainer.tree_engine import TreeTrainEngine
    cfg = Qwen35Config(d_model=256, vocab_size=512, n_layers=4, max_position_embeddings=128, gqa_n_q_heads=4,
                       gqa_n_kv_heads=2, gqa_head_dim=64, delta_n_qk_heads=2, delta_n_v_heads=4, delta_qk_head_dim=32,
                       delta_v_head_dim=32, delta_chunk_size=16, n_routed_experts=8, n_experts_per_token=2,
                       moe_intermediate_size=256, shared_expert_intermediate_size=256)
    B, T = 2, 64
    full = init_params(cfg, 0, torch.float32)
    hyper = dict(lr=2e-3, min_lr=2e-3, warmup_steps=0, grad_clip=1.0)
    opt = FusedShardedAdamW(device=device, wait_seconds=10.0)
    layer = FusedEPMoE(opt.comm, B * T, cfg.d_model, cfg.moe_intermediate_size, cfg.n_routed_experts,
                       cfg.n_experts_per_token, training=True)
    ep = EPMoERuntime(layer)
    eng = TreeTrainEngine(shard_experts(full, rank, world), qwen35_loss_fn(cfg, ep), device=device, local=is_expert_leaf,
                          dist_optimizer=opt, **hyper)
    ref = TreeTrainEngine(full, qwen35_loss_fn(cfg, None), device=device, **hyper)
    res = {"ep_loss": [], "ref_loss": []}
    for step in range(4):
        g = torch.Generator().manual_seed(1000)   # the same batch every step: the loss must fall
        tok_all = torch.randint(0, cfg.vocab_size, (world, B, T + 1), generator=g).to(device)
        mine = tok_all[rank]
        out = eng.train_step(mine[:, :-1].contiguous(), mine[:, 1:].contiguous())
        loss = out["loss"].clone()
        dist.all_reduce(loss)
        for r in range(world):
            ref.micro_step(tok_all[r][:, :-1].contiguous(), tok_all[r][:, 1:].contiguous())
        rout = ref.apply_gradients()
        torch.cuda.synchronize()
        _ext.check_status(device)
        res["ep_loss"].append(loss.item() / world)
        res["ref_loss"].append(rout["loss"].item())
        res.setdefault("gnorm_ep", []).append(out["grad_norm_sq"].item() ** 0.5 / world)
        res.setdefault("gnorm_ref", []).append(rout["grad_norm_sq"].item() ** 0.5 / world)
    return res


def main():
    what = sys.argv[1]
    out_path = sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    if what == "fsdp":
        res = run_fsdp(rank, world, device, False)
    elif what == "fsdp_multimem":
        res = run_fsdp(rank, world, device, True)
    elif what == "ckpt_manager":
        res = run_ckpt_manager(rank, world, device, out_path + ".ckpt")
    elif what == "pp":
        res = run_pp(rank, world, device)
    elif what == "tp":
        res = run_tp(rank, world, device)
    elif what == "sp":
        res = run_sp(rank, world, device)
    elif what == "cp":
        res = run_cp(rank, world, device)
    elif what == "fsdp_ag":
        res = run_fsdp_ag(rank, world, device)
    elif what == "ep":
        res = run_ep(rank, world, device)
    elif what == "ep_bwd":
        res = run_ep_bwd(rank, world, device)
    elif what == "tp_attention":
        res = run_tp_attention(rank, world, device)
    elif what == "vocab_ce":
        res = run_vocab_ce(rank, world, device)
    elif what == "ep_fp8":
        res = run_ep_fp8(rank, world, device)
    elif what == "moe_train":
        res = run_moe_train(rank, world, device)
    else:
        raise SystemExit(f"unknown test {what}")
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(res, f)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
