"""Benchmarks of the expert-parallel paths as library functions: the fused EP-MoE layer (forward, backward, FP8
forward, roofline fraction) and a training step of the MoE model families at a chosen depth. ``bench.py`` reports
them next to the headline number when it runs on two or more GPUs; ``scripts/moe_microbench.py`` and
``scripts/bench_moe_train.py`` are their command-line fronts. All times are CUDA events, maximum over ranks.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def _timed(fn, warmup: int, iters: int, device):
    from .profiling import max_over_ranks
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


def make_router_logits(tokens: int, experts: int, mode: str, device, gen):
    """N(0,1) logits, optionally with a Zipf(s = 1.2) prior over a fixed random permutation of the experts."""
    logits = torch.randn(tokens, experts, device=device, generator=gen)
    if mode == "zipf":
        ranks = torch.arange(1, experts + 1, device=device, dtype=torch.float32)
        prior = torch.log(ranks.pow(-1.2) / ranks.pow(-1.2).sum())
        perm = torch.randperm(experts, device=device, generator=torch.Generator(device=device).manual_seed(7))
        logits = logits + prior[perm] - prior.mean()
    return logits


def ep_moe_layer_bench(device, rank: int, world: int, tokens: int = 4096, d_model: int = 7168, inter: int = 2048,
                       experts: int = 256, top_k: int = 8, n_group: int = 8, topk_group: int = 4, router: str = "normal",
                       warmup: int = 3, iters: int = 5, backward: bool = True, fp8: bool = True, baseline: bool = False,
                       check: bool = False, comm=None) -> dict:
    """One expert-parallel MoE layer of the DeepSeek-V3 shape: every rank owns ``tokens`` bf16 activations ~N(0,1),
    routing is the group-limited sigmoid top-k. Roofline of the busiest rank:
    ``max(FLOPs / measured GEMM rate, NVLink bytes / measured link rate) / time``."""
    from .. import _ext
    from ..comm.symm import Communicator
    from ..ops.router import deepseek_router_from_logits
    from ..parallel.expert_parallel import FusedEPMoE, NcclEPMoE
    from . import roofline as R
    E, D, I, k, T = experts, d_model, inter, top_k, tokens
    el = E // world
    gen = torch.Generator(device=device).manual_seed(11 + rank)
    wgen = torch.Generator(device=device).manual_seed(5)
    local = {n: (torch.randn(el, a, b, device=device, generator=wgen, dtype=torch.bfloat16) * 0.02)
             for n, (a, b) in (("gate_proj", (D, I)), ("up_proj", (D, I)), ("down_proj", (I, D)))}
    x = torch.randn(T, D, device=device, generator=gen).to(torch.bfloat16)
    logits = make_router_logits(T, E, router, device, gen)
    w, idx = deepseek_router_from_logits(logits, torch.zeros(E, device=device), k, n_group, topk_group, 2.5)
    comm = comm or Communicator(device=device, wait_seconds=20.0)
    fused = FusedEPMoE(comm, T, D, I, E, k, training=backward)
    ms_fused = _timed(lambda: fused.forward(x, w, idx, local), warmup, iters, device)
    _ext.check_status(device)
    rows = fused.rows_out.sum().item()
    res = {"world": world, "tokens_per_rank": T, "router": router, "d_model": D, "inter": I, "experts": E, "top_k": k,
           "dtype": "bf16", "fused_fwd_ms": ms_fused, "rows_this_rank": rows}
    if moe_phase_timeline(0) is not None:
        res["fwd_timeline_us"] = moe_phase_timeline(0)
    if backward:
        dout = torch.randn(T, D, device=device, generator=gen).to(torch.bfloat16)
        grads = {n: torch.zeros_like(t, dtype=torch.float32) for n, t in local.items()}
        fused.forward(x, w, idx, local)
        ms_bwd = _timed(lambda: fused.backward(x, dout, w, idx, local, grads), warmup, iters, device)
        _ext.check_status(device)
        res["fused_bwd_ms"] = ms_bwd
        res["bwd_tflops_this_rank"] = 2.0 * rows * 6 * D * I / ms_bwd / 1e9
        if moe_phase_timeline(1) is not None:
            res["bwd_timeline_us"] = moe_phase_timeline(1)
        del grads
    if fp8:
        from ..parallel.expert_parallel import FusedEPMoEFp8, quantize_expert_weights_fp8
        qw = quantize_expert_weights_fp8(local)
        f8 = FusedEPMoEFp8(comm, T, D, I, E, k)
        ms8 = _timed(lambda: f8.forward(x, w, idx, qw), warmup, iters, device)
        _ext.check_status(device)
        res["fused_fp8_fwd_ms"] = ms8
        res["fp8_tflops_this_rank"] = 2.0 * rows * 3 * D * I / ms8 / 1e9
        if check:
            a8 = f8.forward(x, w, idx, qw).float().clone()
            b16 = fused.forward(x, w, idx, local).float()
            res["fp8_vs_bf16_rel"] = ((a8 - b16).norm() / b16.norm()).item()
        del qw, f8
    if baseline and world > 1:
        base = NcclEPMoE(dist.group.WORLD, E)
        res["nccl_fwd_ms"] = _timed(lambda: base.forward(x, w, idx, local), 1, max(1, iters // 2), device)
        res["speedup"] = res["nccl_fwd_ms"] / ms_fused
        if check:
            a = fused.forward(x, w, idx, local).float()
            b = base.forward(x, w, idx, local).float()
            res["fused_vs_nccl_rel"] = ((a - b).norm() / b.norm()).item()
    t = torch.tensor([float(rows)], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    max_rows = t.item()
    flops = 2.0 * max_rows * 3 * D * I
    remote = (world - 1) / world
    nv_bytes = max(max_rows, T * k) * remote * (D * 2 + D * 4)   # bf16 row in, fp32 reduction out
    peaks = R.load_peaks()
    bound = max(flops / (peaks["bf16_tflops"] * 1e12), nv_bytes / (R.NVLINK_GBS_MEASURED * 1e9))
    # HBM floors (bytes every launch has to move once): forward = the rank's expert weights, the received rows
    # written and read, act written and read, the pre-activations written; backward = weights read, fp32 weight
    # gradients read and written by the accumulation, dY rows written and read twice, x / act / pre-activations read,
    # dGU written and read twice
    w_elems = 3.0 * (E // world) * D * I
    hbm = peaks["hbm_gbs"] * 1e9
    fwd_bytes = w_elems * 2 + max_rows * (2 * D * 2 + 2 * I * 2 + 2 * I * 2)
    bwd_bytes = w_elems * 2 + w_elems * 8 + max_rows * (3 * D * 2 + D * 2 + I * 2 + 2 * I * 2 + 3 * 2 * I * 2)
    res.update(hbm_floor_fwd_ms=fwd_bytes / hbm * 1e3, hbm_floor_bwd_ms=bwd_bytes / hbm * 1e3)
    if backward:
        bwd_bound = max(2.0 * flops / (peaks["bf16_tflops"] * 1e12), bwd_bytes / hbm,
                        nv_bytes / (R.NVLINK_GBS_MEASURED * 1e9))
        res["roofline_fraction_bwd_with_hbm"] = bwd_bound * 1e3 / res["fused_bwd_ms"]
    res["roofline_fraction_fwd_with_hbm"] = max(bound, fwd_bytes / hbm) * 1e3 / ms_fused
    res.update(max_rows_any_rank=max_rows, tflops_busiest_rank=flops / ms_fused / 1e9, roofline_ms=bound * 1e3,
               roofline_fraction=bound * 1e3 / ms_fused, denominators=peaks["source"],
               tokens_per_s=T * world / (ms_fused / 1e3))
    if backward:
        res["roofline_fraction_fwd_bwd"] = 3.0 * bound * 1e3 / (ms_fused + res["fused_bwd_ms"])
    del fused, local
    torch.cuda.empty_cache()
    return res


def moe_phase_timeline(which: int) -> Optional[dict]:
    """Summary (microseconds; median and max over the CTAs) of the phase timeline the fused MoE forward
    (``which`` = 0) or backward (1) kernel recorded on its last launch; None unless ``B200_MOE_PROFILE=1`` was set
    before the first launch. Wait columns are SM cycles converted with the launch's own cycles-per-nanosecond."""
    import os
    from .. import _ext
    if os.environ.get("B200_MOE_PROFILE", "0") != "1":
        return None
    p = _ext.ops().moe_profile(which).double()
    p = p[p[:, 0] > 0]
    if p.numel() == 0:
        return None
    start = p[:, 0].min()
    us = lambda col: {"median": round(((p[:, col] - start).median() / 1e3).item(), 1),
                      "max": round(((p[:, col] - start).max() / 1e3).item(), 1)}
    cyc_per_ns = (p[:, 9] / (p[:, 4] - p[:, 0]).clamp_min(1.0)).median().item()
    wait = lambda col: {"median": round((p[:, col] / cyc_per_ns / 1e3).median().item(), 1),
                        "max": round((p[:, col] / cyc_per_ns / 1e3).max().item(), 1)}
    return {"ctas": int(p.shape[0]), "sm_mhz": round(cyc_per_ns * 1e3), "tables_built": us(1), "dispatch_done": us(2),
            "loads_issued": us(3), "epilogue_done": us(8), "end": us(4), "load_warp_dependency_wait": wait(5),
            "mma_operand_wait": wait(6), "mma_accumulator_wait": wait(7)}


def moe_train_bench(device, rank: int, world: int, model: str = "qwen35", layers: int = 4, experts: int = 64,
                    seq: int = 4096, batch: int = 1, accum: int = 1, vocab: int = 0, buffer_sets: int = 4,
                    fp8: bool = False, lowmem: bool = False, steps: int = 3, warmup: int = 2, dist_opt=None) -> dict:
    """Training steps of the Qwen3.5-style hybrid or the DeepSeek-V3-style model at benchmark widths: experts sharded
    over the ranks (fused dispatch / grouped GEMM / combine kernels, forward and backward), dense weights through
    the fused sharded optimizer, parameters drawn on the device per shard. ``lowmem``: expert weights without an
    fp32 master and with bf16 moments. ``accum`` micro-batches of ``batch`` sequences per optimizer step."""
    from .. import _ext
    from ..trainer.lm_loss import deepseek_v3_loss_fn, deepseek_v3_unstack, qwen35_loss_fn, qwen35_unstack
    from ..trainer.tree_engine import TreeTrainEngine
    from .profiling import max_over_ranks
    if model == "qwen35":
        from ..models.qwen35.config import Qwen35Config
        from ..models.qwen35.model import init_params
        cfg = Qwen35Config.ns().replace(n_layers=layers, n_routed_experts=experts, max_position_embeddings=seq)
        make_loss, unstack = qwen35_loss_fn, qwen35_unstack
    else:
        from ..models.deepseek_v3.config import DeepSeekV3Config
        from ..models.deepseek_v3.model import init_params
        cfg = DeepSeekV3Config.full().replace(n_layers=layers, first_k_dense=1, n_routed_experts=experts,
                                              max_position_embeddings=seq)
        make_loss, unstack = deepseek_v3_loss_fn, deepseek_v3_unstack
    if vocab:
        cfg = cfg.replace(vocab_size=vocab)
    shard = (rank, world) if world > 1 else None
    params = init_params(cfg, 0, torch.bfloat16, device=device, on_device=True, expert_shard=shard)
    n_moe = cfg.n_layers if model == "qwen35" else cfg.n_layers - cfg.first_k_dense
    n_sets = max(1, min(buffer_sets, n_moe))
    from ..comm.symm import Communicator
    from ..parallel.expert_parallel import EPMoERuntime, FusedEPMoE, is_expert_leaf
    if world > 1 and dist_opt is None:
        from ..parallel.fsdp import FusedShardedAdamW
        dist_opt = FusedShardedAdamW(device=device)
    comm = dist_opt.comm if dist_opt is not None else Communicator(device=device)
    moe_layers = [FusedEPMoE(comm, batch * seq, cfg.d_model, cfg.moe_intermediate_size, cfg.n_routed_experts,
                             cfg.n_experts_per_token, training=True) for _ in range(n_sets)]
    ep, local = EPMoERuntime(moe_layers), is_expert_leaf
    eng = TreeTrainEngine(params, make_loss(cfg, ep, fp8=fp8), device=device, local=local, lr=1e-4, min_lr=1e-4,
                          warmup_steps=0, dist_optimizer=dist_opt, unstack=unstack, consume_params=True,
                          local_state_dtype=torch.bfloat16 if lowmem else torch.float32)
    del params
    torch.cuda.empty_cache()
    g = torch.Generator().manual_seed(1 + rank)
    toks = [torch.randint(0, cfg.vocab_size, (batch, seq + 1), generator=g).to(device) for _ in range(accum)]

    def step():
        for t in toks:
            eng.micro_step(t[:, :-1].contiguous(), t[:, 1:].contiguous())
        return eng.apply_gradients()
    for _ in range(warmup):
        out = step()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a.record()
    for _ in range(steps):
        out = step()
    b.record()
    torch.cuda.synchronize()
    _ext.check_status(device)
    ms = a.elapsed_time(b) / steps
    ms = max_over_ranks(ms, device) if world > 1 else ms
    res = {"model": model, "layers": layers, "experts": experts, "seq_len": seq, "global_batch": batch * accum * world,
           "n_gpus": world, "params_this_rank_M": eng.n_params() / 1e6, "ms_per_step": ms,
           "tokens_per_s": batch * accum * seq * world / (ms / 1e3), "loss": float(out["loss"]),
           "dtype": "bf16 + fp8 dense GEMMs" if fp8 else "bf16",
           "expert_state": "bf16 weights and moments, stochastic rounding" if lowmem else "fp32 master and moments",
           "parallelism": f"ep{world} + sharded optimizer (dp{world})" if world > 1 else "1gpu",
           "peak_mem_GB": torch.cuda.max_memory_allocated() / 2 ** 30}
    del eng, ep, moe_layers
    torch.cuda.empty_cache()
    return res


def tp_fused_gemm_bench(device, rank: int, world: int, rows: int = 4096, K: int = 7168, N: int = 16384, warmup: int = 3,
                        iters: int = 10, link_gbs: float = 770.0) -> dict:
    """The three fused collective + GEMM kernels (all-gather -> GEMM, GEMM -> reduce-scatter, FSDP weight gather ->
    GEMM) against the same math done with a library collective around this package's plain GEMM: CUDA events, max
    over ranks. Roofline per path: the slower of (FLOPs of this rank / measured bf16 GEMM rate) and (bytes this rank
    must move over NVLink / ``link_gbs`` per direction); reported as bound / time."""
    from .. import _ext
    from ..ops.gemm import gemm
    from ..parallel.fsdp import ShardedWeight
    from ..parallel.tensor_parallel import TPContext, all_gather_matmul_nccl, matmul_reduce_scatter_nccl
    from . import roofline as R
    assert K % (world * 64) == 0 and N % (world * 128) == 0 and rows % 128 == 0
    peaks = R.load_peaks()
    peak, link = peaks["bf16_tflops"] * 1e12, link_gbs * 1e9

    def timed(fn):
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

    ctx = TPContext(device=device)
    g = torch.Generator(device=device).manual_seed(1 + rank)
    res = {"world": world, "rows_per_rank": rows, "K": K, "N": N, "denominators": peaks["source"], "link_gbs": link_gbs}

    def report(name, ms, ms_base, flops, nvlink_bytes):
        t_c, t_l = flops / peak * 1e3, nvlink_bytes / link * 1e3
        res[name] = {"fused_ms": ms, "nccl_plus_gemm_ms": ms_base, "speedup": ms_base / ms, "compute_bound_ms": t_c,
                     "nvlink_bound_ms": t_l, "roofline_fraction": max(t_c, t_l) / ms, "tflops": flops / ms / 1e9}

    x_local = torch.randn(rows, K, device=device, generator=g).to(torch.bfloat16)
    w_col = (torch.randn(K, N // world, device=device, generator=g) * 0.02).to(torch.bfloat16)
    report("all_gather_gemm", timed(lambda: ctx.all_gather_matmul(x_local, w_col)),
           timed(lambda: all_gather_matmul_nccl(x_local, w_col)), 2.0 * rows * world * K * (N // world),
           2.0 * rows * (world - 1) * K)
    x_full = torch.randn(rows * world, K // world, device=device, generator=g).to(torch.bfloat16)
    w_row = (torch.randn(K // world, N, device=device, generator=g) * 0.02).to(torch.bfloat16)
    report("gemm_reduce_scatter", timed(lambda: ctx.matmul_reduce_scatter(x_full, w_row)),
           timed(lambda: matmul_reduce_scatter_nccl(x_full, w_row)), 2.0 * rows * world * (K // world) * N,
           2.0 * rows * (world - 1) * N)        # bf16 partials
    w_full = (torch.randn(K, N, device=device, generator=torch.Generator(device=device).manual_seed(7)) * 0.02).to(torch.bfloat16)
    sw = ShardedWeight(ctx.comm, w_full)
    del w_full

    def base():
        parts = torch.empty(world, K, N // world, device=device, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(parts, sw.shard)
        out = torch.empty(rows, N, device=device, dtype=torch.bfloat16)
        for s_ in range(world):
            gemm(x_local, parts[s_], b_mn_major=True, out=out[:, s_ * (N // world):(s_ + 1) * (N // world)])
        return out
    report("sharded_weight_gemm", timed(lambda: sw.matmul(x_local)), timed(base), 2.0 * rows * K * N,
           2.0 * K * N * (world - 1) / world)
    torch.cuda.synchronize()
    _ext.check_status(device)
    return res
