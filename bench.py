"""Headline benchmark: GPT-2 small training throughput (tokens/s) on N B200s of one node.

    python bench.py --gpus N --steps K --warmup W        # this framework
    python bench.py --impl reference ...                 # the unmodified reference, if it can run

Prints ONE JSON line on rank 0. `value` is the whole-job tokens/s of the device-timed step
loop (CUDA events, max over ranks); `e2e` is the same metric through the public trainer API
(`jax_gpt_b200.trainer.train_step`) including, every step, the host->device copy of that
step's tokens from pinned memory and a device->host read of the loss.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

BASELINE_TOKENS_PER_S = None  # the reference publishes no training throughput


def reference_arm(args):
    """Runs the UNMODIFIED reference from baseline/_ref through its own public API: ``GPT``, ``create_optimizer``,
    ``create_train_state`` and ``train_step`` (jax_gpt/trainer/train_step.py:34-76), the step wrapped in ``nnx.jit``
    as that file's header prescribes, on the same model, batch shape, step and warm-up counts as the b200 arm, and
    prints the same JSON line with ``"impl": "reference"``. The reference imports jax / flax / optax at module
    load; where they are missing (no wheel in the offline image) it cannot run and says so."""
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(here, "baseline", "_ref"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))

    def unavailable(why):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    try:
        import jax
        import jax.numpy as jnp
        import numpy as np
        from flax import nnx
        from jax_gpt.models.gpt2.config import GPTConfig
        from jax_gpt.models.gpt2.model import GPT
        from jax_gpt.trainer.config import TrainConfig
        from jax_gpt.trainer.optimizer import create_optimizer
        from jax_gpt.trainer.train_state import TrainState, create_train_state
        from jax_gpt.trainer.train_step import train_step as ref_train_step
    except Exception as e:  # pragma: no cover - depends on the image
        return unavailable(f"reference needs jax/flax/optax, not installed and no wheel offline ({type(e).__name__}: {e})")
    if world > 1:
        # its train_step has no data-parallel path: batches are never placed with a dp spec and gradients are not
        # reduced across processes (jax_gpt/trainer/sharding.py annotates tensor-parallel specs only)
        return unavailable("the reference's train_step has no multi-process data-parallel path (no gradient reduction "
                           "across processes); it is measured on one GPU only")
    try:
        if not any(d.platform == "gpu" for d in jax.devices()):
            return unavailable(f"jax has no GPU backend here (devices: {[d.platform for d in jax.devices()]})")
        cfg = GPTConfig.from_model_type(args.model)
        B, T = args.micro_batch, args.seq_len
        tc = TrainConfig(micro_batch_size=B, seq_len=T)
        model = GPT(cfg, rngs=nnx.Rngs(0))
        tx = create_optimizer(model, tc)
        state = create_train_state(model, tx)

        @nnx.jit
        def step_fn(model, opt_state, x, y):
            st, metrics = ref_train_step(TrainState(step=0, model=model, tx=tx, opt_state=opt_state), (x, y))
            return st.opt_state, metrics

        rng = np.random.default_rng(1234)
        n = args.steps + args.warmup
        host = [rng.integers(0, cfg.vocab_size, (B, T + 1), dtype=np.int32) for _ in range(n)]
        dev = [(jnp.asarray(h[:, :-1]), jnp.asarray(h[:, 1:])) for h in host]
        opt_state = state.opt_state
        for i in range(args.warmup):
            opt_state, m = step_fn(model, opt_state, *dev[i])
        jax.block_until_ready(m["loss"])
        t0 = time.perf_counter()
        for i in range(args.steps):
            opt_state, m = step_fn(model, opt_state, *dev[args.warmup + i])
        jax.block_until_ready(m["loss"])
        ms = (time.perf_counter() - t0) * 1e3
        final_loss = float(m["loss"])
        # end to end: host arrays in, loss read back, every step
        t0 = time.perf_counter()
        for i in range(args.steps):
            h = host[args.warmup + i]
            opt_state, m = step_fn(model, opt_state, jnp.asarray(h[:, :-1]), jnp.asarray(h[:, 1:]))
            loss_host = float(m["loss"])
        e2e_ms = (time.perf_counter() - t0) * 1e3
        tokens = B * T * args.steps
        print(json.dumps({
            "impl": "reference", "metric": "train tokens/s/box", "value": tokens / (ms / 1e3), "unit": "tokens/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp32 parameters and activations (the reference never consumes its dtype field)",
            "data": "synthetic uniform-random token ids, random-init weights",
            "config": {"model": "GPT-2 small (12L, d768, 12 heads, ctx 1024, vocab 50257, tied embeddings)",
                       "global_batch": B, "seq_len": T, "parallelism": "1gpu",
                       "step": "jax_gpt.trainer.train_step under nnx.jit (XLA:GPU)", "timing": "host clock around block_until_ready"},
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": 2 * B * T * 4, "d2h_bytes_per_step": 4},
            "final_loss": final_loss, "e2e_final_loss": loss_host}))
    except Exception as e:  # pragma: no cover - needs a jax install to exercise
        return unavailable(f"reference runner failed: {type(e).__name__}: {str(e)[:300]}")
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "200"], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # samples under load = the upper half of the observed clocks' time line with power above idle
        busy = [c for c, p in zip(sm, power) if p > 250] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "power_w_max": max(power) if power else None}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--model", default="gpt2")
    ap.add_argument("--micro-batch", type=int, default=16)
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--overlap", action="store_true", help="several GPUs: reduce-scatter each layer's gradients during backward")
    ap.add_argument("--multimem", action="store_true",
                    help="several GPUs: the optimizer kernel reduces and broadcasts through NVSwitch multicast (multimem.ld_reduce / "
                         "multimem.st) instead of peer loads and stores")
    ap.add_argument("--no-extra", action="store_true",
                    help="2+ GPUs: skip the expert-parallel extras (fused EP-MoE layer, Qwen3.5-style MoE training step)")
    ap.add_argument("--extra-budget-s", type=float, default=420.0, help="wall-clock limit of the extras; past it the line is printed without them")
    ap.add_argument("--extras-child", default="", help=argparse.SUPPRESS)   # internal: run only the extras, write them to this file
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.extras_child:
        return extras_child(args.extras_child)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus and world > 1:
        args.gpus = world
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    from jax_gpt_b200 import _ext
    from jax_gpt_b200.models.gpt2 import GPT, GPTConfig
    from jax_gpt_b200.trainer import TrainConfig, create_optimizer, create_train_state, train_step

    cfg = GPTConfig.from_model_type(args.model)
    B, T = args.micro_batch, args.seq_len
    tc = TrainConfig(micro_batch_size=B, seq_len=T, dp=world, cuda_graph=not args.no_graph,
                     overlap_grad_reduce=args.overlap)
    model = GPT(cfg, seed=0)
    dist_opt = None
    if world > 1:
        from jax_gpt_b200.parallel.fsdp import FusedShardedAdamW
        dist_opt = FusedShardedAdamW(dist.group.WORLD, device, use_multimem=args.multimem)
    state = create_train_state(model, create_optimizer(model, tc), train_config=tc, device=device,
                               dist_optimizer=dist_opt)
    eng = state.engine

    # synthetic uniform-random token ids, a different pinned host batch for every step
    gen = torch.Generator().manual_seed(1234 + rank)
    n_batches = args.steps + args.warmup
    host = [torch.randint(0, cfg.vocab_size, (B, T + 1), generator=gen, dtype=torch.int32) for _ in range(n_batches)]
    host_x = [h[:, :-1].contiguous().pin_memory() for h in host]
    host_y = [h[:, 1:].contiguous().pin_memory() for h in host]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed loop: the fused step on device-resident batches -------------------------
    dev_x = [x.to(device) for x in host_x]
    dev_y = [y.to(device) for y in host_y]
    for i in range(args.warmup):
        eng.train_step(dev_x[i], dev_y[i])
    barrier()
    _ext.check_status(device)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for i in range(args.steps):
        eng.train_step(dev_x[args.warmup + i], dev_y[args.warmup + i])
    t1.record()
    barrier()
    ms = t0.elapsed_time(t1)
    clocks = sampler.stop() if rank == 0 else None
    _ext.check_status(device)
    final_loss = float(eng.last_loss)

    # ---- end-to-end loop through the public trainer API ---------------------------------------
    for i in range(min(3, args.warmup)):
        state, m = train_step(state, (host_x[i], host_y[i]))
        float(m["loss"])
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    wall0 = time.perf_counter()
    for i in range(args.steps):
        state, m = train_step(state, (host_x[args.warmup + i], host_y[args.warmup + i]))
        loss_host = float(m["loss"])  # device -> host read every step
    e1.record()
    barrier()
    e2e_ms = max(e0.elapsed_time(e1), (time.perf_counter() - wall0) * 1e3)

    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()
    tokens_per_step = B * T * world
    value = tokens_per_step * args.steps / (ms / 1e3)
    e2e_value = tokens_per_step * args.steps / (e2e_ms / 1e3)
    launches = eng.kernel_launches_per_step() * args.steps
    out = None
    if rank == 0:
        out = {
            "metric": "train tokens/s/box", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None, "dtype": "bf16",
            "data": "synthetic uniform-random token ids, random-init weights",
            "config": {"model": "GPT-2 small (12L, d768, 12 heads, ctx 1024, vocab 50257, tied embeddings)",
                       "global_batch": B * world, "seq_len": T, "parallelism": f"dp{world}" if world > 1 else "1gpu",
                       "optimizer": "AdamW + global-norm clip, fp32 master weights, inside the timed step",
                       "l2": "per-step working set (~7 GB of activations and logits) exceeds the 126 MB L2; no flush",
                       "cuda_graph": not args.no_graph,
                       "grad_reduce": ("per-layer reduce-scatter kernels on a side stream during backward" if world > 1 and args.overlap
                                       else (("inside the fused optimizer kernel after backward" + (" (multimem)" if args.multimem else "")) if world > 1 else "none (1 GPU)"))},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": 2 * B * T * 4, "d2h_bytes_per_step": 4,
                    "api": "jax_gpt_b200.trainer.train_step(state, (x, y))"},
            "gpu_launches": launches,
            "final_loss": final_loss, "e2e_final_loss": loss_host, "impl": "b200",
        }
    if world >= 2 and not args.no_extra:
        # The all-to-all paths on the same GPUs: the fused EP-MoE layer of the DeepSeek-V3 shape and a training step
        # of the Qwen3.5-style hybrid MoE at the depth that fits N GPUs. They run in CHILD processes (one per rank, a
        # process group of their own), so that nothing that happens there (an error, a fault, an overrun) can cost
        # the headline line: the parent only waits, with a time limit, and reads the child's result file.
        import tempfile
        del state, eng, model, dev_x, dev_y, dist_opt
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        dist.barrier()
        dist.destroy_process_group()
        path = os.path.join(tempfile.gettempdir(), f"b200_bench_extras_{os.environ.get('MASTER_PORT', '0')}.json")
        if rank == 0 and os.path.exists(path):
            os.remove(path)
        # a rendezvous of the children's own: another port, and rank 0 hosts the store itself (under torchrun the
        # workers are clients of the agent's store, which only exists on the original port)
        env = dict(os.environ, MASTER_PORT=str(int(os.environ.get("MASTER_PORT", "29500")) + 17),
                   TORCHELASTIC_USE_AGENT_STORE="False")
        err = None
        try:
            r = subprocess.run([sys.executable, os.path.abspath(__file__), "--extras-child", path, "--gpus", str(world)],
                               env=env, timeout=args.extra_budget_s, capture_output=True, text=True)
            if r.returncode != 0:
                err = f"extras exited with code {r.returncode}: {(r.stderr or '')[-300:]}"
        except subprocess.TimeoutExpired:
            err = f"extras exceeded {args.extra_budget_s:.0f} s and were stopped"
        if rank == 0:
            try:
                with open(path) as f:
                    out["extra"] = json.load(f)
            except Exception:
                out["extra"] = {"error": err or "the extras left no result"}
        print(json.dumps(out), flush=True) if rank == 0 else None
        return 0
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def extras_child(path: str) -> int:
    """Child process of one rank: own process group, the extras, rank 0 writes them to ``path``."""
    import torch
    import torch.distributed as dist
    rank, local_rank, world = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1")))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=device)
    extra = run_extras(device, rank, world, dist)
    if rank == 0:
        with open(path + ".tmp", "w") as f:
            json.dump(extra, f)
        os.replace(path + ".tmp", path)
    dist.barrier()
    dist.destroy_process_group()
    return 0


def run_extras(device, rank, world, dist):
    """{"ep_moe_layer": ..., "qwen35_moe_train": ...}; a failed part carries {"error": ...} and the ranks agree on it."""
    import torch
    from jax_gpt_b200.utils.bench_extras import ep_moe_layer_bench, moe_train_bench, tp_fused_gemm_bench
    extra = {}

    def guarded(name, fn):
        import gc
        err = None
        try:
            res = fn()
        except Exception as e:  # out of memory, a kernel status error ...
            res, err = None, f"{type(e).__name__}: {str(e)[:200]}"
        # the parts are sized to fill a GPU: drop what the last one still holds (engines sit in reference cycles;
        # symmetric buffers are freed with their owners) before the next one allocates
        gc.collect()
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        flag = torch.tensor([0 if err is None else 1], device=device)
        dist.all_reduce(flag)
        if int(flag) > 0:
            extra[name] = {"error": err or "failed on another rank"}
            return False
        extra[name] = res
        return True

    # BASELINE config 1: 4096 tokens per rank, N(0,1) router, forward + backward in bf16, FP8 forward
    guarded("ep_moe_layer", lambda: ep_moe_layer_bench(device, rank, world, tokens=4096, router="normal", backward=True,
                                                        fp8=True, warmup=2, iters=4))
    # BASELINE config 2 shape at the depth that fits: 512 experts of inter 512, top-10, seq 4096, global batch 32
    depth = {2: 8, 4: 24}.get(world, 48 if world >= 8 else 4)
    guarded("qwen35_moe_train", lambda: moe_train_bench(device, rank, world, model="qwen35", layers=depth, experts=512,
                                                         seq=4096, batch=1, accum=max(1, 32 // world), lowmem=True,
                                                         steps=2, warmup=1))
    # the fused collective + GEMM kernels (all-gather -> GEMM, GEMM -> reduce-scatter, FSDP weight gather -> GEMM)
    # against NCCL + GEMM on the MLA output-projection shape, with their roofline fractions
    guarded("tp_fused_gemms", lambda: tp_fused_gemm_bench(device, rank, world, rows=4096, K=7168, N=16384, warmup=2, iters=5))
    # BASELINE config 3 at the depth that fits: DeepSeek-V3 widths, 256 experts, seq 4096, global batch 32, FP8 dense GEMMs
    ds_depth = {2: 2, 4: 4}.get(world, 8 if world >= 8 else 2)
    guarded("deepseek_v3_train", lambda: moe_train_bench(device, rank, world, model="deepseek_v3", layers=ds_depth,
                                                          experts=256, seq=4096, batch=1, accum=max(1, 32 // world),
                                                          fp8=True, lowmem=True, steps=2, warmup=1))
    return extra


if __name__ == "__main__":
    sys.exit(main())
