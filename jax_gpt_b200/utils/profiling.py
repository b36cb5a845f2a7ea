"""Named scopes and phase timers.

``scope(name)`` opens an NVTX range (visible to Nsight tools and ``torch.profiler``) with the
scope names the reference attaches through ``jax.named_scope`` (embedding, qkv_proj, sdpa,
moe_routing, moe_experts, deltanet_attn, gqa_attn, output_head, ...;
jax_gpt/models/qwen35/model.py:237,319, jax_gpt/models/qwen35/block.py:31-86).
``CudaTimer`` times a region with CUDA events on the current stream; multi-rank callers take
the maximum over ranks with :func:`max_over_ranks`.
"""
from __future__ import annotations

import contextlib
import os

import torch

_ENABLED = os.environ.get("B200_NVTX", "0") not in ("0", "", "false")


@contextlib.contextmanager
def scope(name: str):
    if _ENABLED and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class CudaTimer:
    """``with CudaTimer() as t: ...`` then ``t.ms`` (synchronises on exit)."""

    def __enter__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.end = torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        self.start.record()
        return self

    def __exit__(self, *exc):
        self.end.record()
        torch.cuda.synchronize()
        self.ms = self.start.elapsed_time(self.end)
        return False


def max_over_ranks(value: float, device=None) -> float:
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device or ("cuda" if torch.cuda.is_available() else "cpu"))
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


@contextlib.contextmanager
def profiler_trace(out_dir: str = ""):
    """torch.profiler trace written to ``out_dir`` (or $PROFILE_DIR); a no-op when neither is set,
    mirroring the PROFILE_DIR switch of scripts/qwen35_benchmark.py:197-207."""
    out_dir = out_dir or os.environ.get("PROFILE_DIR", "")
    if not out_dir:
        yield None
        return
    os.makedirs(out_dir, exist_ok=True)
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    with torch.profiler.profile(activities=acts) as prof:
        yield prof
    prof.export_chrome_trace(os.path.join(out_dir, "trace.json"))
