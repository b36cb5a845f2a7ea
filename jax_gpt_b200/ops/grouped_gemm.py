"""Grouped (ragged) GEMMs for MoE experts: rows are contiguous per expert.

Reference semantics: ``jax.lax.ragged_dot`` as used by jax_gpt/models/qwen35/moe.py:83-87.
On CUDA bf16 inputs the experts run on the tcgen05 GEMM kernel, one launch per non-empty
expert (the persistent fused variant lives with the expert-parallel kernels); elsewhere a
PyTorch loop over the groups.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .gemm import linear


def grouped_matmul(xs: torch.Tensor, group_sizes, w: torch.Tensor) -> torch.Tensor:
    """xs (R, K); w (E, K, N); rows of group e multiply w[e]. Returns (R, N)."""
    sizes = group_sizes.tolist() if torch.is_tensor(group_sizes) else list(group_sizes)
    out = xs.new_empty(xs.shape[0], w.shape[2])
    s = 0
    for e, n in enumerate(sizes):
        if n:
            out[s:s + n] = linear(xs[s:s + n], w[e])
        s += n
    return out


def grouped_swiglu(xs, group_sizes, gate_w, up_w, down_w) -> torch.Tensor:
    """``down_e(silu(x @ gate_e) * (x @ up_e))`` per group."""
    g = grouped_matmul(xs, group_sizes, gate_w)
    u = grouped_matmul(xs, group_sizes, up_w)
    return grouped_matmul(F.silu(g) * u, group_sizes, down_w)
