"""Grouped (ragged) GEMMs for MoE experts: rows are contiguous per expert.

Reference semantics: ``jax.lax.ragged_dot`` as used by jax_gpt/models/qwen35/moe.py:83-87.
This is the FALLBACK of the single-device MoE path, taken when the fused expert kernels' shape guards fail (the
persistent fused dispatch / grouped GEMM / combine kernels live in csrc/moe_kernels.cu): with device-side group
sizes one library grouped GEMM (no host read-back), otherwise a loop of GEMMs over the groups.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .gemm import linear


class _ContiguousGrad(torch.autograd.Function):
    """Identity whose backward makes the incoming gradient contiguous (the library grouped GEMM's backward rejects
    expanded, stride-0 gradients such as the one ``sum()`` produces)."""

    @staticmethod
    def forward(ctx, x):
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g.contiguous()


def grouped_matmul(xs: torch.Tensor, group_sizes, w: torch.Tensor) -> torch.Tensor:
    """xs (R, K); w (E, K, N); rows of group e multiply w[e]. Returns (R, N). With the group sizes in a device tensor
    and bf16 operands whose widths are multiples of 8, the groups run as ONE library grouped GEMM addressed by the
    cumulative sizes, so nothing is read back to the host; otherwise one GEMM per non-empty group."""
    if (torch.is_tensor(group_sizes) and xs.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and xs.shape[1] % 8 == 0
            and w.shape[2] % 8 == 0 and hasattr(torch, "_grouped_mm") and (xs.is_cuda or not xs.requires_grad)):
        offs = group_sizes.to(device=xs.device).cumsum(0).to(torch.int32)
        return _ContiguousGrad.apply(torch._grouped_mm(xs.contiguous(), w.contiguous(), offs=offs))
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
