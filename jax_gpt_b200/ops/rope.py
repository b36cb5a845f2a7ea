"""Fused per-head RMSNorm + partial rotary embedding (kernels of csrc/seq_kernels.cu).

PyTorch references: ``rms_norm`` / ``apply_rotary_emb`` of models/qwen35/primitives.py (the
semantics of jax_gpt/models/qwen35/primitives.py:29-32,79-109).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _ext



def rmsnorm_rope_ref(x, norm_w, freqs, rope_dim: int, pos0: int = 0, eps: float = 1e-6, one_plus: bool = True):
    """x (B,T,H,dh); freqs (n_pos, rope_dim/2, 2)."""
    from ..models.qwen35.primitives import apply_rotary_emb
    xf = x.float()
    if norm_w is not None:
        xf = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * ((1.0 + norm_w.float()) if one_plus else norm_w.float())
    if rope_dim:
        xf = apply_rotary_emb(xf, freqs[pos0:pos0 + x.shape[1]], rope_dim)
    return xf.to(x.dtype)


class _RmsnormRopeFn(torch.autograd.Function):
    """Forward and backward on the fused kernels (per-head RMSNorm with (1 + w) or w gain, partial half-split rotary)."""

    @staticmethod
    def forward(ctx, x, norm_w, freqs, rope_dim, pos0, eps, one_plus):
        B, T, H, dh = x.shape
        xc = x.contiguous().view(B * T, H, dh)
        y = torch.empty_like(xc)
        fr = freqs.contiguous() if freqs is not None else None
        _ext.ops().rmsnorm_rope(xc, norm_w, fr, y, T, rope_dim, pos0, eps, one_plus)
        ctx.save_for_backward(xc, norm_w, fr)
        ctx.meta = (B, T, H, dh, rope_dim, pos0, eps, one_plus)
        return y.view(B, T, H, dh)

    @staticmethod
    def backward(ctx, dy):
        xc, norm_w, fr = ctx.saved_tensors
        B, T, H, dh, rope_dim, pos0, eps, one_plus = ctx.meta
        dyc = dy.contiguous().view(B * T, H, dh)
        dx = torch.empty_like(xc)
        dw = torch.zeros(dh, device=xc.device, dtype=torch.float32) if norm_w is not None else None
        _ext.ops().rmsnorm_rope_bwd(xc, dyc, norm_w, fr, dx, dw, T, rope_dim, pos0, eps, one_plus)
        return dx.view(B, T, H, dh), (dw.to(norm_w.dtype) if dw is not None else None), None, None, None, None, None


def rmsnorm_rope(x, norm_w, freqs, rope_dim: int, pos0: int = 0, eps: float = 1e-6, one_plus: bool = True):
    B, T, H, dh = x.shape
    per = dh // 32 if dh % 32 == 0 else 0
    ok = (x.is_cuda and x.dtype == torch.bfloat16 and per and dh <= 256 and
          (rope_dim == 0 or ((rope_dim // 2) % per == 0)))
    if not ok or (norm_w is not None and norm_w.dtype != torch.bfloat16):
        return rmsnorm_rope_ref(x, norm_w, freqs, rope_dim, pos0, eps, one_plus)
    if torch.is_grad_enabled() and (x.requires_grad or (norm_w is not None and norm_w.requires_grad)):
        return _RmsnormRopeFn.apply(x, norm_w, freqs, rope_dim, pos0, eps, one_plus)
    xc = x.contiguous().view(B * T, H, dh)
    y = torch.empty_like(xc)
    _ext.ops().rmsnorm_rope(xc, norm_w, freqs.contiguous() if freqs is not None else None, y, T, rope_dim, pos0, eps, one_plus)
    return y.view(B, T, H, dh)
