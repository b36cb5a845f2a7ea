"""LayerNorm / RMSNorm: fused CUDA kernels with an fp32 PyTorch reference.

Conventions of the reference: LayerNorm eps 1e-5 with scale and bias
(jax_gpt/models/gpt2/model.py:60-65); RMSNorm in fp32, ``x / sqrt(mean(x^2) + eps) * (1 + w)``
(jax_gpt/models/qwen35/primitives.py:29-32); DeepSeek-style RMSNorm multiplies by ``w`` directly.
"""
from __future__ import annotations

import torch

from .. import _ext

LAYERNORM, RMSNORM, RMSNORM_1P = 0, 1, 2


def norm_ref(mode: int, x: torch.Tensor, gamma: torch.Tensor, beta=None, eps: float = 1e-5) -> torch.Tensor:
    xf = x.float()
    if mode == LAYERNORM:
        mu = xf.mean(-1, keepdim=True)
        var = ((xf - mu) ** 2).mean(-1, keepdim=True)
        y = (xf - mu) * torch.rsqrt(var + eps) * gamma.float()
        if beta is not None:
            y = y + beta.float()
    else:
        y = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps)
        y = y * (gamma.float() if mode == RMSNORM else (1.0 + gamma.float()))
    return y.to(x.dtype)


def norm_fwd(mode, x, gamma, beta, eps, y=None, mean=None, rstd=None):
    """Raw CUDA forward; returns (y, mean, rstd) with the statistics needed by backward."""
    M = x.numel() // x.shape[-1]
    if y is None:
        y = torch.empty_like(x)
    if rstd is None:
        rstd = torch.empty(M, device=x.device, dtype=torch.float32)
    if mean is None and mode == LAYERNORM:
        mean = torch.empty(M, device=x.device, dtype=torch.float32)
    _ext.ops().norm_fwd(mode, x, gamma, beta, y, mean, rstd, eps)
    return y, mean, rstd


_SCRATCH = {}


def bwd_scratch(device, D: int) -> torch.Tensor:
    """Per-device scratch for the partial dgamma/dbeta sums of the backward kernel."""
    n = int(_ext.ops().norm_bwd_scratch_floats(D))   # per-block partial rows; the library knows its grid cap
    key = (torch.device(device).index, n)
    t = _SCRATCH.get(key)
    if t is None:
        t = torch.empty(n, device=device, dtype=torch.float32)
        _SCRATCH[key] = t
    return t


def norm_bwd(mode, dy, x, gamma, mean, rstd, dgamma, dbeta, dres=None, dx=None, scratch=None):
    """Raw CUDA backward; ACCUMULATES into fp32 ``dgamma`` / ``dbeta``; adds ``dres`` to dx.
    ``scratch`` (see :func:`bwd_scratch`) holds per-block partial sums between the two kernels."""
    if dx is None:
        dx = torch.empty_like(x)
    if scratch is None:
        scratch = bwd_scratch(x.device, x.shape[-1])
    _ext.ops().norm_bwd(mode, dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, scratch)
    return dx


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, mode, eps):
        xc = x.contiguous()
        y, mean, rstd = norm_fwd(mode, xc, gamma, beta, eps)
        ctx.save_for_backward(xc, gamma, mean if mean is not None else rstd, rstd)
        ctx.mode = mode
        ctx.has_beta = beta is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gamma, mean, rstd = ctx.saved_tensors
        dgamma = torch.zeros(gamma.shape, device=x.device, dtype=torch.float32)
        dbeta = torch.zeros(gamma.shape, device=x.device, dtype=torch.float32) if ctx.has_beta else None
        dx = norm_bwd(ctx.mode, dy.contiguous(), x, gamma, mean if ctx.mode == LAYERNORM else None, rstd, dgamma, dbeta)
        return dx, dgamma.to(gamma.dtype), (dbeta.to(gamma.dtype) if ctx.has_beta else None), None, None


def layer_norm(x, gamma, beta, eps: float = 1e-5):
    if x.is_cuda and x.dtype == torch.bfloat16:
        return _NormFn.apply(x, gamma, beta, LAYERNORM, eps)
    return norm_ref(LAYERNORM, x, gamma, beta, eps)


def rms_norm(x, w, eps: float = 1e-6, one_plus_w: bool = True):
    """RMSNorm; ``one_plus_w=True`` is the Qwen3.5 convention, ``False`` the DeepSeek one."""
    mode = RMSNORM_1P if one_plus_w else RMSNORM
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return _NormFn.apply(x, w, None, mode, eps)
    return norm_ref(mode, x, w, None, eps)
