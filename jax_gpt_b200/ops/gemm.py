"""GEMM entry points: the tcgen05 kernel on CUDA tensors, an fp32 PyTorch reference elsewhere.

``gemm`` computes ``out[M,N] = epilogue(alpha * A @ B^T)`` where A is logically [M,K] and B is
logically [N,K]; either may be stored transposed ("MN-major": A as [K,M], B as [K,N]), which
is how forward ``x @ W`` with (in,out) kernels, dgrad ``dy @ W^T`` and wgrad ``x^T @ dy`` all
run without a transpose in memory. Linear kernels keep the reference's (in,out) orientation
(jax_gpt/models/gpt2/model.py:80-90, jax_gpt/models/qwen35/model.py:25-36).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _ext

EPI_NONE, EPI_GELU, EPI_GELU_GRAD = 0, 1, 2
OUT_BF16, OUT_F32, OUT_F32_ATOMIC = 0, 1, 2


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.gelu(x, approximate="tanh")


def gelu_tanh_grad(x: torch.Tensor) -> torch.Tensor:
    k0, k1 = 0.7978845608028654, 0.044715
    u = k0 * (x + k1 * x ** 3)
    t = torch.tanh(u)
    return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * k0 * (1 + 3 * k1 * x * x)


def gemm_ref(a, b, *, a_mn_major=False, b_mn_major=False, out=None, bias=None, residual=None, aux=None,
             epilogue=EPI_NONE, out_mode=OUT_BF16, alpha=1.0, split_k=1):
    """fp32 reference of :func:`gemm` with identical argument conventions."""
    A = a.float().t() if a_mn_major else a.float()
    Bm = b.float() if b_mn_major else b.float().t()
    acc = alpha * (A @ Bm)
    if bias is not None:
        acc = acc + bias.float()
    if epilogue == EPI_GELU:
        pre = acc.to(torch.bfloat16)
        if aux is not None:
            aux.copy_(pre)
        acc = gelu_tanh(pre.float())
    elif epilogue == EPI_GELU_GRAD:
        acc = acc * gelu_tanh_grad(aux.float())
    if residual is not None:
        acc = acc + residual.float()
    if out is None:
        return acc.to(torch.bfloat16 if out_mode == OUT_BF16 else torch.float32)
    if out_mode == OUT_F32_ATOMIC:
        out.add_(acc.to(out.dtype))
    else:
        out.copy_(acc.to(out.dtype))
    return out


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn_major: bool = False, b_mn_major: bool = False,
         out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, aux: Optional[torch.Tensor] = None, epilogue: int = EPI_NONE,
         out_mode: int = OUT_BF16, alpha: float = 1.0, split_k: int = 1) -> torch.Tensor:
    """See module docstring. ``out_mode=OUT_F32_ATOMIC`` accumulates into ``out`` (fp32)."""
    if not a.is_cuda:
        return gemm_ref(a, b, a_mn_major=a_mn_major, b_mn_major=b_mn_major, out=out, bias=bias, residual=residual,
                        aux=aux, epilogue=epilogue, out_mode=out_mode, alpha=alpha, split_k=split_k)
    M = a.shape[1] if a_mn_major else a.shape[0]
    N = b.shape[1] if b_mn_major else b.shape[0]
    if out is None:
        if out_mode == OUT_F32_ATOMIC:
            out = torch.zeros(M, N, device=a.device, dtype=torch.float32)
        else:
            out = torch.empty(M, N, device=a.device, dtype=torch.bfloat16 if out_mode == OUT_BF16 else torch.float32)
    _ext.ops().gemm(a, a_mn_major, b, b_mn_major, out, bias, residual, aux, epilogue, out_mode, alpha, split_k)
    return out


def _weight_grad(x2, dy2, w):
    """dW = x^T dy on the split-K GEMM. A weight that carries a ``grad_buf`` attribute (an fp32 tensor of its shape:
    the trainer's flat gradient buffer) gets the product ACCUMULATED there by the GEMM's own epilogue and no
    autograd gradient, which saves the bf16 round trip and the separate accumulation pass."""
    split = max(1, min(16, x2.shape[0] // 2048))
    buf = getattr(w, "grad_buf", None)
    if buf is not None and buf.dtype == torch.float32 and buf.shape == w.shape and buf.is_contiguous():
        gemm(x2, dy2, a_mn_major=True, b_mn_major=True, out=buf, out_mode=OUT_F32_ATOMIC, split_k=split)
        return None
    return gemm(x2, dy2, a_mn_major=True, b_mn_major=True, out_mode=OUT_F32_ATOMIC, split_k=split).to(w.dtype)


class _LinearF32OutFn(torch.autograd.Function):
    """y = x @ W with bf16 operands and an fp32 result (router logits: the products are exact, the sum is fp32,
    which is what an fp32 GEMM on the upcast operands computes)."""

    @staticmethod
    def forward(ctx, x, w):
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm(x2, w, b_mn_major=True, out_mode=OUT_F32)
        ctx.save_for_backward(x2, w)
        ctx.xshape = x.shape
        return y.reshape(*x.shape[:-1], w.shape[1])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).to(torch.bfloat16).contiguous()
        dx = gemm(dy2, w).reshape(ctx.xshape) if ctx.needs_input_grad[0] else None
        dw = _weight_grad(x2, dy2, w) if ctx.needs_input_grad[1] else None
        return dx, dw


def linear_f32out(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w`` as fp32, ``w`` of shape (in, out). CUDA bf16 operands with row strides the TMA accepts (both widths
    multiples of 8) run on the tcgen05 GEMM; anything else is computed in fp32 by PyTorch."""
    if (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0
            and w.shape[0] % 8 == 0 and w.is_contiguous()):
        return _LinearF32OutFn.apply(x, w)
    return x.float() @ w.float()


class _LinearFn(torch.autograd.Function):
    """y = x @ W (+ b) with W stored (in,out); bf16 compute, fp32 parameter gradients."""

    @staticmethod
    def forward(ctx, x, w, bias):
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm(x2, w, b_mn_major=True, bias=bias)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.xshape = x.shape
        return y.reshape(*x.shape[:-1], w.shape[1])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = gemm(dy2, w).reshape(ctx.xshape) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            dw = _weight_grad(x2, dy2, w)
        db = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            from .misc import bias_grad
            db = bias_grad(dy2).to(w.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w + bias`` with ``w`` of shape (in, out). CUDA bf16 tensors run on the tcgen05 GEMM; inside
    ``ops.fp8_linear.fp8_training()`` eligible layers run their three GEMMs in block-scaled FP8."""
    from . import fp8_linear as F8
    if F8.fp8_enabled() and F8.fp8_eligible(x, w):
        return F8.fp8_linear(x, w, bias)
    if x.is_cuda and x.dtype == torch.bfloat16:
        return _LinearFn.apply(x, w, bias)
    y = x @ w
    return y + bias if bias is not None else y
