"""Block-scaled FP8 TRAINING path for linear layers: forward, input gradient and weight gradient all run as
e4m3 GEMMs whose 1x128 / 128x128 power-of-two block scales are applied by the tensor core
(``tcgen05.mma.kind::mxf8f6f4.block_scale``, see csrc/gemm_mxfp8_sm100.cu); master weights, the optimizer and
everything between the GEMMs stay in bf16 / fp32.

    forward   y  = x  @ W        x  [M, in]   1x128 blocks along in     W^T [out, in] 128x128 blocks
    dgrad     dx = dy @ W^T      dy [M, out]  1x128 blocks along out    W   [in, out] 128x128 blocks (same blocks)
    wgrad     dW^T = dy^T @ x    dy^T [out, M] 1x128 blocks along M     x^T [in, M]   128x128 blocks

Every operand is produced by ONE kernel (csrc/seq_kernels.cu:fp8_quant_mx_kernel) that reads a 128 x 128 bf16 tile,
optionally transposes it through shared memory (the weight-gradient operands need the token dimension
contiguous), quantises it and writes the e4m3 bytes plus the exponent bytes in the packed layout the GEMM copies
into tensor memory. The weight gradient leaves the GEMM in bf16.

Use: ``with fp8_training(): loss = loss_fn(...)`` makes ``ops.gemm.linear`` take this path for every weight whose
dimensions and token count are multiples of 128; other calls keep the bf16 kernel.

The reference only has per-row W8A8 *inference* (jax_gpt/models/qwen35/fp8.py:50-150, quantize.py); the
block-scaled training recipe is the DeepSeek-V3 one.
"""
from __future__ import annotations

import contextlib
from typing import Optional

import torch

from .fp8 import fp8_gemm_ref, fp8_quant_mx, mxfp8_gemm_packed

_STATE = {"on": False}


@contextlib.contextmanager
def fp8_training(enabled: bool = True):
    """Inside the block eligible ``linear`` calls run forward and backward in block-scaled FP8."""
    old = _STATE["on"]
    _STATE["on"] = bool(enabled)
    try:
        yield
    finally:
        _STATE["on"] = old


def fp8_enabled() -> bool:
    return _STATE["on"]


def fp8_eligible(x: torch.Tensor, w: torch.Tensor) -> bool:
    if w.dim() != 2 or x.shape[-1] != w.shape[0]:
        return False
    tokens = x.numel() // max(1, x.shape[-1])
    return tokens % 128 == 0 and tokens > 0 and w.shape[0] % 128 == 0 and w.shape[1] % 128 == 0


def _quant(x: torch.Tensor, transpose: bool, block: bool):
    """(q, scales in the form :func:`_mm` wants on x's device): one kernel on CUDA (quantise, transpose and pack
    the exponent bytes), the reference functions elsewhere."""
    q, sf, sc = fp8_quant_mx(x, transpose, block)
    return (q, sf) if x.is_cuda else (q, sc)


def _mm(a, b):
    """a = (q [M,K], scales 1x128), b = (q [N,K], scales 128x128) -> bf16 [M,N]."""
    if a[0].is_cuda:
        return mxfp8_gemm_packed(a[0], a[1], b[0], b[1])
    return fp8_gemm_ref(a[0], a[1], b[0], b[1]).to(torch.bfloat16)


class _Fp8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        K, N = w.shape
        x2 = x.reshape(-1, K).to(torch.bfloat16).contiguous()
        wb = w.detach().to(torch.bfloat16).contiguous()
        y = _mm(_quant(x2, False, False), _quant(wb, True, True))            # x [M,in] x (W^T [out,in])^T
        if bias is not None:
            y = y + bias.to(y.dtype)
        ctx.save_for_backward(x2, wb)
        ctx.has_bias = bias is not None
        ctx.xshape, ctx.x_dtype, ctx.w_dtype = x.shape, x.dtype, w.dtype
        return y.to(x.dtype).reshape(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        x2, wb = ctx.saved_tensors
        N = wb.shape[1]
        dy2 = dy.reshape(-1, N).to(torch.bfloat16).contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = _mm(_quant(dy2, False, False), _quant(wb, False, True))       # dy [M,out] x (W [in,out])^T
            dx = dx.to(ctx.x_dtype).reshape(ctx.xshape)
        if ctx.needs_input_grad[1]:
            dwt = _mm(_quant(dy2, True, False), _quant(x2, True, True))        # dy^T [out,M] x (x^T [in,M])^T
            dw = dwt.t().to(ctx.w_dtype)                                       # [out,in] -> (in,out)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(ctx.w_dtype)
        return dx, dw, db


def fp8_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w + bias`` (w of shape (in, out)) with the three GEMMs of the layer in block-scaled FP8."""
    assert fp8_eligible(x, w), "fp8_linear: token count and both weight dimensions must be multiples of 128"
    return _Fp8LinearFn.apply(x, w, bias)
