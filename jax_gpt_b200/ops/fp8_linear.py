"""Block-scaled FP8 TRAINING path for linear layers: forward, input gradient and weight gradient all run as
e4m3 GEMMs whose 1x128 / 128x128 power-of-two block scales are applied by the tensor core
(``tcgen05.mma.kind::mxf8f6f4.block_scale``, see csrc/gemm_mxfp8_sm100.cu); master weights, the optimizer and
everything between the GEMMs stay in bf16 / fp32.

    forward   y  = x  @ W        x  [M, in]   1x128 blocks along in     W^T [out, in] 128x128 blocks
    dgrad     dx = dy @ W^T      dy [M, out]  1x128 blocks along out    W   [in, out] 128x128 blocks (same blocks)
    wgrad     dW^T = dy^T @ x    dy^T [out, M] 1x128 blocks along M     x^T [in, M]   128x128 blocks

The weight is quantised once per step (its [in, out] block scales serve the forward through a transposed copy of
the e4m3 bytes); activations and gradients are quantised per call, the weight-gradient operands after a
transposing copy so that the token dimension is the contiguous one. The weight gradient leaves the GEMM in bf16.

Use: ``with fp8_training(): loss = loss_fn(...)`` makes ``ops.gemm.linear`` take this path for every weight whose
dimensions and token count are multiples of 128; other calls keep the bf16 kernel.

The reference only has per-row W8A8 *inference* (jax_gpt/models/qwen35/fp8.py:50-150, quantize.py); the
block-scaled training recipe is the DeepSeek-V3 one.
"""
from __future__ import annotations

import contextlib
from typing import Optional

import torch

from .rope import fp8_quant_1x128, fp8_quant_128x128, mxfp8_gemm

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


def _t8(q: torch.Tensor) -> torch.Tensor:
    """Transposed contiguous copy of an e4m3 matrix (moved as bytes)."""
    return q.view(torch.uint8).t().contiguous().view(torch.float8_e4m3fn)


class _Fp8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        K, N = w.shape
        x2 = x.reshape(-1, K).to(torch.bfloat16).contiguous()
        xq, xs = fp8_quant_1x128(x2, True)
        wq, ws = fp8_quant_128x128(w.detach().to(torch.bfloat16).contiguous(), True)     # blocks of W [in, out]
        y = mxfp8_gemm(xq, xs, _t8(wq), ws.t().contiguous())
        if bias is not None:
            y = y + bias.to(y.dtype)
        ctx.save_for_backward(x2, wq, ws)
        ctx.has_bias = bias is not None
        ctx.xshape, ctx.x_dtype, ctx.w_dtype = x.shape, x.dtype, w.dtype
        return y.to(x.dtype).reshape(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        x2, wq, ws = ctx.saved_tensors
        N = wq.shape[1]
        dy2 = dy.reshape(-1, N).to(torch.bfloat16).contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dyq, dys = fp8_quant_1x128(dy2, True)
            dx = mxfp8_gemm(dyq, dys, wq, ws).to(ctx.x_dtype).reshape(ctx.xshape)       # [M, out] x [in, out]^T
        if ctx.needs_input_grad[1]:
            dytq, dyts = fp8_quant_1x128(dy2.t().contiguous(), True)                     # [out, M]
            xtq, xts = fp8_quant_128x128(x2.t().contiguous(), True)                      # [in, M]
            dw = mxfp8_gemm(dytq, dyts, xtq, xts).t().to(ctx.w_dtype)                    # [out, in] -> (in, out)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(ctx.w_dtype)
        return dx, dw, db


def fp8_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w + bias`` (w of shape (in, out)) with the three GEMMs of the layer in block-scaled FP8."""
    assert fp8_eligible(x, w), "fp8_linear: token count and both weight dimensions must be multiples of 128"
    return _Fp8LinearFn.apply(x, w, bias)
