"""FP8 (e4m3) helpers with per-row scales (jax_gpt/models/qwen35/fp8.py:26-193).

One convention everywhere: a quantised weight is ``{'w': e4m3 (..., out, in), 'scale_inv': f32
(..., out, 1)}`` with ``w = round(weight^T * scale_inv)``, i.e. ``scale_inv = 448 / amax`` is the
QUANTISATION multiplier and de-quantisation DIVIDES by it (``scale_inv = 2`` halves the weight).
The reference applies this to 2-D weights but multiplies for stacked expert weights
(jax_gpt/models/qwen35/fp8.py:146); here 2-D and 3-D follow the same rule.
"""
from __future__ import annotations

import torch

FP8_DTYPE = torch.float8_e4m3fn
FP8_MAX = 448.0


def is_fp8_weight(w) -> bool:
    return isinstance(w, dict) and "w" in w and "scale_inv" in w


def dynamic_quantize_fp8(x: torch.Tensor):
    """Per-row (last dim) dynamic quantisation: returns (x_fp8, scale) with x ~= x_fp8 * scale."""
    xf = x.float()
    amax = xf.abs().amax(dim=-1, keepdim=True)
    scale = (amax / FP8_MAX).clamp_min(torch.finfo(torch.float32).tiny)
    q = (xf / scale).clamp(-FP8_MAX, FP8_MAX).to(FP8_DTYPE)
    return q, scale


def fp8_matmul(x: torch.Tensor, w_fp8: torch.Tensor, w_scale_inv: torch.Tensor) -> torch.Tensor:
    """``x @ dequant(w)`` with dynamic activation quantisation; w_fp8 (out, in), w_scale_inv (out, 1).
    fp32 accumulation, then ``* x_scale / w_scale_inv``."""
    xq, xs = dynamic_quantize_fp8(x)
    acc = xq.float() @ w_fp8.float().t()
    return (acc * xs / w_scale_inv.reshape(1, -1).float()).to(x.dtype if x.dtype != FP8_DTYPE else torch.bfloat16)


def fp8_linear(x: torch.Tensor, params: dict, key: str = "weight") -> torch.Tensor:
    w = params[key]
    return fp8_matmul(x, w["w"], w["scale_inv"])


def dequantize_weight(w: dict, dtype=torch.float32) -> torch.Tensor:
    """(…, out, in) fp8 + scales -> (…, in, out) dense."""
    return (w["w"].float() / w["scale_inv"].float()).transpose(-1, -2).to(dtype)


def matmul_maybe_fp8(x: torch.Tensor, w) -> torch.Tensor:
    """``x @ w`` for a dense (in,out) kernel or an FP8 dict (2-D: quantised matmul; stacked 3-D
    expert weights: de-quantise then matmul)."""
    if is_fp8_weight(w):
        if w["w"].dim() == 2:
            shp = x.shape
            y = fp8_matmul(x.reshape(-1, shp[-1]), w["w"], w["scale_inv"])
            return y.reshape(*shp[:-1], -1)
        return x @ dequantize_weight(w, x.dtype)
    from ...ops.gemm import linear
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dim() == 2 and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0:
        return linear(x, w)
    return x @ w


def fp8_ragged_dot(x: torch.Tensor, w_fp8: torch.Tensor, group_sizes: torch.Tensor, w_scale_inv: torch.Tensor):
    """Grouped matmul over contiguous row groups: rows of group e use expert e's weight.
    x (M, in); w_fp8 (E, out, in); w_scale_inv (E, out, 1). Activation and weight scales both applied."""
    xq, xs = dynamic_quantize_fp8(x)
    out = x.new_zeros(x.shape[0], w_fp8.shape[1], dtype=torch.float32)
    start = 0
    for e, n in enumerate(group_sizes.tolist()):
        if n:
            acc = xq[start:start + n].float() @ w_fp8[e].float().t()
            out[start:start + n] = acc * xs[start:start + n] / w_scale_inv[e].reshape(1, -1).float()
        start += n
    return out.to(x.dtype)
