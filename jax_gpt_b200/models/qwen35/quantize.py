"""Whole-tree FP8 quantisation (jax_gpt/models/qwen35/quantize.py:18-109): per output-row scales
of the transposed (out,in) weight; norms, A_log, dt_bias, embeddings, conv weights and small
tensors stay dense."""
from __future__ import annotations

import torch

from .fp8 import FP8_DTYPE, FP8_MAX, dequantize_weight, is_fp8_weight

SKIP_TOKENS = ("norm", "A_log", "dt_bias", "scale_inv", "embed", "conv_weight")


def quantize_weight(w: torch.Tensor) -> dict:
    """(…, in, out) dense -> {'w': (…, out, in) e4m3, 'scale_inv': (…, out, 1)}."""
    wt = w.float().transpose(-1, -2)
    amax = wt.abs().amax(dim=-1, keepdim=True).clamp_min(1e-12)
    scale_inv = FP8_MAX / amax
    return {"w": (wt * scale_inv).clamp(-FP8_MAX, FP8_MAX).to(FP8_DTYPE), "scale_inv": scale_inv}


def should_quantize(name: str, t: torch.Tensor) -> bool:
    if t.dim() < 2 or min(t.shape[-2:]) < 32:
        return False
    return not any(tok in name for tok in SKIP_TOKENS)


def quantize_params_fp8(params, _prefix: str = ""):
    if isinstance(params, dict) and not is_fp8_weight(params):
        return {k: quantize_params_fp8(v, f"{_prefix}.{k}" if _prefix else k) for k, v in params.items()}
    if torch.is_tensor(params) and should_quantize(_prefix, params):
        return quantize_weight(params)
    return params


def dequantize_params(params, dtype=torch.float32):
    if is_fp8_weight(params):
        return dequantize_weight(params, dtype)
    if isinstance(params, dict):
        return {k: dequantize_params(v, dtype) for k, v in params.items()}
    return params


def count_fp8_params(params):
    """Returns (total parameter count, count stored in FP8)."""
    total = fp8 = 0
    if is_fp8_weight(params):
        n = params["w"].numel()
        return n, n
    if isinstance(params, dict):
        for v in params.values():
            t, f = count_fp8_params(v)
            total, fp8 = total + t, fp8 + f
        return total, fp8
    if torch.is_tensor(params):
        return params.numel(), 0
    return 0, 0
