"""Pure-function primitives of the Qwen3.5 model (jax_gpt/models/qwen35/primitives.py:16-134):
RMSNorm with the (1 + w) convention, RoPE tables, half-split partial rotary, SwiGLU."""
from __future__ import annotations

import torch

from ...ops import norm as norm_ops


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """fp32 ``x / sqrt(mean(x^2) + eps) * (1 + w)``, cast back to x's dtype."""
    return norm_ops.rms_norm(x, weight, eps, one_plus_w=True)


def precompute_rope_freqs(dim: int, max_seq_len: int, theta: float = 10_000_000.0, device=None) -> torch.Tensor:
    """Table of shape (max_seq_len, dim // 2, 2) holding (cos, sin) of ``t * theta^(-2i/dim)``."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
    ang = torch.arange(max_seq_len, dtype=torch.float32, device=device)[:, None] * inv[None, :]
    return torch.stack([ang.cos(), ang.sin()], dim=-1)


def apply_rotary_emb(x: torch.Tensor, freqs: torch.Tensor, rope_dim: int) -> torch.Tensor:
    """Rotates the first ``rope_dim`` features of x (..., T, H, dh) with half-split pairing
    (x[i], x[i + rope_dim/2]); the remaining features pass through. ``freqs``: (T, rope_dim/2, 2)."""
    rot, rest = x[..., :rope_dim], x[..., rope_dim:]
    half = rope_dim // 2
    x1, x2 = rot[..., :half].float(), rot[..., half:].float()
    cos = freqs[:, None, :, 0]
    sin = freqs[:, None, :, 1]
    o1 = x1 * cos - x2 * sin
    o2 = x2 * cos + x1 * sin
    return torch.cat([o1.to(x.dtype), o2.to(x.dtype), rest], dim=-1)


def swiglu(x: torch.Tensor, gate_w, up_w, down_w) -> torch.Tensor:
    """``down(silu(x @ gate) * (x @ up))`` with (in,out) kernels (possibly FP8 dicts)."""
    from .fp8 import matmul_maybe_fp8
    g = matmul_maybe_fp8(x, gate_w)
    u = matmul_maybe_fp8(x, up_w)
    return matmul_maybe_fp8(torch.nn.functional.silu(g) * u, down_w)
