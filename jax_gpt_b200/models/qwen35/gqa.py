"""Gated grouped-query attention (jax_gpt/models/qwen35/gqa.py:20-130): a 2x-wide q projection
split per head into query and output gate, per-head RMSNorm(1+w) on q and k, partial half-split
RoPE, causal softmax attention, ``out * sigmoid(gate)``, output projection. The cached path
attends over the filled prefix only (the reference spans the whole zero-padded buffer and masks)."""
from __future__ import annotations

from typing import Optional

import torch

from ...ops import attention as attn_ops
from .fp8 import matmul_maybe_fp8
from .primitives import apply_rotary_emb, rms_norm


def gqa_attention(x, params, n_q_heads: int, n_kv_heads: int, head_dim: int, rope_freqs, rope_dim: int,
                  cache_k: Optional[torch.Tensor] = None, cache_v: Optional[torch.Tensor] = None,
                  cache_pos: Optional[int] = None):
    """x (B,T,D) -> (out (B,T,D), new_k, new_v). Caches are (B, Hkv, max_len, dh), updated in place."""
    B, T, _ = x.shape
    qg = matmul_maybe_fp8(x, params["q_proj"]).reshape(B, T, n_q_heads, 2 * head_dim)
    q, gate = qg[..., :head_dim], qg[..., head_dim:]
    k = matmul_maybe_fp8(x, params["k_proj"]).reshape(B, T, n_kv_heads, head_dim)
    v = matmul_maybe_fp8(x, params["v_proj"]).reshape(B, T, n_kv_heads, head_dim)
    pos = int(cache_pos) if cache_pos is not None else 0
    if x.is_cuda and x.dtype == torch.bfloat16:
        # per-head RMSNorm(1 + w) and partial rotary in one kernel
        from ...ops.rope import rmsnorm_rope
        q = rmsnorm_rope(q, params["q_norm"], rope_freqs, rope_dim, pos)
        k = rmsnorm_rope(k, params["k_norm"], rope_freqs, rope_dim, pos)
    else:
        q = rms_norm(q.contiguous(), params["q_norm"])
        k = rms_norm(k.contiguous(), params["k_norm"])
        fr = rope_freqs[pos:pos + T]
        q = apply_rotary_emb(q, fr, rope_dim)
        k = apply_rotary_emb(k, fr, rope_dim)
    if cache_k is not None:
        cache_k[:, :, pos:pos + T] = k.permute(0, 2, 1, 3).to(cache_k.dtype)
        cache_v[:, :, pos:pos + T] = v.permute(0, 2, 1, 3).to(cache_v.dtype)
        if T == 1:
            # decode: one token per sequence against the filled prefix of the cache, split over the keys
            out = attn_ops.attention_decode(q[:, 0], cache_k, cache_v, kv_len=pos + 1)[:, None]
        elif pos == 0:
            out = attn_ops.attention(q.contiguous(), k.contiguous(), v.contiguous(), causal=True)
        else:
            # a later chunk of a prompt: the forward kernel reads the cache in place, queries at pos + i
            out = attn_ops.attention_cached(q.contiguous(), cache_k, cache_v, pos + T, pos)
    else:
        out = attn_ops.attention(q.contiguous(), k.contiguous(), v.contiguous(), causal=True)
    out = out * torch.sigmoid(gate.float()).to(out.dtype)
    y = matmul_maybe_fp8(out.reshape(B, T, n_q_heads * head_dim), params["o_proj"])
    return y, cache_k, cache_v
