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


def _q_proj_cols(w) -> int:
    return w["w"].shape[-2] if isinstance(w, dict) else w.shape[-1]


def gqa_attention(x, params, n_q_heads: int, n_kv_heads: int, head_dim: int, rope_freqs, rope_dim: int,
                  cache_k: Optional[torch.Tensor] = None, cache_v: Optional[torch.Tensor] = None,
                  cache_pos: Optional[int] = None, tp_group=None):
    """x (B,T,D) -> (out (B,T,D), new_k, new_v). Caches are (B, Hkv, max_len, dh), updated in place.

    Tensor parallel (``tp_group`` and a head-sharded ``q_proj`` / ``o_proj``, models/qwen35/sharding.py rules A):
    this rank computes its query heads against the kv heads they belong to; k and v (replicated weights, as in the
    reference's rules, where two kv heads do not divide over the mesh) are computed in full on every rank, so the
    cache stays whole, and the row-parallel output projection is summed over the group."""
    from ...parallel.tp_ops import copy_to_tp, reduce_from_tp, tp_rank
    B, T, _ = x.shape
    hq_all, hkv_all = n_q_heads, n_kv_heads
    n_q_heads = _q_proj_cols(params["q_proj"]) // (2 * head_dim)
    sharded = n_q_heads < hq_all
    kv_lo = 0
    if sharded:
        g = hq_all // hkv_all
        assert n_q_heads % g == 0 or g % n_q_heads == 0, "query-head shard must align with the kv groups"
        kv_lo = (tp_rank(tp_group) * n_q_heads) // g
        n_kv_heads = max(1, n_q_heads // g)
    qg = matmul_maybe_fp8(copy_to_tp(x, tp_group) if sharded else x, params["q_proj"]).reshape(B, T, n_q_heads, 2 * head_dim)
    q, gate = qg[..., :head_dim], qg[..., head_dim:]
    k = matmul_maybe_fp8(x, params["k_proj"]).reshape(B, T, hkv_all, head_dim)
    v = matmul_maybe_fp8(x, params["v_proj"]).reshape(B, T, hkv_all, head_dim)
    pos = int(cache_pos) if cache_pos is not None else 0
    q_norm_w = copy_to_tp(params["q_norm"], tp_group) if sharded else params["q_norm"]   # used on this rank's heads only
    if x.is_cuda and x.dtype == torch.bfloat16:
        # per-head RMSNorm(1 + w) and partial rotary in one kernel
        from ...ops.rope import rmsnorm_rope
        q = rmsnorm_rope(q, q_norm_w, rope_freqs, rope_dim, pos)
        k = rmsnorm_rope(k, params["k_norm"], rope_freqs, rope_dim, pos)
    else:
        q = rms_norm(q.contiguous(), q_norm_w)
        k = rms_norm(k.contiguous(), params["k_norm"])
        fr = rope_freqs[pos:pos + T]
        q = apply_rotary_emb(q, fr, rope_dim)
        k = apply_rotary_emb(k, fr, rope_dim)
    if sharded:
        # every rank has the full k / v; each uses the heads of its queries, and the gradients of the slices add up
        k = copy_to_tp(k, tp_group)
        v = copy_to_tp(v, tp_group)
    if cache_k is not None:
        cache_k[:, :, pos:pos + T] = k.permute(0, 2, 1, 3).to(cache_k.dtype)
        cache_v[:, :, pos:pos + T] = v.permute(0, 2, 1, 3).to(cache_v.dtype)
    if sharded:
        k, v = k[:, :, kv_lo:kv_lo + n_kv_heads], v[:, :, kv_lo:kv_lo + n_kv_heads]
        full_k, full_v = cache_k, cache_v
        if cache_k is not None:
            cache_k = cache_k[:, kv_lo:kv_lo + n_kv_heads].contiguous()
            cache_v = cache_v[:, kv_lo:kv_lo + n_kv_heads].contiguous()
    if cache_k is not None:
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
    if sharded:
        return reduce_from_tp(y, tp_group), full_k, full_v
    return y, cache_k, cache_v
