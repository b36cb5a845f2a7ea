"""Hybrid inference cache (jax_gpt/models/qwen35/cache.py:20-102): a fixed-size recurrent state
and conv window per DeltaNet layer, a KV cache per gated-attention layer, one position."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .config import Qwen35Config


@dataclass
class HybridCache:
    delta_M: torch.Tensor      # (G, 3, B, Hv, dk, dv)
    delta_conv: torch.Tensor   # (G, 3, B, conv_dim, K)
    gqa_k: torch.Tensor        # (G, B, Hkv, max_len, dh)
    gqa_v: torch.Tensor        # (G, B, Hkv, max_len, dh)
    pos: int                   # tokens already in the cache (same for the whole batch)


def init_cache(config: Qwen35Config, batch_size: int, max_len: Optional[int] = None, dtype=torch.float32,
               device="cpu") -> HybridCache:
    G, nd = config.n_groups, config.n_delta_per_group
    max_len = max_len or config.max_position_embeddings
    z = lambda *s: torch.zeros(*s, dtype=dtype, device=device)
    return HybridCache(
        delta_M=z(G, nd, batch_size, config.delta_n_v_heads, config.delta_qk_head_dim, config.delta_v_head_dim),
        delta_conv=z(G, nd, batch_size, config.delta_conv_dim, config.delta_conv_kernel),
        gqa_k=z(G, batch_size, config.gqa_n_kv_heads, max_len, config.gqa_head_dim),
        gqa_v=z(G, batch_size, config.gqa_n_kv_heads, max_len, config.gqa_head_dim),
        pos=0)
