"""MoE routers: softmax top-k with renormalisation (Qwen3.5; jax_gpt/models/qwen35/moe.py:50-55)
and DeepSeek-V3's group-limited sigmoid router. PyTorch reference here; the fused CUDA kernel
(logits -> weights, ids, per-expert counts) is dispatched for CUDA inputs when built."""
from __future__ import annotations

import torch


def softmax_topk_router(logits: torch.Tensor, k: int):
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = probs.topk(k, dim=-1)
    return w / w.sum(-1, keepdim=True), idx


def deepseek_router_from_logits(logits: torch.Tensor, bias: torch.Tensor, k: int, n_group: int, topk_group: int,
                                scale: float, norm_topk: bool = True):
    M, E = logits.shape
    s = torch.sigmoid(logits.float())
    choice = s + bias.float()
    group_scores = choice.view(M, n_group, E // n_group).topk(2, dim=-1)[0].sum(-1)
    gidx = group_scores.topk(topk_group, dim=-1)[1]
    gmask = torch.zeros_like(group_scores).scatter_(1, gidx, 1.0)
    mask = gmask[:, :, None].expand(M, n_group, E // n_group).reshape(M, E).bool()
    idx = choice.masked_fill(~mask, 0.0).topk(k, dim=-1)[1]
    w = s.gather(1, idx)
    if norm_topk:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * scale, idx


def deepseek_router(x: torch.Tensor, gate_weight: torch.Tensor, bias: torch.Tensor, k: int, n_group: int,
                    topk_group: int, scale: float, norm_topk: bool = True):
    """x (M,D), gate_weight (D,E) -> (weights (M,k) fp32, ids (M,k)). Logits in fp32."""
    logits = x.float() @ gate_weight.float()
    return deepseek_router_from_logits(logits, bias, k, n_group, topk_group, scale, norm_topk)
