"""MoE routers: softmax top-k with renormalisation (Qwen3.5; jax_gpt/models/qwen35/moe.py:50-55)
and DeepSeek-V3's group-limited sigmoid router. PyTorch reference here; the fused CUDA kernel
(logits -> weights, ids, per-expert counts) is dispatched for CUDA inputs when built."""
from __future__ import annotations

import torch


def _cuda_ok(logits, k, n_group=1):
    E = logits.shape[-1]
    return logits.is_cuda and E % 32 == 0 and E <= 512 and k <= 32 and (n_group <= 1 or (32 % n_group == 0 and E % n_group == 0))


def router_cuda(mode: int, logits, bias, k, n_group=1, topk_group=1, scale=1.0, counts=None):
    """Fused router kernel: (weights fp32 [M,k], ids int32 [M,k]); adds pair counts into ``counts`` when given."""
    from .. import _ext
    lf = logits.float().contiguous()
    M = lf.shape[0]
    w = torch.empty(M, k, device=lf.device, dtype=torch.float32)
    ids = torch.empty(M, k, device=lf.device, dtype=torch.int32)
    _ext.ops().router(mode, lf, None if bias is None else bias.float().contiguous(), k, n_group, topk_group, scale, w,
                      ids, counts)
    return w, ids


def _needs_grad(t):
    return torch.is_grad_enabled() and t.requires_grad


def softmax_topk_router(logits: torch.Tensor, k: int):
    if _cuda_ok(logits, k):
        w, ids = router_cuda(0, logits.detach(), None, k)
        if _needs_grad(logits):  # the kernel picks the experts; the weights are re-derived differentiably
            w = torch.softmax(logits.float(), dim=-1).gather(1, ids.long())
            w = w / w.sum(-1, keepdim=True)
        return w, ids.long()
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = probs.topk(k, dim=-1)
    return w / w.sum(-1, keepdim=True), idx


def deepseek_router_from_logits(logits: torch.Tensor, bias: torch.Tensor, k: int, n_group: int, topk_group: int,
                                scale: float, norm_topk: bool = True):
    M, E = logits.shape
    if _cuda_ok(logits, k, n_group) and norm_topk:
        w, ids = router_cuda(1, logits.detach(), bias, k, n_group, topk_group, scale)
        if _needs_grad(logits):
            w = torch.sigmoid(logits.float()).gather(1, ids.long())
            w = w / (w.sum(-1, keepdim=True) + 1e-20) * scale
        return w, ids.long()
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
    from .gemm import linear_f32out
    logits = linear_f32out(x, gate_weight)
    return deepseek_router_from_logits(logits, bias, k, n_group, topk_group, scale, norm_topk)
