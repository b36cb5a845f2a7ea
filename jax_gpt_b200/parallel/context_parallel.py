"""Context parallelism for causal attention (long sequences split over the ranks).

The sequence of length T is cut into ``2 * world`` chunks; rank r holds chunks r and ``2 * world - 1 - r`` (the
zig-zag layout), so that under the causal mask every rank owns the same number of (query chunk, key chunk) blocks:
``2 * world + 1``. Keys and values are all-gathered once; each rank then runs the flash-attention kernel block by
block: a square causal block where a query chunk meets its own keys, full (unmasked) blocks against every earlier
chunk, and merges the partial results with their log-sum-exps. The backward pass calls the attention backward
kernel per block with the GLOBAL output and log-sum-exp of the query chunk (so every block yields exactly its share
of the gradient), accumulates dQ locally and sums dK / dV over the ranks.

The reference lists ring / context-parallel attention as an optional extension of its sharding rules
(jax_gpt/trainer/sharding.py:24-55 shards only batch and model axes); the block decomposition here is what a ring
schedule computes, with the key / value exchange done by one all-gather instead of ``world`` point-to-point steps.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist

_LN2 = math.log(2.0)


def zigzag_split(x: torch.Tensor, world: int, rank: int, dim: int = 1) -> torch.Tensor:
    """The two chunks of ``x`` (split in ``2 * world`` along ``dim``) that rank ``rank`` owns, concatenated."""
    chunks = x.chunk(2 * world, dim=dim)
    return torch.cat([chunks[rank], chunks[2 * world - 1 - rank]], dim=dim)


def zigzag_merge(parts: List[torch.Tensor], dim: int = 1) -> torch.Tensor:
    """Inverse of ``zigzag_split`` given every rank's local tensor (in rank order)."""
    world = len(parts)
    chunks = [None] * (2 * world)
    for r, p in enumerate(parts):
        a, b = p.chunk(2, dim=dim)
        chunks[r], chunks[2 * world - 1 - r] = a, b
    return torch.cat(chunks, dim=dim)


def _use_kernel(q, k, v) -> bool:
    from ..ops.attention import supports_cuda_kernel
    return q.is_cuda and q.dtype == torch.bfloat16 and supports_cuda_kernel(q, k, v) and q.shape[1] % 128 == 0


def _block_fwd(q, k, v, causal: bool, scale: float):
    """One (query chunk, key chunk) block: (out fp32 (B,c,H,Dv), lse (B,H,c) in log2 units)."""
    if _use_kernel(q, k, v):
        from ..ops.attention import attn_fwd
        out, lse = attn_fwd(q.contiguous(), k.contiguous(), v.contiguous(), causal, scale)
        return out.float(), lse
    B, c, H, D = q.shape
    rep = H // k.shape[2]
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = (qf @ kf.transpose(-1, -2)) * scale
    if causal:
        s = s.masked_fill(~torch.ones(c, k.shape[1], dtype=torch.bool, device=q.device).tril(), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    out = torch.exp(s - lse[..., None]) @ vf
    return out.permute(0, 2, 1, 3), lse / _LN2


def _block_bwd(q, k, v, out, dout, lse2, causal: bool, scale: float):
    """Gradient share of one block given the GLOBAL ``out`` / ``lse2`` of the query chunk: (dq, dk, dv) fp32."""
    if _use_kernel(q, k, v):
        from ..ops.attention import attn_bwd
        dq, dk, dv = attn_bwd(q.contiguous(), k.contiguous(), v.contiguous(), out.to(torch.bfloat16).contiguous(),
                              dout.to(torch.bfloat16).contiguous(), lse2.contiguous(), causal, scale)
        return dq.float(), dk.float(), dv.float()
    B, c, H, D = q.shape
    Hkv = k.shape[2]
    rep = H // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    do = dout.float().permute(0, 2, 1, 3)
    of = out.float().permute(0, 2, 1, 3)
    s = (qf @ kf.transpose(-1, -2)) * scale
    if causal:
        s = s.masked_fill(~torch.ones(c, k.shape[1], dtype=torch.bool, device=q.device).tril(), float("-inf"))
    p = torch.exp(s - (lse2 * _LN2)[..., None])
    dv = p.transpose(-1, -2) @ do
    dp = do @ vf.transpose(-1, -2)
    delta = (do * of).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = ds @ kf
    dk = ds.transpose(-1, -2) @ qf
    fold = lambda t: t.reshape(B, Hkv, rep, t.shape[2], t.shape[3]).sum(2).permute(0, 2, 1, 3)
    return dq.permute(0, 2, 1, 3), fold(dk), fold(dv)


def _gather_chunks(t_local: torch.Tensor, group) -> List[torch.Tensor]:
    """All ranks' local (two-chunk) tensors -> the ``2 * world`` global chunks in sequence order."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(t_local) for _ in range(world)]
    dist.all_gather(parts, t_local.contiguous(), group=group)
    chunks = [None] * (2 * world)
    for r, p in enumerate(parts):
        a, b = p.chunk(2, dim=1)
        chunks[r], chunks[2 * world - 1 - r] = a, b
    return chunks


class _ContextParallelAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, group, scale):
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        kc, vc = _gather_chunks(k, group), _gather_chunks(v, group)
        outs, lses = [], []
        for qi, gq in enumerate((rank, 2 * world - 1 - rank)):
            qc = q.chunk(2, dim=1)[qi]
            acc = lse_tot = None
            for gk in range(gq + 1):
                o, l2 = _block_fwd(qc, kc[gk], vc[gk], gk == gq, scale)
                if acc is None:
                    acc, lse_tot = o, l2
                else:
                    new = torch.logaddexp(lse_tot * _LN2, l2 * _LN2) / _LN2
                    w_old = torch.exp2(lse_tot - new).permute(0, 2, 1)[..., None]
                    w_new = torch.exp2(l2 - new).permute(0, 2, 1)[..., None]
                    acc, lse_tot = acc * w_old + o * w_new, new
            outs.append(acc)
            lses.append(lse_tot)
        out = torch.cat(outs, dim=1).to(q.dtype)
        ctx.save_for_backward(q, k, v, out, torch.stack(lses))
        ctx.group, ctx.scale = group, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lses = ctx.saved_tensors
        group, scale = ctx.group, ctx.scale
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        kc, vc = _gather_chunks(k, group), _gather_chunks(v, group)
        dk_all = [torch.zeros(c.shape, device=c.device, dtype=torch.float32) for c in kc]
        dv_all = [torch.zeros(c.shape, device=c.device, dtype=torch.float32) for c in vc]
        dqs = []
        for qi, gq in enumerate((rank, 2 * world - 1 - rank)):
            qc, oc, doc = [t.chunk(2, dim=1)[qi] for t in (q, out, dout)]
            dq = torch.zeros(qc.shape, device=q.device, dtype=torch.float32)
            for gk in range(gq + 1):
                a, b, c = _block_bwd(qc, kc[gk], vc[gk], oc, doc, lses[qi], gk == gq, scale)
                dq += a
                dk_all[gk] += b
                dv_all[gk] += c
            dqs.append(dq)
        # every rank holds partial dK / dV of every chunk: sum over the ranks, keep the two own chunks
        dk_sum, dv_sum = torch.stack(dk_all), torch.stack(dv_all)
        dist.all_reduce(dk_sum, group=group)
        dist.all_reduce(dv_sum, group=group)
        own = (rank, 2 * world - 1 - rank)
        dk = torch.cat([dk_sum[i] for i in own], dim=1).to(k.dtype)
        dv = torch.cat([dv_sum[i] for i in own], dim=1).to(v.dtype)
        return torch.cat(dqs, dim=1).to(q.dtype), dk, dv, None, None


def context_parallel_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group=None,
                               scale: Optional[float] = None) -> torch.Tensor:
    """Causal attention over a sequence sharded in the zig-zag layout: q (B, T / world, H, D), k / v
    (B, T / world, Hkv, D[v]) are this rank's two chunks (``zigzag_split``); returns the local rows of the output,
    (B, T / world, H, Dv), differentiable. bf16 CUDA tensors whose chunk length is a multiple of 128 run on the
    flash-attention kernels; anything else (CPU ranks over gloo included) on the PyTorch restatement."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    group = group if group is not None else dist.group.WORLD
    assert q.shape[1] % 2 == 0, "every rank holds two chunks"
    return _ContextParallelAttnFn.apply(q, k, v, group, scale)
