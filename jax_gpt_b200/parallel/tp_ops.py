"""Tensor-parallel building blocks with gradients: the collectives that sit between the replicated and the
sharded regions of a layer, as ``autograd.Function``s over a ``torch.distributed`` group (NCCL on GPUs, gloo for
CPU ranks), plus the vocabulary-parallel embedding.

A tensor-parallel layer in this package is written Megatron-style on REPLICATED activations:

    h   = norm(x)                      # replicated
    hs  = copy_to_tp(h)                # identity forward, all-reduce of the gradient backward
    y_r = row_parallel(act(column_parallel(hs)))        # this rank's heads / intermediate slice
    y   = reduce_from_tp(y_r)          # all-reduce forward, identity backward

so every replicated parameter (norm weights, router, k/v projections of the gated attention) sees the FULL
gradient on every rank and no cross-rank reduction of parameter gradients is needed for the TP group; sharded
parameters receive the gradient of their shard. The reference gets the same collectives from GSPMD annotations
(jax_gpt/models/qwen35/sharding.py:104-267, jax_gpt/trainer/sharding.py:24-55); its row-parallel projections
imply the all-reduce that ``reduce_from_tp`` spells out. The fused kernels (all-gather -> GEMM, GEMM ->
reduce-scatter over peer memory) are the sequence-parallel variant of the same pair: parallel/tensor_parallel.py.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def tp_world(group) -> int:
    return dist.get_world_size(group) if group is not None and dist.is_available() and dist.is_initialized() else 1


def tp_rank(group) -> int:
    return dist.get_rank(group) if group is not None and dist.is_available() and dist.is_initialized() else 0


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        y = x.contiguous().clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherFromTP(torch.autograd.Function):
    """Concatenates the ranks' slices along ``dim`` (forward); hands each rank its slice of the gradient."""

    @staticmethod
    def forward(ctx, x, group, dim):
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        ctx.dim, ctx.rank, ctx.n = dim, rank, x.shape[dim]
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=dim)

    @staticmethod
    def backward(ctx, g):
        return g.narrow(ctx.dim, ctx.rank * ctx.n, ctx.n).contiguous(), None, None


def copy_to_tp(x: torch.Tensor, group) -> torch.Tensor:
    """Entry of a sharded region: identity forward, sum of the ranks' gradients backward."""
    return x if tp_world(group) == 1 else _CopyToTP.apply(x, group)


def reduce_from_tp(x: torch.Tensor, group) -> torch.Tensor:
    """Exit of a sharded region: sum over the ranks forward, identity backward."""
    return x if tp_world(group) == 1 else _ReduceFromTP.apply(x, group)


def gather_from_tp(x: torch.Tensor, group, dim: int = -1) -> torch.Tensor:
    if tp_world(group) == 1:
        return x
    return _GatherFromTP.apply(x, group, dim if dim >= 0 else x.dim() + dim)


def vocab_parallel_embedding(tokens: torch.Tensor, table_shard: torch.Tensor, group, vocab_size: Optional[int] = None):
    """Rows of a vocabulary-sharded table: each rank looks up the ids it owns (others give zero rows), the sum over
    the ranks is the embedding (jax_gpt/models/qwen35/sharding.py:43: 'embed' split over the vocabulary)."""
    world = tp_world(group)
    if world == 1 or (vocab_size is not None and table_shard.shape[0] == vocab_size):
        return table_shard[tokens.long()]
    n = table_shard.shape[0]
    lo = tp_rank(group) * n
    t = tokens.long() - lo
    mine = (t >= 0) & (t < n)
    rows = table_shard[t.clamp(0, n - 1)] * mine[..., None].to(table_shard.dtype)
    return reduce_from_tp(rows, group)
