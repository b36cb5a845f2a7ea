"""GPT-2 with tensor + sequence parallelism on the fused collective GEMM kernels.

Between the blocks the token rows are sharded over the ranks (rank r holds rows ``[r M / W, (r + 1) M / W)`` of
the flattened (batch, time) axis); inside a block the attention heads and the MLP columns are sharded. The four
projections of a block are exactly the two fused patterns of ``parallel/tensor_parallel.py``:

    LN -> all-gather rows -> @ W_qkv[:, local heads]      column_parallel_linear   (all-gather -> GEMM, one kernel)
    attention over the whole sequence, local heads
    @ W_proj[local heads, :] -> reduce-scatter rows       row_parallel_linear      (GEMM -> reduce-scatter, one kernel)
    LN -> all-gather rows -> @ W_fc[:, local columns] -> GELU -> @ W_proj2[local columns, :] -> reduce-scatter rows

LayerNorms, residuals, embeddings, the tied head and the loss work on local rows only, so activation memory of those
parts shrinks by the number of ranks. Parameters that are not sharded (LayerNorm, embeddings, the biases added after
a reduce-scatter) see only the local rows' contribution to their gradient: ``sync_replicated_grads`` sums them over
the group. The reference reaches the same layout through GSPMD annotations on the batch / model axes
(jax_gpt/trainer/sharding.py:24-55); here the collectives are explicit and fused into the GEMMs.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import Dict

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..ops import attention as attn_ops
from ..ops import gemm as gemm_ops
from ..ops import norm as norm_ops
from .tensor_parallel import TPContext, column_parallel_linear, row_parallel_linear

SHARDED = ("h.attn.c_attn.kernel", "h.attn.c_attn.bias", "h.attn.c_proj.kernel", "h.mlp.c_fc.kernel", "h.mlp.c_fc.bias",
           "h.mlp.c_proj.kernel")


def shard_gpt2_for_sequence_parallel(params: Dict[str, torch.Tensor], cfg, world: int, rank: int) -> Dict[str, torch.Tensor]:
    """This rank's parameters: the four projections of every block sharded by heads / MLP columns (head-aligned
    q | k | v split, as ``trainer/sharding.py:shard_gpt2_tensor``), everything else replicated."""
    from ..trainer.sharding import shard_gpt2_tensor
    mesh = SimpleNamespace(size=lambda ax: world if ax == "tp" else 1, rank=lambda ax: rank if ax == "tp" else 0)
    return {k: (shard_gpt2_tensor(k, v.detach(), cfg, mesh) if k in SHARDED else v.detach().clone()) for k, v in params.items()}


def gpt2_sequence_parallel_loss(params: Dict[str, torch.Tensor], cfg, tokens: torch.Tensor, targets: torch.Tensor,
                                tp: TPContext) -> torch.Tensor:
    """Mean next-token cross-entropy over ALL rows of the batch, computed from this rank's rows: the returned scalar
    is this rank's share (local sum / total rows), so that ``backward()`` on it followed by
    ``sync_replicated_grads`` yields the gradients of the global mean loss, and the sum over the ranks is the loss.
    tokens, targets (B, T) are the full batch on every rank; bf16 CUDA parameters; B * T / world % 128 == 0."""
    p = params
    W, r = tp.world, tp.rank
    B, T = tokens.shape
    M = B * T
    assert M % (W * 128) == 0, "rows per rank must be a multiple of 128"
    rows = M // W
    lo = r * rows
    d, dh = cfg.d_model, cfg.d_head
    flat_tok = tokens.reshape(-1)[lo:lo + rows].long()
    pos = (torch.arange(lo, lo + rows, device=tokens.device) % T)
    x = p["wte.embedding"][flat_tok] + p["wpe.embedding"][pos]                    # (rows, d): local rows only
    for l in range(cfg.n_layers):
        h1 = norm_ops.layer_norm(x, p["h.ln_1.layer_norm.scale"][l], p["h.ln_1.layer_norm.bias"][l], 1e-5)
        qkv = column_parallel_linear(h1, p["h.attn.c_attn.kernel"][l], tp) + p["h.attn.c_attn.bias"][l]   # (M, 3 d / W)
        dl = qkv.shape[-1] // 3
        q, k, v = [t.reshape(B, T, dl // dh, dh) for t in qkv.split(dl, dim=-1)]
        y = attn_ops.attention(q, k, v, causal=True).reshape(M, dl)
        x = x + row_parallel_linear(y, p["h.attn.c_proj.kernel"][l], tp) + p["h.attn.c_proj.bias"][l]
        h2 = norm_ops.layer_norm(x, p["h.ln_2.layer_norm.scale"][l], p["h.ln_2.layer_norm.bias"][l], 1e-5)
        f = gemm_ops.gelu_tanh(column_parallel_linear(h2, p["h.mlp.c_fc.kernel"][l], tp) + p["h.mlp.c_fc.bias"][l])
        x = x + row_parallel_linear(f, p["h.mlp.c_proj.kernel"][l], tp) + p["h.mlp.c_proj.bias"][l]
    h = norm_ops.layer_norm(x, p["ln_f.layer_norm.scale"], p["ln_f.layer_norm.bias"], 1e-5)
    logits = (h @ p["wte.embedding"].t()).float()
    tgt = targets.reshape(-1)[lo:lo + rows].long()
    return F.cross_entropy(logits, tgt, reduction="sum") / M


def sync_replicated_grads(params: Dict[str, torch.Tensor], group=None) -> None:
    """Sums over the group the gradients of the parameters every rank holds in full (each rank differentiated only
    its own rows). Call after ``backward()`` and before the optimizer step."""
    for k, v in params.items():
        if k not in SHARDED and v.grad is not None:
            dist.all_reduce(v.grad, group=group)
