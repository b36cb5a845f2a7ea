"""Tensor-parallel attention layers on the fused collective GEMMs (sequence parallel outside attention).

Tokens are sharded over the TP ranks between layers. Inside the attention block

* the input projections are ONE all-gather -> GEMM launch (``TPContext.all_gather_matmul``): the peers'
  token shards are read by TMA tile loads straight out of their memory while the local shard's tiles
  are already being multiplied;
* attention runs on this rank's heads over the full sequence;
* the output projection is ONE GEMM -> reduce-scatter launch (``TPContext.matmul_reduce_scatter``) whose
  epilogue adds each tile into the owner rank's rows over NVLink.

``mla_prefill_tp`` is DeepSeek-V3's MLA (heads split over the ranks; the small low-rank projections
q_a / kv_a are computed for all tokens on every rank inside the gathered GEMM), ``gqa_attention_tp`` the
Qwen3.5 gated attention (q heads split; the 2 KV heads are replicated, as the reference's sharding rules
also do, jax_gpt/models/qwen35/sharding.py:41-90).
"""
from __future__ import annotations

import torch

from ..ops import attention as attn_ops
from ..ops.gemm import linear
from .tensor_parallel import TPContext


def shard_mla_params(ap: dict, c, rank: int, world: int) -> dict:
    """Per-rank MLA weights: q_b / kv_b split by head (columns), o_proj by head (rows); q_a | kv_a fused and replicated."""
    H, dn, dr, dv = c.n_heads, c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim
    assert H % world == 0
    hl = H // world
    hs = slice(rank * hl, (rank + 1) * hl)
    qb = ap["q_b_proj"].reshape(-1, H, dn + dr)[:, hs].reshape(-1, hl * (dn + dr)).contiguous()
    kvb = ap["kv_b_proj"].reshape(-1, H, dn + dv)[:, hs].reshape(-1, hl * (dn + dv)).contiguous()
    o = ap["o_proj"].reshape(H, dv, -1)[hs].reshape(hl * dv, -1).contiguous()
    qa_kva = torch.cat([ap["q_a_proj"], ap["kv_a_proj_with_mqa"]], dim=1).contiguous()
    return {"qa_kva": qa_kva, "q_a_norm": ap["q_a_norm"], "kv_a_norm": ap["kv_a_norm"], "q_b_proj": qb, "kv_b_proj": kvb,
            "o_proj": o, "heads_local": hl}


def mla_prefill_tp(ctx: TPContext, x_local: torch.Tensor, sp: dict, c, rope: torch.Tensor, batch: int, seq: int):
    """x_local (rows_local, D): this rank's token shard of a (batch, seq) prefill (rows are batch-major,
    ``rows_local * world == batch * seq``). Returns this rank's rows of the attention block's output."""
    from ..models.deepseek_v3.model import rms_norm, rope_half_split
    dn, dr, dv, kvr, qr = c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim, c.kv_lora_rank, c.q_lora_rank
    hl = sp["heads_local"]
    B, T = batch, seq
    low = ctx.all_gather_matmul(x_local, sp["qa_kva"])                     # (B*T, q_lora + kv_lora + dr), all tokens
    q = linear(rms_norm(low[:, :qr].contiguous(), sp["q_a_norm"], c.rms_norm_eps), sp["q_b_proj"]).reshape(B, T, hl, dn + dr)
    c_kv = rms_norm(low[:, qr:qr + kvr].contiguous(), sp["kv_a_norm"], c.rms_norm_eps)
    fr = rope[:T]
    q_rope = rope_half_split(q[..., dn:], fr)
    k_rope = rope_half_split(low[:, qr + kvr:].reshape(B, T, 1, dr), fr)
    kvb = linear(c_kv, sp["kv_b_proj"]).reshape(B, T, hl, dn + dv)
    k = torch.cat([kvb[..., :dn], k_rope.expand(B, T, hl, dr)], dim=-1)
    qf = torch.cat([q[..., :dn], q_rope], dim=-1)
    out = attn_ops.mla_attention(qf, k, kvb[..., dn:], c.softmax_scale)     # (B, T, hl, dv)
    return ctx.matmul_reduce_scatter(out.reshape(B * T, hl * dv).contiguous(), sp["o_proj"])


def shard_gqa_params(ap: dict, n_q_heads: int, n_kv_heads: int, head_dim: int, rank: int, world: int) -> dict:
    """Per-rank gated-attention weights: the 2x-wide q projection and o_proj split by q head; k / v replicated
    and fused with q into one column block so that the input projection is a single gathered GEMM."""
    assert n_q_heads % world == 0
    hl = n_q_heads // world
    hs = slice(rank * hl, (rank + 1) * hl)
    D = ap["q_proj"].shape[0]
    q = ap["q_proj"].reshape(D, n_q_heads, 2 * head_dim)[:, hs].reshape(D, hl * 2 * head_dim)
    qkv = torch.cat([q, ap["k_proj"], ap["v_proj"]], dim=1).contiguous()
    o = ap["o_proj"].reshape(n_q_heads, head_dim, -1)[hs].reshape(hl * head_dim, -1).contiguous()
    return {"qkv": qkv, "o_proj": o, "q_norm": ap["q_norm"], "k_norm": ap["k_norm"], "heads_local": hl}


def gqa_attention_tp(ctx: TPContext, x_local: torch.Tensor, sp: dict, n_kv_heads: int, head_dim: int, rope_freqs,
                     rope_dim: int, batch: int, seq: int):
    """Qwen3.5 gated attention, prefill, tokens sharded over the ranks. Returns this rank's output rows."""
    from ..ops.rope import rmsnorm_rope
    hl = sp["heads_local"]
    B, T = batch, seq
    qkv = ctx.all_gather_matmul(x_local, sp["qkv"])                         # all tokens x (hl*2*dh + 2*Hkv*dh)
    nq = hl * 2 * head_dim
    qg = qkv[:, :nq].reshape(B, T, hl, 2 * head_dim)
    q, gate = qg[..., :head_dim], qg[..., head_dim:]
    k = qkv[:, nq:nq + n_kv_heads * head_dim].reshape(B, T, n_kv_heads, head_dim)
    v = qkv[:, nq + n_kv_heads * head_dim:].reshape(B, T, n_kv_heads, head_dim)
    q = rmsnorm_rope(q.contiguous(), sp["q_norm"], rope_freqs, rope_dim, 0)
    k = rmsnorm_rope(k.contiguous(), sp["k_norm"], rope_freqs, rope_dim, 0)
    # local q heads attend to the replicated KV heads: group the local heads by their KV head
    rep_total = (hl * ctx.world) // n_kv_heads
    first = ctx.rank * hl
    kv_idx = torch.arange(first, first + hl, device=q.device) // rep_total
    out = attn_ops.attention(q, k[:, :, kv_idx].contiguous(), v[:, :, kv_idx].contiguous(), causal=True)
    out = out * torch.sigmoid(gate.float()).to(out.dtype)
    return ctx.matmul_reduce_scatter(out.reshape(B * T, hl * head_dim).contiguous(), sp["o_proj"])
