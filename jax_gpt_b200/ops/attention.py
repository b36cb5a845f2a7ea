"""Causal / full softmax attention: tcgen05 flash kernels on CUDA, dense fp32 reference elsewhere.

The reference materialises (B,H,T,S) scores (jax_gpt/models/gpt2/model.py:167-176,
jax_gpt/models/qwen35/gqa.py:103-119); the kernels tile the same math with an online softmax.
Tensors are [B, T, H, D]; q/k/v may be column slices of one fused projection output.

CUDA bf16 paths, none of which calls a library matmul or materialises scores:
  * ``attention`` / ``mla_attention``: forward and backward kernels for head widths 64, 128, 256 and the MLA
    prefill shape (q/k 192, v 128);
  * ``attention_cached``: the forward kernel reading K / V straight from a (B, Hkv, max_len, D) cache with the
    queries at positions ``q_pos0 + i`` (prefill on top of a cache);
  * ``attention_decode``: one query token per sequence, split over the keys of the cache.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _ext


def attention_ref(q, k, v, causal: bool = True, scale: Optional[float] = None, q_pos0: int = 0):
    """fp32 dense attention; q [B,T,H,D], k/v [B,S,Hkv,D]; query i sits at position q_pos0 + i."""
    B, T, H, D = q.shape
    S, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(H // Hkv, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(H // Hkv, dim=1)
    s = (qf @ kf.transpose(-1, -2)) * scale
    if causal:
        qp = torch.arange(T, device=q.device)[:, None] + q_pos0
        kp = torch.arange(S, device=q.device)[None, :]
        s = s.masked_fill(kp > qp, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return (p @ vf).permute(0, 2, 1, 3).to(q.dtype)


def _as2d(t):
    B, T, H, D = t.shape
    assert t.stride(3) == 1 and t.stride(2) == D and t.stride(0) == T * t.stride(1), "unsupported attention layout"
    return t.as_strided((B * T, H * D), (t.stride(1), 1))


def attn_fwd(q, k, v, causal=True, scale=None, out=None, lse=None):
    """Raw CUDA forward. Returns (out [B,T,H,D] bf16, lse [B,H,T] fp32 in log2 units)."""
    B, T, H, D = q.shape
    Hkv, Dv = k.shape[2], v.shape[3]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty(B, T, H, Dv, device=q.device, dtype=torch.bfloat16)
    if lse is None:
        lse = torch.empty(B, H, T, device=q.device, dtype=torch.float32)
    _ext.ops().attn_fwd(_as2d(q), _as2d(k), _as2d(v), _as2d(out), lse, B, T, H, Hkv, D, scale, causal, Dv)
    return out, lse


def attn_bwd(q, k, v, out, dout, lse, causal=True, scale=None, dq=None, dk=None, dv=None, dq_accum=None, delta=None):
    """Raw CUDA backward. Returns (dq, dk, dv) in bf16 with the layouts of q/k/v. Head widths 64 / 128 run the
    key-block-stationary kernel, 256 and the MLA shape (192 / 128) the 64-query-tile kernel for wide heads."""
    B, T, H, D = q.shape
    Hkv, Dv = k.shape[2], v.shape[3]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if dq_accum is None:
        dq_accum = torch.zeros(B * T, H * D, device=q.device, dtype=torch.float32)
    if delta is None:
        delta = torch.empty(B, H, T, device=q.device, dtype=torch.float32)
    if dq is None:
        dq = torch.empty(B, T, H, D, device=q.device, dtype=torch.bfloat16)
    if dk is None:
        dk = torch.empty(B, T, Hkv, D, device=q.device, dtype=torch.bfloat16)
    if dv is None:
        dv = torch.empty(B, T, Hkv, Dv, device=q.device, dtype=torch.bfloat16)
    if D in (64, 128) and Dv == D:
        _ext.ops().attn_bwd(_as2d(q), _as2d(k), _as2d(v), _as2d(out), _as2d(dout), lse, delta, dq_accum, _as2d(dk),
                            _as2d(dv), B, T, H, Hkv, D, scale, causal)
    else:
        _ext.ops().attn_bwd_wide(_as2d(q), _as2d(k), _as2d(v), _as2d(out), _as2d(dout), lse, delta, dq_accum,
                                 _as2d(dk), _as2d(dv), B, T, H, Hkv, D, Dv, scale, causal)
    _ext.ops().cast_rows(dq_accum, _as2d(dq))
    return dq, dk, dv


def attn_fwd_cached(q, cache_k, cache_v, kv_len: int, q_pos0: int, causal=True, scale=None, out=None, lse=None):
    """Raw CUDA forward with K / V read from caches (B, Hkv, max_len, D) bf16: q (B, Tq, H, D) sits at positions
    ``q_pos0 + i`` and attends over the first ``kv_len`` cache rows. Rows of the last 128-row tile past ``kv_len``
    are read and masked, so the cache must hold finite values there (zeros from ``init_cache``)."""
    B, T, H, D = q.shape
    Dv = cache_v.shape[3]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty(B, T, H, Dv, device=q.device, dtype=torch.bfloat16)
    if lse is None:
        lse = torch.empty(B, H, T, device=q.device, dtype=torch.float32)
    _ext.ops().attn_fwd_cached(_as2d(q), cache_k, cache_v, _as2d(out), lse, B, T, H, int(kv_len), int(q_pos0), scale,
                               causal)
    return out, lse


def decode_splits(batch: int, n_kv_heads: int, max_len: int) -> int:
    """Key ranges per (sequence, kv head) for ``attention_decode``: enough CTAs to cover the SMs about twice,
    at least 64 keys per range."""
    want = max(1, 296 // max(1, batch * n_kv_heads))
    return int(max(1, min(want, (max_len + 63) // 64, 64)))


def attention_decode(q, cache_k, cache_v, kv_len=None, pos: Optional[torch.Tensor] = None, scale=None,
                     scratch=None, out=None):
    """One query token per sequence over a dense cache. q (B, H, D) (any view with contiguous heads); caches
    (B, Hkv, max_len, D). The number of valid keys is ``kv_len`` (host int) or ``pos + 1`` with ``pos`` an int32
    DEVICE scalar (CUDA-graph decode loops). ``scratch = (part_o [B,H,S,D], part_ml [B,H,S,2])`` fp32 may be
    preallocated; S is the number of key ranges. Returns (B, H, D)."""
    B, H, D = q.shape
    Hkv = cache_k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    cuda_ok = (q.is_cuda and q.dtype == torch.bfloat16 and cache_k.dtype == torch.bfloat16 and D in (64, 128, 256)
               and H % Hkv == 0 and (H // Hkv) in (1, 2, 4, 8))
    if not cuda_ok:
        n = int(kv_len) if kv_len is not None else int(pos.item()) + 1
        kk = cache_k[:B, :, :n].permute(0, 2, 1, 3).to(q.dtype)
        vv = cache_v[:B, :, :n].permute(0, 2, 1, 3).to(q.dtype)
        return attention_ref(q[:, None], kk, vv, causal=False, scale=scale)[:, 0]
    q2 = q.reshape(B, H * D)
    if q2.stride(1) != 1 or q2.stride(0) % 8 != 0 or q2.data_ptr() % 16 != 0:
        q2 = q2.contiguous()
    if scratch is None:
        S = decode_splits(B, Hkv, cache_k.shape[2])
        scratch = (torch.empty(B, H, S, D, device=q.device, dtype=torch.float32),
                   torch.empty(B, H, S, 2, device=q.device, dtype=torch.float32))
    if out is None:
        out = torch.empty(B, H * D, device=q.device, dtype=torch.bfloat16)
    _ext.ops().attn_decode(q2, cache_k, cache_v, pos, int(kv_len) if kv_len is not None else 0, 1, H, scale,
                           scratch[0], scratch[1], out)
    return out.view(B, H, D)


def attention_decode_paged(q, pool, block_table, seq_ids, seq_lens, n_kv_heads: int, len_add: int = 1, scale=None,
                           scratch=None, out=None, max_len: Optional[int] = None):
    """One query token per sequence over a PAGED cache (cache/paged.py): ``pool`` (n_pages, page_size, 2 * Hkv * D)
    holds K of every kv head then V per cached token, ``block_table`` (max_seqs, max_pages) the page ids,
    ``seq_ids`` (B,) the sequence of every query row, ``seq_lens`` (max_seqs,) the committed lengths, all on the
    device; ``len_add`` keys beyond the committed length are attended (1: the new token's row is written, the length
    not yet advanced). q (B, H, D). Returns (B, H, D)."""
    B, H, D = q.shape
    Hkv = n_kv_heads
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    cuda_ok = (q.is_cuda and q.dtype == torch.bfloat16 and pool.dtype == torch.bfloat16 and D in (64, 128, 256)
               and H % Hkv == 0 and (H // Hkv) in (1, 2, 4, 8) and pool.shape[-1] == 2 * Hkv * D)
    if not cuda_ok:
        outs = []
        ps = pool.shape[1]
        for b in range(B):
            sid = int(seq_ids[b])
            n = int(seq_lens[sid]) + len_add
            pos = torch.arange(n, device=pool.device)
            rows = pool[block_table[sid, (pos // ps).long()].long(), (pos % ps).long()]          # (n, 2 Hkv D)
            kk = rows[:, :Hkv * D].reshape(1, n, Hkv, D).to(q.dtype)
            vv = rows[:, Hkv * D:].reshape(1, n, Hkv, D).to(q.dtype)
            outs.append(attention_ref(q[b:b + 1, None], kk, vv, causal=False, scale=scale)[:, 0])
        return torch.cat(outs)
    q2 = q.reshape(B, H * D)
    if q2.stride(1) != 1 or q2.stride(0) % 8 != 0 or q2.data_ptr() % 16 != 0:
        q2 = q2.contiguous()
    if scratch is None:
        S = decode_splits(B, Hkv, max_len or block_table.shape[1] * pool.shape[1])
        scratch = (torch.empty(B, H, S, D, device=q.device, dtype=torch.float32),
                   torch.empty(B, H, S, 2, device=q.device, dtype=torch.float32))
    if out is None:
        out = torch.empty(B, H * D, device=q.device, dtype=torch.bfloat16)
    _ext.ops().attn_decode_paged(q2, pool, block_table, seq_ids, seq_lens, int(len_add), H, Hkv, scale, scratch[0],
                                 scratch[1], out)
    return out.view(B, H, D)


class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        out, lse = attn_fwd(q, k, v, causal, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.scale = causal, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = attn_bwd(q, k, v, out, _kernel_layout(dout), lse, ctx.causal, ctx.scale)
        return dq, dk, dv, None, None


def attn_bwd_chunked(q, k, v, out, dout, lse, causal=True, scale=None, chunk: Optional[int] = None):
    """Gradients from the forward kernel's (out, lse) with the probabilities recomputed one query
    chunk at a time, ALL heads of a sequence per step: batched library matmuls over the kv heads for the four
    products, and on CUDA one elementwise kernel that rewrites the bf16 scores and dO V^T in place as P and dS
    (chunks sized to about 8 GB of those two). A library-matmul cross-check of the backward kernels (tests) and
    the gradient path for tensors the kernels do not take; ``attention`` never calls it for CUDA bf16 inputs.
    q (B,T,H,D), k (B,T,Hkv,D), v (B,T,Hkv,Dv); lse (B,H,T) is the log2-sum-exp of scale*log2(e)*scores."""
    B, T, H, D = q.shape
    Hkv, Dv = k.shape[2], v.shape[3]
    g = H // Hkv
    scale = float(scale) if scale is not None else D ** -0.5
    c2 = scale * 1.4426950408889634
    fused = q.is_cuda and q.dtype == torch.bfloat16 and T % 8 == 0
    if chunk is None:
        # fused path: scores and dP are kept as bf16 and rewritten in place (4 bytes per score element);
        # library path: fp32 temporaries (about 16 bytes per element)
        budget = (1 << 33) // 4 if fused else (1 << 28)
        chunk = max(64, min(T, budget // max(1, H * T) // 64 * 64))
    dq = torch.empty_like(q)
    dk = torch.zeros(B, Hkv, T, D, device=q.device, dtype=torch.float32)
    dv = torch.zeros(B, Hkv, T, Dv, device=q.device, dtype=torch.float32)
    delta = (out.float() * dout.float()).sum(-1)          # (B,T,H)
    pos = torch.arange(T, device=q.device)
    for b in range(B):
        kb, vb = k[b].permute(1, 0, 2), v[b].permute(1, 0, 2)                    # (Hkv, T, D), (Hkv, T, Dv)
        for q0 in range(0, T, chunk):
            q1 = min(T, q0 + chunk)
            c = q1 - q0
            kv1 = q1 if causal else T
            kk, vv = kb[:, :kv1], vb[:, :kv1]
            # rows of a kv head: its g query heads one after the other, c positions each
            qs = q[b, q0:q1].reshape(c, Hkv, g, D).permute(1, 2, 0, 3).reshape(Hkv, g * c, D)
            do = dout[b, q0:q1].reshape(c, Hkv, g, Dv).permute(1, 2, 0, 3).reshape(Hkv, g * c, Dv)
            l2 = lse[b, :, q0:q1].reshape(Hkv, g * c, 1)
            dl = delta[b, q0:q1].t().reshape(Hkv, g * c, 1)
            if fused:
                # one elementwise kernel turns (scores, dO V^T) into (P, dS) in place
                pb = torch.matmul(qs, kk.transpose(1, 2))                                   # (Hkv, g*c, kv1) bf16
                ds = torch.matmul(do, vv.transpose(1, 2))
                _ext.ops().attn_bwd_probs(pb, ds, l2.contiguous(), dl.contiguous(), c, q0, scale, causal)
            else:
                p = torch.matmul(qs, kk.transpose(1, 2)).float().mul_(c2).sub_(l2).exp2_()  # (Hkv, g*c, kv1)
                if causal:
                    p.view(Hkv, g, c, kv1).masked_fill_(pos[None, :kv1] > pos[q0:q1, None], 0.0)
                ds = torch.matmul(do, vv.transpose(1, 2)).float().sub_(dl).mul_(p).mul_(scale).to(q.dtype)
                pb = p.to(q.dtype)
                del p
            dq[b, q0:q1] = torch.matmul(ds, kk).reshape(Hkv, g, c, D).permute(2, 0, 1, 3).reshape(c, H, D)
            dk[b, :, :kv1] += torch.matmul(ds.transpose(1, 2), qs)
            dv[b, :, :kv1] += torch.matmul(pb.transpose(1, 2), do)
    return dq, dk.permute(0, 2, 1, 3).to(k.dtype), dv.permute(0, 2, 1, 3).to(v.dtype)


def supports_cuda_kernel(q, k, v=None) -> bool:
    """True when forward and backward run on the tcgen05 kernels: bf16 on CUDA, self-attention lengths, head
    widths 64 / 128 / 256 or the MLA shape (q/k 192 wide, v 128 wide)."""
    d = q.shape[-1]
    dv = v.shape[-1] if v is not None else d
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[1] == k.shape[1] and
            ((d == dv and d in (64, 128, 256)) or (d == 192 and dv == 128)))


supports_cuda_forward = supports_cuda_kernel


def _kernel_layout(t):
    """The kernels take [B, T, H, D] views whose heads are contiguous column blocks of one row per token."""
    B, T, H, D = t.shape
    ok = (t.stride(3) == 1 and t.stride(2) == D and t.stride(0) == T * t.stride(1) and t.stride(1) % 8 == 0
          and t.data_ptr() % 16 == 0)
    return t if ok else t.contiguous()


def attention(q, k, v, causal: bool = True, scale: Optional[float] = None):
    """Softmax attention over [B,T,H,D] tensors (GQA when k/v have fewer heads). On CUDA in bf16, head widths
    64 / 128 / 256 and the MLA shape (192 / 128) run forward and backward on the tcgen05 kernels; anything else
    takes the dense fp32 reference."""
    if supports_cuda_kernel(q, k, v):
        return _AttnFn.apply(_kernel_layout(q), _kernel_layout(k), _kernel_layout(v), causal, scale)
    return attention_ref(q, k, v, causal, scale)


def attention_cached(q, cache_k, cache_v, kv_len: int, q_pos0: int, scale: Optional[float] = None):
    """Causal attention of q (B,T,H,D) at positions ``q_pos0 + i`` over the first ``kv_len`` rows of caches laid
    out as (B, Hkv, max_len, D) (jax_gpt/models/qwen35/gqa.py:88-119 attends over the whole padded buffer and
    masks). Inference path: no gradient. The tcgen05 forward kernel reads the cache in place when it is bf16."""
    d, dv = q.shape[-1], cache_v.shape[-1]
    if (q.is_cuda and q.dtype == torch.bfloat16 and cache_k.dtype == torch.bfloat16 and cache_k.is_contiguous()
            and cache_v.is_contiguous() and ((d == dv and d in (64, 128, 256)) or (d == 192 and dv == 128))):
        return attn_fwd_cached(_kernel_layout(q), cache_k, cache_v, kv_len, q_pos0, True, scale)[0]
    B = q.shape[0]
    kk = cache_k[:B, :, :kv_len].permute(0, 2, 1, 3).to(q.dtype)
    vv = cache_v[:B, :, :kv_len].permute(0, 2, 1, 3).to(q.dtype)
    return attention_ref(q, kk, vv, causal=True, scale=scale, q_pos0=q_pos0)


def mla_attention(q, k, v, scale: float):
    """Causal attention with different q/k and v head widths (MLA prefill: 192 / 128).
    q,k (B,T,H,dqk); v (B,T,H,dv)."""
    if supports_cuda_kernel(q, k, v):
        return _AttnFn.apply(_kernel_layout(q), _kernel_layout(k), _kernel_layout(v), True, scale)
    B, T, H, dqk = q.shape
    qf, kf, vf = [t.float().permute(0, 2, 1, 3) for t in (q, k, v)]
    s = (qf @ kf.transpose(-1, -2)) * scale
    mask = torch.ones(T, T, dtype=torch.bool, device=q.device).tril()
    p = torch.softmax(s.masked_fill(~mask, float("-inf")), dim=-1)
    return (p @ vf).permute(0, 2, 1, 3).to(q.dtype)
