"""Causal / full softmax attention: tcgen05 flash kernels on CUDA, dense fp32 reference elsewhere.

The reference materialises (B,H,T,S) scores (jax_gpt/models/gpt2/model.py:167-176,
jax_gpt/models/qwen35/gqa.py:103-119); the kernels tile the same math with an online softmax.
Tensors are [B, T, H, D]; q/k/v may be column slices of one fused projection output.
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
    """Raw CUDA backward. Returns (dq, dk, dv) in bf16 with the layouts of q/k/v."""
    B, T, H, D = q.shape
    Hkv = k.shape[2]
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
        dv = torch.empty(B, T, Hkv, D, device=q.device, dtype=torch.bfloat16)
    _ext.ops().attn_bwd(_as2d(q), _as2d(k), _as2d(v), _as2d(out), _as2d(dout), lse, delta, dq_accum, _as2d(dk),
                        _as2d(dv), B, T, H, Hkv, D, scale, causal)
    _ext.ops().cast_rows(dq_accum, _as2d(dq))
    return dq, dk, dv


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
        dq, dk, dv = attn_bwd(q, k, v, out, dout.contiguous(), lse, ctx.causal, ctx.scale)
        return dq, dk, dv, None, None


def attn_bwd_chunked(q, k, v, out, dout, lse, causal=True, scale=None, chunk: Optional[int] = None):
    """Gradients from the forward kernel's (out, lse) with the probabilities recomputed one query
    chunk at a time, ALL heads of a sequence per step: batched library matmuls over the kv heads for the four
    products, and on CUDA one elementwise kernel that rewrites the bf16 scores and dO V^T in place as P and dS
    (chunks sized to about 8 GB of those two). Covers the head widths that have a forward kernel but no
    tensor-core backward kernel: 256 and the MLA shape 192 / 128.
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


class _AttnFwdKernelFn(torch.autograd.Function):
    """Forward on the tcgen05 kernel, backward by chunked recomputation (head widths without a backward kernel)."""

    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        out, lse = attn_fwd(q, k, v, causal, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.scale = causal, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = attn_bwd_chunked(q, k, v, out, dout.contiguous(), lse, ctx.causal, ctx.scale)
        return dq, dk, dv, None, None


def supports_cuda_kernel(q, k) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128) and q.shape[1] == k.shape[1])


def supports_cuda_forward(q, k, v) -> bool:
    d, dv = q.shape[-1], v.shape[-1]
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[1] == k.shape[1] and
            ((d == dv and d in (64, 128, 256)) or (d == 192 and dv == 128)))


def attention(q, k, v, causal: bool = True, scale: Optional[float] = None):
    """Softmax attention over [B,T,H,D] tensors (GQA when k/v have fewer heads). Head widths
    64 / 128 run forward and backward on the tcgen05 kernels; 256 and the MLA shape (192 / 128)
    run the forward kernel, and their gradients come from a chunked recomputation."""
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    if supports_cuda_kernel(q, k) and v.shape[-1] == q.shape[-1]:
        return _AttnFn.apply(q, k, v, causal, scale)
    if supports_cuda_forward(q, k, v):
        if needs_grad:
            return _AttnFwdKernelFn.apply(q.contiguous(), k.contiguous(), v.contiguous(), causal, scale)
        return attn_fwd(q.contiguous(), k.contiguous(), v.contiguous(), causal, scale)[0]
    return attention_ref(q, k, v, causal, scale)


def mla_attention(q, k, v, scale: float):
    """Causal attention with different q/k and v head widths (MLA prefill: 192 / 128).
    q,k (B,T,H,dqk); v (B,T,H,dv)."""
    if supports_cuda_forward(q, k, v):
        if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
            return _AttnFwdKernelFn.apply(q.contiguous(), k.contiguous(), v.contiguous(), True, scale)
        return attn_fwd(q.contiguous(), k.contiguous(), v.contiguous(), True, scale)[0]
    B, T, H, dqk = q.shape
    qf, kf, vf = [t.float().permute(0, 2, 1, 3) for t in (q, k, v)]
    s = (qf @ kf.transpose(-1, -2)) * scale
    mask = torch.ones(T, T, dtype=torch.bool, device=q.device).tril()
    p = torch.softmax(s.masked_fill(~mask, float("-inf")), dim=-1)
    return (p @ vf).permute(0, 2, 1, 3).to(q.dtype)
