"""Embedding, fused cross-entropy, bias gradient and optimizer kernels with fp32 references.

Loss semantics: mean softmax cross-entropy with integer labels computed in fp32
(jax_gpt/trainer/train_step.py:56-60). AdamW chain: clip by global norm, Adam moments with
eps 1e-8, decoupled masked weight decay, learning-rate scaling (jax_gpt/trainer/optimizer.py:48-63).
"""
from __future__ import annotations

import torch

from .. import _ext


def embed_ref(idx, wte, wpe=None, pos0: int = 0):
    out = wte[idx.long()]
    if wpe is not None:
        T = idx.shape[-1]
        out = out + wpe[pos0:pos0 + T]
    return out


def embed_fwd(idx, wte, wpe=None, pos0: int = 0, out=None):
    """idx [B,T] int32 -> [B,T,D] = wte[idx] (+ wpe[pos0 + t])."""
    if not idx.is_cuda:
        return embed_ref(idx, wte, wpe, pos0)
    B, T = idx.shape
    if out is None:
        out = torch.empty(B, T, wte.shape[1], device=idx.device, dtype=wte.dtype)
    _ext.ops().embed_fwd(idx.contiguous(), wte, wpe, out, T, pos0)
    return out


def embed_bwd(idx, dout, dwte, dwpe=None, pos0: int = 0):
    """Accumulates the embedding gradients into fp32 ``dwte`` / ``dwpe``."""
    B, T = idx.shape
    _ext.ops().embed_bwd(idx.contiguous(), dout.contiguous(), dwte, dwpe, T, pos0)


def cross_entropy_ref(logits, targets, vocab: int):
    lf = logits[..., :vocab].float()
    return torch.nn.functional.cross_entropy(lf.reshape(-1, vocab), targets.reshape(-1).long(), reduction="none",
                                             ignore_index=-1)


def cross_entropy_fwd_bwd(logits, targets, vocab: int, scale: float, write_grad: bool = True, loss=None):
    """Per-row loss; overwrites ``logits`` [M, ldl] with ``scale * (softmax - onehot)`` in place."""
    M = logits.shape[0]
    if loss is None:
        loss = torch.empty(M, device=logits.device, dtype=torch.float32)
    _ext.ops().ce_fwd_bwd(logits, targets, loss, vocab, scale, write_grad)
    return loss


class _CrossEntropyMeanFn(torch.autograd.Function):
    """Mean token cross-entropy on the fused kernel: one pass produces the per-row losses and overwrites
    the logits with ``(softmax - onehot) / n_valid``; the backward hands that buffer on."""

    @staticmethod
    def forward(ctx, logits, targets, vocab):
        n_valid = (targets >= 0).sum().clamp_min(1).float()
        rows = cross_entropy_fwd_bwd(logits, targets, vocab, 1.0, True)
        ctx.save_for_backward(logits, n_valid)
        return rows.sum() / n_valid

    @staticmethod
    def backward(ctx, g):
        dlogits, n_valid = ctx.saved_tensors
        return dlogits.mul_((g / n_valid).to(dlogits.dtype)), None, None


def cross_entropy_mean(logits, targets, vocab=None):
    """Mean cross-entropy over rows with target >= 0. logits (M, V') with V' >= vocab (padding columns
    ignored). CUDA bf16 logits are CONSUMED (overwritten with their gradient)."""
    vocab = logits.shape[-1] if vocab is None else vocab
    logits = logits.reshape(-1, logits.shape[-1])
    targets = targets.reshape(-1)
    if logits.is_cuda and logits.dtype == torch.bfloat16 and logits.stride(1) == 1:
        return _CrossEntropyMeanFn.apply(logits, targets.to(torch.int32).contiguous(), vocab)
    rows = cross_entropy_ref(logits, targets, vocab)
    return rows.sum() / (targets >= 0).sum().clamp_min(1)


def bias_grad(dy, out=None):
    """Column sums of a [M,N] bf16 matrix, accumulated into an fp32 vector."""
    if not dy.is_cuda:
        s = dy.float().sum(0)
        return s if out is None else out.add_(s)
    if out is None:
        out = torch.zeros(dy.shape[1], device=dy.device, dtype=torch.float32)
    _ext.ops().bias_grad(dy, out)
    return out


def sumsq(g, out=None):
    if not g.is_cuda:
        s = (g.float() ** 2).sum()
        return s if out is None else out.add_(s)
    if out is None:
        out = torch.zeros(1, device=g.device, dtype=torch.float32)
    _ext.ops().sumsq(g, out)
    return out


def adamw_ref(p, g, m, v, hp, gnorm_sq, beta1, beta2, eps, wd, clip, p_bf16=None, zero_grad=True):
    """Reference of the fused AdamW step; ``hp = [lr, 1-beta1^t, 1-beta2^t, grad_scale]``."""
    lr, bc1, bc2, gscale = [float(x) for x in hp]
    coef = gscale
    if gnorm_sq is not None and clip > 0:
        norm = float(gnorm_sq) ** 0.5 * gscale
        coef *= min(1.0, clip / (norm + 1e-6))
    gi = g * coef
    m.mul_(beta1).add_(gi, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gi, gi, value=1 - beta2)
    u = (m / bc1) / ((v / bc2).sqrt() + eps) + wd * p
    p.sub_(lr * u)
    if p_bf16 is not None:
        p_bf16.copy_(p)
    if zero_grad:
        g.zero_()


def adamw_bf16_state(p, g, m, v, hp, gnorm_sq=None, *, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.0, clip=0.0,
                     zero_grad=True, seed=0):
    """AdamW whose whole state is bf16: ``p`` (the weights, no fp32 master), ``m`` and ``v``; ``g`` fp32. Stores are
    rounded stochastically on CUDA (``seed`` should change every step); the CPU path rounds to nearest."""
    if p.is_cuda:
        _ext.ops().adamw_bf16_state(p, g, m, v, hp, gnorm_sq, beta1, beta2, eps, wd, clip, zero_grad, int(seed) & 0x7fffffff)
        return
    pf, mf, vf = p.float(), m.float(), v.float()
    adamw_ref(pf, g.clone(), mf, vf, hp, gnorm_sq, beta1, beta2, eps, wd, clip, None, zero_grad=False)
    p.copy_(pf)
    m.copy_(mf)
    v.copy_(vf)
    if zero_grad:
        g.zero_()


def adamw(p, g, m, v, hp, gnorm_sq=None, *, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.0, clip=0.0, p_bf16=None,
          zero_grad=True):
    """Fused AdamW over flat fp32 buffers; also refreshes the bf16 compute copy and zeroes the grad."""
    if not p.is_cuda:
        return adamw_ref(p, g, m, v, hp, gnorm_sq, beta1, beta2, eps, wd, clip, p_bf16, zero_grad)
    _ext.ops().adamw(p, g, m, v, p_bf16, hp, gnorm_sq, beta1, beta2, eps, wd, clip, zero_grad)
