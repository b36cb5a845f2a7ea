"""train / eval steps with the reference's signatures (jax_gpt/trainer/train_step.py:34-165).

``train_step(state, batch, mesh=None) -> (state, {'loss', 'grad_norm', 'lr'})`` (``mesh``: a
``trainer.sharding.DeviceMesh``; with tensor-parallel shards in the state the model runs its TP forward and the
clipping norm is the global one): forward,
fp32 mean softmax cross-entropy with integer labels, gradients, global norm, AdamW update,
step + 1. ``batch`` is ``(x, y)`` of shape (B, T). With a fused engine in the state the whole
step is a CUDA-graph replay and the returned metrics are device tensors (read them with
``float()`` when needed); otherwise PyTorch autograd differentiates the model.
"""
from __future__ import annotations

from typing import Sequence

import torch

from .train_state import TrainState


def _loss_fn(model, x, y, mesh=None):
    logits, _ = model(x, deterministic=False, mesh=mesh)
    lf = logits.float()
    return torch.nn.functional.cross_entropy(lf.reshape(-1, lf.shape[-1]), y.reshape(-1).long())


def _autograd_grads(model, micro_batches, mesh=None):
    params = model.params
    leaves = list(params.values())
    for p in leaves:
        p.requires_grad_(True)
    total = 0.0
    sums = None
    for x, y in micro_batches:
        loss = _loss_fn(model, x, y, mesh)
        grads = torch.autograd.grad(loss, leaves, allow_unused=True)
        grads = [g if g is not None else torch.zeros_like(p) for g, p in zip(grads, leaves)]
        sums = grads if sums is None else [a + b for a, b in zip(sums, grads)]
        total = total + loss.detach()
    n = len(micro_batches)
    for p in leaves:
        p.requires_grad_(False)
    return total / n, {k: g / n for k, g in zip(params.keys(), sums)}


def train_step_with_accumulation(state: TrainState, micro_batches: Sequence, mesh=None):
    """Sums gradients over the micro-batches, scales by 1/n, applies ONE optimizer update."""
    if state.engine is not None:
        eng = state.engine
        for x, y in micro_batches:
            eng.micro_step(x, y)
        out = eng.apply_gradients()
        state.step += 1
        state.opt_state.count = eng.step_count
        gn = out["grad_norm_sq"].sqrt() * out["grad_scale"]
        return state, {"loss": out["loss"], "grad_norm": gn, "lr": out["lr"]}
    loss, grads = _autograd_grads(state.model, micro_batches, mesh)
    gnorm, lr = state.tx.update(grads, state.opt_state, state.model.params, mesh=mesh,
                                model_config=getattr(state.model, "config", None))
    state.step += 1
    return state, {"loss": loss, "grad_norm": gnorm, "lr": lr}


def train_step(state: TrainState, batch, mesh=None):
    return train_step_with_accumulation(state, [batch], mesh)


@torch.no_grad()
def eval_step(model, batch, engine=None):
    """Loss only; parameters untouched."""
    x, y = batch
    if engine is not None:
        return engine.eval_loss(x, y)
    logits, _ = model(x, deterministic=True)
    lf = logits.float()
    return torch.nn.functional.cross_entropy(lf.reshape(-1, lf.shape[-1]), y.reshape(-1).long())


jitted_eval_step = eval_step
