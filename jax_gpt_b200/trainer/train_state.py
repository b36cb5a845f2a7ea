"""Training state ``{step, model, tx, opt_state}`` (jax_gpt/trainer/train_state.py:7-34).

``engine`` is this runtime's addition: when the model is a GPT-2 on a CUDA device the state
carries the fused fixed-shape engine that owns the flat parameter, gradient and moment
buffers; ``model.params`` then aliases the engine's fp32 master views.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

import torch


@dataclass
class TrainState:
    step: int
    model: Any
    tx: Any
    opt_state: Any
    engine: Optional[Any] = None


def create_train_state(model, tx, *, train_config=None, device=None, dist_optimizer=None) -> TrainState:
    """``tx.init`` over the model's parameters. With ``train_config`` and a CUDA ``device`` a
    GPT-2 model is moved onto the fused engine (bf16 compute, fp32 master weights)."""
    from ..models.gpt2.model import GPT
    if (train_config is not None and device is not None and torch.device(device).type == "cuda" and isinstance(model, GPT)
            and model.config.dropout == 0.0):   # dropout > 0 trains under autograd: the engine's kernels carry no masks
        from ..models.gpt2.engine import GPT2TrainEngine
        c = train_config
        eng = GPT2TrainEngine(model.config, c.micro_batch_size, c.seq_len, device=device, lr=c.learning_rate,
                              min_lr=c.min_lr, warmup_steps=c.warmup_steps, lr_decay_steps=c.lr_decay_steps,
                              weight_decay=c.weight_decay, beta1=c.beta1, beta2=c.beta2, grad_clip=c.grad_clip,
                              init={k: v.detach().cpu() for k, v in model.params.items()},
                              use_cuda_graph=c.cuda_graph, dist_optimizer=dist_optimizer,
                              overlap_grad_reduce=getattr(c, "overlap_grad_reduce", False))
        # the model's tree aliases the engine's buffers: the fp32 master weights on one GPU; with a sharded optimizer
        # no rank holds those in full, so the tree aliases the (always current) bf16 compute copy instead and the
        # checkpoint manager gathers the fp32 values when it saves
        model.params = eng.params() if dist_optimizer is None else eng.flat.tree(eng.flat.compute)
        from .optimizer import AdamWState
        st = eng.opt_state()
        return TrainState(0, model, tx, AdamWState(0, st["mu"], st["nu"]), eng)
    params = model.params if isinstance(getattr(model, "params", None), dict) else dict(model.named_parameters())
    return TrainState(0, model, tx, tx.init(params), None)
