"""Next-token losses of the function-style model families, in the form ``TreeTrainEngine`` expects
(``loss_fn(tree, tokens, targets)``). The reference has no training path for these models (its
trainer only knows GPT-2, jax_gpt/trainer/train_step.py:34-84); the loss is the same mean token
cross-entropy."""
from __future__ import annotations

import torch

from ..ops.fp8_linear import fp8_training
from ..ops.misc import cross_entropy_mean


def qwen35_loss_fn(config, ep=None, fp8: bool = False):
    """``ep``: None (all experts local), a process group (all-to-all path) or an ``EPMoERuntime``.
    ``fp8``: run the dense projections (forward, input and weight gradients) as block-scaled FP8 GEMMs."""
    from ..models.qwen35.model import forward

    def loss_fn(tree, tokens, targets):
        with fp8_training(fp8):
            logits, _ = forward(tree, tokens, config, ep_group=ep)
        return cross_entropy_mean(logits, targets, config.vocab_size)
    return loss_fn


def deepseek_v3_loss_fn(config, ep=None, fp8: bool = False):
    """``fp8``: the DeepSeek-V3 recipe for the dense projections (1x128 activation / 128x128 weight blocks in
    forward, dgrad and wgrad); the routed experts keep their own kernels."""
    from ..models.deepseek_v3.model import forward

    def loss_fn(tree, tokens, targets):
        with fp8_training(fp8):
            logits = forward(tree, tokens, config, ep=ep)
        return cross_entropy_mean(logits, targets, config.vocab_size)
    return loss_fn


def qwen35_unstack(path, tensor) -> int:
    """Leading layer axes of the Qwen3.5 tree (``TreeTrainEngine(unstack=...)``): everything under ``groups`` is
    stacked over the groups, the DeltaNet layers additionally over their position in the group."""
    if path[0] != "groups":
        return 0
    return 2 if "delta_layers" in path else 1


def deepseek_v3_unstack(path, tensor) -> int:
    """Leading layer axis of the DeepSeek-V3 tree: ``dense_layers`` and ``moe_layers`` are stacked over layers."""
    return 1 if path[0] in ("dense_layers", "moe_layers") else 0
