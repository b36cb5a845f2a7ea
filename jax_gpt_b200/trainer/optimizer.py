"""AdamW with warmup-cosine schedule, decay mask and global-norm clipping.

Chain and ordering of the reference (jax_gpt/trainer/optimizer.py:48-63): clip by global norm
FIRST, Adam moments (eps 1e-8, bias-corrected), decoupled weight decay on masked-in leaves,
then the learning rate. The mask leaves out any leaf whose path contains ``bias``,
``embedding`` or ``scale`` (jax_gpt/trainer/optimizer.py:23-33).

On CUDA the update of each leaf runs on the fused AdamW kernel; on CPU the same formula runs
in PyTorch. The fused GPT-2 engine bypasses the per-leaf loop and updates two flat ranges.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Optional

import torch

from ..models.gpt2.engine import lr_schedule
from ..ops import misc

NO_DECAY_TOKENS = ("bias", "embedding", "scale")


def _params_of(model) -> Dict[str, torch.Tensor]:
    if hasattr(model, "params") and isinstance(model.params, dict):
        return model.params
    if callable(getattr(model, "params", None)):
        return model.params()
    return dict(model.named_parameters())


def build_decay_mask(model) -> Dict[str, bool]:
    """path -> True if the leaf is weight-decayed."""
    mask = {}
    for name in _params_of(model):
        parts = name.split(".")
        mask[name] = not any(tok in part for part in parts for tok in NO_DECAY_TOKENS)
    return mask


@dataclass
class AdamWState:
    count: int
    mu: Dict[str, torch.Tensor]
    nu: Dict[str, torch.Tensor]


@dataclass
class AdamW:
    """The transformation object (``tx``): ``init(params)`` and ``update(grads, state, params)``."""
    learning_rate: float
    min_lr: float
    warmup_steps: int
    lr_decay_steps: int
    weight_decay: float
    beta1: float
    beta2: float
    grad_clip: float
    mask: Dict[str, bool] = field(default_factory=dict)
    eps: float = 1e-8

    def schedule(self, step: int) -> float:
        return lr_schedule(step, self.learning_rate, self.min_lr, self.warmup_steps, self.lr_decay_steps)

    def init(self, params: Dict[str, torch.Tensor]) -> AdamWState:
        return AdamWState(0, {k: torch.zeros_like(v, dtype=torch.float32) for k, v in params.items()},
                          {k: torch.zeros_like(v, dtype=torch.float32) for k, v in params.items()})

    @torch.no_grad()
    def update(self, grads: Dict[str, torch.Tensor], state: AdamWState, params: Dict[str, torch.Tensor], mesh=None,
               model_config=None, global_sq: Optional[torch.Tensor] = None):
        """Applies one step IN PLACE to ``params`` and the moments; returns (grad_norm, lr). With a tensor-parallel
        ``mesh`` the leaves are shards: the squared norms of the sharded leaves are summed over the group, those of
        the replicated leaves counted once, so every rank clips by the same global norm as a single process."""
        if global_sq is not None:
            # the caller already summed the squared gradient norm over its process group (pipeline stages)
            return self._apply(grads, state, params, global_sq.float().reshape(()).cpu())
        sq = None
        sq_sharded = None
        tp = mesh is not None and getattr(mesh, "group", None) is not None and mesh.size("tp") > 1
        for k, g in grads.items():
            s = (g.float() ** 2).sum()
            if tp and _is_tp_sharded(k, g, model_config, mesh):
                sq_sharded = s if sq_sharded is None else sq_sharded + s
            else:
                sq = s if sq is None else sq + s
        if sq_sharded is not None:
            import torch.distributed as dist
            dist.all_reduce(sq_sharded, group=mesh.group)
            sq = sq_sharded if sq is None else sq + sq_sharded
        return self._apply(grads, state, params, sq)

    def _apply(self, grads, state, params, sq):
        gnorm = float(sq.sqrt())
        lr = self.schedule(state.count)
        t = state.count + 1
        hp = torch.tensor([lr, 1 - self.beta1 ** t, 1 - self.beta2 ** t, 1.0], dtype=torch.float32)
        for k, p in params.items():
            g = grads[k]
            wd = self.weight_decay if self.mask.get(k, True) else 0.0
            if p.is_cuda and p.dtype == torch.float32 and p.is_contiguous():
                misc.adamw(p.view(-1), g.float().contiguous().view(-1), state.mu[k].view(-1), state.nu[k].view(-1),
                           hp.to(p.device), sq.reshape(1).to(p.device), beta1=self.beta1, beta2=self.beta2,
                           eps=self.eps, wd=wd, clip=self.grad_clip, zero_grad=False)
            else:
                pf = p.float()
                misc.adamw_ref(pf, g.float().clone(), state.mu[k], state.nu[k], hp, sq, self.beta1, self.beta2,
                               self.eps, wd, self.grad_clip, None, zero_grad=False)
                p.copy_(pf)
        state.count = t
        return gnorm, lr


def _is_tp_sharded(name: str, t: torch.Tensor, model_config, mesh) -> bool:
    """True when leaf ``name`` is a tensor-parallel shard under the trainer's rules (trainer/sharding.py)."""
    from .sharding import param_spec
    if "tp" not in param_spec(name, t.dim()):
        return False
    if model_config is None:
        return True
    from .sharding import shard_gpt2_tensor
    full_shape = _full_shape(name, model_config)
    return full_shape is None or tuple(t.shape) != tuple(full_shape)


def _full_shape(name: str, c):
    L, d, f, V = c.n_layers, c.d_model, c.d_ff, c.vocab_size
    return {"wte.embedding": (V, d), "h.attn.c_attn.kernel": (L, d, 3 * d), "h.attn.c_attn.bias": (L, 3 * d),
            "h.attn.c_proj.kernel": (L, d, d), "h.mlp.c_fc.kernel": (L, d, f), "h.mlp.c_fc.bias": (L, f),
            "h.mlp.c_proj.kernel": (L, f, d), "lm_head.kernel": (d, V)}.get(name)


def create_optimizer(model, config) -> AdamW:
    return AdamW(config.learning_rate, config.min_lr, config.warmup_steps, config.lr_decay_steps, config.weight_decay,
                 config.beta1, config.beta2, config.grad_clip, build_decay_mask(model))
