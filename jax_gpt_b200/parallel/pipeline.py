"""Pipeline parallelism: a 1F1B schedule over point-to-point sends and receives.

The layers of a model are split into ``pp`` contiguous stages, one per rank of the pipeline
group; a global batch is cut into micro-batches that flow through the stages. Activations go
forward and gradients go backward with ``torch.distributed`` p2p operations (NCCL on GPUs,
gloo in the CPU tests), posted with ``batch_isend_irecv`` so that a stage's send of
micro-batch i overlaps its compute on micro-batch i+1. This is the one place where the product
path stays on NCCL: the messages are whole activation tensors between neighbouring stages,
not a collective that could be fused into a GEMM.

The reference has no pipeline parallelism (``assert config.pp == 1``,
jax_gpt/trainer/sharding.py:68; hooks are only discussed in phase2_plan.md:598-614).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


def split_layers(n_layers: int, n_stages: int) -> List[range]:
    """Contiguous, as-even-as-possible layer ranges; earlier stages get the remainder."""
    base, rem = divmod(n_layers, n_stages)
    out, start = [], 0
    for s in range(n_stages):
        n = base + (1 if s < rem else 0)
        out.append(range(start, start + n))
        start += n
    return out


def one_f_one_b_order(stage: int, n_stages: int, n_micro: int) -> List[tuple]:
    """The sequence of ('F', i) / ('B', i) steps a stage executes: warm-up forwards, steady
    one-forward-one-backward, cool-down backwards."""
    warm = min(n_stages - stage - 1, n_micro)
    order = [("F", i) for i in range(warm)]
    f, b = warm, 0
    while f < n_micro:
        order.append(("F", f))
        order.append(("B", b))
        f += 1
        b += 1
    while b < n_micro:
        order.append(("B", b))
        b += 1
    return order


@dataclass
class PipelineStage:
    """One stage. ``forward_fn(x_or_tokens, micro_batch_index) -> activation`` (the last stage
    returns the scalar loss of the micro-batch). ``act_shape``/``act_dtype`` describe the tensor
    passed between stages."""
    forward_fn: Callable
    params: Sequence[torch.Tensor]
    act_shape: tuple
    act_dtype: torch.dtype
    group: Optional[object] = None
    device: Optional[torch.device] = None

    def __post_init__(self):
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.first, self.last = self.rank == 0, self.rank == self.world - 1
        self.device = self.device or torch.device("cpu")

    def _peer(self, delta: int) -> int:
        r = self.rank + delta
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    def run(self, micro_inputs: Sequence, loss_scale: Optional[float] = None):
        """Runs one optimizer step's worth of micro-batches with the 1F1B order. ``micro_inputs``
        are this stage's own inputs (tokens on the first stage, targets on the last; None
        elsewhere). Gradients accumulate in ``p.grad``. Returns the mean loss on the last stage."""
        n_micro = len(micro_inputs)
        scale = loss_scale if loss_scale is not None else 1.0 / n_micro
        inputs, outputs = {}, {}
        pending: List = []
        losses = []

        def flush():
            for w in pending:
                w.wait()
            pending.clear()

        for kind, i in one_f_one_b_order(self.rank, self.world, n_micro):
            if kind == "F":
                if self.first:
                    x = micro_inputs[i]
                else:
                    x = torch.empty(self.act_shape, dtype=self.act_dtype, device=self.device)
                    for w in dist.batch_isend_irecv([dist.P2POp(dist.irecv, x, self._peer(-1), self.group)]):
                        w.wait()
                    x.requires_grad_(True)
                inputs[i] = x
                if self.last and not self.first:
                    y = self.forward_fn((x, micro_inputs[i]), i)   # (activation from upstream, targets)
                else:
                    y = self.forward_fn(x, i)
                outputs[i] = y
                if self.last:
                    losses.append(y.detach())
                else:
                    flush()
                    pending.extend(dist.batch_isend_irecv([dist.P2POp(dist.isend, y.detach().contiguous(),
                                                                      self._peer(+1), self.group)]))
            else:
                y = outputs.pop(i)
                if self.last:
                    (y * scale).backward()
                else:
                    gy = torch.empty(self.act_shape, dtype=self.act_dtype, device=self.device)
                    for w in dist.batch_isend_irecv([dist.P2POp(dist.irecv, gy, self._peer(+1), self.group)]):
                        w.wait()
                    y.backward(gy)
                x = inputs.pop(i)
                if not self.first:
                    flush()
                    pending.extend(dist.batch_isend_irecv([dist.P2POp(dist.isend, x.grad.contiguous(), self._peer(-1),
                                                                      self.group)]))
        flush()
        return torch.stack(losses).mean() if losses else None


def gpt2_stage(model, stage: int, n_stages: int, micro_batch: int, seq_len: int, group=None, device=None,
               act_dtype: Optional[torch.dtype] = None) -> PipelineStage:
    """The pipeline stage ``stage`` of a GPT-2 (models/gpt2/model.py): its contiguous range of blocks, plus the
    embeddings on the first stage and the final norm, tied head and mean cross-entropy on the last. ``model`` holds
    the full parameter dict on every rank (only the stage's layers are used and receive gradients). The last stage
    takes ``targets`` as its micro-batch input, the first stage ``tokens``."""
    from ..ops import norm as norm_ops
    cfg, p = model.config, model.params
    layers = split_layers(cfg.n_layers, n_stages)[stage]
    first, last = stage == 0, stage == n_stages - 1
    dtype = act_dtype or p["wte.embedding"].dtype

    def fwd(inp, i):
        x, tgt = (inp if (last and not first) else (inp, None))
        if first:
            tokens = x if not last else x[0]
            tgt = None if not last else inp[1]
            T = tokens.shape[1]
            x = p["wte.embedding"][tokens.long()] + p["wpe.embedding"][:T]
        for l in layers:
            x, _, _ = model._block(l, x, None, None, 0, None)
        if not last:
            return x
        h = norm_ops.layer_norm(x, p["ln_f.layer_norm.scale"], p["ln_f.layer_norm.bias"], 1e-5)
        logits = (h @ p["wte.embedding"].t()).float()
        return torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]), tgt.reshape(-1).long())

    used = [v for k, v in p.items() if not k.startswith("h.")] + [v for k, v in p.items() if k.startswith("h.")]
    return PipelineStage(fwd, used, (micro_batch, seq_len, cfg.d_model), dtype, group, device)


def sync_tied_embedding_grad(model, group=None) -> None:
    """GPT-2 ties the token embedding to the output head, so under pipeline parallelism its gradient is split between
    the first stage (lookup) and the last stage (head). Sums it over the pipeline group (middle stages add zeros);
    call after ``PipelineStage.run`` and before the optimizer step."""
    w = model.params["wte.embedding"]
    if w.grad is None:
        w.grad = torch.zeros_like(w)
    dist.all_reduce(w.grad, group=group)
