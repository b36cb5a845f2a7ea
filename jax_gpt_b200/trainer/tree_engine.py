"""Training engine for models written as functions over a nested parameter dict (the Qwen3.5
and DeepSeek-V3 families): flat fp32 master / compute-dtype / fp32 gradient buffers with the
tree's leaves as views, autograd for the backward pass, the fused AdamW kernels for the update.

Two parameter classes:

* dense leaves are replicated over the data-parallel ranks. Their gradients are accumulated into one
  flat fp32 buffer by post-accumulate hooks, and the update is either the single-GPU AdamW kernel
  or a sharded optimizer of parallel/fsdp.py (gradient reduce-scatter + AdamW + parameter all-gather
  in one kernel over NVLink);
* expert-parallel leaves (``local(path)`` true) exist only on their owner. They stay outside
  autograd: the fused MoE backward kernel adds their fp32 gradients into the ``<name>@grad``
  buffers that sit beside them in the tree, and they are updated locally. Their squared norm joins
  the global clipping norm.

The optimizer chain is the reference's (jax_gpt/trainer/optimizer.py:48-63): global-norm clip,
Adam, decoupled weight decay on >=2-D weights, schedule.
"""
from __future__ import annotations

import math
from types import SimpleNamespace
from typing import Callable, Dict, Optional

import torch

from ..ops import misc
from .optimizer import lr_schedule


def _walk(tree, prefix=()):
    for k in sorted(tree.keys()):
        v = tree[k]
        if isinstance(v, dict):
            yield from _walk(v, prefix + (k,))
        else:
            yield prefix + (k,), v


def _set(tree, path, value):
    for k in path[:-1]:
        tree = tree.setdefault(k, {})
    tree[path[-1]] = value


def default_decay(path, t) -> bool:
    """Weight decay on matrices only (norm scales, biases, per-head vectors are exempt)."""
    return t.dim() >= 2 and "norm" not in path[-1]


def _drop(tree: dict, path) -> None:
    """Removes a leaf from a nested dict (its storage is freed once nothing else refers to it)."""
    node = tree
    for k in path[:-1]:
        node = node[k]
    node.pop(path[-1], None)


class TreeTrainEngine:
    def __init__(self, params: dict, loss_fn: Callable, *, device=None, compute_dtype=torch.bfloat16,
                 local: Optional[Callable] = None, decay: Callable = default_decay, lr: float = 3e-4,
                 min_lr: float = 3e-5, warmup_steps: int = 100, lr_decay_steps: int = 10000, weight_decay: float = 0.1,
                 beta1: float = 0.9, beta2: float = 0.95, grad_clip: float = 1.0, dist_optimizer=None,
                 dp_world: int = 1, unstack: Optional[Callable] = None, local_state_dtype=torch.float32,
                 consume_params: bool = False):
        """``params``: nested dict of tensors (any device / dtype; copied). ``loss_fn(tree, *batch)``
        returns a scalar. ``local(path, tensor)`` marks expert-parallel leaves. ``unstack(path, tensor)`` gives
        the number of leading (layer) axes of a dense leaf that the model indexes one slice at a time: the tree then
        holds nested lists of per-slice autograd leaves instead of one stacked leaf, so that a layer's gradient is
        added to its own slice of the flat buffer (a stacked leaf receives one FULL-size gradient per slice from
        the select-backward of every layer, which costs layers^2 traffic).

        ``local_state_dtype=torch.bfloat16`` keeps the expert-parallel leaves WITHOUT an fp32 master and with bf16
        moments (stochastically rounded AdamW, csrc/elementwise.cu): 6 bytes of state per expert parameter instead
        of 16 plus the fp32 gradient, which is what lets the 512-expert / 48-layer benchmark shape fit eight GPUs.
        ``consume_params=True`` frees every leaf of ``params`` as soon as it has been copied into the flat buffers
        (the tree is emptied), so that a model initialised on the device is not held twice."""
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.loss_fn = loss_fn
        self.hyper = dict(lr=lr, min_lr=min_lr, warmup=warmup_steps, decay=lr_decay_steps, wd=weight_decay,
                          b1=beta1, b2=beta2, clip=grad_clip)
        self.dist_optimizer = dist_optimizer
        self.dp_world = dist_optimizer.world if dist_optimizer is not None else dp_world
        leaves = list(_walk(params))
        is_local = (lambda p, t: False) if local is None else local
        dense = [(p, t) for p, t in leaves if not is_local(p, t)]
        loc = [(p, t) for p, t in leaves if is_local(p, t)]
        dense = [x for x in dense if decay(*x)] + [x for x in dense if not decay(*x)]
        n_dec = sum(1 for x in dense if decay(*x))
        dev = self.device

        # ---- dense group: [decay | no decay], every view 256-byte aligned ----
        self.offsets: Dict[tuple, tuple] = {}
        off = 0
        n_decay = 0
        for i, (p, t) in enumerate(dense):
            self.offsets[p] = (off, t.numel(), tuple(t.shape))
            off += (t.numel() + 63) // 64 * 64
            if i == n_dec - 1:
                n_decay = off
        total = (off + 511) // 512 * 512
        alloc_c = getattr(dist_optimizer, "alloc_compute", None)
        alloc_g = getattr(dist_optimizer, "alloc_grad", None)
        master = torch.zeros(total, device=dev, dtype=torch.float32)
        if alloc_c is not None and compute_dtype == torch.bfloat16:
            compute = alloc_c(total)
        else:
            compute = torch.zeros(total, device=dev, dtype=compute_dtype)
        grad = alloc_g(total) if alloc_g is not None else torch.zeros(total, device=dev, dtype=torch.float32)
        del leaves
        for i, (p, t) in enumerate(dense):
            o, n, _ = self.offsets[p]
            master[o:o + n].copy_(t.reshape(-1).to(torch.float32))
            if consume_params:          # keep only the shape: the caller's tree and these lists let go of the storage
                _drop(params, p)
                dense[i] = (p, torch.empty(t.shape, device="meta", dtype=t.dtype))
        del t
        compute.copy_(master)
        grad.zero_()
        self.flat = SimpleNamespace(total=total, n_decay=n_decay, master=master, compute=compute, grad=grad)

        # ---- expert-parallel group (all weight-decayed matrices) ----
        self.local_offsets: Dict[tuple, tuple] = {}
        off = 0
        for p, t in loc:
            self.local_offsets[p] = (off, t.numel(), tuple(t.shape))
            off += (t.numel() + 63) // 64 * 64
        self.local_total = off
        self.local_lowmem = bool(off) and local_state_dtype == torch.bfloat16 and compute_dtype == torch.bfloat16
        if off:
            self.local_compute = torch.zeros(off, device=dev, dtype=compute_dtype)
            self.local_grad = torch.zeros(off, device=dev, dtype=torch.float32)
            sdt = torch.bfloat16 if self.local_lowmem else torch.float32
            self.local_m = torch.zeros(off, device=dev, dtype=sdt)
            self.local_v = torch.zeros(off, device=dev, dtype=sdt)
            # without an fp32 master the bf16 compute copy IS the master
            self.local_master = self.local_compute if self.local_lowmem else torch.zeros(off, device=dev, dtype=torch.float32)
            for i, (p, t) in enumerate(loc):
                o, n, _ = self.local_offsets[p]
                self.local_master[o:o + n].copy_(t.reshape(-1).to(self.local_master.dtype))
                if consume_params:
                    _drop(params, p)
                    loc[i] = (p, torch.empty(t.shape, device="meta", dtype=t.dtype))
            del t
            if not self.local_lowmem:
                self.local_compute.copy_(self.local_master)
        self.local_sq = torch.zeros(1, device=dev, dtype=torch.float32)

        # ---- the tree the model sees ----
        self.tree: dict = {}
        self._leaf_params = []
        def make_leaves(cview, gview, depth):
            if depth == 0:
                leaf = cview.requires_grad_(True)
                leaf.register_post_accumulate_grad_hook(self._make_hook(gview))
                if leaf.is_cuda and leaf.dim() == 2:
                    leaf.grad_buf = gview    # ops.gemm's weight-gradient GEMM accumulates straight into the flat buffer
                self._leaf_params.append(leaf)
                return leaf
            return [make_leaves(cview[i], gview[i], depth - 1) for i in range(cview.shape[0])]

        for p, t in dense:
            o, n, shape = self.offsets[p]
            depth = min(int(unstack(p, t)), len(shape) - 1) if unstack is not None else 0
            _set(self.tree, p, make_leaves(compute[o:o + n].view(shape), grad[o:o + n].view(shape), max(depth, 0)))
        for p, _ in loc:
            o, n, shape = self.local_offsets[p]
            _set(self.tree, p, self.local_compute[o:o + n].view(shape))
            _set(self.tree, p[:-1] + (p[-1] + "@grad",), self.local_grad[o:o + n].view(shape))

        if dist_optimizer is not None:
            dist_optimizer.attach(self)
            self.m = self.v = None
        else:
            self.m = torch.zeros(total, device=dev, dtype=torch.float32)
            self.v = torch.zeros(total, device=dev, dtype=torch.float32)
        self.gnorm_sq = torch.zeros(1, device=dev, dtype=torch.float32)
        self.hp = torch.zeros(4, device=dev, dtype=torch.float32)
        self._hp_host = torch.zeros(4, dtype=torch.float32)
        if dev.type == "cuda":
            self._hp_host = self._hp_host.pin_memory()
        self.step_count = 0
        self._micro = 0
        self.loss_sum = torch.zeros((), device=dev, dtype=torch.float32)

    @staticmethod
    def _make_hook(gview):
        def hook(param):
            if param.grad is not None:   # a function may return no gradient for the leaf (autograd still calls the hook)
                gview.add_(param.grad)   # bf16 -> fp32 accumulate
                param.grad = None
        return hook

    # ------------------------------------------------------------------------------------------
    def micro_step(self, *batch):
        """Forward + backward of one micro-batch; gradients accumulate. Returns the detached loss."""
        loss = self.loss_fn(self.tree, *batch)
        loss.backward()
        self.loss_sum += loss.detach().float()
        self._micro += 1
        return loss.detach()

    def _set_hyper(self, n_micro: int):
        h = self.hyper
        t = self.step_count + 1
        lr = lr_schedule(self.step_count, h["lr"], h["min_lr"], h["warmup"], h["decay"])
        self._hp_host[0] = lr
        self._hp_host[1] = 1.0 - h["b1"] ** t
        self._hp_host[2] = 1.0 - h["b2"] ** t
        self._hp_host[3] = 1.0 / (n_micro * self.dp_world)
        self.hp.copy_(self._hp_host, non_blocking=True)
        return lr

    def apply_gradients(self):
        h = self.hyper
        n = max(1, self._micro)
        lr = self._set_hyper(n)
        fl = self.flat
        extra = None
        if self.local_total:
            self.local_sq.zero_()
            misc.sumsq(self.local_grad, self.local_sq)
            extra = self.local_sq
        if self.dist_optimizer is not None:
            self.dist_optimizer.step(self, extra_sq=extra) if extra is not None else self.dist_optimizer.step(self)
            gsq = self.dist_optimizer.grad_norm_sq()
        else:
            self.gnorm_sq.zero_()
            misc.sumsq(fl.grad, self.gnorm_sq)
            if extra is not None:
                if self.dp_world > 1:   # expert gradients of the other ranks belong to the global norm too
                    import torch.distributed as dist
                    dist.all_reduce(extra)
                self.gnorm_sq += extra
            gsq = self.gnorm_sq
            nd = fl.n_decay
            kw = dict(beta1=h["b1"], beta2=h["b2"], eps=1e-8, clip=h["clip"])
            cdt = fl.compute.dtype
            pb = (lambda a, b: fl.compute[a:b]) if cdt == torch.bfloat16 else (lambda a, b: None)
            if nd:
                misc.adamw(fl.master[:nd], fl.grad[:nd], self.m[:nd], self.v[:nd], self.hp, gsq, wd=h["wd"],
                           p_bf16=pb(0, nd), **kw)
            if fl.total > nd:
                misc.adamw(fl.master[nd:], fl.grad[nd:], self.m[nd:], self.v[nd:], self.hp, gsq, wd=0.0,
                           p_bf16=pb(nd, fl.total), **kw)
            if cdt != torch.bfloat16:
                fl.compute.copy_(fl.master)
        if self.local_total and self.local_lowmem:
            misc.adamw_bf16_state(self.local_compute, self.local_grad, self.local_m, self.local_v, self.hp, gsq,
                                  beta1=h["b1"], beta2=h["b2"], eps=1e-8, wd=h["wd"], clip=h["clip"],
                                  seed=0x9e3779b1 * (self.step_count + 1))
        elif self.local_total:
            lb = self.local_compute if self.local_compute.dtype == torch.bfloat16 else None
            misc.adamw(self.local_master, self.local_grad, self.local_m, self.local_v, self.hp, gsq, beta1=h["b1"],
                       beta2=h["b2"], eps=1e-8, wd=h["wd"], clip=h["clip"], p_bf16=lb)
            if lb is None:
                self.local_compute.copy_(self.local_master)
        self.step_count += 1
        self._micro = 0
        loss = self.loss_sum / n
        self.loss_sum = torch.zeros_like(self.loss_sum)
        return {"loss": loss, "grad_norm_sq": gsq, "lr": lr, "grad_scale": 1.0 / (n * self.dp_world)}

    def train_step(self, *batch):
        self.micro_step(*batch)
        return self.apply_gradients()

    # ------------------------------------------------------------------------------------------
    def master_tree(self) -> dict:
        """fp32 master parameters as a nested dict (checkpointing)."""
        master = self.dist_optimizer.gather_master(self) if self.dist_optimizer is not None else self.flat.master
        out: dict = {}
        for p, (o, n, shape) in self.offsets.items():
            _set(out, p, master[o:o + n].view(shape))
        for p, (o, n, shape) in self.local_offsets.items():
            _set(out, p, self.local_master[o:o + n].view(shape))
        return out

    # ---- checkpoint state ------------------------------------------------------------------------
    def dense_state(self):
        """(master, m, v) of the dense group as nested dicts of full-size fp32 tensors keyed like the parameter
        tree. With a sharded optimizer this gathers the shards: a COLLECTIVE call on every rank; the result does not
        depend on the number of ranks."""
        if self.dist_optimizer is not None:
            master = self.dist_optimizer.gather_master(self)
            m, v = self.dist_optimizer.gather_moments(self)
        else:
            master, m, v = self.flat.master, self.m, self.v
        out = ({}, {}, {})
        for p, (o, n, shape) in self.offsets.items():
            for tree, buf in zip(out, (master, m, v)):
                _set(tree, p, buf[o:o + n].view(shape))
        return out

    def local_state(self):
        """(master, m, v) of this rank's expert-parallel leaves as nested dicts (empty without such leaves)."""
        out = ({}, {}, {})
        for p, (o, n, shape) in self.local_offsets.items():
            for tree, buf in zip(out, (self.local_master, self.local_m, self.local_v)):
                _set(tree, p, buf[o:o + n].view(shape))
        return out

    def load_state(self, dense=None, local=None, step: Optional[int] = None):
        """Inverse of ``dense_state`` / ``local_state``: ``dense`` and ``local`` are (master, m, v) triples of nested
        dicts (moments may be None). Every rank loads the full dense trees; the sharded optimizer re-slices."""
        def get(tree, p):
            for k in p:
                tree = tree[k]
            return tree
        if dense is not None:
            master, m, v = dense
            # with a sharded optimizer the replicated fp32 master was released: load through a temporary
            full = self.flat.master if self.flat.master is not None else torch.zeros(
                self.flat.total, device=self.flat.compute.device, dtype=torch.float32)
            full_m = torch.zeros_like(full) if m is not None else None
            full_v = torch.zeros_like(full) if v is not None else None
            for p, (o, n, shape) in self.offsets.items():
                full[o:o + n].copy_(get(master, p).reshape(-1).to(full))
                if m is not None:
                    full_m[o:o + n].copy_(get(m, p).reshape(-1).to(full_m))
                    full_v[o:o + n].copy_(get(v, p).reshape(-1).to(full_v))
            self.flat.compute.copy_(full)
            if self.dist_optimizer is not None:
                self.dist_optimizer.scatter_state(self, full, full_m, full_v)
            elif m is not None:
                self.m.copy_(full_m)
                self.v.copy_(full_v)
        if local is not None and self.local_total:
            master, m, v = local
            for p, (o, n, shape) in self.local_offsets.items():
                self.local_master[o:o + n].copy_(get(master, p).reshape(-1).to(self.local_master))
                if m is not None:
                    self.local_m[o:o + n].copy_(get(m, p).reshape(-1).to(self.local_m))
                    self.local_v[o:o + n].copy_(get(v, p).reshape(-1).to(self.local_v))
            if not self.local_lowmem:
                self.local_compute.copy_(self.local_master)
        if step is not None:
            self.step_count = int(step)

    def n_params(self) -> int:
        return sum(n for _, n, _ in self.offsets.values()) + sum(n for _, n, _ in self.local_offsets.values())
