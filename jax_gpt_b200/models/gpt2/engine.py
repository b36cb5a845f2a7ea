"""Fused GPT-2 training engine for one B200.

Everything a training step launches is one of this package's sm_100a kernels, called on
preallocated buffers with fixed shapes so the whole step (forward, backward, gradient-norm,
AdamW) can be captured once in a CUDA graph and replayed:

* parameters live in three flat buffers (fp32 master, bf16 compute copy, fp32 gradient) laid
  out as [decayed kernels | everything else]; the tree exposed to users and checkpoints is a
  set of views with the reference's names and shapes (see models/gpt2/model.py);
* linear layers run on the tcgen05 GEMM with bias / GELU / residual fused in the epilogue,
  dgrad and wgrad use the same kernel through MN-major operand descriptors, wgrad
  accumulates in fp32 with split-K;
* attention is the tcgen05 flash kernel reading q/k/v straight out of the fused qkv buffer;
* cross-entropy overwrites the logits with their gradient; AdamW applies the global-norm
  clip from a device scalar, refreshes the bf16 copy and zeroes the gradient in one pass.

The math is the reference's train step (jax_gpt/trainer/train_step.py:34-76) with its
optimizer chain (jax_gpt/trainer/optimizer.py:48-63).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ... import _ext
from ...ops import attention as attn_ops
from ...ops import gemm as G
from ...ops import misc, norm
from .config import GPTConfig
from .model import PARAM_ORDER_DECAY, PARAM_ORDER_NO_DECAY, init_params, param_shapes


def lr_schedule(step: int, peak: float, min_lr: float, warmup: int, decay_steps: int) -> float:
    """Linear 0 -> peak over ``warmup`` steps, cosine to ``min_lr`` at ``decay_steps``
    (optax.warmup_cosine_decay_schedule as used by jax_gpt/trainer/optimizer.py:48-57)."""
    if warmup > 0 and step < warmup:
        return peak * step / warmup
    if step >= decay_steps:
        return min_lr
    frac = (step - warmup) / max(1, decay_steps - warmup)
    return min_lr + 0.5 * (peak - min_lr) * (1.0 + math.cos(math.pi * frac))


class FlatParams:
    """Flat master / compute / gradient / moment buffers with named views."""

    def __init__(self, cfg: GPTConfig, device, seed: int = 0, init: Optional[Dict[str, torch.Tensor]] = None,
                 alloc_grad=None, alloc_compute=None):
        shapes = param_shapes(cfg)
        self.names = PARAM_ORDER_DECAY + PARAM_ORDER_NO_DECAY
        self.offsets = {}
        off = 0
        for n in self.names:
            numel = math.prod(shapes[n])
            self.offsets[n] = (off, numel, shapes[n])
            off += (numel + 63) // 64 * 64  # keep every view 256-byte aligned
            if n == PARAM_ORDER_DECAY[-1]:
                self.n_decay = off
        self.total = off
        # the flat size is padded so that it splits evenly across up to 8 ranks in 16-byte units
        self.total = (self.total + 511) // 512 * 512
        self.master = torch.zeros(self.total, device=device, dtype=torch.float32)
        # gradient and compute buffers may come from a peer-visible (symmetric) allocator
        self.compute = (alloc_compute(self.total) if alloc_compute is not None
                        else torch.zeros(self.total, device=device, dtype=torch.bfloat16))
        self.grad = (alloc_grad(self.total) if alloc_grad is not None
                     else torch.zeros(self.total, device=device, dtype=torch.float32))
        src = init if init is not None else init_params(cfg, seed, "cpu", torch.float32)
        for n in self.names:
            o, numel, shape = self.offsets[n]
            self.master[o:o + numel].copy_(src[n].reshape(-1).to(torch.float32))
        self.compute.copy_(self.master)

    def view(self, buf: torch.Tensor, name: str) -> torch.Tensor:
        o, numel, shape = self.offsets[name]
        return buf[o:o + numel].view(shape)

    def tree(self, buf: torch.Tensor) -> Dict[str, torch.Tensor]:
        return {n: self.view(buf, n) for n in self.names}


class GPT2TrainEngine:
    """Fixed-shape fused training step for GPT-2 on one GPU (optionally one rank of a
    data-parallel group, see parallel/fsdp.py for the fused reduce-scatter + AdamW path)."""

    def __init__(self, cfg: GPTConfig, batch: int, seq: int, *, device=None, seed: int = 0, lr: float = 6e-4,
                 min_lr: float = 6e-5, warmup_steps: int = 2000, lr_decay_steps: int = 600000,
                 weight_decay: float = 0.1, beta1: float = 0.9, beta2: float = 0.95, grad_clip: float = 1.0,
                 init: Optional[Dict[str, torch.Tensor]] = None, use_cuda_graph: bool = True, dist_optimizer=None,
                 overlap_grad_reduce: bool = False):
        assert cfg.n_head == cfg.n_kv_head and cfg.d_head in (64, 128)
        assert cfg.d_model % 8 == 0 and seq <= cfg.d_context
        if cfg.dropout > 0.0:
            raise NotImplementedError("the fused engine has no dropout masks in its kernels; train with "
                                      "GPT(..., deterministic=False) under autograd (trainer.train_step without "
                                      "an engine) or set dropout=0.0 as the reference's training configs do")
        self.cfg, self.B, self.T = cfg, batch, seq
        self.device = torch.device(device if device is not None else ("cuda", torch.cuda.current_device()))
        _ext.load()
        self.hyper = dict(lr=lr, min_lr=min_lr, warmup=warmup_steps, decay=lr_decay_steps, wd=weight_decay,
                          b1=beta1, b2=beta2, clip=grad_clip)
        self.dist_optimizer = dist_optimizer
        self.dp_world = 1
        self._overlap = False
        self._overlap_now = False
        self._pre_reduced = False
        self._sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        if dist_optimizer is not None:
            self.flat = FlatParams(cfg, self.device, seed, init, getattr(dist_optimizer, "alloc_grad", None),
                                   getattr(dist_optimizer, "alloc_compute", None))
            dist_optimizer.attach(self)
            self.dp_world = dist_optimizer.world
            self._overlap = bool(overlap_grad_reduce) and hasattr(dist_optimizer, "setup_buckets") and self.dp_world > 1
            if self._overlap:
                # one bucket per transformer layer (its slice of every stacked parameter), completed in reverse
                # layer order by backward, then one bucket with everything else (embeddings, final norm)
                L = cfg.n_layers
                layer_b = [[] for _ in range(L)]
                rest = []
                for n in self.flat.names:
                    o, numel, shape = self.flat.offsets[n]
                    if n.startswith("h."):
                        per = numel // L
                        for l in range(L):
                            layer_b[l].append((o + l * per, per))
                    else:
                        rest.append((o, numel))
                dist_optimizer.setup_buckets(layer_b + [rest])
                self._rs_stream = torch.cuda.Stream(device=self.device)
            self.m = self.v = None  # moments live in the optimizer's shards
        else:
            self.flat = FlatParams(cfg, self.device, seed, init)
            self.m = torch.zeros_like(self.flat.master)
            self.v = torch.zeros_like(self.flat.master)
        self.step_count = 0
        self.p = self.flat.tree(self.flat.compute)   # bf16 compute views
        self.g = self.flat.tree(self.flat.grad)      # fp32 gradient views
        self._alloc()
        self.use_cuda_graph = use_cuda_graph
        self._graphs = {}
        self._warm = False
        self._micro = 0
        self._side = torch.cuda.Stream(device=self.device)

    # ------------------------------------------------------------------------------------------
    def _alloc(self):
        cfg, dev = self.cfg, self.device
        M, d, f, L = self.B * self.T, cfg.d_model, cfg.d_ff, cfg.n_layers
        bf = dict(device=dev, dtype=torch.bfloat16)
        f32 = dict(device=dev, dtype=torch.float32)
        self.tokens = torch.zeros(self.B, self.T, device=dev, dtype=torch.int32)
        self.targets = torch.zeros(self.B * self.T, device=dev, dtype=torch.int32)
        self.x = [torch.empty(M, d, **bf) for _ in range(L + 1)]       # residual stream at block inputs
        self.ln1 = [torch.empty(M, d, **bf) for _ in range(L)]
        self.ln1_mean = [torch.empty(M, **f32) for _ in range(L)]
        self.ln1_rstd = [torch.empty(M, **f32) for _ in range(L)]
        self.qkv = [torch.empty(M, 3 * d, **bf) for _ in range(L)]
        self.att = [torch.empty(M, d, **bf) for _ in range(L)]
        self.lse = [torch.empty(self.B, cfg.n_head, self.T, **f32) for _ in range(L)]
        self.xmid = [torch.empty(M, d, **bf) for _ in range(L)]
        self.ln2 = [torch.empty(M, d, **bf) for _ in range(L)]
        self.ln2_mean = [torch.empty(M, **f32) for _ in range(L)]
        self.ln2_rstd = [torch.empty(M, **f32) for _ in range(L)]
        self.fc_pre = [torch.empty(M, f, **bf) for _ in range(L)]
        self.fc_act = [torch.empty(M, f, **bf) for _ in range(L)]
        self.lnf = torch.empty(M, d, **bf)
        self.lnf_mean = torch.empty(M, **f32)
        self.lnf_rstd = torch.empty(M, **f32)
        self.logits = torch.empty(M, cfg.padded_vocab, **bf)
        self.loss_rows = torch.empty(M, **f32)
        self.loss = torch.zeros(1, **f32)
        self.loss_sum = torch.zeros(1, **f32)
        self.last_loss = torch.zeros(1, **f32)
        # backward scratch
        self.dx_a = torch.empty(M, d, **bf)
        self.dx_b = torch.empty(M, d, **bf)
        self.dtmp = torch.empty(M, d, **bf)
        self.dfc = torch.empty(M, f, **bf)
        self.dqkv = torch.empty(M, 3 * d, **bf)
        self.dq_acc = torch.empty(M, d, **f32)
        self.delta = torch.empty(self.B, cfg.n_head, self.T, **f32)
        self.gnorm_sq = torch.zeros(1, **f32)
        self.hp = torch.zeros(4, **f32)
        self._hp_host = torch.zeros(4, dtype=torch.float32).pin_memory()

    # ------------------------------------------------------------------------------------------
    def _heads(self, buf2d: torch.Tensor, which: int) -> torch.Tensor:
        cfg = self.cfg
        d = cfg.d_model
        return buf2d.view(self.B, self.T, 3 * d)[..., which * d:(which + 1) * d].unflatten(-1, (cfg.n_head, cfg.d_head))

    def forward(self, compute_loss: bool = True, write_grad: bool = True):
        cfg, p = self.cfg, self.p
        L, d = cfg.n_layers, cfg.d_model
        M = self.B * self.T
        misc.embed_fwd(self.tokens, p["wte.embedding"], p["wpe.embedding"], 0, out=self.x[0].view(self.B, self.T, d))
        for l in range(L):
            x = self.x[l]
            norm.norm_fwd(norm.LAYERNORM, x, p["h.ln_1.layer_norm.scale"][l], p["h.ln_1.layer_norm.bias"][l], 1e-5,
                          y=self.ln1[l], mean=self.ln1_mean[l], rstd=self.ln1_rstd[l])
            G.gemm(self.ln1[l], p["h.attn.c_attn.kernel"][l], b_mn_major=True, bias=p["h.attn.c_attn.bias"][l],
                   out=self.qkv[l])
            attn_ops.attn_fwd(self._heads(self.qkv[l], 0), self._heads(self.qkv[l], 1), self._heads(self.qkv[l], 2),
                              causal=True, out=self.att[l].view(self.B, self.T, cfg.n_head, cfg.d_head),
                              lse=self.lse[l])
            G.gemm(self.att[l], p["h.attn.c_proj.kernel"][l], b_mn_major=True, bias=p["h.attn.c_proj.bias"][l],
                   residual=x, out=self.xmid[l])
            norm.norm_fwd(norm.LAYERNORM, self.xmid[l], p["h.ln_2.layer_norm.scale"][l],
                          p["h.ln_2.layer_norm.bias"][l], 1e-5, y=self.ln2[l], mean=self.ln2_mean[l],
                          rstd=self.ln2_rstd[l])
            G.gemm(self.ln2[l], p["h.mlp.c_fc.kernel"][l], b_mn_major=True, bias=p["h.mlp.c_fc.bias"][l],
                   aux=self.fc_pre[l], epilogue=G.EPI_GELU, out=self.fc_act[l])
            G.gemm(self.fc_act[l], p["h.mlp.c_proj.kernel"][l], b_mn_major=True, bias=p["h.mlp.c_proj.bias"][l],
                   residual=self.xmid[l], out=self.x[l + 1])
        norm.norm_fwd(norm.LAYERNORM, self.x[L], p["ln_f.layer_norm.scale"], p["ln_f.layer_norm.bias"], 1e-5,
                      y=self.lnf, mean=self.lnf_mean, rstd=self.lnf_rstd)
        # tied head: logits = lnf @ wte^T ; the buffer is padded to a multiple of 64 columns
        G.gemm(self.lnf, p["wte.embedding"], out=self.logits[:, :cfg.vocab_size])
        if compute_loss:
            misc.cross_entropy_fwd_bwd(self.logits, self.targets, cfg.vocab_size, 1.0 / M, write_grad=write_grad,
                                       loss=self.loss_rows)
            torch.sum(self.loss_rows, dim=0, keepdim=True, out=self.loss)
            self.loss.mul_(1.0 / M)

    def backward(self):
        cfg, p, g = self.cfg, self.p, self.g
        L, d = cfg.n_layers, cfg.d_model
        M = self.B * self.T
        sms = self._sm_count

        def split_for(out_rows: int, out_cols: int) -> int:
            """Split-K factor of a weight-gradient GEMM (K = tokens): the number of (tile, split) work items should
            fill whole waves of the persistent kernel's CTAs (128 x 256 tiles on every SM) or CTA pairs (256 x 256
            tiles on every two SMs, whichever the launcher picks for that count); every split keeps at least
            1024 tokens."""
            tiles1 = ((out_rows + 127) // 128) * ((out_cols + 255) // 256)
            tiles2 = ((out_rows + 255) // 256) * ((out_cols + 255) // 256)
            uses_pair = _ext.ops().gemm_uses_pair
            best, best_eff = 1, 0.0
            lo = max(1, min(4, M // 4096))
            for sp in range(lo, max(lo, min(16, M // 1024)) + 1):
                if uses_pair(out_rows, out_cols, sp):
                    items, units = tiles2 * sp, sms // 2
                else:
                    items, units = tiles1 * sp, sms
                eff = items / (-(-items // units) * units)
                if eff > best_eff + 0.02:
                    best, best_eff = sp, eff
            return best

        f = cfg.d_ff
        sp_lm, sp_proj2, sp_fc = split_for(cfg.vocab_size, d), split_for(f, d), split_for(d, f)
        sp_proj, sp_attn = split_for(d, d), split_for(d, 3 * d)
        dlog = self.logits[:, :cfg.vocab_size]
        # lm head (tied): dlnf = dlogits @ wte ; dwte += dlogits^T @ lnf
        G.gemm(dlog, p["wte.embedding"], b_mn_major=True, out=self.dtmp)
        G.gemm(dlog, self.lnf, a_mn_major=True, b_mn_major=True, out=g["wte.embedding"], out_mode=G.OUT_F32_ATOMIC,
               split_k=sp_lm)
        dx, dx_other = self.dx_a, self.dx_b
        norm.norm_bwd(norm.LAYERNORM, self.dtmp, self.x[L], p["ln_f.layer_norm.scale"], self.lnf_mean, self.lnf_rstd,
                      g["ln_f.layer_norm.scale"], g["ln_f.layer_norm.bias"], dx=dx)
        for l in reversed(range(L)):
            # MLP: x[l+1] = fc_act @ W2 + b2 + xmid
            G.gemm(self.fc_act[l], dx, a_mn_major=True, b_mn_major=True, out=g["h.mlp.c_proj.kernel"][l],
                   out_mode=G.OUT_F32_ATOMIC, split_k=sp_proj2)
            misc.bias_grad(dx, g["h.mlp.c_proj.bias"][l])
            G.gemm(dx, p["h.mlp.c_proj.kernel"][l], aux=self.fc_pre[l], epilogue=G.EPI_GELU_GRAD, out=self.dfc)
            G.gemm(self.ln2[l], self.dfc, a_mn_major=True, b_mn_major=True, out=g["h.mlp.c_fc.kernel"][l],
                   out_mode=G.OUT_F32_ATOMIC, split_k=sp_fc)
            misc.bias_grad(self.dfc, g["h.mlp.c_fc.bias"][l])
            G.gemm(self.dfc, p["h.mlp.c_fc.kernel"][l], out=self.dtmp)
            norm.norm_bwd(norm.LAYERNORM, self.dtmp, self.xmid[l], p["h.ln_2.layer_norm.scale"][l], self.ln2_mean[l],
                          self.ln2_rstd[l], g["h.ln_2.layer_norm.scale"][l], g["h.ln_2.layer_norm.bias"][l], dres=dx,
                          dx=dx_other)
            dx, dx_other = dx_other, dx  # dx = gradient w.r.t. xmid
            # attention: xmid = att @ Wo + bo + x[l]
            G.gemm(self.att[l], dx, a_mn_major=True, b_mn_major=True, out=g["h.attn.c_proj.kernel"][l],
                   out_mode=G.OUT_F32_ATOMIC, split_k=sp_proj)
            misc.bias_grad(dx, g["h.attn.c_proj.bias"][l])
            G.gemm(dx, p["h.attn.c_proj.kernel"][l], out=self.dtmp)
            self.dq_acc.zero_()
            attn_ops.attn_bwd(self._heads(self.qkv[l], 0), self._heads(self.qkv[l], 1), self._heads(self.qkv[l], 2),
                              self.att[l].view(self.B, self.T, cfg.n_head, cfg.d_head),
                              self.dtmp.view(self.B, self.T, cfg.n_head, cfg.d_head), self.lse[l], causal=True,
                              dq=self._heads(self.dqkv, 0), dk=self._heads(self.dqkv, 1), dv=self._heads(self.dqkv, 2),
                              dq_accum=self.dq_acc, delta=self.delta)
            G.gemm(self.ln1[l], self.dqkv, a_mn_major=True, b_mn_major=True, out=g["h.attn.c_attn.kernel"][l],
                   out_mode=G.OUT_F32_ATOMIC, split_k=sp_attn)
            misc.bias_grad(self.dqkv, g["h.attn.c_attn.bias"][l])
            G.gemm(self.dqkv, p["h.attn.c_attn.kernel"][l], out=self.dtmp)
            norm.norm_bwd(norm.LAYERNORM, self.dtmp, self.x[l], p["h.ln_1.layer_norm.scale"][l], self.ln1_mean[l],
                          self.ln1_rstd[l], g["h.ln_1.layer_norm.scale"][l], g["h.ln_1.layer_norm.bias"][l], dres=dx,
                          dx=dx_other)
            dx, dx_other = dx_other, dx
            if self._overlap_now:
                self._reduce_bucket_async(l)
        misc.embed_bwd(self.tokens, dx.view(self.B, self.T, d), g["wte.embedding"], g["wpe.embedding"], 0)
        if self._overlap_now:
            self.dist_optimizer.reduce_bucket(L, blocks=1184)   # embeddings / final norm: nothing left to overlap with
            torch.cuda.current_stream().wait_stream(self._rs_stream)

    def _reduce_bucket_async(self, b: int):
        """Reduce-scatter of layer ``b``'s gradients on the side stream, behind the kernels that produced them."""
        ev = torch.cuda.Event()
        ev.record()
        with torch.cuda.stream(self._rs_stream):
            self._rs_stream.wait_event(ev)
            self.dist_optimizer.reduce_bucket(b)

    def optimizer_step(self):
        """clip -> Adam -> decoupled decay (kernels only) -> lr; also refreshes bf16 weights, zeroes grads."""
        h = self.hyper
        fl = self.flat
        if self.dist_optimizer is not None:
            if self._pre_reduced:
                self.dist_optimizer.step(self, pre_reduced=True)
            else:
                self.dist_optimizer.step(self)
            return
        self.gnorm_sq.zero_()
        misc.sumsq(fl.grad, self.gnorm_sq)
        nd = fl.n_decay
        misc.adamw(fl.master[:nd], fl.grad[:nd], self.m[:nd], self.v[:nd], self.hp, self.gnorm_sq, beta1=h["b1"],
                   beta2=h["b2"], eps=1e-8, wd=h["wd"], clip=h["clip"], p_bf16=fl.compute[:nd])
        misc.adamw(fl.master[nd:], fl.grad[nd:], self.m[nd:], self.v[nd:], self.hp, self.gnorm_sq, beta1=h["b1"],
                   beta2=h["b2"], eps=1e-8, wd=0.0, clip=h["clip"], p_bf16=fl.compute[nd:])

    # ------------------------------------------------------------------------------------------
    def _set_hyper(self, n_micro: int = 1):
        h = self.hyper
        t = self.step_count + 1
        lr = lr_schedule(self.step_count, h["lr"], h["min_lr"], h["warmup"], h["decay"])
        self._hp_host[0] = lr
        self._hp_host[1] = 1.0 - h["b1"] ** t
        self._hp_host[2] = 1.0 - h["b2"] ** t
        self._hp_host[3] = 1.0 / (n_micro * self.dp_world)
        self.hp.copy_(self._hp_host, non_blocking=True)
        return lr

    def _fwd_bwd(self):
        self.forward(True, True)
        self.backward()
        self.loss_sum.add_(self.loss)

    def _fwd_bwd_reduce(self):
        """Forward + backward of the step's ONLY micro-batch with the gradient reduce-scatter of every layer
        launched on a side stream as soon as that layer's backward is enqueued."""
        self.dist_optimizer.epoch_t.add_(1)
        self._overlap_now = True
        try:
            self._fwd_bwd()
        finally:
            self._overlap_now = False

    def _run(self, name: str, fn):
        """Runs ``fn`` eagerly, or through a CUDA graph captured on first use."""
        if not self.use_cuda_graph:
            fn()
            return
        graph = self._graphs.get(name)
        if graph is None:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                fn()
            self._graphs[name] = graph
        graph.replay()

    def _warm_up(self):
        """One throw-away eager step on a side stream before any capture: sets kernel attributes,
        fills the allocator, and leaves parameters, moments and gradients exactly as they were."""
        if self._warm:
            return
        self._side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._side):
            self._fwd_bwd()
            if self.dist_optimizer is None:
                # single GPU: also exercise the optimizer kernels, then restore the state
                saved = (self.flat.master.clone(), self.m.clone(), self.v.clone())
                self.optimizer_step()
                self.flat.master.copy_(saved[0]); self.m.copy_(saved[1]); self.v.copy_(saved[2])
                self.flat.compute.copy_(self.flat.master)
            if self._overlap:
                # first launch of the bucket kernel outside any capture (epoch 0: no flag to wait for)
                for b in range(self.cfg.n_layers + 1):
                    self.dist_optimizer.reduce_bucket(b)
            self.flat.grad.zero_()
            self.loss_sum.zero_()
        torch.cuda.current_stream().wait_stream(self._side)
        torch.cuda.synchronize(self.device)
        _ext.check_status(self.device)
        self._warm = True

    def micro_step(self, tokens: Optional[torch.Tensor] = None, targets: Optional[torch.Tensor] = None):
        """Forward + backward of one micro-batch; gradients accumulate in the flat fp32 buffer."""
        if tokens is not None:
            self.tokens.copy_(tokens, non_blocking=True)
            self.targets.copy_(targets.reshape(-1), non_blocking=True)
        self._warm_up()
        self._run("fwd_bwd", self._fwd_bwd)
        self._micro += 1

    def apply_gradients(self):
        """Optimizer step over the accumulated gradients (mean over the micro-batches seen)."""
        lr = self._set_hyper(max(1, self._micro))
        self._run("opt_pre" if self._pre_reduced else "opt", self.optimizer_step)
        self._pre_reduced = False
        self.step_count += 1
        n = max(1, self._micro)
        self._micro = 0
        self.last_loss.copy_(self.loss_sum)
        self.last_loss.mul_(1.0 / n)
        self.loss_sum.zero_()
        gsq = self.gnorm_sq if self.dist_optimizer is None else self.dist_optimizer.grad_norm_sq()
        return {"loss": self.last_loss, "grad_norm_sq": gsq, "lr": lr, "grad_scale": 1.0 / (n * self.dp_world)}

    def train_step(self, tokens: Optional[torch.Tensor] = None, targets: Optional[torch.Tensor] = None):
        """One optimizer step on one micro-batch. ``tokens``/``targets`` [B,T] int32 (device or
        pinned host); when omitted the static input buffers are re-used. Returns device scalars
        ``loss`` and ``grad_norm_sq`` (no host sync) plus the learning rate used."""
        if self._overlap and self._micro == 0:
            # a step of one micro-batch: its gradients are final layer by layer, so their reduce-scatter
            # overlaps the rest of backward
            if tokens is not None:
                self.tokens.copy_(tokens, non_blocking=True)
                self.targets.copy_(targets.reshape(-1), non_blocking=True)
            self._warm_up()
            self._run("fwd_bwd_reduce", self._fwd_bwd_reduce)
            self._micro += 1
            self._pre_reduced = True
            return self.apply_gradients()
        self.micro_step(tokens, targets)
        return self.apply_gradients()

    @torch.no_grad()
    def eval_loss(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        self.tokens.copy_(tokens, non_blocking=True)
        self.targets.copy_(targets.reshape(-1), non_blocking=True)
        self.forward(True, False)
        return self.loss.clone()

    # -- parameter access (reference tree) -------------------------------------------------------
    def params(self) -> Dict[str, torch.Tensor]:
        """fp32 master parameters as the reference tree. With a sharded optimizer this is a collective call
        (the shards are gathered first): every rank must make it."""
        if self.dist_optimizer is not None:
            return self.flat.tree(self.dist_optimizer.gather_master(self))
        return self.flat.tree(self.flat.master)

    def opt_state(self) -> Dict[str, Dict[str, torch.Tensor]]:
        """Adam moments as trees shaped like the parameters. Collective with a sharded optimizer; the result
        does not depend on the number of ranks."""
        if self.m is None:
            m, v = self.dist_optimizer.gather_moments(self)
            return {"count": self.step_count, "mu": self.flat.tree(m), "nu": self.flat.tree(v)}
        return {"count": self.step_count, "mu": self.flat.tree(self.m), "nu": self.flat.tree(self.v)}

    def load(self, params: Dict[str, torch.Tensor], opt_state=None, step: Optional[int] = None):
        with torch.no_grad():
            # with a sharded optimizer the replicated fp32 master was released: a temporary full vector takes
            # the checkpoint's values, the bf16 copy and this rank's shard are cut from it
            master = self.flat.master if self.flat.master is not None else torch.zeros(
                self.flat.total, device=self.flat.compute.device, dtype=torch.float32)
            for n, t in params.items():
                self.flat.view(master, n).copy_(t)
            self.flat.compute.copy_(master)
            if self.dist_optimizer is not None:
                # sharded optimizer: assemble full-length moments, then keep this rank's slices
                m = v = None
                if opt_state is not None:
                    m, v = torch.zeros_like(master), torch.zeros_like(master)
                    for n, t in opt_state["mu"].items():
                        self.flat.view(m, n).copy_(t)
                    for n, t in opt_state["nu"].items():
                        self.flat.view(v, n).copy_(t)
                self.dist_optimizer.scatter_state(self, master, m, v)
            elif opt_state is not None:
                for n, t in opt_state["mu"].items():
                    self.flat.view(self.m, n).copy_(t)
                for n, t in opt_state["nu"].items():
                    self.flat.view(self.v, n).copy_(t)
            if step is not None:
                self.step_count = int(step)

    def kernel_launches_per_step(self) -> int:
        """Number of this package's kernels launched by one train step (for bench reporting)."""
        L = self.cfg.n_layers
        fwd = 1 + L * 7 + 1 + 1 + 1
        bwd = 2 + 1 + L * (3 + 3 + 3 + 2 + 2 + 3 + 2) + 1  # gemms, bias grads, norms, attention (delta+bwd+cast)
        opt = 3
        return fwd + bwd + opt
