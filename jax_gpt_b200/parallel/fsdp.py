"""Sharded optimizer (ZeRO / FSDP style) fused with its collectives.

``FusedShardedAdamW`` replaces "reduce-scatter gradients (NCCL) -> AdamW on the shard ->
all-gather parameters (NCCL)" by ONE kernel per rank that reads every peer's gradient slice
over NVLink, clips, updates its fp32 master shard and pushes the new bf16 values into every
peer's compute buffer (csrc/comm_kernels.cu). ``NcclShardedAdamW`` is the library baseline
with the same math. ``sharded_adamw_reference`` restates the protocol with ordinary
collectives so the host-side sharding logic is testable on CPU (gloo) ranks.

The reference only declares an ``fsdp`` mesh axis (jax_gpt/trainer/sharding.py:58-69); its
optimizer chain is jax_gpt/trainer/optimizer.py:48-63.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import _ext
from ..comm.symm import Communicator, shard_range
from ..ops import misc


def sharded_adamw_reference(group, grad: torch.Tensor, master_shard: torch.Tensor, m: torch.Tensor, v: torch.Tensor,
                            compute: torch.Tensor, hp, n_decay: int, beta1, beta2, eps, wd, clip):
    """Same result as the fused kernel using reduce_scatter / all_reduce / all_gather.
    ``grad`` is the full local fp32 gradient, ``compute`` the full compute-dtype parameter copy."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    n = grad.numel()
    lo, hi = shard_range(n, world, rank)
    red = torch.empty(hi - lo, dtype=grad.dtype, device=grad.device)
    if grad.is_cuda:
        dist.reduce_scatter_tensor(red, grad, group=group)
    else:  # gloo has no reduce_scatter: all-reduce a copy and slice
        full = grad.clone()
        dist.all_reduce(full, group=group)
        red.copy_(full[lo:hi])
    sq = (red.double() ** 2).sum().float().reshape(1)
    dist.all_reduce(sq, group=group)
    lr, bc1, bc2, gscale = [float(x) for x in hp]
    coef = gscale
    if clip > 0:
        coef *= min(1.0, clip / (float(sq) ** 0.5 * gscale + 1e-6))
    gi = red * coef
    m.mul_(beta1).add_(gi, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gi, gi, value=1 - beta2)
    idx = torch.arange(lo, hi, device=grad.device)
    wdv = torch.where(idx < n_decay, torch.tensor(wd, device=grad.device), torch.tensor(0.0, device=grad.device))
    u = (m / bc1) / ((v / bc2).sqrt() + eps) + wdv * master_shard
    master_shard.sub_(lr * u)
    pieces = [torch.empty(hi - lo, dtype=compute.dtype, device=compute.device) for _ in range(world)]
    dist.all_gather(pieces, master_shard.to(compute.dtype), group=group)
    compute.copy_(torch.cat(pieces))
    return sq


class _ShardedBase:
    """Owns this rank's fp32 master / moment shards of an engine's flat parameter vector."""

    def __init__(self, group=None, device=None):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = device
        self.master = self.m = self.v = None

    def _make_shards(self, engine):
        n = engine.flat.total
        assert n % (self.world * 8) == 0
        lo, hi = shard_range(n, self.world, self.rank)
        self.lo, self.hi = lo, hi
        self.master = engine.flat.master[lo:hi].clone()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        # from here on the fp32 master weights exist only as shards (ZeRO-style: 4 bytes per parameter and rank
        # instead of 4 per parameter): the engine's replicated copy is released
        engine.flat.master = None

    def gather_master(self, engine) -> torch.Tensor:
        """The full fp32 master vector assembled from the shards (checkpointing path): a temporary. Collective."""
        full = torch.empty(engine.flat.total, device=self.master.device, dtype=torch.float32)
        dist.all_gather_into_tensor(full, self.master, group=self.group)
        return full

    def gather_moments(self, engine):
        """Full-length Adam moments (m, v) assembled from every rank's shard. Collective; the result is
        independent of the number of ranks, so a checkpoint can be resumed at another sharding degree."""
        m = torch.empty(engine.flat.total, device=self.master.device, dtype=torch.float32)
        v = torch.empty_like(m)
        dist.all_gather_into_tensor(m, self.m, group=self.group)
        dist.all_gather_into_tensor(v, self.v, group=self.group)
        return m, v

    def scatter_state(self, engine, master_full, m_full=None, v_full=None):
        """Re-slices this rank's shards from full-length buffers (after a checkpoint was loaded into the engine)."""
        self.master.copy_(master_full[self.lo:self.hi])
        if m_full is not None:
            self.m.copy_(m_full[self.lo:self.hi])
        if v_full is not None:
            self.v.copy_(v_full[self.lo:self.hi])


class FusedShardedAdamW(_ShardedBase):
    """One-kernel reduce-scatter + AdamW + all-gather over NVLink peer memory."""

    def __init__(self, group=None, device=None, use_multimem: bool = False, wait_seconds: float = 20.0):
        super().__init__(group, device)
        self.comm = Communicator(self.group, device, wait_seconds)
        self.use_multimem = use_multimem
        self.grad_buf = self.param_buf = None

    # allocation hook used by the engine so that gradients and bf16 weights are peer-visible
    def alloc_grad(self, numel: int):
        self.grad_buf = self.comm.alloc(numel, torch.float32)
        return self.grad_buf.tensor

    def alloc_compute(self, numel: int):
        self.param_buf = self.comm.alloc(numel, torch.bfloat16)
        return self.param_buf.tensor

    def attach(self, engine):
        self._make_shards(engine)
        self.n_total, self.n_decay = engine.flat.total, engine.flat.n_decay

    # ---- gradient reduce-scatter overlapped with backward ------------------------------------------
    def setup_buckets(self, buckets, blocks: int = 74):
        """``buckets``: list (in the order backward completes them) of lists of (offset, length) element ranges
        of the flat gradient vector. Each bucket's part inside this rank's shard is reduced by one small
        kernel on a side stream as soon as backward has produced it (``reduce_bucket``)."""
        dev = self.comm.device
        self._bucket_ranges = []
        for ranges in buckets:
            mine = []
            for off, n in ranges:
                a, b = max(off, self.lo), min(off + n, self.hi)
                if b > a:
                    assert a % 4 == 0 and (b - a) % 4 == 0
                    mine.append((a, b - a))
            self._bucket_ranges.append(torch.tensor(mine, dtype=torch.int64, device=dev).reshape(-1, 2))
        self._bucket_flags = self.comm.alloc(len(buckets) * 8, torch.int32)
        self.epoch_t = torch.zeros(1, device=dev, dtype=torch.int32)
        self._bucket_blocks = blocks
        dist.barrier(self.group)

    def reduce_bucket(self, b: int, blocks: Optional[int] = None):
        """Launch on the CURRENT stream (the caller puts it on a side stream behind the producing kernels).
        ``blocks``: CTAs of 256 threads; few for a kernel that shares the GPU with backward, many for one that runs alone."""
        _ext.ops().rs_bucket(self.world, self.rank, self.grad_buf.peer_ptrs, self._bucket_flags.peer_ptrs,
                             self._bucket_ranges[b], b, self.epoch_t, blocks or self._bucket_blocks, self.comm.wait_seconds)

    def step(self, engine, extra_sq=None, pre_reduced: bool = False):
        """``extra_sq``: device scalar with this rank's sum of squared gradients of parameters kept
        outside the flat vector (expert-parallel weights); it joins the global clipping norm.
        ``pre_reduced``: every bucket was already reduce-scattered during backward."""
        h = engine.hyper
        mc_g = self.grad_buf.multicast_ptr if self.use_multimem else 0
        mc_p = self.param_buf.multicast_ptr if self.use_multimem else 0
        _ext.ops().sharded_adamw(self.world, self.rank, self.n_total, self.n_decay, self.grad_buf.peer_ptrs,
                                 self.param_buf.peer_ptrs, self.comm.ctrl.peer_ptrs, mc_g, mc_p, self.master, self.m,
                                 self.v, engine.hp, h["b1"], h["b2"], 1e-8, h["wd"], h["clip"], self.comm.wait_seconds,
                                 extra_sq, pre_reduced)
        engine.flat.grad.zero_()

    def grad_norm_sq(self) -> torch.Tensor:
        """Device scalar: global sum of squared gradients of the last step (before scaling)."""
        # CommCtrl layout: flags 8*8 int32, norm_slots 8 fp32, epoch, bar_epoch, sq_local, sq_total
        return self.comm.ctrl.tensor.view(torch.float32)[8 * 8 + 8 + 3:8 * 8 + 8 + 4]


class NcclShardedAdamW(_ShardedBase):
    """Baseline: NCCL reduce-scatter, the fused single-GPU AdamW kernel on the shard, NCCL all-gather."""

    def attach(self, engine):
        self._make_shards(engine)
        self.n_total, self.n_decay = engine.flat.total, engine.flat.n_decay
        self.red = torch.empty_like(self.master)
        self.sq = torch.zeros(1, device=self.master.device)
        self.shard_bf16 = torch.empty(self.master.numel(), device=self.master.device, dtype=torch.bfloat16)

    def step(self, engine, extra_sq=None):
        h = engine.hyper
        dist.reduce_scatter_tensor(self.red, engine.flat.grad, group=self.group)
        self.sq.zero_()
        misc.sumsq(self.red, self.sq)
        if extra_sq is not None:
            self.sq += extra_sq
        dist.all_reduce(self.sq, group=self.group)
        nd = min(max(self.n_decay - self.lo, 0), self.hi - self.lo)
        for a, b, wd in ((0, nd, h["wd"]), (nd, self.hi - self.lo, 0.0)):
            if b > a:
                misc.adamw(self.master[a:b], self.red[a:b], self.m[a:b], self.v[a:b], engine.hp, self.sq,
                           beta1=h["b1"], beta2=h["b2"], eps=1e-8, wd=wd, clip=h["clip"],
                           p_bf16=self.shard_bf16[a:b], zero_grad=False)
        dist.all_gather_into_tensor(engine.flat.compute, self.shard_bf16, group=self.group)
        engine.flat.grad.zero_()

    def grad_norm_sq(self):
        return self.sq


class ShardedWeight:
    """A weight W (K, N) kept sharded across the ranks (FSDP: rank r owns the columns ``[r N / W, (r + 1) N / W)``
    as a contiguous (K, N / W) matrix), gathered INSIDE the GEMM that consumes it: ``matmul(x)`` is one kernel whose
    copier CTAs push this rank's shard into every peer's gather buffer (every byte over NVLink once, published 64
    rows at a time) while its compute CTAs run the tcgen05 GEMM on their own gather buffer, the output columns of
    the local shard first, then each peer's once its shard has landed. The gather buffers (two, alternating, so
    that a peer one call ahead never overwrites a shard still being read) are shared by all weights of one shape:
    resident memory stays one shard per weight plus two full-size buffers per distinct shape."""

    _scratch = {}

    def __init__(self, comm: Communicator, w_full_or_shard: torch.Tensor, is_shard: bool = False):
        self.comm = comm
        W = comm.world
        if is_shard:
            shard = w_full_or_shard
            self.K, self.N = shard.shape[0], shard.shape[1] * W
        else:
            self.K, self.N = w_full_or_shard.shape
            npr = self.N // W
            shard = w_full_or_shard[:, comm.rank * npr:(comm.rank + 1) * npr]
        assert self.N % (W * 128) == 0 and self.K % 64 == 0, "columns per rank: a multiple of 128; K: a multiple of 64"
        self.shard = shard.to(device=comm.device, dtype=torch.bfloat16).contiguous().clone()
        key = (id(comm), self.K, self.N)
        if key not in ShardedWeight._scratch:
            bufs = [comm.alloc(self.K * self.N, torch.bfloat16, zero=False) for _ in range(2)]
            ready = [comm.alloc(W * self.K // 64, torch.int32) for _ in range(2)]
            torch.cuda.synchronize(comm.device)
            dist.barrier(comm.group)          # zeroed ready arrays are in place everywhere
            ShardedWeight._scratch[key] = [bufs, ready, 0]
        self._key = key

    def matmul(self, x: torch.Tensor, bias=None) -> torch.Tensor:
        st = ShardedWeight._scratch[self._key]
        st[2] += 1
        epoch = st[2]
        buf, rdy = st[0][epoch & 1], st[1][epoch & 1]
        W, r = self.comm.world, self.comm.rank
        buf.tensor.view(W, self.K, self.N // W)[r].copy_(self.shard)
        x2 = x.reshape(-1, self.K)
        out = torch.empty(x2.shape[0], self.N, device=x.device, dtype=torch.bfloat16)
        _ext.ops().gemm_sharded_b_staged(x2, buf.peer_ptrs, rdy.peer_ptrs, self.N, r, out, bias, epoch,
                                         self.comm.wait_seconds)
        return out.reshape(*x.shape[:-1], self.N)
