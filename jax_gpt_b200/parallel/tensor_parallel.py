"""Tensor-parallel linear pairs with the collective fused into the GEMM kernel.

Under sequence parallelism the tokens are sharded between the TP regions, so

* a column-parallel projection is ``all-gather(x) @ W_col``  -> :meth:`TPContext.all_gather_matmul`
  runs the tcgen05 GEMM with one TMA tensor map per rank: M-tiles of the local shard are
  computed first while the peers' shards are read straight out of their memory by ordinary
  (non-multicast) TMA tile loads over NVLink;
* a row-parallel projection is ``reduce-scatter(x @ W_row)`` -> :meth:`TPContext.matmul_reduce_scatter`
  whose epilogue adds each output tile into the owning rank's fp32 buffer with vectorised
  ``red.global.add`` over NVLink instead of writing a full partial result and calling NCCL.

Used for the MLA / gated-attention projections (q/k/v in, o out). The reference gets the same
collectives implicitly from GSPMD annotations (jax_gpt/models/qwen35/sharding.py:41-90,
jax_gpt/trainer/sharding.py:24-55).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import _ext
from ..comm.symm import Communicator


class TPContext:
    def __init__(self, group=None, device=None, wait_seconds: float = 20.0):
        self.comm = Communicator(group, device, wait_seconds)
        self.rank, self.world = self.comm.rank, self.comm.world
        self.device = self.comm.device
        self._ag = {}
        self._rs = {}

    # ---- all-gather -> GEMM ------------------------------------------------------------------
    def all_gather_matmul(self, x_local: torch.Tensor, w: torch.Tensor, bias=None) -> torch.Tensor:
        """``concat_ranks(x_local) @ w`` with ``w`` (in, out_local); x_local [rows, K] bf16, rows % 128 == 0."""
        rows, K = x_local.shape
        assert rows % 128 == 0 and x_local.dtype == torch.bfloat16
        key = (rows, K)
        if key not in self._ag:
            self._ag[key] = self.comm.alloc(rows * K, torch.bfloat16)
        buf = self._ag[key]
        buf.tensor.view(rows, K).copy_(x_local)
        self.comm.barrier()  # every rank's shard is in place
        out = torch.empty(rows * self.world, w.shape[1], device=self.device, dtype=torch.bfloat16)
        _ext.ops().gemm_gathered_a(buf.peer_ptrs, rows, self.rank, K, K, w, True, out, bias)
        self.comm.barrier()  # nobody still reads this rank's staging buffer
        return out

    # ---- GEMM -> reduce-scatter ----------------------------------------------------------------
    def matmul_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """Rows ``[rank*R, (rank+1)*R)`` of ``sum_ranks(x @ w)``; x [R*world, K_local] bf16, w (K_local, N)."""
        M, K = x.shape
        N = w.shape[1]
        assert M % self.world == 0
        R = M // self.world
        key = (R, N)
        if key not in self._rs:
            self._rs[key] = self.comm.alloc(R * N, torch.float32)
        buf = self._rs[key]
        buf.tensor.zero_()
        self.comm.barrier()  # every destination is zeroed
        _ext.ops().gemm_reduce_scatter(x, w, True, buf.peer_ptrs, R, N)
        self.comm.barrier()  # every rank's contributions have landed
        return buf.tensor.view(R, N).to(torch.bfloat16)


def all_gather_matmul_nccl(x_local, w, group=None):
    """Library baseline: NCCL all-gather, then the local GEMM."""
    world = dist.get_world_size(group)
    full = torch.empty(x_local.shape[0] * world, x_local.shape[1], device=x_local.device, dtype=x_local.dtype)
    dist.all_gather_into_tensor(full, x_local.contiguous(), group=group)
    from ..ops.gemm import gemm
    return gemm(full, w, b_mn_major=True)


def matmul_reduce_scatter_nccl(x, w, group=None):
    """Library baseline: local GEMM to fp32, then NCCL reduce-scatter."""
    from ..ops.gemm import OUT_F32, gemm
    world = dist.get_world_size(group)
    part = gemm(x, w, b_mn_major=True, out_mode=OUT_F32)
    out = torch.empty(x.shape[0] // world, w.shape[1], device=x.device, dtype=torch.float32)
    dist.reduce_scatter_tensor(out, part, group=group)
    return out.to(torch.bfloat16)


# ---- vocabulary-parallel cross-entropy --------------------------------------------------------
def vocab_parallel_ce_reference(logits_local: torch.Tensor, targets: torch.Tensor, v0: int, group=None):
    """Per-row loss and the local-shard gradient ``softmax - onehot`` with library collectives
    (all_reduce of max / sum-exp / target logit). Works on CPU (gloo) ranks: the host-side protocol."""
    lf = logits_local.float()
    m = lf.max(dim=-1).values
    dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
    e = torch.exp(lf - m[:, None])
    s = e.sum(-1)
    dist.all_reduce(s, group=group)
    tg = targets.long() - v0
    mine = (tg >= 0) & (tg < lf.shape[1])
    tl = torch.where(mine, lf.gather(1, tg.clamp(0, lf.shape[1] - 1)[:, None])[:, 0], torch.zeros_like(m))
    dist.all_reduce(tl, group=group)
    valid = targets >= 0
    loss = torch.where(valid, torch.log(s) + m - tl, torch.zeros_like(m))
    grad = e / s[:, None]
    grad[mine, tg[mine]] -= 1.0
    grad = grad * valid[:, None]
    return loss, grad


class _VocabParallelCEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits_local, targets, vp):
        M = logits_local.shape[0]
        loss = torch.empty(M, device=logits_local.device, dtype=torch.float32)
        n_valid = (targets >= 0).sum().clamp_min(1).float()
        c = vp.comm
        _ext.ops().vocab_parallel_ce(c.world, c.rank, logits_local, targets, vp.v_local, vp.v0, vp.stats(M).peer_ptrs,
                                     c.ctrl.peer_ptrs, loss, 1.0, True, c.wait_seconds)
        ctx.save_for_backward(logits_local, n_valid)
        return loss.sum() / n_valid

    @staticmethod
    def backward(ctx, g):
        dlogits, n_valid = ctx.saved_tensors
        return dlogits.mul_((g / n_valid).to(dlogits.dtype)), None, None


class VocabParallelCE:
    """Mean token cross-entropy over logits whose vocabulary axis is sharded across the ranks of ``comm``
    (rank r holds columns ``[r * v_local, (r + 1) * v_local)``): ONE kernel computes the shard statistics,
    exchanges them through peer memory, and turns the shard into its gradient in place - the (M, V)
    logits are never gathered (the reference all-gathers them implicitly through GSPMD when it evaluates
    ``optax.softmax_cross_entropy_with_integer_labels``, jax_gpt/trainer/train_step.py:24-31)."""

    def __init__(self, comm: Communicator, vocab_size: int):
        assert vocab_size % comm.world == 0
        self.comm = comm
        self.v_local = vocab_size // comm.world
        self.v0 = comm.rank * self.v_local
        self._stats = {}

    def stats(self, M: int):
        if M not in self._stats:
            self._stats[M] = self.comm.alloc(2 * self.comm.world * M * 4, torch.float32)
        return self._stats[M]

    def __call__(self, logits_local: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """logits_local (M, >= v_local) bf16, CONSUMED (overwritten with its gradient); targets (M,) global ids."""
        logits_local = logits_local.reshape(-1, logits_local.shape[-1])
        return _VocabParallelCEFn.apply(logits_local, targets.reshape(-1).to(torch.int32).contiguous(), self)
