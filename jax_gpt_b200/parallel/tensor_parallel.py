"""Tensor-parallel linear pairs with the collective fused into the GEMM kernel.

Under sequence parallelism the tokens are sharded between the TP regions, so

* a column-parallel projection is ``all-gather(x) @ W_col``  -> :meth:`TPContext.all_gather_matmul`:
  ONE kernel whose last CTAs push this rank's row block into every peer's gather buffer (bulk copies local ->
  shared-memory ring -> peer, and plain 16-byte loads and stores, so every byte crosses NVLink once) and publish
  it 128 rows at a time in the peer's ready array, while the other CTAs run the tcgen05 GEMM on their own gather
  buffer, the tiles of the local rows first, waiting block by block for the flags the peers set. No barrier:
  the gather buffers alternate between two copies;
* a row-parallel projection is ``reduce-scatter(x @ W_row)`` -> :meth:`TPContext.matmul_reduce_scatter`
  whose epilogue stores each bf16 output tile into the owning rank's receive slot over NVLink and whose second
  phase sums the slots of the rows this rank owns, instead of writing a full partial result and calling NCCL.

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
        """``concat_ranks(x_local) @ w`` with ``w`` (in, out_local); x_local [rows, K] bf16, rows % 128 == 0.
        The gather buffers and their ready arrays alternate between two copies per shape: a rank can only be one
        call ahead of a peer (its next call needs that peer's rows of the call in between), so nobody overwrites
        rows that are still being read."""
        rows, K = x_local.shape
        assert rows % 128 == 0 and x_local.dtype == torch.bfloat16
        key = (rows, K)
        if key not in self._ag:
            bufs = [self.comm.alloc(self.world * rows * K, torch.bfloat16, zero=False) for _ in range(2)]
            ready = [self.comm.alloc(self.world * rows // 128, torch.int32) for _ in range(2)]
            torch.cuda.synchronize(self.device)
            dist.barrier(self.comm.group)                  # every ready array is zero before anyone publishes
            self._ag[key] = [bufs, ready, 0]
        bufs, ready, epoch = self._ag[key]
        epoch += 1
        self._ag[key][2] = epoch
        buf, rdy = bufs[epoch & 1], ready[epoch & 1]
        buf.tensor.view(self.world * rows, K)[self.rank * rows:(self.rank + 1) * rows].copy_(x_local)
        out = torch.empty(rows * self.world, w.shape[1], device=self.device, dtype=torch.bfloat16)
        _ext.ops().gemm_gathered_a_staged(buf.peer_ptrs, rdy.peer_ptrs, rows, K, self.rank, w, True, out, bias, epoch,
                                          self.comm.wait_seconds)
        return out

    # ---- GEMM -> reduce-scatter ----------------------------------------------------------------
    def matmul_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """Rows ``[rank*R, (rank+1)*R)`` of ``sum_ranks(x @ w)``; x [R*world, K_local] bf16, w (K_local, N).
        One kernel: every 128 x BN tile is stored as bf16 into this rank's slot of the row owner's receive buffer
        (plain 128-byte stores over NVLink, the owners after this rank first, its own rows last), every epilogue
        warp bumps the owner's arrival counter of the row block, and when the tiles are done the CTAs sum the
        ``world`` slots of the blocks this rank owns. No barrier and no zeroing: the receive buffers and counters
        alternate between two copies (a rank cannot be two calls ahead of a peer whose partials it needs)."""
        M, K = x.shape
        N = w.shape[1]
        assert M % self.world == 0 and x.dtype == torch.bfloat16
        R = M // self.world
        assert R % 128 == 0 and N % 64 == 0, "rows per rank must be a multiple of 128 and N of 64"
        key = (R, N)
        if key not in self._rs:
            recv = [self.comm.alloc(self.world * R * N, torch.bfloat16, zero=False) for _ in range(2)]
            cnt = [self.comm.alloc(R // 128, torch.int32) for _ in range(2)]
            torch.cuda.synchronize(self.device)
            dist.barrier(self.comm.group)                  # counters are zero everywhere before the first arrival
            self._rs[key] = [recv, cnt, 0]
        recv, cnt, calls = self._rs[key]
        self._rs[key][2] = calls + 1
        par = calls & 1
        expected = (calls // 2 + 1) * self.world * 4 * (N // 64)     # four lane quarters x 64-column groups per source
        out = torch.empty(R, N, device=self.device, dtype=torch.bfloat16)
        _ext.ops().gemm_reduce_scatter_push(x, w, True, recv[par].peer_ptrs, cnt[par].peer_ptrs, self.rank, R, out, expected,
                                            self.comm.wait_seconds)
        return out

class _ColumnParallelFn(torch.autograd.Function):
    """``concat_ranks(x_local) @ w`` (sequence-parallel input, column-parallel weight) with the fused kernels in
    both directions: the backward's input gradient is the fused GEMM -> reduce-scatter of ``dy @ w^T``; the weight
    gradient needs the gathered input again, which is re-gathered (NCCL) rather than kept alive."""

    @staticmethod
    def forward(ctx, x_local, w, tp):
        ctx.tp = tp
        ctx.save_for_backward(x_local, w)
        return tp.all_gather_matmul(x_local, w)

    @staticmethod
    def backward(ctx, dy):
        from ..ops.gemm import OUT_F32_ATOMIC, gemm
        x_local, w = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        dx = tp.matmul_reduce_scatter(dy, w.t().contiguous()) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            full = torch.empty(x_local.shape[0] * tp.world, x_local.shape[1], device=x_local.device, dtype=x_local.dtype)
            dist.all_gather_into_tensor(full, x_local.contiguous(), group=tp.comm.group)
            dw = gemm(full, dy, a_mn_major=True, b_mn_major=True, out_mode=OUT_F32_ATOMIC).to(w.dtype)
        return dx, dw, None


class _RowParallelFn(torch.autograd.Function):
    """Rows of ``sum_ranks(x @ w_r)`` owned by this rank (row-parallel weight, sequence-parallel output): forward is
    the fused GEMM -> reduce-scatter, the input gradient the fused all-gather -> GEMM of ``dy_local`` with ``w^T``."""

    @staticmethod
    def forward(ctx, x, w, tp):
        ctx.tp = tp
        ctx.save_for_backward(x, w)
        return tp.matmul_reduce_scatter(x, w)

    @staticmethod
    def backward(ctx, dy_local):
        from ..ops.gemm import OUT_F32_ATOMIC, gemm
        x, w = ctx.saved_tensors
        tp = ctx.tp
        dy_local = dy_local.contiguous()
        dx = tp.all_gather_matmul(dy_local, w.t().contiguous()) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            full = torch.empty(dy_local.shape[0] * tp.world, dy_local.shape[1], device=x.device, dtype=dy_local.dtype)
            dist.all_gather_into_tensor(full, dy_local, group=tp.comm.group)
            dw = gemm(x, full, a_mn_major=True, b_mn_major=True, out_mode=OUT_F32_ATOMIC).to(w.dtype)
        return dx, dw, None


def column_parallel_linear(x_local, w, tp: "TPContext"):
    """Differentiable ``all-gather(x_local) @ w``; x_local [rows, K] bf16 (rows % 128 == 0), w (K, N_local)."""
    return _ColumnParallelFn.apply(x_local, w, tp)


def row_parallel_linear(x, w, tp: "TPContext"):
    """Differentiable ``reduce-scatter(x @ w)``; x [rows * world, K_local] bf16, w (K_local, N), N % 64 == 0."""
    return _RowParallelFn.apply(x, w, tp)


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
