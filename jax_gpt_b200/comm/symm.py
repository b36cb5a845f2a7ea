"""Symmetric (peer-mapped) device memory and cross-rank flags for in-kernel communication.

One process per GPU; `torch.distributed` (NCCL) provides rendezvous, the CUDA-VMM symmetric
allocator of ``torch.distributed._symmetric_memory`` provides buffers that every rank of the
group can address directly (and, where the fabric supports it, an NVLS multicast alias).
Kernels of this package receive the resulting raw peer addresses and do the loads, stores,
reductions and flag waits themselves; nothing here moves data.

The reference has no explicit communication layer: XLA inserts collectives from sharding
annotations and the only hand-written one is a ``psum`` (jax_gpt/models/qwen35/moe.py:218).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import _ext

CTRL_INT32_WORDS = 1024  # 4 KB control block per rank (flags, norm slots, epochs)


@dataclass
class SymmetricBuffer:
    tensor: torch.Tensor          # this rank's buffer
    peer_ptrs: List[int]          # address of every rank's buffer as seen from this rank
    multicast_ptr: int            # NVLS alias covering all ranks' buffers, 0 if unavailable
    handle: object


class Communicator:
    """Rendezvous of one process group: symmetric allocations, a control block, a barrier."""

    def __init__(self, group=None, device=None, wait_seconds: float = 20.0):
        import torch.distributed._symmetric_memory as symm_mem
        self._symm = symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.device = torch.device(device if device is not None else ("cuda", torch.cuda.current_device()))
        self.wait_seconds = wait_seconds
        self.ctrl = self.alloc(CTRL_INT32_WORDS, torch.int32, zero=True)
        self.ctrl_ptr_table = torch.tensor(self.ctrl.peer_ptrs, device=self.device, dtype=torch.int64)
        dist.barrier(self.group)  # control blocks are zero everywhere before any kernel signals

    def alloc(self, numel: int, dtype, zero: bool = True) -> SymmetricBuffer:
        t = self._symm.empty(numel, dtype=dtype, device=self.device)
        if zero:
            t.zero_()
        hdl = self._symm.rendezvous(t, self.group)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        mc = int(hdl.multicast_ptr) if getattr(hdl, "multicast_ptr", 0) else 0
        return SymmetricBuffer(t, ptrs, mc, hdl)

    def barrier(self):
        """Device-side barrier on the current stream (bounded flag waits, no host sync)."""
        _ext.ops().comm_barrier(self.ctrl_ptr_table, self.world, self.rank, self.wait_seconds)


def shard_range(n_total: int, world: int, rank: int):
    """[start, end) of rank's contiguous shard of a flat vector of ``n_total`` elements."""
    assert n_total % world == 0
    s = n_total // world
    return rank * s, (rank + 1) * s
