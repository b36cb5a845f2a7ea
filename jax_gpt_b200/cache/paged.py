"""Paged KV cache: fixed-size pages, a per-sequence block table and per-sequence lengths.

The reference keeps dense ``(B, Hkv, max_len, dh)`` caches with ONE scalar position for the
whole batch (jax_gpt/models/qwen35/cache.py:36-48) and lists paged attention as future work
(project_plan.md:58). Here every sequence owns a list of 64-token pages taken from a shared
pool, so ragged batches and early finishes do not waste memory. For MLA one cached token is
the 576-wide latent (compressed KV + rotary key); for gated-attention layers it is K and V of
the 2 KV heads. The allocator is host-side bookkeeping (free list); the pool, block table and
lengths are device tensors read directly by the decode kernels.
"""
from __future__ import annotations

from typing import List, Optional

import torch


class PageAllocator:
    """Free-list page allocator with per-sequence ownership."""

    def __init__(self, n_pages: int):
        self.n_pages = n_pages
        self.free: List[int] = list(range(n_pages - 1, -1, -1))
        self.owned = {}

    def alloc(self, seq_id: int, n: int) -> List[int]:
        if n > len(self.free):
            raise MemoryError(f"paged cache exhausted: want {n} pages, {len(self.free)} free")
        pages = [self.free.pop() for _ in range(n)]
        self.owned.setdefault(seq_id, []).extend(pages)
        return pages

    def release(self, seq_id: int) -> None:
        self.free.extend(reversed(self.owned.pop(seq_id, [])))

    @property
    def n_free(self) -> int:
        return len(self.free)


class PagedCache:
    """``pool``: (n_layers, n_pages, page_size, width). ``block_table``: (max_seqs, max_pages_per_seq)
    int32 page ids (-1 = unassigned). ``seq_lens``: (max_seqs,) int32 tokens stored per sequence."""

    def __init__(self, n_layers: int, width: int, n_pages: int, page_size: int = 64, max_seqs: int = 64,
                 max_pages_per_seq: int = 64, dtype=torch.bfloat16, device="cpu"):
        self.page_size, self.width, self.n_layers = page_size, width, n_layers
        self.pool = torch.zeros(n_layers, n_pages, page_size, width, dtype=dtype, device=device)
        self.block_table = torch.full((max_seqs, max_pages_per_seq), -1, dtype=torch.int32, device=device)
        self.seq_lens = torch.zeros(max_seqs, dtype=torch.int32, device=device)
        self._lens_host = [0] * max_seqs
        self.alloc = PageAllocator(n_pages)

    def reserve(self, seq_id: int, new_len: int) -> None:
        """Makes sure sequence ``seq_id`` owns enough pages for ``new_len`` tokens."""
        have = len(self.alloc.owned.get(seq_id, []))
        need = (new_len + self.page_size - 1) // self.page_size
        if need > self.block_table.shape[1]:
            raise ValueError("sequence exceeds max_pages_per_seq")
        if need > have:
            pages = self.alloc.alloc(seq_id, need - have)
            self.block_table[seq_id, have:need] = torch.tensor(pages, dtype=torch.int32, device=self.block_table.device)

    def slots(self, seq_id: int, start: int, n: int):
        """(page ids, in-page offsets) of tokens [start, start+n) of a sequence, as device tensors."""
        pos = torch.arange(start, start + n, device=self.block_table.device)
        pages = self.block_table[seq_id, (pos // self.page_size).long()].long()
        return pages, (pos % self.page_size).long()

    def append(self, layer: int, seq_ids, rows: torch.Tensor, commit: bool = False) -> None:
        """rows (B, T, width): writes T new tokens of every listed sequence at its current length.
        ``commit`` advances the lengths (do it once per model step, after the last layer)."""
        B, T, _ = rows.shape
        for b, sid in enumerate(seq_ids):
            start = self._lens_host[sid]
            self.reserve(sid, start + T)
            pages, offs = self.slots(sid, start, T)
            self.pool[layer, pages, offs] = rows[b].to(self.pool.dtype)
        if commit:
            self.commit(seq_ids, T)

    def commit(self, seq_ids, n_new: int) -> None:
        for sid in seq_ids:
            self._lens_host[sid] += n_new
        self.seq_lens.copy_(torch.tensor(self._lens_host, dtype=torch.int32))

    def gather(self, layer: int, seq_id: int, length: Optional[int] = None) -> torch.Tensor:
        """Dense (length, width) view of one sequence (reference path and tests)."""
        length = self._lens_host[seq_id] if length is None else length
        pages, offs = self.slots(seq_id, 0, length)
        return self.pool[layer, pages, offs]

    def length(self, seq_id: int) -> int:
        return self._lens_host[seq_id]

    def release(self, seq_id: int) -> None:
        self.alloc.release(seq_id)
        self.block_table[seq_id].fill_(-1)
        self._lens_host[seq_id] = 0
        self.seq_lens[seq_id] = 0
