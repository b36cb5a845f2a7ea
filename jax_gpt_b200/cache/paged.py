"""Paged KV cache: fixed-size pages, a per-sequence block table and per-sequence lengths.

The reference keeps dense ``(B, Hkv, max_len, dh)`` caches with ONE scalar position for the
whole batch (jax_gpt/models/qwen35/cache.py:36-48) and lists paged attention as future work
(project_plan.md:58). Here every sequence owns a list of 64-token pages taken from a shared
pool, so ragged batches and early finishes do not waste memory. For MLA one cached token is
the 576-wide latent (compressed KV + rotary key); for gated-attention layers it is K and V of
the 2 KV heads.

Bookkeeping (free list, page lists, lengths) lives in the native ``PageTable`` of
csrc/runtime.cpp, which owns host mirrors of the block table and the length vector; the cache
uploads them when they changed (the upload snapshots the pageable mirrors at call time). Without the library the same
bookkeeping runs in ``PageAllocator`` (Python). On CUDA, new rows are scattered into their pages
by the ``paged_kv_write`` kernel and read by the paged decode kernel (csrc/mla_decode_sm100.cu).
"""
from __future__ import annotations

from typing import List, Optional

import torch


class PageAllocator:
    """Free-list page allocator with per-sequence ownership (Python fallback of the native table)."""

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


class _PyTable:
    """Same interface as the native page table, in Python."""

    def __init__(self, n_pages, page_size, max_seqs, max_pages, pin):
        self.page_size, self.max_pages = page_size, max_pages
        self.alloc = PageAllocator(n_pages)
        self.table = torch.full((max_seqs, max_pages), -1, dtype=torch.int32)
        self.lens = torch.zeros(max_seqs, dtype=torch.int32)
        self.version = 0

    def reserve(self, seqs, new_lens) -> int:
        added = 0
        for s, n in zip(seqs, new_lens):
            have = len(self.alloc.owned.get(s, []))
            need = (n + self.page_size - 1) // self.page_size
            if need > self.max_pages:
                raise ValueError("sequence exceeds max_pages_per_seq")
            if need > have:
                pages = self.alloc.alloc(s, need - have)
                self.table[s, have:need] = torch.tensor(pages, dtype=torch.int32)
                added += need - have
        self.version += added > 0
        return added

    def advance(self, seqs, n):
        for s in seqs:
            self.lens[s] += n
        self.version += 1

    def release(self, s):
        self.alloc.release(s)
        self.table[s].fill_(-1)
        self.lens[s] = 0
        self.version += 1

    def length(self, s) -> int:
        return int(self.lens[s])

    def n_free(self) -> int:
        return self.alloc.n_free


class _NativeTable:
    def __init__(self, ops, n_pages, page_size, max_seqs, max_pages, pin):
        self._ops = ops
        self._h = ops.pagetable_create(n_pages, page_size, max_seqs, max_pages, pin)
        self.table, self.lens = ops.pagetable_tensors(self._h)

    def reserve(self, seqs, new_lens) -> int:
        try:
            return self._ops.pagetable_reserve(self._h, list(seqs), list(new_lens))
        except RuntimeError as e:
            if "exhausted" in str(e):
                raise MemoryError(str(e).splitlines()[0]) from None
            if "block table has" in str(e):
                raise ValueError(str(e).splitlines()[0]) from None
            raise

    def advance(self, seqs, n):
        self._ops.pagetable_advance(self._h, list(seqs), n)

    def release(self, s):
        self._ops.pagetable_release(self._h, s)

    def length(self, s) -> int:
        return self._ops.pagetable_length(self._h, s)

    def n_free(self) -> int:
        return self._ops.pagetable_n_free(self._h)

    @property
    def version(self) -> int:
        return self._ops.pagetable_version(self._h)

    def __del__(self):
        try:
            self._ops.pagetable_close(self._h)
        except Exception:
            pass


class PagedCache:
    """``pool``: (n_layers, n_pages, page_size, width). ``block_table``: (max_seqs, max_pages_per_seq)
    int32 page ids (-1 = unassigned). ``seq_lens``: (max_seqs,) int32 tokens stored per sequence."""

    def __init__(self, n_layers: int, width: int, n_pages: int, page_size: int = 64, max_seqs: int = 64,
                 max_pages_per_seq: int = 64, dtype=torch.bfloat16, device="cpu", native: Optional[bool] = None):
        self.page_size, self.width, self.n_layers = page_size, width, n_layers
        self.device = torch.device(device)
        self.pool = torch.zeros(n_layers, n_pages, page_size, width, dtype=dtype, device=device)
        on_gpu = self.device.type == "cuda"
        ops = None
        if native is not False:
            try:
                from .. import _ext
                ops = _ext.ops()
            except Exception:
                if native or on_gpu:
                    raise
        self._ops = ops
        mk = (lambda *a: _NativeTable(ops, *a)) if ops is not None else _PyTable
        # pageable mirrors: an upload snapshots them at call time, so later bookkeeping cannot race the copy
        self._tab = mk(n_pages, page_size, max_seqs, max_pages_per_seq, False)
        self.block_table = self._tab.table.to(device).clone()
        self.seq_lens = self._tab.lens.to(device).clone()
        self._synced = self._tab.version
        self._id_cache = {}

    # ---- bookkeeping ------------------------------------------------------------------------
    @property
    def alloc(self):
        """Free-page view (``n_free``) for callers that size batches by the remaining pages."""
        tab = self._tab

        class _View:
            n_free = property(lambda s: tab.n_free())
        return _View()

    def _sync(self) -> None:
        v = self._tab.version
        if v != self._synced:
            self.block_table.copy_(self._tab.table, non_blocking=True)
            self.seq_lens.copy_(self._tab.lens, non_blocking=True)
            self._synced = v

    def reserve(self, seq_id: int, new_len: int) -> None:
        """Makes sure sequence ``seq_id`` owns enough pages for ``new_len`` tokens."""
        self._tab.reserve([seq_id], [new_len])
        self._sync()

    def seq_id_tensor(self, seq_ids) -> torch.Tensor:
        key = tuple(seq_ids)
        t = self._id_cache.get(key)
        if t is None:
            t = torch.tensor(list(key), dtype=torch.int32, device=self.device)
            if len(self._id_cache) > 64:
                self._id_cache.clear()
            self._id_cache[key] = t
        return t

    def slots(self, seq_id: int, start: int, n: int):
        """(page ids, in-page offsets) of tokens [start, start+n) of a sequence, as device tensors."""
        pos = torch.arange(start, start + n, device=self.block_table.device)
        pages = self.block_table[seq_id, (pos // self.page_size).long()].long()
        return pages, (pos % self.page_size).long()

    def append(self, layer: int, seq_ids, rows: torch.Tensor, commit: bool = False) -> None:
        """rows (B, T, width): writes T new tokens of every listed sequence at its current length.
        ``commit`` advances the lengths (do it once per model step, after the last layer)."""
        B, T, _ = rows.shape
        seq_ids = list(seq_ids)
        starts = [self._tab.length(s) for s in seq_ids]
        self._tab.reserve(seq_ids, [s + T for s in starts])
        self._sync()
        if rows.is_cuda and self.pool.dtype == torch.bfloat16 and self.width % 8 == 0:
            ids = self.seq_id_tensor(seq_ids)
            start = self.seq_lens[ids.long()]   # device lengths equal the host ones after _sync
            self._ops.paged_kv_write(rows.to(torch.bfloat16).contiguous(), self.pool[layer], self.block_table, ids, start)
        else:
            for b, sid in enumerate(seq_ids):
                pages, offs = self.slots(sid, starts[b], T)
                self.pool[layer, pages, offs] = rows[b].to(self.pool.dtype)
        if commit:
            self.commit(seq_ids, T)

    def commit(self, seq_ids, n_new: int) -> None:
        self._tab.advance(list(seq_ids), n_new)
        self._sync()

    def gather(self, layer: int, seq_id: int, length: Optional[int] = None) -> torch.Tensor:
        """Dense (length, width) view of one sequence (reference path and tests)."""
        length = self._tab.length(seq_id) if length is None else length
        pages, offs = self.slots(seq_id, 0, length)
        return self.pool[layer, pages, offs]

    def length(self, seq_id: int) -> int:
        return self._tab.length(seq_id)

    def release(self, seq_id: int) -> None:
        self._tab.release(seq_id)
        self._sync()
