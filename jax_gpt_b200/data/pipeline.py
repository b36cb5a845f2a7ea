"""Token-window data pipeline (jax_gpt/data/pipeline.py:36-150).

``<local_data_path>/<split>.bin`` is a flat uint16 array. Window ``i`` is tokens
``[i*S, i*S + S + 1)``; a batch stacks ``micro_batch_size`` windows and returns
``x = w[:, :-1], y = w[:, 1:]`` as int32. Each data-parallel rank reads windows
``rank, rank + world, ...``. The native loader (csrc/runtime.cpp) memory-maps the file and a
prefetch thread fills pinned host tensors ahead of the training loop, so the host->device copy
of step n+1 never waits for the page cache. ``skip_to_step`` seeks in O(1); the reference
replays ``step * accum * micro_batch`` items (jax_gpt/data/pipeline.py:142-150).

``data_source='gcs'`` names ``gs://<gcs_bucket>/<gcs_dataset_path>/<split>`` (jax_gpt/data/pipeline.py:29-30,
93-98, where grain reads ArrayRecord shards from the bucket). Here the bucket is read through a file-system mount
(gcsfuse or any other): ``<mount>/<gcs_bucket>/<gcs_dataset_path>/<split>.bin`` in the same flat uint16 format, with
``<mount>`` taken from the environment variable ``B200_GCS_MOUNT`` (default ``/gcs``), so the memory-mapped native
loader serves both sources. Without such a mount the constructor says what it looked for.
"""
from __future__ import annotations

import os

import numpy as np
import torch


def _world():
    try:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            return dist.get_rank(), dist.get_world_size()
    except Exception:
        pass
    return 0, 1


def gcs_mounted_path(config, split: str) -> str:
    """File behind ``gs://<gcs_bucket>/<gcs_dataset_path>/<split>`` on the bucket's file-system mount."""
    if not config.gcs_bucket:
        raise ValueError("data_source='gcs' needs gcs_bucket (and gcs_dataset_path)")
    root = os.environ.get("B200_GCS_MOUNT", "/gcs")
    path = os.path.join(root, config.gcs_bucket, config.gcs_dataset_path.strip("/"), f"{split}.bin")
    if not os.path.exists(path):
        raise FileNotFoundError(
            f"gs://{config.gcs_bucket}/{config.gcs_dataset_path}/{split}: expected the bucket mounted at {root} "
            f"(set B200_GCS_MOUNT) with the flat uint16 token file {path}")
    return path


class DataPipeline:
    def __init__(self, config, split: str = "train", *, _shard_index=None, _shard_count=None, use_native: bool = True,
                 prefetch: int = 8):
        if config.data_source == "local":
            self.path = os.path.join(config.local_data_path, f"{split}.bin")
            if not os.path.exists(self.path):
                raise FileNotFoundError(self.path)
        elif config.data_source == "gcs":
            self.path = gcs_mounted_path(config, split)
        else:
            raise ValueError(f"Unknown data_source '{config.data_source}'. Expected 'local' or 'gcs'.")
        rank, world = _world()
        self.shard_index = rank if _shard_index is None else _shard_index
        self.shard_count = world if _shard_count is None else _shard_count
        self.seq_len, self.mb = config.seq_len, config.micro_batch_size
        self._cursor = 0
        self._handle = None
        n_tokens = os.path.getsize(self.path) // 2
        self.num_windows = (n_tokens - 1) // self.seq_len
        self.num_local_windows = (self.num_windows - self.shard_index + self.shard_count - 1) // self.shard_count
        if use_native:
            try:
                from .. import _ext
                self._ops = _ext.ops()
                # num_workers (worker processes of the reference's grain loader, jax_gpt/data/pipeline.py:117-125) sizes
                # the prefetch queue of the single native reader thread: batches kept ready ahead of the training loop
                depth = max(prefetch, 2 * int(getattr(config, "num_workers", 0)))
                self._handle = self._ops.loader_create(self.path, self.seq_len, self.mb, self.shard_index,
                                                       self.shard_count, depth, torch.cuda.is_available())
            except Exception:
                self._handle = None
        if self._handle is None:
            self._data = np.memmap(self.path, dtype=np.uint16, mode="r")

    def get_batch(self):
        """(x, y): int32 tensors of shape (micro_batch_size, seq_len); pinned when CUDA is present."""
        if self._handle is not None:
            self._cursor += self.mb
            return self._ops.loader_next(self._handle)
        rows = []
        for b in range(self.mb):
            local = (self._cursor + b) % self.num_local_windows
            w = self.shard_index + local * self.shard_count
            rows.append(np.asarray(self._data[w * self.seq_len:w * self.seq_len + self.seq_len + 1], dtype=np.int32))
        self._cursor += self.mb
        t = torch.from_numpy(np.stack(rows))
        return t[:, :-1].contiguous(), t[:, 1:].contiguous()

    def skip_to_step(self, step: int, grad_accum_steps: int = 1) -> None:
        """Positions the stream where a run that already did ``step`` optimizer steps would be."""
        self._cursor = step * grad_accum_steps * self.mb
        if self._handle is not None:
            self._ops.loader_seek(self._handle, self._cursor)

    def state(self) -> dict:
        return {"cursor": self._cursor}

    def close(self):
        if self._handle is not None:
            self._ops.loader_close(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
