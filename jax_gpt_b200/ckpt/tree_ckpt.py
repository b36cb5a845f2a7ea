"""Periodic checkpoints of the function-style (MoE) training engines, sharded by rank and re-shardable on load.

The GPT-2 trainer state goes through ``ckpt/manager.py`` (the reference's payload and API,
jax_gpt/trainer/checkpointing.py:47-101, which knows GPT-2 only). ``TreeTrainEngine`` holds two kinds of state:
the dense group, whose optimizer state is sharded over the data-parallel ranks, and the expert-parallel leaves,
of which every rank owns the experts ``[rank * E / world, (rank + 1) * E / world)``. A checkpoint is

    <dir>/<step>/dense.safetensors            master / mu / nu of the dense leaves, gathered, written by rank 0
    <dir>/<step>/experts_rank<r>.safetensors  master / mu / nu of rank r's experts, written by rank r
    <dir>/<step>/manifest.json                step, expert-parallel degree, expert axis of every leaf; written LAST

so a directory without a manifest is unfinished and ignored. ``load`` works at ANY expert-parallel degree that
divides the expert count: each rank assembles its expert range from the files that overlap it.
"""
from __future__ import annotations

import json
import os
import shutil
from typing import Optional

import torch

from ..models.qwen35.sharding import flatten
from .manager import _unflatten


def _flat3(triple, prefix):
    out = {}
    for name, tree in zip(("master", "mu", "nu"), triple):
        for k, v in flatten(tree).items():
            out[f"{prefix}{name}/{k}"] = v.detach().to("cpu").contiguous()
    return out


class TreeCheckpointer:
    def __init__(self, directory: str, keep: int = 3, rank: int = 0, world: int = 1, barrier=None):
        self.dir, self.keep, self.rank, self.world = directory, keep, rank, world
        self._barrier = barrier or (lambda: None)
        os.makedirs(directory, exist_ok=True)

    # ------------------------------------------------------------------------------------------------
    def complete_steps(self):
        out = []
        for n in os.listdir(self.dir) if os.path.isdir(self.dir) else []:
            if n.isdigit() and os.path.exists(os.path.join(self.dir, n, "manifest.json")):
                out.append(int(n))
        return sorted(out)

    def latest_step(self) -> Optional[int]:
        s = self.complete_steps()
        return s[-1] if s else None

    def save(self, step: int, engine, extra: Optional[dict] = None) -> None:
        """COLLECTIVE over the ranks of the job: every rank calls it (the dense state is gathered, every rank writes
        its experts, rank 0 writes the manifest after all files exist)."""
        from safetensors.torch import save_file
        d = os.path.join(self.dir, str(step))
        os.makedirs(d, exist_ok=True)
        self._barrier()
        dense = engine.dense_state()                      # collective with a sharded optimizer
        if self.rank == 0:
            save_file(_flat3(dense, ""), os.path.join(d, "dense.safetensors.tmp"))
            os.replace(os.path.join(d, "dense.safetensors.tmp"), os.path.join(d, "dense.safetensors"))
        local = engine.local_state()
        axes = {}
        if engine.local_offsets:
            flat = _flat3(local, "")
            for k, v in flatten(local[0]).items():
                axes[k] = v.dim() - 3                     # stacked routed experts: the expert axis is third from last
            path = os.path.join(d, f"experts_rank{self.rank}.safetensors")
            save_file(flat, path + ".tmp")
            os.replace(path + ".tmp", path)
        self._barrier()
        if self.rank == 0:
            manifest = {"step": int(step), "ep_world": self.world if engine.local_offsets else 0,
                        "expert_axes": axes, "extra": extra or {}}
            with open(os.path.join(d, "manifest.json.tmp"), "w") as f:
                json.dump(manifest, f)
            os.replace(os.path.join(d, "manifest.json.tmp"), os.path.join(d, "manifest.json"))
            for s in self.complete_steps()[:-self.keep] if self.keep > 0 else []:
                shutil.rmtree(os.path.join(self.dir, str(s)), ignore_errors=True)
        self._barrier()

    def load(self, engine, step: Optional[int] = None) -> Optional[dict]:
        """Restores ``engine`` from ``step`` (default: the latest complete one). Returns the manifest or None when
        there is nothing to restore. The expert-parallel degree may differ from the one that saved."""
        from safetensors import safe_open
        from safetensors.torch import load_file
        step = step if step is not None else self.latest_step()
        if step is None:
            return None
        d = os.path.join(self.dir, str(step))
        with open(os.path.join(d, "manifest.json")) as f:
            manifest = json.load(f)
        flat = load_file(os.path.join(d, "dense.safetensors"))
        dense = tuple(_unflatten({k.split("/", 1)[1]: v for k, v in flat.items() if k.startswith(name + "/")})
                      for name in ("master", "mu", "nu"))
        local = None
        if engine.local_offsets:
            old = int(manifest["ep_world"])
            assert old > 0, "the checkpoint has no expert-parallel leaves"
            files = [safe_open(os.path.join(d, f"experts_rank{r}.safetensors"), framework="pt", device="cpu")
                     for r in range(old)]
            trees = ({}, {}, {})
            for p, (_, _, shape) in engine.local_offsets.items():
                key = ".".join(p)
                ax = int(manifest["expert_axes"][key])
                e_new = shape[ax]
                lo, hi = self.rank * e_new, (self.rank + 1) * e_new          # this rank's global expert range
                for name, tree in zip(("master", "mu", "nu"), trees):
                    parts = []
                    for r, fh in enumerate(files):
                        sl = fh.get_slice(f"{name}/{key}")
                        e_old = sl.get_shape()[ax]
                        a, b = max(lo, r * e_old), min(hi, (r + 1) * e_old)
                        if a < b:
                            idx = [slice(None)] * len(shape)
                            idx[ax] = slice(a - r * e_old, b - r * e_old)
                            parts.append(sl[tuple(idx)])
                    t = torch.cat(parts, dim=ax) if len(parts) > 1 else parts[0]
                    node = tree
                    for k in p[:-1]:
                        node = node.setdefault(k, {})
                    node[p[-1]] = t
            local = trees
        engine.load_state(dense, local, manifest["step"])
        return manifest
