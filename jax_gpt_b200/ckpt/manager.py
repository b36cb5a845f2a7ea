"""Asynchronous checkpointing with the reference's payload and API
(jax_gpt/trainer/checkpointing.py:16-113).

Payload: ``{"step", "params", "opt_state"}``. ``params`` is the model's parameter tree with the
reference's names, shapes, (in,out) orientation and layer stacking; the optimizer state keeps
the optax chain's content: Adam ``count`` / ``mu`` / ``nu`` (mirroring the parameter tree) and
the schedule ``count``. On disk::

    <checkpoint_dir>/<step>/params.safetensors       # flattened tree, '.'-joined keys
    <checkpoint_dir>/<step>/opt_state.safetensors    # mu.<key>, nu.<key>
    <checkpoint_dir>/<step>/manifest.json            # step, counts, data cursor, key lists; written LAST

``save`` copies device tensors into pinned host memory and returns; a native writer thread
(csrc/runtime.cpp) streams them to ``*.tmp`` files and renames them, then writes the manifest,
so a directory without a manifest is an unfinished checkpoint and is ignored. If a file of a checkpoint
fails to write, the writer drops the rest of that checkpoint (no manifest appears) and the error is raised
by ``wait_until_finished``. Older checkpoints are only deleted once enough NEWER ones are complete on disk
(at the next ``save`` and in ``wait_until_finished``), never while the newest is still in flight.

With a sharded optimizer (``state.engine.dist_optimizer``) the weights and moments live as per-rank shards:
``save`` then assembles them itself, which makes it a COLLECTIVE call that every rank must make; only rank 0
writes. The saved tree does not depend on the number of ranks. Orbax's OCDBT
container cannot be produced without TensorStore; the tree is the same, the container differs.
"""
from __future__ import annotations

import json
import os
import shutil
from typing import Optional

import torch

from ..models.qwen35.sharding import flatten


def _unflatten(flat):
    out = {}
    for k, v in flat.items():
        d = out
        parts = k.split(".")
        for p in parts[:-1]:
            d = d.setdefault(p, {})
        d[parts[-1]] = v
    return out


def save_tree(path: str, tree: dict) -> None:
    """Writes a nested tensor dict as ONE safetensors file with '.'-joined keys (written to ``.tmp`` and renamed)."""
    from safetensors.torch import save_file
    flat = {k: v.detach().to("cpu").contiguous() for k, v in flatten(tree).items()}
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    save_file(flat, path + ".tmp")
    os.replace(path + ".tmp", path)


def load_tree(path: str, device="cpu") -> dict:
    from safetensors.torch import load_file
    return _unflatten(load_file(path, device=str(device)))


def _model_params(model):
    if hasattr(model, "params"):
        return model.params() if callable(model.params) else model.params
    return dict(model.named_parameters())


class CheckpointManager:
    def __init__(self, config, model_config=None, timeout_secs: float = 300.0):
        self._config = config
        self._model_config = model_config
        self._dir = config.checkpoint_dir
        self._keep = config.max_checkpoints_to_keep
        self._timeout = timeout_secs
        os.makedirs(self._dir, exist_ok=True)
        self._writer = None
        self._ops = None
        try:
            from .. import _ext
            self._ops = _ext.ops()
            self._writer = self._ops.writer_create()
        except Exception:
            self._writer = None

    # ---------------------------------------------------------------------------------------
    def _stage(self, tree_flat):
        """Device -> pinned host copies (non-blocking), returns names and CPU tensors."""
        names, tensors = [], []
        cuda = False
        for k, v in tree_flat.items():
            t = v.detach()
            if t.is_cuda:
                cuda = True
                h = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                h.copy_(t, non_blocking=True)
                t = h
            else:
                t = t.contiguous().clone()
            names.append(k)
            tensors.append(t)
        if cuda:
            torch.cuda.current_stream().synchronize()
        return names, tensors

    def save(self, step: int, state, data_state: Optional[dict] = None) -> None:
        """Non-blocking: returns once the tensors are staged in host memory. With a sharded optimizer every rank
        must call it (the shards are gathered collectively) and only rank 0 writes."""
        eng = getattr(state, "engine", None)
        gathered = None
        if eng is not None and getattr(eng, "dist_optimizer", None) is not None:
            # the optimizer kernels update per-rank shards and no rank holds the full fp32 weights: gather them
            # (and the moments) now, into temporaries that only this save uses
            gathered = eng.params()
            st = eng.opt_state()
            state.opt_state.mu, state.opt_state.nu = st["mu"], st["nu"]
            if getattr(eng.dist_optimizer, "rank", 0) != 0:
                return
        self._prune()      # complete checkpoints only; the one about to be written does not count yet
        params = gathered if gathered is not None else _model_params(state.model)
        flat_p = flatten(params) if any(isinstance(v, dict) for v in params.values()) else dict(params)
        opt = state.opt_state
        mu = getattr(opt, "mu", None) or (opt.get("mu") if isinstance(opt, dict) else {})
        nu = getattr(opt, "nu", None) or (opt.get("nu") if isinstance(opt, dict) else {})
        flat_o = {f"mu.{k}": v for k, v in (flatten(mu) if any(isinstance(v, dict) for v in mu.values()) else mu).items()}
        flat_o.update({f"nu.{k}": v for k, v in (flatten(nu) if any(isinstance(v, dict) for v in nu.values()) else nu).items()})
        d = os.path.join(self._dir, str(step))
        os.makedirs(d, exist_ok=True)
        count = int(getattr(opt, "count", step) if not isinstance(opt, dict) else opt.get("count", step))
        manifest = {"step": int(step), "opt_count": count, "schedule_count": count, "format": "safetensors",
                    "params": sorted(flat_p), "opt_state": sorted(flat_o), "data_state": data_state or {}}
        pn, pt = self._stage(flat_p)
        on, ot = self._stage(flat_o)
        if self._writer is not None:
            self._ops.writer_submit_safetensors(self._writer, os.path.join(d, "params.safetensors"), pn, pt)
            self._ops.writer_submit_safetensors(self._writer, os.path.join(d, "opt_state.safetensors"), on, ot)
            self._ops.writer_submit_bytes(self._writer, os.path.join(d, "manifest.json"), json.dumps(manifest))
        else:
            from safetensors.torch import save_file
            save_file(dict(zip(pn, pt)), os.path.join(d, "params.safetensors"))
            save_file(dict(zip(on, ot)), os.path.join(d, "opt_state.safetensors"))
            with open(os.path.join(d, "manifest.json"), "w") as f:
                json.dump(manifest, f)
            self._prune()

    def _complete_steps(self):
        out = []
        if os.path.isdir(self._dir):
            for n in os.listdir(self._dir):
                if n.isdigit() and os.path.exists(os.path.join(self._dir, n, "manifest.json")):
                    out.append(int(n))
        return sorted(out)

    def _prune(self):
        """Keeps the newest ``max_checkpoints_to_keep`` COMPLETE checkpoints (those with a manifest)."""
        steps = self._complete_steps()
        for s in steps[:-self._keep] if self._keep > 0 else []:
            shutil.rmtree(os.path.join(self._dir, str(s)), ignore_errors=True)

    # ---------------------------------------------------------------------------------------
    def restore(self, step: Optional[int], state):
        """Loads ``step`` (or the latest complete checkpoint) INTO ``state``: parameters in place,
        moments, counts. Returns the state; unchanged if there is nothing to restore."""
        self.wait_until_finished()
        s = step if step is not None else self.latest_step()
        if s is None:
            return state
        from safetensors.torch import load_file
        d = os.path.join(self._dir, str(s))
        with open(os.path.join(d, "manifest.json")) as f:
            manifest = json.load(f)
        flat_p = load_file(os.path.join(d, "params.safetensors"))
        flat_o = load_file(os.path.join(d, "opt_state.safetensors"))
        mu = {k[3:]: v for k, v in flat_o.items() if k.startswith("mu.")}
        nu = {k[3:]: v for k, v in flat_o.items() if k.startswith("nu.")}
        if getattr(state, "engine", None) is not None:
            state.engine.load(flat_p, {"mu": mu, "nu": nu}, manifest["opt_count"])
        else:
            params = _model_params(state.model)
            cur = flatten(params) if any(isinstance(v, dict) for v in params.values()) else params
            with torch.no_grad():
                for k, v in flat_p.items():
                    cur[k].copy_(v.to(cur[k].dtype))
                omu = flatten(state.opt_state.mu) if any(isinstance(v, dict) for v in state.opt_state.mu.values()) else state.opt_state.mu
                onu = flatten(state.opt_state.nu) if any(isinstance(v, dict) for v in state.opt_state.nu.values()) else state.opt_state.nu
                for k, v in mu.items():
                    omu[k].copy_(v)
                for k, v in nu.items():
                    onu[k].copy_(v)
        state.opt_state.count = manifest["opt_count"]
        state.step = manifest["step"]
        self.last_manifest = manifest
        return state

    def wait_until_finished(self) -> None:
        if self._writer is not None:
            ok = self._ops.writer_wait(self._writer, self._timeout)
            err = self._ops.writer_last_error(self._writer)
            if err:
                raise RuntimeError(f"checkpoint write failed: {err}")
            if not ok:
                raise TimeoutError(f"checkpoint writes did not finish within {self._timeout} s")
            self._prune()

    def latest_step(self) -> Optional[int]:
        steps = self._complete_steps()
        return steps[-1] if steps else None

    def should_save(self, step: int) -> bool:
        return self._config.save_interval > 0 and step % self._config.save_interval == 0   # 0 = never save periodically

    def close(self):
        if self._writer is not None:
            self.wait_until_finished()
            self._ops.writer_close(self._writer)
            self._writer = None
