"""Layer-streaming forward (jax_gpt/models/qwen35/offload.py:51-383): the weights stay on disk
in HF safetensors shards; one 4-layer group at a time is read, placed on the device, run and
released, so the resident footprint is one group plus embedding, final norm and head.
On a B200 the copy of group g+1 (pinned host buffer, side stream) overlaps the compute of g.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import torch

from .block import group_forward
from .cache import HybridCache
from .config import Qwen35Config
from .fp8 import matmul_maybe_fp8
from .primitives import precompute_rope_freqs, rms_norm
from .sharding import tree_map
from .weight_loader import _stack, _t, detect_prefixes, load_delta_layer, load_gqa_layer


class LazySafetensors:
    """Mapping name -> tensor over a directory of ``*.safetensors`` files; tensors are read on access."""

    def __init__(self, model_dir: str):
        from safetensors import safe_open
        self._open = safe_open
        self.dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        self.where: Dict[str, str] = {}
        if os.path.exists(index):
            with open(index) as f:
                self.where = dict(json.load(f)["weight_map"])
        else:
            for fn in sorted(os.listdir(model_dir)):
                if fn.endswith(".safetensors"):
                    with safe_open(os.path.join(model_dir, fn), framework="pt") as f:
                        for k in f.keys():
                            self.where[k] = fn
        self._handles = {}

    def __iter__(self):
        return iter(self.where)

    def __contains__(self, k):
        return k in self.where

    def keys(self):
        return self.where.keys()

    def __getitem__(self, k):
        fn = self.where[k]
        h = self._handles.get(fn)
        if h is None:
            h = self._open(os.path.join(self.dir, fn), framework="pt")
            self._handles[fn] = h
        return h.get_tensor(k)


def load_group(sd, gi: int, c: Qwen35Config, dtype, shard=None) -> dict:
    layers, _, _ = detect_prefixes(sd)
    base = gi * c.full_attention_interval
    deltas = [load_delta_layer(sd, f"{layers}.{base + i}", c, dtype, shard) for i in range(c.n_delta_per_group)]
    return {"delta_layers": _stack(deltas), "gqa_layer": load_gqa_layer(sd, f"{layers}.{base + c.n_delta_per_group}", c, dtype, shard)}


def forward_offload(tokens, config: Qwen35Config, model_dir, mesh=None, axis_rules=None,
                    cache: Optional[HybridCache] = None, is_decode: bool = False, verbose: bool = True,
                    dtype=torch.bfloat16, device=None, state_dict=None):
    """Same result as ``forward`` with weights streamed group by group from ``model_dir``
    (or from an in-memory ``state_dict`` of HF names). Returns (logits, new_cache | None)."""
    c = config
    sd = state_dict if state_dict is not None else LazySafetensors(model_dir)
    device = torch.device(device) if device is not None else tokens.device
    _, embed_key, norm_key = detect_prefixes(sd)
    embed = sd[embed_key].to(dtype).to(device)
    final_norm = sd[norm_key].to(dtype).to(device)
    lm_head = _t(sd["lm_head.weight"], dtype).to(device)
    x = embed[tokens.to(device).long()]
    B, T = tokens.shape
    pos = cache.pos if cache is not None else 0
    max_pos = cache.gqa_k.shape[3] if cache is not None else pos + T
    rope = precompute_rope_freqs(c.gqa_rope_dim, max(max_pos, pos + T), c.gqa_rope_theta, device=device)
    copy_stream = torch.cuda.Stream(device) if device.type == "cuda" else None

    def fetch(gi):
        gp = load_group(sd, gi, c, dtype)
        if copy_stream is None:
            return tree_map(lambda t: t.to(device), gp), None
        with torch.cuda.stream(copy_stream):
            gp = tree_map(lambda t: t.pin_memory().to(device, non_blocking=True), gp)
            ev = torch.cuda.Event()
            ev.record(copy_stream)
        return gp, ev

    new_M, new_conv = [], []
    nxt = fetch(0)
    for gi in range(c.n_groups):
        gp, ev = nxt
        if gi + 1 < c.n_groups:
            nxt = fetch(gi + 1)  # overlaps with this group's compute
        if ev is not None:
            torch.cuda.current_stream(device).wait_event(ev)
        if cache is not None:
            dM, dC, ck, cv = cache.delta_M[gi], cache.delta_conv[gi], cache.gqa_k[gi], cache.gqa_v[gi]
        else:
            dM = dC = ck = cv = None
        x, M, conv, _, _ = group_forward(x, gp, dM, dC, ck, cv, pos, c, rope, is_decode)
        new_M.append(M)
        new_conv.append(conv)
        if verbose:
            print(f"[offload] group {gi + 1}/{c.n_groups} done", flush=True)
        del gp
    x = rms_norm(x, final_norm, c.rms_norm_eps)
    logits = matmul_maybe_fp8(x, lm_head)
    new_cache = None
    if cache is not None:
        new_cache = HybridCache(torch.stack(new_M).to(cache.delta_M.dtype),
                                torch.stack(new_conv).to(cache.delta_conv.dtype), cache.gqa_k, cache.gqa_v, pos + T)
    return logits, new_cache
