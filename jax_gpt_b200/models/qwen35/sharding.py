"""Tensor / expert sharding rules for the Qwen3.5 tree (jax_gpt/models/qwen35/sharding.py:35-373).

Every parameter suffix has logical axes; a rule set maps logical axes to the mesh axis (or
None = replicated). ``shard_params`` slices a full tree into the local shard of ``rank``:

* rules A: heads / intermediate / experts / vocab all split over the one ``tp`` axis;
* rules B: only experts and vocab are split (attention replicated).

A dimension that the mesh size does not divide stays replicated. Unlike the reference, which
splits ``in_proj_qkv`` on the concatenated q|k|v axis (jax_gpt/models/qwen35/sharding.py:49),
q, k and v segments are split head-aligned so that a rank holds whole heads.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from .config import Qwen35Config

# suffix -> logical axes of the TRAILING dims (leading stack axes are never sharded)
LOGICAL_AXES: Dict[str, Tuple[Optional[str], ...]] = {
    "embed": ("vocab", None), "lm_head": (None, "vocab"), "final_norm": (None,),
    "attn_norm": (None,), "moe_norm": (None,),
    "attn.in_proj_qkv": (None, "delta_qkv"), "attn.in_proj_z": (None, "delta_v"), "attn.in_proj_b": (None, "delta_heads"),
    "attn.in_proj_a": (None, "delta_heads"), "attn.conv_weight": ("delta_qkv", None), "attn.A_log": ("delta_heads",),
    "attn.dt_bias": ("delta_heads",), "attn.norm_weight": (None,), "attn.out_proj": ("delta_v", None),
    "attn.q_proj": (None, "q_heads"), "attn.k_proj": (None, "kv_heads"), "attn.v_proj": (None, "kv_heads"),
    "attn.o_proj": ("q_heads_out", None), "attn.q_norm": (None,), "attn.k_norm": (None,),
    "moe.gate_weight": (None, None), "moe.gate_proj": ("experts", None, None), "moe.up_proj": ("experts", None, None),
    "moe.down_proj": ("experts", None, None), "moe.shared_gate_proj": (None, None), "moe.shared_up_proj": (None, None),
    "moe.shared_down_proj": (None, None), "moe.shared_expert_gate_weight": (None, None),
}

AXIS_RULES_A = {"vocab": "tp", "experts": "tp", "q_heads": "tp", "q_heads_out": "tp", "kv_heads": None,
                "delta_qkv": "tp", "delta_v": "tp", "delta_heads": "tp"}
AXIS_RULES_B = {"vocab": "tp", "experts": "tp", "q_heads": None, "q_heads_out": None, "kv_heads": None,
                "delta_qkv": None, "delta_v": None, "delta_heads": None}


@dataclass
class Mesh:
    """A 1-D device mesh: ``n_devices`` ranks on one axis; ``group`` is the process group of that axis (None: the
    default group when torch.distributed is initialised, else a single process)."""
    n_devices: int
    axis_name: str = "tp"
    group: object = None


def make_mesh(n_devices: Optional[int] = None, axis_name: str = "tp", group=None) -> Mesh:
    import torch.distributed as dist
    live = dist.is_available() and dist.is_initialized()
    if n_devices is None:
        n_devices = dist.get_world_size(group) if live else 1
    if group is None and live and n_devices == dist.get_world_size():
        group = dist.group.WORLD
    return Mesh(n_devices, axis_name, group)


def tree_map(fn, tree):
    if isinstance(tree, dict):
        return {k: tree_map(fn, v) for k, v in tree.items()}
    return fn(tree)


def flatten(tree, prefix=""):
    out = {}
    for k, v in tree.items():
        name = f"{prefix}.{k}" if prefix else k
        if isinstance(v, dict) and not ("w" in v and "scale_inv" in v):
            out.update(flatten(v, name))
        else:
            out[name] = v
    return out


def resolve_logical_axes(name: str):
    """Longest-suffix match of a flattened parameter name against LOGICAL_AXES."""
    best = None
    for suffix in LOGICAL_AXES:
        if name == suffix or name.endswith("." + suffix):
            if best is None or len(suffix) > len(best):
                best = suffix
    if best is None:
        raise KeyError(f"no logical axes for parameter {name!r}")
    return LOGICAL_AXES[best]


def _split_sizes(axis: str, c: Qwen35Config):
    """Segments that must be split separately so shards stay head-aligned."""
    if axis == "delta_qkv":
        return [c.delta_key_dim, c.delta_key_dim, c.delta_value_dim]
    return None


def shard_tensor(name: str, t: torch.Tensor, c: Qwen35Config, rules, world: int, rank: int) -> torch.Tensor:
    axes = resolve_logical_axes(name)
    lead = t.dim() - len(axes)
    for i, ax in enumerate(axes):
        if ax is None or rules.get(ax) is None or world == 1:
            continue
        dim = lead + i
        segs = _split_sizes(ax, c) or [t.shape[dim]]
        unit = {"q_heads": 2 * c.gqa_head_dim, "q_heads_out": c.gqa_head_dim, "delta_heads": 1,
                "delta_v": c.delta_v_head_dim, "delta_qkv": c.delta_qk_head_dim}.get(ax, 1)
        if any(s % (world * unit) != 0 for s in segs):
            continue  # not divisible: keep replicated
        parts, off = [], 0
        for s in segs:
            n = s // world
            parts.append(t.narrow(dim, off + rank * n, n))
            off += s
        t = torch.cat(parts, dim=dim) if len(parts) > 1 else parts[0]
    return t.contiguous()


def shard_params(params, mesh: Mesh, config: Qwen35Config, axis_rules=None, rank: Optional[int] = None):
    """Returns the local shard of ``params`` for ``rank`` (default: this process's rank)."""
    rules = axis_rules or AXIS_RULES_A
    if rank is None:
        import torch.distributed as dist
        rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0

    def rec(tree, prefix):
        out = {}
        for k, v in tree.items():
            name = f"{prefix}.{k}" if prefix else k
            out[k] = rec(v, name) if isinstance(v, dict) else shard_tensor(name, v, config, rules, mesh.n_devices, rank)
        return out
    return rec(params, "")


def make_cache_sharding(config: Qwen35Config, mesh: Mesh, axis_rules=None):
    """Which cache dims are split: DeltaNet state / conv over v heads when divisible, KV replicated."""
    rules = axis_rules or AXIS_RULES_A
    w = mesh.n_devices
    heads = rules.get("delta_heads") is not None and config.delta_n_v_heads % w == 0
    return {"delta_M": ("heads" if heads else None), "delta_conv": ("channels" if heads else None), "gqa_kv": None}


def shard_cache(cache, mesh: Mesh, config: Qwen35Config, axis_rules=None, rank: int = 0):
    from .cache import HybridCache
    spec = make_cache_sharding(config, mesh, axis_rules)
    w = mesh.n_devices
    M, conv = cache.delta_M, cache.delta_conv
    if spec["delta_M"] and w > 1:
        h = config.delta_n_v_heads // w
        M = M[:, :, :, rank * h:(rank + 1) * h].contiguous()
        conv = shard_tensor("attn.conv_weight", conv.transpose(-1, -2).transpose(-2, -1), config, axis_rules or AXIS_RULES_A,
                            w, rank)
    return HybridCache(M, conv, cache.gqa_k, cache.gqa_v, cache.pos)


def get_output_shardings(config: Qwen35Config, mesh: Mesh, axis_rules=None):
    """Logits are replicated; caches follow :func:`make_cache_sharding`."""
    return {"logits": None, **make_cache_sharding(config, mesh, axis_rules)}
