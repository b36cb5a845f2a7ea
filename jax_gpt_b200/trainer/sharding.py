"""Trainer-side sharding: the device mesh of a training job, the GPT-2 sharding rules and the functions that turn
a full train state into the local shard (jax_gpt/trainer/sharding.py:24-194 in the reference).

The reference annotates parameters with logical axes, maps them to the mesh axes ``('dp','fsdp','tp','sp')`` and
lets the XLA partitioner insert the collectives. Here the mesh is a set of ``torch.distributed`` process groups
(one per axis, one process per GPU), the rules are the same table, and the collectives are explicit:
``GPT.__call__(..., mesh=mesh)`` runs the Megatron-style tensor-parallel forward of parallel/tp_ops.py on the
shards that :func:`shard_train_state` produces, data-parallel gradients go through the fused sharded optimizer
(parallel/fsdp.py) and pipeline stages through parallel/pipeline.py.

Unlike the reference, which splits the fused ``c_attn`` output on the concatenated q|k|v axis, the q, k and v
segments are split separately so that a rank holds whole heads of all three.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

import torch

# logical axis name -> mesh axis (None: replicated); change this table to rearrange the parallelism
LOGICAL_AXIS_RULES: Dict[str, Optional[str]] = {
    "vocab": "tp", "embed": None, "joined_heads": "tp", "heads": "tp", "mlp": "tp", "context": None, "layers": "pp",
}

# parameter name -> logical axes of its TRAILING dims (a leading stacked-layer axis is handled by padding)
LOGICAL_SPECS: Dict[str, Tuple[Optional[str], ...]] = {
    "wte.embedding": ("vocab", "embed"), "wpe.embedding": ("context", "embed"),
    "h.attn.c_attn.kernel": ("embed", "joined_heads"), "h.attn.c_attn.bias": ("joined_heads",),
    "h.attn.c_proj.kernel": ("heads", "embed"), "h.attn.c_proj.bias": ("embed",),
    "h.mlp.c_fc.kernel": ("embed", "mlp"), "h.mlp.c_fc.bias": ("mlp",),
    "h.mlp.c_proj.kernel": ("mlp", "embed"), "h.mlp.c_proj.bias": ("embed",),
    "h.ln_1.layer_norm.scale": ("embed",), "h.ln_1.layer_norm.bias": ("embed",),
    "h.ln_2.layer_norm.scale": ("embed",), "h.ln_2.layer_norm.bias": ("embed",),
    "ln_f.layer_norm.scale": ("embed",), "ln_f.layer_norm.bias": ("embed",),
    "lm_head.kernel": ("embed", "vocab"),
}

AXES = ("pp", "dp", "fsdp", "tp", "sp")


@dataclass
class DeviceMesh:
    """Axis sizes, this process's coordinate on every axis and one process group per axis (None for an axis of
    size 1 or without torch.distributed). Ranks are laid out with ``sp`` fastest, then ``tp``, ``fsdp``, ``dp``,
    ``pp``, so a tensor-parallel group is a run of consecutive ranks (neighbouring GPUs)."""
    sizes: Dict[str, int]
    coords: Dict[str, int] = field(default_factory=dict)
    groups: Dict[str, object] = field(default_factory=dict)

    @property
    def shape(self):
        return {a: self.sizes[a] for a in AXES}

    def size(self, axis: str) -> int:
        return self.sizes.get(axis, 1)

    def rank(self, axis: str) -> int:
        return self.coords.get(axis, 0)

    @property
    def group(self):
        """The tensor-parallel group (what model code takes as ``mesh.group``)."""
        return self.groups.get("tp")

    @property
    def n_devices(self) -> int:
        return self.sizes.get("tp", 1)


def make_mesh(config, world: Optional[int] = None, rank: Optional[int] = None, create_groups: bool = True) -> DeviceMesh:
    """Mesh of a training job from ``TrainConfig`` (dp, fsdp, tp, sp, pp). ``dp * fsdp * tp * sp * pp`` must equal
    the number of processes. Collective: every process has to call it (it creates the per-axis groups)."""
    import torch.distributed as dist
    live = dist.is_available() and dist.is_initialized()
    world = world if world is not None else (dist.get_world_size() if live else 1)
    rank = rank if rank is not None else (dist.get_rank() if live else 0)
    sizes = {a: int(getattr(config, a, 1)) for a in AXES}
    total = 1
    for a in AXES:
        total *= sizes[a]
    if total != world:
        raise ValueError(f"dp*fsdp*tp*sp*pp = {total} does not match the number of processes ({world})")
    # coordinates: sp fastest
    coords, rem = {}, rank
    for a in reversed(AXES):
        coords[a] = rem % sizes[a]
        rem //= sizes[a]
    groups: Dict[str, object] = {}
    if live and create_groups and world > 1:
        strides, s = {}, 1
        for a in reversed(AXES):
            strides[a] = s
            s *= sizes[a]
        for a in AXES:
            if sizes[a] == 1:
                continue
            # every set of ranks that differ only in coordinate `a` forms one group; all processes create all of them
            seen = set()
            for r in range(world):
                base = r - ((r // strides[a]) % sizes[a]) * strides[a]
                if base in seen:
                    continue
                seen.add(base)
                members = [base + i * strides[a] for i in range(sizes[a])]
                g = dist.new_group(members)
                if rank in members:
                    groups[a] = g
    return DeviceMesh(sizes, coords, groups)


def logical_to_physical(logical_spec, ndim: int) -> tuple:
    """Maps a tuple of logical axis names to mesh axes with LOGICAL_AXIS_RULES; when the array has more dims than
    the spec (a leading stacked-layers axis) the front is padded with None."""
    axes = list(logical_spec)
    if ndim > len(axes):
        axes = [None] * (ndim - len(axes)) + axes
    return tuple(LOGICAL_AXIS_RULES.get(a) if a is not None else None for a in axes)


def param_spec(name: str, ndim: int) -> tuple:
    """Physical spec of a GPT-2 parameter (longest matching name of LOGICAL_SPECS; unknown names are replicated)."""
    best = None
    for k in LOGICAL_SPECS:
        if (name == k or name.endswith(k) or k in name) and (best is None or len(k) > len(best)):
            best = k
    return logical_to_physical(LOGICAL_SPECS[best], ndim) if best is not None else (None,) * ndim


def shard_gpt2_tensor(name: str, t: torch.Tensor, model_config, mesh: DeviceMesh) -> torch.Tensor:
    """The tensor-parallel shard of one GPT-2 parameter (or of an optimizer moment of the same name and shape)."""
    w, r = mesh.size("tp"), mesh.rank("tp")
    if w == 1:
        return t
    spec = param_spec(name, t.dim())
    d = model_config.d_model
    for dim, ax in enumerate(spec):
        if ax != "tp":
            continue
        n = t.shape[dim]
        fused_qkv = "c_attn" in name and n == 3 * d
        segs = [d, d, d] if fused_qkv else [n]
        unit = model_config.d_head if ("c_attn" in name or "attn.c_proj.kernel" in name) else 1
        if any(s % (w * unit) != 0 for s in segs):
            continue          # not divisible: stays replicated
        parts, off = [], 0
        for s in segs:
            parts.append(t.narrow(dim, off + r * (s // w), s // w))
            off += s
        t = torch.cat(parts, dim=dim) if len(parts) > 1 else parts[0]
    return t.contiguous()


def shard_train_state(state, mesh: DeviceMesh, model_config=None):
    """Replaces the model's parameters and the Adam moments of ``state`` by this rank's tensor-parallel shards
    (optimizer leaves follow the parameter of the same name). Data / FSDP axes do not slice the state here: the
    sharded optimizer owns that split (parallel/fsdp.py). Returns the state."""
    cfg = model_config or getattr(state.model, "config", None)
    if mesh.size("tp") == 1:
        return state
    params = state.model.params
    state.model.params = {k: shard_gpt2_tensor(k, v.detach(), cfg, mesh).requires_grad_(v.requires_grad)
                          for k, v in params.items()}
    opt = state.opt_state
    for slot in ("mu", "nu"):
        tree = getattr(opt, slot, None)
        if isinstance(tree, dict):
            setattr(opt, slot, {k: shard_gpt2_tensor(k, v, cfg, mesh) for k, v in tree.items()})
    return state


def activation_sharding_constraint(x: torch.Tensor, spec, mesh: Optional[DeviceMesh]):
    """The reference's hint to the partitioner (jax_gpt/trainer/sharding.py:190-194). Collectives are explicit in
    this runtime, so the activation is returned as it is; the spec is checked against the mesh so that a layout
    that cannot exist (a dim the axis size does not divide) is reported where it is written."""
    if mesh is None:
        return x
    for dim, ax in enumerate(spec):
        if ax is not None and mesh.size(ax) > 1 and dim < x.dim() and x.shape[dim] % mesh.size(ax) != 0 and ax != "tp":
            raise ValueError(f"activation dim {dim} of size {x.shape[dim]} cannot be split over '{ax}' ({mesh.size(ax)})")
    return x
