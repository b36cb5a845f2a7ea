"""HF Qwen3.5-MoE state dict -> this package's parameter tree
(jax_gpt/models/qwen35/weight_loader.py:26-252).

HF linear weights are (out,in) and become (in,out); the fused expert tensor ``gate_up_proj``
(E, 2I, D) splits into ``gate_proj`` / ``up_proj`` (E, D, I); ``down_proj`` (E, D, I) becomes
(E, I, D); the depthwise conv weight (C,1,K) is squeezed to (C,K). Both the text-only prefix
``model.layers`` and the multimodal ``model.language_model.layers`` are recognised.

With ``shard=(rank, world)`` the expert axis is sliced while loading, so a rank only ever
materialises its own experts (the reference achieves the same with per-shard callbacks,
jax_gpt/models/qwen35/weight_loader.py:151-196).
"""
from __future__ import annotations

from typing import Optional

import torch

from .config import Qwen35Config


def _t(w, dtype):
    return w.detach().to(dtype).transpose(-1, -2).contiguous()


def _moe(sd, prefix, c: Qwen35Config, dtype, shard):
    I = c.moe_intermediate_size
    gate_up = sd[f"{prefix}.mlp.experts.gate_up_proj"].detach()
    down = sd[f"{prefix}.mlp.experts.down_proj"].detach()
    if shard is not None:
        r, w = shard
        e = c.n_routed_experts // w
        gate_up, down = gate_up[r * e:(r + 1) * e], down[r * e:(r + 1) * e]
    return {
        "gate_weight": _t(sd[f"{prefix}.mlp.gate.weight"], dtype),
        "gate_proj": gate_up[:, :I, :].to(dtype).transpose(1, 2).contiguous(),
        "up_proj": gate_up[:, I:, :].to(dtype).transpose(1, 2).contiguous(),
        "down_proj": down.to(dtype).transpose(1, 2).contiguous(),
        "shared_gate_proj": _t(sd[f"{prefix}.mlp.shared_expert.gate_proj.weight"], dtype),
        "shared_up_proj": _t(sd[f"{prefix}.mlp.shared_expert.up_proj.weight"], dtype),
        "shared_down_proj": _t(sd[f"{prefix}.mlp.shared_expert.down_proj.weight"], dtype),
        "shared_expert_gate_weight": _t(sd[f"{prefix}.mlp.shared_expert_gate.weight"], dtype),
    }


def load_delta_layer(sd, prefix, c, dtype, shard=None):
    g = lambda k: sd[f"{prefix}.{k}"].detach().to(dtype)
    attn = {
        "in_proj_qkv": _t(sd[f"{prefix}.linear_attn.in_proj_qkv.weight"], dtype),
        "in_proj_z": _t(sd[f"{prefix}.linear_attn.in_proj_z.weight"], dtype),
        "in_proj_b": _t(sd[f"{prefix}.linear_attn.in_proj_b.weight"], dtype),
        "in_proj_a": _t(sd[f"{prefix}.linear_attn.in_proj_a.weight"], dtype),
        "conv_weight": g("linear_attn.conv1d.weight").squeeze(1),
        "A_log": g("linear_attn.A_log"), "dt_bias": g("linear_attn.dt_bias"), "norm_weight": g("linear_attn.norm.weight"),
        "out_proj": _t(sd[f"{prefix}.linear_attn.out_proj.weight"], dtype),
    }
    return {"attn_norm": g("input_layernorm.weight"), "attn": attn, "moe_norm": g("post_attention_layernorm.weight"),
            "moe": _moe(sd, prefix, c, dtype, shard)}


def load_gqa_layer(sd, prefix, c, dtype, shard=None):
    g = lambda k: sd[f"{prefix}.{k}"].detach().to(dtype)
    attn = {k: _t(sd[f"{prefix}.self_attn.{k}.weight"], dtype) for k in ("q_proj", "k_proj", "v_proj", "o_proj")}
    attn["q_norm"] = g("self_attn.q_norm.weight")
    attn["k_norm"] = g("self_attn.k_norm.weight")
    return {"attn_norm": g("input_layernorm.weight"), "attn": attn, "moe_norm": g("post_attention_layernorm.weight"),
            "moe": _moe(sd, prefix, c, dtype, shard)}


def _stack(trees):
    if isinstance(trees[0], dict):
        return {k: _stack([t[k] for t in trees]) for k in trees[0]}
    return torch.stack(trees)


def detect_prefixes(sd):
    multimodal = any("language_model" in k for k in sd)
    base = "model.language_model" if multimodal else "model"
    return f"{base}.layers", f"{base}.embed_tokens.weight", f"{base}.norm.weight"


def load_from_hf_state_dict(sd, config: Qwen35Config, mesh=None, axis_rules=None, dtype=torch.bfloat16,
                            shard: Optional[tuple] = None, device="cpu") -> dict:
    """``sd``: mapping of HF names to tensors (lazy mappings work: each key is read once)."""
    c = config
    layers, embed_key, norm_key = detect_prefixes(sd)
    groups = []
    for gi in range(c.n_groups):
        base = gi * c.full_attention_interval
        deltas = [load_delta_layer(sd, f"{layers}.{base + i}", c, dtype, shard) for i in range(c.n_delta_per_group)]
        gqa = load_gqa_layer(sd, f"{layers}.{base + c.n_delta_per_group}", c, dtype, shard)
        groups.append({"delta_layers": _stack(deltas), "gqa_layer": gqa})
    params = {
        "embed": sd[embed_key].detach().to(dtype), "final_norm": sd[norm_key].detach().to(dtype),
        "lm_head": _t(sd["lm_head.weight"], dtype), "groups": _stack(groups),
    }
    if device != "cpu":
        from .sharding import tree_map
        params = tree_map(lambda t: t.to(device), params)
    return params
