"""Layer and group assembly (jax_gpt/models/qwen35/block.py:19-137): every layer is
``x += mixer(norm(x)); x += moe(norm(x))``; a group is three Gated-DeltaNet layers followed by
one gated-attention layer."""
from __future__ import annotations

import torch

from ...parallel.tp_ops import copy_to_tp, reduce_from_tp
from ...utils.profiling import scope
from .deltanet import deltanet_prefill, deltanet_recurrent_step
from .gqa import gqa_attention
from .moe import moe_layer
from .primitives import rms_norm


def _slice(tree, i):
    if isinstance(tree, dict):
        if "w" in tree and "scale_inv" in tree:
            return {"w": tree["w"][i], "scale_inv": tree["scale_inv"][i]}
        return {k: _slice(v, i) for k, v in tree.items()}
    return tree[i]


def _local_delta_heads(attn_params, config):
    """(qk heads, v heads) held by this rank: the head axis of ``in_proj_a`` tells whether the layer is a
    tensor-parallel shard (head-aligned split, models/qwen35/sharding.py)."""
    w = attn_params["in_proj_a"]
    n_v = (w["w"].shape[-2] if isinstance(w, dict) else w.shape[-1])
    return config.delta_n_qk_heads * n_v // config.delta_n_v_heads, n_v


def deltanet_layer_forward(x, lp, delta_M, delta_conv, config, is_decode: bool, ep_group=None, tp_group=None):
    """One DeltaNet layer. Returns (x, new_state, new_conv_state). With ``tp_group`` and head-sharded weights the
    mixer runs on this rank's heads (state and conv window are the matching shards) and the row-parallel output
    projection is summed over the group."""
    c = config
    n_qk, n_v = _local_delta_heads(lp["attn"], c)
    sharded = n_v < c.delta_n_v_heads
    with scope("deltanet_attn"):
        h = rms_norm(x, lp["attn_norm"], c.rms_norm_eps)
        ap = lp["attn"]
        if sharded:
            h = copy_to_tp(h, tp_group)
            # a replicated weight used INSIDE the sharded region (the per-head output norm): each rank sees the
            # gradient of its heads only, so its gradient is summed over the group like an activation's
            ap = dict(ap, norm_weight=copy_to_tp(ap["norm_weight"], tp_group))
        if is_decode:
            a, M, conv = deltanet_recurrent_step(h, ap, delta_M, delta_conv, n_qk, n_v, c.delta_qk_head_dim,
                                                 c.delta_v_head_dim)
        else:
            a, M, conv = deltanet_prefill(h, ap, n_qk, n_v, c.delta_qk_head_dim, c.delta_v_head_dim,
                                          c.delta_conv_kernel, c.delta_chunk_size)
        if sharded:
            a = reduce_from_tp(a, tp_group)
        x = x + a
    with scope("deltanet_moe"):
        h = rms_norm(x, lp["moe_norm"], c.rms_norm_eps)
        x = x + moe_layer(h, lp["moe"], c.n_experts_per_token, group=ep_group, n_experts=c.n_routed_experts,
                          tp_group=tp_group)
    return x, M, conv


def gqa_layer_forward(x, lp, cache_k, cache_v, cache_pos, config, rope_freqs, ep_group=None, tp_group=None):
    """One gated-attention layer. Returns (x, new_k, new_v)."""
    c = config
    with scope("gqa_attn"):
        h = rms_norm(x, lp["attn_norm"], c.rms_norm_eps)
        a, nk, nv = gqa_attention(h, lp["attn"], c.gqa_n_q_heads, c.gqa_n_kv_heads, c.gqa_head_dim, rope_freqs,
                                  c.gqa_rope_dim, cache_k, cache_v, cache_pos, tp_group=tp_group)
        x = x + a
    with scope("gqa_moe"):
        h = rms_norm(x, lp["moe_norm"], c.rms_norm_eps)
        x = x + moe_layer(h, lp["moe"], c.n_experts_per_token, group=ep_group, n_experts=c.n_routed_experts,
                          tp_group=tp_group)
    return x, nk, nv


def group_forward(x, group_params, delta_Ms, delta_convs, gqa_k, gqa_v, cache_pos, config, rope_freqs,
                  is_decode: bool, n_devices: int = 1, mesh=None, axis_name: str = "tp", ep_group=None, tp_group=None):
    """One 4-layer group. delta_Ms (3,B,Hv,dk,dv) / delta_convs (3,B,C,K) or None; gqa_k/gqa_v
    (B,Hkv,max_len,dh) or None. Returns (x, new_delta_Ms, new_delta_convs, new_k, new_v)."""
    nd = config.n_delta_per_group
    if tp_group is None and mesh is not None:
        tp_group = getattr(mesh, "group", None)
    new_M, new_conv = [], []
    for i in range(nd):
        lp = _slice(group_params["delta_layers"], i)
        M_i = delta_Ms[i] if delta_Ms is not None else None
        c_i = delta_convs[i] if delta_convs is not None else None
        x, M, conv = deltanet_layer_forward(x, lp, M_i, c_i, config, is_decode, ep_group, tp_group)
        new_M.append(M)
        new_conv.append(conv)
    if tp_group is None and mesh is not None:
        tp_group = getattr(mesh, "group", None)
    x, nk, nv = gqa_layer_forward(x, group_params["gqa_layer"], gqa_k, gqa_v, cache_pos, config, rope_freqs, ep_group,
                                  tp_group)
    return x, torch.stack(new_M), torch.stack(new_conv), nk, nv
