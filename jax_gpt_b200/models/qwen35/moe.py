"""Mixture-of-experts FFN (jax_gpt/models/qwen35/moe.py:19-282).

Router: fp32 softmax over all experts, top-k, renormalise to sum 1. Experts: SwiGLU. Output:
weighted sum of the chosen experts plus a shared SwiGLU expert scaled by ``sigmoid(x @ w)``.
No capacity limit, no token dropping, no auxiliary loss.

Single device: tokens are grouped by expert and run through a grouped GEMM. Expert parallel:
``expert_forward_ep`` sends every (token, expert) row to the rank that owns the expert with an
all-to-all, computes only local experts and returns the weighted rows with a second all-to-all
(the reference replicates tokens, computes all rows on every rank and sums with one ``psum``,
jax_gpt/models/qwen35/moe.py:117-222). The fused CUDA path lives in parallel/expert_parallel.py.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from .fp8 import dequantize_weight, is_fp8_weight, matmul_maybe_fp8


def moe_routing(x: torch.Tensor, gate_weight, k: int):
    """x (M, D) -> (weights (M,k) fp32 summing to 1, expert ids (M,k) int64)."""
    from ...ops.router import softmax_topk_router
    from ...ops.gemm import linear_f32out
    logits = matmul_maybe_fp8(x, gate_weight).float() if is_fp8_weight(gate_weight) else linear_f32out(x, gate_weight)
    return softmax_topk_router(logits, k)


def _dense(w, dtype):
    return dequantize_weight(w, dtype) if is_fp8_weight(w) else w


def grouped_swiglu(xs: torch.Tensor, group_sizes, gate_proj, up_proj, down_proj, expert_offset: int = 0):
    """Rows of ``xs`` are contiguous per expert; expert e (global id expert_offset + e) owns
    ``group_sizes[e]`` rows. Kernels are stacked (E, D, I) / (E, I, D)."""
    from ...ops import grouped_gemm
    return grouped_gemm.grouped_swiglu(xs, group_sizes, _dense(gate_proj, xs.dtype), _dense(up_proj, xs.dtype),
                                       _dense(down_proj, xs.dtype))


def _n_local_experts(params) -> int:
    g = params["gate_proj"]
    return (g["w"] if is_fp8_weight(g) else g).shape[0]


def expert_forward_single(x: torch.Tensor, weights: torch.Tensor, idx: torch.Tensor, params) -> torch.Tensor:
    """x (M,D); weights/idx (M,k). Returns sum_k w_k * expert_{idx_k}(x)."""
    M, D = x.shape
    k = idx.shape[1]
    E = (params["gate_proj"]["w"] if is_fp8_weight(params["gate_proj"]) else params["gate_proj"]).shape[0]
    flat = idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    tok = order // k
    sizes = torch.bincount(flat, minlength=E)
    ys = grouped_swiglu(x[tok], sizes, params["gate_proj"], params["up_proj"], params["down_proj"])
    ys = ys * weights.reshape(-1)[order][:, None].to(ys.dtype)
    out = torch.zeros(M, D, dtype=torch.float32, device=x.device)
    out.index_add_(0, tok, ys.float())
    return out.to(x.dtype)


def expert_forward_ep(x: torch.Tensor, weights: torch.Tensor, idx: torch.Tensor, params, group, n_experts: int):
    """Expert-parallel forward over ``group`` with all-to-all dispatch and combine (library
    collectives; the baseline of the fused kernels). ``params`` hold only the local experts."""
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    M, D = x.shape
    k = idx.shape[1]
    e_local = n_experts // world
    flat = idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    tok = order // k
    dest = flat[order] // e_local
    send_counts = torch.bincount(dest, minlength=world)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    sc, rc = send_counts.tolist(), recv_counts.tolist()
    rows = x[tok].contiguous()
    eid = (flat[order] % e_local).contiguous()
    recv_rows = rows.new_empty(sum(rc), D)
    recv_eid = eid.new_empty(sum(rc))
    dist.all_to_all_single(recv_rows, rows, rc, sc, group=group)
    dist.all_to_all_single(recv_eid, eid, rc, sc, group=group)
    lorder = torch.argsort(recv_eid, stable=True)
    sizes = torch.bincount(recv_eid, minlength=e_local)
    ys = grouped_swiglu(recv_rows[lorder], sizes, params["gate_proj"], params["up_proj"], params["down_proj"])
    back = torch.empty_like(ys)
    back[lorder] = ys
    ret = rows.new_empty(rows.shape[0], D)
    dist.all_to_all_single(ret, back.contiguous(), sc, rc, group=group)
    ret = ret * weights.reshape(-1)[order][:, None].to(ret.dtype)
    out = torch.zeros(M, D, dtype=torch.float32, device=x.device)
    out.index_add_(0, tok, ret.float())
    return out.to(x.dtype)


def expert_forward_tp(x: torch.Tensor, weights: torch.Tensor, idx: torch.Tensor, params, group, n_experts: int):
    """Experts split over a TENSOR-parallel group whose ranks all hold the same tokens: every rank runs the
    (token, expert) rows of its own experts and the partial outputs are summed over the group, the scheme of the
    reference's expert parallelism (jax_gpt/models/qwen35/moe.py:117-222), without its full-size masked work."""
    from ...parallel.tp_ops import reduce_from_tp, tp_rank, tp_world
    world, rank = tp_world(group), tp_rank(group)
    M, D = x.shape
    k = idx.shape[1]
    e_local = n_experts // world
    flat = idx.reshape(-1) - rank * e_local
    sel = ((flat >= 0) & (flat < e_local)).nonzero(as_tuple=True)[0]
    eid = flat[sel]
    order = torch.argsort(eid, stable=True)
    sel = sel[order]
    tok = sel // k
    sizes = torch.bincount(eid, minlength=e_local)
    ys = grouped_swiglu(x[tok], sizes, params["gate_proj"], params["up_proj"], params["down_proj"])
    ys = ys * weights.reshape(-1)[sel][:, None].to(ys.dtype)
    out = torch.zeros(M, D, dtype=torch.float32, device=x.device)
    out = out.index_add(0, tok, ys.float())
    return reduce_from_tp(out, group).to(x.dtype)


def shared_expert_forward(x: torch.Tensor, params) -> torch.Tensor:
    if "shared_gate_up_proj" in params:       # gate | up as one GEMM over concatenated weights (decode engine)
        gu = matmul_maybe_fp8(x, params["shared_gate_up_proj"])
        half = gu.shape[-1] // 2
        return matmul_maybe_fp8(F.silu(gu[..., :half]) * gu[..., half:], params["shared_down_proj"])
    g = matmul_maybe_fp8(x, params["shared_gate_proj"])
    u = matmul_maybe_fp8(x, params["shared_up_proj"])
    return matmul_maybe_fp8(F.silu(g) * u, params["shared_down_proj"])


def moe_layer(x: torch.Tensor, params, n_experts_per_token: int, n_devices: int = 1, axis_name: str = "tp",
              mesh=None, group=None, n_experts: Optional[int] = None, tp_group=None) -> torch.Tensor:
    """x (B,T,D) -> (B,T,D). With ``group`` the routed experts run expert-parallel: a process group
    selects the all-to-all library path, a callable ``group(x, weights, idx, params, grads)`` (the fused
    kernel runtime of parallel/expert_parallel.py) the one-kernel path; ``params`` then hold only this
    rank's experts and, when training, their fp32 gradient buffers under ``<name>@grad``. ``tp_group``: the
    ranks hold the SAME tokens (tensor parallelism) and, when the expert axis of ``params`` is a shard, split
    the experts among them (partial outputs summed over the group)."""
    B, T, D = x.shape
    xf = x.reshape(B * T, D)
    w, idx = moe_routing(xf, params["gate_weight"], n_experts_per_token)
    if callable(group):
        grads = {n: params.get(n + "@grad") for n in ("gate_proj", "up_proj", "down_proj")}
        routed = group(xf, w, idx, params, grads).to(x.dtype)
    elif group is not None:
        routed = expert_forward_ep(xf, w, idx, params, group, n_experts)
    elif tp_group is not None and n_experts is not None and _n_local_experts(params) < n_experts:
        from ...parallel.tp_ops import copy_to_tp
        # entry of the sharded region: activations and routing weights get the SUM of the ranks' gradients
        routed = expert_forward_tp(copy_to_tp(xf, tp_group), copy_to_tp(w, tp_group), idx, params, tp_group, n_experts)
    else:
        routed = expert_forward_single(xf, w, idx, params)
    shared = shared_expert_forward(xf, params)
    sg = torch.sigmoid(matmul_maybe_fp8(xf, params["shared_expert_gate_weight"]).float()).to(x.dtype)
    return (routed + shared * sg).reshape(B, T, D)
