"""Analytic roofline for the Qwen3.5 / DeepSeek building blocks and for fused
compute+collective kernels.

The reference derives FLOPs and bytes from ``jax.experimental.roofline`` with TPU v5p constants
(459 TFLOP/s, 2.8 TB/s; scripts/qwen35_benchmark.py:78-194). Here the counts are written out
per module and the denominators are the rates MEASURED on the B200 pool (``MEASURED_PEAKS.json``
in the repository root when present, otherwise the documented fallback). A fused
compute+collective kernel is bounded by ``max(FLOPs / GEMM rate, NVLink bytes / link rate)``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NVLINK_GBS_MEASURED = 770.0   # peer copy, per direction per GPU
NVLINK_GBS_NOMINAL = 900.0


def load_peaks(root: str = ""):
    root = root or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return dict(FALLBACK, source="fallback")


@dataclass
class Roofline:
    name: str
    flops: float
    hbm_bytes: float
    nvlink_bytes: float = 0.0

    def bound(self, peaks=None, sustained: bool = False):
        peaks = peaks or load_peaks()
        rate = peaks["bf16_tflops_sustained" if sustained else "bf16_tflops"] * 1e12
        t_c = self.flops / rate
        t_m = self.hbm_bytes / (peaks["hbm_gbs"] * 1e9)
        t_l = self.nvlink_bytes / (NVLINK_GBS_MEASURED * 1e9)
        t = max(t_c, t_m, t_l)
        kind = "compute" if t == t_c else ("hbm" if t == t_m else "nvlink")
        return {"name": self.name, "seconds": t, "bound": kind, "flops": self.flops, "hbm_bytes": self.hbm_bytes,
                "nvlink_bytes": self.nvlink_bytes, "intensity": self.flops / max(self.hbm_bytes, 1.0),
                "denominators": peaks["source"]}

    def fraction(self, measured_seconds: float, peaks=None, sustained: bool = False) -> float:
        return self.bound(peaks, sustained)["seconds"] / measured_seconds


def linear(name, M, K, N, bytes_per=2):
    return Roofline(name, 2.0 * M * K * N, bytes_per * (M * K + K * N + M * N))


def qwen35_modules(c, B: int, T: int, decode: bool = False, bytes_per: int = 2):
    """Per-layer module rooflines of the Qwen3.5 hybrid for B sequences of T new tokens."""
    M, D = B * T, c.d_model
    Kd, Vd, Hv = c.delta_key_dim, c.delta_value_dim, c.delta_n_v_heads
    dk, dv, C = c.delta_qk_head_dim, c.delta_v_head_dim, c.delta_chunk_size
    out = [linear("deltanet.in_proj", M, D, 2 * Kd + 2 * Vd + 2 * Hv, bytes_per), linear("deltanet.out_proj", M, Vd, D, bytes_per)]
    if decode:
        out.append(Roofline("deltanet.state_update", B * Hv * 6.0 * dk * dv, B * Hv * dk * dv * 4 * 2))
    else:
        per_chunk = 2.0 * C * C * dk * 2 + 2.0 * C * C * dv + 2.0 * C * dk * dv * 3 + C * C * C / 3.0 * 2
        out.append(Roofline("deltanet.chunk_scan", B * Hv * (T / C) * per_chunk, bytes_per * M * (2 * Kd + 2 * Vd)))
    Hq, Hkv, dh = c.gqa_n_q_heads, c.gqa_n_kv_heads, c.gqa_head_dim
    out += [linear("gqa.qkv_proj", M, D, 2 * Hq * dh + 2 * Hkv * dh, bytes_per), linear("gqa.o_proj", M, Hq * dh, D, bytes_per)]
    S = T if not decode else T
    out.append(Roofline("gqa.sdpa", 4.0 * B * Hq * T * S * dh * (0.5 if not decode else 1.0),
                        bytes_per * (M * Hq * dh * 2 + B * S * Hkv * dh * 2)))
    E, k, I, SI = c.n_routed_experts, c.n_experts_per_token, c.moe_intermediate_size, c.shared_expert_intermediate_size
    active = min(E, M * k)
    out.append(Roofline("moe.experts", 2.0 * M * k * 3 * D * I, bytes_per * (active * 3 * D * I + 2 * M * k * D)))
    out.append(Roofline("moe.shared_expert", 2.0 * M * 3 * D * SI, bytes_per * (3 * D * SI + 2 * M * D)))
    out.append(linear("moe.router", M, D, E, bytes_per))
    return out


def ep_moe_layer(tokens_per_rank: int, d_model: int, inter: int, top_k: int, max_dest_ranks: int, world: int,
                 fp8: bool = True):
    """Roofline of the fused expert-parallel MoE forward on one rank (balanced routing)."""
    flops = 2.0 * tokens_per_rank * top_k * 3 * d_model * inter
    remote = (world - 1) / world
    disp = tokens_per_rank * max_dest_ranks * remote * (d_model * (1 if fp8 else 2) + (d_model // 128) * 4)
    comb = tokens_per_rank * max_dest_ranks * remote * d_model * 2
    r = Roofline("ep_moe_fwd", flops, 0.0, disp + comb)
    if fp8:
        r.flops = flops / 2.0  # fp8 tensor rate is twice the bf16 rate used as the denominator
    return r
