"""Block-scaled FP8 (e4m3) API in one place: quantisation (1x128 activation blocks, 128x128 weight blocks,
optional power-of-two scales), the two GEMMs (fp32 scales with software promotion; power-of-two scales applied by
the tensor core), the packed exponent-byte layout, the inference layer, and (re-exported from ops/fp8_linear.py) the
training path. Kernels: csrc/seq_kernels.cu (quantisers), gemm_fp8_sm100.cu, gemm_mxfp8_sm100.cu. Reference
counterpart: per-row W8A8 inference in jax_gpt/models/qwen35/fp8.py:50-150 and quantize.py.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _ext

FP8_MAX = 448.0


def _pow2_ceil(s):
    return torch.exp2(torch.ceil(torch.log2(s)))


def fp8_quant_1x128_ref(x, pow2: bool = False):
    M, K = x.shape
    xb = x.float().view(M, K // 128, 128)
    sc = xb.abs().amax(-1).clamp_min(1e-12) / FP8_MAX
    if pow2:
        sc = _pow2_ceil(sc)
    q = (xb / sc[..., None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(M, K)
    return q, sc


def fp8_quant_128x128_ref(w, pow2: bool = False):
    R, C = w.shape
    wb = w.float().view(R // 128, 128, C // 128, 128)
    sc = wb.abs().amax(dim=(1, 3)).clamp_min(1e-12) / FP8_MAX
    if pow2:
        sc = _pow2_ceil(sc)
    q = (wb / sc[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(R, C)
    return q, sc


def fp8_quant_1x128(x, pow2: bool = False):
    """x (M,K) bf16 -> (q (M,K) e4m3, scales (M,K/128) fp32) with x ~= q * scale per 1x128 block."""
    if not (x.is_cuda and x.dtype == torch.bfloat16):
        return fp8_quant_1x128_ref(x, pow2)
    M, K = x.shape
    q = torch.empty(M, K, device=x.device, dtype=torch.float8_e4m3fn)
    sc = torch.empty(M, K // 128, device=x.device, dtype=torch.float32)
    _ext.ops().fp8_quant(x.contiguous(), q, sc, False, pow2)
    return q, sc


def fp8_quant_128x128(w, pow2: bool = False):
    """w (R,C) bf16 -> (q (R,C) e4m3, scales (R/128,C/128) fp32), one scale per 128x128 block."""
    if not (w.is_cuda and w.dtype == torch.bfloat16):
        return fp8_quant_128x128_ref(w, pow2)
    R, C = w.shape
    q = torch.empty(R, C, device=w.device, dtype=torch.float8_e4m3fn)
    sc = torch.empty(R // 128, C // 128, device=w.device, dtype=torch.float32)
    _ext.ops().fp8_quant(w.contiguous(), q, sc, True, pow2)
    return q, sc


def fp8_gemm_ref(a_q, a_s, b_q, b_s):
    """fp32 reference of the block-scaled product: de-quantise both operands, multiply."""
    M, K = a_q.shape
    N = b_q.shape[0]
    a = a_q.float().view(M, K // 128, 128) * a_s[..., None]
    bs = b_s.repeat_interleave(128, dim=0)[:N]
    b = b_q.float().view(N, K // 128, 128) * bs[..., None]
    return a.view(M, K) @ b.view(N, K).t()


def fp8_gemm(a_q, a_s, b_q, b_s, out_dtype=torch.bfloat16):
    """a_q [M,K] e4m3 with 1x128 scales, b_q [N,K] e4m3 with 128x128 scales -> [M,N]."""
    if not a_q.is_cuda:
        return fp8_gemm_ref(a_q, a_s, b_q, b_s).to(out_dtype)
    out = torch.empty(a_q.shape[0], b_q.shape[0], device=a_q.device, dtype=out_dtype)
    _ext.ops().gemm_fp8(a_q, a_s, b_q, b_s, out)
    return out


def pack_scales_ue8m0(scales: torch.Tensor, rows: int, per_row: bool) -> torch.Tensor:
    """Power-of-two fp32 block scales -> the packed UE8M0 layout the hardware-scaled GEMM reads:
    ``[ceil(rows/128), K/128, 512]`` bytes, byte ``(r % 32) * 16 + (r / 32) * 4 + j`` of a chunk being the
    exponent of row r for the j-th 32-wide K block of the slab (all four j equal here).
    ``per_row``: scales are (rows, K/128) (1x128 activation scales); else (ceil(rows/128), K/128)
    (128x128 weight scales)."""
    e = (torch.log2(scales.float()).round() + 127).clamp(0, 254).to(torch.uint8)
    KS = e.shape[1]
    MB = (rows + 127) // 128
    if per_row:
        pad = torch.full((MB * 128, KS), 127, dtype=torch.uint8, device=e.device)
        pad[:rows] = e
        t = pad.view(MB, 4, 32, KS).permute(0, 3, 2, 1)                  # (MB, KS, lane, group)
        return t.unsqueeze(-1).expand(MB, KS, 32, 4, 4).reshape(MB, KS, 512).contiguous()
    return e[:MB, :, None].expand(MB, KS, 512).contiguous()


def mxfp8_gemm(a_q, a_s, b_q, b_s):
    """Same product as ``fp8_gemm`` for POWER-OF-TWO scales, with the scaling done by the tensor core
    (tcgen05 block-scaled MMA). a_s (M, K/128), b_s (ceil(N/128), K/128) fp32 powers of two. Returns bf16."""
    if not a_q.is_cuda:
        return fp8_gemm_ref(a_q, a_s, b_q, b_s).to(torch.bfloat16)
    M, N = a_q.shape[0], b_q.shape[0]
    sfa = pack_scales_ue8m0(a_s, M, True)
    sfb = pack_scales_ue8m0(b_s, N, False)
    out = torch.empty(M, N, device=a_q.device, dtype=torch.bfloat16)
    _ext.ops().gemm_mxfp8(a_q, sfa, b_q, sfb, out)
    return out


def fp8_quant_mx(x: torch.Tensor, transpose: bool = False, block: bool = False):
    """One-pass quantisation for the hardware-scaled GEMM. x (R, C) bf16, R and C multiples of 128. Returns
    ``(q, sf_packed, scales)``: q is x (or x^T when ``transpose``) in e4m3 with power-of-two scales per 1x128
    block of an output row (``block=False``) or per 128x128 tile; ``sf_packed`` the exponent bytes in the
    operand layout of :func:`mxfp8_gemm_packed`; ``scales`` the same scales in fp32."""
    R, C = x.shape
    rows, kc = (C, R) if transpose else (R, C)
    if not (x.is_cuda and x.dtype == torch.bfloat16):
        xt = (x.t() if transpose else x).contiguous()
        q, sc = (fp8_quant_128x128_ref if block else fp8_quant_1x128_ref)(xt, True)
        return q, pack_scales_ue8m0(sc, rows, not block), sc
    q = torch.empty(rows, kc, device=x.device, dtype=torch.float8_e4m3fn)
    sf = torch.empty(rows // 128, kc // 128, 512, device=x.device, dtype=torch.uint8)
    sc = torch.empty(rows // 128 if block else rows, kc // 128, device=x.device, dtype=torch.float32)
    _ext.ops().fp8_quant_mx(x.contiguous(), q, sc, sf, transpose, block)
    return q, sf, sc


def mxfp8_gemm_packed(a_q, sfa, b_q, sfb):
    """a_q [M,K] @ b_q [N,K]^T in e4m3 with packed exponent-byte scales (see :func:`fp8_quant_mx`) -> bf16 [M,N]."""
    out = torch.empty(a_q.shape[0], b_q.shape[0], device=a_q.device, dtype=torch.bfloat16)
    _ext.ops().gemm_mxfp8(a_q, sfa, b_q, sfb, out)
    return out


class Fp8Linear:
    """y = x @ W with W (in, out) held as block-scaled FP8: the weight is quantised once
    (transposed to [out, in] so K is contiguous), activations are quantised per call."""

    def __init__(self, w: torch.Tensor, pow2: bool = False):
        self.in_features, self.out_features = w.shape
        self.w_q, self.w_s = fp8_quant_128x128(w.t().contiguous().to(torch.bfloat16), pow2)
        self.pow2 = pow2

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        shp = x.shape
        x2 = x.reshape(-1, shp[-1]).to(torch.bfloat16).contiguous()
        xq, xs = fp8_quant_1x128(x2, self.pow2)
        return fp8_gemm(xq, xs, self.w_q, self.w_s).reshape(*shp[:-1], self.out_features)


_TRAINING_NAMES = ("fp8_eligible", "fp8_enabled", "fp8_linear", "fp8_training")


def __getattr__(name):
    """The training path lives in ops/fp8_linear.py, which imports this module: its names are resolved on first use
    instead of at import time, so that either module may be imported first."""
    if name in _TRAINING_NAMES:
        from . import fp8_linear
        return getattr(fp8_linear, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
