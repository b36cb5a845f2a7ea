"""Gated DeltaNet (jax_gpt/models/qwen35/deltanet.py:26-443).

Per head the layer maintains a state S (dk x dv) with the gated delta rule

    S <- exp(g) S;   S <- S + k (beta (v - S^T k))^T;   o = S^T q

where beta = sigmoid(b), g = -exp(A_log) softplus(a + dt_bias), q and k are L2-normalised
(q scaled by dk^-1/2) after a causal depthwise conv (width 4) + SiLU over the concatenated
q|k|v channels, and the output passes a gated RMSNorm ``w * rmsnorm(o) * silu(z)``.

``deltanet_prefill`` evaluates the same recurrence chunk-parallel: inside a chunk the
dependence of the corrected values on earlier tokens is a unit lower-triangular system, solved
here with one triangular solve per chunk (the reference unrolls a forward substitution,
jax_gpt/models/qwen35/deltanet.py:325-329); between chunks only S is carried, in fp32
(the reference carries it in the activation dtype, jax_gpt/models/qwen35/deltanet.py:344-345).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .fp8 import matmul_maybe_fp8


def _l2_norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def _gated_rms_norm(x: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf, zf = x.float(), z.float()
    y = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps)
    return (weight.float() * y * F.silu(zf)).to(x.dtype)


def causal_conv1d_update(x_new: torch.Tensor, conv_state: torch.Tensor, weight: torch.Tensor):
    """x_new (B, C), conv_state (B, C, K) of raw inputs, newest last. Returns (silu(conv), new_state)."""
    state = torch.cat([conv_state[:, :, 1:], x_new[:, :, None].to(conv_state.dtype)], dim=-1)
    y = (state.float() * weight.float()[None]).sum(-1)
    return F.silu(y).to(x_new.dtype), state


class _ConvSiluFn(torch.autograd.Function):
    """Depthwise causal FIR (width 4) + SiLU on the CUDA kernels, forward and backward; also returns the final
    conv state (the last K raw inputs), which carries no gradient."""

    @staticmethod
    def forward(ctx, x, weight):
        from ... import _ext
        B, T, C = x.shape
        xc = x.contiguous()
        wb = weight.to(torch.bfloat16).contiguous()
        y = torch.empty_like(xc)
        state = torch.empty(B, C, weight.shape[-1], device=x.device, dtype=torch.float32)
        _ext.ops().gdn_conv_silu(xc, wb, y, state)
        ctx.save_for_backward(xc, wb)
        ctx.w_dtype = weight.dtype
        state = state.to(x.dtype)
        ctx.mark_non_differentiable(state)
        return y, state

    @staticmethod
    def backward(ctx, dy, _dstate):
        from ... import _ext
        xc, wb = ctx.saved_tensors
        dx = torch.empty_like(xc)
        dw = torch.zeros(wb.shape, device=xc.device, dtype=torch.float32)
        _ext.ops().gdn_conv_silu_bwd(xc, wb, dy.to(torch.bfloat16).contiguous(), dx, dw)
        return dx, dw.to(ctx.w_dtype)


def causal_conv1d_prefill(x: torch.Tensor, weight: torch.Tensor):
    """x (B, T, C); depthwise causal FIR of width K then SiLU. Final state = last K raw inputs."""
    B, T, C = x.shape
    K = weight.shape[-1]
    if x.is_cuda and x.dtype == torch.bfloat16 and K == 4 and C % 8 == 0:
        return _ConvSiluFn.apply(x, weight)
    xc = F.pad(x.transpose(1, 2).float(), (K - 1, 0))
    y = F.conv1d(xc, weight.float()[:, None, :], groups=C)
    state = xc[:, :, -K:] if T >= 1 else xc
    return F.silu(y).transpose(1, 2).to(x.dtype), state.to(x.dtype)


def _project(x, params, n_qk, n_v, dk, dv):
    if "in_proj_all" in params:
        # the four projections as ONE GEMM over the concatenated weights (decode engine): column slices of its output
        y = matmul_maybe_fp8(x, params["in_proj_all"])
        c, vd = 2 * n_qk * dk + n_v * dv, n_v * dv
        return y[..., :c], y[..., c:c + vd], y[..., c + vd:c + vd + n_v], y[..., c + vd + n_v:c + vd + 2 * n_v]
    mixed = matmul_maybe_fp8(x, params["in_proj_qkv"])
    z = matmul_maybe_fp8(x, params["in_proj_z"])
    b = matmul_maybe_fp8(x, params["in_proj_b"])
    a = matmul_maybe_fp8(x, params["in_proj_a"])
    return mixed, z, b, a


def _gates(b, a, params):
    beta = torch.sigmoid(b.float())
    g = -torch.exp(params["A_log"].float()) * F.softplus(a.float() + params["dt_bias"].float())
    return beta, g


def gated_delta_step(q, k, v, beta, g, state):
    """One token. q,k (B,H,dk) already normalised; v (B,H,dv); beta,g (B,H); state (B,H,dk,dv) fp32."""
    state = state * torch.exp(g)[..., None, None]
    kv = torch.einsum("bhkv,bhk->bhv", state, k)
    delta = (v - kv) * beta[..., None]
    state = state + torch.einsum("bhk,bhv->bhkv", k, delta)
    return torch.einsum("bhkv,bhk->bhv", state, q), state


def deltanet_recurrent_step(x, params, state, conv_state, n_qk: int, n_v: int, dk: int, dv: int):
    """Decode: x (B,1,D) -> (out (B,1,D), new_state (B,Hv,dk,dv), new_conv_state (B,conv_dim,K))."""
    B = x.shape[0]
    key_dim, rep = n_qk * dk, n_v // n_qk
    mixed, z, b, a = _project(x, params, n_qk, n_v, dk, dv)
    if (x.is_cuda and x.dtype == torch.bfloat16 and state.dtype == torch.float32 and conv_state.dtype == torch.float32
            and max(dk, dv) <= 256 and not isinstance(params["out_proj"], dict)):
        # fused CUDA step: conv window update, gates, delta rule, gated RMSNorm; states updated in place
        from ... import _ext
        out = torch.empty(B, n_v * dv, device=x.device, dtype=torch.bfloat16)
        state_c, conv_c = state.contiguous(), conv_state.contiguous()
        bf = lambda t: t.to(torch.bfloat16).contiguous()
        # the kernel takes row strides: column slices of a merged projection output are read in place
        _ext.ops().gdn_decode_step(mixed[:, 0], z[:, 0], b[:, 0], a[:, 0], conv_c, bf(params["conv_weight"]), bf(params["A_log"]),
                                   bf(params["dt_bias"]), bf(params["norm_weight"]), state_c, out, n_qk, n_v, dk, dv, 1e-6)
        y = matmul_maybe_fp8(out, params["out_proj"])
        return y[:, None, :], state_c, conv_c
    mixed, new_conv = causal_conv1d_update(mixed[:, 0], conv_state, params["conv_weight"])
    q = mixed[:, :key_dim].reshape(B, n_qk, dk).float()
    k = mixed[:, key_dim:2 * key_dim].reshape(B, n_qk, dk).float()
    v = mixed[:, 2 * key_dim:].reshape(B, n_v, dv).float()
    beta, g = _gates(b[:, 0], a[:, 0], params)
    q = (_l2_norm(q) * dk ** -0.5).repeat_interleave(rep, dim=1)
    k = _l2_norm(k).repeat_interleave(rep, dim=1)
    o, new_state = gated_delta_step(q, k, v, beta, g, state.float())
    o = _gated_rms_norm(o.reshape(B * n_v, dv), z[:, 0].reshape(B * n_v, dv), params["norm_weight"])
    y = matmul_maybe_fp8(o.reshape(B, n_v * dv).to(x.dtype), params["out_proj"])
    return y[:, None, :], new_state.to(state.dtype), new_conv


class _GdnScanFn(torch.autograd.Function):
    """Inter-chunk scan of the gated delta rule on the tcgen05 kernels. Inputs per (batch*head, chunk):
    kq (128, dk) = [k_cum ; q exp(G)], intra (64, 64), kdec (64, dk), veff (64, dv) in bf16, e fp32, optional
    initial state. Returns (o (BH, N, 64, dv) bf16, final state fp32)."""

    @staticmethod
    def forward(ctx, kq, intra, kdec, veff, e, s0):
        from ... import _ext
        kq, intra, kdec, veff, e = [t.contiguous() for t in (kq, intra, kdec, veff, e)]
        BH, N = kq.shape[0], kq.shape[1]
        dev = kq.device
        o = torch.empty(BH, N, 64, 128, device=dev, dtype=torch.bfloat16)
        s_out = torch.empty(BH, 128, 128, device=dev, dtype=torch.float32)
        needs = any(ctx.needs_input_grad)
        s_save = torch.empty(BH, N, 128, 128, device=dev, dtype=torch.bfloat16) if needs else None
        vn_save = torch.empty(BH, N, 64, 128, device=dev, dtype=torch.bfloat16) if needs else None
        s0c = s0.contiguous() if s0 is not None else None
        _ext.ops().gdn_scan(kq, intra, kdec, veff, e, s0c, o, s_out, s_save, vn_save)
        if needs:
            ctx.save_for_backward(kq, intra, kdec, e, s_save, vn_save)
            ctx.has_s0 = s0 is not None
        return o, s_out

    @staticmethod
    def backward(ctx, d_o, d_s_out):
        from ... import _ext
        kq, intra, kdec, e, s_save, vn_save = ctx.saved_tensors
        BH, N = kq.shape[0], kq.shape[1]
        dev = kq.device
        bf = torch.bfloat16
        d_kq = torch.empty_like(kq)
        d_intra = torch.empty_like(intra)
        d_kdec = torch.empty_like(kdec)
        d_veff = torch.empty(BH, N, 64, 128, device=dev, dtype=bf)
        d_e = torch.zeros(BH, N, device=dev, dtype=torch.float32)
        ds0 = torch.empty(BH, 128, 128, device=dev, dtype=torch.float32)
        dsf = d_s_out.float().contiguous() if d_s_out is not None else None
        _ext.ops().gdn_scan_bwd(kq, intra, kdec, s_save, vn_save, e, d_o.to(bf).contiguous(), dsf, d_kq, d_intra, d_kdec,
                                d_veff, d_e, ds0)
        return d_kq, d_intra, d_kdec, d_veff, d_e, (ds0 if ctx.has_s0 else None)


class _GdnChunkPrepFn(torch.autograd.Function):
    """Everything of the chunked rule that does not depend on the running state, as one CUDA kernel forward and one
    backward (csrc/gdn_chunk_kernels.cu): gates, L2 norms of q and k, in-chunk decays, the two 64 x 64 Gram
    matrices, and the unit-lower-triangular solve. Inputs: ``mixed`` (B, T, 2 Kd + Vd) bf16 after conv + SiLU, the
    gate pre-activations ``b``, ``a`` (B, T, Hv) bf16, ``A_log``, ``dt_bias`` (Hv,). Outputs: the operands of
    ``_GdnScanFn`` for chunks of 64 (head widths 128). The backward recomputes the forward from the inputs, so
    nothing but the inputs is kept alive."""

    @staticmethod
    def forward(ctx, mixed, b, a, A_log, dt_bias, n_qk, n_v):
        from ... import _ext
        B, T, _ = mixed.shape
        N = (T + 63) // 64
        dev, bf = mixed.device, torch.bfloat16
        mixed, b, a = mixed.contiguous(), b.to(bf).contiguous(), a.to(bf).contiguous()
        al, dt = A_log.float().contiguous(), dt_bias.float().contiguous()
        BH = B * n_v
        kq = torch.empty(BH, N, 128, 128, device=dev, dtype=bf)
        intra = torch.empty(BH, N, 64, 64, device=dev, dtype=bf)
        kdec = torch.empty(BH, N, 64, 128, device=dev, dtype=bf)
        veff = torch.empty(BH, N, 64, 128, device=dev, dtype=bf)
        e = torch.empty(BH, N, device=dev, dtype=torch.float32)
        _ext.ops().gdn_chunk_prep(mixed, b, a, al, dt, kq, intra, kdec, veff, e, n_qk, n_v)
        ctx.save_for_backward(mixed, b, a, al, dt)
        ctx.heads = (n_qk, n_v)
        ctx.param_dtypes = (A_log.dtype, dt_bias.dtype)
        return kq, intra, kdec, veff, e

    @staticmethod
    def backward(ctx, d_kq, d_intra, d_kdec, d_veff, d_e):
        from ... import _ext
        mixed, b, a, al, dt = ctx.saved_tensors
        n_qk, n_v = ctx.heads
        bf = torch.bfloat16
        d_mixed = torch.empty_like(mixed)
        d_b = torch.empty(b.shape, device=b.device, dtype=torch.float32)
        d_a = torch.empty_like(d_b)
        d_al, d_dt = torch.zeros_like(al), torch.zeros_like(dt)
        _ext.ops().gdn_chunk_prep_bwd(mixed, b, a, al, dt, d_kq.to(bf).contiguous(), d_intra.to(bf).contiguous(),
                                      d_kdec.to(bf).contiguous(), d_veff.to(bf).contiguous(), d_e.float().contiguous(),
                                      d_mixed, d_b, d_a, d_al, d_dt, n_qk, n_v)
        return (d_mixed, d_b.to(b.dtype), d_a.to(a.dtype), d_al.to(ctx.param_dtypes[0]), d_dt.to(ctx.param_dtypes[1]),
                None, None)


class _GdnGatedNormFn(torch.autograd.Function):
    """``w * rmsnorm(o) * silu(z)`` on the scan kernel's head-major output ``o`` (B*Hv, N, 64, 128), written
    token-major as (B, T, Hv * 128): the transpose, the norm and the gate in one kernel, forward and backward."""

    @staticmethod
    def forward(ctx, o, z, weight, n_v, eps):
        from ... import _ext
        zc = z.contiguous()
        w = weight.float().contiguous()
        y = torch.empty_like(zc)
        _ext.ops().gdn_gated_norm(o, zc, w, y, n_v, eps)
        ctx.save_for_backward(o, zc, w)
        ctx.meta = (n_v, eps, weight.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        from ... import _ext
        o, z, w = ctx.saved_tensors
        n_v, eps, w_dtype = ctx.meta
        T, Tpad = z.shape[1], o.shape[1] * o.shape[2]
        d_o = torch.empty_like(o) if Tpad == T else torch.zeros_like(o)
        dz = torch.empty_like(z)
        dw = torch.zeros(128, device=o.device, dtype=torch.float32)
        _ext.ops().gdn_gated_norm_bwd(o, z, w, dy.to(torch.bfloat16).contiguous(), d_o, dz, dw, n_v, eps)
        return d_o, dz, dw.to(w_dtype), None, None


def gated_delta_prefill_cuda(mixed, b, a, A_log, dt_bias, n_qk: int, n_v: int, initial_state=None, head_major=False):
    """The whole gated-delta-rule prefill on this package's kernels (no library call): ``mixed`` (B, T, conv_dim)
    bf16 after conv + SiLU and the gate pre-activations -> (o (B, T, Hv, 128) bf16, final state (B, Hv, 128, 128)
    fp32). Chunks of 64 whatever the configured chunk size (the result does not depend on it). ``head_major``
    returns o as the scan kernel wrote it, (B*Hv, N, 64, 128) with zero-padded tail, for the fused gated norm."""
    B, T, _ = mixed.shape
    kq, intra, kdec, veff, e = _GdnChunkPrepFn.apply(mixed, b, a, A_log, dt_bias, n_qk, n_v)
    s0 = initial_state.float().reshape(B * n_v, 128, 128) if initial_state is not None else None
    o, s_out = _GdnScanFn.apply(kq, intra, kdec, veff, e, s0)
    if not head_major:
        o = o.reshape(B, n_v, -1, 128)[:, :, :T].transpose(1, 2)
    return o, s_out.reshape(B, n_v, 128, 128)


def chunk_gated_delta_rule(q, k, v, beta, g, chunk_size: int, initial_state=None):
    """Chunk-parallel gated delta rule in fp32.
    q,k (B,H,T,dk) normalised; v (B,H,T,dv); beta,g (B,H,T). Returns (o (B,H,T,dv), final state)."""
    B, H, T, dk = q.shape
    dv = v.shape[-1]
    C = chunk_size
    pad = (-T) % C
    if pad:
        q, k, v = [F.pad(t, (0, 0, 0, pad)) for t in (q, k, v)]
        beta, g = F.pad(beta, (0, pad)), F.pad(g, (0, pad))
    N = (T + pad) // C
    q, k, v = [t.reshape(B, H, N, C, -1) for t in (q, k, v)]
    beta, g = beta.reshape(B, H, N, C), g.reshape(B, H, N, C)
    G = g.cumsum(-1)                                              # cumulative log-decay inside the chunk
    decay = torch.exp((G[..., :, None] - G[..., None, :]).tril())  # exp(G_i - G_j), j <= i
    strict = torch.ones(C, C, device=q.device, dtype=torch.bool).tril(-1)
    causal = torch.ones(C, C, device=q.device, dtype=torch.bool).tril(0)
    kb = k * beta[..., None]
    A = (kb @ k.transpose(-1, -2)) * decay
    A = A.masked_fill(~strict, 0.0)
    eye = torch.eye(C, device=q.device, dtype=q.dtype)
    # (I + A) X = rhs  for the corrected values and the decayed keys
    rhs = torch.cat([v * beta[..., None], kb * torch.exp(G)[..., None]], dim=-1)
    sol = torch.linalg.solve_triangular(eye + A, rhs, upper=False, unitriangular=True)
    v_eff, k_cum = sol[..., :dv], sol[..., dv:]
    if q.is_cuda and dk == 128 and dv == 128 and C == 64:
        # the sequential part runs as ONE kernel per (batch, head) with the state on chip, forward and
        # backward (csrc/gdn_kernels.cu); the batched algebra around it stays differentiable PyTorch
        bf = torch.bfloat16
        g_end = G[..., -1]
        kq = torch.cat([k_cum, q * torch.exp(G)[..., None]], dim=-2).to(bf).reshape(B * H, N, 2 * C, dk)
        intra = ((q @ k.transpose(-1, -2)) * decay).masked_fill(~causal, 0.0).to(bf).reshape(B * H, N, C, C)
        kdec = (k * torch.exp(g_end[..., None] - G)[..., None]).to(bf).reshape(B * H, N, C, dk)
        veff = v_eff.to(bf).reshape(B * H, N, C, dv)
        e = torch.exp(g_end).float().reshape(B * H, N)
        s0 = initial_state.float().reshape(B * H, dk, dv) if initial_state is not None else None
        o, s_out = _GdnScanFn.apply(kq, intra, kdec, veff, e, s0)
        return o.reshape(B, H, N * C, dv)[:, :, :T].float(), s_out.reshape(B, H, dk, dv)
    S = initial_state.float() if initial_state is not None else q.new_zeros(B, H, dk, dv)
    outs = []
    for n in range(N):
        qn, kn = q[:, :, n], k[:, :, n]
        Gn = G[:, :, n]
        intra = (qn @ kn.transpose(-1, -2)) * decay[:, :, n]
        intra = intra.masked_fill(~causal, 0.0)
        v_new = v_eff[:, :, n] - k_cum[:, :, n] @ S
        o = (qn * torch.exp(Gn)[..., None]) @ S + intra @ v_new
        outs.append(o)
        g_end = Gn[..., -1]
        S = S * torch.exp(g_end)[..., None, None] + (kn * torch.exp(g_end[..., None] - Gn)[..., None]).transpose(-1, -2) @ v_new
    o = torch.stack(outs, dim=2).reshape(B, H, N * C, dv)[:, :, :T]
    return o, S


def deltanet_prefill(x, params, n_qk: int, n_v: int, dk: int, dv: int, conv_kernel: int, chunk_size: int = 256,
                     initial_state=None):
    """Prefill: x (B,T,D) -> (out (B,T,D), final_state (B,Hv,dk,dv) fp32, final_conv_state (B,conv_dim,K))."""
    B, T, _ = x.shape
    key_dim, rep = n_qk * dk, n_v // n_qk
    mixed, z, b, a = _project(x, params, n_qk, n_v, dk, dv)
    mixed, conv_state = causal_conv1d_prefill(mixed, params["conv_weight"])
    if mixed.is_cuda and mixed.dtype == torch.bfloat16 and dk == 128 and dv == 128 and n_v % n_qk == 0:
        o, S = gated_delta_prefill_cuda(mixed, b, a, params["A_log"], params["dt_bias"], n_qk, n_v, initial_state,
                                        head_major=True)
        o = _GdnGatedNormFn.apply(o, z, params["norm_weight"], n_v, 1e-6)
        return matmul_maybe_fp8(o, params["out_proj"]), S, conv_state
    q = mixed[..., :key_dim].reshape(B, T, n_qk, dk).float()
    k = mixed[..., key_dim:2 * key_dim].reshape(B, T, n_qk, dk).float()
    v = mixed[..., 2 * key_dim:].reshape(B, T, n_v, dv).float()
    beta, g = _gates(b, a, params)                                   # (B,T,Hv)
    q = (_l2_norm(q) * dk ** -0.5).repeat_interleave(rep, dim=2)
    k = _l2_norm(k).repeat_interleave(rep, dim=2)
    o, S = chunk_gated_delta_rule(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), beta.transpose(1, 2),
                                  g.transpose(1, 2), chunk_size, initial_state)
    o = o.transpose(1, 2)                                            # (B,T,Hv,dv)
    o = _gated_rms_norm(o.reshape(B * T * n_v, dv), z.reshape(B * T * n_v, dv), params["norm_weight"])
    y = matmul_maybe_fp8(o.reshape(B, T, n_v * dv).to(x.dtype), params["out_proj"])
    return y, S, conv_state
