"""Router, RMSNorm+RoPE, FP8 quantisation and Gated-DeltaNet decode kernels vs PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("E,k", [(512, 10), (64, 2), (256, 8)])
def test_softmax_router(cuda_device, E, k):
    from jax_gpt_b200.ops import router as R
    torch.manual_seed(0)
    logits = torch.randn(777, E, device=cuda_device)
    counts = torch.zeros(E, device=cuda_device, dtype=torch.int32)
    w, ids = R.router_cuda(0, logits, None, k, counts=counts)
    probs = torch.softmax(logits, -1)
    rw, ri = probs.topk(k, -1)
    rw = rw / rw.sum(-1, keepdim=True)
    assert torch.equal(ids.long(), ri) and torch.allclose(w, rw, atol=1e-5)
    assert torch.equal(counts.long(), torch.bincount(ri.reshape(-1), minlength=E))


@pytest.mark.parametrize("E,k,G,kg", [(256, 8, 8, 4), (64, 6, 8, 3), (128, 4, 4, 2)])
def test_deepseek_router(cuda_device, E, k, G, kg):
    from jax_gpt_b200.ops import router as R
    torch.manual_seed(1)
    logits = torch.randn(500, E, device=cuda_device) * 2
    bias = torch.randn(E, device=cuda_device) * 0.1
    w, ids = R.router_cuda(1, logits, bias, k, G, kg, 2.5)
    rw, ri = R.deepseek_router_from_logits(logits.cpu(), bias.cpu(), k, G, kg, 2.5)
    # same expert set per token (order may differ) and the same weight per expert
    a = torch.zeros(500, E).scatter_(1, ids.long().cpu(), w.cpu())
    b = torch.zeros(500, E).scatter_(1, ri, rw)
    assert torch.allclose(a, b, atol=1e-5)


@pytest.mark.parametrize("dh,rope,norm", [(256, 64, True), (128, 32, True), (64, 64, False), (32, 8, True)])
def test_rmsnorm_rope(cuda_device, dh, rope, norm):
    from jax_gpt_b200.models.qwen35.primitives import precompute_rope_freqs
    from jax_gpt_b200.ops import rope as RP
    torch.manual_seed(2)
    B, T, H = 2, 37, 3
    x = torch.randn(B, T, H, dh, device=cuda_device).to(torch.bfloat16)
    w = (torch.randn(dh, device=cuda_device) * 0.2).to(torch.bfloat16) if norm else None
    fr = precompute_rope_freqs(rope, 64, 10000.0, device=cuda_device)
    y = RP.rmsnorm_rope(x, w, fr, rope, pos0=5)
    ref = RP.rmsnorm_rope_ref(x, w, fr, rope, pos0=5)
    assert _rel(y, ref) < 1e-2
    # backward kernel vs autograd of the fp32 restatement
    xg = x.clone().requires_grad_(True)
    wg = w.clone().requires_grad_(True) if norm else None
    dy = torch.randn_like(x)
    RP.rmsnorm_rope(xg, wg, fr, rope, pos0=5).backward(dy)
    xr = x.float().requires_grad_(True)
    wr = w.float().requires_grad_(True) if norm else None
    RP.rmsnorm_rope_ref(xr, wr, fr, rope, pos0=5).backward(dy.float())
    assert _rel(xg.grad, xr.grad) < 1.5e-2
    if norm:
        assert _rel(wg.grad, wr.grad) < 1.5e-2


@pytest.mark.parametrize("pow2", [False, True])
def test_fp8_block_quant(cuda_device, pow2):
    from jax_gpt_b200.ops import fp8 as RP
    torch.manual_seed(3)
    x = (torch.randn(300, 512, device=cuda_device) * torch.rand(300, 1, device=cuda_device) * 5).to(torch.bfloat16)
    q, sc = RP.fp8_quant_1x128(x, pow2)
    rq, rsc = RP.fp8_quant_1x128_ref(x, pow2)
    assert torch.allclose(sc, rsc, rtol=1e-6)
    deq = q.float().view(300, 4, 128) * sc[..., None]
    assert ((deq.view(300, 512) - x.float()).abs().max() / x.float().abs().max()) < 0.07
    assert (q.float() - rq.float()).abs().max() <= 32  # at most one e4m3 step apart near the top of the range
    w = torch.randn(256, 384, device=cuda_device).to(torch.bfloat16)
    qw, sw = RP.fp8_quant_128x128(w, pow2)
    _, rsw = RP.fp8_quant_128x128_ref(w, pow2)
    assert torch.allclose(sw, rsw, rtol=1e-6)
    deq = (qw.float().view(2, 128, 3, 128) * sw[:, None, :, None]).view(256, 384)
    assert _rel(deq, w) < 0.05
    if pow2:
        assert torch.equal(torch.exp2(torch.round(torch.log2(sw))), sw)


def test_gdn_decode_step(cuda_device):
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.models.qwen35 import deltanet as DN
    torch.manual_seed(4)
    B, Hqk, Hv, dk, dv, Kc = 3, 2, 4, 128, 128, 4
    Kd, Vd = Hqk * dk, Hv * dv
    C = 2 * Kd + Vd
    bf = lambda *s: (torch.randn(*s, device=cuda_device)).to(torch.bfloat16)
    mixed, z, bp, ap = bf(B, C), bf(B, Vd), bf(B, Hv), bf(B, Hv)
    conv_w = (torch.randn(C, Kc, device=cuda_device) * 0.5).to(torch.bfloat16)
    A_log = torch.log(torch.rand(Hv, device=cuda_device) * 4 + 0.1).to(torch.bfloat16)
    dt_bias = torch.ones(Hv, device=cuda_device, dtype=torch.bfloat16)
    norm_w = (torch.randn(dv, device=cuda_device) * 0.3 + 1).to(torch.bfloat16)
    conv_state = torch.randn(B, C, Kc, device=cuda_device)
    state = torch.randn(B, Hv, dk, dv, device=cuda_device) * 0.1
    # reference (fp32 torch)
    cs_ref, st_ref = conv_state.clone(), state.clone()
    mx, cs_ref = DN.causal_conv1d_update(mixed.float(), cs_ref, conv_w.float())
    q = DN._l2_norm(mx[:, :Kd].reshape(B, Hqk, dk)) * dk ** -0.5
    k = DN._l2_norm(mx[:, Kd:2 * Kd].reshape(B, Hqk, dk))
    v = mx[:, 2 * Kd:].reshape(B, Hv, dv)
    beta, g = DN._gates(bp.float(), ap.float(), {"A_log": A_log.float(), "dt_bias": dt_bias.float()})
    o, st_ref = DN.gated_delta_step(q.repeat_interleave(Hv // Hqk, 1), k.repeat_interleave(Hv // Hqk, 1), v, beta, g, st_ref)
    o = DN._gated_rms_norm(o.reshape(B * Hv, dv), z.float().reshape(B * Hv, dv), norm_w.float()).reshape(B, Vd)
    out = torch.empty(B, Vd, device=cuda_device, dtype=torch.bfloat16)
    _ext.ops().gdn_decode_step(mixed, z, bp, ap, conv_state, conv_w, A_log, dt_bias, norm_w, state, out, Hqk, Hv, dk, dv, 1e-6)
    assert _rel(out, o) < 1e-2
    assert _rel(state, st_ref) < 1e-4 and _rel(conv_state, cs_ref) < 1e-6


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 256, 512), (1024, 2048, 7168), (4096, 4096, 2048)])
def test_fp8_blockscaled_gemm(cuda_device, M, N, K):
    from jax_gpt_b200.ops import fp8 as RP
    torch.manual_seed(5)
    x = (torch.randn(M, K, device=cuda_device) * (torch.rand(M, 1, device=cuda_device) * 3 + 0.1)).to(torch.bfloat16)
    w = (torch.randn(N, K, device=cuda_device) * 0.05).to(torch.bfloat16)
    xq, xs = RP.fp8_quant_1x128(x)
    wq, ws = RP.fp8_quant_128x128(w) if N % 128 == 0 else RP.fp8_quant_128x128_ref(torch.nn.functional.pad(w, (0, 0, 0, (-N) % 128)))
    if N % 128:
        wq = wq[:N].contiguous()
    out = RP.fp8_gemm(xq, xs, wq, ws)
    ref = RP.fp8_gemm_ref(xq, xs, wq, ws)
    assert _rel(out, ref) < 1e-2                      # kernel vs exact arithmetic on the same quantised operands
    assert _rel(out, x.float() @ w.float().t()) < 6e-2   # and the quantisation error itself stays small
    lin = RP.Fp8Linear(w.t().contiguous())
    assert _rel(lin(x), x.float() @ w.float().t()) < 6e-2


@pytest.mark.parametrize("heads,n_splits", [(16, 1), (16, 0), (128, 3), (40, 0)])
def test_mla_paged_decode_and_paged_write(cuda_device, heads, n_splits):
    """Ragged batch over the paged latent cache: the tcgen05 decode kernel vs fp32 math on the gathered
    pages; the rows get into their pages through the paged write kernel."""
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.cache.paged import PagedCache
    from jax_gpt_b200.ops.mla_decode import mla_paged_decode, mla_paged_decode_ref
    lens = [1, 63, 64, 65, 128, 200, 1000, 2309]
    B = len(lens)
    g = torch.Generator(device=cuda_device).manual_seed(5)
    cache = PagedCache(2, 576, n_pages=80, page_size=64, max_seqs=16, max_pages_per_seq=40, device=cuda_device)
    ids = [3, 0, 7, 1, 12, 5, 9, 2]
    # interleave the appends so that the page lists are not contiguous
    for chunk in range(3):
        for b, sid in enumerate(ids):
            n = lens[b] // 3 if chunk < 2 else lens[b] - 2 * (lens[b] // 3)
            if n:
                rows = torch.randn(1, n, 576, device=cuda_device, generator=g).to(torch.bfloat16)
                cache.append(1, [sid], rows, commit=True)
    assert [cache.length(s) for s in ids] == lens
    q = (torch.randn(B, heads, 576, device=cuda_device, generator=g) * 0.3).to(torch.bfloat16)
    scale = 192 ** -0.5
    out = mla_paged_decode(q, cache, 1, ids, scale, n_splits=n_splits)
    torch.cuda.synchronize()
    _ext.check_status(cuda_device)
    ref = mla_paged_decode_ref(q, cache, 1, ids, scale, 512)
    err = (out.float() - ref.float()).abs().max().item()
    assert err < 3e-2, err
    rel = ((out.float() - ref.float()).norm() / ref.float().norm()).item()
    assert rel < 1.5e-2, rel


@pytest.mark.parametrize("M,N,K", [(300, 512, 1024), (256, 384, 512), (1024, 2048, 7168)])
def test_mxfp8_gemm_hardware_block_scales(cuda_device, M, N, K):
    """tcgen05 block-scaled MMA (UE8M0 scales in TMEM) vs the de-quantised fp32 product."""
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.ops import fp8 as Q
    torch.manual_seed(3)
    x = (torch.randn(M, K, device=cuda_device) * torch.rand(M, 1, device=cuda_device) * 4).to(torch.bfloat16)
    w = (torch.randn(N, K, device=cuda_device) * 0.05).to(torch.bfloat16)
    wp = torch.zeros((N + 127) // 128 * 128, K, device=cuda_device, dtype=torch.bfloat16)
    wp[:N] = w
    xq, xs = Q.fp8_quant_1x128(x, pow2=True)
    wq, ws = Q.fp8_quant_128x128(wp, pow2=True)
    out = Q.mxfp8_gemm(xq, xs, wq[:N].contiguous(), ws)
    torch.cuda.synchronize()
    _ext.check_status(cuda_device)
    ref = Q.fp8_gemm_ref(xq, xs, wq[:N], ws)
    assert _rel(out, ref) < 5e-3, _rel(out, ref)
    assert _rel(out, x.float() @ w.float().t()) < 6e-2


def test_gdn_conv_silu_kernel(cuda_device):
    from jax_gpt_b200.models.qwen35 import deltanet as D
    torch.manual_seed(0)
    B, T, C = 2, 70, 1024
    x = torch.randn(B, T, C, device=cuda_device).to(torch.bfloat16)
    w = (torch.randn(C, 4, device=cuda_device) * 0.5).to(torch.bfloat16)
    with torch.no_grad():
        y, st = D.causal_conv1d_prefill(x, w)
        y_ref, st_ref = D.causal_conv1d_prefill(x.float().cpu(), w.float().cpu())
    assert _rel(y.cpu(), y_ref) < 1e-2
    assert torch.equal(st.float().cpu(), st_ref)
    with torch.no_grad():
        _, st1 = D.causal_conv1d_prefill(x[:, :2].contiguous(), w)      # shorter than the window: zero padded
    assert torch.equal(st1.float().cpu(), D.causal_conv1d_prefill(x[:, :2].float().cpu(), w.float().cpu())[1])


@pytest.mark.parametrize("B,T,C", [(2, 70, 1024), (1, 33, 256), (1, 257, 2048)])
def test_gdn_conv_silu_backward_kernel(cuda_device, B, T, C):
    """dx and dw of the depthwise causal FIR + SiLU kernel against autograd of the fp32 library path (strips of 32
    steps: T = 70 / 33 / 257 cover a ragged last strip and taps that cross strip boundaries)."""
    from jax_gpt_b200.models.qwen35 import deltanet as D
    torch.manual_seed(4)
    x = torch.randn(B, T, C, device=cuda_device).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(C, 4, device=cuda_device) * 0.5).requires_grad_()          # fp32 master weight
    dy = torch.randn(B, T, C, device=cuda_device).to(torch.bfloat16)
    y, _ = D.causal_conv1d_prefill(x, w)
    y.backward(dy)
    xr = x.detach().float().cpu().requires_grad_()
    wr = w.detach().to(torch.bfloat16).float().cpu().requires_grad_()
    yr, _ = D.causal_conv1d_prefill(xr, wr)
    yr.backward(dy.float().cpu())
    assert w.grad.dtype == torch.float32
    assert _rel(x.grad.float().cpu(), xr.grad) < 1e-2
    assert _rel(w.grad.cpu(), wr.grad) < 1e-2


@pytest.mark.parametrize("T,with_state", [(64, False), (200, False), (1024, True)])
def test_gdn_chunk_scan_kernel(cuda_device, T, with_state):
    """Chunked gated delta rule with the tcgen05 inter-chunk scan vs the token-by-token recurrence in fp32."""
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.models.qwen35 import deltanet as D
    torch.manual_seed(1)
    B, H, dk, dv = 2, 3, 128, 128
    q = D._l2_norm(torch.randn(B, H, T, dk)) * dk ** -0.5
    k = D._l2_norm(torch.randn(B, H, T, dk))
    v = torch.randn(B, H, T, dv)
    beta = torch.sigmoid(torch.randn(B, H, T))
    g = -torch.rand(B, H, T) * 0.2
    s0 = torch.randn(B, H, dk, dv) * 0.1 if with_state else None
    S = s0.clone() if with_state else torch.zeros(B, H, dk, dv)
    outs = []
    for t in range(T):
        o, S = D.gated_delta_step(q[:, :, t], k[:, :, t], v[:, :, t], beta[:, :, t], g[:, :, t], S)
        outs.append(o)
    ref = torch.stack(outs, dim=2)
    dev = lambda t: None if t is None else t.to(cuda_device)
    with torch.no_grad():
        o_k, S_k = D.chunk_gated_delta_rule(dev(q), dev(k), dev(v), dev(beta), dev(g), 64, dev(s0))
    torch.cuda.synchronize()
    _ext.check_status(cuda_device)
    assert _rel(o_k.cpu(), ref) < 2e-2, _rel(o_k.cpu(), ref)
    assert _rel(S_k.cpu(), S) < 2e-2, _rel(S_k.cpu(), S)


@pytest.mark.parametrize("T,with_state", [(128, False), (300, True)])
def test_gdn_chunk_scan_backward_kernel(cuda_device, T, with_state):
    """Gradients through the tcgen05 forward + backward scan kernels vs autograd of the fp32 PyTorch chunk loop."""
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.models.qwen35 import deltanet as D
    torch.manual_seed(4)
    B, H, dk, dv = 1, 2, 128, 128
    q0 = D._l2_norm(torch.randn(B, H, T, dk)) * dk ** -0.5
    k0 = D._l2_norm(torch.randn(B, H, T, dk))
    v0 = torch.randn(B, H, T, dv)
    b0 = torch.sigmoid(torch.randn(B, H, T))
    g0 = -torch.rand(B, H, T) * 0.2
    s0 = torch.randn(B, H, dk, dv) * 0.1 if with_state else None
    wo, ws = torch.randn(B, H, T, dv), torch.randn(B, H, dk, dv) * 0.1

    def run(device):
        leaves = [t.clone().to(device).requires_grad_(True) for t in (q0, k0, v0, b0, g0)]
        st = s0.clone().to(device).requires_grad_(True) if with_state else None
        o, S = D.chunk_gated_delta_rule(*leaves, 64, st)
        ((o * wo.to(device)).sum() + (S * ws.to(device)).sum()).backward()
        grads = [t.grad.float().cpu() for t in leaves] + ([st.grad.float().cpu()] if with_state else [])
        return o.detach().float().cpu(), grads

    o_ref, g_ref = run("cpu")
    o_k, g_k = run(cuda_device)
    torch.cuda.synchronize()
    _ext.check_status(cuda_device)
    assert _rel(o_k, o_ref) < 2e-2
    names = ["q", "k", "v", "beta", "g"] + (["s0"] if with_state else [])
    for n, a, b in zip(names, g_k, g_ref):
        assert _rel(a, b) < 4e-2, (n, _rel(a, b))


def _gdn_inputs(B, T, n_qk, n_v, seed):
    g = torch.Generator().manual_seed(seed)
    conv_dim = (2 * n_qk + n_v) * 128
    mixed = torch.nn.functional.silu(torch.randn(B, T, conv_dim, generator=g)).to(torch.bfloat16)
    b = torch.randn(B, T, n_v, generator=g).to(torch.bfloat16)
    a = torch.randn(B, T, n_v, generator=g).to(torch.bfloat16)
    A_log = torch.log(torch.rand(n_v, generator=g) * 3.9 + 0.1)
    dt_bias = torch.ones(n_v) + 0.1 * torch.randn(n_v, generator=g)
    return mixed, b, a, A_log, dt_bias


def _gdn_reference(mixed, b, a, A_log, dt_bias, n_qk, n_v, s0=None):
    """fp32 PyTorch: split q | k | v, gates, L2 norms, chunked rule (triangular solve + chunk loop)."""
    from jax_gpt_b200.models.qwen35 import deltanet as D
    B, T, _ = mixed.shape
    Kd, rep = n_qk * 128, n_v // n_qk
    q = mixed[..., :Kd].reshape(B, T, n_qk, 128).float()
    k = mixed[..., Kd:2 * Kd].reshape(B, T, n_qk, 128).float()
    v = mixed[..., 2 * Kd:].reshape(B, T, n_v, 128).float()
    beta, g = D._gates(b, a, {"A_log": A_log, "dt_bias": dt_bias})
    q = (D._l2_norm(q) * 128 ** -0.5).repeat_interleave(rep, dim=2)
    k = D._l2_norm(k).repeat_interleave(rep, dim=2)
    o, S = D.chunk_gated_delta_rule(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), beta.transpose(1, 2),
                                    g.transpose(1, 2), 64, s0)
    return o.transpose(1, 2), S


@pytest.mark.parametrize("B,T,n_qk,n_v", [(2, 64, 1, 1), (1, 200, 2, 4), (2, 1024, 2, 2)])
def test_gdn_chunk_prep_kernel(cuda_device, B, T, n_qk, n_v):
    """The fused state-independent kernel (gates, L2 norms, decays, Gram matrices, triangular solve) against the
    same quantities computed in fp32 PyTorch with ``solve_triangular``."""
    from jax_gpt_b200.models.qwen35 import deltanet as D
    mixed, b, a, A_log, dt_bias = _gdn_inputs(B, T, n_qk, n_v, 7)
    dev = lambda t: t.to(cuda_device)
    with torch.no_grad():
        kq, intra, kdec, veff, e = D._GdnChunkPrepFn.apply(dev(mixed), dev(b), dev(a), dev(A_log), dev(dt_bias), n_qk, n_v)
    torch.cuda.synchronize()
    # reference, chunk by chunk on zero-padded inputs
    C, N, pad = 64, (T + 63) // 64, (-T) % 64
    Kd, rep = n_qk * 128, n_v // n_qk
    F = torch.nn.functional
    q = (D._l2_norm(mixed[..., :Kd].reshape(B, T, n_qk, 128).float()) * 128 ** -0.5).repeat_interleave(rep, 2)
    k = D._l2_norm(mixed[..., Kd:2 * Kd].reshape(B, T, n_qk, 128).float()).repeat_interleave(rep, 2)
    v = mixed[..., 2 * Kd:].reshape(B, T, n_v, 128).float()
    beta, g = D._gates(b, a, {"A_log": A_log, "dt_bias": dt_bias})
    q, k, v = [F.pad(t.transpose(1, 2), (0, 0, 0, pad)).reshape(B * n_v, N, C, 128) for t in (q, k, v)]
    beta, g = [F.pad(t.transpose(1, 2), (0, pad)).reshape(B * n_v, N, C) for t in (beta, g)]
    G = g.cumsum(-1)
    decay = torch.exp((G[..., :, None] - G[..., None, :]).tril())
    kb = k * beta[..., None]
    A = ((kb @ k.transpose(-1, -2)) * decay).tril(-1)
    rhs = torch.cat([v * beta[..., None], kb * torch.exp(G)[..., None]], dim=-1)
    sol = torch.linalg.solve_triangular(torch.eye(C) + A, rhs, upper=False, unitriangular=True)
    ref_kq = torch.cat([sol[..., 128:], q * torch.exp(G)[..., None]], dim=-2)
    ref_intra = ((q @ k.transpose(-1, -2)) * decay).tril()
    ref_kdec = k * torch.exp(G[..., -1:] - G)[..., None]
    for name, got, ref in (("kq", kq, ref_kq), ("intra", intra, ref_intra), ("kdec", kdec, ref_kdec),
                           ("veff", veff, sol[..., :128]), ("e", e, torch.exp(G[..., -1]))):
        assert _rel(got.float().cpu(), ref) < 8e-3, (name, _rel(got.float().cpu(), ref))


@pytest.mark.parametrize("B,T,n_qk,n_v,with_state", [(1, 128, 1, 1, False), (2, 200, 2, 4, True)])
def test_gated_delta_prefill_cuda_gradients(cuda_device, B, T, n_qk, n_v, with_state):
    """The whole prefill on the kernels (chunk preparation + inter-chunk scan, forward and backward) against
    autograd of the fp32 PyTorch path: outputs, final state, and the gradients of every input and gate parameter."""
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.models.qwen35 import deltanet as D
    ins = _gdn_inputs(B, T, n_qk, n_v, 9)
    torch.manual_seed(10)
    s0 = torch.randn(B, n_v, 128, 128) * 0.1 if with_state else None
    wo, ws = torch.randn(B, T, n_v, 128), torch.randn(B, n_v, 128, 128) * 0.1

    def run(device):
        leaves = [t.clone().float().to(device).requires_grad_(True) for t in ins]
        st = s0.clone().to(device).requires_grad_(True) if with_state else None
        mixed, b, a = [t.to(torch.bfloat16) for t in leaves[:3]]          # the cast carries the gradient back in fp32
        if device == "cpu":
            o, S = _gdn_reference(mixed, b, a, leaves[3], leaves[4], n_qk, n_v, st)
        else:
            o, S = D.gated_delta_prefill_cuda(mixed, b, a, leaves[3], leaves[4], n_qk, n_v, st)
        ((o.float() * wo.to(device)).sum() + (S * ws.to(device)).sum()).backward()
        grads = [t.grad.float().cpu() for t in leaves] + ([st.grad.float().cpu()] if with_state else [])
        return o.detach().float().cpu(), S.detach().float().cpu(), grads

    o_ref, S_ref, g_ref = run("cpu")
    o_k, S_k, g_k = run(cuda_device)
    torch.cuda.synchronize()
    _ext.check_status(cuda_device)
    assert _rel(o_k, o_ref) < 2e-2 and _rel(S_k, S_ref) < 2e-2, (_rel(o_k, o_ref), _rel(S_k, S_ref))
    names = ["mixed", "b", "a", "A_log", "dt_bias"] + (["s0"] if with_state else [])
    bad = [(n, _rel(x, y)) for n, x, y in zip(names, g_k, g_ref) if _rel(x, y) > 5e-2]
    assert not bad, bad


@pytest.mark.parametrize("B,T,Hv", [(2, 64, 2), (1, 200, 4)])
def test_gdn_gated_norm_kernel(cuda_device, B, T, Hv):
    """Fused transpose + RMSNorm + SiLU gate on the scan kernel's head-major layout (zero-padded to chunks of
    64), forward and backward, against the fp32 PyTorch expression on the token-major tensor."""
    from jax_gpt_b200.models.qwen35 import deltanet as D
    torch.manual_seed(12)
    N = (T + 63) // 64
    o_tm = torch.randn(B, T, Hv, 128)                                   # token-major values
    o_hm = torch.zeros(B, Hv, N * 64, 128)
    o_hm[:, :, :T] = o_tm.transpose(1, 2)
    z = torch.randn(B, T, Hv * 128)
    w = torch.rand(128) + 0.5
    dy = torch.randn(B, T, Hv * 128)
    bf = torch.bfloat16
    o_k = o_hm.to(bf).reshape(B * Hv, N, 64, 128).to(cuda_device).requires_grad_()
    z_k = z.to(bf).to(cuda_device).requires_grad_()
    w_k = w.to(cuda_device).requires_grad_()
    y = D._GdnGatedNormFn.apply(o_k, z_k, w_k, Hv, 1e-6)
    y.backward(dy.to(bf).to(cuda_device))
    o_r = o_tm.to(bf).float().requires_grad_()
    z_r = z.to(bf).float().requires_grad_()
    w_r = w.clone().requires_grad_()
    y_r = D._gated_rms_norm(o_r.reshape(-1, 128), z_r.reshape(-1, 128), w_r).reshape(B, T, Hv * 128)
    y_r.backward(dy.to(bf).float())
    assert _rel(y.float().cpu(), y_r) < 1e-2
    d_o = o_k.grad.float().cpu().reshape(B, Hv, N * 64, 128)
    assert d_o[:, :, T:].abs().max().item() == 0 if N * 64 > T else True
    assert _rel(d_o[:, :, :T].transpose(1, 2), o_r.grad) < 1e-2
    assert _rel(z_k.grad.float().cpu(), z_r.grad) < 1e-2
    assert _rel(w_k.grad.cpu(), w_r.grad) < 1e-2


def test_linear_with_fp32_output_and_gradient_buffer(cuda_device):
    """Router-style GEMM (bf16 operands, fp32 logits) and the weight gradient accumulated by the GEMM epilogue
    straight into an fp32 buffer attached to the weight (``grad_buf``), twice, as in gradient accumulation."""
    from jax_gpt_b200.ops.gemm import linear, linear_f32out
    torch.manual_seed(13)
    M, K, N = 4096, 512, 64
    x = torch.randn(M, K, device=cuda_device).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(K, N, device=cuda_device) * 0.05).to(torch.bfloat16).requires_grad_()
    y = linear_f32out(x, w)
    assert y.dtype == torch.float32
    ref = x.detach().float() @ w.detach().float()
    assert _rel(y, ref) < 1e-5
    dy = torch.randn(M, N, device=cuda_device)
    y.backward(dy)
    assert _rel(x.grad, dy @ w.detach().float().t()) < 1e-2
    assert _rel(w.grad, x.detach().float().t() @ dy) < 1e-2
    # with a gradient buffer: no autograd gradient, two backward passes add up in fp32
    w2 = w.detach().clone().requires_grad_()
    w2.grad_buf = torch.zeros(K, N, device=cuda_device)
    for fn in (linear, linear_f32out):
        out = fn(x.detach(), w2)
        out.backward(dy.to(out.dtype))
    assert w2.grad is None
    assert _rel(w2.grad_buf, 2 * (x.detach().float().t() @ dy)) < 1e-2


def test_fp8_linear_training_path_on_gpu(cuda_device):
    """Forward / dgrad / wgrad of a linear layer on the hardware block-scaled FP8 GEMM: against the same recipe
    evaluated by the CPU reference kernels (same quantisation, so only summation order and bf16 rounding differ)
    and against the bf16 layer (e4m3 rounding)."""
    from jax_gpt_b200.ops.fp8_linear import fp8_training
    from jax_gpt_b200.ops.gemm import linear
    torch.manual_seed(5)
    M, K, N = 512, 512, 768
    xc = torch.randn(M, K).to(torch.bfloat16)
    wc = (torch.randn(K, N) * 0.05).to(torch.bfloat16)
    dyc = torch.randn(M, N).to(torch.bfloat16)
    outs = {}
    for name, dev, fp8 in (("gpu_fp8", cuda_device, True), ("cpu_fp8", "cpu", True), ("gpu_bf16", cuda_device, False)):
        x = xc.detach().clone().to(dev).requires_grad_()
        w = wc.detach().clone().to(dev).requires_grad_()
        with fp8_training(fp8):
            y = linear(x, w)
        y.backward(dyc.to(dev))
        outs[name] = (y.detach().float().cpu(), x.grad.float().cpu(), w.grad.float().cpu())
    for i, what in enumerate(("y", "dx", "dw")):
        assert _rel(outs["gpu_fp8"][i], outs["cpu_fp8"][i]) < 2e-2, what
        assert _rel(outs["gpu_fp8"][i], outs["gpu_bf16"][i]) < 6e-2, what
    assert outs["gpu_fp8"][2].shape == (K, N)


@pytest.mark.parametrize("transpose", [False, True])
@pytest.mark.parametrize("block", [False, True])
def test_fp8_quant_mx_kernel_matches_reference(cuda_device, transpose, block):
    """One-pass quantise (+ transpose) + packed exponent bytes against the reference functions: same e4m3 bytes,
    same power-of-two scales, same packed layout."""
    from jax_gpt_b200.ops import fp8 as R
    torch.manual_seed(6)
    x = (torch.randn(384, 256) * torch.logspace(-2, 2, 256)[None, :]).to(torch.bfloat16)
    q, sf, sc = R.fp8_quant_mx(x.to(cuda_device), transpose, block)
    q_ref, sf_ref, sc_ref = R.fp8_quant_mx(x, transpose, block)
    assert q.shape == q_ref.shape == ((256, 384) if transpose else (384, 256))
    assert torch.equal(sc.cpu(), sc_ref)
    assert torch.equal(sf.cpu(), sf_ref)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))

