"""Numerics of the sm_100a kernels against plain PyTorch fp32 references of the same ops."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 256), (384, 768, 192), (200, 136, 72), (2048, 2304, 768)])
def test_gemm_layouts(cuda_device, M, N, K, a_mn, b_mn):
    from jax_gpt_b200.ops import gemm as G
    torch.manual_seed(0)
    if (a_mn and M % 8) or (b_mn and N % 8) or K % 8:
        pytest.skip("row strides must be multiples of 8 elements")
    a = torch.randn((K, M) if a_mn else (M, K), device=cuda_device).to(torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device=cuda_device).to(torch.bfloat16)
    out = G.gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn)
    ref = G.gemm_ref(a, b, a_mn_major=a_mn, b_mn_major=b_mn)
    assert _rel_err(out, ref) < 1e-2


def test_gemm_epilogues(cuda_device):
    from jax_gpt_b200.ops import gemm as G
    torch.manual_seed(1)
    M, N, K = 512, 768, 256
    a = torch.randn(M, K, device=cuda_device).to(torch.bfloat16)
    w = (torch.randn(K, N, device=cuda_device) * 0.05).to(torch.bfloat16)
    bias = torch.randn(N, device=cuda_device).to(torch.bfloat16)
    res = torch.randn(M, N, device=cuda_device).to(torch.bfloat16)
    out = G.gemm(a, w, b_mn_major=True, bias=bias, residual=res)
    ref = G.gemm_ref(a, w, b_mn_major=True, bias=bias, residual=res)
    assert _rel_err(out, ref) < 1e-2
    aux = torch.empty(M, N, device=cuda_device, dtype=torch.bfloat16)
    aux_ref = torch.empty_like(aux)
    out = G.gemm(a, w, b_mn_major=True, bias=bias, aux=aux, epilogue=G.EPI_GELU)
    ref = G.gemm_ref(a, w, b_mn_major=True, bias=bias, aux=aux_ref, epilogue=G.EPI_GELU)
    assert _rel_err(aux, aux_ref) < 1e-2 and _rel_err(out, ref) < 1e-2
    out = G.gemm(a, w, b_mn_major=True, aux=aux_ref, epilogue=G.EPI_GELU_GRAD)
    ref = G.gemm_ref(a, w, b_mn_major=True, aux=aux_ref, epilogue=G.EPI_GELU_GRAD)
    assert _rel_err(out, ref) < 1e-2
    # fp32 accumulate with split-K (the wgrad path): two accumulations into one buffer
    acc = torch.zeros(K, N, device=cuda_device)
    dy = torch.randn(M, N, device=cuda_device).to(torch.bfloat16)
    G.gemm(a, dy, a_mn_major=True, b_mn_major=True, out=acc, out_mode=G.OUT_F32_ATOMIC, split_k=4)
    G.gemm(a, dy, a_mn_major=True, b_mn_major=True, out=acc, out_mode=G.OUT_F32_ATOMIC, split_k=1)
    ref = 2 * (a.float().t() @ dy.float())
    assert _rel_err(acc, ref) < 1e-3


@pytest.mark.parametrize("M,N,K", [(4096, 3072, 256), (4000, 3080, 192), (8192, 768, 320)])
def test_gemm_pair_kernel_epilogues(cuda_device, M, N, K):
    """Shapes whose 256 x 256 tiles fill the GPU, so the CTA-pair kernel (cta_group::2) runs: every fused
    epilogue, ragged M (rows past the end of a pair tile) and an N that is not a multiple of the 64-column
    staging group, against the fp32 reference."""
    from jax_gpt_b200 import _ext
    from jax_gpt_b200.ops import gemm as G
    assert _ext.ops().gemm_uses_pair(M, N, 1) or N < 1024
    torch.manual_seed(3)
    a = torch.randn(M, K, device=cuda_device).to(torch.bfloat16)
    w = (torch.randn(K, N, device=cuda_device) * 0.05).to(torch.bfloat16)
    bias = torch.randn(N, device=cuda_device).to(torch.bfloat16)
    res = torch.randn(M, N, device=cuda_device).to(torch.bfloat16)
    out = G.gemm(a, w, b_mn_major=True, bias=bias, residual=res)
    assert _rel_err(out, G.gemm_ref(a, w, b_mn_major=True, bias=bias, residual=res)) < 1e-2
    aux = torch.empty(M, N, device=cuda_device, dtype=torch.bfloat16)
    aux_ref = torch.empty_like(aux)
    out = G.gemm(a, w, b_mn_major=True, bias=bias, aux=aux, epilogue=G.EPI_GELU)
    ref = G.gemm_ref(a, w, b_mn_major=True, bias=bias, aux=aux_ref, epilogue=G.EPI_GELU)
    assert _rel_err(aux, aux_ref) < 1e-2 and _rel_err(out, ref) < 1e-2
    out = G.gemm(a, w, b_mn_major=True, aux=aux_ref, epilogue=G.EPI_GELU_GRAD)
    assert _rel_err(out, G.gemm_ref(a, w, b_mn_major=True, aux=aux_ref, epilogue=G.EPI_GELU_GRAD)) < 1e-2
    # K-major B (the dgrad layout) and fp32 output
    wt = w.t().contiguous()
    out32 = G.gemm(a, wt, out_mode=G.OUT_F32)
    assert _rel_err(out32, a.float() @ w.float()) < 1e-2
    # weight-gradient layout with split-K accumulation: [K, N] += a^T @ dy, twice
    dy = torch.randn(M, N, device=cuda_device).to(torch.bfloat16)
    a2 = torch.randn(M, 1024, device=cuda_device).to(torch.bfloat16)
    big = torch.zeros(N, 1024, device=cuda_device)
    G.gemm(dy, a2, a_mn_major=True, b_mn_major=True, out=big, out_mode=G.OUT_F32_ATOMIC, split_k=4)
    G.gemm(dy, a2, a_mn_major=True, b_mn_major=True, out=big, out_mode=G.OUT_F32_ATOMIC, split_k=1)
    assert _rel_err(big, 2 * (dy.float().t() @ a2.float())) < 1e-3


def test_linear_autograd(cuda_device):
    from jax_gpt_b200.ops.gemm import linear
    torch.manual_seed(2)
    x = torch.randn(4, 96, 256, device=cuda_device).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(256, 512, device=cuda_device) * 0.05).to(torch.bfloat16).requires_grad_()
    b = torch.randn(512, device=cuda_device).to(torch.bfloat16).requires_grad_()
    y = linear(x, w, b)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr, br = [t.detach().float().requires_grad_() for t in (x, w, b)]
    yr = xr @ wr + br
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 1e-2
    assert _rel_err(b.grad, br.grad) < 1e-2


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("D", [64, 768, 1600, 2048, 7168])
def test_norms(cuda_device, mode, D):
    from jax_gpt_b200.ops import norm as N
    torch.manual_seed(3)
    M = 333
    x = torch.randn(M, D, device=cuda_device).to(torch.bfloat16).requires_grad_()
    g = (torch.randn(D, device=cuda_device) * 0.3 + (1 if mode < 2 else 0)).to(torch.bfloat16).requires_grad_()
    b = torch.randn(D, device=cuda_device).to(torch.bfloat16).requires_grad_() if mode == 0 else None
    eps = 1e-5
    y = N._NormFn.apply(x, g, b, mode, eps)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    gr = g.detach().float().requires_grad_()
    br = b.detach().float().requires_grad_() if b is not None else None
    yr = N.norm_ref(mode, xr, gr, br, eps)
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 2e-2
    assert _rel_err(g.grad, gr.grad) < 2e-2
    if b is not None:
        assert _rel_err(b.grad, br.grad) < 2e-2


def test_embedding_and_ce(cuda_device):
    from jax_gpt_b200.ops import misc
    torch.manual_seed(4)
    V, D, B, T = 1000, 128, 3, 50
    wte = torch.randn(V, D, device=cuda_device).to(torch.bfloat16)
    wpe = torch.randn(64, D, device=cuda_device).to(torch.bfloat16)
    idx = torch.randint(0, V, (B, T), device=cuda_device, dtype=torch.int32)
    out = misc.embed_fwd(idx, wte, wpe, pos0=3)
    ref = misc.embed_ref(idx, wte.float(), wpe.float(), pos0=3)
    assert _rel_err(out, ref) < 1e-2
    dout = torch.randn(B, T, D, device=cuda_device).to(torch.bfloat16)
    dwte = torch.zeros(V, D, device=cuda_device)
    dwpe = torch.zeros(64, D, device=cuda_device)
    misc.embed_bwd(idx, dout, dwte, dwpe, pos0=3)
    ref_wte = torch.zeros_like(dwte).index_add_(0, idx.reshape(-1).long(), dout.float().reshape(-1, D))
    ref_wpe = torch.zeros_like(dwpe)
    ref_wpe[3:3 + T] = dout.float().sum(0)
    assert _rel_err(dwte, ref_wte) < 1e-3 and _rel_err(dwpe, ref_wpe) < 1e-3
    # cross entropy with a padded vocabulary
    M, Vp = 77, 1024
    logits = (torch.randn(M, Vp, device=cuda_device) * 3).to(torch.bfloat16)
    tg = torch.randint(0, V, (M,), device=cuda_device, dtype=torch.int32)
    tg[5] = -1
    lf = logits[:, :V].float().requires_grad_()
    ref_loss = torch.nn.functional.cross_entropy(lf, tg.long(), ignore_index=-1, reduction="none")
    (ref_loss.sum() / M).backward()
    work = logits.clone()
    loss = misc.cross_entropy_fwd_bwd(work, tg, V, 1.0 / M)
    assert torch.allclose(loss, ref_loss, atol=2e-2, rtol=1e-2)
    assert _rel_err(work[:, :V], lf.grad) < 2e-2
    assert work[:, V:].abs().max().item() == 0


def test_bias_grad_sumsq_adamw(cuda_device):
    from jax_gpt_b200.ops import misc
    torch.manual_seed(5)
    dy = torch.randn(1000, 776, device=cuda_device).to(torch.bfloat16)
    assert _rel_err(misc.bias_grad(dy), dy.float().sum(0)) < 1e-3
    n = 100003
    p = torch.randn(n, device=cuda_device)
    g = torch.randn(n, device=cuda_device)
    m = torch.rand(n, device=cuda_device) * 0.1
    v = torch.rand(n, device=cuda_device) * 0.1
    ss = misc.sumsq(g)
    assert abs(ss.item() - (g.double() ** 2).sum().item()) / ss.item() < 1e-4
    hp = torch.tensor([1e-2, 1 - 0.9 ** 3, 1 - 0.95 ** 3, 0.5], device=cuda_device)
    pr, gr, mr, vr = p.clone().cpu(), g.clone().cpu(), m.clone().cpu(), v.clone().cpu()
    pb = torch.empty(n, device=cuda_device, dtype=torch.bfloat16)
    misc.adamw(p, g, m, v, hp, ss, wd=0.1, clip=1.0, p_bf16=pb)
    misc.adamw_ref(pr, gr, mr, vr, hp.cpu(), ss.cpu(), 0.9, 0.95, 1e-8, 0.1, 1.0)
    assert _rel_err(p.cpu(), pr) < 1e-5 and _rel_err(m.cpu(), mr) < 1e-5 and _rel_err(v.cpu(), vr) < 1e-5
    assert g.abs().max().item() == 0 and _rel_err(pb.float().cpu(), pr) < 1e-2


@pytest.mark.parametrize("B,T,H,Hkv,D,causal", [
    (2, 128, 2, 2, 64, True), (1, 256, 3, 3, 64, True), (2, 512, 4, 4, 64, True), (1, 200, 2, 2, 64, True),
    (1, 384, 4, 2, 64, True), (1, 256, 2, 2, 64, False), (1, 256, 2, 1, 128, True),
])
def test_attention_fwd_bwd(cuda_device, B, T, H, Hkv, D, causal):
    from jax_gpt_b200.ops import attention as A
    torch.manual_seed(6)
    q = torch.randn(B, T, H, D, device=cuda_device).to(torch.bfloat16).requires_grad_()
    k = torch.randn(B, T, Hkv, D, device=cuda_device).to(torch.bfloat16).requires_grad_()
    v = torch.randn(B, T, Hkv, D, device=cuda_device).to(torch.bfloat16).requires_grad_()
    out = A.attention(q, k, v, causal=causal)
    dout = torch.randn_like(out)
    out.backward(dout)
    qr, kr, vr = [t.detach().float().requires_grad_() for t in (q, k, v)]
    ref = A.attention_ref(qr, kr, vr, causal=causal)
    ref.backward(dout.float())
    assert _rel_err(out, ref) < 2e-2
    assert _rel_err(v.grad, vr.grad) < 3e-2
    assert _rel_err(k.grad, kr.grad) < 3e-2
    assert _rel_err(q.grad, qr.grad) < 3e-2


@pytest.mark.parametrize("B,T,H,Hkv,D,Dv", [(2, 256, 4, 2, 256, 256), (1, 384, 4, 4, 192, 128),
                                            (1, 200, 8, 1, 256, 256), (2, 330, 2, 2, 192, 128),
                                            (1, 64, 2, 2, 256, 256), (1, 1024, 2, 1, 192, 128)])
def test_attention_wide_heads_gradients(cuda_device, B, T, H, Hkv, D, Dv):
    """Wide heads (gated attention 256, MLA 192 / 128): forward kernel and the 64-query-tile backward kernel
    against autograd of the fp32 reference; the library-matmul recomputation is checked against the same
    gradients (with a small chunk, so that the key / value gradients accumulate over chunks)."""
    from jax_gpt_b200.ops import attention as A
    torch.manual_seed(9)
    q = torch.randn(B, T, H, D, device=cuda_device).to(torch.bfloat16).requires_grad_()
    k = torch.randn(B, T, Hkv, D, device=cuda_device).to(torch.bfloat16).requires_grad_()
    v = torch.randn(B, T, Hkv, Dv, device=cuda_device).to(torch.bfloat16).requires_grad_()
    dout = torch.randn(B, T, H, Dv, device=cuda_device).to(torch.bfloat16)
    out = A.attention(q, k, v, causal=True)
    out.backward(dout)
    qr, kr, vr = [t.detach().float().requires_grad_() for t in (q, k, v)]
    ref = A.attention_ref(qr, kr, vr, causal=True)
    ref.backward(dout.float())
    assert _rel_err(out, ref) < 2e-2
    for got, want in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        assert _rel_err(got, want) < 3e-2
    lse = A.attn_fwd(q.detach(), k.detach(), v.detach(), True, None)[1]
    dq, dk, dv = A.attn_bwd_chunked(q.detach(), k.detach(), v.detach(), out.detach(), dout, lse, True, None, chunk=128)
    for got, want in ((dq, qr.grad), (dk, kr.grad), (dv, vr.grad)):
        assert _rel_err(got, want) < 3e-2


def test_attention_fused_qkv_views(cuda_device):
    """q/k/v given as column slices of one [B*T, 3*H*D] projection output."""
    from jax_gpt_b200.ops import attention as A
    torch.manual_seed(7)
    B, T, H, D = 2, 256, 4, 64
    qkv = torch.randn(B, T, 3 * H * D, device=cuda_device).to(torch.bfloat16)
    q, k, v = [qkv[..., i * H * D:(i + 1) * H * D].unflatten(-1, (H, D)) for i in range(3)]
    out, _ = A.attn_fwd(q, k, v, causal=True)
    ref = A.attention_ref(q, k, v, causal=True)
    assert _rel_err(out, ref) < 2e-2


@pytest.mark.parametrize("B,T,H,Hkv,D,Dv", [(1, 256, 4, 1, 256, 256), (2, 384, 4, 4, 192, 128), (1, 200, 2, 2, 192, 128)])
def test_attention_forward_wide_heads(cuda_device, B, T, H, Hkv, D, Dv):
    """Forward-only kernels: gated attention with 256-wide heads and the MLA prefill shape 192 / 128."""
    from jax_gpt_b200.ops import attention as A
    torch.manual_seed(8)
    q = torch.randn(B, T, H, D, device=cuda_device).to(torch.bfloat16)
    k = torch.randn(B, T, Hkv, D, device=cuda_device).to(torch.bfloat16)
    v = torch.randn(B, T, Hkv, Dv, device=cuda_device).to(torch.bfloat16)
    with torch.no_grad():
        out = A.attention(q, k, v, causal=True, scale=D ** -0.5) if D == Dv else A.mla_attention(q, k, v, D ** -0.5)
    kk = k.float().repeat_interleave(H // Hkv, 2)
    vv = v.float().repeat_interleave(H // Hkv, 2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kk) * D ** -0.5
    s = s.masked_fill(~torch.ones(T, T, dtype=torch.bool, device=cuda_device).tril(), float("-inf"))
    ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), vv)
    assert out.shape == (B, T, H, Dv) and _rel_err(out, ref) < 2e-2


def test_adamw_with_bf16_state_is_unbiased(cuda_device):
    """AdamW whose weights and moments are bf16 (no fp32 master): every element within one bf16 ulp of the fp32
    update, and, because the stores round stochastically, the mean error far below the half-ulp bias that
    round-to-nearest would leave on updates smaller than an ulp."""
    from jax_gpt_b200.ops import misc
    torch.manual_seed(4)
    n = 1 << 20
    p0 = (torch.randn(n, device=cuda_device) * 0.02).to(torch.bfloat16)
    g = torch.randn(n, device=cuda_device) * 1e-3
    m0 = (torch.randn(n, device=cuda_device) * 1e-4).to(torch.bfloat16)
    v0 = (torch.rand(n, device=cuda_device) * 1e-6).to(torch.bfloat16)
    hp = torch.tensor([1e-4, 0.1, 0.05, 1.0], device=cuda_device)
    pr, mr, vr = p0.float().cpu(), m0.float().cpu(), v0.float().cpu()
    misc.adamw_ref(pr, g.cpu().clone(), mr, vr, hp.cpu(), None, 0.9, 0.95, 1e-8, 0.1, 0.0, None, zero_grad=False)
    p, m, v, gg = p0.clone(), m0.clone(), v0.clone(), g.clone()
    misc.adamw_bf16_state(p, gg, m, v, hp, None, wd=0.1, seed=123)
    assert gg.abs().max().item() == 0
    ulp = (torch.maximum(p0.float().abs().cpu(), pr.abs()) * 2 ** -7).clamp_min(1e-30)   # bf16 spacing at the result
    err = p.float().cpu() - pr
    assert (err.abs() <= ulp * 1.01).all()
    step = (pr - p0.float().cpu())
    # the true update is a small fraction of an ulp for most elements, yet its mean survives the rounding
    assert step.abs().median() < 0.5 * ulp.median()
    assert abs(err.mean().item()) < 0.02 * step.abs().mean().item()
    assert _rel_err(m.cpu(), mr) < 1e-2 and _rel_err(v.cpu(), vr) < 1e-2
    # a different seed rounds differently
    p2, m2, v2, g2 = p0.clone(), m0.clone(), v0.clone(), g.clone()
    misc.adamw_bf16_state(p2, g2, m2, v2, hp, None, wd=0.1, seed=124)
    assert not torch.equal(p, p2)


def test_grouped_matmul_without_host_sync_matches_the_loop(cuda_device):
    """The single-device MoE fallback with device-side group sizes (one grouped GEMM, nothing read back to the host)
    against the loop of per-group GEMMs, values and gradients, with an empty group."""
    from jax_gpt_b200.ops.grouped_gemm import grouped_swiglu
    torch.manual_seed(21)
    E, D, I = 6, 128, 64
    sizes = torch.tensor([40, 0, 17, 128, 3, 60], device=cuda_device)
    R = int(sizes.sum())
    mk = lambda *sh: (torch.randn(*sh, device=cuda_device) * 0.2).to(torch.bfloat16)
    x0, g0, u0, d0 = mk(R, D), mk(E, D, I), mk(E, D, I), mk(E, I, D)
    dy = mk(R, D)
    outs = []
    for sz in (sizes, sizes.tolist()):
        leaves = [t.clone().requires_grad_() for t in (x0, g0, u0, d0)]
        y = grouped_swiglu(leaves[0], sz, leaves[1], leaves[2], leaves[3])
        y.backward(dy)
        outs.append([y.detach()] + [t.grad for t in leaves])
    for a, b in zip(*outs):
        assert _rel_err(a, b) < 2e-2
