"""Attention kernels beyond the plain training shapes: the two-tile forward at awkward lengths, prefill on top
of a cache (keys / values read from the cache buffer, queries offset) and single-token decode over the cache,
each against the fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("B,T,H,Hkv,causal", [
    (1, 64, 1, 1, True), (2, 130, 2, 1, True), (1, 257, 3, 3, True), (3, 1024, 2, 2, True), (1, 640, 4, 2, False),
    (2, 1000, 12, 12, True),
])
def test_forward_two_tile_kernel_odd_lengths(cuda_device, B, T, H, Hkv, causal):
    """Head width 64: one, an odd number and many query tiles per sequence, ragged last tile, GQA."""
    from jax_gpt_b200.ops import attention as A
    torch.manual_seed(11)
    q = torch.randn(B, T, H, 64, device=cuda_device).to(torch.bfloat16)
    k = torch.randn(B, T, Hkv, 64, device=cuda_device).to(torch.bfloat16)
    v = torch.randn(B, T, Hkv, 64, device=cuda_device).to(torch.bfloat16)
    out, lse = A.attn_fwd(q, k, v, causal=causal)
    ref = A.attention_ref(q, k, v, causal=causal)
    assert _rel_err(out, ref) < 2e-2
    # log2-sum-exp of the scaled scores
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float().repeat_interleave(H // Hkv, 2)) / 8.0
    if causal:
        s = s.masked_fill(~torch.ones(T, T, dtype=torch.bool, device=cuda_device).tril(), float("-inf"))
    want = torch.logsumexp(s, -1) / math.log(2.0)
    assert (lse - want).abs().max().item() < 2e-2


@pytest.mark.parametrize("D,Dv,H,Hkv", [(64, 64, 4, 4), (64, 64, 4, 2), (128, 128, 2, 1), (256, 256, 8, 1),
                                        (192, 128, 2, 2)])
@pytest.mark.parametrize("pos,T", [(0, 200), (128, 128), (100, 60), (300, 257)])
def test_prefill_on_top_of_a_cache(cuda_device, D, Dv, H, Hkv, pos, T):
    """Queries at positions pos .. pos+T-1 against keys / values read in place from (B, Hkv, max_len, D) caches."""
    from jax_gpt_b200.ops import attention as A
    torch.manual_seed(12)
    B, max_len = 2, 640
    ck = torch.zeros(B, Hkv, max_len, D, device=cuda_device, dtype=torch.bfloat16)
    cv = torch.zeros(B, Hkv, max_len, Dv, device=cuda_device, dtype=torch.bfloat16)
    ck[:, :, :pos + T] = torch.randn(B, Hkv, pos + T, D, device=cuda_device).to(torch.bfloat16)
    cv[:, :, :pos + T] = torch.randn(B, Hkv, pos + T, Dv, device=cuda_device).to(torch.bfloat16)
    q = torch.randn(B, T, H, D, device=cuda_device).to(torch.bfloat16)
    out = A.attention_cached(q, ck, cv, pos + T, pos, scale=D ** -0.5)
    kk = ck[:, :, :pos + T].permute(0, 2, 1, 3)
    vv = cv[:, :, :pos + T].permute(0, 2, 1, 3)
    ref = A.attention_ref(q, kk, vv, causal=True, scale=D ** -0.5, q_pos0=pos)
    assert out.shape == (B, T, H, Dv) and _rel_err(out, ref) < 2e-2


@pytest.mark.parametrize("D,H,Hkv", [(64, 12, 12), (64, 4, 2), (128, 8, 2), (256, 16, 2), (256, 4, 4)])
@pytest.mark.parametrize("n", [1, 37, 64, 1000])
def test_decode_over_dense_cache(cuda_device, D, H, Hkv, n):
    """One token per sequence over the first n cache rows; key count from the host and from a device counter."""
    from jax_gpt_b200.ops import attention as A
    torch.manual_seed(13)
    B, max_len = 3, 1024
    ck = torch.randn(B, Hkv, max_len, D, device=cuda_device).to(torch.bfloat16)
    cv = torch.randn(B, Hkv, max_len, D, device=cuda_device).to(torch.bfloat16)
    q = torch.randn(B, H, D, device=cuda_device).to(torch.bfloat16)
    kk = ck[:, :, :n].permute(0, 2, 1, 3)
    vv = cv[:, :, :n].permute(0, 2, 1, 3)
    ref = A.attention_ref(q[:, None], kk, vv, causal=False)[:, 0]
    out = A.attention_decode(q, ck, cv, kv_len=n)
    assert _rel_err(out, ref) < 2e-2
    pos = torch.tensor([n - 1], device=cuda_device, dtype=torch.int32)
    out2 = A.attention_decode(q, ck, cv, pos=pos)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("D,H,Hkv", [(64, 4, 2), (256, 16, 2)])
def test_decode_over_paged_cache(cuda_device, D, H, Hkv):
    """One token per sequence over a paged cache with ragged lengths and shuffled page ownership, against the dense
    attention over the rows gathered through the block table."""
    from jax_gpt_b200.cache.paged import PagedCache
    from jax_gpt_b200.ops import attention as A
    torch.manual_seed(14)
    lens = [1, 63, 64, 200, 517]
    B = len(lens)
    cache = PagedCache(1, 2 * Hkv * D, n_pages=64, page_size=64, max_seqs=8, max_pages_per_seq=16, device=cuda_device)
    order = [3, 0, 4, 1, 2]                       # sequences take their pages in this order: ids are interleaved
    rows = {}
    for sid in order:
        r = torch.randn(1, lens[sid], 2 * Hkv * D, device=cuda_device).to(torch.bfloat16)
        cache.append(0, [sid], r, commit=True)
        rows[sid] = r[0]
    q = torch.randn(B, H, D, device=cuda_device).to(torch.bfloat16)
    ids = cache.seq_id_tensor(list(range(B)))
    out = A.attention_decode_paged(q, cache.pool[0], cache.block_table, ids, cache.seq_lens, Hkv, len_add=0)
    for b in range(B):
        kk = rows[b][:, :Hkv * D].reshape(1, lens[b], Hkv, D)
        vv = rows[b][:, Hkv * D:].reshape(1, lens[b], Hkv, D)
        ref = A.attention_ref(q[b:b + 1, None], kk, vv, causal=False)[:, 0]
        assert _rel_err(out[b:b + 1], ref) < 2e-2, b


def test_gqa_layer_cached_paths_match_uncached(cuda_device):
    """The gated-attention layer: prompt in two chunks plus one decode token through the cache == one pass."""
    from jax_gpt_b200.models.qwen35.gqa import gqa_attention
    from jax_gpt_b200.models.qwen35.primitives import precompute_rope_freqs
    torch.manual_seed(14)
    B, T, Dm, Hq, Hkv, dh = 2, 200, 256, 4, 2, 64
    dt = torch.bfloat16
    p = {"q_proj": torch.randn(Dm, 2 * Hq * dh, device=cuda_device).mul(0.05).to(dt),
         "k_proj": torch.randn(Dm, Hkv * dh, device=cuda_device).mul(0.05).to(dt),
         "v_proj": torch.randn(Dm, Hkv * dh, device=cuda_device).mul(0.05).to(dt),
         "o_proj": torch.randn(Hq * dh, Dm, device=cuda_device).mul(0.05).to(dt),
         "q_norm": torch.zeros(dh, device=cuda_device, dtype=dt), "k_norm": torch.zeros(dh, device=cuda_device, dtype=dt)}
    x = torch.randn(B, T, Dm, device=cuda_device).to(dt)
    rope = precompute_rope_freqs(16, 512, 1e4, device=cuda_device)
    with torch.no_grad():
        full, _, _ = gqa_attention(x, p, Hq, Hkv, dh, rope, 16)
        ck = torch.zeros(B, Hkv, 512, dh, device=cuda_device, dtype=dt)
        cv = torch.zeros_like(ck)
        a, _, _ = gqa_attention(x[:, :120], p, Hq, Hkv, dh, rope, 16, ck, cv, 0)
        b, _, _ = gqa_attention(x[:, 120:199], p, Hq, Hkv, dh, rope, 16, ck, cv, 120)
        c, _, _ = gqa_attention(x[:, 199:], p, Hq, Hkv, dh, rope, 16, ck, cv, 199)
    got = torch.cat([a, b, c], dim=1)
    assert _rel_err(got, full) < 2e-2
