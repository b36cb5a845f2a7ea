"""Host-side pieces of the FP8 expert path and the paged cache on CPU: packed UE8M0 scale layout, expert weight
preparation, the fp32 restatement of the kernel's quantised arithmetic, the native page table."""
import pytest
import torch

from jax_gpt_b200.ops import fp8 as Q


def test_packed_scale_layout_per_row_and_per_block():
    s = torch.exp2(torch.randint(-6, 6, (200, 3)).float())
    p = Q.pack_scales_ue8m0(s, 200, True)
    assert p.shape == (2, 3, 512) and p.dtype == torch.uint8
    for r, ks in ((0, 0), (37, 2), (137, 1), (199, 0)):
        mb, rr = divmod(r, 128)
        for j in range(4):
            assert int(p[mb, ks, (rr % 32) * 16 + (rr // 32) * 4 + j]) == int(torch.log2(s[r, ks])) + 127
    assert int(p[1, 0, (100 % 32) * 16 + (100 // 32) * 4]) == 127          # padding rows: scale 1
    w = torch.exp2(torch.randint(-6, 6, (2, 3)).float())
    pw = Q.pack_scales_ue8m0(w, 256, False)
    assert pw.shape == (2, 3, 512) and bool((pw[1, 2] == int(torch.log2(w[1, 2])) + 127).all())


def test_pow2_block_quantisation_is_exact_in_the_reference_gemm():
    torch.manual_seed(0)
    x = (torch.randn(64, 256) * 3).to(torch.bfloat16)
    w = (torch.randn(128, 256) * 0.1).to(torch.bfloat16)
    xq, xs = Q.fp8_quant_1x128_ref(x, pow2=True)
    wq, ws = Q.fp8_quant_128x128_ref(w, pow2=True)
    assert bool((torch.log2(xs) == torch.log2(xs).round()).all()) and bool((torch.log2(ws) == torch.log2(ws).round()).all())
    out = Q.fp8_gemm_ref(xq, xs, wq, ws)
    ref = x.float() @ w.float().t()
    assert ((out - ref).norm() / ref.norm()) < 6e-2


def test_expert_weight_preparation_and_quantised_reference():
    from jax_gpt_b200.models.qwen35.moe import expert_forward_single
    from jax_gpt_b200.parallel.expert_parallel import (fp8_moe_reference, quantize_expert_weights_fp8,
                                                       quantize_stacked_experts_fp8)
    torch.manual_seed(1)
    E, D, I, k, T = 4, 256, 128, 2, 48
    full = {n: (torch.randn(E, a, b) * 0.05).to(torch.bfloat16)
            for n, (a, b) in (("gate_proj", (D, I)), ("up_proj", (D, I)), ("down_proj", (I, D)))}
    qw = quantize_expert_weights_fp8(full)
    assert qw["gate_q"].shape == (E, I, D) and qw["down_q"].shape == (E, D, I)
    assert qw["sfb1"].shape == (E, I // 128, D // 128, 512) and qw["sfb2"].shape == (E, D // 128, I // 128, 512)
    c = qw["sfb1"][2, 0, 1]
    for r, src in ((10, "gate_e"), (40, "gate_e"), (70, "up_e"), (127, "up_e")):       # rows 0-63 gate, 64-127 up
        assert int(c[(r % 32) * 16 + (r // 32) * 4 + 3]) == int(qw[src][2, 0, 1])
    x = torch.randn(T, D).to(torch.bfloat16)
    w, idx = torch.softmax(torch.randn(T, E), -1).topk(k, -1)
    ref = expert_forward_single(x.float(), w, idx, {n: t.float() for n, t in full.items()})
    out = fp8_moe_reference(x, w, idx, qw)
    assert ((out - ref).norm() / ref.norm()) < 0.1
    stacked = quantize_stacked_experts_fp8({n: torch.stack([t, t]) for n, t in full.items()} | {"gate_weight": torch.zeros(2, D, E)})
    assert stacked["gate_q"].shape == (2, E, I, D) and "gate_proj" not in stacked and "gate_weight" in stacked


@pytest.mark.parametrize("native", [True, False])
def test_page_table_bookkeeping(native):
    from jax_gpt_b200.cache.paged import PagedCache
    if native:
        pytest.importorskip("torch")
        try:
            from jax_gpt_b200 import _ext
            _ext.load(build_if_missing=False)
        except Exception:
            pytest.skip("extension not built")
    c = PagedCache(1, 16, n_pages=6, page_size=4, max_seqs=4, max_pages_per_seq=3, dtype=torch.float32, native=native)
    r = torch.arange(5 * 16, dtype=torch.float32).reshape(1, 5, 16)
    c.append(0, [2], r, commit=True)
    assert c.length(2) == 5 and c.alloc.n_free == 4 and torch.equal(c.gather(0, 2), r[0])
    assert c.seq_lens.tolist() == [0, 0, 5, 0] and (c.block_table[2, :2] >= 0).all() and c.block_table[2, 2] == -1
    with pytest.raises(ValueError):
        c.reserve(1, 100)
    c.reserve(1, 12)
    with pytest.raises(MemoryError):
        c.reserve(0, 12)
    c.release(2)
    assert c.alloc.n_free == 3 and c.length(2) == 0 and c.seq_lens.tolist()[2] == 0


def test_tensor_parallel_attention_weight_shards_cover_the_heads():
    from jax_gpt_b200.models.deepseek_v3.config import DeepSeekV3Config
    from jax_gpt_b200.models.deepseek_v3.model import _attn_params
    from jax_gpt_b200.parallel.tp_attention import shard_gqa_params, shard_mla_params
    c = DeepSeekV3Config.tiny()
    g = torch.Generator().manual_seed(0)
    ap = _attn_params(c, (), lambda *s: torch.randn(*s, generator=g), lambda *s: torch.ones(*s))
    parts = [shard_mla_params(ap, c, r, 2) for r in range(2)]
    H, dn, dr, dv = c.n_heads, c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim
    qb = torch.cat([p["q_b_proj"].reshape(-1, H // 2, dn + dr) for p in parts], dim=1).reshape(-1, H * (dn + dr))
    assert torch.equal(qb, ap["q_b_proj"])
    assert torch.equal(torch.cat([p["o_proj"] for p in parts], dim=0), ap["o_proj"])
    assert parts[0]["qa_kva"].shape[1] == c.q_lora_rank + c.kv_lora_rank + dr
    gp = {"q_proj": torch.randn(32, 2 * 4 * 8), "k_proj": torch.randn(32, 2 * 8), "v_proj": torch.randn(32, 2 * 8),
          "o_proj": torch.randn(4 * 8, 32), "q_norm": torch.zeros(8), "k_norm": torch.zeros(8)}
    sp = [shard_gqa_params(gp, 4, 2, 8, r, 2) for r in range(2)]
    assert sp[0]["qkv"].shape == (32, 2 * 2 * 8 + 2 * 2 * 8) and torch.equal(torch.cat([p["o_proj"] for p in sp]), gp["o_proj"])


def test_forward_tile_order_keeps_producers_ahead_of_consumers():
    """Static tile order of the fused expert kernels (host model): every tile appears once, every down-projection
    tile comes after all gate|up tiles of its rows (so a persistent CTA never waits for a later tile), and with
    enough work the two are at least a round of CTAs apart."""
    import random
    from jax_gpt_b200.parallel.expert_parallel import forward_tile_order
    rng = random.Random(0)
    for E, grid, n1, n2 in ((8, 148, 16, 28), (64, 148, 4, 8), (512, 148, 4, 8), (512, 16, 4, 8)):
        for fill in ("dense", "sparse", "empty"):
            rows = [0 if fill == "empty" or (fill == "sparse" and rng.random() < 0.8) else rng.randint(1, 400)
                    for _ in range(E)]
            lag, tiles = forward_tile_order(rows, n1, n2, grid)
            assert 1 <= lag <= E
            expect = sum(((r + 127) // 128) * (n1 + n2) for r in rows)
            assert len(tiles) == expect == len(set(tiles))
            last_g1 = {}
            for t, (e, phase, m, n) in enumerate(tiles):
                assert 0 <= m < (rows[e] + 127) // 128 and 0 <= n < (n1 if phase == 0 else n2)
                if phase == 0:
                    last_g1[(e, m)] = t
            gaps = [t - last_g1[(e, m)] for t, (e, phase, m, n) in enumerate(tiles) if phase == 1]
            assert all(g > 0 for g in gaps)
            if fill == "dense" and expect > 8 * grid:
                first = {}
                for t, (e, phase, m, n) in enumerate(tiles):
                    if phase == 1:
                        first.setdefault(e, t)
                # except near the end of the order, an expert's first GEMM2 tile is a round of CTAs behind its GEMM1 tiles
                early = [first[e] - max(v for (ee, _), v in last_g1.items() if ee == e) for e in first if e < E - lag]
                assert sorted(early)[len(early) // 2] >= grid      # the lag is sized from the average expert
