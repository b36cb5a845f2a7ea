"""DeepSeek-V3-style model on CPU: HF oracle, router rules, paged absorbed decode == prefill."""
import pytest
import torch

from jax_gpt_b200.cache.paged import PagedCache
from jax_gpt_b200.models.deepseek_v3 import (DeepSeekV3Config, forward, generate, init_params, load_from_hf_state_dict,
                                             make_cache)
from jax_gpt_b200.ops.router import deepseek_router_from_logits


def _hf(c, interleave):
    tfm = pytest.importorskip("transformers.models.deepseek_v3.modeling_deepseek_v3")
    from transformers.models.deepseek_v3.configuration_deepseek_v3 import DeepseekV3Config
    hc = DeepseekV3Config(
        vocab_size=c.vocab_size, hidden_size=c.d_model, intermediate_size=c.dense_intermediate_size,
        moe_intermediate_size=c.moe_intermediate_size, num_hidden_layers=c.n_layers, num_attention_heads=c.n_heads,
        num_key_value_heads=c.n_heads, n_shared_experts=1, n_routed_experts=c.n_routed_experts,
        routed_scaling_factor=c.routed_scaling_factor, kv_lora_rank=c.kv_lora_rank, q_lora_rank=c.q_lora_rank,
        qk_rope_head_dim=c.qk_rope_head_dim, v_head_dim=c.v_head_dim, qk_nope_head_dim=c.qk_nope_head_dim,
        n_group=c.n_group, topk_group=c.topk_group, num_experts_per_tok=c.n_experts_per_token,
        first_k_dense_replace=c.first_k_dense, max_position_embeddings=256, rope_interleave=interleave,
        rope_parameters={"rope_type": "default", "rope_theta": c.rope_theta})
    torch.manual_seed(0)
    hf = tfm.DeepseekV3ForCausalLM(hc).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.add_(torch.randn_like(p) * 0.1)
        for n, b in hf.named_buffers():
            if "e_score_correction_bias" in n:
                b.copy_(torch.randn_like(b) * 0.1)
    return hf


@pytest.mark.parametrize("interleave", [False, True])
def test_matches_hf(interleave):
    c = DeepSeekV3Config.tiny()
    hf = _hf(c, interleave)
    p = load_from_hf_state_dict(hf.state_dict(), c, dtype=torch.float32, rope_interleave=interleave)
    tok = torch.randint(0, c.vocab_size, (2, 11))
    with torch.no_grad():
        ref = hf(tok).logits
    assert (forward(p, tok, c) - ref).abs().max() < 1e-4


def test_paged_absorbed_decode_equals_prefill():
    c = DeepSeekV3Config.tiny()
    p = init_params(c, 1)
    tok = torch.randint(0, c.vocab_size, (2, 11))
    full = forward(p, tok, c)
    cache = make_cache(c, 32, 2, 8, torch.float32)
    outs = [forward(p, tok[:, :7], c, cache, [0, 1])]
    for t in range(7, 11):
        outs.append(forward(p, tok[:, t:t + 1], c, cache, [0, 1], is_decode=True))
    assert torch.allclose(torch.cat(outs, 1), full, atol=1e-5)
    assert cache.length(0) == 11 and cache.length(1) == 11
    out = generate(p, tok, c, 4)
    assert out.shape == (2, 4) and torch.equal(out[:, 0], full[:, -1].argmax(-1))


def test_router_group_limit_and_weights():
    torch.manual_seed(0)
    M, E, k, G, kg = 64, 32, 4, 8, 2
    logits = torch.randn(M, E)
    bias = torch.randn(E) * 0.1
    w, idx = deepseek_router_from_logits(logits, bias, k, G, kg, 2.5)
    assert torch.allclose(w.sum(-1), torch.full((M,), 2.5), atol=1e-5)
    groups = idx // (E // G)
    assert all(len(set(g.tolist())) <= kg for g in groups)          # at most topk_group groups per token
    s = torch.sigmoid(logits)
    assert torch.allclose(w, 2.5 * s.gather(1, idx) / s.gather(1, idx).sum(-1, keepdim=True), atol=1e-6)


def test_page_allocator_reuse_and_exhaustion():
    pc = PagedCache(1, 8, n_pages=4, page_size=4, max_seqs=3, max_pages_per_seq=4, dtype=torch.float32)
    pc.append(0, [0], torch.ones(1, 6, 8), commit=True)      # 2 pages
    pc.append(0, [1], 2 * torch.ones(1, 5, 8), commit=True)  # 2 pages
    assert pc.alloc.n_free == 0
    with pytest.raises(MemoryError):
        pc.append(0, [2], torch.ones(1, 1, 8))
    pc.release(0)
    assert pc.alloc.n_free == 2 and pc.length(0) == 0
    pc.append(0, [2], 3 * torch.ones(1, 3, 8), commit=True)
    assert torch.equal(pc.gather(0, 1), 2 * torch.ones(5, 8)) and torch.equal(pc.gather(0, 2), 3 * torch.ones(3, 8))
