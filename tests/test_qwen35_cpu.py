"""Qwen3.5 hybrid model on CPU: op properties, prefill == recurrence, cache == no cache,
causality, FP8 bounds, HF oracle, sharding rules, offload forward."""
import math

import pytest
import torch

from jax_gpt_b200.models.qwen35 import Qwen35Config, forward, generate, init_cache, init_params
from jax_gpt_b200.models.qwen35 import deltanet as DN
from jax_gpt_b200.models.qwen35 import fp8 as F8
from jax_gpt_b200.models.qwen35 import moe as MOE
from jax_gpt_b200.models.qwen35 import quantize as Q
from jax_gpt_b200.models.qwen35 import sharding as SH
from jax_gpt_b200.models.qwen35.block import _slice
from jax_gpt_b200.models.qwen35.gqa import gqa_attention
from jax_gpt_b200.models.qwen35.primitives import apply_rotary_emb, precompute_rope_freqs, rms_norm


@pytest.fixture(scope="module")
def cfg():
    return Qwen35Config.tiny()


@pytest.fixture(scope="module")
def params(cfg):
    return init_params(cfg, 0)


def test_config_presets():
    f = Qwen35Config.full()
    assert f.n_groups == 15 and f.gqa_rope_dim == 64 and f.layer_type(3) == "full" and f.layer_type(4) == "linear"
    assert Qwen35Config.mini().n_routed_experts == 32 and Qwen35Config.ns().delta_chunk_size == 64


def test_rms_norm_conventions():
    x = torch.randn(4, 7, 64)
    y = rms_norm(x, torch.zeros(64))
    assert torch.allclose((y * y).mean(-1), torch.ones(4, 7), atol=1e-3)
    assert torch.allclose(rms_norm(x, torch.ones(64)), 2 * y, atol=1e-5)


def test_rope_norm_preserving_and_partial():
    fr = precompute_rope_freqs(8, 16)
    x = torch.randn(2, 16, 3, 32)
    y = apply_rotary_emb(x, fr, 8)
    assert torch.allclose(y[..., 8:], x[..., 8:])
    assert torch.allclose(y[..., :8].norm(dim=-1), x[..., :8].norm(dim=-1), atol=1e-5)
    assert torch.allclose(y[:, 0], x[:, 0], atol=1e-6)  # position 0 is the identity


def test_fp8_roundtrip_and_matmul():
    x = torch.randn(16, 128)
    q, s = F8.dynamic_quantize_fp8(x)
    assert ((q.float() * s - x).abs().max() / x.abs().max()) < 0.15
    w = torch.randn(128, 64) * 0.1
    qw = Q.quantize_weight(w)
    assert (F8.fp8_matmul(x, qw["w"], qw["scale_inv"]) - x @ w).abs().max() < 0.5
    # scale semantics: doubling scale_inv halves the de-quantised weight
    y1 = F8.fp8_matmul(x, qw["w"], qw["scale_inv"])
    y2 = F8.fp8_matmul(x, qw["w"], qw["scale_inv"] * 2)
    assert torch.allclose(y2, y1 / 2, atol=1e-5)
    # grouped variant applies both scales
    ws = torch.randn(3, 128, 64) * 0.1
    qws = Q.quantize_weight(ws)
    sizes = torch.tensor([5, 0, 11])
    out = F8.fp8_ragged_dot(x, qws["w"], sizes, qws["scale_inv"])
    ref = torch.cat([x[:5] @ ws[0], x[5:] @ ws[2]])
    assert (out - ref).abs().max() < 0.5


def test_quantize_tree_skips_and_counts(cfg, params):
    qp = Q.quantize_params_fp8(params)
    assert F8.is_fp8_weight(qp["lm_head"]) and not F8.is_fp8_weight(qp["embed"])
    assert not F8.is_fp8_weight(qp["groups"]["delta_layers"]["attn"]["conv_weight"])
    total, n8 = Q.count_fp8_params(qp)
    assert 0 < n8 < total
    dq = Q.dequantize_params(qp)
    assert (dq["lm_head"] - params["lm_head"]).abs().max() < 0.01
    lg, _ = forward(qp, torch.randint(0, cfg.vocab_size, (1, 6)), cfg)
    assert torch.isfinite(lg).all()


def test_moe_routing_and_layer(cfg, params):
    lp = _slice(_slice(params["groups"], 0)["gqa_layer"], slice(None))["moe"] if False else _slice(params["groups"], 0)["gqa_layer"]["moe"]
    x = torch.randn(10, cfg.d_model)
    w, idx = MOE.moe_routing(x, lp["gate_weight"], cfg.n_experts_per_token)
    assert torch.allclose(w.sum(-1), torch.ones(10), atol=1e-5) and idx.shape == (10, cfg.n_experts_per_token)
    y = MOE.moe_layer(x.reshape(2, 5, -1), lp, cfg.n_experts_per_token)
    assert y.shape == (2, 5, cfg.d_model) and torch.isfinite(y).all()
    # grouped path equals a per-token dense evaluation
    dense = torch.zeros(10, cfg.d_model)
    for t in range(10):
        for j in range(cfg.n_experts_per_token):
            e = idx[t, j]
            h = torch.nn.functional.silu(x[t] @ lp["gate_proj"][e]) * (x[t] @ lp["up_proj"][e])
            dense[t] += w[t, j] * (h @ lp["down_proj"][e])
    assert torch.allclose(MOE.expert_forward_single(x, w, idx, lp), dense, atol=1e-5)


def test_gqa_cache_equals_no_cache_and_causal(cfg, params):
    lp = _slice(params["groups"], 0)["gqa_layer"]["attn"]
    lp = dict(lp, q_norm=torch.randn(cfg.gqa_head_dim) * 0.1, k_norm=torch.randn(cfg.gqa_head_dim) * 0.1)
    rope = precompute_rope_freqs(cfg.gqa_rope_dim, 32, cfg.gqa_rope_theta)
    x = torch.randn(2, 12, cfg.d_model)
    args = (cfg.gqa_n_q_heads, cfg.gqa_n_kv_heads, cfg.gqa_head_dim, rope, cfg.gqa_rope_dim)
    full, _, _ = gqa_attention(x, lp, *args)
    ck = torch.zeros(2, cfg.gqa_n_kv_heads, 32, cfg.gqa_head_dim)
    cv = torch.zeros_like(ck)
    a, _, _ = gqa_attention(x[:, :7], lp, *args, ck, cv, 0)
    b, _, _ = gqa_attention(x[:, 7:], lp, *args, ck, cv, 7)
    assert torch.allclose(torch.cat([a, b], 1), full, atol=1e-5)
    x2 = x.clone()
    x2[:, 6:] += 1.0
    pert, _, _ = gqa_attention(x2, lp, *args)
    assert torch.allclose(pert[:, :6], full[:, :6], atol=1e-6)


def test_deltanet_prefill_matches_recurrence(cfg, params):
    lp = dict(_slice(_slice(params["groups"], 0)["delta_layers"], 2)["attn"])
    lp["norm_weight"] = torch.randn(cfg.delta_v_head_dim) * 0.5 + 1.0  # non-trivial gated-norm weight
    args = (cfg.delta_n_qk_heads, cfg.delta_n_v_heads, cfg.delta_qk_head_dim, cfg.delta_v_head_dim)
    x = torch.randn(2, 3 * 8 + 5, cfg.d_model)
    y, S, conv = DN.deltanet_prefill(x, lp, *args, cfg.delta_conv_kernel, 8)
    st = torch.zeros(2, cfg.delta_n_v_heads, cfg.delta_qk_head_dim, cfg.delta_v_head_dim)
    cs = torch.zeros(2, cfg.delta_conv_dim, cfg.delta_conv_kernel)
    outs = []
    for t in range(x.shape[1]):
        o, st, cs = DN.deltanet_recurrent_step(x[:, t:t + 1], lp, st, cs, *args)
        outs.append(o)
    assert y.abs().max() > 1e-4
    assert torch.allclose(torch.cat(outs, 1), y, atol=1e-4)
    assert torch.allclose(st, S, atol=1e-4) and torch.allclose(cs, conv, atol=1e-5)
    # the state decays under zero input
    zero = torch.zeros(2, 1, cfg.d_model)
    _, st2, _ = DN.deltanet_recurrent_step(zero, lp, st, cs, *args)
    assert st2.abs().sum() < st.abs().sum()


def test_model_shapes_cache_and_generate(cfg, params):
    tok = torch.randint(0, cfg.vocab_size, (2, 9))
    lg, c0 = forward(params, tok, cfg)
    assert lg.shape == (2, 9, cfg.vocab_size) and c0 is None
    cache = init_cache(cfg, 2, 16)
    l1, cache = forward(params, tok[:, :4], cfg, cache=cache)
    assert cache.pos == 4
    l2, cache = forward(params, tok[:, 4:5], cfg, cache=cache, is_decode=True)
    assert cache.pos == 5
    assert torch.allclose(l1, lg[:, :4], atol=1e-5) and torch.allclose(l2[:, 0], lg[:, 4], atol=1e-4)
    out = generate(params, tok, cfg, 6, key=3)
    assert out.shape == (2, 6) and out.min() >= 0 and out.max() < cfg.vocab_size
    greedy = generate(params, tok, cfg, 3, temperature=0.0)
    assert torch.equal(greedy[:, 0], lg[:, -1].argmax(-1))


def test_hf_oracle_and_offload(cfg):
    tfm = pytest.importorskip("transformers.models.qwen3_5_moe.modeling_qwen3_5_moe")
    from transformers.models.qwen3_5_moe.configuration_qwen3_5_moe import Qwen3_5MoeTextConfig
    from jax_gpt_b200.models.qwen35.offload import forward_offload
    from jax_gpt_b200.models.qwen35.weight_loader import load_from_hf_state_dict
    c = cfg
    hc = Qwen3_5MoeTextConfig(
        vocab_size=c.vocab_size, hidden_size=c.d_model, num_hidden_layers=c.n_layers, num_attention_heads=c.gqa_n_q_heads,
        num_key_value_heads=c.gqa_n_kv_heads, head_dim=c.gqa_head_dim, max_position_embeddings=128,
        linear_conv_kernel_dim=4, linear_key_head_dim=c.delta_qk_head_dim, linear_value_head_dim=c.delta_v_head_dim,
        linear_num_key_heads=c.delta_n_qk_heads, linear_num_value_heads=c.delta_n_v_heads,
        moe_intermediate_size=c.moe_intermediate_size, shared_expert_intermediate_size=c.shared_expert_intermediate_size,
        num_experts_per_tok=c.n_experts_per_token, num_experts=c.n_routed_experts,
        rope_parameters={"rope_type": "default", "rope_theta": c.gqa_rope_theta, "partial_rotary_factor": 0.25})
    torch.manual_seed(0)
    hf = tfm.Qwen3_5MoeForCausalLM(hc).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.add_(torch.randn_like(p) * 0.1)
    sd = hf.state_dict()
    p = load_from_hf_state_dict(sd, c, dtype=torch.float32)
    tok = torch.randint(0, c.vocab_size, (2, 13))
    with torch.no_grad():
        ref = hf(tok).logits
    out, _ = forward(p, tok, c)
    assert (out - ref).abs().max() < 1e-4
    off, _ = forward_offload(tok, c, None, dtype=torch.float32, verbose=False, state_dict=sd)
    assert torch.allclose(off, out, atol=1e-5)


def test_sharding_rules(cfg, params):
    flat = SH.flatten(params)
    for name in flat:
        SH.resolve_logical_axes(name)  # every parameter resolves
    mesh = SH.make_mesh(2)
    shards = [SH.shard_params(params, mesh, cfg, SH.AXIS_RULES_A, rank=r) for r in range(2)]
    e = cfg.n_routed_experts // 2
    gp = params["groups"]["gqa_layer"]["moe"]["gate_proj"]
    assert torch.equal(shards[1]["groups"]["gqa_layer"]["moe"]["gate_proj"], gp[:, e:])
    # replicated where rules B say so, split where rules A do
    sB = SH.shard_params(params, mesh, cfg, SH.AXIS_RULES_B, rank=1)
    assert sB["groups"]["gqa_layer"]["attn"]["q_proj"].shape == params["groups"]["gqa_layer"]["attn"]["q_proj"].shape
    assert shards[0]["groups"]["gqa_layer"]["attn"]["q_proj"].shape[-1] == params["groups"]["gqa_layer"]["attn"]["q_proj"].shape[-1] // 2
    # q|k|v segments of in_proj_qkv are split head-aligned: concatenating the rank shards per segment restores them
    full = params["groups"]["delta_layers"]["attn"]["in_proj_qkv"]
    Kd, Vd = cfg.delta_key_dim, cfg.delta_value_dim
    a, b = [s["groups"]["delta_layers"]["attn"]["in_proj_qkv"] for s in shards]
    rec = torch.cat([a[..., :Kd // 2], b[..., :Kd // 2], a[..., Kd // 2:Kd], b[..., Kd // 2:Kd], a[..., Kd:], b[..., Kd:]], -1)
    assert torch.equal(rec, full)
    # expert-sharded forward (each rank computes its experts, outputs summed) equals the full MoE
    lp = _slice(params["groups"], 0)["gqa_layer"]["moe"]
    x = torch.randn(6, cfg.d_model)
    w, idx = MOE.moe_routing(x, lp["gate_weight"], cfg.n_experts_per_token)
    ref = MOE.expert_forward_single(x, w, idx, lp)
    acc = torch.zeros_like(ref)
    for r in range(2):
        lpr = _slice(shards[r]["groups"], 0)["gqa_layer"]["moe"]
        mine = (idx // e) == r
        wr = torch.where(mine, w, torch.zeros_like(w))
        acc += MOE.expert_forward_single(x, wr, torch.where(mine, idx - r * e, torch.zeros_like(idx)), lpr)
    assert torch.allclose(acc, ref, atol=1e-5)


def test_decode_engine_matches_function_style_decode(cfg, params):
    """The in-place decode engine (device-side position, masked attention over the whole cache, states updated
    in place) produces the logits of ``forward(..., is_decode=True)`` step after step."""
    from jax_gpt_b200.models.qwen35.decode_engine import Qwen35DecodeEngine
    torch.manual_seed(11)
    B, T, steps = 2, 6, 4
    tok = torch.randint(0, cfg.vocab_size, (B, T))
    with torch.no_grad():
        cache_a = init_cache(cfg, B, T + steps + 2)
        logits, cache_a = forward(params, tok, cfg, cache=cache_a)
        cache_b = init_cache(cfg, B, T + steps + 2)
        _, cache_b = forward(params, tok, cfg, cache=cache_b)
        eng = Qwen35DecodeEngine(params, cfg, cache_b, use_cuda_graph=False)
        nxt = logits[:, -1].argmax(-1)
        for _ in range(steps):
            ref, cache_a = forward(params, nxt[:, None], cfg, cache=cache_a, is_decode=True)
            got = eng.step(nxt)
            assert torch.allclose(eng.logits, ref[:, -1], atol=2e-4, rtol=1e-4)
            assert torch.equal(got, ref[:, -1].argmax(-1))
            nxt = got.clone()
        assert eng.pos == cache_a.pos == T + steps
        back = eng.cache(torch.float32)
        assert torch.allclose(back.delta_M, cache_a.delta_M, atol=1e-5)
        assert torch.allclose(back.gqa_k[:, :, :, :eng.pos], cache_a.gqa_k[:, :, :, :eng.pos], atol=1e-5)


def test_decode_engine_with_paged_kv_matches_dense_engine(cfg, params):
    """The engine with its gated-attention keys / values in a paged cache (pages, block table, per-sequence
    lengths) produces the logits of the engine on the dense buffers, step after step."""
    from jax_gpt_b200.models.qwen35.decode_engine import Qwen35DecodeEngine
    torch.manual_seed(12)
    B, T, steps = 2, 70, 5                      # 70 prompt tokens: the second 64-token page is in use
    tok = torch.randint(0, cfg.vocab_size, (B, T))
    with torch.no_grad():
        ca = init_cache(cfg, B, T + steps + 2)
        logits, ca = forward(params, tok, cfg, cache=ca)
        cb = init_cache(cfg, B, T + steps + 2)
        _, cb = forward(params, tok, cfg, cache=cb)
        dense = Qwen35DecodeEngine(params, cfg, ca, use_cuda_graph=False)
        paged = Qwen35DecodeEngine(params, cfg, cb, use_cuda_graph=False, paged_kv=True)
        assert paged.k is None and paged.paged.length(0) == T
        nxt = logits[:, -1].argmax(-1)
        for _ in range(steps):
            a = dense.step(nxt).clone()
            b = paged.step(nxt).clone()
            assert torch.allclose(paged.logits, dense.logits, atol=2e-4, rtol=1e-4)
            assert torch.equal(a, b)
            nxt = a


def test_generate_with_engine_matches_generate(cfg, params):
    """Same continuation as ``generate`` for greedy decoding and for sampling with the same seed."""
    from jax_gpt_b200.models.qwen35.decode_engine import generate_with_engine
    prompt = torch.randint(0, cfg.vocab_size, (2, 5), generator=torch.Generator().manual_seed(4))
    for kw in (dict(temperature=0.0), dict(temperature=0.9, top_k=8, key=3)):
        a = generate(params, prompt, cfg, 6, **kw)
        b = generate_with_engine(params, prompt, cfg, 6, **kw)
        assert a.shape == b.shape == (2, 6) and torch.equal(a, b), kw
