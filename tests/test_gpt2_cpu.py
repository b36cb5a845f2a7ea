"""GPT-2 model on CPU: shapes, cache, generation length, HF parity, lm-eval scoring core."""
import torch

from jax_gpt_b200.models.gpt2 import GPT, GPTConfig
from jax_gpt_b200.models.gpt2.lm_eval_adapter import loglikelihood_tokens

CFG = GPTConfig(d_model=64, d_head=16, d_ff=256, d_context=32, n_head=4, n_kv_head=4, n_layers=2, vocab_size=100)


def test_presets():
    c = GPTConfig.from_model_type("gpt2-medium")
    assert (c.n_layers, c.n_head, c.d_model, c.d_ff, c.d_head) == (24, 16, 1024, 4096, 64)
    assert GPTConfig.from_model_type("gpt2", d_context=256).d_context == 256


def test_forward_cache_generate():
    m = GPT(CFG, seed=0)
    x = torch.randint(0, 100, (2, 8))
    logits, cache = m(x)
    assert logits.shape == (2, 8, 100) and cache is None
    c = m.init_cache(2)
    l1, c = m(x[:, :5], cache=c)
    assert c.pos == 5
    l2, c = m(x[:, 5:], cache=c)
    assert c.pos == 8 and torch.allclose(torch.cat([l1, l2], 1), logits, atol=1e-5)
    out = m.generate(x, 5, temperature=0.8, top_k=10, rngs=1)
    assert out.shape == (2, 13) and torch.equal(out[:, :8], x)
    _, _, acts = m(x, return_activations=True)
    assert {"initial_embedding", "block_0_ln1_output", "block_1_mlp_output_pre_residual", "final_layernorm", "final_logits"} <= set(acts)
    # the unused lm_head parameter is part of the tree for checkpoint parity
    assert m.params["lm_head.kernel"].shape == (64, 100)


def test_hf_parity_and_activation_compare():
    from transformers import GPT2Config, GPT2LMHeadModel
    hf = GPT2LMHeadModel(GPT2Config(vocab_size=100, n_positions=32, n_embd=64, n_layer=2, n_head=4,
                                    activation_function="gelu_new", resid_pdrop=0, embd_pdrop=0, attn_pdrop=0)).eval()
    m = GPT.from_hf_state_dict(hf.state_dict(), CFG)
    x = torch.randint(0, 100, (2, 9))
    with torch.no_grad():
        assert (m(x)[0] - hf(x).logits).abs().max() < 1e-4
    assert max(r[3] for r in m.compare_activations(hf, 2, 8)) < 1e-4


def test_loglikelihood_tokens():
    m = GPT(CFG, seed=1)
    reqs = [([1, 2, 3], [4, 5]), ([7], [8, 9, 10]), ([11, 12, 13, 14], [15])]
    got = loglikelihood_tokens(m, reqs, batch_size=2, max_len=32)
    for (ctx, cont), (ll, greedy) in zip(reqs, got):
        full = torch.tensor([ctx + cont])
        lp = torch.log_softmax(m(full[:, :-1])[0].float(), -1)[0]
        want = sum(lp[len(ctx) - 1 + i, t].item() for i, t in enumerate(cont))
        assert abs(ll - want) < 1e-4 and isinstance(greedy, bool)


def test_dropout_is_applied_only_when_training():
    """``config.dropout`` acts in ``deterministic=False`` passes (embedding, attention probabilities, both residual
    branches) and never in evaluation or cached decoding; p = 0 leaves the training pass equal to evaluation."""
    cfg = GPTConfig(d_model=64, d_head=16, d_ff=256, d_context=32, n_head=4, n_kv_head=4, n_layers=2, vocab_size=100,
                    dropout=0.5)
    m = GPT(cfg, seed=0)
    x = torch.randint(0, 100, (2, 8))
    ev1, _ = m(x, deterministic=True)
    ev2, _ = m(x)
    assert torch.equal(ev1, ev2)
    torch.manual_seed(0)
    tr1, _ = m(x, deterministic=False)
    tr2, _ = m(x, deterministic=False)
    assert not torch.allclose(tr1, ev1, atol=1e-3) and not torch.allclose(tr1, tr2, atol=1e-3)
    m0 = GPT(CFG, seed=0)                      # dropout 0.0
    a, _ = m0(x, deterministic=False)
    b, _ = m0(x, deterministic=True)
    assert torch.allclose(a, b, atol=1e-6)
    # gradients flow through the dropout path
    for p in m.params.values():
        p.requires_grad_(True)
    m(x, deterministic=False)[0].sum().backward()
    assert m.params["h.attn.c_attn.kernel"].grad.abs().sum() > 0


def test_golden_log_script_matches_the_pytorch_model():
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "scripts", "debug_golden_log.py")
    spec = importlib.util.spec_from_file_location("debug_golden_log", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    rc = mod.main(["--random", "--n-layers", "2", "--n-head", "2", "--d-model", "64", "--ctx", "64", "--vocab", "300",
                   "--new-tokens", "4", "--tolerance", "1e-3"])
    assert rc == 0
