"""TreeTrainEngine on CPU: flat-buffer bookkeeping, gradient parity with plain autograd, AdamW parity with
torch.optim.AdamW, loss decrease on the tiny Qwen3.5 and DeepSeek-V3 configs, chunked attention backward."""
import math

import pytest
import torch

from jax_gpt_b200.trainer.lm_loss import deepseek_v3_loss_fn, qwen35_loss_fn
from jax_gpt_b200.trainer.tree_engine import TreeTrainEngine, _walk


def _batch(vocab, B=2, T=16, seed=0):
    g = torch.Generator().manual_seed(seed)
    tok = torch.randint(0, vocab, (B, T + 1), generator=g)
    return tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


def test_qwen35_tiny_grads_match_autograd_and_loss_decreases():
    from jax_gpt_b200.models.qwen35.config import Qwen35Config
    from jax_gpt_b200.models.qwen35.model import init_params
    cfg = Qwen35Config.tiny()
    params = init_params(cfg, 0, torch.float32)
    loss_fn = qwen35_loss_fn(cfg)
    eng = TreeTrainEngine(params, loss_fn, compute_dtype=torch.float32, lr=3e-3, min_lr=3e-3, warmup_steps=0,
                          grad_clip=1.0)
    tokens, targets = _batch(cfg.vocab_size)
    # gradient parity: engine's flat buffer vs autograd on an independent copy of the tree
    ref = {}
    for p, t in _walk(params):
        d = ref
        for k in p[:-1]:
            d = d.setdefault(k, {})
        d[p[-1]] = t.clone().requires_grad_(True)
    l_ref = loss_fn(ref, tokens, targets)
    l_ref.backward()
    l = eng.micro_step(tokens, targets)
    assert abs(float(l) - float(l_ref)) < 1e-5
    for p, t in _walk(ref):
        o, n, shape = eng.offsets[p]
        g = eng.flat.grad[o:o + n].view(shape)
        if t.grad is None:
            assert float(g.abs().max()) == 0.0
        else:
            assert torch.allclose(g, t.grad, atol=1e-5, rtol=1e-4), p
    first = float(l)
    assert abs(first - math.log(cfg.vocab_size)) < 1.0
    eng.apply_gradients()
    for _ in range(8):
        out = eng.train_step(tokens, targets)
    assert float(out["loss"]) < first - 0.5


def test_adamw_matches_torch_optimizer():
    torch.manual_seed(0)
    params = {"w": torch.randn(8, 8), "norm": torch.ones(8), "b": {"v": torch.randn(4, 8)}}
    x = torch.randn(16, 8)

    def loss_fn(tree, x):
        h = torch.tanh(x @ tree["w"]) * tree["norm"]
        return (h @ tree["b"]["v"].t()).pow(2).mean()

    eng = TreeTrainEngine(params, loss_fn, compute_dtype=torch.float32, lr=1e-2, min_lr=1e-2, warmup_steps=0,
                          weight_decay=0.1, grad_clip=0.0)
    ref = {k: v.clone().requires_grad_(True) for k, v in (("w", params["w"]), ("norm", params["norm"]), ("v", params["b"]["v"]))}
    opt = torch.optim.AdamW([{"params": [ref["w"], ref["v"]], "weight_decay": 0.1},
                             {"params": [ref["norm"]], "weight_decay": 0.0}], lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    for _ in range(5):
        eng.train_step(x)
        opt.zero_grad()
        loss_fn({"w": ref["w"], "norm": ref["norm"], "b": {"v": ref["v"]}}, x).backward()
        opt.step()
    assert torch.allclose(eng.tree["w"], ref["w"], atol=1e-5)
    assert torch.allclose(eng.tree["norm"], ref["norm"], atol=1e-5)
    assert torch.allclose(eng.tree["b"]["v"], ref["v"], atol=1e-5)


def test_deepseek_v3_tiny_loss_decreases_and_local_group():
    from jax_gpt_b200.models.deepseek_v3.config import DeepSeekV3Config
    from jax_gpt_b200.models.deepseek_v3.model import init_params
    from jax_gpt_b200.parallel.expert_parallel import is_expert_leaf, shard_experts
    cfg = DeepSeekV3Config.tiny()
    params = init_params(cfg, 0, torch.float32)
    # sharding helper: world 2 halves the routed experts and leaves dense MLPs alone
    half = shard_experts(params, 1, 2)
    assert half["moe_layers"]["moe"]["gate_proj"].shape[1] == cfg.n_routed_experts // 2
    assert half["dense_layers"]["mlp"]["gate_proj"].shape == params["dense_layers"]["mlp"]["gate_proj"].shape
    leaves = dict(_walk(params))
    assert is_expert_leaf(("moe_layers", "moe", "gate_proj"), leaves[("moe_layers", "moe", "gate_proj")])
    assert not is_expert_leaf(("dense_layers", "mlp", "gate_proj"), leaves[("dense_layers", "mlp", "gate_proj")])
    eng = TreeTrainEngine(params, deepseek_v3_loss_fn(cfg), compute_dtype=torch.float32, lr=3e-3, min_lr=3e-3,
                          warmup_steps=0)
    tokens, targets = _batch(cfg.vocab_size)
    first = float(eng.train_step(tokens, targets)["loss"])
    for _ in range(8):
        out = eng.train_step(tokens, targets)
    assert float(out["loss"]) < first - 0.3


@pytest.mark.parametrize("shape", [(2, 48, 4, 2, 32, 32), (1, 40, 4, 4, 24, 16)])
def test_chunked_attention_backward_matches_autograd(shape):
    from jax_gpt_b200.ops.attention import attention_ref, attn_bwd_chunked
    B, T, H, Hkv, D, Dv = shape
    g = torch.Generator().manual_seed(1)
    q = torch.randn(B, T, H, D, generator=g, requires_grad=True)
    k = torch.randn(B, T, Hkv, D, generator=g, requires_grad=True)
    v = torch.randn(B, T, Hkv, Dv, generator=g, requires_grad=True)
    scale = D ** -0.5
    rep = H // Hkv
    kf, vf = k.repeat_interleave(rep, 2), v.repeat_interleave(rep, 2)
    s = torch.einsum("bthd,bshd->bhts", q, kf) * scale
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    out = torch.einsum("bhts,bshd->bthd", torch.softmax(s, -1), vf)
    dout = torch.randn(B, T, H, Dv, generator=g)
    out.backward(dout)
    lse2 = torch.logsumexp(s, dim=-1) * 1.4426950408889634    # (B,H,T) in log2 units
    dq, dk, dv = attn_bwd_chunked(q.detach(), k.detach(), v.detach(), out.detach(), dout, lse2.detach(), True, scale,
                                  chunk=16)
    assert torch.allclose(dq, q.grad, atol=1e-4)
    assert torch.allclose(dk, k.grad, atol=1e-4)
    assert torch.allclose(dv, v.grad, atol=1e-4)


@pytest.mark.parametrize("family", ["qwen35", "deepseek_v3"])
def test_unstacked_layer_leaves_train_like_stacked_leaves(family):
    """``unstack``: per-layer autograd leaves (nested lists in the tree the model indexes) give the same
    parameters after a few steps as one stacked leaf per parameter, and the layer slices are real leaves."""
    from jax_gpt_b200.trainer.lm_loss import (deepseek_v3_loss_fn, deepseek_v3_unstack, qwen35_loss_fn,
                                              qwen35_unstack)
    if family == "qwen35":
        from jax_gpt_b200.models.qwen35 import Qwen35Config, init_params
        cfg = Qwen35Config.tiny()
        params, make_loss, unstack = init_params(cfg, 0), qwen35_loss_fn, qwen35_unstack
    else:
        from jax_gpt_b200.models.deepseek_v3.config import DeepSeekV3Config
        from jax_gpt_b200.models.deepseek_v3.model import init_params
        cfg = DeepSeekV3Config.tiny()
        params, make_loss, unstack = init_params(cfg, 0, torch.float32), deepseek_v3_loss_fn, deepseek_v3_unstack
    tokens, targets = _batch(cfg.vocab_size)
    engines = [TreeTrainEngine(params, make_loss(cfg), compute_dtype=torch.float32, lr=3e-3, min_lr=3e-3, warmup_steps=0,
                               unstack=u) for u in (None, unstack)]
    for _ in range(3):
        losses = [float(e.train_step(tokens, targets)["loss"]) for e in engines]
        assert abs(losses[0] - losses[1]) < 1e-4, losses
    a, b = engines[0].master_tree(), engines[1].master_tree()
    for (pa, ta), (pb, tb) in zip(_walk(a), _walk(b)):
        assert pa == pb and torch.allclose(ta, tb, atol=1e-5), pa
    key = "groups" if family == "qwen35" else "moe_layers"
    node = engines[1].tree[key]
    while isinstance(node, dict):
        node = node[sorted(node.keys())[0]]
    assert isinstance(node, list)
    leaf = node[0][0] if isinstance(node[0], list) else node[0]
    assert leaf.is_leaf and leaf.requires_grad
