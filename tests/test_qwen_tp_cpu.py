"""Tensor-parallel Qwen3.5 forward on CPU ranks (gloo): the local shards of ``shard_params`` fed through
``forward(..., tp_group=...)`` give the unsharded logits, with rules A (heads, experts and vocabulary split) and
rules B (experts and vocabulary only), with and without a cache, and the gradients of a sharded training step are
the matching slices of the single-process gradients. The reference checks the same equivalence on fake XLA
devices (tests/qwen35/test_sharding_multidevice.py:108-120)."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from jax_gpt_b200.models.qwen35 import Qwen35Config, forward, init_cache, init_params
from jax_gpt_b200.models.qwen35.sharding import (AXIS_RULES_A, AXIS_RULES_B, flatten, make_mesh, shard_cache,
                                                 shard_params, shard_tensor)


def _worker(rank, world, path, rules_name):
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
    torch.manual_seed(0)
    cfg = Qwen35Config.tiny()
    rules = AXIS_RULES_A if rules_name == "A" else AXIS_RULES_B
    params = init_params(cfg, 0)
    # non-trivial norms so that every path matters
    g = torch.Generator().manual_seed(1)
    for k, v in flatten(params).items():
        if k.endswith("norm") or k.endswith("norm_weight"):
            v.add_(torch.randn(v.shape, generator=g) * 0.1)
    tok = torch.randint(0, cfg.vocab_size, (2, 12), generator=g)
    mesh = make_mesh(world)
    local = shard_params(params, mesh, cfg, rules, rank=rank)
    n_sharded = sum(1 for (k, a), (_, b) in zip(flatten(params).items(), flatten(local).items()) if a.shape != b.shape)
    assert n_sharded > 0

    # ---- plain forward
    ref, _ = forward(params, tok, cfg)
    got, _ = forward(local, tok, cfg, tp_group=mesh.group)
    assert got.shape == ref.shape and (got - ref).abs().max().item() < 2e-4, (rank, (got - ref).abs().max().item())
    # the mesh argument carries the group as well
    got2, _ = forward(local, tok, cfg, mesh=mesh)
    assert torch.equal(got, got2)

    # ---- prefill + two decode steps through sharded caches
    cache = init_cache(cfg, 2, 16)
    lcache = shard_cache(init_cache(cfg, 2, 16), mesh, cfg, rules, rank=rank)
    r1, cache = forward(params, tok[:, :10], cfg, cache=cache)
    g1, lcache = forward(local, tok[:, :10], cfg, cache=lcache, tp_group=mesh.group)
    assert (g1 - r1).abs().max().item() < 2e-4
    for t in (10, 11):
        r1, cache = forward(params, tok[:, t:t + 1], cfg, cache=cache, is_decode=True)
        g1, lcache = forward(local, tok[:, t:t + 1], cfg, cache=lcache, is_decode=True, tp_group=mesh.group)
        assert (g1 - r1).abs().max().item() < 2e-4, (rank, t)

    # ---- gradients of a training step
    def loss_of(tree, **kw):
        logits, _ = forward(tree, tok[:, :-1], cfg, **kw)
        return torch.nn.functional.cross_entropy(logits.reshape(-1, cfg.vocab_size).float(), tok[:, 1:].reshape(-1))
    full_leaves = {k: v.clone().requires_grad_() for k, v in flatten(params).items()}
    loc_leaves = {k: v.clone().requires_grad_() for k, v in flatten(local).items()}

    def unflat(flat):
        out = {}
        for k, v in flat.items():
            d = out
            parts = k.split(".")
            for p in parts[:-1]:
                d = d.setdefault(p, {})
            d[parts[-1]] = v
        return out
    l_ref = loss_of(unflat(full_leaves))
    l_ref.backward()
    l_tp = loss_of(unflat(loc_leaves), tp_group=mesh.group)
    l_tp.backward()
    assert abs(float(l_ref) - float(l_tp)) < 1e-5
    worst = 0.0
    for k, v in loc_leaves.items():
        want = shard_tensor(k, full_leaves[k].grad, cfg, rules, world, rank)
        got_g = v.grad if v.grad is not None else torch.zeros_like(v)
        err = (got_g - want).abs().max().item() / (want.abs().max().item() + 1e-8)
        worst = max(worst, err)
        assert err < 2e-3, (rank, k, err)
    dist.destroy_process_group()


@pytest.mark.parametrize("world,rules", [(2, "A"), (2, "B"), (4, "B")])
def test_sharded_forward_and_gradients_match_unsharded(world, rules):
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(world, os.path.join(d, "rdv"), rules), nprocs=world, join=True)


def test_sharded_tree_without_a_group_is_rejected():
    cfg = Qwen35Config.tiny()
    params = init_params(cfg, 0)
    local = shard_params(params, make_mesh(2), cfg, AXIS_RULES_A, rank=0)
    with pytest.raises(ValueError, match="process group"):
        forward(local, torch.zeros(1, 4, dtype=torch.long), cfg)
