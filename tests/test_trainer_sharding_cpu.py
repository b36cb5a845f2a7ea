"""Trainer sharding API: mesh construction, the logical -> physical spec mapping, and the tensor-parallel GPT-2
forward on the shards of ``shard_train_state`` against the unsharded model, on CPU ranks (gloo). Mirrors the
reference's tests/trainer/test_sharding.py (trivial mesh, spec table, vmap padding, TP forward == unsharded)."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from jax_gpt_b200.models.gpt2 import GPT, GPTConfig
from jax_gpt_b200.trainer.config import TrainConfig
from jax_gpt_b200.trainer.optimizer import create_optimizer
from jax_gpt_b200.trainer.sharding import (LOGICAL_SPECS, activation_sharding_constraint, logical_to_physical, make_mesh,
                                           param_spec, shard_train_state)
from jax_gpt_b200.trainer.train_state import create_train_state

CFG = GPTConfig(d_model=64, d_head=16, d_ff=256, d_context=32, n_head=4, n_kv_head=4, n_layers=2, vocab_size=96)


def test_logical_to_physical_and_spec_table():
    assert logical_to_physical(("embed", "joined_heads"), 2) == (None, "tp")
    assert logical_to_physical(("embed", "joined_heads"), 3) == (None, None, "tp")      # stacked-layers axis padded
    assert logical_to_physical(("vocab", "embed"), 2) == ("tp", None)
    assert param_spec("h.attn.c_proj.kernel", 3) == (None, "tp", None)
    assert param_spec("h.mlp.c_fc.bias", 2) == (None, "tp")
    assert param_spec("ln_f.layer_norm.scale", 1) == (None,)
    model = GPT(CFG, rngs=0)
    assert set(model.params) <= set(LOGICAL_SPECS)


def test_trivial_mesh_is_the_identity():
    tc = TrainConfig(micro_batch_size=2, seq_len=16)
    mesh = make_mesh(tc, world=1, rank=0)
    assert mesh.shape == {"pp": 1, "dp": 1, "fsdp": 1, "tp": 1, "sp": 1} and mesh.group is None
    model = GPT(CFG, rngs=0)
    state = create_train_state(model, create_optimizer(model, tc))
    before = {k: v.clone() for k, v in model.params.items()}
    state = shard_train_state(state, mesh)
    assert all(torch.equal(before[k], state.model.params[k]) for k in before)
    x = torch.randn(2, 4, 8)
    assert activation_sharding_constraint(x, ("dp", None, "tp"), mesh) is x
    with pytest.raises(ValueError):
        make_mesh(TrainConfig(tp=2), world=1, rank=0)


def test_mesh_coordinates():
    tc = TrainConfig(dp=2, tp=2, pp=2)
    seen = set()
    for r in range(8):
        m = make_mesh(tc, world=8, rank=r, create_groups=False)
        seen.add((m.rank("pp"), m.rank("dp"), m.rank("tp")))
        assert m.rank("tp") == r % 2 and m.rank("dp") == (r // 2) % 2 and m.rank("pp") == r // 4
    assert len(seen) == 8


def _worker(rank, world, path):
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
    tc = TrainConfig(tp=world, micro_batch_size=2, seq_len=16)
    mesh = make_mesh(tc)
    full = GPT(CFG, rngs=3)
    g = torch.Generator().manual_seed(5)
    for k, v in full.params.items():       # biases and norms away from their trivial init
        if "bias" in k or "scale" in k:
            v.data.add_(torch.randn(v.shape, generator=g) * 0.1)
    tok = torch.randint(0, CFG.vocab_size, (2, 16), generator=g)
    ref, _ = full(tok)
    model = GPT(CFG, rngs=3)
    model.load_state_dict(full.state_dict())
    state = create_train_state(model, create_optimizer(model, tc))
    state = shard_train_state(state, mesh)
    p = state.model.params
    assert p["h.attn.c_attn.kernel"].shape == (2, 64, 192 // world) and p["wte.embedding"].shape == (96 // world, 64)
    assert state.opt_state.mu["h.mlp.c_fc.kernel"].shape == (2, 64, 256 // world)
    got, _ = state.model(tok, mesh=mesh)
    assert got.shape == ref.shape and torch.allclose(got, ref, rtol=1e-4, atol=1e-5), (got - ref).abs().max()
    # gradients: shard of the full gradient for sharded leaves, the full gradient for replicated ones
    for m in (full, state.model):
        m.requires_grad_(True)
    loss_ref = torch.nn.functional.cross_entropy(full(tok[:, :-1])[0].reshape(-1, CFG.vocab_size), tok[:, 1:].reshape(-1))
    loss_ref.backward()
    loss = torch.nn.functional.cross_entropy(state.model(tok[:, :-1], mesh=mesh)[0].reshape(-1, CFG.vocab_size),
                                             tok[:, 1:].reshape(-1))
    loss.backward()
    from jax_gpt_b200.trainer.sharding import shard_gpt2_tensor
    for k, v in state.model.params.items():
        if k == "lm_head.kernel":
            continue
        want = shard_gpt2_tensor(k, full.params[k].grad, CFG, mesh)
        assert torch.allclose(v.grad, want, rtol=2e-3, atol=1e-6), (k, (v.grad - want).abs().max())
    # without the mesh the sharded model refuses to run
    with pytest.raises(ValueError, match="shard"):
        state.model(tok)
    dist.destroy_process_group()


def _train_worker(rank, world, path):
    """Three optimizer steps tensor parallel == the same steps in one process (weights of the shard, loss, norm)."""
    from jax_gpt_b200.trainer.sharding import shard_gpt2_tensor
    from jax_gpt_b200.trainer.train_step import train_step
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
    tc = TrainConfig(tp=world, micro_batch_size=2, seq_len=16, learning_rate=1e-2, warmup_steps=0, lr_decay_steps=100,
                     grad_clip=0.5)
    mesh = make_mesh(tc)
    single = GPT(CFG, rngs=7)
    model = GPT(CFG, rngs=7)
    s_state = create_train_state(single, create_optimizer(single, tc))
    t_state = shard_train_state(create_train_state(model, create_optimizer(model, tc)), mesh)
    g = torch.Generator().manual_seed(11)
    for step in range(3):
        tok = torch.randint(0, CFG.vocab_size, (2, 17), generator=g)
        batch = (tok[:, :-1], tok[:, 1:])
        s_state, sm = train_step(s_state, batch)
        t_state, tm = train_step(t_state, batch, mesh=mesh)
        assert abs(float(sm["loss"]) - float(tm["loss"])) < 1e-5, (step, float(sm["loss"]), float(tm["loss"]))
        assert abs(float(sm["grad_norm"]) - float(tm["grad_norm"])) < 1e-4 * max(1.0, float(sm["grad_norm"]))
    for k, v in t_state.model.params.items():
        if k == "lm_head.kernel":
            continue
        want = shard_gpt2_tensor(k, single.params[k], CFG, mesh)
        assert torch.allclose(v, want, rtol=1e-3, atol=3e-4), (k, (v - want).abs().max())   # Adam amplifies rounding of tiny gradients
    dist.destroy_process_group()


def test_tensor_parallel_training_steps_match_single_process():
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_train_worker, args=(2, os.path.join(d, "rdv")), nprocs=2, join=True)


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_gpt2_matches_unsharded(world):
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(world, os.path.join(d, "rdv")), nprocs=world, join=True)
