"""Checkpoints of the function-style training engine: save / resume gives the same next step, and the expert
shards written at one expert-parallel degree load at another."""
import os

import torch

from jax_gpt_b200.ckpt.tree_ckpt import TreeCheckpointer
from jax_gpt_b200.models.qwen35 import Qwen35Config
from jax_gpt_b200.models.qwen35.model import init_params
from jax_gpt_b200.parallel.expert_parallel import is_expert_leaf, shard_experts
from jax_gpt_b200.trainer.lm_loss import qwen35_loss_fn, qwen35_unstack
from jax_gpt_b200.trainer.tree_engine import TreeTrainEngine


def _engine(cfg, params, local=None, seed_lr=1e-2):
    return TreeTrainEngine(params, qwen35_loss_fn(cfg, None), device="cpu", compute_dtype=torch.float32, local=local,
                           unstack=qwen35_unstack, lr=seed_lr, warmup_steps=0, lr_decay_steps=100)


def _batch(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    t = torch.randint(0, cfg.vocab_size, (2, 17), generator=g)
    return t[:, :-1], t[:, 1:]


def test_save_resume_continues_identically(tmp_path):
    cfg = Qwen35Config.tiny()
    a = _engine(cfg, init_params(cfg, 0, torch.float32))
    for s in range(3):
        a.train_step(*_batch(cfg, s))
    ck = TreeCheckpointer(str(tmp_path), keep=2)
    ck.save(3, a, extra={"cursor": 11})
    assert ck.latest_step() == 3
    b = _engine(cfg, init_params(cfg, 1, torch.float32))            # different init, then restored
    man = TreeCheckpointer(str(tmp_path)).load(b)
    assert man["step"] == 3 and man["extra"] == {"cursor": 11} and b.step_count == 3
    la = a.train_step(*_batch(cfg, 9))["loss"]
    lb = b.train_step(*_batch(cfg, 9))["loss"]
    assert abs(float(la) - float(lb)) < 1e-6
    assert torch.allclose(a.flat.master, b.flat.master, atol=1e-7)
    # keep-N and unfinished directories
    for s in (4, 5):
        ck.save(s, a)
    os.makedirs(tmp_path / "99")
    assert ck.complete_steps() == [4, 5] and ck.latest_step() == 5


def test_expert_shards_load_at_another_degree(tmp_path):
    """Two 'ranks' save their halves of the experts; one engine holding all experts (degree 1) and four engines
    holding a quarter each (degree 4) restore exactly the slices they own."""
    cfg = Qwen35Config.tiny()
    full = init_params(cfg, 0, torch.float32)
    engines = [_engine(cfg, shard_experts(full, r, 2), local=is_expert_leaf) for r in range(2)]
    for r, e in enumerate(engines):                                   # distinguishable optimizer state per rank
        e.local_m.fill_(0.5 + r)
        e.local_v.fill_(0.25 + r)
        e.step_count = 7
    # sequential stand-in for the two processes of a job: rank 1 first, rank 0 last (it writes the manifest)
    TreeCheckpointer(str(tmp_path), rank=1, world=2).save(7, engines[1])
    TreeCheckpointer(str(tmp_path), rank=0, world=2).save(7, engines[0])
    for world in (1, 4):
        for r in range(world):
            other = init_params(cfg, 5, torch.float32)
            e = _engine(cfg, shard_experts(other, r, world), local=is_expert_leaf)
            TreeCheckpointer(str(tmp_path), rank=r, world=world).load(e)
            want = shard_experts(full, r, world)
            got_master, got_m, _ = e.local_state()
            k = ("groups", "delta_layers", "moe", "gate_proj")
            w, g_ = want, got_master
            for key in k:
                w, g_ = w[key], g_[key]
            assert torch.equal(g_, w) and e.step_count == 7
            m = got_m
            for key in k:
                m = m[key]
            E = cfg.n_routed_experts // world
            first_global = r * E
            assert float(m.select(m.dim() - 3, 0).mean()) == (0.5 if first_global < cfg.n_routed_experts // 2 else 1.5)
