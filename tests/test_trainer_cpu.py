"""Trainer library on CPU: config 0 smoke (GPT-2 small, 10 AdamW steps), optimizer mask and
schedule, accumulation, metrics, checkpoint round-trip, data pipeline, config overrides."""
import json
import math
import os

import numpy as np
import pytest
import torch

from jax_gpt_b200.data.pipeline import DataPipeline
from jax_gpt_b200.data.tokenize import tokenize, write_synthetic
from jax_gpt_b200.models.gpt2 import GPT, GPTConfig
from jax_gpt_b200.trainer import (MetricsLogger, TrainConfig, apply_overrides, build_decay_mask, compute_mfu,
                                  compute_model_flops, create_optimizer, create_train_state, eval_step, train_step,
                                  train_step_with_accumulation)
from jax_gpt_b200.trainer.checkpointing import CheckpointManager

TINY = GPTConfig(d_model=64, d_head=16, d_ff=256, d_context=64, n_head=4, n_kv_head=4, n_layers=2, vocab_size=100)


def _state(seed=0, **kw):
    tc = TrainConfig(learning_rate=1e-2, warmup_steps=0, lr_decay_steps=1000, **kw)
    m = GPT(TINY, seed=seed)
    return tc, create_train_state(m, create_optimizer(m, tc))


def _batch(seed=0, B=4, T=32):
    g = torch.Generator().manual_seed(seed)
    tok = torch.randint(0, TINY.vocab_size, (B, T + 1), generator=g)
    return tok[:, :-1], tok[:, 1:]


def test_gpt2_small_cpu_ten_adamw_steps():
    """GPT-2 small, fp32, batch 4 x 256 uniform-random ids from seed 0, lr 6e-4: the loss
    starts near ln(50257) and decreases."""
    cfg = GPTConfig.from_model_type("gpt2")
    tc = TrainConfig(learning_rate=6e-4, warmup_steps=0, lr_decay_steps=1000)
    model = GPT(cfg, seed=0)
    state = create_train_state(model, create_optimizer(model, tc))
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (4, 257), generator=g)
    batch = (tok[:, :-1], tok[:, 1:])
    losses = []
    for _ in range(10):
        state, m = train_step(state, batch)
        losses.append(float(m["loss"]))
    assert abs(losses[0] - math.log(cfg.vocab_size)) < 0.5, losses
    assert losses[-1] < losses[0] - 0.5, losses
    assert all(b < a + 0.05 for a, b in zip(losses, losses[1:])), losses


def test_train_step_basics():
    tc, st = _state()
    b = _batch()
    st, m0 = train_step(st, b)
    assert abs(float(m0["loss"]) - math.log(TINY.vocab_size)) < 1.5
    assert set(m0) >= {"loss", "grad_norm", "lr"} and m0["grad_norm"] > 0
    for _ in range(49):
        st, m = train_step(st, b)
    assert st.step == 50 and float(m["loss"]) < float(m0["loss"])
    before = {k: v.clone() for k, v in st.model.params.items()}
    ev = eval_step(st.model, b)
    assert math.isfinite(float(ev)) and all(torch.equal(before[k], v) for k, v in st.model.params.items())


def test_accumulation_matches_single_step():
    _, a = _state()
    _, b = _state()
    batch = _batch()
    a, _ = train_step(a, batch)
    b, _ = train_step_with_accumulation(b, [batch, batch])
    for k in a.model.params:
        assert torch.allclose(a.model.params[k], b.model.params[k], rtol=1e-4, atol=1e-6), k


def test_decay_mask_and_schedule():
    m = GPT(TINY)
    mask = build_decay_mask(m)
    assert not mask["wte.embedding"] and not mask["h.attn.c_attn.bias"] and not mask["ln_f.layer_norm.scale"]
    assert mask["h.attn.c_attn.kernel"] and mask["h.mlp.c_proj.kernel"]
    tx = create_optimizer(m, TrainConfig(learning_rate=1.0, min_lr=0.1, warmup_steps=10, lr_decay_steps=110))
    assert tx.schedule(0) == 0.0 and abs(tx.schedule(5) - 0.5) < 1e-9 and abs(tx.schedule(10) - 1.0) < 1e-9
    assert abs(tx.schedule(60) - 0.55) < 1e-9 and tx.schedule(110) == 0.1 and tx.schedule(500) == 0.1


def test_metrics():
    f = compute_model_flops(GPTConfig.from_model_type("gpt2"))
    assert 1.5e8 < f < 2.0e8
    mfu = compute_mfu(f, 1e6, "b200", 1)
    assert 0 < mfu < 1 and abs(compute_mfu(f, 1e6, "b200", 2) - mfu / 2) < 1e-12
    assert abs(compute_mfu(f, 1e6, "h100", 1, compat=True) - 6 * f * 1e6 / 989e12) < 1e-12
    lg = MetricsLogger(TrainConfig(), TINY)
    d = lg.log(10, {"loss": 1.0, "grad_norm": 2.0, "lr": 1e-3}, 1000)
    assert d["tokens_per_sec"] > 0
    lg.log_val(10, 1.5)


def test_checkpoint_roundtrip(tmp_path):
    tc, st = _state(seed=1, checkpoint_dir=str(tmp_path / "ck"), max_checkpoints_to_keep=2, save_interval=5)
    batch = _batch()
    for _ in range(3):
        st, _ = train_step(st, batch)
    mgr = CheckpointManager(tc, TINY)
    assert mgr.latest_step() is None and mgr.should_save(10) and not mgr.should_save(7)
    mgr.save(42, st, data_state={"cursor": 7})
    mgr.wait_until_finished()
    assert mgr.latest_step() == 42
    _, other = _state(seed=2)
    other = mgr.restore(None, other)
    assert other.step == 42 and other.opt_state.count == st.opt_state.count
    for k in st.model.params:
        assert torch.equal(other.model.params[k], st.model.params[k])
        assert torch.equal(other.opt_state.mu[k], st.opt_state.mu[k])
    assert mgr.last_manifest["data_state"] == {"cursor": 7}
    # same next step from the restored state
    st, m1 = train_step(st, batch)
    other, m2 = train_step(other, batch)
    assert abs(float(m1["loss"]) - float(m2["loss"])) < 1e-6
    for s in (43, 44, 45):
        mgr.save(s, st)
    mgr.wait_until_finished()
    kept = sorted(int(n) for n in os.listdir(tmp_path / "ck"))
    assert kept == [44, 45]
    # an unfinished checkpoint (no manifest) is ignored
    os.makedirs(tmp_path / "ck" / "99")
    assert mgr.latest_step() == 45
    # the files are ordinary safetensors with the reference's key tree
    from safetensors.torch import load_file
    flat = load_file(str(tmp_path / "ck" / "45" / "params.safetensors"))
    assert flat["h.attn.c_attn.kernel"].shape == (2, 64, 192) and flat["lm_head.kernel"].shape == (64, 100)
    mgr.close()


def test_checkpoint_failed_write_leaves_no_manifest_and_keeps_the_older_step(tmp_path):
    """A checkpoint whose data file cannot be written must not look complete, and with keep = 1 the older,
    complete checkpoint must survive it."""
    tc, st = _state(seed=3, checkpoint_dir=str(tmp_path / "ck"), max_checkpoints_to_keep=1, save_interval=1)
    st, _ = train_step(st, _batch())
    mgr = CheckpointManager(tc, TINY)
    if mgr._writer is None:
        pytest.skip("native writer not built")
    mgr.save(1, st)
    mgr.wait_until_finished()
    assert mgr.latest_step() == 1
    # make params.safetensors of step 2 unwritable: its path is taken by a directory
    os.makedirs(tmp_path / "ck" / "2" / "params.safetensors.tmp")
    mgr.save(2, st)
    with pytest.raises(RuntimeError, match="checkpoint write failed"):
        mgr.wait_until_finished()
    assert not os.path.exists(tmp_path / "ck" / "2" / "manifest.json")
    assert mgr.latest_step() == 1 and os.path.exists(tmp_path / "ck" / "1" / "manifest.json")
    # the writer recovers: the next checkpoint is complete and only then is step 1 pruned
    mgr.save(3, st)
    mgr.wait_until_finished()
    assert mgr.latest_step() == 3 and not os.path.exists(tmp_path / "ck" / "1")
    mgr.close()


def test_checkpoint_save_refreshes_sharded_state_and_only_rank0_writes(tmp_path):
    """With a sharded optimizer the manager itself gathers weights and moments (a collective on every rank)
    instead of writing the snapshot taken when the state was created."""
    tc, st = _state(seed=4, checkpoint_dir=str(tmp_path / "ck"), max_checkpoints_to_keep=2, save_interval=1)
    fresh = {k: v.detach().clone() + 1.0 for k, v in st.model.params.items()}
    calls = []

    class FakeEngine:
        def __init__(self, rank):
            self.dist_optimizer = type("D", (), {"rank": rank})()

        def params(self):
            calls.append("params")
            for k in st.model.params:
                st.model.params[k].data.copy_(fresh[k])      # what gather_master does: refresh in place
            return st.model.params

        def opt_state(self):
            calls.append("opt_state")
            return {"count": 5, "mu": {k: torch.full_like(v, 0.25) for k, v in fresh.items()},
                    "nu": {k: torch.full_like(v, 0.5) for k, v in fresh.items()}}

    mgr = CheckpointManager(tc, TINY)
    st.engine = FakeEngine(rank=1)
    mgr.save(7, st)
    mgr.wait_until_finished()
    assert calls == ["params", "opt_state"] and mgr.latest_step() is None      # took part, wrote nothing
    st.engine = FakeEngine(rank=0)
    mgr.save(7, st)
    mgr.wait_until_finished()
    from safetensors.torch import load_file
    flat = load_file(str(tmp_path / "ck" / "7" / "params.safetensors"))
    opt = load_file(str(tmp_path / "ck" / "7" / "opt_state.safetensors"))
    k = "h.attn.c_attn.kernel"
    assert torch.equal(flat[k], fresh[k]) and float(opt["mu." + k].mean()) == 0.25 and float(opt["nu." + k].mean()) == 0.5
    mgr.close()


@pytest.mark.parametrize("native", [True, False])
def test_data_pipeline(tmp_path, native):
    write_synthetic(str(tmp_path), 20000, vocab_size=1000, seed=0)
    tc = TrainConfig(local_data_path=str(tmp_path), micro_batch_size=4, seq_len=32)
    p = DataPipeline(tc, "train", use_native=native)
    x, y = p.get_batch()
    assert x.shape == (4, 32) and y.shape == (4, 32) and x.dtype == torch.int32
    assert torch.equal(x[:, 1:], y[:, :-1])
    raw = np.fromfile(tmp_path / "train.bin", dtype=np.uint16)
    assert x[1, 0].item() == raw[32] and y[0, -1].item() == raw[32]
    a = DataPipeline(tc, "train", _shard_index=0, _shard_count=2, use_native=native)
    b = DataPipeline(tc, "train", _shard_index=1, _shard_count=2, use_native=native)
    xa, _ = a.get_batch()
    xb, _ = b.get_batch()
    assert not torch.equal(xa, xb) and xb[0, 0].item() == raw[32]
    # O(1) resume: skipping to step 3 equals reading three batches
    q = DataPipeline(tc, "train", use_native=native)
    for _ in range(3):
        q.get_batch()
    want, _ = q.get_batch()
    r = DataPipeline(tc, "train", use_native=native)
    r.skip_to_step(3, 1)
    got, _ = r.get_batch()
    assert torch.equal(want, got)
    for d in (p, a, b, q, r):
        d.close()


def test_tokenizer_cli_paths(tmp_path):
    (tmp_path / "docs").mkdir()
    (tmp_path / "docs" / "a.txt").write_text("hello world " * 50)
    (tmp_path / "docs" / "b.txt").write_text("second document " * 50)
    train, val = tokenize(str(tmp_path / "docs"), 0.1)
    assert train.dtype == np.uint16 and len(val) >= 1 and (np.concatenate([val, train]) == 50256).sum() == 2
    with open(tmp_path / "c.jsonl", "w") as f:
        f.write(json.dumps({"text": "one"}) + "\n" + json.dumps({"text": "two"}) + "\n")
    t2, v2 = tokenize(str(tmp_path / "c.jsonl"), 0.5)
    assert len(t2) + len(v2) >= 4


def test_config_overrides():
    cfg, rest = apply_overrides(TrainConfig(), ["--max_steps=7", "--learning_rate", "0.5", "--log_to_wandb", "--foo", "1"])
    assert cfg.max_steps == 7 and cfg.learning_rate == 0.5 and cfg.log_to_wandb is True and rest == ["--foo", "1"]


def test_data_pipeline_gcs_source_reads_the_mounted_bucket(tmp_path, monkeypatch):
    """data_source='gcs' resolves gs://bucket/path/split to the bucket's mount and yields the same windows as the local
    source; without the mount the error names what was looked for."""
    import numpy as np
    from jax_gpt_b200.trainer.config import TrainConfig
    toks = (np.arange(4 * 65 + 1) % 50000).astype(np.uint16)
    d = tmp_path / "mnt" / "my-bucket" / "datasets" / "owt"
    d.mkdir(parents=True)
    toks.tofile(d / "train.bin")
    (tmp_path / "local").mkdir()
    toks.tofile(tmp_path / "local" / "train.bin")
    monkeypatch.setenv("B200_GCS_MOUNT", str(tmp_path / "mnt"))
    g = DataPipeline(TrainConfig(data_source="gcs", gcs_bucket="my-bucket", gcs_dataset_path="datasets/owt", seq_len=64,
                                 micro_batch_size=2), "train", use_native=False)
    l = DataPipeline(TrainConfig(data_source="local", local_data_path=str(tmp_path / "local"), seq_len=64,
                                 micro_batch_size=2), "train", use_native=False)
    (gx, gy), (lx, ly) = g.get_batch(), l.get_batch()
    assert torch.equal(gx, lx) and torch.equal(gy, ly)
    with pytest.raises(FileNotFoundError, match="B200_GCS_MOUNT"):
        DataPipeline(TrainConfig(data_source="gcs", gcs_bucket="other", gcs_dataset_path="x", seq_len=64,
                                 micro_batch_size=2), "val", use_native=False)
    with pytest.raises(ValueError):
        DataPipeline(TrainConfig(data_source="s3", seq_len=64, micro_batch_size=2), "train", use_native=False)
