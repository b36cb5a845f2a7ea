"""Pipeline schedule and failure detection on CPU (gloo) ranks."""
import os
import tempfile
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from jax_gpt_b200.parallel.pipeline import one_f_one_b_order, split_layers


def test_schedule_shapes():
    assert [list(r) for r in split_layers(10, 4)] == [[0, 1, 2], [3, 4, 5], [6, 7], [8, 9]]
    for S, M in [(4, 8), (2, 3), (3, 1)]:
        for s in range(S):
            order = one_f_one_b_order(s, S, M)
            assert [i for k, i in order if k == "F"] == list(range(M)) and [i for k, i in order if k == "B"] == list(range(M))
            done = set()
            live = 0
            for k, i in order:      # a backward never precedes its forward; at most S - s in flight
                if k == "F":
                    done.add(i); live += 1
                else:
                    assert i in done; live -= 1
                assert live <= S - s
    assert one_f_one_b_order(0, 4, 8)[:4] == [("F", 0), ("F", 1), ("F", 2), ("F", 3)]


def _pp_worker(rank, world, path):
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
    from jax_gpt_b200.parallel.pipeline import PipelineStage
    torch.manual_seed(0)
    D, n_layers, n_micro, B = 16, 4, 4, 3
    Ws = [torch.randn(D, D) * 0.3 for _ in range(n_layers)]     # same weights on every rank
    xs = [torch.randn(B, D) for _ in range(n_micro)]
    ys = [torch.randn(B, D) for _ in range(n_micro)]
    mine = split_layers(n_layers, world)[rank]
    params = [Ws[i].clone().requires_grad_(True) for i in mine]

    def fwd(inp, i):
        x, tgt = (inp, None)
        if rank == world - 1:
            x, tgt = inp if world > 1 else (inp[0], inp[1])
        for w in params:
            x = torch.tanh(x @ w)
        return ((x - tgt) ** 2).mean() if tgt is not None else x

    stage = PipelineStage(fwd, params, (B, D), torch.float32)
    inputs = xs if rank == 0 else (ys if rank == world - 1 else [None] * n_micro)
    loss = stage.run(inputs)
    # single-process reference
    ref_params = [w.clone().requires_grad_(True) for w in Ws]
    tot = 0
    for x, y in zip(xs, ys):
        h = x
        for w in ref_params:
            h = torch.tanh(h @ w)
        tot = tot + ((h - y) ** 2).mean() / n_micro
    tot.backward()
    for j, i in enumerate(mine):
        assert torch.allclose(params[j].grad, ref_params[i].grad, atol=1e-6), (rank, i)
    if rank == world - 1:
        assert abs(float(loss) - float(tot)) < 1e-6
    dist.destroy_process_group()


def test_pipeline_1f1b_matches_single_process():
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_pp_worker, args=(2, os.path.join(d, "rdv")), nprocs=2, join=True)


def _pp_gpt2_worker(rank, world, path):
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
    from jax_gpt_b200.models.gpt2 import GPT, GPTConfig
    from jax_gpt_b200.parallel.pipeline import gpt2_stage, sync_tied_embedding_grad
    cfg = GPTConfig(d_model=32, d_head=16, d_ff=64, d_context=16, n_head=2, n_kv_head=2, n_layers=4, vocab_size=64)
    model, ref = GPT(cfg, seed=9), GPT(cfg, seed=9)
    for m in (model, ref):
        m.requires_grad_(True)
    g = torch.Generator().manual_seed(3)
    toks = [torch.randint(0, 64, (2, 17), generator=g) for _ in range(4)]
    stage = gpt2_stage(model, rank, world, 2, 16)
    inputs = [t[:, :-1] for t in toks] if rank == 0 else ([t[:, 1:] for t in toks] if rank == world - 1 else [None] * 4)
    loss = stage.run(inputs)
    sync_tied_embedding_grad(model)
    tot = 0.0
    for t in toks:
        part = torch.nn.functional.cross_entropy(ref(t[:, :-1])[0].reshape(-1, 64), t[:, 1:].reshape(-1)) / 4
        part.backward()
        tot += float(part.detach())
    mine = split_layers(cfg.n_layers, world)[rank]
    for k, v in model.params.items():
        if k.startswith("h."):
            assert torch.allclose(v.grad[mine.start:mine.stop], ref.params[k].grad[mine.start:mine.stop], atol=1e-6), k
    assert torch.allclose(model.params["wte.embedding"].grad, ref.params["wte.embedding"].grad, atol=1e-6)
    if rank == world - 1:
        assert abs(float(loss) - tot) < 1e-5
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_pipeline_gpt2_stages_match_single_process(world):
    """GPT-2 cut into pipeline stages (embeddings first, tied head and loss last): block gradients per stage and the
    tied embedding gradient after its cross-stage sum equal one process."""
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_pp_gpt2_worker, args=(world, os.path.join(d, "rdv")), nprocs=world, join=True)


def _wd_worker(rank, world, path, result_path):
    from jax_gpt_b200.utils.watchdog import PeerFailure, Watchdog
    store = dist.FileStore(path, world)
    wd = Watchdog(store, rank, world, interval=0.1, timeout=1.0, startup_grace=60.0).start()
    # every rank waits until it has seen the first beat of all the others (start-up skew is not a failure)
    t0 = time.time()
    while time.time() - t0 < 50 and len(wd.peers_seen()) < world - 1:
        time.sleep(0.05)
    store.set(f"ready/{rank}", "1")
    store.wait([f"ready/{r}" for r in range(world)])
    if rank == 1:
        os._exit(0)          # this rank dies between steps, without saying goodbye
    if rank == 3:
        wd.stop()            # this one finishes cleanly: not a failure
        with open(f"{result_path}.{rank}", "w") as f:
            f.write("done")
        return
    t0 = time.time()
    seen = None
    while time.time() - t0 < 20:
        try:
            wd.check()
        except PeerFailure as e:
            seen = e.dead
            break
        time.sleep(0.05)
    with open(f"{result_path}.{rank}", "w") as f:
        f.write(repr(seen))
    wd.stop()


def test_watchdog_detects_a_dead_rank():
    """Four ranks: 1 dies silently after everyone has seen everyone, 3 stops cleanly; 0 and 2 must report [1] only."""
    with tempfile.TemporaryDirectory() as d:
        ctx = mp.spawn(_wd_worker, args=(4, os.path.join(d, "store"), os.path.join(d, "res")), nprocs=4, join=False)
        t0 = time.time()
        while time.time() - t0 < 90 and not all(os.path.exists(os.path.join(d, f"res.{r}")) for r in (0, 2)):
            time.sleep(0.1)
        for r in (0, 2):
            assert open(os.path.join(d, f"res.{r}")).read() == "[1]"
        for p in ctx.processes:
            p.join(timeout=5)


def test_watchdog_start_up_skew_is_not_a_failure():
    """A peer that has not beaten yet is covered by the start-up grace, not by the beat timeout."""
    from jax_gpt_b200.utils.watchdog import Watchdog
    with tempfile.TemporaryDirectory() as d:
        store = dist.FileStore(os.path.join(d, "s"), 2)
        wd = Watchdog(store, 0, 2, interval=0.05, timeout=0.2, startup_grace=30.0).start()
        time.sleep(0.8)                      # four timeouts long, rank 1 still silent
        wd.check()
        assert wd.dead_ranks == [] and wd.peers_seen() == []
        late = Watchdog(store, 1, 2, interval=0.05, timeout=0.2, startup_grace=30.0).start()
        time.sleep(0.3)
        assert wd.peers_seen() == [1]
        late.stop()                          # clean exit
        time.sleep(0.6)
        wd.check()
        wd.stop()


def _vce_worker(rank, world, path):
    from jax_gpt_b200.parallel.tensor_parallel import vocab_parallel_ce_reference
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(0)
    M, V = 33, 64
    logits = torch.randn(M, V, generator=g) * 3
    targets = torch.randint(0, V, (M,), generator=g)
    targets[4] = -1
    vl = V // world
    loss, grad = vocab_parallel_ce_reference(logits[:, rank * vl:(rank + 1) * vl].clone(), targets, rank * vl)
    lf = logits.clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lf, targets, ignore_index=-1, reduction="none")
    ref.sum().backward()
    assert torch.allclose(loss, ref, atol=1e-5)
    assert torch.allclose(grad, lf.grad[:, rank * vl:(rank + 1) * vl], atol=1e-5)
    dist.destroy_process_group()


def test_vocab_parallel_cross_entropy_protocol_on_cpu_ranks():
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_vce_worker, args=(2, os.path.join(d, "rdv")), nprocs=2, join=True)


def test_train_script_pipeline_parallel_matches_single_process(tmp_path):
    """``scripts/train.py --pp=2`` (two gloo processes, 1F1B over four micro-batches) follows the same loss curve as
    the single-process run on the same data windows, seed and schedule."""
    import json
    import subprocess
    import sys
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
    common = ["--preset", "gpt2-tiny", "--synthetic", "--synthetic_tokens=60000", "--max_steps=4", "--micro_batch_size=2",
              "--seq_len=32", "--grad_accum_steps=4", "--log_interval=1", "--learning_rate=1e-3", "--warmup_steps=0",
              "--eval_interval=0", "--save_interval=0", f"--local_data_path={tmp_path}/data"]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MASTER_ADDR="127.0.0.1")
    one = subprocess.run([sys.executable, os.path.join(root, "scripts", "train.py"), *common, f"--jsonl={tmp_path}/one.jsonl",
                          f"--checkpoint_dir={tmp_path}/ck1"], env=env, capture_output=True, text=True, timeout=600)
    assert one.returncode == 0, one.stdout[-2000:] + one.stderr[-2000:]
    two = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29841", os.path.join(root, "scripts", "train.py"),
                          *common, "--pp=2", f"--jsonl={tmp_path}/two.jsonl"], env=env, capture_output=True, text=True,
                         timeout=600)
    assert two.returncode == 0, two.stdout[-2000:] + two.stderr[-2000:]
    read = lambda p: [json.loads(l) for l in open(p) if l.strip()]
    a, b = read(f"{tmp_path}/one.jsonl"), read(f"{tmp_path}/two.jsonl")
    la = [r["loss"] for r in a if "loss" in r]
    lb = [r["loss"] for r in b if "loss" in r]
    assert len(la) == len(lb) == 4
    assert max(abs(x - y) for x, y in zip(la, lb)) < 2e-3, (la, lb)
