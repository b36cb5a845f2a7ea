"""Host-side sharding logic of the sharded optimizer on CPU (gloo) ranks."""
import os
import tempfile

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, path, n, n_decay):
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
    from jax_gpt_b200.ops import misc
    from jax_gpt_b200.parallel.fsdp import shard_range, sharded_adamw_reference
    torch.manual_seed(0)
    p0 = torch.randn(n)
    grads = [torch.randn(n, generator=torch.Generator().manual_seed(10 + r)) for r in range(world)]
    lo, hi = shard_range(n, world, rank)
    master = p0[lo:hi].clone()
    m = torch.zeros(hi - lo)
    v = torch.zeros(hi - lo)
    compute = p0.clone()
    hp = [1e-2, 1 - 0.9, 1 - 0.95, 1.0 / world]
    sq = sharded_adamw_reference(dist.group.WORLD, grads[rank].clone(), master, m, v, compute, hp, n_decay, 0.9, 0.95,
                                 1e-8, 0.1, 1.0)
    # single-process answer on the summed gradient
    g = sum(grads)
    pr, mr, vr = p0.clone(), torch.zeros(n), torch.zeros(n)
    ss = (g.double() ** 2).sum().float()
    misc.adamw_ref(pr[:n_decay], g[:n_decay].clone(), mr[:n_decay], vr[:n_decay], hp, ss, 0.9, 0.95, 1e-8, 0.1, 1.0,
                   zero_grad=False)
    misc.adamw_ref(pr[n_decay:], g[n_decay:].clone(), mr[n_decay:], vr[n_decay:], hp, ss, 0.9, 0.95, 1e-8, 0.0, 1.0,
                   zero_grad=False)
    assert torch.allclose(compute, pr, atol=1e-6), (compute - pr).abs().max()
    assert torch.allclose(master, pr[lo:hi], atol=1e-6)
    assert abs(float(sq) - float(ss)) / float(ss) < 1e-5
    dist.destroy_process_group()


def test_sharded_adamw_reference_matches_single_process():
    world, n, n_decay = 2, 4096, 2560
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(world, os.path.join(d, "rdv"), n, n_decay), nprocs=world, join=True)
