"""Context-parallel (zig-zag) causal attention on gloo ranks against dense attention on one process."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, path, H, Hkv):
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world)
    from jax_gpt_b200.ops.attention import attention_ref
    from jax_gpt_b200.parallel.context_parallel import context_parallel_attention, zigzag_merge, zigzag_split
    g = torch.Generator().manual_seed(5)
    B, T, D = 2, 24 * world, 16
    q = torch.randn(B, T, H, D, generator=g)
    k = torch.randn(B, T, Hkv, D, generator=g)
    v = torch.randn(B, T, Hkv, D, generator=g)
    w = torch.randn(B, T, H, D, generator=g)
    # dense reference with gradients
    qr, kr, vr = [t.clone().requires_grad_() for t in (q, k, v)]
    ref = attention_ref(qr, kr, vr, causal=True)
    (ref * w).sum().backward()
    # sharded
    ql, kl, vl = [zigzag_split(t, world, rank).clone().requires_grad_() for t in (q, k, v)]
    out = context_parallel_attention(ql, kl, vl)
    (out * zigzag_split(w, world, rank)).sum().backward()
    err = lambda a, b: float((a - b).abs().max())
    assert err(out, zigzag_split(ref, world, rank)) < 1e-5
    assert err(ql.grad, zigzag_split(qr.grad, world, rank)) < 1e-5
    assert err(kl.grad, zigzag_split(kr.grad, world, rank)) < 1e-5
    assert err(vl.grad, zigzag_split(vr.grad, world, rank)) < 1e-5
    # the merge helper inverts the split
    parts = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(parts, out.detach())
    assert err(zigzag_merge(parts), ref.detach()) < 1e-5
    dist.destroy_process_group()


@pytest.mark.parametrize("world,H,Hkv", [(2, 4, 4), (3, 4, 2)])
def test_context_parallel_attention_matches_dense(world, H, Hkv):
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(world, os.path.join(d, "rdv"), H, Hkv), nprocs=world, join=True)
