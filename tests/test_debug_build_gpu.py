"""The range-checked build (``-DB200_DEBUG``) runs valid workloads without reporting a violation.

Only in-range inputs are used: the point is that the checks compile into the indexed paths (routing slots,
source ranks, page ids) and stay silent on correct programs."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_PROG = r"""
import torch
from jax_gpt_b200 import _ext
assert _ext.DEBUG and _ext.LIB_PATH.endswith("_C_debug.so")
from jax_gpt_b200.cache.paged import PagedCache
from jax_gpt_b200.ops.mla_decode import mla_paged_decode, mla_paged_decode_ref
dev = torch.device("cuda", 0)
cache = PagedCache(1, 576, n_pages=16, page_size=64, max_seqs=4, max_pages_per_seq=8, device=dev)
for sid, n in ((1, 70), (3, 300)):
    cache.append(0, [sid], torch.randn(1, n, 576, device=dev).to(torch.bfloat16), commit=True)
q = (torch.randn(2, 16, 576, device=dev) * 0.3).to(torch.bfloat16)
out = mla_paged_decode(q, cache, 0, [1, 3], 192 ** -0.5)
ref = mla_paged_decode_ref(q, cache, 0, [1, 3], 192 ** -0.5, 512)
assert (out.float() - ref.float()).abs().max() < 3e-2
import os, torch.distributed as dist
os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29541")
dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
from jax_gpt_b200.comm.symm import Communicator
from jax_gpt_b200.parallel.expert_parallel import FusedEPMoE
from jax_gpt_b200.models.qwen35.moe import expert_forward_single
T, D, I, E, k = 256, 512, 256, 8, 2
g = torch.Generator(device=dev).manual_seed(0)
p = {n: (torch.randn(E, a, b, device=dev, generator=g) * 0.05).to(torch.bfloat16)
     for n, (a, b) in (("gate_proj", (D, I)), ("up_proj", (D, I)), ("down_proj", (I, D)))}
x = torch.randn(T, D, device=dev, generator=g).to(torch.bfloat16)
w, idx = torch.softmax(torch.randn(T, E, device=dev, generator=g), -1).topk(k, -1)
layer = FusedEPMoE(Communicator(device=dev, wait_seconds=5.0), T, D, I, E, k, training=True)
out = layer.forward(x, w, idx, p).clone()
grads = {n: torch.zeros_like(t, dtype=torch.float32) for n, t in p.items()}
layer.backward(x, torch.randn_like(x), w, idx, p, grads)
torch.cuda.synchronize()
_ext.check_status(dev)          # raises on any recorded violation or timeout
ref = expert_forward_single(x.float(), w, idx, {n: t.float() for n, t in p.items()})
assert ((out - ref).norm() / ref.norm()) < 2e-2
print("debug build ok")
"""


def test_range_checked_build_is_silent_on_valid_programs():
    if not os.path.exists(os.path.join(ROOT, "jax_gpt_b200", "_C_debug.so")):
        from jax_gpt_b200 import build as b
        b.build(debug=True)
    env = dict(os.environ, B200_DEBUG="1", NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-c", _PROG], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "debug build ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
