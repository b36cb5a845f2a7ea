"""CUDA-graph decode engine of the Qwen3.5-style model against the function-style decode, on one GPU with the
fused expert kernel (a single-rank process group carries its symmetric buffers), run as a child process so that
the process group does not leak into the other tests."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_PROG = r"""
import os, torch, torch.distributed as dist
from jax_gpt_b200 import _ext
from jax_gpt_b200.comm.symm import Communicator
from jax_gpt_b200.models.qwen35 import Qwen35Config, forward, init_cache, init_params
from jax_gpt_b200.models.qwen35.decode_engine import Qwen35DecodeEngine
from jax_gpt_b200.models.qwen35.sharding import tree_map
from jax_gpt_b200.parallel.expert_parallel import EPMoEInferenceRuntime
dev = torch.device("cuda", 0)
os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29543")
dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
cfg = Qwen35Config(d_model=256, vocab_size=512, n_layers=8, max_position_embeddings=256, gqa_n_q_heads=4,
                   gqa_n_kv_heads=2, gqa_head_dim=64, delta_n_qk_heads=2, delta_n_v_heads=4, delta_qk_head_dim=64,
                   delta_v_head_dim=64, delta_chunk_size=16, n_routed_experts=32, n_experts_per_token=4,
                   moe_intermediate_size=128, shared_expert_intermediate_size=128)
params = tree_map(lambda t: t.to(dev).to(torch.bfloat16) if t.is_floating_point() else t.to(dev), init_params(cfg, 0))
ep = EPMoEInferenceRuntime(Communicator(device=dev, wait_seconds=5.0), cfg.d_model, cfg.moe_intermediate_size,
                           cfg.n_routed_experts, cfg.n_experts_per_token)
B, T, steps = 4, 40, 6
tok = torch.randint(0, cfg.vocab_size, (B, T), generator=torch.Generator().manual_seed(3)).to(dev)

def fresh_cache():
    c = init_cache(cfg, B, T + steps + 2, dtype=torch.float32, device=dev)
    c.gqa_k, c.gqa_v = c.gqa_k.to(torch.bfloat16), c.gqa_v.to(torch.bfloat16)
    return c

from jax_gpt_b200.models.qwen35.cache import HybridCache

def rows_close(a, b, tol):
    a, b = a.float(), b.float()
    err = (a - b).norm(dim=-1) / b.norm(dim=-1)
    return (err < tol).float().mean().item()

with torch.no_grad():
    logits, _ = forward(params, tok, cfg, cache=fresh_cache(), ep_group=ep)
    _, cache_b = forward(params, tok, cfg, cache=fresh_cache(), ep_group=ep)
    _, cache_c = forward(params, tok, cfg, cache=fresh_cache(), ep_group=ep)
    graph_eng = Qwen35DecodeEngine(params, cfg, cache_b, ep=ep, use_cuda_graph=True)
    eager_eng = Qwen35DecodeEngine(params, cfg, cache_c, ep=ep, use_cuda_graph=False)
    assert graph_eng.use_graph
    nxt = logits[:, -1].argmax(-1)
    for s in range(steps):
        # every step starts from the graph engine's state in all three paths, so that a step is compared and not
        # the drift of three bf16 trajectories (a near-tie in a router flips an expert and changes a whole row)
        ref_cache = HybridCache(graph_eng.M.clone(), graph_eng.conv.clone(), graph_eng.k.clone(), graph_eng.v.clone(),
                                graph_eng.pos)
        for dst, src in ((eager_eng.M, graph_eng.M), (eager_eng.conv, graph_eng.conv), (eager_eng.k, graph_eng.k),
                         (eager_eng.v, graph_eng.v), (eager_eng.pos_t, graph_eng.pos_t)):
            dst.copy_(src)
        ref, ref_cache = forward(params, nxt[:, None], cfg, cache=ref_cache, is_decode=True, ep_group=ep)
        eager_eng.step(nxt)
        graph_eng.step(nxt)
        # the graph replays the eager engine's kernels (only the fp32 atomics of the expert combine may reorder)
        assert rows_close(graph_eng.logits, eager_eng.logits, 1e-2) >= 0.75, (s, "graph vs eager engine")
        assert rows_close(graph_eng.logits, ref[:, -1], 3e-2) >= 0.75, (s, "engine vs function-style decode")
        assert rows_close(graph_eng.M, ref_cache.delta_M, 2e-2) >= 0.9, (s, "recurrent state")
        nxt = graph_eng.next_tokens.clone()
    assert graph_eng.pos == eager_eng.pos == T + steps and int(graph_eng.pos_t) == T + steps
    # the same engine with the gated-attention keys / values in a paged cache, captured in a graph as well: every
    # step starts from the dense graph engine's recurrent state and is compared with it
    _, cache_d = forward(params, tok, cfg, cache=fresh_cache(), ep_group=ep)
    _, cache_e = forward(params, tok, cfg, cache=fresh_cache(), ep_group=ep)
    dense_eng = Qwen35DecodeEngine(params, cfg, cache_d, ep=ep, use_cuda_graph=True)
    paged_eng = Qwen35DecodeEngine(params, cfg, cache_e, ep=ep, use_cuda_graph=True, paged_kv=True)
    nxt = logits[:, -1].argmax(-1)
    for s in range(steps):
        paged_eng.M.copy_(dense_eng.M)
        paged_eng.conv.copy_(dense_eng.conv)
        dense_eng.step(nxt)
        paged_eng.step(nxt)
        assert rows_close(paged_eng.logits, dense_eng.logits, 1e-2) >= 0.75, (s, "paged vs dense engine")
        nxt = dense_eng.next_tokens.clone()
    assert int(paged_eng.paged_lens[0]) == T + steps
worst = 0.0
torch.cuda.synchronize()
_ext.check_status(dev)
print("qwen engine ok", worst)
dist.destroy_process_group()
"""


def test_qwen35_graph_decode_engine_matches_function_style_decode():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-c", _PROG], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "qwen engine ok" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
