"""Helpers shared by the command-line scripts: model presets, distributed set-up, tokenisers."""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def init_distributed():
    """One process per GPU under torchrun; returns (rank, world, device). Single process otherwise."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
    else:
        device = torch.device("cpu")
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if device.type == "cuda":
            dist.init_process_group("nccl", device_id=device)
        else:
            dist.init_process_group("gloo")
    return rank, world, device


def make_tp_dp_groups(tp: int, dp: int):
    """Splits the default group into ``dp`` replicas of ``tp`` consecutive ranks. Returns
    (tp_group | None, tp_rank, dp_rank). Every rank has to call it (new_group is collective)."""
    import torch.distributed as dist
    world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    if tp * dp != world:
        raise SystemExit(f"--tp {tp} x --dp {dp} must equal the number of processes ({world}); launch with torchrun "
                         f"--nproc-per-node {tp * dp}")
    if world == 1:
        return None, 0, 0
    rank = dist.get_rank()
    mine = None
    for r in range(dp):
        g = dist.new_group(list(range(r * tp, (r + 1) * tp)))
        if rank // tp == r:
            mine = g
    return (mine if tp > 1 else None), rank % tp, rank // tp


def load_hf_dir(model_dir: str):
    """All ``*.safetensors`` shards of a Hugging Face directory as one lazy name -> tensor mapping."""
    import glob
    from safetensors import safe_open
    files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not files:
        raise SystemExit(f"no *.safetensors files in {model_dir}")

    class _Lazy(dict):
        def __init__(self):
            super().__init__()
            self._where = {}
            self._open = {}
            for f in files:
                h = safe_open(f, framework="pt", device="cpu")
                self._open[f] = h
                for k in h.keys():
                    self._where[k] = f

        def __contains__(self, k):
            return k in self._where

        def keys(self):
            return self._where.keys()

        def __iter__(self):
            return iter(self._where)

        def __len__(self):
            return len(self._where)

        def __getitem__(self, k):
            return self._open[self._where[k]].get_tensor(k)
    return _Lazy()


def fake_quant_w8a8(params):
    """The reference's "W8A8" benchmark mode (scripts/bench_prefill_decode.py:84-102 there): every weight matrix
    is rounded through fp8 e4m3 with ONE scale per tensor and stored back in its own dtype, so the run measures
    the accuracy of 8-bit weights at the speed of the unquantised kernels."""
    from jax_gpt_b200.models.qwen35.sharding import tree_map

    def q(t):
        if not torch.is_tensor(t) or t.dim() < 2 or not t.is_floating_point():
            return t
        scale = t.abs().max().float().clamp_min(1e-12) / 448.0
        return ((t.float() / scale).to(torch.float8_e4m3fn).float() * scale).to(t.dtype)
    return tree_map(q, params)


def gpt_config(preset: str):
    from jax_gpt_b200.models.gpt2 import GPTConfig
    if preset == "gpt2-tiny":
        return GPTConfig(d_model=128, d_head=64, d_ff=512, d_context=256, n_head=2, n_kv_head=2, n_layers=2, vocab_size=50257)
    return GPTConfig.from_model_type(preset)


def qwen_config(name: str):
    from jax_gpt_b200.models.qwen35 import Qwen35Config
    return {"mini": Qwen35Config.mini, "mid": Qwen35Config.mid, "mid_large": Qwen35Config.mid_large,
            "full": Qwen35Config.full, "ns": Qwen35Config.ns, "tiny": Qwen35Config.tiny}[name]()


class ByteTokenizer:
    """Fallback when the GPT-2 BPE vocabulary is not available offline."""
    eot = 50256

    def encode(self, text):
        return list(text.encode("utf-8"))

    def decode(self, ids):
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", errors="replace")


def get_tokenizer():
    try:
        import tiktoken
        enc = tiktoken.get_encoding("gpt2")
        enc.encode_ordinary("probe")

        class _T:
            eot = 50256
            encode = staticmethod(enc.encode_ordinary)
            decode = staticmethod(enc.decode)
        return _T()
    except Exception:
        return ByteTokenizer()
