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
