"""GPT-2 configuration (field names and presets of jax_gpt/models/gpt2/config.py:5-35)."""
from __future__ import annotations

from dataclasses import dataclass, replace


@dataclass
class GPTConfig:
    d_model: int = 768
    d_head: int = 64
    d_ff: int = 3072
    d_context: int = 1024
    n_head: int = 12
    n_kv_head: int = 12
    n_layers: int = 12
    vocab_size: int = 50257
    use_bias: bool = True
    dropout: float = 0.0

    @classmethod
    def from_model_type(cls, model_type: str, **override) -> "GPTConfig":
        """Presets gpt2 / gpt2-medium / gpt2-large / gpt2-xl; d_ff = 4 d_model, d_head = d_model / n_head."""
        table = {
            "gpt2": dict(n_layers=12, n_head=12, d_model=768),
            "gpt2-medium": dict(n_layers=24, n_head=16, d_model=1024),
            "gpt2-large": dict(n_layers=36, n_head=20, d_model=1280),
            "gpt2-xl": dict(n_layers=48, n_head=25, d_model=1600),
        }
        if model_type not in table:
            raise ValueError(f"unknown model type {model_type!r}; choose from {sorted(table)}")
        base = dict(table[model_type])
        base.update(override)
        base.setdefault("n_kv_head", base["n_head"])
        base.setdefault("d_ff", 4 * base["d_model"])
        base.setdefault("d_head", base["d_model"] // base["n_head"])
        return cls(**base)

    def replace(self, **kw) -> "GPTConfig":
        return replace(self, **kw)

    @property
    def padded_vocab(self) -> int:
        """Vocabulary rounded up to a multiple of 64 (row stride of the logits buffer)."""
        return (self.vocab_size + 63) // 64 * 64
