from .config import GPTConfig
from .model import GPT, KVCache, init_params, param_shapes, sample_logits

__all__ = ["GPTConfig", "GPT", "KVCache", "init_params", "param_shapes", "sample_logits"]
