from .cache import HybridCache, init_cache
from .config import Qwen35Config
from .model import forward, generate, init_params

__all__ = ["Qwen35Config", "HybridCache", "init_cache", "init_params", "forward", "generate"]
