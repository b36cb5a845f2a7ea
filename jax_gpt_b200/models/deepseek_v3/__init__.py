from .config import DeepSeekV3Config
from .model import forward, generate, init_params, load_from_hf_state_dict, make_cache

__all__ = ["DeepSeekV3Config", "init_params", "forward", "generate", "make_cache", "load_from_hf_state_dict"]
