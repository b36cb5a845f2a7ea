from .config import TrainConfig, apply_overrides
from .metrics import HARDWARE_PEAK_TFLOPS, MetricsLogger, compute_mfu, compute_model_flops
from .optimizer import AdamW, AdamWState, build_decay_mask, create_optimizer
from .train_state import TrainState, create_train_state
from .train_step import eval_step, jitted_eval_step, train_step, train_step_with_accumulation

__all__ = [
    "TrainConfig", "apply_overrides", "HARDWARE_PEAK_TFLOPS", "MetricsLogger", "compute_mfu", "compute_model_flops",
    "AdamW", "AdamWState", "build_decay_mask", "create_optimizer", "TrainState", "create_train_state", "eval_step",
    "jitted_eval_step", "train_step", "train_step_with_accumulation",
]
