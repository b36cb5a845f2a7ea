"""``CheckpointManager`` at the reference's import path (jax_gpt/trainer/checkpointing.py)."""
from ..ckpt.manager import CheckpointManager

__all__ = ["CheckpointManager"]
