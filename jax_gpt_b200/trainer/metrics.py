"""Throughput / MFU metrics and the step logger (jax_gpt/trainer/metrics.py:9-113).

``compute_model_flops`` keeps the reference's estimate 2 * 12 * L * d^2 per token (forward).
``compute_mfu`` by default uses the conventional 3x forward FLOPs for a training step; the
reference multiplies by 6 (jax_gpt/trainer/metrics.py:40), reproducible with ``compat=True``.
"""
from __future__ import annotations

import json
import time

from ..models.gpt2.config import GPTConfig

HARDWARE_PEAK_TFLOPS = {
    "tpu_v3": 123e12, "tpu_v4": 275e12, "tpu_v5e": 393e12, "a100": 312e12, "h100": 989e12,
    "b200": 2250e12,  # dense bf16, nominal
    "cpu": 1e12,
}


def compute_model_flops(config: GPTConfig) -> int:
    return 2 * 12 * config.n_layers * config.d_model ** 2


def compute_mfu(flops_per_token: int, tokens_per_second: float, hardware: str, num_devices: int,
                compat: bool = False) -> float:
    peak = HARDWARE_PEAK_TFLOPS.get(hardware, HARDWARE_PEAK_TFLOPS["cpu"])
    mult = 6 if compat else 3
    return mult * flops_per_token * tokens_per_second / (peak * num_devices)


def _world():
    try:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            return dist.get_rank(), dist.get_world_size()
    except Exception:
        pass
    return 0, 1


class MetricsLogger:
    """Prints ``step | loss | lr | gnorm | tok/s | tok/s/chip | TFLOPs/chip | MFU`` on rank 0,
    optionally mirrors to wandb and to a JSONL file."""

    def __init__(self, config, model_config, jsonl_path: str = "", num_devices: int = 0):
        self._flops_per_token = compute_model_flops(model_config)
        self._config = config
        self._last_time = time.monotonic()
        self._last_step = 0
        self._wandb = None
        self._jsonl = open(jsonl_path, "a") if jsonl_path else None
        self._num_devices = num_devices
        if config.log_to_wandb:
            import wandb
            self._wandb = wandb.init(project=config.wandb_project, name=config.wandb_run_name or None, resume="allow")

    def log(self, step: int, metrics: dict, num_tokens_this_interval: int) -> dict:
        now = time.monotonic()
        dt = now - self._last_time
        rank, world = _world()
        ndev = self._num_devices or world
        tps = num_tokens_this_interval / dt if dt > 0 else 0.0
        mfu = compute_mfu(self._flops_per_token, tps, self._config.hardware, ndev)
        tflops = 3 * self._flops_per_token * tps / ndev / 1e12
        d = {
            "step": step, "loss": float(metrics.get("loss", float("nan"))),
            "grad_norm": float(metrics.get("grad_norm", float("nan"))), "lr": float(metrics.get("lr", float("nan"))),
            "tokens_per_sec": tps, "tokens_per_sec_per_device": tps / ndev, "mfu_pct": mfu * 100,
            "tflops_per_chip": tflops,
        }
        if rank == 0:
            print(f"step {step:6d} | loss {d['loss']:.4f} | lr {d['lr']:.2e} | gnorm {d['grad_norm']:.3f} | "
                  f"tok/s {tps:,.0f} | tok/s/chip {tps / ndev:,.0f} | TFLOPs/chip {tflops:.1f} | "
                  f"MFU {d['mfu_pct']:.1f}%", flush=True)
            if self._jsonl is not None:
                self._jsonl.write(json.dumps(d) + "\n")
                self._jsonl.flush()
        if self._wandb is not None:
            self._wandb.log({k: v for k, v in d.items() if k != "step"}, step=step)
        self._last_time, self._last_step = now, step
        return d

    def log_val(self, step: int, val_loss: float) -> None:
        rank, _ = _world()
        if rank == 0:
            print(f"step {step:6d} | val_loss {float(val_loss):.4f}", flush=True)
            if self._jsonl is not None:
                self._jsonl.write(json.dumps({"step": step, "val_loss": float(val_loss)}) + "\n")
                self._jsonl.flush()
        if self._wandb is not None:
            self._wandb.log({"val_loss": float(val_loss)}, step=step)
