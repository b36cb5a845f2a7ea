"""Training configuration: the reference's fields (jax_gpt/trainer/config.py:4-58) plus the
knobs this runtime consumes (``cuda_graph``, ``hardware='b200'``)."""
from __future__ import annotations

from dataclasses import dataclass, fields, replace


@dataclass
class TrainConfig:
    # batch & sequence
    global_batch_tokens: int = 524288
    micro_batch_size: int = 16
    seq_len: int = 1024
    grad_accum_steps: int = 1
    # optimizer
    learning_rate: float = 6e-4
    min_lr: float = 6e-5
    warmup_steps: int = 2000
    lr_decay_steps: int = 600000
    weight_decay: float = 0.1
    beta1: float = 0.9
    beta2: float = 0.95
    grad_clip: float = 1.0
    # precision: compute dtype of activations / GEMM inputs, dtype of the master weights
    dtype: str = "bfloat16"
    param_dtype: str = "float32"
    # parallel layout (all 1 = single device)
    dp: int = 1
    fsdp: int = 1
    tp: int = 1
    sequence_parallel: bool = False  # with --tp=N on GPUs: token rows sharded between the blocks, fused collective GEMMs
    sp: int = 1
    pp: int = 1                      # pipeline stages (scripts/train.py --pp=N, GPT-2)
    ep: int = 1
    # data
    data_source: str = "local"
    gcs_bucket: str = ""
    gcs_dataset_path: str = ""
    local_data_path: str = "data/"
    num_workers: int = 4
    # duration
    max_steps: int = 600000
    eval_interval: int = 250
    eval_steps: int = 20
    log_interval: int = 10
    save_interval: int = 1000
    # checkpointing
    checkpoint_dir: str = "checkpoints/"
    max_checkpoints_to_keep: int = 3
    resume_from: str = ""
    # logging
    wandb_project: str = ""
    wandb_run_name: str = ""
    log_to_wandb: bool = False
    hardware: str = "b200"
    # runtime
    cuda_graph: bool = True
    overlap_grad_reduce: bool = False  # several GPUs: reduce-scatter each layer's gradients during backward
    seed: int = 0

    def replace(self, **kw) -> "TrainConfig":
        return replace(self, **kw)


def apply_overrides(cfg, argv):
    """Applies ``--name=value`` / ``--name value`` overrides to a dataclass instance, converting
    each value to the type of the field's current value. Returns (new_cfg, leftover_args)."""
    names = {f.name: f for f in fields(cfg)}
    updates, rest = {}, []
    i = 0
    while i < len(argv):
        a = argv[i]
        if a.startswith("--"):
            key, eq, val = a[2:].partition("=")
            key = key.replace("-", "_")
            if key in names:
                if not eq:
                    cur = getattr(cfg, key)
                    if isinstance(cur, bool) and (i + 1 >= len(argv) or argv[i + 1].startswith("--")):
                        val = "true"
                    else:
                        i += 1
                        val = argv[i]
                cur = getattr(cfg, key)
                if isinstance(cur, bool):
                    updates[key] = val.lower() in ("1", "true", "yes", "on")
                elif isinstance(cur, int):
                    updates[key] = int(val)
                elif isinstance(cur, float):
                    updates[key] = float(val)
                else:
                    updates[key] = val
                i += 1
                continue
        rest.append(a)
        i += 1
    return replace(cfg, **updates), rest
