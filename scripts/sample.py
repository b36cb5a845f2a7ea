"""Sampler (the reference's scripts/sample.py:1-7 is a stub): load a checkpoint, encode a prompt
with the GPT-2 BPE, generate with the KV cache, decode and print.

    python scripts/sample.py --checkpoint_dir checkpoints/ --prompt "Hello" --new_tokens 50 --top_k 40
    python scripts/sample.py --preset gpt2-tiny --random-weights --prompt "abc"
"""
from __future__ import annotations

import argparse

from utils import get_tokenizer, gpt_config

import torch


def main(argv=None):
    from jax_gpt_b200.models.gpt2 import GPT
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--preset", default="gpt2")
    ap.add_argument("--checkpoint_dir", default="")
    ap.add_argument("--step", type=int, default=-1, help="-1 = latest")
    ap.add_argument("--hf", default="", help="load HF weights by name or path instead of a checkpoint")
    ap.add_argument("--random-weights", action="store_true")
    ap.add_argument("--prompt", default="Hello, my name is")
    ap.add_argument("--new_tokens", type=int, default=32)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top_k", type=int, default=0)
    ap.add_argument("--num_samples", type=int, default=1)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)

    cfg = gpt_config(args.preset)
    if args.hf:
        model = GPT.from_pretrained(args.hf)
    else:
        model = GPT(cfg, seed=args.seed)
        if args.checkpoint_dir and not args.random_weights:
            from jax_gpt_b200.trainer import TrainConfig, create_optimizer, create_train_state
            from jax_gpt_b200.trainer.checkpointing import CheckpointManager
            tc = TrainConfig(checkpoint_dir=args.checkpoint_dir)
            state = create_train_state(model, create_optimizer(model, tc))
            state = CheckpointManager(tc, cfg).restore(None if args.step < 0 else args.step, state)
            print(f"loaded checkpoint step {state.step}")
    tok = get_tokenizer()
    ids = tok.encode(args.prompt) or [tok.eot]
    idx = torch.tensor([ids] * args.num_samples, dtype=torch.long)
    out = model.generate(idx, args.new_tokens, temperature=args.temperature, top_k=args.top_k or None, rngs=args.seed)
    for i, row in enumerate(out.tolist()):
        print(f"--- sample {i} ---")
        print(tok.decode(row))


if __name__ == "__main__":
    main()
