"""Greedy generation with this package's GPT-2 next to the HF implementation on the same
weights (scripts/verify_generation.py:1-48); with ``--random`` a tiny random HF model is used."""
from __future__ import annotations

import argparse

from utils import gpt_config  # noqa: F401

import torch


def main(argv=None):
    from transformers import GPT2Config, GPT2LMHeadModel
    from jax_gpt_b200.models.gpt2 import GPT, GPTConfig
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model", default="gpt2")
    ap.add_argument("--random", action="store_true")
    ap.add_argument("--new-tokens", type=int, default=8)
    args = ap.parse_args(argv)
    if args.random:
        cfg = GPTConfig(d_model=64, d_head=16, d_ff=256, d_context=64, n_head=4, n_kv_head=4, n_layers=2, vocab_size=100)
        hf = GPT2LMHeadModel(GPT2Config(vocab_size=100, n_positions=64, n_embd=64, n_layer=2, n_head=4,
                                        activation_function="gelu_new", resid_pdrop=0, embd_pdrop=0, attn_pdrop=0)).eval()
    else:
        cfg = GPTConfig.from_model_type(args.model)
        hf = GPT2LMHeadModel.from_pretrained(args.model).eval()
    ours = GPT.from_hf_state_dict(hf.state_dict(), cfg)
    idx = torch.randint(0, cfg.vocab_size, (1, 5), generator=torch.Generator().manual_seed(0))
    a = ours.generate(idx, args.new_tokens, temperature=0.0)
    b = hf.generate(idx, max_new_tokens=args.new_tokens, do_sample=False, pad_token_id=0)
    print("ours:", a.tolist()[0])
    print("hf:  ", b.tolist()[0])
    print("match:", a.tolist() == b.tolist())
    rows = ours.compare_activations(hf, 2, 8)
    print("max activation diff:", max(r[3] for r in rows))


if __name__ == "__main__":
    main()
