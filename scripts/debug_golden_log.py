"""Golden activation log of GPT-2: a plain PyTorch model and this framework's GPT side by side.

    python scripts/debug_golden_log.py --model-dir /path/to/hf/gpt2        # pre-trained weights from a local folder
    python scripts/debug_golden_log.py --random --n-layers 4 --seed 0      # random weights, no files needed

Builds the ``transformers`` GPT-2 (the PyTorch reference: weights from ``--model-dir`` or random), copies its
weights into ``jax_gpt_b200.models.gpt2.GPT``, runs ONE forward pass of a prompt through both, and prints for
every site of the residual stream (after the embedding, after every attention block, after every MLP block, after
the final LayerNorm, the logits) the mean and standard deviation seen by each model and the largest absolute
difference: the log one reads to find the first layer where two implementations part ways (the reference's
scripts/debug_pytorch.py:91-157 prints the PyTorch half of it). Ends with a short greedy continuation from both
models. ``--device cuda`` runs this framework's half on the GPU kernels (bf16), so the same log doubles as a kernel
sanity check.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import torch


def _hf_model(args):
    from transformers import GPT2Config, GPT2LMHeadModel
    if args.model_dir:
        return GPT2LMHeadModel.from_pretrained(args.model_dir, local_files_only=True).eval()
    torch.manual_seed(args.seed)
    cfg = GPT2Config(vocab_size=args.vocab, n_positions=args.ctx, n_embd=args.d_model, n_layer=args.n_layers,
                     n_head=args.n_head, activation_function="gelu_new", resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    return GPT2LMHeadModel(cfg).eval()


def _prompt_ids(args, vocab):
    if args.model_dir:
        try:
            from transformers import AutoTokenizer
            tok = AutoTokenizer.from_pretrained(args.model_dir, local_files_only=True)
            return torch.tensor([tok.encode(args.prompt)], dtype=torch.long), tok
        except Exception:
            pass
    g = torch.Generator().manual_seed(args.seed)
    return torch.randint(0, vocab, (1, args.prompt_tokens), generator=g), None


def golden_log(hf, ids):
    """[(site, tensor)] of the residual stream of the PyTorch model, in forward order."""
    sites = []
    hooks = []
    tr = hf.transformer
    hooks.append(tr.drop.register_forward_hook(lambda m, i, o: sites.append(("Start      | After Embed    ", o.detach()))))
    for n, blk in enumerate(tr.h):
        state = {}
        hooks.append(blk.register_forward_pre_hook(lambda m, i, st=state: st.__setitem__("x", i[0].detach())))
        hooks.append(blk.attn.register_forward_hook(
            lambda m, i, o, st=state, n=n: sites.append((f"Block {n:<2} | After Attention", st["x"] + (o[0] if isinstance(o, tuple) else o).detach()))))
        hooks.append(blk.register_forward_hook(
            lambda m, i, o, n=n: sites.append((f"Block {n:<2} | After MLP      ", (o[0] if isinstance(o, tuple) else o).detach()))))
    hooks.append(tr.ln_f.register_forward_hook(lambda m, i, o: sites.append(("End        | After Final LN ", o.detach()))))
    with torch.no_grad():
        logits = hf(ids).logits
    for h in hooks:
        h.remove()
    sites.append(("End        | Final Logits   ", logits))
    return sites


def framework_log(model, ids):
    with torch.no_grad():
        _, _, acts = model(ids, return_activations=True)
    n_layers = model.config.n_layers
    x = acts["initial_embedding"].float()
    sites = [("Start      | After Embed    ", x)]
    for n in range(n_layers):
        x = x + acts[f"block_{n}_attn_output_pre_residual"].float()
        sites.append((f"Block {n:<2} | After Attention", x))
        x = x + acts[f"block_{n}_mlp_output_pre_residual"].float()
        sites.append((f"Block {n:<2} | After MLP      ", x))
    sites.append(("End        | After Final LN ", acts["final_layernorm"].float()))
    sites.append(("End        | Final Logits   ", acts["final_logits"].float()))
    return sites


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model-dir", default="", help="local Hugging Face GPT-2 folder (weights and tokenizer)")
    ap.add_argument("--random", action="store_true", help="random weights of the given shape instead of --model-dir")
    ap.add_argument("--prompt", default="The answer to the ultimate question of life, the universe, and everything is")
    ap.add_argument("--prompt-tokens", type=int, default=16, help="length of the random prompt when there is no tokenizer")
    ap.add_argument("--new-tokens", type=int, default=20)
    ap.add_argument("--n-layers", type=int, default=12)
    ap.add_argument("--n-head", type=int, default=12)
    ap.add_argument("--d-model", type=int, default=768)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--vocab", type=int, default=50257)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--tolerance", type=float, default=0.0, help="exit 1 if a site differs by more (0 = only report)")
    args = ap.parse_args(argv)
    if not args.model_dir and not args.random:
        ap.error("give --model-dir or --random")
    from jax_gpt_b200.models.gpt2 import GPT, GPTConfig
    hf = _hf_model(args)
    ids, tok = _prompt_ids(args, hf.config.vocab_size)
    dtype = torch.bfloat16 if args.device.startswith("cuda") else torch.float32
    hc = hf.config
    cfg = GPTConfig(d_model=hc.n_embd, d_head=hc.n_embd // hc.n_head, d_ff=4 * hc.n_embd, d_context=hc.n_positions,
                    n_head=hc.n_head, n_kv_head=hc.n_head, n_layers=hc.n_layer, vocab_size=hc.vocab_size)
    model = GPT.from_hf_state_dict(hf.state_dict(), cfg, device=args.device, dtype=dtype)
    ref = golden_log(hf, ids)
    own = framework_log(model, ids.to(args.device))
    print(f"{'site':<29} | {'PyTorch mean':>12} {'std':>10} | {'this mean':>12} {'std':>10} | max abs diff")
    worst = 0.0
    for (name, a), (_, b) in zip(ref, own):
        b = b.to("cpu", torch.float32)
        d = float((a.float() - b).abs().max())
        worst = max(worst, d)
        print(f"{name} | {float(a.mean()):12.6f} {float(a.std()):10.6f} | {float(b.mean()):12.6f} {float(b.std()):10.6f} | {d:.3e}")
    last = ref[-1][1][0, -1]
    print(f"\nReference logits (last token): shape {tuple(last.shape)}, mean {float(last.mean()):.6f}, std {float(last.std()):.6f}")
    with torch.no_grad():
        out_ref = hf.generate(ids, max_new_tokens=args.new_tokens, do_sample=False, pad_token_id=0)[0, ids.shape[1]:]
        out_own = model.generate(ids.to(args.device), args.new_tokens, temperature=0.0)[0, ids.shape[1]:].cpu()
    same = int((out_ref == out_own).sum())
    print(f"greedy continuation: {same}/{args.new_tokens} tokens equal")
    if tok is not None:
        print("PyTorch :", tok.decode(out_ref.tolist()))
        print("this    :", tok.decode(out_own.tolist()))
    if args.tolerance and worst > args.tolerance:
        print(f"FAILED: largest difference {worst:.3e} > {args.tolerance:.3e}")
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
