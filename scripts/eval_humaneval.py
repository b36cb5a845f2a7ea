"""HumanEval-style evaluation of the Qwen3.5 hybrid model (scripts/eval_humaneval.py:50-818).

The processes form ``--dp`` replicas of ``--tp`` tensor-parallel ranks (``--sharding`` picks the rule set of
models/qwen35/sharding.py). Each replica takes every ``dp``-th problem, generates a completion with the
KV / recurrent-state cache (prefill, then one recurrent step per token until a stop id or
``--max-new-tokens``), runs the problem's tests in a subprocess with a 10 s limit, writes its
results to ``--output-dir`` and waits on a file barrier (600 s, then merges what exists).
The prompt goes through the tokenizer's chat template when it has one (``--enable-thinking`` is passed to it),
otherwise through the plain-text fallback below.
Without the ``datasets`` package or network a single built-in problem is used, as in the
reference (scripts/eval_humaneval.py:423-448).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

from utils import get_tokenizer, init_distributed, make_tp_dp_groups, qwen_config

import torch

DUMMY_PROBLEM = {
    "task_id": "dummy/0",
    "prompt": 'def add(a, b):\n    """Return the sum of a and b.\n    >>> add(1, 2)\n    3\n    """\n',
    "test": "def check(candidate):\n    assert candidate(1, 2) == 3\n    assert candidate(-1, 1) == 0\n",
    "entry_point": "add",
}


def load_problems(n: int):
    try:
        from datasets import load_dataset
        ds = load_dataset("openai_humaneval", split="test")
        probs = [dict(p) for p in ds]
    except Exception:
        probs = [DUMMY_PROBLEM]
    return probs[:n] if n > 0 else probs


def evaluate_completion(problem: dict, completion: str, timeout: float = 10.0) -> bool:
    """Runs prompt + completion + tests in a fresh interpreter; True when it exits 0 in time."""
    code = problem["prompt"] + completion + "\n" + problem["test"] + f"\ncheck({problem['entry_point']})\n"
    with tempfile.NamedTemporaryFile(mode="w", suffix=".py", delete=False) as f:
        f.write(code)
        path = f.name
    try:
        return subprocess.run([sys.executable, path], capture_output=True, text=True, timeout=timeout).returncode == 0
    except subprocess.TimeoutExpired:
        return False
    finally:
        os.unlink(path)


def file_barrier(out_dir: str, rank: int, world: int, timeout: float = 600.0) -> bool:
    """Each rank drops a sentinel; returns True when all are present, False after ``timeout``."""
    open(os.path.join(out_dir, f".done_{rank}"), "w").close()
    t0 = time.time()
    while time.time() - t0 < timeout:
        if all(os.path.exists(os.path.join(out_dir, f".done_{r}")) for r in range(world)):
            return True
        time.sleep(0.2)
    return False


INSTRUCTION = ("Complete the following Python function. Return only the code that continues the given prefix.\n\n"
               "```python\n{prompt}```")


def build_prompt(problem_prompt: str, hf_tok, enable_thinking: bool) -> str:
    """Chat-formatted prompt as the reference builds it (scripts/eval_humaneval.py:311-360 there): the
    tokenizer's own chat template when it has one, with ``enable_thinking`` handed through; without a template
    (byte / GPT-2 fallback tokenizers) a ChatML-style frame with an opened or pre-closed think block."""
    msg = [{"role": "user", "content": INSTRUCTION.format(prompt=problem_prompt)}]
    if hf_tok is not None and getattr(hf_tok, "chat_template", None):
        try:
            return hf_tok.apply_chat_template(msg, tokenize=False, add_generation_prompt=True,
                                              enable_thinking=enable_thinking)
        except TypeError:
            return hf_tok.apply_chat_template(msg, tokenize=False, add_generation_prompt=True)
    think = "<think>\n" if enable_thinking else "<think>\n\n</think>\n\n"
    return f"<|im_start|>user\n{msg[0]['content']}<|im_end|>\n<|im_start|>assistant\n{think}"


def extract_code(text: str) -> str:
    """The completion's code: what follows a closed think block, inside a ```python fence when there is one."""
    if "</think>" in text:
        text = text.split("</think>", 1)[1]
    if "```" in text:
        body = text.split("```", 1)[1]
        body = body.split("\n", 1)[1] if body.startswith(("python", "py")) and "\n" in body else body
        text = body.split("```", 1)[0]
    return text


@torch.no_grad()
def generate_completion(params, cfg, prompt_ids, max_new_tokens, stop_ids, sampler_kw, device, gen, cache_dtype,
                        tp=None, use_engine=False):
    """``tp = (group, mesh, rules, rank)`` for tensor-parallel parameters: every rank of the group runs the same
    loop on the same tokens (the sampler is seeded alike), so they stay in lock step as in the reference
    (scripts/eval_humaneval.py:388-408 there). ``use_engine``: decode through the in-place CUDA-graph engine."""
    from jax_gpt_b200.models.qwen35 import forward, init_cache
    from jax_gpt_b200.utils.sampling import sample
    tok = torch.tensor([prompt_ids], device=device)
    cache = init_cache(cfg, 1, len(prompt_ids) + max_new_tokens, dtype=cache_dtype, device=device)
    tp_group = None
    if tp is not None:
        from jax_gpt_b200.models.qwen35.sharding import shard_cache
        tp_group, mesh, rules, tp_rank = tp
        cache = shard_cache(cache, mesh, cfg, rules, rank=tp_rank)
    seen = torch.zeros(1, cfg.vocab_size, device=device)
    seen[0, tok[0]] = 1.0
    logits, cache = forward(params, tok, cfg, cache=cache, tp_group=tp_group)
    engine = None
    if use_engine and tp is None:
        from jax_gpt_b200.models.qwen35.decode_engine import Qwen35DecodeEngine
        engine = Qwen35DecodeEngine(params, cfg, cache, use_cuda_graph=False)
    out = []
    last = logits[:, -1]
    for _ in range(max_new_tokens):
        nxt = sample(last, presence_mask=seen, generator=gen, **sampler_kw)
        t = int(nxt)
        if t in stop_ids:
            break
        out.append(t)
        seen[0, t] = 1.0
        if engine is not None:
            engine.step(nxt)
            last = engine.logits
        else:
            logits, cache = forward(params, nxt[:, None], cfg, cache=cache, is_decode=True, tp_group=tp_group)
            last = logits[:, -1]
    return out


def main(argv=None):
    from jax_gpt_b200.models.qwen35 import init_params
    from jax_gpt_b200.models.qwen35.sharding import tree_map
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model-dir", default="")
    ap.add_argument("--output-dir", default="humaneval_out")
    ap.add_argument("--n-problems", type=int, default=0)
    ap.add_argument("--max-new-tokens", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=0.0)
    ap.add_argument("--presence-penalty", type=float, default=0.0)
    ap.add_argument("--sharding", default="A", choices=["A", "B"])
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--dp", type=int, default=1)
    ap.add_argument("--config", default="mini")
    ap.add_argument("--tokenizer", default="")
    ap.add_argument("--random-weights", action="store_true")
    ap.add_argument("--enable-thinking", action="store_true")
    ap.add_argument("--engine", action="store_true", help="decode on the in-place engine (not with --tp)")
    args = ap.parse_args(argv)
    rank, world, device = init_distributed()
    if args.tp * args.dp == 1 and world > 1:
        args.dp = world                       # plain data parallelism over the launched processes
    tp_group, tp_rank, dp_rank = make_tp_dp_groups(args.tp, args.dp)
    cfg = qwen_config(args.config)
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    if args.model_dir and not args.random_weights:
        from jax_gpt_b200.models.qwen35.offload import LazySafetensors
        from jax_gpt_b200.models.qwen35.weight_loader import load_from_hf_state_dict
        params = load_from_hf_state_dict(LazySafetensors(args.model_dir), cfg, dtype=dtype)
    else:
        params = init_params(cfg, 0, dtype=dtype)
    tp = None
    if args.tp > 1:
        from jax_gpt_b200.models.qwen35.sharding import AXIS_RULES_A, AXIS_RULES_B, make_mesh, shard_params
        rules = AXIS_RULES_A if args.sharding == "A" else AXIS_RULES_B
        mesh = make_mesh(args.tp, group=tp_group)
        params = shard_params(params, mesh, cfg, rules, rank=tp_rank)
        tp = (tp_group, mesh, rules, tp_rank)
    params = tree_map(lambda t: t.to(device), params)
    hf_tok = None
    if args.tokenizer:
        from transformers import AutoTokenizer
        hf_tok = AutoTokenizer.from_pretrained(args.tokenizer)
        encode, decode = hf_tok.encode, hf_tok.decode
        stop_ids = {i for i in [hf_tok.eos_token_id] if i is not None}
    else:
        bt = get_tokenizer()
        encode = lambda s: [i % cfg.vocab_size for i in bt.encode(s)]
        decode, stop_ids = bt.decode, {bt.eot % cfg.vocab_size}
    os.makedirs(args.output_dir, exist_ok=True)
    problems = load_problems(args.n_problems)
    mine = problems[dp_rank::args.dp]
    gen = torch.Generator().manual_seed(dp_rank)        # the ranks of a tensor-parallel group sample alike
    kw = dict(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, presence_penalty=args.presence_penalty)
    results = []
    for p in mine:
        t0 = time.time()
        prompt = build_prompt(p["prompt"], hf_tok, args.enable_thinking)
        ids = generate_completion(params, cfg, encode(prompt), args.max_new_tokens, stop_ids, kw, device, gen, dtype,
                                  tp=tp, use_engine=args.engine)
        text = extract_code(decode(ids))
        if tp_rank == 0:
            results.append({"task_id": p["task_id"], "completion": text, "passed": evaluate_completion(p, text),
                            "n_tokens": len(ids), "seconds": time.time() - t0})
    if tp_rank == 0:
        with open(os.path.join(args.output_dir, f"results_rank{dp_rank}.json"), "w") as f:
            json.dump(results, f)
    complete = file_barrier(args.output_dir, rank, world)
    if rank == 0:
        merged = []
        for r in range(args.dp):
            path = os.path.join(args.output_dir, f"results_rank{r}.json")
            if os.path.exists(path):
                merged += json.load(open(path))
        n_pass = sum(r["passed"] for r in merged)
        summary = {"n_problems": len(merged), "pass@1": n_pass / max(1, len(merged)), "all_ranks_reported": complete,
                   "tokens_per_second": sum(r["n_tokens"] for r in merged) / max(1e-9, sum(r["seconds"] for r in merged))}
        with open(os.path.join(args.output_dir, "summary.json"), "w") as f:
            json.dump({"summary": summary, "results": merged}, f, indent=1)
        print(json.dumps(summary))
    return 0


if __name__ == "__main__":
    main()
