"""Benchmark-shaped inference tests, as in the reference's tests/*/test_inference_benchmark.py: a prefill run
repeated a few times and a decode loop, timed and printed (run pytest with -s to see the lines); the assertions
are shapes, finiteness and, for the decode paths, agreement between the step-by-step cache and the prefill."""
import time

import torch

from jax_gpt_b200.models.gpt2 import GPT, GPTConfig
from jax_gpt_b200.models.qwen35 import Qwen35Config, forward, init_cache, init_params


def _timed(fn, n):
    fn()                                    # warm-up
    t0 = time.perf_counter()
    for _ in range(n):
        out = fn()
    return out, (time.perf_counter() - t0) / n * 1e3


def test_gpt2_prefill_and_decode_benchmark():
    cfg = GPTConfig(d_model=128, d_head=32, d_ff=512, d_context=160, n_head=4, n_kv_head=4, n_layers=4, vocab_size=512)
    model = GPT(cfg, seed=0)
    B, T, steps = 4, 96, 32
    x = torch.randint(0, cfg.vocab_size, (B, T))
    with torch.no_grad():
        (logits, _), ms = _timed(lambda: model(x), 3)
        print(f"gpt2 prefill  B={B} T={T}: {ms:.2f} ms, {B * T / ms * 1e3:.0f} tok/s")
        assert logits.shape == (B, T, cfg.vocab_size) and torch.isfinite(logits).all()

        def decode():
            cache = model.init_cache(B)
            lg, cache = model(x, cache=cache)
            nxt = lg[:, -1].argmax(-1)
            for _ in range(steps):
                lg, cache = model(nxt[:, None], cache=cache)
                nxt = lg[:, -1].argmax(-1)
            return lg, cache
        (lg, cache), ms = _timed(decode, 2)
        print(f"gpt2 prefill+{steps} decode steps: {ms:.2f} ms, {ms / steps:.2f} ms/step upper bound")
        assert cache.pos == T + steps and lg.shape == (B, 1, cfg.vocab_size) and torch.isfinite(lg).all()


def test_qwen35_prefill_decode_and_engine_benchmark():
    from jax_gpt_b200.models.qwen35.decode_engine import Qwen35DecodeEngine
    cfg = Qwen35Config.tiny()
    params = init_params(cfg, 0)
    B, T, steps = 2, 24, 8
    tok = torch.randint(0, cfg.vocab_size, (B, T))
    with torch.no_grad():
        (logits, _), ms = _timed(lambda: forward(params, tok, cfg), 3)
        print(f"qwen35 prefill B={B} T={T}: {ms:.2f} ms, {B * T / ms * 1e3:.0f} tok/s")
        assert logits.shape == (B, T, cfg.vocab_size) and torch.isfinite(logits).all()

        def loop():
            cache = init_cache(cfg, B, T + steps)
            lg, cache = forward(params, tok, cfg, cache=cache)
            nxt = lg[:, -1].argmax(-1)
            outs = []
            for _ in range(steps):
                lg, cache = forward(params, nxt[:, None], cfg, cache=cache, is_decode=True)
                nxt = lg[:, -1].argmax(-1)
                outs.append(nxt)
            return torch.stack(outs, 1), cache

        def engine():
            cache = init_cache(cfg, B, T + steps)
            lg, cache = forward(params, tok, cfg, cache=cache)
            eng = Qwen35DecodeEngine(params, cfg, cache, use_cuda_graph=False)
            nxt = lg[:, -1].argmax(-1)
            outs = []
            for _ in range(steps):
                nxt = eng.step(nxt).clone()
                outs.append(nxt)
            return torch.stack(outs, 1), eng
        (a, cache), ms_loop = _timed(loop, 2)
        (b, eng), ms_eng = _timed(engine, 2)
        print(f"qwen35 prefill+{steps} decode: function-style {ms_loop:.1f} ms, in-place engine {ms_eng:.1f} ms")
        assert cache.pos == eng.pos == T + steps
        assert a.shape == (B, steps) and torch.equal(a, b)
        assert int(a.min()) >= 0 and int(a.max()) < cfg.vocab_size
