"""Fused GPT-2 engine on a B200 vs the PyTorch fp32 reference model (autograd)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _setup(cuda_device, graph):
    from jax_gpt_b200.models.gpt2 import GPT, GPTConfig
    from jax_gpt_b200.models.gpt2.engine import GPT2TrainEngine
    cfg = GPTConfig(d_model=128, d_head=64, d_ff=512, d_context=256, n_head=2, n_kv_head=2, n_layers=2, vocab_size=1003)
    ref = GPT(cfg, seed=3, device=cuda_device, dtype=torch.float32)
    eng = GPT2TrainEngine(cfg, 2, 256, device=cuda_device, init={k: v.cpu() for k, v in ref.params.items()},
                          lr=1e-3, warmup_steps=0, lr_decay_steps=1000, use_cuda_graph=graph)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (2, 257), generator=g)
    x = tok[:, :-1].to(cuda_device, torch.int32)
    y = tok[:, 1:].to(cuda_device, torch.int32)
    return cfg, ref, eng, x, y


def test_engine_loss_and_grads_match_reference(cuda_device):
    cfg, ref, eng, x, y = _setup(cuda_device, graph=False)
    eng.tokens.copy_(x)
    eng.targets.copy_(y.reshape(-1))
    eng.forward(True, True)
    eng.backward()
    torch.cuda.synchronize()
    for p in ref.params.values():
        p.requires_grad_(True)
    logits, _ = ref(x)
    loss = torch.nn.functional.cross_entropy(logits.float().reshape(-1, cfg.vocab_size), y.reshape(-1).long())
    loss.backward()
    assert abs(eng.loss.item() - loss.item()) < 2e-2
    assert abs(loss.item() - math.log(cfg.vocab_size)) < 1.0
    bad = []
    for name, g in eng.g.items():
        rg = ref.params[name].grad
        if rg is None or name == "lm_head.kernel":
            assert g.abs().max().item() == 0
            continue
        e = _rel(g, rg)
        if e > 6e-2:
            bad.append((name, e))
    assert not bad, bad


@pytest.mark.parametrize("graph", [False, True])
def test_engine_trains(cuda_device, graph):
    cfg, ref, eng, x, y = _setup(cuda_device, graph=graph)
    losses = []
    for _ in range(12):
        out = eng.train_step(x, y)
        losses.append(out["loss"].item())
    assert losses[0] > losses[-1] + 0.5, losses
    assert all(math.isfinite(v) for v in losses)
    # bf16 compute copy tracks the fp32 master
    assert _rel(eng.flat.compute.float(), eng.flat.master) < 1e-2


def test_engine_accumulation_matches_single_step(cuda_device):
    """Two identical micro-batches then one update == one micro-batch then one update."""
    cfg, ref, eng_a, x, y = _setup(cuda_device, graph=False)
    _, _, eng_b, _, _ = _setup(cuda_device, graph=False)
    eng_a.train_step(x, y)
    eng_b.micro_step(x, y)
    eng_b.micro_step(x, y)
    eng_b.apply_gradients()
    torch.cuda.synchronize()
    assert _rel(eng_b.flat.master, eng_a.flat.master) < 1e-4


def test_trainer_api_on_gpu(cuda_device):
    from jax_gpt_b200.models.gpt2 import GPT, GPTConfig
    from jax_gpt_b200.trainer import TrainConfig, create_optimizer, create_train_state, eval_step, train_step
    cfg = GPTConfig(d_model=128, d_head=64, d_ff=512, d_context=128, n_head=2, n_kv_head=2, n_layers=2, vocab_size=512)
    tc = TrainConfig(micro_batch_size=2, seq_len=128, learning_rate=1e-3, warmup_steps=0, lr_decay_steps=100)
    model = GPT(cfg, seed=0)
    state = create_train_state(model, create_optimizer(model, tc), train_config=tc, device=cuda_device)
    g = torch.Generator().manual_seed(1)
    tok = torch.randint(0, 512, (2, 129), generator=g, dtype=torch.int32)
    batch = (tok[:, :-1].contiguous().pin_memory(), tok[:, 1:].contiguous().pin_memory())
    first = None
    for i in range(8):
        state, m = train_step(state, batch)
        first = float(m["loss"]) if first is None else first
    assert state.step == 8 and float(m["loss"]) < first
    assert float(m["grad_norm"]) > 0
    ev = eval_step(model, batch, engine=state.engine)
    assert math.isfinite(float(ev))


def test_engine_matches_autograd_at_the_benchmark_shape(cuda_device):
    """Width 768, 12 heads, sequence 1024, the real vocabulary (50257, not a multiple of the tile), batch 16, two
    layers: the shapes at which the CTA-pair GEMM, the split-K weight gradients (K = 16384 tokens), the two-tile
    attention forward and the pipelined attention backward actually run in ``bench.py``. Loss and every gradient
    against autograd of the fp32 reference model fed the same bf16-rounded weights."""
    from jax_gpt_b200.models.gpt2 import GPT, GPTConfig
    from jax_gpt_b200.models.gpt2.engine import GPT2TrainEngine
    cfg = GPTConfig(d_model=768, d_head=64, d_ff=3072, d_context=1024, n_head=12, n_kv_head=12, n_layers=2,
                    vocab_size=50257)
    B, T = 16, 1024
    ref = GPT(cfg, seed=11, device=cuda_device, dtype=torch.float32)
    with torch.no_grad():
        for v in ref.params.values():          # the engine computes with bf16 copies of the weights
            v.copy_(v.to(torch.bfloat16).float())
    eng = GPT2TrainEngine(cfg, B, T, device=cuda_device, init={k: v.cpu() for k, v in ref.params.items()},
                          lr=1e-3, warmup_steps=0, lr_decay_steps=1000, use_cuda_graph=False)
    g = torch.Generator().manual_seed(2)
    tok = torch.randint(0, cfg.vocab_size, (B, T + 1), generator=g)
    x, y = tok[:, :-1].to(cuda_device, torch.int32), tok[:, 1:].to(cuda_device, torch.int32)
    eng.tokens.copy_(x)
    eng.targets.copy_(y.reshape(-1))
    eng.forward(True, True)
    eng.backward()
    torch.cuda.synchronize()
    for p in ref.params.values():
        p.requires_grad_(True)
    loss = 0.0
    for b0 in range(0, B, 4):                  # the fp32 reference in slices of four sequences (logits are 0.8 GB each)
        logits, _ = ref(x[b0:b0 + 4])
        part = torch.nn.functional.cross_entropy(logits.float().reshape(-1, cfg.vocab_size),
                                                 y[b0:b0 + 4].reshape(-1).long(), reduction="sum") / (B * T)
        part.backward()
        loss += part.item()
    assert abs(eng.loss.item() - loss) < 2e-2, (eng.loss.item(), loss)
    bad = []
    for name, gr in eng.g.items():
        rg = ref.params[name].grad
        if rg is None or name == "lm_head.kernel":
            continue
        e = _rel(gr, rg)
        if e > 6e-2:
            bad.append((name, e))
    assert not bad, bad


def test_loss_decreases_at_the_benchmark_shape(cuda_device):
    """Twenty optimizer steps at the peak learning rate (6e-4, no warm-up) on the full GPT-2 small shape of
    ``bench.py``, CUDA graphs on, one fixed batch: the loss must fall well below ln(vocab)."""
    from jax_gpt_b200.models.gpt2 import GPTConfig
    from jax_gpt_b200.models.gpt2.engine import GPT2TrainEngine
    cfg = GPTConfig.from_model_type("gpt2")
    eng = GPT2TrainEngine(cfg, 16, 1024, device=cuda_device, lr=6e-4, min_lr=6e-4, warmup_steps=0,
                          lr_decay_steps=1000, use_cuda_graph=True, seed=0)
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(0, cfg.vocab_size, (16, 1025), generator=g)
    x, y = tok[:, :-1].to(cuda_device, torch.int32), tok[:, 1:].to(cuda_device, torch.int32)
    losses = [eng.train_step(x, y)["loss"].item() for _ in range(20)]
    assert abs(losses[0] - math.log(cfg.vocab_size)) < 0.5, losses[0]
    assert all(math.isfinite(v) for v in losses) and losses[-1] < losses[0] - 2.0, losses
    del eng
    torch.cuda.empty_cache()
