"""Qwen3.5-style hybrid model: parameter init, forward, generate, sampling
(jax_gpt/models/qwen35/model.py:25-416).

Parameter tree (nested dict, (in,out) kernels, leading (G,) group axis and (G,3) for the
DeltaNet layers)::

    embed (V,D)  final_norm (D)  lm_head (D,V)
    groups.delta_layers.{attn_norm,moe_norm} (G,3,D)
    groups.delta_layers.attn.{in_proj_qkv (G,3,D,2Kd+Vd), in_proj_z (G,3,D,Vd), in_proj_b, in_proj_a (G,3,D,Hv),
                              conv_weight (G,3,2Kd+Vd,Kc), A_log, dt_bias (G,3,Hv), norm_weight (G,3,dv), out_proj (G,3,Vd,D)}
    groups.delta_layers.moe.{gate_weight (G,3,D,E), gate_proj, up_proj (G,3,E,D,I), down_proj (G,3,E,I,D),
                             shared_gate_proj, shared_up_proj (G,3,D,SI), shared_down_proj (G,3,SI,D),
                             shared_expert_gate_weight (G,3,D,1)}
    groups.gqa_layer.{attn_norm,moe_norm} (G,D)
    groups.gqa_layer.attn.{q_proj (G,D,2 Hq dh), k_proj, v_proj (G,D,Hkv dh), o_proj (G,Hq dh,D), q_norm, k_norm (G,dh)}
    groups.gqa_layer.moe.{... same keys with a leading (G,) ...}

Init: N(0, 0.02) for every linear, embedding and conv weight; RMSNorm weights 0 (the (1+w)
convention); ``A_log = log U(0.1, 16)``; ``dt_bias = 1``; gated-norm weight 1.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ...utils.profiling import scope
from .block import _slice, group_forward
from .cache import HybridCache, init_cache
from .config import Qwen35Config
from .fp8 import matmul_maybe_fp8
from .primitives import precompute_rope_freqs, rms_norm
from .quantize import quantize_params_fp8


def _normal(g, device, dtype):
    """``n(*shape)``: N(0, 0.02) of that shape. A generator that lives on the target device draws there, in the
    target dtype (no host copy of the tree); a CPU generator draws in fp32 on the host and moves the result."""
    if g.device.type != "cpu":
        return lambda *s: torch.randn(*s, generator=g, device=g.device, dtype=dtype).mul_(0.02)
    return lambda *s: (torch.randn(*s, generator=g) * 0.02).to(device=device, dtype=dtype)


def _moe_params(c: Qwen35Config, lead, g, dtype, device, g_experts=None, n_local=None):
    D, E, I, SI = c.d_model, c.n_routed_experts, c.moe_intermediate_size, c.shared_expert_intermediate_size
    nn = _normal(g, device, dtype)
    n = lambda *s: nn(*lead, *s)
    if n_local is not None:           # only this rank's experts, from the rank's own stream
        ne = _normal(g_experts, device, dtype)
        e = lambda *s: ne(*lead, *s)
        El = n_local
    else:
        e, El = n, E
    return {
        "gate_weight": n(D, E), "gate_proj": e(El, D, I), "up_proj": e(El, D, I), "down_proj": e(El, I, D),
        "shared_gate_proj": n(D, SI), "shared_up_proj": n(D, SI), "shared_down_proj": n(SI, D),
        "shared_expert_gate_weight": n(D, 1),
    }


def init_params(config: Qwen35Config, key=0, dtype=torch.float32, fp8: bool = False, device="cpu",
                on_device: bool = False, expert_shard=None) -> dict:
    """``key``: integer seed (or a torch.Generator). ``on_device=True`` draws every tensor on ``device`` in ``dtype``
    (nothing of the tree ever exists on the host: the 77 B-parameter benchmark shape cannot be initialised there).
    ``expert_shard=(rank, world)`` creates only this rank's ``E / world`` routed experts, from a stream of their own
    seeded with (key, rank); everything else is drawn identically on every rank."""
    c = config
    if on_device and torch.device(device).type != "cpu" and not isinstance(key, torch.Generator):
        g = torch.Generator(device=device).manual_seed(int(key))
    else:
        g = key if isinstance(key, torch.Generator) else torch.Generator().manual_seed(int(key))
    g_experts = n_local = None
    if expert_shard is not None:
        rank, world = expert_shard
        assert c.n_routed_experts % world == 0
        n_local = c.n_routed_experts // world
        g_experts = torch.Generator(device=g.device).manual_seed((int(g.initial_seed()) + 1) * 1000003 + rank)
    G, nd, D = c.n_groups, c.n_delta_per_group, c.d_model
    Kd, Vd, Hv = c.delta_key_dim, c.delta_value_dim, c.delta_n_v_heads
    Hq, Hkv, dh = c.gqa_n_q_heads, c.gqa_n_kv_heads, c.gqa_head_dim
    dev = dict(device=device, dtype=dtype)
    n = _normal(g, device, dtype)
    zeros = lambda *s: torch.zeros(*s, **dev)
    ones = lambda *s: torch.ones(*s, **dev)
    delta_attn = {
        "in_proj_qkv": n(G, nd, D, 2 * Kd + Vd), "in_proj_z": n(G, nd, D, Vd), "in_proj_b": n(G, nd, D, Hv),
        "in_proj_a": n(G, nd, D, Hv), "conv_weight": n(G, nd, 2 * Kd + Vd, c.delta_conv_kernel),
        "A_log": torch.log(torch.rand(G, nd, Hv, generator=g, device=g.device) * 15.9 + 0.1).to(**dev),
        "dt_bias": ones(G, nd, Hv),
        "norm_weight": ones(G, nd, c.delta_v_head_dim), "out_proj": n(G, nd, Vd, D),
    }
    gqa_attn = {
        "q_proj": n(G, D, 2 * Hq * dh), "k_proj": n(G, D, Hkv * dh), "v_proj": n(G, D, Hkv * dh),
        "o_proj": n(G, Hq * dh, D), "q_norm": zeros(G, dh), "k_norm": zeros(G, dh),
    }
    params = {
        "embed": n(c.vocab_size, D), "final_norm": zeros(D), "lm_head": n(D, c.vocab_size),
        "groups": {
            "delta_layers": {"attn_norm": zeros(G, nd, D), "moe_norm": zeros(G, nd, D), "attn": delta_attn,
                             "moe": _moe_params(c, (G, nd), g, dtype, device, g_experts, n_local)},
            "gqa_layer": {"attn_norm": zeros(G, D), "moe_norm": zeros(G, D), "attn": gqa_attn,
                          "moe": _moe_params(c, (G,), g, dtype, device, g_experts, n_local)},
        },
    }
    return quantize_params_fp8(params) if fp8 else params


def forward(params, tokens, config: Qwen35Config, cache: Optional[HybridCache] = None, is_decode: bool = False,
            cache_sharding=None, n_devices: int = 1, axis_name: str = "tp", mesh=None, ep_group=None, tp_group=None):
    """tokens (B,T) -> (logits (B,T,V), new_cache | None). ``is_decode`` selects the recurrent
    DeltaNet step (T must be 1); otherwise the chunked prefill runs (a prefill starts from an
    empty DeltaNet state, as in the reference).

    Tensor parallel: pass the local shard from ``shard_params`` together with ``tp_group`` (or a ``mesh`` made by
    ``make_mesh(..., group=...)``): every rank feeds the same tokens, sharded axes are recognised by their shapes,
    and the logits come back whole on every rank, as in the reference's sharded forward
    (jax_gpt/models/qwen35/model.py:207-331 with the specs of sharding.py). ``n_devices``, ``axis_name`` and
    ``cache_sharding`` are accepted for signature parity: the group and the shapes carry that information here.
    A sharded tree without a group is an error rather than a silent wrong answer."""
    from ...parallel.tp_ops import copy_to_tp, gather_from_tp, tp_world, vocab_parallel_embedding
    c = config
    B, T = tokens.shape
    if tp_group is None and mesh is not None:
        tp_group = getattr(mesh, "group", None)
    vocab_sharded = params["embed"].shape[0] < c.vocab_size
    if (vocab_sharded or _lm_head_cols(params["lm_head"]) < c.vocab_size) and tp_world(tp_group) == 1:
        raise ValueError("forward() got a tensor-parallel shard of the parameters but no process group: pass "
                         "tp_group= (or mesh=make_mesh(n, group=...)) and run one process per shard")
    with scope("embedding"):
        x = vocab_parallel_embedding(tokens, params["embed"], tp_group, c.vocab_size)
    pos = cache.pos if cache is not None else 0
    max_pos = (cache.gqa_k.shape[3] if cache is not None else pos + T)
    rope = precompute_rope_freqs(c.gqa_rope_dim, max(max_pos, pos + T), c.gqa_rope_theta, device=x.device)
    new_M, new_conv = [], []
    for gi in range(c.n_groups):
        gp = _slice(params["groups"], gi)
        if cache is not None:
            dM, dC = cache.delta_M[gi], cache.delta_conv[gi]
            ck, cv = cache.gqa_k[gi], cache.gqa_v[gi]
        else:
            dM = dC = ck = cv = None
        x, M, conv, _, _ = group_forward(x, gp, dM, dC, ck, cv, pos, c, rope, is_decode, ep_group=ep_group,
                                         tp_group=tp_group)
        new_M.append(M)
        new_conv.append(conv)
    with scope("output_head"):
        x = rms_norm(x, params["final_norm"], c.rms_norm_eps)
        from ...ops.fp8_linear import fp8_training
        with fp8_training(False):          # the head stays in bf16 also when the layers train in FP8
            if _lm_head_cols(params["lm_head"]) < c.vocab_size:
                # vocabulary-parallel head: local logit columns, gathered to whole logits on every rank
                logits = gather_from_tp(matmul_maybe_fp8(copy_to_tp(x, tp_group), params["lm_head"]), tp_group, -1)
            else:
                logits = matmul_maybe_fp8(x, params["lm_head"])
    new_cache = None
    if cache is not None:
        new_cache = HybridCache(torch.stack(new_M).to(cache.delta_M.dtype),
                                torch.stack(new_conv).to(cache.delta_conv.dtype), cache.gqa_k, cache.gqa_v, pos + T)
    return logits, new_cache


def _lm_head_cols(w) -> int:
    return w["w"].shape[-2] if isinstance(w, dict) else w.shape[-1]


def _sample(logits: torch.Tensor, temperature: float = 1.0, top_k: Optional[int] = None, generator=None):
    """(B,V) -> (B,) token ids: T <= 0 -> argmax; else logits/T, keep logits >= k-th, sample."""
    from ..gpt2.model import sample_logits
    return sample_logits(logits, temperature, top_k, generator)


@torch.no_grad()
def generate(params, prompt_tokens, config: Qwen35Config, max_new_tokens: int, max_seq_len: Optional[int] = None,
             temperature: float = 1.0, top_k: Optional[int] = None, key=None, cache_dtype=None):
    """Prefill + recurrent decode. Returns ONLY the continuation, shape (B, max_new_tokens)."""
    B, T = prompt_tokens.shape
    max_seq_len = max_seq_len or (T + max_new_tokens)
    gen = key if isinstance(key, torch.Generator) else torch.Generator().manual_seed(int(key) if key is not None else 0)
    dtype = cache_dtype or params["embed"].dtype
    cache = init_cache(config, B, max_seq_len, dtype=dtype, device=prompt_tokens.device)
    logits, cache = forward(params, prompt_tokens, config, cache=cache, is_decode=False)
    nxt = _sample(logits[:, -1], temperature, top_k, gen)
    out = [nxt]
    for _ in range(max_new_tokens - 1):
        logits, cache = forward(params, nxt[:, None], config, cache=cache, is_decode=True)
        nxt = _sample(logits[:, -1], temperature, top_k, gen)
        out.append(nxt)
    return torch.stack(out, dim=1)


def count_params(params) -> int:
    from .quantize import count_fp8_params
    return count_fp8_params(params)[0]
