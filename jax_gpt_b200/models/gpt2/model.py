"""GPT-2 with the reference's parameter tree, API and semantics.

Parameter tree (jax_gpt/models/gpt2/model.py:229-242, jax_gpt/trainer/sharding.py:37-55):
linear kernels are (in, out), block parameters carry a leading ``n_layers`` axis::

    wte.embedding (V,d)   wpe.embedding (ctx,d)   ln_f.layer_norm.{scale,bias} (d)
    h.ln_1.layer_norm.{scale,bias} (L,d)          h.ln_2.layer_norm.{scale,bias} (L,d)
    h.attn.c_attn.{kernel (L,d,3d), bias (L,3d)}  h.attn.c_proj.{kernel (L,d,d), bias (L,d)}
    h.mlp.c_fc.{kernel (L,d,4d), bias (L,4d)}     h.mlp.c_proj.{kernel (L,4d,d), bias (L,d)}
    lm_head.kernel (d,V)                          # kept for layout parity, unused by forward

Forward: wte + wpe, pre-LN blocks, tanh-GELU MLP, logits tied to wte
(jax_gpt/models/gpt2/model.py:245-326). The cached path applies the causal rule on true
positions ``pos + i >= k_pos`` and attends only over the filled part of the cache; the
reference masks every query row of a multi-token cached pass with the incoming position
(jax_gpt/models/gpt2/model.py:170-172), which is only right for single-token decode.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional

import torch
import torch.nn.functional as F

from ...ops import attention as attn_ops
from ...ops import gemm as gemm_ops
from ...ops import norm as norm_ops
from .config import GPTConfig

PARAM_ORDER_DECAY = [
    "h.attn.c_attn.kernel", "h.attn.c_proj.kernel", "h.mlp.c_fc.kernel", "h.mlp.c_proj.kernel", "lm_head.kernel",
]
PARAM_ORDER_NO_DECAY = [
    "wte.embedding", "wpe.embedding",
    "h.ln_1.layer_norm.scale", "h.ln_1.layer_norm.bias", "h.ln_2.layer_norm.scale", "h.ln_2.layer_norm.bias",
    "h.attn.c_attn.bias", "h.attn.c_proj.bias", "h.mlp.c_fc.bias", "h.mlp.c_proj.bias",
    "ln_f.layer_norm.scale", "ln_f.layer_norm.bias",
]


def param_shapes(cfg: GPTConfig) -> Dict[str, tuple]:
    L, d, f, V, C = cfg.n_layers, cfg.d_model, cfg.d_ff, cfg.vocab_size, cfg.d_context
    return {
        "wte.embedding": (V, d), "wpe.embedding": (C, d),
        "h.ln_1.layer_norm.scale": (L, d), "h.ln_1.layer_norm.bias": (L, d),
        "h.ln_2.layer_norm.scale": (L, d), "h.ln_2.layer_norm.bias": (L, d),
        "h.attn.c_attn.kernel": (L, d, 3 * d), "h.attn.c_attn.bias": (L, 3 * d),
        "h.attn.c_proj.kernel": (L, d, d), "h.attn.c_proj.bias": (L, d),
        "h.mlp.c_fc.kernel": (L, d, f), "h.mlp.c_fc.bias": (L, f),
        "h.mlp.c_proj.kernel": (L, f, d), "h.mlp.c_proj.bias": (L, d),
        "ln_f.layer_norm.scale": (d,), "ln_f.layer_norm.bias": (d,),
        "lm_head.kernel": (d, V),
    }


def init_params(cfg: GPTConfig, seed: int = 0, device="cpu", dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """N(0, 0.02) kernels and embeddings, zero biases, unit LN scales, both c_proj kernels
    N(0, 0.02 / sqrt(2 L)) (jax_gpt/models/gpt2/model.py:328-379)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    out = {}
    for name, shape in param_shapes(cfg).items():
        if name.endswith(".bias"):
            t = torch.zeros(shape)
        elif name.endswith(".scale"):
            t = torch.ones(shape)
        else:
            std = 0.02 / math.sqrt(2 * cfg.n_layers) if "c_proj.kernel" in name else 0.02
            t = torch.randn(shape, generator=g) * std
        out[name] = t.to(device=device, dtype=dtype)
    return out


@dataclass
class KVCache:
    """Stacked cache: key/value (L, B, H, d_context, dh); pos = number of filled positions."""
    key: torch.Tensor
    value: torch.Tensor
    pos: int


class GPT:
    """GPT-2. ``model(x)`` returns ``(logits, cache)``; parameters live in ``self.params``."""

    def __init__(self, config: GPTConfig, *, rngs=None, init_mesh=None, seed: Optional[int] = None, device="cpu",
                 dtype=torch.float32):
        self.config = config
        if seed is None:
            seed = int(rngs) if isinstance(rngs, int) else 0
        self.params = init_params(config, seed, device, dtype)
        self.training = False

    # -- small conveniences ----------------------------------------------------------------
    def parameters(self):
        return list(self.params.values())

    def named_parameters(self):
        return list(self.params.items())

    def to(self, device=None, dtype=None):
        self.params = {k: v.to(device=device, dtype=dtype) for k, v in self.params.items()}
        return self

    def requires_grad_(self, flag: bool = True):
        for v in self.params.values():
            v.requires_grad_(flag)
        return self

    def state_dict(self):
        return {k: v.detach() for k, v in self.params.items()}

    def load_state_dict(self, sd):
        for k, v in sd.items():
            with torch.no_grad():
                self.params[k].copy_(v.to(self.params[k].dtype))

    # -- forward ------------------------------------------------------------------------------
    def _block(self, l, x, cache_k, cache_v, pos, acts, tp_group=None, drop: float = 0.0):
        """``tp_group`` with sharded projections (trainer/sharding.py): this rank's heads and its slice of the MLP,
        row-parallel outputs summed over the group, their biases added once after the sum."""
        from ...parallel.tp_ops import copy_to_tp, reduce_from_tp
        p, cfg = self.params, self.config
        B, T, d = x.shape
        dh = cfg.d_head
        dl = p["h.attn.c_attn.kernel"].shape[-1] // 3        # local width of q, k and v
        H = dl // dh
        tp = tp_group if dl < d else None
        h1 = norm_ops.layer_norm(x, p["h.ln_1.layer_norm.scale"][l], p["h.ln_1.layer_norm.bias"][l], 1e-5)
        qkv = gemm_ops.linear(copy_to_tp(h1, tp), p["h.attn.c_attn.kernel"][l], p["h.attn.c_attn.bias"][l])
        q, k, v = [t.unflatten(-1, (H, dh)) for t in qkv.split(dl, dim=-1)]
        new_k = new_v = None
        if cache_k is not None:
            # cache layout (B, H, ctx, dh); write the new rows, attend over the filled prefix
            cache_k[:, :, pos:pos + T] = k.permute(0, 2, 1, 3)
            cache_v[:, :, pos:pos + T] = v.permute(0, 2, 1, 3)
            if T == 1:
                y = attn_ops.attention_decode(q[:, 0], cache_k, cache_v, kv_len=pos + 1)[:, None]
            elif pos == 0:
                y = attn_ops.attention(q, k, v, causal=True)
            else:
                y = attn_ops.attention_cached(q, cache_k, cache_v, pos + T, pos)
            new_k, new_v = cache_k, cache_v
        elif drop > 0.0:
            # dropout on the attention probabilities (jax_gpt/models/gpt2/model.py:175) cannot pass through the
            # flash kernels, which never materialise them: the stock fused attention applies it
            y = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                               dropout_p=drop, is_causal=True).transpose(1, 2)
        else:
            y = attn_ops.attention(q, k, v, causal=True)
        if tp is None:
            a = gemm_ops.linear(y.reshape(B, T, dl), p["h.attn.c_proj.kernel"][l], p["h.attn.c_proj.bias"][l])
        else:
            a = reduce_from_tp(gemm_ops.linear(y.reshape(B, T, dl), p["h.attn.c_proj.kernel"][l]), tp) \
                + p["h.attn.c_proj.bias"][l]
        x = x + F.dropout(a, drop, training=drop > 0.0)
        h2 = norm_ops.layer_norm(x, p["h.ln_2.layer_norm.scale"][l], p["h.ln_2.layer_norm.bias"][l], 1e-5)
        mlp_tp = tp_group if p["h.mlp.c_fc.kernel"].shape[-1] < cfg.d_ff else None
        f = gemm_ops.linear(copy_to_tp(h2, mlp_tp), p["h.mlp.c_fc.kernel"][l], p["h.mlp.c_fc.bias"][l])
        f = gemm_ops.gelu_tanh(f)
        if mlp_tp is None:
            m = gemm_ops.linear(f, p["h.mlp.c_proj.kernel"][l], p["h.mlp.c_proj.bias"][l])
        else:
            m = reduce_from_tp(gemm_ops.linear(f, p["h.mlp.c_proj.kernel"][l]), mlp_tp) + p["h.mlp.c_proj.bias"][l]
        if acts is not None:
            acts[f"block_{l}_ln1_output"] = h1
            acts[f"block_{l}_attn_output_pre_residual"] = a
            acts[f"block_{l}_mlp_output_pre_residual"] = m
        return x + F.dropout(m, drop, training=drop > 0.0), new_k, new_v

    def __call__(self, x, *, deterministic: bool = True, cache: Optional[KVCache] = None,
                 return_activations: bool = False, mesh=None):
        p, cfg = self.params, self.config
        B, T = x.shape
        pos = cache.pos if cache is not None else 0
        assert pos + T <= cfg.d_context, "sequence exceeds d_context"
        acts = {} if return_activations else None
        idx = x.long()
        from ...parallel.tp_ops import copy_to_tp, gather_from_tp, tp_world, vocab_parallel_embedding
        tp_group = getattr(mesh, "group", None) if mesh is not None else None
        vocab_sharded = p["wte.embedding"].shape[0] < cfg.vocab_size
        if (vocab_sharded or p["h.attn.c_attn.kernel"].shape[-1] < 3 * cfg.d_model) and tp_world(tp_group) == 1:
            raise ValueError("the parameters are a tensor-parallel shard: pass mesh=make_mesh(config) "
                             "(trainer/sharding.py) and run one process per shard")
        h = vocab_parallel_embedding(idx, p["wte.embedding"], tp_group, cfg.vocab_size) + p["wpe.embedding"][pos:pos + T]
        # ``deterministic=False`` with ``config.dropout > 0``: embedding, attention-probability and residual dropout
        # as in the reference modules (jax_gpt/models/gpt2/model.py:93-102, 132-180, 234)
        drop = float(cfg.dropout) if (not deterministic and cache is None) else 0.0
        h = F.dropout(h, drop, training=drop > 0.0)
        if acts is not None:
            acts["initial_embedding"] = h
        for l in range(cfg.n_layers):
            ck = cache.key[l] if cache is not None else None
            cv = cache.value[l] if cache is not None else None
            h, _, _ = self._block(l, h, ck, cv, pos, acts, tp_group, drop)
        h = norm_ops.layer_norm(h, p["ln_f.layer_norm.scale"], p["ln_f.layer_norm.bias"], 1e-5)
        if vocab_sharded:
            # tied, vocabulary-parallel head: this rank's logit columns, gathered to whole logits
            logits = gather_from_tp(copy_to_tp(h, tp_group) @ p["wte.embedding"].t(), tp_group, -1)
            logits = logits[..., :cfg.vocab_size]
        else:
            logits = h @ p["wte.embedding"].t()
        new_cache = KVCache(cache.key, cache.value, pos + T) if cache is not None else None
        if acts is not None:
            acts["final_layernorm"] = h
            acts["final_logits"] = logits
            return logits, new_cache, acts
        return logits, new_cache

    # -- generation ----------------------------------------------------------------------------
    def init_cache(self, batch: int, device=None, dtype=torch.float32) -> KVCache:
        cfg = self.config
        device = device or self.params["wte.embedding"].device
        shape = (cfg.n_layers, batch, cfg.n_head, cfg.d_context, cfg.d_head)
        return KVCache(torch.zeros(shape, device=device, dtype=dtype), torch.zeros(shape, device=device, dtype=dtype), 0)

    @torch.no_grad()
    def generate(self, idx, new_tokens: int, temperature: float = 1.0, top_k: Optional[int] = None, *, rngs=None):
        """Returns prompt + continuation, shape (B, T_prompt + new_tokens)
        (jax_gpt/models/gpt2/model.py:381-418). ``rngs``: int seed or torch.Generator."""
        gen = rngs if isinstance(rngs, torch.Generator) else torch.Generator(device="cpu").manual_seed(
            int(rngs) if rngs is not None else 0)
        dtype = self.params["wte.embedding"].dtype
        cache = self.init_cache(idx.shape[0], dtype=dtype)
        logits, cache = self(idx, cache=cache)
        for _ in range(new_tokens):
            nxt = sample_logits(logits[:, -1, :], temperature, top_k, gen)
            idx = torch.cat([idx, nxt.to(idx.dtype)[:, None]], dim=1)
            if idx.shape[1] >= self.config.d_context + 1:
                break
            logits, cache = self(nxt[:, None].to(idx.dtype), cache=cache)
        return idx

    # -- HF import -----------------------------------------------------------------------------
    @classmethod
    def from_hf_state_dict(cls, sd, config: GPTConfig, device="cpu", dtype=torch.float32) -> "GPT":
        """HF GPT2LMHeadModel weights -> stacked tree. HF Conv1D kernels are already (in,out),
        so nothing is transposed (jax_gpt/models/gpt2/model.py:419-465)."""
        m = cls(config, seed=0, device=device, dtype=dtype)
        L = config.n_layers
        get = lambda k: sd[k].detach().to(dtype)
        stack = lambda fmt: torch.stack([get(fmt.format(i)) for i in range(L)])
        new = {
            "wte.embedding": get("transformer.wte.weight"), "wpe.embedding": get("transformer.wpe.weight"),
            "h.ln_1.layer_norm.scale": stack("transformer.h.{}.ln_1.weight"),
            "h.ln_1.layer_norm.bias": stack("transformer.h.{}.ln_1.bias"),
            "h.ln_2.layer_norm.scale": stack("transformer.h.{}.ln_2.weight"),
            "h.ln_2.layer_norm.bias": stack("transformer.h.{}.ln_2.bias"),
            "h.attn.c_attn.kernel": stack("transformer.h.{}.attn.c_attn.weight"),
            "h.attn.c_attn.bias": stack("transformer.h.{}.attn.c_attn.bias"),
            "h.attn.c_proj.kernel": stack("transformer.h.{}.attn.c_proj.weight"),
            "h.attn.c_proj.bias": stack("transformer.h.{}.attn.c_proj.bias"),
            "h.mlp.c_fc.kernel": stack("transformer.h.{}.mlp.c_fc.weight"),
            "h.mlp.c_fc.bias": stack("transformer.h.{}.mlp.c_fc.bias"),
            "h.mlp.c_proj.kernel": stack("transformer.h.{}.mlp.c_proj.weight"),
            "h.mlp.c_proj.bias": stack("transformer.h.{}.mlp.c_proj.bias"),
            "ln_f.layer_norm.scale": get("transformer.ln_f.weight"), "ln_f.layer_norm.bias": get("transformer.ln_f.bias"),
            "lm_head.kernel": get("transformer.wte.weight").t().contiguous(),
        }
        m.load_state_dict(new)
        return m

    @classmethod
    def from_pretrained(cls, model_type: str, override_args=None) -> "GPT":
        from transformers import GPT2LMHeadModel
        cfg = GPTConfig.from_model_type(model_type, **(override_args or {}))
        hf = GPT2LMHeadModel.from_pretrained(model_type)
        return cls.from_hf_state_dict(hf.state_dict(), cfg)

    def compare_activations(self, hf_model, batch_size: int = 2, sequence_length: int = 16, seed: int = 0):
        """Runs the same random tokens through ``hf_model`` (a transformers GPT2LMHeadModel with
        ``gelu_new``) and this model and returns per-site (mean, std, max-abs-diff) rows, the
        forward-hook comparison of jax_gpt/models/gpt2/model.py:467-590."""
        g = torch.Generator().manual_seed(seed)
        tok = torch.randint(0, self.config.vocab_size, (batch_size, sequence_length), generator=g)
        captured = {}
        hooks = []
        def grab(name):
            def fn(_m, _i, o):
                captured[name] = (o[0] if isinstance(o, tuple) else o).detach()
            return fn
        hooks.append(hf_model.transformer.drop.register_forward_hook(grab("initial_embedding")))
        for i, blk in enumerate(hf_model.transformer.h):
            hooks.append(blk.ln_1.register_forward_hook(grab(f"block_{i}_ln1_output")))
            hooks.append(blk.attn.register_forward_hook(grab(f"block_{i}_attn_output_pre_residual")))
            hooks.append(blk.mlp.register_forward_hook(grab(f"block_{i}_mlp_output_pre_residual")))
        hooks.append(hf_model.transformer.ln_f.register_forward_hook(grab("final_layernorm")))
        with torch.no_grad():
            captured["final_logits"] = hf_model(tok).logits
            _, _, acts = self(tok, return_activations=True)
        for h in hooks:
            h.remove()
        rows = []
        for k, v in acts.items():
            ref = captured[k].to(v.dtype)
            rows.append((k, float(v.mean()), float(v.std()), float((v - ref).abs().max())))
        return rows


def sample_logits(logits, temperature: float = 1.0, top_k: Optional[int] = None, generator=None):
    """T <= 0 -> argmax; else logits / T, keep logits >= k-th largest, categorical sample
    (jax_gpt/models/qwen35/model.py:399-416, jax_gpt/models/gpt2/model.py:399-407)."""
    if temperature <= 0:
        return logits.argmax(-1)
    lf = logits.float() / temperature
    if top_k is not None and top_k < lf.shape[-1]:
        kth = lf.topk(top_k, dim=-1).values[..., -1:]
        lf = lf.masked_fill(lf < kth, float("-inf"))
    probs = torch.softmax(lf, dim=-1)
    return torch.multinomial(probs.cpu(), 1, generator=generator).squeeze(-1).to(logits.device)
