"""DeepSeek-V3-style model: MLA attention, group-limited sigmoid router, MoE with a shared expert.

Parameter tree (nested dict, (in,out) kernels, homogeneous runs stacked on a leading axis)::

    embed (V,D)  final_norm (D)  lm_head (D,V)
    dense_layers.{attn_norm, ffn_norm (Ld,D), attn.*, mlp.{gate_proj, up_proj (Ld,D,I), down_proj (Ld,I,D)}}
    moe_layers.{attn_norm, ffn_norm (Lm,D), attn.*, moe.{gate_weight (Lm,D,E), e_score_correction_bias (Lm,E),
                gate_proj, up_proj (Lm,E,D,I), down_proj (Lm,E,I,D), shared_gate_proj, shared_up_proj (Lm,D,SI),
                shared_down_proj (Lm,SI,D)}}
    attn.* = q_a_proj (D,qr)  q_a_norm (qr)  q_b_proj (qr,H*(dn+dr))  kv_a_proj_with_mqa (D,kvr+dr)
             kv_a_norm (kvr)  kv_b_proj (kvr,H*(dn+dv))  o_proj (H*dv,D)

MLA: ``q = q_b(norm(q_a(x)))`` split per head into [nope | rope]; ``kv_a(x)`` gives the
compressed KV ``c`` and ONE rotary key shared by all heads; ``kv_b(norm(c))`` gives per-head
[k_nope | v]. Prefill attends with the decompressed keys/values; decode absorbs ``W_uk`` into
the query and ``W_uv`` into the output and attends over the cached 576-wide latent
(post-norm ``c`` + post-RoPE key) held in 64-token pages. RoPE pairs features half-split.
RMSNorm multiplies by ``w`` (init 1). Router: sigmoid scores, selection on score + bias,
groups ranked by the sum of their top-2, top-k over the kept groups, weights = unbiased
scores normalised to 1 and multiplied by ``routed_scaling_factor``.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn.functional as F

from ...cache.paged import PagedCache
from ...ops import attention as attn_ops
from ...ops import grouped_gemm
from ...ops import norm as norm_ops
from ...ops.gemm import linear
from ...utils.profiling import scope
from ..qwen35.block import _slice
from ..qwen35.primitives import precompute_rope_freqs
from .config import DeepSeekV3Config


def rms_norm(x, w, eps):
    return norm_ops.rms_norm(x, w, eps, one_plus_w=False)


def rope_half_split(x: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """x (..., T, H, dr); freqs (T, dr/2, 2). Rotates pairs (x[i], x[i + dr/2])."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half].float(), x[..., half:].float()
    cos, sin = freqs[:, None, :, 0], freqs[:, None, :, 1]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


# ------------------------------------------------------------------------------------------------
def _attn_params(c: DeepSeekV3Config, lead, n, ones):
    H = c.n_heads
    return {
        "q_a_proj": n(*lead, c.d_model, c.q_lora_rank), "q_a_norm": ones(*lead, c.q_lora_rank),
        "q_b_proj": n(*lead, c.q_lora_rank, H * c.qk_head_dim),
        "kv_a_proj_with_mqa": n(*lead, c.d_model, c.latent_dim), "kv_a_norm": ones(*lead, c.kv_lora_rank),
        "kv_b_proj": n(*lead, c.kv_lora_rank, H * (c.qk_nope_head_dim + c.v_head_dim)),
        "o_proj": n(*lead, H * c.v_head_dim, c.d_model),
    }


def init_params(config: DeepSeekV3Config, key=0, dtype=torch.float32, device="cpu", on_device: bool = False,
                expert_shard=None) -> dict:
    """``on_device=True`` draws every tensor on ``device`` in ``dtype`` (no host copy); ``expert_shard=(rank, world)``
    creates only this rank's routed experts from a stream of their own (see models/qwen35/model.py:init_params)."""
    from ..qwen35.model import _normal
    c = config
    if on_device and torch.device(device).type != "cpu" and not isinstance(key, torch.Generator):
        g = torch.Generator(device=device).manual_seed(int(key))
    else:
        g = key if isinstance(key, torch.Generator) else torch.Generator().manual_seed(int(key))
    dev = dict(device=device, dtype=dtype)
    n = _normal(g, device, dtype)
    e, n_local = n, c.n_routed_experts
    if expert_shard is not None:
        rank, world = expert_shard
        assert c.n_routed_experts % world == 0
        n_local = c.n_routed_experts // world
        e = _normal(torch.Generator(device=g.device).manual_seed((int(g.initial_seed()) + 1) * 1000003 + rank), device, dtype)
    ones = lambda *s: torch.ones(*s, **dev)
    Ld, Lm, D = c.first_k_dense, c.n_moe_layers, c.d_model
    E, I, SI = c.n_routed_experts, c.moe_intermediate_size, c.moe_intermediate_size * c.n_shared_experts
    p = {"embed": n(c.vocab_size, D), "final_norm": ones(D), "lm_head": n(D, c.vocab_size)}
    if Ld:
        p["dense_layers"] = {
            "attn_norm": ones(Ld, D), "ffn_norm": ones(Ld, D), "attn": _attn_params(c, (Ld,), n, ones),
            "mlp": {"gate_proj": n(Ld, D, c.dense_intermediate_size), "up_proj": n(Ld, D, c.dense_intermediate_size),
                    "down_proj": n(Ld, c.dense_intermediate_size, D)},
        }
    if Lm:
        p["moe_layers"] = {
            "attn_norm": ones(Lm, D), "ffn_norm": ones(Lm, D), "attn": _attn_params(c, (Lm,), n, ones),
            "moe": {"gate_weight": n(Lm, D, E), "e_score_correction_bias": torch.zeros(Lm, E, **dev),
                    "gate_proj": e(Lm, n_local, D, I), "up_proj": e(Lm, n_local, D, I), "down_proj": e(Lm, n_local, I, D),
                    "shared_gate_proj": n(Lm, D, SI), "shared_up_proj": n(Lm, D, SI), "shared_down_proj": n(Lm, SI, D)},
        }
    return p


# ------------------------------------------------------------------------------------------------
def route_tokens(x: torch.Tensor, gate_weight, bias, c: DeepSeekV3Config):
    """x (M,D) -> (weights (M,k) fp32, expert ids (M,k))."""
    from ...ops.router import deepseek_router
    return deepseek_router(x, gate_weight, bias, c.n_experts_per_token, c.n_group, c.topk_group,
                           c.routed_scaling_factor, c.norm_topk_prob)


def swiglu_mlp(x, gate, up, down):
    return linear(F.silu(linear(x, gate)) * linear(x, up), down)


def moe_ffn(x: torch.Tensor, mp, c: DeepSeekV3Config, ep=None) -> torch.Tensor:
    """x (B,T,D). ``ep``: an expert-parallel dispatcher (parallel/expert_parallel.py) or None."""
    B, T, D = x.shape
    xf = x.reshape(B * T, D)
    with scope("moe_routing"):
        w, idx = route_tokens(xf, mp["gate_weight"], mp["e_score_correction_bias"], c)
    with scope("moe_experts"):
        if ep is not None:
            routed = ep.forward(xf, w, idx, mp).to(x.dtype)
        else:
            from ..qwen35.moe import expert_forward_single
            routed = expert_forward_single(xf, w, idx, mp)
    with scope("moe_shared_expert"):
        shared = swiglu_mlp(xf, mp["shared_gate_proj"], mp["shared_up_proj"], mp["shared_down_proj"])
    return (routed + shared).reshape(B, T, D)


# ------------------------------------------------------------------------------------------------
def mla_project(x, ap, c: DeepSeekV3Config, rope, pos0: int):
    """Returns q_nope (B,T,H,dn), q_rope (B,T,H,dr) rotated, c_kv (B,T,kvr) normed, k_rope (B,T,dr) rotated."""
    B, T, _ = x.shape
    H, dn, dr = c.n_heads, c.qk_nope_head_dim, c.qk_rope_head_dim
    q = linear(rms_norm(linear(x, ap["q_a_proj"]), ap["q_a_norm"], c.rms_norm_eps), ap["q_b_proj"])
    q = q.reshape(B, T, H, dn + dr)
    kv = linear(x, ap["kv_a_proj_with_mqa"])
    c_kv = rms_norm(kv[..., :c.kv_lora_rank].contiguous(), ap["kv_a_norm"], c.rms_norm_eps)
    fr = rope[pos0:pos0 + T]
    q_rope = rope_half_split(q[..., dn:], fr)
    k_rope = rope_half_split(kv[..., c.kv_lora_rank:].reshape(B, T, 1, dr), fr)[:, :, 0]
    return q[..., :dn], q_rope, c_kv, k_rope


def mla_prefill(x, ap, c: DeepSeekV3Config, rope, pos0: int = 0):
    """Causal MLA over the tokens of ``x`` with decompressed K/V. Returns (out (B,T,D), latent (B,T,kvr+dr))."""
    B, T, _ = x.shape
    H, dn, dr, dv = c.n_heads, c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim
    q_nope, q_rope, c_kv, k_rope = mla_project(x, ap, c, rope, pos0)
    kvb = linear(c_kv, ap["kv_b_proj"]).reshape(B, T, H, dn + dv)
    k = torch.cat([kvb[..., :dn], k_rope[:, :, None, :].expand(B, T, H, dr)], dim=-1)
    q = torch.cat([q_nope, q_rope], dim=-1)
    v = kvb[..., dn:]
    out = attn_ops.mla_attention(q, k, v, c.softmax_scale)
    y = linear(out.reshape(B, T, H * dv), ap["o_proj"])
    return y, torch.cat([c_kv, k_rope], dim=-1)


def mla_decode_absorbed(x, ap, c: DeepSeekV3Config, rope, cache: PagedCache, layer: int, seq_ids: List[int]):
    """One new token per sequence over the paged latent cache (weights absorbed). x (B,1,D).
    The new token's latent is appended to the cache here (lengths are committed once per model step)."""
    from ...ops.mla_decode import mla_paged_decode
    B = x.shape[0]
    H, dn, dr, dv, kvr = c.n_heads, c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim, c.kv_lora_rank
    wkv = ap["kv_b_proj"].reshape(kvr, H, dn + dv)
    w_uk, w_uv = wkv[..., :dn], wkv[..., dn:]          # (kvr,H,dn), (kvr,H,dv)
    lens = [cache.length(s) for s in seq_ids]
    if len(set(lens)) == 1:
        q_nope, q_rope, c_new, k_new = mla_project(x, ap, c, rope, lens[0])
    else:  # ragged batch: every sequence has its own rotary position
        parts = [mla_project(x[b:b + 1], ap, c, rope, lens[b]) for b in range(B)]
        q_nope, q_rope, c_new, k_new = [torch.cat([p[i] for p in parts], dim=0) for i in range(4)]
    cache.append(layer, seq_ids, torch.cat([c_new, k_new], dim=-1))
    # absorb W_uk into the query: (B,H,dn) x (kvr,H,dn) -> (B,H,kvr)
    q_lat = torch.einsum("bhd,khd->bhk", q_nope[:, 0], w_uk.to(q_nope.dtype))
    q_full = torch.cat([q_lat, q_rope[:, 0]], dim=-1).contiguous()
    if _decode_kernel_ok(q_full, cache, kvr):
        # the kernel reads the lengths from the device: they must count the token appended above
        o_lat = _decode_with_pending_token(q_full, cache, layer, seq_ids, c.softmax_scale)
    else:
        outs = []
        for b, sid in enumerate(seq_ids):
            lat = cache.gather(layer, sid, lens[b] + 1).float()
            s = (q_full[b].float() @ lat.t()) * c.softmax_scale
            outs.append(torch.softmax(s, dim=-1) @ lat[:, :kvr])
        o_lat = torch.stack(outs).to(x.dtype)
    o = torch.einsum("bhk,khd->bhd", o_lat, w_uv.to(o_lat.dtype)).reshape(B, 1, H * dv)
    return linear(o, ap["o_proj"])


def _decode_kernel_ok(q_full, cache, kvr) -> bool:
    from ...ops.mla_decode import supports_cuda
    return supports_cuda(q_full, cache, kvr)


def _decode_with_pending_token(q_full, cache, layer, seq_ids, scale):
    from ...ops.mla_decode import mla_paged_decode
    ids = cache.seq_id_tensor(seq_ids).long()
    cache.seq_lens[ids] += 1          # count the appended, not yet committed token for this launch
    try:
        return mla_paged_decode(q_full, cache, layer, seq_ids, scale, n_splits=_splits_for(cache, seq_ids, q_full))
    finally:
        cache.seq_lens[ids] -= 1


def _splits_for(cache, seq_ids, q_full) -> int:
    B, H, _ = q_full.shape
    sms = torch.cuda.get_device_properties(q_full.device).multi_processor_count
    ctas = B * (1 if H <= 16 else (H + 31) // 32)
    longest = max(cache.length(s) for s in seq_ids) + 1
    return max(1, min(sms // max(ctas, 1), (longest + 127) // 128, 32))


# ------------------------------------------------------------------------------------------------
def _layer(x, lp, c, rope, pos0, is_moe, cache, layer_idx, seq_ids, is_decode, ep):
    with scope("mla_attn"):
        h = rms_norm(x, lp["attn_norm"], c.rms_norm_eps)
        if is_decode:
            a = mla_decode_absorbed(h, lp["attn"], c, rope, cache, layer_idx, seq_ids)
        else:
            a, latent = mla_prefill(h, lp["attn"], c, rope, pos0)
            if cache is not None:
                cache.append(layer_idx, seq_ids, latent)
        x = x + a
    with scope("ffn"):
        h = rms_norm(x, lp["ffn_norm"], c.rms_norm_eps)
        if is_moe:
            x = x + moe_ffn(h, lp["moe"], c, ep)
        else:
            m = lp["mlp"]
            x = x + swiglu_mlp(h, m["gate_proj"], m["up_proj"], m["down_proj"])
    return x


def forward(params, tokens, config: DeepSeekV3Config, cache: Optional[PagedCache] = None,
            seq_ids: Optional[List[int]] = None, is_decode: bool = False, ep=None):
    """tokens (B,T) -> logits (B,T,V). Prefill (``is_decode=False``) starts every listed sequence at
    position 0 and, with a ``cache``, stores the latents; decode takes one token per sequence."""
    c = config
    B, T = tokens.shape
    seq_ids = list(range(B)) if seq_ids is None else seq_ids
    x = params["embed"][tokens.long()]
    rope = precompute_rope_freqs(c.qk_rope_head_dim, c.max_position_embeddings, c.rope_theta, device=x.device)
    li = 0
    for name, is_moe, n in (("dense_layers", False, c.first_k_dense), ("moe_layers", True, c.n_moe_layers)):
        for i in range(n):
            lp = _slice(params[name], i)
            x = _layer(x, lp, c, rope, 0, is_moe, cache, li, seq_ids, is_decode, ep)
            li += 1
    if cache is not None:
        cache.commit(seq_ids, T)
    with scope("output_head"):
        x = rms_norm(x, params["final_norm"], c.rms_norm_eps)
        from ...ops.fp8_linear import fp8_training
        with fp8_training(False):          # the head stays in bf16 also when the layers train in FP8
            return linear(x, params["lm_head"])


def make_cache(config: DeepSeekV3Config, n_pages: int, max_seqs: int, max_pages_per_seq: int, dtype=torch.bfloat16,
               device="cpu") -> PagedCache:
    return PagedCache(config.n_layers, config.latent_dim, n_pages, config.page_size, max_seqs, max_pages_per_seq,
                      dtype, device)


@torch.no_grad()
def generate(params, prompt_tokens, config: DeepSeekV3Config, max_new_tokens: int, temperature: float = 0.0,
             top_k: Optional[int] = None, key=None, cache: Optional[PagedCache] = None):
    """Greedy / sampled continuation (B, max_new_tokens) with the paged latent cache."""
    from ..gpt2.model import sample_logits
    B, T = prompt_tokens.shape
    gen = key if isinstance(key, torch.Generator) else torch.Generator().manual_seed(int(key) if key is not None else 0)
    if cache is None:
        per_seq = (T + max_new_tokens + config.page_size - 1) // config.page_size
        cache = make_cache(config, B * per_seq, B, per_seq, params["embed"].dtype, prompt_tokens.device)
    ids = list(range(B))
    logits = forward(params, prompt_tokens, config, cache, ids)
    nxt = sample_logits(logits[:, -1], temperature, top_k, gen)
    out = [nxt]
    for _ in range(max_new_tokens - 1):
        logits = forward(params, nxt[:, None], config, cache, ids, is_decode=True)
        nxt = sample_logits(logits[:, -1], temperature, top_k, gen)
        out.append(nxt)
    return torch.stack(out, dim=1)


def load_from_hf_state_dict(sd, config: DeepSeekV3Config, dtype=torch.bfloat16, rope_interleave: bool = True) -> dict:
    """HF ``deepseek_v3`` names -> this tree. HF checkpoints store the rotary features of q and k
    interleaved (pairs (2i, 2i+1)); with ``rope_interleave`` they are permuted to the half-split
    order used here, which leaves the attention scores unchanged."""
    c = config
    H, dn, dr = c.n_heads, c.qk_nope_head_dim, c.qk_rope_head_dim
    t = lambda k: sd[k].detach().to(dtype).t().contiguous()
    g = lambda k: sd[k].detach().to(dtype)
    perm = torch.cat([torch.arange(0, dr, 2), torch.arange(1, dr, 2)]) if rope_interleave else torch.arange(dr)

    def attn(pfx):
        qb = t(f"{pfx}.self_attn.q_b_proj.weight").reshape(c.q_lora_rank, H, dn + dr)
        qb = torch.cat([qb[..., :dn], qb[..., dn:][..., perm]], dim=-1).reshape(c.q_lora_rank, H * (dn + dr))
        kva = t(f"{pfx}.self_attn.kv_a_proj_with_mqa.weight")
        kva = torch.cat([kva[:, :c.kv_lora_rank], kva[:, c.kv_lora_rank:][:, perm]], dim=-1)
        return {"q_a_proj": t(f"{pfx}.self_attn.q_a_proj.weight"), "q_a_norm": g(f"{pfx}.self_attn.q_a_layernorm.weight"),
                "q_b_proj": qb.contiguous(), "kv_a_proj_with_mqa": kva.contiguous(),
                "kv_a_norm": g(f"{pfx}.self_attn.kv_a_layernorm.weight"), "kv_b_proj": t(f"{pfx}.self_attn.kv_b_proj.weight"),
                "o_proj": t(f"{pfx}.self_attn.o_proj.weight")}

    from ..qwen35.weight_loader import _stack
    dense, moe = [], []
    for i in range(c.n_layers):
        pfx = f"model.layers.{i}"
        base = {"attn_norm": g(f"{pfx}.input_layernorm.weight"), "ffn_norm": g(f"{pfx}.post_attention_layernorm.weight"),
                "attn": attn(pfx)}
        if i < c.first_k_dense:
            base["mlp"] = {k: t(f"{pfx}.mlp.{k}.weight") for k in ("gate_proj", "up_proj", "down_proj")}
            dense.append(base)
        else:
            I = c.moe_intermediate_size
            if f"{pfx}.mlp.experts.gate_up_proj" in sd:
                gu = sd[f"{pfx}.mlp.experts.gate_up_proj"].detach().to(dtype)
                gate, up = gu[:, :I, :].transpose(1, 2).contiguous(), gu[:, I:, :].transpose(1, 2).contiguous()
                down = sd[f"{pfx}.mlp.experts.down_proj"].detach().to(dtype).transpose(1, 2).contiguous()
            else:
                gate = torch.stack([t(f"{pfx}.mlp.experts.{e}.gate_proj.weight") for e in range(c.n_routed_experts)])
                up = torch.stack([t(f"{pfx}.mlp.experts.{e}.up_proj.weight") for e in range(c.n_routed_experts)])
                down = torch.stack([t(f"{pfx}.mlp.experts.{e}.down_proj.weight") for e in range(c.n_routed_experts)])
            base["moe"] = {"gate_weight": t(f"{pfx}.mlp.gate.weight"),
                           "e_score_correction_bias": g(f"{pfx}.mlp.gate.e_score_correction_bias"),
                           "gate_proj": gate, "up_proj": up, "down_proj": down,
                           "shared_gate_proj": t(f"{pfx}.mlp.shared_experts.gate_proj.weight"),
                           "shared_up_proj": t(f"{pfx}.mlp.shared_experts.up_proj.weight"),
                           "shared_down_proj": t(f"{pfx}.mlp.shared_experts.down_proj.weight")}
            moe.append(base)
    p = {"embed": g("model.embed_tokens.weight"), "final_norm": g("model.norm.weight"), "lm_head": t("lm_head.weight")}
    if dense:
        p["dense_layers"] = _stack(dense)
    if moe:
        p["moe_layers"] = _stack(moe)
    return p
