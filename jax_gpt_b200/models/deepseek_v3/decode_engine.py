"""CUDA-graph decode engine for the DeepSeek-V3 model: one graph replay per generated token.

The eager decode path (model.py:mla_decode_absorbed) does host bookkeeping inside every layer (page
reservation, lengths, rotary positions), which makes a decode step launch-bound. Here the host work
of a step is done ONCE up front - reserve the page of the next token for every sequence, upload the
block table if it changed - and everything else reads its inputs from device memory: rotary
positions and write slots come from the device length vector, the new latent rows are scattered by
the paged-write kernel, attention is the paged MLA kernel, the routed experts are the fused
expert-parallel kernel. The whole token step (all layers, logits, arg-max, length increment) is
captured in a CUDA graph the first time it runs and replayed afterwards.

The reference decodes with one jitted forward per token over a dense cache
(jax_gpt/models/qwen35/model.py:338-396); it has no MLA model.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn.functional as F

from ... import _ext
from ...cache.paged import PagedCache
from ...ops.gemm import linear
from ...ops.router import deepseek_router
from ..qwen35.block import _slice
from ..qwen35.primitives import precompute_rope_freqs
from .config import DeepSeekV3Config
from .model import rms_norm


def _rope_rows(x: torch.Tensor, fr: torch.Tensor) -> torch.Tensor:
    """x (B, H, dr) or (B, dr); fr (B, dr/2, 2): every row has its own position."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half].float(), x[..., half:].float()
    cos, sin = fr[..., 0], fr[..., 1]
    if x.dim() == 3:
        cos, sin = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


class DeepSeekV3DecodeEngine:
    def __init__(self, params: dict, config: DeepSeekV3Config, cache: PagedCache, seq_ids: List[int], ep=None,
                 use_cuda_graph: bool = True, max_len: Optional[int] = None):
        """``cache`` already holds the prompts of ``seq_ids`` (prefill done, lengths committed). ``ep``: an
        expert-parallel dispatcher with ``forward(x, weights, idx, layer_params)`` (required for graphs: the
        single-GPU grouped path sizes its groups on the host)."""
        c = config
        assert c.kv_lora_rank == 512 and c.qk_rope_head_dim == 64 and cache.page_size == 64, "paged MLA kernel shape"
        self.p, self.c, self.cache, self.ep = params, c, cache, ep
        self.seq_ids = list(seq_ids)
        self.B = len(self.seq_ids)
        self.device = cache.pool.device
        self.ids_t = cache.seq_id_tensor(self.seq_ids)
        self.ids_long = self.ids_t.long()
        self.rope = precompute_rope_freqs(c.qk_rope_head_dim, c.max_position_embeddings, c.rope_theta, device=self.device)
        self.tokens = torch.zeros(self.B, device=self.device, dtype=torch.long)
        self.next_tokens = torch.zeros(self.B, device=self.device, dtype=torch.long)
        self.logits = None
        self.use_graph = use_cuda_graph and ep is not None and self.device.type == "cuda"
        self._graph = None
        longest = max_len or (max(cache.length(s) for s in self.seq_ids) + 1024)
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        ctas = self.B * (1 if c.n_heads <= 16 else (c.n_heads + 31) // 32)
        self.n_splits = max(1, min(sms // max(ctas, 1), (longest + 127) // 128, 32))
        H = c.n_heads
        self._part_out = torch.empty(2 * self.B * self.n_splits * H * 512, device=self.device, dtype=torch.float32)
        self._part_lse = torch.empty(2 * self.B * self.n_splits * H, device=self.device, dtype=torch.float32)

    # ---- one layer, everything on the device -----------------------------------------------------
    def _attention(self, x, ap, layer: int, pos):
        c = self.c
        B, H, dn, dr, dv, kvr = self.B, c.n_heads, c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim, c.kv_lora_rank
        q = linear(rms_norm(linear(x, ap["q_a_proj"]), ap["q_a_norm"], c.rms_norm_eps), ap["q_b_proj"]).reshape(B, H, dn + dr)
        kv = linear(x, ap["kv_a_proj_with_mqa"])
        c_kv = rms_norm(kv[:, :kvr].contiguous(), ap["kv_a_norm"], c.rms_norm_eps)
        fr = self.rope.index_select(0, pos)                                   # (B, dr/2, 2)
        q_rope = _rope_rows(q[..., dn:], fr)
        k_rope = _rope_rows(kv[:, kvr:], fr)
        cache = self.cache
        rows = torch.cat([c_kv, k_rope], dim=-1).to(torch.bfloat16).reshape(B, 1, kvr + dr).contiguous()
        ops = _ext.ops()
        ops.paged_kv_write(rows, cache.pool[layer], cache.block_table, self.ids_t, pos.to(torch.int32))
        wkv = ap["kv_b_proj"].reshape(kvr, H, dn + dv)
        q_lat = torch.einsum("bhd,khd->bhk", q[..., :dn], wkv[..., :dn])
        q_full = torch.cat([q_lat, q_rope], dim=-1).contiguous()
        o_lat = torch.empty(B, H, 512, device=x.device, dtype=torch.bfloat16)
        # self._lens1 = lengths + 1: the token written above is attended to as well
        ops.mla_paged_decode(q_full, cache.pool[layer], cache.block_table, self._lens1, self.ids_t, c.softmax_scale,
                             self.n_splits, self._part_out, self._part_lse, o_lat)
        o = torch.einsum("bhk,khd->bhd", o_lat, wkv[..., dn:]).reshape(B, H * dv)
        return linear(o, ap["o_proj"])

    def _ffn(self, h, lp, is_moe: bool):
        c = self.c
        if not is_moe:
            m = lp["mlp"]
            return linear(F.silu(linear(h, m["gate_proj"])) * linear(h, m["up_proj"]), m["down_proj"])
        mp = lp["moe"]
        w, idx = deepseek_router(h, mp["gate_weight"], mp["e_score_correction_bias"], c.n_experts_per_token, c.n_group,
                                 c.topk_group, c.routed_scaling_factor, c.norm_topk_prob)
        if self.ep is not None:
            routed = self.ep.forward(h, w, idx, mp).to(h.dtype)
        else:
            from ..qwen35.moe import expert_forward_single
            routed = expert_forward_single(h, w, idx, mp)
        shared = linear(F.silu(linear(h, mp["shared_gate_proj"])) * linear(h, mp["shared_up_proj"]), mp["shared_down_proj"])
        return routed + shared

    def _token_step(self):
        c, p = self.c, self.p
        # positions of the new tokens = current lengths (device); the full block table row of a sequence is
        # indexed by its id, the length vector likewise
        pos = self.cache.seq_lens.index_select(0, self.ids_long).long()
        self._lens1.copy_(self.cache.seq_lens)
        self._lens1.index_add_(0, self.ids_long, torch.ones_like(self.ids_t))
        x = p["embed"][self.tokens]
        li = 0
        for name, is_moe, n in (("dense_layers", False, c.first_k_dense), ("moe_layers", True, c.n_moe_layers)):
            for i in range(n):
                lp = _slice(p[name], i)
                x = x + self._attention(rms_norm(x, lp["attn_norm"], c.rms_norm_eps), lp["attn"], li, pos)
                x = x + self._ffn(rms_norm(x, lp["ffn_norm"], c.rms_norm_eps), lp, is_moe)
                li += 1
        logits = linear(rms_norm(x, p["final_norm"], c.rms_norm_eps), p["lm_head"])
        self.next_tokens.copy_(logits.argmax(-1))
        self.cache.seq_lens.copy_(self._lens1)           # the step's tokens are now part of the sequences
        return logits

    # ---- public ---------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens (B,) ids of the last generated token of every sequence. Returns the greedy next ids (B,)
        (a device tensor that the next call may consume directly); ``self.logits`` holds the step's logits."""
        cache = self.cache
        # host part: make sure every sequence owns the page of its next token, then advance the host lengths
        lens = [cache.length(s) for s in self.seq_ids]
        cache._tab.reserve(self.seq_ids, [n + 1 for n in lens])
        if cache._tab.version != cache._synced:
            cache.block_table.copy_(cache._tab.table, non_blocking=True)
            cache._synced = cache._tab.version
        self.tokens.copy_(tokens)
        if not hasattr(self, "_lens1"):
            self._lens1 = torch.zeros_like(cache.seq_lens)
        if not self.use_graph:
            self.logits = self._token_step()
        elif self._graph is None:
            # one eager step on a side stream first (kernel attributes, symmetric buffers, allocator), then capture
            saved = cache.seq_lens.clone()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._token_step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            cache.seq_lens.copy_(saved)                  # the warm-up wrote the same rows the real step rewrites
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self.logits = self._token_step()
            cache.seq_lens.copy_(saved)                  # capture does not execute; replay does the real step
            self._graph.replay()
        else:
            self._graph.replay()
        # the device lengths were advanced inside the step; mirror that on the host without another upload
        cache._tab.advance(self.seq_ids, 1)
        cache._synced = cache._tab.version
        return self.next_tokens
