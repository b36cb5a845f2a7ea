"""CUDA-graph decode engine for the Qwen3.5-style hybrid model: one graph replay per generated token.

The function-style decode (model.py:forward with ``is_decode=True``) rebuilds the cache object every step
(stacking all recurrent states), passes the position as a host integer and launches a few hundred small
kernels, so a token step is bound by the host. Here the state lives in place and everything a step needs is in
device memory:

* the Gated-DeltaNet states and conv windows are fp32 buffers updated in place by the fused decode kernel
  (csrc/seq_kernels.cu: conv window, gates, delta rule, gated RMSNorm in one launch per layer);
* the position is a device scalar: rotary angles are gathered with it, the new key / value row is written with
  ``index_copy_`` and the attention of the gated-attention layers is the split-KV decode kernel
  (csrc/attention_decode.cu), which reads the number of valid keys from that scalar, so every shape is static;
* the routed experts go through the fused dispatch / grouped GEMM / combine kernel when an expert runtime is
  given (a launch per expert otherwise, which cannot be captured: the engine then runs eagerly);
* projections that share their input run as one GEMM over weights concatenated once at construction (the four
  DeltaNet input projections, attention q | k | v, the shared expert's gate | up); the fused decode kernel reads
  the column slices of that GEMM's output in place;
* embedding, all layers, the head, the arg-max and the position increment are captured in one CUDA graph the
  first time a step runs and replayed afterwards.

The reference decodes with one jitted forward per token over the same dense cache
(jax_gpt/models/qwen35/model.py:338-396, block.py:19-137, gqa.py:60-119, deltanet.py decode step).
"""
from __future__ import annotations

from typing import Optional

import torch

from ...ops import attention as attn_ops
from .block import _slice
from .cache import HybridCache
from .config import Qwen35Config
from .deltanet import deltanet_recurrent_step
from .fp8 import matmul_maybe_fp8
from .moe import moe_layer
from .primitives import apply_rotary_emb, precompute_rope_freqs, rms_norm


class Qwen35DecodeEngine:
    def __init__(self, params: dict, config: Qwen35Config, cache: HybridCache, ep=None, use_cuda_graph: bool = True,
                 paged_kv: bool = False):
        """``cache`` holds the prompts (prefill done); its key / value buffers are used in place, the recurrent
        states are copied once into fp32 buffers. ``ep``: callable expert runtime
        (parallel/expert_parallel.py:EPMoEInferenceRuntime) or None. ``paged_kv``: the gated-attention layers keep
        their keys and values in a paged cache (cache/paged.py: 64-token pages, block table, per-sequence lengths;
        one pool row = K of both kv heads, then V) instead of the dense buffers: the prompt rows are copied into
        pages here, a step scatters the new row with ``paged_kv_write`` and attends through the block table."""
        c = config
        self.p, self.c, self.ep = params, c, ep
        self.device = cache.gqa_k.device
        self.B = cache.gqa_k.shape[1]
        self.max_len = cache.gqa_k.shape[3]
        self.M = cache.delta_M.float().contiguous()          # (G, nd, B, Hv, dk, dv)
        self.conv = cache.delta_conv.float().contiguous()    # (G, nd, B, conv_dim, K)
        self.k, self.v = cache.gqa_k, cache.gqa_v            # (G, B, Hkv, max_len, dh)
        act_dtype = params["embed"].dtype
        if self.device.type == "cuda" and act_dtype == torch.bfloat16 and self.k.dtype != torch.bfloat16:
            # the decode kernel streams a bf16 cache; a cache of another type is converted once and owned here
            self.k, self.v = self.k.to(torch.bfloat16), self.v.to(torch.bfloat16)
        self.pos = int(cache.pos)
        self.pos_t = torch.tensor([self.pos], device=self.device, dtype=torch.long)
        self.pos_i32 = torch.tensor([self.pos], device=self.device, dtype=torch.int32)
        n_splits = attn_ops.decode_splits(self.B, c.gqa_n_kv_heads, self.max_len)
        self.dec_scratch = (torch.empty(self.B, c.gqa_n_q_heads, n_splits, c.gqa_head_dim, device=self.device,
                                        dtype=torch.float32),
                            torch.empty(self.B, c.gqa_n_q_heads, n_splits, 2, device=self.device, dtype=torch.float32))
        self.rope = precompute_rope_freqs(c.gqa_rope_dim, self.max_len, c.gqa_rope_theta, device=self.device)
        self.tokens = torch.zeros(self.B, device=self.device, dtype=torch.long)
        self.next_tokens = torch.zeros(self.B, device=self.device, dtype=torch.long)
        self.logits = None
        self.use_graph = bool(use_cuda_graph) and self.device.type == "cuda" and callable(ep)
        self._graph = None
        self._layers = self._build_layers()
        self.paged = None
        if paged_kv:
            from ...cache.paged import PagedCache
            ps = 64
            per_seq = (self.max_len + ps - 1) // ps
            Hkv, dh = c.gqa_n_kv_heads, c.gqa_head_dim
            self.paged = PagedCache(c.n_groups, 2 * Hkv * dh, n_pages=self.B * per_seq, page_size=ps, max_seqs=self.B,
                                    max_pages_per_seq=per_seq, dtype=self.k.dtype, device=self.device)
            self.seq_ids = list(range(self.B))
            for sid in self.seq_ids:                      # every page a sequence can ever need: the table is static
                self.paged.reserve(sid, self.max_len)
            if self.pos > 0:
                for gi in range(c.n_groups):              # (B, Hkv, pos, dh) x 2 -> rows (B, pos, 2 Hkv dh)
                    kk = self.k[gi][:, :, :self.pos].permute(0, 2, 1, 3).reshape(self.B, self.pos, Hkv * dh)
                    vv = self.v[gi][:, :, :self.pos].permute(0, 2, 1, 3).reshape(self.B, self.pos, Hkv * dh)
                    self.paged.append(gi, self.seq_ids, torch.cat([kk, vv], dim=-1))
                self.paged.commit(self.seq_ids, self.pos)
            self.seq_id_t = self.paged.seq_id_tensor(self.seq_ids)
            self.paged_lens = self.paged.seq_lens.clone()     # advanced on the device inside the captured step
            self.k = self.v = None                            # the dense buffers are not used any more

    def _build_layers(self):
        """Per-layer parameter dicts, sliced once, with the projections that share an input concatenated so that a
        token step launches one GEMM where the function-style model launches four (DeltaNet q|k|v, z, b, a), three
        (attention q, k, v) or two (shared expert gate, up). Only plain tensors are merged (FP8 dicts stay apart)."""
        c, p = self.c, self.p
        plain = lambda *ts: all(torch.is_tensor(t) for t in ts)
        def merge_moe(moe):
            moe = dict(moe)
            if plain(moe["shared_gate_proj"], moe["shared_up_proj"]):
                moe["shared_gate_up_proj"] = torch.cat([moe["shared_gate_proj"], moe["shared_up_proj"]], dim=1).contiguous()
            return moe
        layers = []
        for gi in range(c.n_groups):
            gp = _slice(p["groups"], gi)
            delta = []
            for i in range(c.n_delta_per_group):
                lp = dict(_slice(gp["delta_layers"], i))
                ap = dict(lp["attn"])
                if plain(ap["in_proj_qkv"], ap["in_proj_z"], ap["in_proj_b"], ap["in_proj_a"]):
                    ap["in_proj_all"] = torch.cat([ap["in_proj_qkv"], ap["in_proj_z"], ap["in_proj_b"], ap["in_proj_a"]],
                                                  dim=1).contiguous()
                lp["attn"], lp["moe"] = ap, merge_moe(lp["moe"])
                delta.append(lp)
            gl = dict(gp["gqa_layer"])
            ap = dict(gl["attn"])
            if plain(ap["q_proj"], ap["k_proj"], ap["v_proj"]):
                ap["qkv_proj"] = torch.cat([ap["q_proj"], ap["k_proj"], ap["v_proj"]], dim=1).contiguous()
            gl["attn"], gl["moe"] = ap, merge_moe(gl["moe"])
            layers.append((delta, gl))
        return layers

    # ---- layers (x is (B, D)) -------------------------------------------------------------------------
    def _moe(self, x, lp):
        c = self.c
        h = rms_norm(x, lp["moe_norm"], c.rms_norm_eps)
        return x + moe_layer(h[:, None, :], lp["moe"], c.n_experts_per_token, group=self.ep,
                             n_experts=c.n_routed_experts)[:, 0]

    def _delta_layer(self, x, lp, gi: int, i: int):
        c = self.c
        h = rms_norm(x, lp["attn_norm"], c.rms_norm_eps)
        state, conv = self.M[gi, i], self.conv[gi, i]
        a, new_state, new_conv = deltanet_recurrent_step(h[:, None, :], lp["attn"], state, conv, c.delta_n_qk_heads,
                                                         c.delta_n_v_heads, c.delta_qk_head_dim, c.delta_v_head_dim)
        if new_state.data_ptr() != state.data_ptr():         # library path returns new tensors; the kernel works in place
            state.copy_(new_state)
            conv.copy_(new_conv)
        return self._moe(x + a[:, 0], lp)

    def _gqa_layer(self, x, lp, gi: int):
        c, ap = self.c, lp["attn"]
        B, Hq, Hkv, dh = self.B, c.gqa_n_q_heads, c.gqa_n_kv_heads, c.gqa_head_dim
        h = rms_norm(x, lp["attn_norm"], c.rms_norm_eps)
        if "qkv_proj" in ap:
            qkv = matmul_maybe_fp8(h, ap["qkv_proj"])
            nq, nk = 2 * Hq * dh, Hkv * dh
            qg = qkv[:, :nq].reshape(B, 1, Hq, 2 * dh)
            k = qkv[:, nq:nq + nk].reshape(B, 1, Hkv, dh)
            v = qkv[:, nq + nk:].reshape(B, 1, Hkv, dh)
        else:
            qg = matmul_maybe_fp8(h, ap["q_proj"]).reshape(B, 1, Hq, 2 * dh)
            k = matmul_maybe_fp8(h, ap["k_proj"]).reshape(B, 1, Hkv, dh)
            v = matmul_maybe_fp8(h, ap["v_proj"]).reshape(B, 1, Hkv, dh)
        q, gate = qg[..., :dh], qg[..., dh:]
        fr = self.rope.index_select(0, self.pos_t)                                   # (1, rope_dim/2, 2)
        q = apply_rotary_emb(rms_norm(q.contiguous(), ap["q_norm"]), fr, c.gqa_rope_dim)
        k = apply_rotary_emb(rms_norm(k.contiguous(), ap["k_norm"]), fr, c.gqa_rope_dim)
        if self.paged is not None:
            pc = self.paged
            row = torch.cat([k.reshape(B, 1, Hkv * dh), v.reshape(B, 1, Hkv * dh)], dim=-1).to(pc.pool.dtype)
            if row.is_cuda:
                pc._ops.paged_kv_write(row.contiguous(), pc.pool[gi], pc.block_table, self.seq_id_t, self.paged_lens)
            else:
                for b in range(B):
                    pg, of = pc.slots(b, self.pos, 1)
                    pc.pool[gi, pg, of] = row[b]
            o = attn_ops.attention_decode_paged(q.reshape(B, Hq, dh), pc.pool[gi], pc.block_table, self.seq_id_t,
                                                self.paged_lens, Hkv, len_add=1, scratch=self.dec_scratch,
                                                max_len=self.max_len)
        else:
            ck, cv = self.k[gi], self.v[gi]                                          # (B, Hkv, max_len, dh)
            ck.index_copy_(2, self.pos_t, k.permute(0, 2, 1, 3).to(ck.dtype))
            cv.index_copy_(2, self.pos_t, v.permute(0, 2, 1, 3).to(cv.dtype))
            o = attn_ops.attention_decode(q.reshape(B, Hq, dh), ck, cv, pos=self.pos_i32, scratch=self.dec_scratch)
        o = (o.float() * torch.sigmoid(gate[:, 0].float())).to(x.dtype)
        return self._moe(x + matmul_maybe_fp8(o.reshape(B, Hq * dh), ap["o_proj"]), lp)

    def _token_step(self):
        c, p = self.c, self.p
        x = p["embed"][self.tokens]
        for gi, (delta, gqa) in enumerate(self._layers):
            for i, lp in enumerate(delta):
                x = self._delta_layer(x, lp, gi, i)
            x = self._gqa_layer(x, gqa, gi)
        logits = matmul_maybe_fp8(rms_norm(x, p["final_norm"], c.rms_norm_eps), p["lm_head"])
        self.next_tokens.copy_(logits.argmax(-1))
        self.pos_t.add_(1)
        self.pos_i32.add_(1)
        if self.paged is not None:
            self.paged_lens.add_(1)
        return logits

    # ---- public ---------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens (B,): the last token of every sequence. Returns the greedy next tokens (B,), a device tensor
        the next call may take directly; ``self.logits`` (B, V) are the step's logits."""
        assert self.pos < self.max_len, "the cache is full"
        self.tokens.copy_(tokens.reshape(-1))
        if not self.use_graph:
            self.logits = self._token_step()
        elif self._graph is None:
            # one eager step on a side stream first (kernel attributes, symmetric buffers, allocator), undone
            # afterwards: the recurrent states and the position are restored, the rewritten cache row is the same
            saved = (self.M.clone(), self.conv.clone(), self.pos_t.clone())
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._token_step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.M.copy_(saved[0])
            self.conv.copy_(saved[1])
            self.pos_t.copy_(saved[2])
            self.pos_i32.copy_(saved[2])
            if self.paged is not None:
                self.paged_lens.sub_(1)
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self.logits = self._token_step()
            self._graph.replay()                      # capture does not execute; the replay is the real step
        else:
            self._graph.replay()
        self.pos += 1
        return self.next_tokens

    def cache(self, dtype: Optional[torch.dtype] = None) -> HybridCache:
        """The state as a ``HybridCache`` (to continue with the function-style forward)."""
        if self.paged is not None:
            raise RuntimeError("a paged engine has no dense key / value buffers to hand back")
        dt = dtype or self.k.dtype
        return HybridCache(self.M.to(dt), self.conv.to(dt), self.k, self.v, self.pos)


@torch.no_grad()
def generate_with_engine(params, prompt_tokens, config: Qwen35Config, max_new_tokens: int,
                         max_seq_len: Optional[int] = None, temperature: float = 1.0, top_k: Optional[int] = None,
                         key=None, cache_dtype=None, ep=None, use_cuda_graph: bool = True):
    """Same contract as ``model.generate`` (returns ONLY the continuation, shape (B, max_new_tokens); same
    sampler and random stream), with the decode steps on the in-place engine: prefill through ``forward``, then
    one engine step (a CUDA-graph replay when ``ep`` is given on a GPU) per token, sampling from its logits."""
    from .cache import init_cache
    from .model import _sample, forward
    B, T = prompt_tokens.shape
    max_seq_len = max_seq_len or (T + max_new_tokens)
    gen = key if isinstance(key, torch.Generator) else torch.Generator().manual_seed(int(key) if key is not None else 0)
    dtype = cache_dtype or params["embed"].dtype
    cache = init_cache(config, B, max_seq_len, dtype=dtype, device=prompt_tokens.device)
    logits, cache = forward(params, prompt_tokens, config, cache=cache, is_decode=False, ep_group=ep)
    nxt = _sample(logits[:, -1], temperature, top_k, gen)
    out = [nxt]
    if max_new_tokens > 1:
        eng = Qwen35DecodeEngine(params, config, cache, ep=ep, use_cuda_graph=use_cuda_graph)
        for _ in range(max_new_tokens - 1):
            eng.step(nxt)
            nxt = _sample(eng.logits, temperature, top_k, gen)
            out.append(nxt)
    return torch.stack(out, dim=1)
