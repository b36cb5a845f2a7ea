"""Paged MLA decode attention with absorbed weights: every sequence's new query attends over its
latent cache (512 compressed-KV + 64 rotary-key values per token, 64-token pages).

``mla_paged_decode`` runs the tcgen05 kernel of csrc/mla_decode_sm100.cu on CUDA bf16 inputs with
the DeepSeek-V3 latent shape and the PyTorch restatement elsewhere. The reference has no MLA and no
paged cache (project_plan.md:58).
"""
from __future__ import annotations

import torch

from .. import _ext

_SM_COUNT = {}


def mla_paged_decode_ref(q_lat, cache, layer: int, seq_ids, scale: float, latent: int):
    """q_lat (B,H,W) -> (B,H,latent). fp32 math over the gathered pages."""
    outs = []
    for b, sid in enumerate(seq_ids):
        c = cache.gather(layer, sid).float()                       # (S, W)
        s = (q_lat[b].float() @ c.t()) * scale
        outs.append(torch.softmax(s, dim=-1) @ c[:, :latent])
    return torch.stack(outs).to(q_lat.dtype)


def supports_cuda(q_lat, cache, latent: int) -> bool:
    return (q_lat.is_cuda and q_lat.dtype == torch.bfloat16 and cache.pool.dtype == torch.bfloat16 and latent == 512 and
            cache.width == 576 and cache.page_size == 64)


def mla_paged_decode(q_lat, cache, layer: int, seq_ids, scale: float, latent: int = 512, n_splits: int = 0):
    """q_lat (B,H,576) bf16; ``cache``: a PagedCache whose lengths already include the new token.
    Returns (B,H,512) bf16."""
    if not supports_cuda(q_lat, cache, latent):
        return mla_paged_decode_ref(q_lat, cache, layer, seq_ids, scale, latent)
    B, H, _ = q_lat.shape
    dev = q_lat.device
    if n_splits <= 0:
        sms = _SM_COUNT.setdefault(dev.index, torch.cuda.get_device_properties(dev).multi_processor_count)
        ctas = B * (1 if H <= 16 else (H + 31) // 32)
        longest = max(cache.length(s) for s in seq_ids)
        n_splits = max(1, min(sms // max(ctas, 1), (longest + 127) // 128, 32))   # at least two tiles per CTA
    part_out = torch.empty(2 * B * n_splits * H * 512, device=dev, dtype=torch.float32)   # two softmax groups per split
    part_lse = torch.empty(2 * B * n_splits * H, device=dev, dtype=torch.float32)
    out = torch.empty(B, H, 512, device=dev, dtype=torch.bfloat16)
    _ext.ops().mla_paged_decode(q_lat.contiguous(), cache.pool[layer], cache.block_table, cache.seq_lens,
                                cache.seq_id_tensor(seq_ids), scale, n_splits, part_out, part_lse, out)
    return out
