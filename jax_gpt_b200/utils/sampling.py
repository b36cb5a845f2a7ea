"""Next-token sampling: argmax / temperature / top-k / top-p / presence penalty.

Rules of the reference's evaluation sampler (scripts/eval_humaneval.py:279-307): the presence
penalty is subtracted from the logits of tokens already seen; ``temperature <= 0`` means
argmax; top-k keeps logits >= the k-th largest; top-p keeps logits >= the value at the first
position where the cumulative probability of the descending-sorted distribution reaches
``top_p``; the survivor set is sampled categorically.
"""
from __future__ import annotations

from typing import Optional

import torch


def filter_logits(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.0,
                  presence_penalty: float = 0.0, presence_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """logits (B, V) -> fp32 scaled logits with rejected entries at -inf."""
    lf = logits.float()
    if presence_penalty > 0.0 and presence_mask is not None:
        lf = lf - presence_penalty * presence_mask.to(lf.dtype)
    if temperature <= 0.0:
        return lf
    lf = lf / temperature
    neg = torch.finfo(torch.float32).min
    if top_k and top_k < lf.shape[-1]:
        kth = lf.sort(dim=-1, descending=True).values[..., top_k - 1:top_k]
        lf = torch.where(lf >= kth, lf, torch.full_like(lf, neg))
    if top_p and top_p > 0.0:
        srt = lf.sort(dim=-1, descending=True).values
        cum = torch.softmax(srt, dim=-1).cumsum(-1)
        cut = torch.searchsorted(cum, torch.full_like(cum[..., :1], top_p)).clamp_max(lf.shape[-1] - 1)
        cutoff = srt.gather(-1, cut)
        lf = torch.where(lf >= cutoff, lf, torch.full_like(lf, neg))
    return lf


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.0,
           presence_penalty: float = 0.0, presence_mask: Optional[torch.Tensor] = None, generator=None) -> torch.Tensor:
    """Returns (B,) token ids."""
    lf = filter_logits(logits, temperature, top_k, top_p, presence_penalty, presence_mask)
    if temperature <= 0.0:
        return lf.argmax(-1)
    probs = torch.softmax(lf, dim=-1)
    return torch.multinomial(probs.cpu(), 1, generator=generator).squeeze(-1).to(logits.device)
