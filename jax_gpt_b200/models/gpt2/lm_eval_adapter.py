"""lm-evaluation-harness adapter (jax_gpt/models/gpt2/jax_gpt_adapter.py:16-94).

``B200GPTLM`` registers as ``b200_gpt_adapter`` when ``lm_eval`` is importable; the scoring
core :func:`loglikelihood_tokens` is independent of the harness: contexts are left-padded and
continuations right-padded with the end-of-text id, one forward pass scores the batch, the
continuation log-probabilities are summed and checked against the greedy prediction.
``generate_until`` and ``loglikelihood_rolling`` are not provided, as in the reference.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

EOT = 50256


@torch.no_grad()
def loglikelihood_tokens(model, requests: Sequence[Tuple[List[int], List[int]]], batch_size: int = 8,
                         max_len: int = 1024, pad_id: int = EOT) -> List[Tuple[float, bool]]:
    """requests: (context ids, continuation ids). Returns (sum log p(continuation | context), is_greedy)."""
    out = []
    vocab = model.config.vocab_size
    pad_id = pad_id % vocab
    for s in range(0, len(requests), batch_size):
        chunk = requests[s:s + batch_size]
        seqs, spans = [], []
        for ctx, cont in chunk:
            full = (list(ctx) + list(cont))[-(max_len + 1):]
            inp = full[:-1]
            spans.append((len(inp) - len(cont), len(inp)))
            seqs.append(inp)
        L = max(len(x) for x in seqs)
        batch = torch.full((len(seqs), L), pad_id, dtype=torch.long)
        for i, x in enumerate(seqs):
            batch[i, :len(x)] = torch.tensor(x)       # right padding keeps positions of real tokens
        logits, _ = model(batch)
        logp = torch.log_softmax(logits.float(), dim=-1)
        for i, ((ctx, cont), (a, b)) in enumerate(zip(chunk, spans)):
            tgt = torch.tensor(list(cont)[-(b - a):])
            rows = logp[i, a:b]
            ll = rows.gather(-1, tgt[:, None]).sum().item()
            out.append((ll, bool((rows.argmax(-1) == tgt).all())))
    return out


try:  # pragma: no cover - lm_eval is not part of the image
    from lm_eval.api.model import TemplateLM
    from lm_eval.api.registry import register_model

    @register_model("b200_gpt_adapter")
    class B200GPTLM(TemplateLM):
        def __init__(self, model_type: str = "gpt2", batch_size: int = 8, **kw):
            super().__init__()
            from .model import GPT
            import tiktoken
            self.model = GPT.from_pretrained(model_type)
            self.enc = tiktoken.get_encoding("gpt2")
            self.batch_size = int(batch_size)

        @property
        def eot_token_id(self):
            return EOT

        def tok_encode(self, string, **kw):
            return self.enc.encode_ordinary(string)

        def _loglikelihood_tokens(self, requests, **kw):
            return loglikelihood_tokens(self.model, [(c, t) for _, c, t in requests], self.batch_size,
                                        self.model.config.d_context)

        def generate_until(self, requests, **kw):
            raise NotImplementedError

        def loglikelihood_rolling(self, requests, **kw):
            raise NotImplementedError
except ImportError:
    B200GPTLM = None
