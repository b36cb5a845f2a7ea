"""Offload forward vs the HF reference model (scripts/test_correctness_offload.py:69-191).

Runs the layer-streaming forward of this package and the HF ``Qwen3_5MoeForCausalLM`` forward
(CPU) on the same prompt and reports max / mean absolute logit difference and top-1 / top-5
agreement of the last position. Passes when max diff < 2.0 and the top-1 tokens agree.
``--model-dir`` is an HF safetensors directory; without one a tiny random HF model is built
in memory so the script is runnable offline.
"""
from __future__ import annotations

import argparse
import json

from utils import qwen_config

import torch


def main(argv=None):
    from jax_gpt_b200.models.qwen35.offload import LazySafetensors, forward_offload
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model-dir", default="")
    ap.add_argument("--prompt", default="The capital of France is")
    ap.add_argument("--max-new-tokens", type=int, default=0)
    ap.add_argument("--sharding", default="A")
    ap.add_argument("--n-devices", type=int, default=1)
    ap.add_argument("--skip-hf", action="store_true")
    ap.add_argument("--config", default="tiny")
    args = ap.parse_args(argv)
    cfg = qwen_config(args.config)
    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    hf = None
    if args.model_dir:
        sd = LazySafetensors(args.model_dir)
        if not args.skip_hf:
            from transformers import AutoModelForCausalLM
            hf = AutoModelForCausalLM.from_pretrained(args.model_dir, torch_dtype=torch.bfloat16).eval()
    else:
        from transformers.models.qwen3_5_moe.configuration_qwen3_5_moe import Qwen3_5MoeTextConfig
        from transformers.models.qwen3_5_moe.modeling_qwen3_5_moe import Qwen3_5MoeForCausalLM
        c = cfg
        hc = Qwen3_5MoeTextConfig(
            vocab_size=c.vocab_size, hidden_size=c.d_model, num_hidden_layers=c.n_layers,
            num_attention_heads=c.gqa_n_q_heads, num_key_value_heads=c.gqa_n_kv_heads, head_dim=c.gqa_head_dim,
            max_position_embeddings=128, linear_conv_kernel_dim=c.delta_conv_kernel,
            linear_key_head_dim=c.delta_qk_head_dim, linear_value_head_dim=c.delta_v_head_dim,
            linear_num_key_heads=c.delta_n_qk_heads, linear_num_value_heads=c.delta_n_v_heads,
            moe_intermediate_size=c.moe_intermediate_size,
            shared_expert_intermediate_size=c.shared_expert_intermediate_size,
            num_experts_per_tok=c.n_experts_per_token, num_experts=c.n_routed_experts,
            rope_parameters={"rope_type": "default", "rope_theta": c.gqa_rope_theta, "partial_rotary_factor": 0.25})
        torch.manual_seed(0)
        hf = Qwen3_5MoeForCausalLM(hc).eval().float()
        sd = hf.state_dict()
    ids = [b % cfg.vocab_size for b in args.prompt.encode("utf-8")]
    tok = torch.tensor([ids])
    dtype = torch.float32 if hf is not None and next(hf.parameters()).dtype == torch.float32 else torch.bfloat16
    with torch.no_grad():
        ours, _ = forward_offload(tok.to(device), cfg, None, dtype=dtype, verbose=False, state_dict=sd, device=device)
        ours = ours.float().cpu()
        res = {"tokens": len(ids)}
        if hf is not None and not args.skip_hf:
            ref = hf(tok).logits.float()
            d = (ours - ref).abs()
            t5a, t5b = ours[0, -1].topk(5).indices.tolist(), ref[0, -1].topk(5).indices.tolist()
            res.update(max_abs_diff=float(d.max()), mean_abs_diff=float(d.mean()), top1_match=t5a[0] == t5b[0],
                       top5_overlap=len(set(t5a) & set(t5b)))
            res["passed"] = bool(res["max_abs_diff"] < 2.0 and res["top1_match"])
    print(json.dumps(res))
    return 0 if res.get("passed", True) else 1


if __name__ == "__main__":
    raise SystemExit(main())
