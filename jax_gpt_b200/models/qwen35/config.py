"""Qwen3.5-style hybrid configuration: Gated-DeltaNet layers with a gated softmax-attention
layer every ``full_attention_interval`` layers, MoE FFN everywhere. Field names and presets
follow jax_gpt/models/qwen35/config.py:12-152; ``ns`` is the training benchmark shape."""
from __future__ import annotations

from dataclasses import dataclass, replace


@dataclass(frozen=True)
class Qwen35Config:
    d_model: int = 4096
    vocab_size: int = 248320
    n_layers: int = 60
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 262144
    full_attention_interval: int = 4
    # gated softmax attention
    gqa_n_q_heads: int = 32
    gqa_n_kv_heads: int = 2
    gqa_head_dim: int = 256
    gqa_partial_rotary_factor: float = 0.25
    gqa_rope_theta: float = 10_000_000.0
    attn_output_gate: bool = True
    # Gated DeltaNet
    delta_n_qk_heads: int = 16
    delta_n_v_heads: int = 64
    delta_qk_head_dim: int = 128
    delta_v_head_dim: int = 128
    delta_conv_kernel: int = 4
    delta_chunk_size: int = 256
    # MoE
    n_routed_experts: int = 512
    n_experts_per_token: int = 10
    moe_intermediate_size: int = 1024
    shared_expert_intermediate_size: int = 1024
    router_aux_loss_coef: float = 0.001
    dtype: str = "bfloat16"

    @classmethod
    def mini(cls) -> "Qwen35Config":
        return cls(d_model=1024, n_layers=8, max_position_embeddings=2048, gqa_n_q_heads=32, gqa_n_kv_heads=2,
                   gqa_head_dim=128, delta_n_qk_heads=16, delta_n_v_heads=64, delta_qk_head_dim=128,
                   delta_v_head_dim=128, delta_chunk_size=4, n_routed_experts=32, n_experts_per_token=2,
                   moe_intermediate_size=512, shared_expert_intermediate_size=512)

    @classmethod
    def mid(cls) -> "Qwen35Config":
        return cls(d_model=4096, n_layers=16, max_position_embeddings=8192, n_routed_experts=16,
                   n_experts_per_token=4, moe_intermediate_size=1024, shared_expert_intermediate_size=1024)

    @classmethod
    def mid_large(cls) -> "Qwen35Config":
        return cls(d_model=4096, n_layers=32, max_position_embeddings=8192, n_routed_experts=64,
                   n_experts_per_token=4, moe_intermediate_size=1024, shared_expert_intermediate_size=1024)

    @classmethod
    def full(cls) -> "Qwen35Config":
        return cls()

    @classmethod
    def ns(cls) -> "Qwen35Config":
        """Training benchmark shape: 48 layers, d 2048, vocab 151936, DeltaNet 16 qk / 32 v heads
        of 128 with chunk 64, attention 16 q / 2 kv heads of 256, 512 experts of 512, top-10."""
        return cls(d_model=2048, vocab_size=151936, n_layers=48, max_position_embeddings=32768, gqa_n_q_heads=16,
                   gqa_n_kv_heads=2, gqa_head_dim=256, delta_n_qk_heads=16, delta_n_v_heads=32,
                   delta_qk_head_dim=128, delta_v_head_dim=128, delta_conv_kernel=4, delta_chunk_size=64,
                   n_routed_experts=512, n_experts_per_token=10, moe_intermediate_size=512,
                   shared_expert_intermediate_size=512)

    @classmethod
    def tiny(cls) -> "Qwen35Config":
        """Unit-test size."""
        return cls(d_model=64, vocab_size=256, n_layers=4, max_position_embeddings=128, gqa_n_q_heads=4,
                   gqa_n_kv_heads=2, gqa_head_dim=32, delta_n_qk_heads=2, delta_n_v_heads=4, delta_qk_head_dim=16,
                   delta_v_head_dim=16, delta_chunk_size=8, n_routed_experts=8, n_experts_per_token=2,
                   moe_intermediate_size=32, shared_expert_intermediate_size=32, dtype="float32")

    def replace(self, **kw) -> "Qwen35Config":
        return replace(self, **kw)

    @property
    def n_groups(self) -> int:
        assert self.n_layers % self.full_attention_interval == 0
        return self.n_layers // self.full_attention_interval

    @property
    def n_delta_per_group(self) -> int:
        return self.full_attention_interval - 1

    @property
    def gqa_rope_dim(self) -> int:
        return int(self.gqa_head_dim * self.gqa_partial_rotary_factor)

    @property
    def delta_key_dim(self) -> int:
        return self.delta_n_qk_heads * self.delta_qk_head_dim

    @property
    def delta_value_dim(self) -> int:
        return self.delta_n_v_heads * self.delta_v_head_dim

    @property
    def delta_conv_dim(self) -> int:
        return 2 * self.delta_key_dim + self.delta_value_dim

    def layer_type(self, layer_idx: int) -> str:
        return "full" if (layer_idx + 1) % self.full_attention_interval == 0 else "linear"
