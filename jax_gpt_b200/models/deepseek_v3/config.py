"""DeepSeek-V3-style configuration: MLA attention, group-limited sigmoid-routed MoE with a shared
expert, the first ``first_k_dense`` layers dense SwiGLU. The reference has no such model; widths
follow the public DeepSeek-V3 architecture and the semantics follow the HF ``deepseek_v3``
implementation, which serves as the CPU oracle in the tests."""
from __future__ import annotations

from dataclasses import dataclass, replace


@dataclass(frozen=True)
class DeepSeekV3Config:
    d_model: int = 7168
    vocab_size: int = 129280
    n_layers: int = 61
    first_k_dense: int = 3
    dense_intermediate_size: int = 18432
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 4096
    rope_theta: float = 10000.0
    # MLA
    n_heads: int = 128
    q_lora_rank: int = 1536
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    # MoE
    n_routed_experts: int = 256
    n_experts_per_token: int = 8
    n_group: int = 8
    topk_group: int = 4
    moe_intermediate_size: int = 2048
    n_shared_experts: int = 1
    routed_scaling_factor: float = 2.5
    norm_topk_prob: bool = True
    # cache
    page_size: int = 64
    dtype: str = "bfloat16"

    @property
    def qk_head_dim(self) -> int:
        return self.qk_nope_head_dim + self.qk_rope_head_dim

    @property
    def n_moe_layers(self) -> int:
        return self.n_layers - self.first_k_dense

    @property
    def latent_dim(self) -> int:
        """Width of one cached token: compressed KV plus the shared rotary key."""
        return self.kv_lora_rank + self.qk_rope_head_dim

    @property
    def softmax_scale(self) -> float:
        return self.qk_head_dim ** -0.5

    def replace(self, **kw) -> "DeepSeekV3Config":
        return replace(self, **kw)

    @classmethod
    def full(cls) -> "DeepSeekV3Config":
        """671B shape: 61 layers, first 3 dense."""
        return cls()

    @classmethod
    def eight_layer(cls) -> "DeepSeekV3Config":
        """Training benchmark shape: full widths, 8 layers, layer 0 dense."""
        return cls(n_layers=8, first_k_dense=1)

    @classmethod
    def tiny(cls) -> "DeepSeekV3Config":
        return cls(d_model=64, vocab_size=256, n_layers=3, first_k_dense=1, dense_intermediate_size=128,
                   max_position_embeddings=256, n_heads=4, q_lora_rank=32, kv_lora_rank=32, qk_nope_head_dim=16,
                   qk_rope_head_dim=8, v_head_dim=16, n_routed_experts=16, n_experts_per_token=4, n_group=4,
                   topk_group=2, moe_intermediate_size=32, page_size=4, dtype="float32")
