"""B200-native LLM framework: GPT-2, Qwen3.5-style hybrid and DeepSeek-V3-style models,
trainer, sampler and benchmarks on hand-written sm_100a kernels."""
__version__ = "0.1.0"
