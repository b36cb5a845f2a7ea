"""Block-scaled FP8 (e4m3) API in one place: quantisation (1x128 activation blocks, 128x128 weight blocks,
optional power-of-two scales), the two GEMMs (fp32 scales with software promotion; power-of-two scales applied by
the tensor core), the packed exponent-byte layout, the inference layer and the training path.

The implementations live in ops/rope.py (kernels of csrc/seq_kernels.cu, gemm_fp8_sm100.cu, gemm_mxfp8_sm100.cu)
and ops/fp8_linear.py; this module only gathers the names. Reference counterpart: per-row W8A8 inference in
jax_gpt/models/qwen35/fp8.py:50-150 and quantize.py.
"""
from .fp8_linear import fp8_eligible, fp8_enabled, fp8_linear, fp8_training  # noqa: F401
from .rope import (Fp8Linear, fp8_gemm, fp8_gemm_ref, fp8_quant_128x128, fp8_quant_128x128_ref,  # noqa: F401
                   fp8_quant_1x128, fp8_quant_1x128_ref, fp8_quant_mx, mxfp8_gemm, mxfp8_gemm_packed,
                   pack_scales_ue8m0)
