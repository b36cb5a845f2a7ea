// Launcher of the block-scaled FP8 GEMM (gemm_fp8_sm100.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// out[M,N] = sum_slabs (a_q[M, slab] . b_q[N, slab]^T) * a_scales[M, K/128] * b_scales[ceil(N/128), K/128].
// a_q [M,K] and b_q [N,K] are e4m3 bytes, K contiguous, K % 128 == 0, N % 8 == 0.
cudaError_t launch_gemm_fp8_blockscaled(const uint8_t* a_q, const float* a_scales, const uint8_t* b_q,
                                        const float* b_scales, void* out, int64_t ldo, int out_f32, int M, int N, int K,
                                        int* status, cudaStream_t stream);

// Hardware block-scaled variant (gemm_mxfp8_sm100.cu): the scales are UE8M0 exponent bytes in the packed
// 512-byte-chunk layout described there ([ceil(rows/128), K/128, 512]); out bf16 [M, ldo].
cudaError_t launch_gemm_mxfp8(const uint8_t* a_q, const uint8_t* sfa_packed, const uint8_t* b_q,
                              const uint8_t* sfb_packed, __nv_bfloat16* out, int64_t ldo, int M, int N, int K, int* status,
                              cudaStream_t stream);

}  // namespace b200
