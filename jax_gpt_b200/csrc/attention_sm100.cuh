// Launchers of the tcgen05 flash-attention kernels (see attention_sm100.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// Q, K, V are 2-D bf16 matrices of B*T rows; head h occupies columns [col0 + h*D, +D).
// For a fused qkv activation the three pointers alias one buffer at different column offsets.
struct AttnTensors {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  int64_t ldq, ldk, ldv;  // row strides in elements (multiples of 8)
};

struct AttnShape {
  int B, T, H, Hkv, D;  // forward: D in {64, 128, 256} or (D, Dv) = (192, 128); backward: D in {64, 128}
  float scale;          // softmax scale (1/sqrt(D) by default)
  int causal;
  int Dv;               // v head width when it differs from D (forward only: 192/128 for MLA); 0 = D
};

// out [B*T, ldo] bf16 with head h at columns [h*D, +D); lse [B, H, T] fp32 holds
// log2-sum-exp of the scaled scores (scale * log2(e) folded in).
cudaError_t launch_attn_fwd(const AttnTensors& t, const AttnShape& s, __nv_bfloat16* out, int64_t ldo, float* lse,
                            int* status, cudaStream_t stream);

// Gradients. dq_accum [B*T, H*D] fp32 must be zero on entry (partial sums arrive through
// fp32 reductions); dk / dv are written as bf16 with the strides given. delta [B, H, T] is
// scratch for rowsum(dO * O).
cudaError_t launch_attn_bwd(const AttnTensors& t, const AttnShape& s, const __nv_bfloat16* out, int64_t ldo,
                            const __nv_bfloat16* dout, int64_t lddo, const float* lse, float* delta, float* dq_accum,
                            __nv_bfloat16* dk, int64_t lddk, __nv_bfloat16* dv, int64_t lddv, int* status,
                            cudaStream_t stream);

// dst[r, c] (bf16, row stride ldd) = src[r, c] (fp32, row stride lds), for an M x N block.
// In-place elementwise step of the recomputed attention backward: s [rows, kv] bf16 scores -> probabilities,
// dp [rows, kv] bf16 (dO V^T) -> dS; lse (log2 units) and delta per row; row r is query position q0 + r % c.
cudaError_t launch_attn_bwd_probs(__nv_bfloat16* s, __nv_bfloat16* dp, const float* lse, const float* delta,
                                  int64_t rows, int kv, int c, int q0, float scale, int causal, cudaStream_t stream);

cudaError_t launch_cast_rows_f32_bf16(const float* src, int64_t lds, __nv_bfloat16* dst, int64_t ldd, int M, int N,
                                      cudaStream_t stream);

}  // namespace b200
