// Launchers of the bandwidth-bound kernels (see elementwise.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// mode 0: LayerNorm(gamma, beta); 1: RMSNorm * w; 2: RMSNorm * (1 + w). D % 8 == 0, D <= 8192.
cudaError_t launch_norm_fwd(int mode, const __nv_bfloat16* x, const __nv_bfloat16* gamma, const __nv_bfloat16* beta,
                            __nv_bfloat16* y, float* mean, float* rstd, int M, int D, float eps, cudaStream_t st);
// dx = norm_bwd(dy) (+ dres); dgamma/dbeta are ACCUMULATED. `partials` is scratch of
// norm_bwd_scratch_floats(D) floats: per-block partial sums, reduced by a second kernel.
constexpr int kNormBwdMaxBlocks = 592;   // four 128-thread blocks per SM: the row loop is latency-bound below that
inline int64_t norm_bwd_scratch_floats(int D) { return static_cast<int64_t>(kNormBwdMaxBlocks) * 4 * 2 * D; }
cudaError_t launch_norm_bwd(int mode, const __nv_bfloat16* dy, const __nv_bfloat16* x, const __nv_bfloat16* gamma,
                            const float* mean, const float* rstd, const __nv_bfloat16* dres, __nv_bfloat16* dx,
                            float* dgamma, float* dbeta, float* partials, int M, int D, cudaStream_t st);
cudaError_t launch_embed_fwd(const int32_t* idx, const __nv_bfloat16* wte, const __nv_bfloat16* wpe,
                             __nv_bfloat16* out, int n_tok, int T, int D, int pos0, cudaStream_t st);
cudaError_t launch_embed_bwd(const int32_t* idx, const __nv_bfloat16* dout, float* dwte, float* dwpe, int n_tok,
                             int T, int D, int pos0, cudaStream_t st);
cudaError_t launch_ce_fwd_bwd(__nv_bfloat16* logits, const int32_t* targets, float* loss, int M, int V, int ldl,
                              float scale, int write_grad, cudaStream_t st);
cudaError_t launch_bias_grad(const __nv_bfloat16* dy, float* dbias, int M, int N, cudaStream_t st);
cudaError_t launch_sumsq(const float* g, int64_t n, float* out, cudaStream_t st);
// AdamW with bf16 weights (no fp32 master) and bf16 moments, stochastically rounded; `seed` should change every step.
cudaError_t launch_adamw_bf16_state(__nv_bfloat16* p, float* g, __nv_bfloat16* m, __nv_bfloat16* v, int64_t n,
                                    const float* hp, const float* gnorm_sq, float beta1, float beta2, float eps,
                                    float wd, float clip, int zero_grad, uint32_t seed, cudaStream_t st);

cudaError_t launch_adamw(float* p, float* g, float* m, float* v, __nv_bfloat16* p_bf16, int64_t n, const float* hp,
                         const float* gnorm_sq, float beta1, float beta2, float eps, float wd, float clip,
                         int zero_grad, cudaStream_t st);
cudaError_t launch_cast_f32_bf16(const float* in, __nv_bfloat16* out, int64_t n, cudaStream_t st);

}  // namespace b200
