// Launchers of the routing, rotary, quantisation and Gated-DeltaNet decode kernels (seq_kernels.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// MoE router on fp32 logits [M, E] (E <= 512, E % 32 == 0).
//  mode 0: softmax over all experts, top-k, renormalise to sum 1 (Qwen3.5).
//  mode 1: sigmoid scores; selection on score + bias; groups ranked by the sum of their top-2;
//          top-k over the kept groups; weights = unbiased scores / their sum * scale (DeepSeek-V3).
// Outputs: weights [M, k] fp32, ids [M, k] int32, and (optional) counts [E] += pairs per expert.
cudaError_t launch_router(int mode, const float* logits, const float* bias, int M, int E, int k, int n_group,
                          int topk_group, float scale, float* weights, int* ids, int* counts, cudaStream_t st);

// x [rows, H, dh] bf16 -> y: per-head RMSNorm over dh (weight w, (1 + w) when one_plus), then
// half-split rotary on the first rope_dim features with the (cos, sin) table [n_pos, rope_dim/2, 2];
// row r uses position pos0 + (r % T). norm_w may be nullptr (rotary only).
cudaError_t launch_rmsnorm_rope(const __nv_bfloat16* x, const __nv_bfloat16* norm_w, const float* freqs,
                                __nv_bfloat16* y, int rows, int T, int H, int dh, int rope_dim, int pos0, float eps,
                                int one_plus, cudaStream_t st);

// Block-scaled FP8 e4m3 quantisation. Activations: one fp32 scale per 1 x 128 block along K
// (x [M, K] bf16 -> q [M, K] fp8, scales [M, K/128]); weights: one scale per 128 x 128 block
// (w [R, C] bf16 -> q [R, C], scales [R/128, C/128]). scale = amax / 448, optionally rounded up to
// a power of two; q = x / scale.
cudaError_t launch_fp8_quant_1x128(const __nv_bfloat16* x, uint8_t* q, float* scales, int M, int K, int pow2,
                                   cudaStream_t st);
cudaError_t launch_fp8_quant_128x128(const __nv_bfloat16* w, uint8_t* q, float* scales, int R, int C, int pow2,
                                     cudaStream_t st);

// Quantisation for the hardware-scaled GEMM in one pass: x [R, C] bf16 (R, C multiples of 128) -> q [R, C], or with
// `transpose` q^T [C, R]; power-of-two scales per 1 x 128 block of an output row (`block` = 0) or per 128 x 128
// tile (`block` = 1), written as fp32 (`scales`, may be null) and as packed exponent bytes
// [rows/128, contraction/128, 512] (`sf_packed`, the operand layout of launch_gemm_mxfp8).
cudaError_t launch_fp8_quant_mx(const __nv_bfloat16* x, uint8_t* q, float* scales, uint8_t* sf_packed, int R, int C,
                                int transpose, int block, cudaStream_t st);

// One decode step of a Gated-DeltaNet layer for B sequences, fused: conv-window update + depthwise
// conv + SiLU, gates, L2-normalised q/k, state decay + delta-rule update, read-out, gated RMSNorm.
//  mixed [B, 2*Kd + Vd] bf16 (projected q|k|v before the conv), z [B, Vd], bproj / aproj [B, Hv] bf16 (row strides
//  ld_*: the four may be column slices of one merged projection output),
//  conv_state [B, C, Kc] fp32 (updated in place), conv_w [C, Kc], A_log / dt_bias [Hv], norm_w [dv],
//  state [B, Hv, dk, dv] fp32 (updated in place), out [B, Vd] bf16.
cudaError_t launch_gdn_decode_step(const __nv_bfloat16* mixed, const __nv_bfloat16* z, const __nv_bfloat16* bproj,
                                   const __nv_bfloat16* aproj, float* conv_state, const __nv_bfloat16* conv_w,
                                   const __nv_bfloat16* A_log, const __nv_bfloat16* dt_bias,
                                   const __nv_bfloat16* norm_w, float* state, __nv_bfloat16* out, int B, int Hqk, int Hv,
                                   int dk, int dv, int Kc, float eps, int ld_mixed, int ld_z, int ld_b, int ld_a,
                                   cudaStream_t st);

// Backward of launch_rmsnorm_rope: dx [rows, H, dh] bf16; dw [dh] fp32 is ACCUMULATED into (may be nullptr).
cudaError_t launch_rmsnorm_rope_bwd(const __nv_bfloat16* x, const __nv_bfloat16* dy, const __nv_bfloat16* norm_w,
                                    const float* freqs, __nv_bfloat16* dx, float* dw, int rows, int T, int H, int dh,
                                    int rope_dim, int pos0, float eps, int one_plus, cudaStream_t st);

// Inter-chunk scan of the chunked gated delta rule (gdn_kernels.cu); head widths dk = dv = 128, chunks of 64.
//   kq    [BH, N, 128, 128] bf16: rows 0-63 k_cum, rows 64-127 q * exp(G) of every chunk
//   intra [BH, N, 64, 64]   bf16: causal-masked (q k^T * decay)
//   kdec  [BH, N, 64, 128]  bf16: k * exp(g_end - G)
//   veff  [BH, N, 64, 128]  bf16: corrected values;  e [BH, N] fp32: exp(g_end);  s0: initial state or nullptr
// Writes o [BH, N, 64, 128] bf16 and the final state s_out [BH, 128, 128] fp32; with s_save / vn_save (optional,
// [BH, N, 128, 128] / [BH, N, 64, 128] bf16) also the state every chunk starts from and its v_new, which the
// backward scan consumes.
cudaError_t launch_gdn_scan(const __nv_bfloat16* kq, const __nv_bfloat16* intra, const __nv_bfloat16* kdec,
                            const __nv_bfloat16* veff, const float* e, const float* s0, __nv_bfloat16* o, float* s_out,
                            __nv_bfloat16* s_save, __nv_bfloat16* vn_save, int bh, int n_chunks, int* status,
                            cudaStream_t stream);

// Backward of the scan (reverse over chunks, dS resident on chip). dO [BH, N, 64, 128] bf16; ds_final optional
// [BH, 128, 128] fp32. Writes d_kq [BH, N, 128, 128] (rows 0-63 d k_cum, 64-127 d q*exp(G)), d_intra, d_kdec,
// d_veff (bf16, shaped like the inputs), ACCUMULATES d_e [BH, N] fp32 (zero it first), writes ds0 [BH, 128, 128] fp32.
cudaError_t launch_gdn_scan_bwd(const __nv_bfloat16* kq, const __nv_bfloat16* intra, const __nv_bfloat16* kdec,
                                const __nv_bfloat16* s_save, const __nv_bfloat16* vn_save, const float* e,
                                const __nv_bfloat16* d_o, const float* ds_final, __nv_bfloat16* d_kq,
                                __nv_bfloat16* d_intra, __nv_bfloat16* d_kdec, __nv_bfloat16* d_veff, float* d_e, float* ds0,
                                int bh, int n_chunks, int* status, cudaStream_t stream);

// State-independent part of the chunked gated delta rule (gdn_chunk_kernels.cu), chunks of 64, dk = dv = 128.
//   mixed [B, T, (2 Hqk + Hv) * 128] bf16: q | k | v after the conv + SiLU;  b_in, a_in [B, T, Hv] bf16: gate
//   pre-activations;  A_log, dt_bias [Hv] fp32.
// Writes the operands of launch_gdn_scan for BH = B * Hv (value head hv reads q/k head hv / (Hv / Hqk)) and
// N = ceil(T / 64) chunks: kq, intra, kdec, veff, e (rows at or beyond T behave as zero-padded tokens).
cudaError_t launch_gdn_chunk_prep(const __nv_bfloat16* mixed, const __nv_bfloat16* b_in, const __nv_bfloat16* a_in,
                                  const float* A_log, const float* dt_bias, __nv_bfloat16* kq, __nv_bfloat16* intra,
                                  __nv_bfloat16* kdec, __nv_bfloat16* veff, float* e, int B, int T, int Hqk, int Hv,
                                  cudaStream_t stream);

// Backward of launch_gdn_chunk_prep: recomputes the forward from the same inputs. d_kq / d_intra / d_kdec / d_veff
// bf16 and d_e fp32 are shaped like the forward outputs. Writes d_mixed [B, T, conv_dim] bf16 (every element),
// d_b, d_a [B, T, Hv] fp32, and ACCUMULATES d_A_log, d_dt_bias [Hv] fp32 (zero them first).
cudaError_t launch_gdn_chunk_prep_bwd(const __nv_bfloat16* mixed, const __nv_bfloat16* b_in, const __nv_bfloat16* a_in,
                                      const float* A_log, const float* dt_bias, const __nv_bfloat16* d_kq,
                                      const __nv_bfloat16* d_intra, const __nv_bfloat16* d_kdec,
                                      const __nv_bfloat16* d_veff, const float* d_e, __nv_bfloat16* d_mixed, float* d_b,
                                      float* d_a, float* d_A_log, float* d_dt_bias, int B, int T, int Hqk, int Hv,
                                      cudaStream_t stream);

// Gated RMSNorm of the scan output, fused with the head-major -> token-major transpose:
//   y[b, t, h, :] = w * o[b, h, t, :] * rsqrt(mean(o^2) + eps) * silu(z[b, t, h, :]),   head width 128
// o [B*Hv, Tpad, 128] bf16 (the layout launch_gdn_scan writes, Tpad >= T), z and y [B, T, Hv * 128] bf16, w [128] fp32.
cudaError_t launch_gdn_gated_norm(const __nv_bfloat16* o, const __nv_bfloat16* z, const float* w, __nv_bfloat16* y, int B,
                                  int T, int Tpad, int Hv, float eps, cudaStream_t stream);
// Backward: writes d_o (rows t < T of the [B*Hv, Tpad, 128] layout; zero the padding yourself) and dz, ACCUMULATES
// dw [128] fp32.
cudaError_t launch_gdn_gated_norm_bwd(const __nv_bfloat16* o, const __nv_bfloat16* z, const float* w,
                                      const __nv_bfloat16* dy, __nv_bfloat16* d_o, __nv_bfloat16* dz, float* dw, int B,
                                      int T, int Tpad, int Hv, float eps, cudaStream_t stream);

// Causal depthwise conv (width 4) + SiLU over x [B, T, C] bf16 with w [C, 4]; `state` (optional) [B, C, 4] fp32
// receives the last four raw inputs of every channel.
cudaError_t launch_gdn_conv_silu(const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* y, float* state, int B,
                                 int T, int C, int K, cudaStream_t stream);
// Backward of the same op: dx [B, T, C] bf16 is written, dw [C, K] fp32 is ACCUMULATED (atomics).
cudaError_t launch_gdn_conv_silu_bwd(const __nv_bfloat16* x, const __nv_bfloat16* w, const __nv_bfloat16* dy,
                                     __nv_bfloat16* dx, float* dw, int B, int T, int C, int K, cudaStream_t stream);

}  // namespace b200
