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

// Where the keys and values of (batch b, kv head hkv) live. Token-major activations: K and V are [B*Tk, Hkv*D]
// matrices (rows_b = Tk, rows_h = 0, k_col_h = D). A cache laid out as (B, Hkv, max_len, D) is one matrix of
// B*Hkv*max_len rows and D columns (rows_b = Hkv*max_len, rows_h = max_len, k_col_h = 0). Rows of the last
// 128-row tile past Tk are read and masked: they must hold finite values.
struct AttnKvLayout {
  int Tk;                 // keys per sequence
  int q_pos0;             // position of query 0; a causal query i sees keys at positions <= q_pos0 + i
  int rows_b, rows_h;     // row of key 0 of (b, hkv) = b * rows_b + hkv * rows_h
  int k_col_h, v_col_h;   // first column of head hkv in K / V = hkv * {k,v}_col_h
  uint64_t rows;          // extent of the K and V matrices
  uint64_t k_cols, v_cols;
};

// out [B*T, ldo] bf16 with head h at columns [h*D, +D); lse [B, H, T] fp32 holds
// log2-sum-exp of the scaled scores (scale * log2(e) folded in).
cudaError_t launch_attn_fwd(const AttnTensors& t, const AttnShape& s, __nv_bfloat16* out, int64_t ldo, float* lse,
                            int* status, cudaStream_t stream);

// The same with an explicit key / value layout and query offset (prefill on top of a cache; s.T counts queries).
cudaError_t launch_attn_fwd_kv(const AttnTensors& t, const AttnShape& s, const AttnKvLayout& kv, __nv_bfloat16* out,
                               int64_t ldo, float* lse, int* status, cudaStream_t stream);
// Head width 64: two query tiles per CTA (attention_fwd2_sm100.cu).
cudaError_t launch_attn_fwd2_d64(const AttnTensors& t, const AttnShape& s, const AttnKvLayout& kv,
                                 __nv_bfloat16* out, int64_t ldo, float* lse, int* status, cudaStream_t stream);

// Gradients. dq_accum [B*T, H*D] fp32 must be zero on entry (partial sums arrive through
// fp32 reductions); dk / dv are written as bf16 with the strides given. delta [B, H, T] is
// scratch for rowsum(dO * O).
cudaError_t launch_attn_bwd(const AttnTensors& t, const AttnShape& s, const __nv_bfloat16* out, int64_t ldo,
                            const __nv_bfloat16* dout, int64_t lddo, const float* lse, float* delta, float* dq_accum,
                            __nv_bfloat16* dk, int64_t lddk, __nv_bfloat16* dv, int64_t lddv, int* status,
                            cudaStream_t stream);

// Head width 64, pipelined over half score tiles (attention_bwd2_sm100.cu); delta must already hold rowsum(dO * O).
cudaError_t launch_attn_bwd2_d64(const AttnTensors& t, const AttnShape& s, const __nv_bfloat16* dout, int64_t lddo,
                                 const float* lse, const float* delta, float* dq_accum, __nv_bfloat16* dk,
                                 int64_t lddk, __nv_bfloat16* dv, int64_t lddv, int* status, cudaStream_t stream);

// delta[b, h, t] = sum_d dO[b, t, h, d] * O[b, t, h, d] for v-head widths 64, 128, 256.
cudaError_t launch_attn_delta(const __nv_bfloat16* out, int64_t ldo, const __nv_bfloat16* dout, int64_t lddo,
                              float* delta, int B, int T, int H, int Dv, cudaStream_t stream);

// Wide heads (attention_bwd_wide_sm100.cu): (D, Dv) = (256, 256) or (192, 128). delta must already hold
// rowsum(dO * O); dq_accum [B*T, H*D] fp32 zero on entry.
cudaError_t launch_attn_bwd_wide(const AttnTensors& t, const AttnShape& s, const __nv_bfloat16* dout, int64_t lddo,
                                 const float* lse, const float* delta, float* dq_accum, __nv_bfloat16* dk,
                                 int64_t lddk, __nv_bfloat16* dv, int64_t lddv, int* status, cudaStream_t stream);

// One query token per sequence against a dense cache (B, Hkv, max_len, D) given by element strides
// (attention_decode.cu). D in {64, 128, 256}, H / Hkv in {1, 2, 4, 8}. The number of valid keys is `len`, or
// pos_ptr[0] + len_add read on the device. part_o [B, H, n_splits, D] and part_ml [B, H, n_splits, 2] fp32 are
// scratch for the key ranges; out [B, H*D] bf16 with row stride ldo.
cudaError_t launch_attn_decode(const __nv_bfloat16* q, int64_t ldq, const __nv_bfloat16* k, const __nv_bfloat16* v,
                               int64_t kv_stride_b, int64_t kv_stride_h, int64_t kv_stride_t, const int* pos_ptr,
                               int len, int len_add, int B, int H, int Hkv, int D, float scale, int n_splits,
                               float* part_o, float* part_ml, __nv_bfloat16* out, int64_t ldo, cudaStream_t stream);

// The same decode attention over a PAGED cache: pool [n_pages, page_size, width] bf16 with width = 2 * Hkv * D (K of
// every kv head, then V), block_table [max_seqs, max_pages] int32, seq_ids [B], seq_lens [max_seqs] (device); the
// number of valid keys of a sequence is seq_lens[seq] + len_add (len_add = 1 when the new token's row has been written
// but the length not yet advanced).
cudaError_t launch_attn_decode_paged(const __nv_bfloat16* q, int64_t ldq, const __nv_bfloat16* pool, int width,
                                     const int* block_table, const int* seq_ids, const int* seq_lens, int len_add,
                                     int page_size, int max_pages, int B, int H, int Hkv, int D, float scale, int n_splits,
                                     float* part_o, float* part_ml, __nv_bfloat16* out, int64_t ldo, cudaStream_t stream);

// dst[r, c] (bf16, row stride ldd) = src[r, c] (fp32, row stride lds), for an M x N block.
// In-place elementwise step of the recomputed attention backward: s [rows, kv] bf16 scores -> probabilities,
// dp [rows, kv] bf16 (dO V^T) -> dS; lse (log2 units) and delta per row; row r is query position q0 + r % c.
cudaError_t launch_attn_bwd_probs(__nv_bfloat16* s, __nv_bfloat16* dp, const float* lse, const float* delta,
                                  int64_t rows, int kv, int c, int q0, float scale, int causal, cudaStream_t stream);

cudaError_t launch_cast_rows_f32_bf16(const float* src, int64_t lds, __nv_bfloat16* dst, int64_t ldd, int M, int N,
                                      cudaStream_t stream);

}  // namespace b200
