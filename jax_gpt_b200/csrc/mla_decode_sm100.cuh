// Paged multi-head-latent-attention decode (absorbed weights) and paged cache writes for sm_100a
// (see mla_decode_sm100.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int kMlaLatent = 512;   // compressed KV width (value part of a cached token)
constexpr int kMlaRope = 64;      // rotary key width
constexpr int kMlaWidth = kMlaLatent + kMlaRope;  // one cached token
constexpr int kMlaPage = 64;      // tokens per page

struct MlaDecodeArgs {
  int batch, heads;               // sequences in this step, query heads per sequence
  int max_pages;                  // columns of the block table
  int n_splits;                   // KV splits per sequence (grid.x)
  int n_pages;                    // pages in the pool (filled in by the launcher)
  const int* block_table;         // [max_seqs, max_pages] page ids
  const int* seq_lens;            // [max_seqs] tokens to attend over (the new token included)
  const int* seq_ids;             // [batch] row of block_table / seq_lens for every batch slot
  float scale_log2;               // softmax scale * log2(e)
  float* part_out;                // [batch, 2 * n_splits, heads, 512] normalised partials (two softmax groups per split)
  float* part_lse;                // [batch, 2 * n_splits, heads] log2-sum-exp of each partial (-inf when empty)
  int* status;
};

// q [batch * heads, 576] bf16 (absorbed nope part | rotated rope part); pool: one layer of the page pool,
// [n_pages * 64, 576] bf16. out [batch, heads, 512] bf16 = softmax(q . c^T) c[:, :512] over each sequence's pages.
// scratch: part_out / part_lse as sized above.
cudaError_t launch_mla_paged_decode(const __nv_bfloat16* q, const __nv_bfloat16* pool, int n_pages,
                                    const MlaDecodeArgs& args, __nv_bfloat16* out, cudaStream_t stream);

// Writes rows [batch, T, width] into the pages of their sequences at positions start[b] + t.
cudaError_t launch_paged_kv_write(const __nv_bfloat16* rows, __nv_bfloat16* pool, const int* block_table,
                                  const int* seq_ids, const int* start, int batch, int T, int width, int page_size,
                                  int max_pages, int n_pages, int* status, cudaStream_t stream);

}  // namespace b200
