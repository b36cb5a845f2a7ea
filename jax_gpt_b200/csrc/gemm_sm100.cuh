// Host-visible argument block of the tcgen05 GEMM family (see gemm_sm100.cu).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

enum GemmEpilogue : int {
  kEpiNone = 0,      // out = alpha * acc (+ bias) (+ residual)
  kEpiGelu = 1,      // pre = acc + bias; aux_out = pre; out = gelu_tanh(pre)
  kEpiGeluGrad = 2,  // out = acc * gelu_tanh'(aux_in)
  kEpiSiluMul = 3,   // reserved for SwiGLU-style epilogues
};
enum GemmOut : int {
  kOutBf16 = 0,       // store bf16
  kOutF32 = 1,        // store fp32
  kOutF32Atomic = 2,  // fp32 atomic accumulate (gradient accumulation, split-K)
  kOutBf16PeerRed = 3 // bf16 reduction into a row-partitioned set of peer buffers (GEMM -> reduce-scatter)
};

constexpr int kMaxPeers = 8;

struct GemmArgs {
  int M, N, K;
  void* out;
  int64_t ldo;
  const __nv_bfloat16* bias;      // [N] or nullptr
  const __nv_bfloat16* residual;  // [M, ldr] or nullptr
  int64_t ldr;
  __nv_bfloat16* aux_out;         // [M, ldaux] pre-activation (kEpiGelu)
  const __nv_bfloat16* aux_in;    // [M, ldaux] pre-activation (kEpiGeluGrad)
  int64_t ldaux;
  int epilogue;
  int out_mode;
  float alpha;
  int split_k;
  int* status;
  // kOutBf16PeerRed: rows [r*rows_per_peer, (r+1)*rows_per_peer) of the logical output live
  // in peer_out[r] (this rank's own buffer included), each [rows_per_peer, ldo] fp32.
  float* peer_out[kMaxPeers];
  int rows_per_peer;
  int n_peers;
};

// A is [M,K]; a_major 0: stored row-major [M,K] (K contiguous), 1: stored row-major [K,M].
// B is [N,K]; b_major 0: stored row-major [N,K] (K contiguous), 1: stored row-major [K,N].
// lda / ldb are the row strides of the stored matrices, in elements.
// Returns cudaSuccess or the launch error; device-side problems land in args.status.
cudaError_t launch_gemm_bf16(const __nv_bfloat16* A, int64_t lda, int a_major, const __nv_bfloat16* B, int64_t ldb,
                             int b_major, const GemmArgs& args, cudaStream_t stream);

// All-gather -> GEMM: the M rows of A are the concatenation of `n_src` row blocks of
// `rows_per_src` rows, block s living at a_src[s] (a peer-mapped pointer for remote ranks,
// read with ordinary non-multicast TMA tile loads). Row blocks are visited starting with
// block `first_src` (the local one), so compute starts before remote data is needed.
cudaError_t launch_gemm_bf16_gathered_a(const __nv_bfloat16* const* a_src, int n_src, int rows_per_src,
                                        int first_src, int64_t lda, const __nv_bfloat16* B, int64_t ldb, int b_major,
                                        const GemmArgs& args, cudaStream_t stream);

// Parameter all-gather fused into the consuming GEMM (FSDP): the weight W [K, N] (MN-major B) is
// split by rows over `b_n_src` ranks; shard s lives at b_src[s] (peer-mapped for remote ranks) and
// is read tile by tile with non-multicast TMA as the K loop reaches it, the local shard first.
cudaError_t launch_gemm_bf16_sharded_b(const __nv_bfloat16* A, int64_t lda, const __nv_bfloat16* const* b_src,
                                       int b_n_src, int b_first_src, int64_t ldb, const GemmArgs& args,
                                       cudaStream_t stream);

// CTA-pair variant (gemm_pair_sm100.cu): 256 x 256 tiles computed by two CTAs of a cluster with
// tcgen05.mma.cta_group::2. launch_gemm_bf16 forwards to it when gemm_pair_wanted() says so
// (environment B200_GEMM_PAIR: 0 never, 1 whenever M, N >= 256, unset: when the 256 x 256 tiles occupy at least 3/4 of the CTA pairs).
cudaError_t launch_gemm_bf16_pair(const __nv_bfloat16* A, int64_t lda, int a_major, const __nv_bfloat16* B, int64_t ldb,
                                  int b_major, const GemmArgs& args, cudaStream_t stream);
bool gemm_pair_wanted(const GemmArgs& args);

int gemm_sm_count();

}  // namespace b200
