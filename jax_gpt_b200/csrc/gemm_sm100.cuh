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
  kOutBf16PeerRed = 3, // fp32 reduction into a row-partitioned set of peer buffers (GEMM -> reduce-scatter, red.add)
  kOutBf16PeerPush = 4 // GEMM -> reduce-scatter: bf16 partial tiles stored into the row owner's receive slot of this
                       // rank, arrival counters, then the owner sums the slots (second phase of the same kernel)
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
  // kOutBf16PeerPush: peer_out[r] is rank r's receive buffer [n_peers, rows_per_peer, ldo] bf16 (slot s = partial of
  // rank s); peer_cnt[r] its arrival counters, one per 128-row block of its rows; every epilogue warp adds the number
  // of 64-column groups it stored, so a block is complete at cnt_expected = calls * n_peers * 4 * (N / 64). rs_out [rows_per_peer, ldo] bf16
  // receives the sum of this rank's slots.
  int* peer_cnt[kMaxPeers];
  int self_rank;
  int cnt_expected;
  __nv_bfloat16* rs_out;
  unsigned long long rs_wait_ns;
};

// Staged gather: extra "copier" CTAs of the GEMM grid PUSH this rank's operand shard into every peer's gather buffer
// (local -> shared-memory ring -> peer with bulk copies, and local -> peer with plain loads and stores: writes over
// NVLink are posted, so a few SMs keep the links busy, which reads from a peer do not), one unit at a time, and
// publish each unit in the peer's `ready` array. The GEMM CTAs read their own gather buffer with TMA and wait, unit
// by unit, for the flags the peers set. Every byte crosses NVLink once. A unit is one 128-row M-block of A
// (all-gather -> GEMM) or 64 rows of one rank's column shard of B (FSDP weight gather).
struct StageCopy {
  int n_copy_ctas;                  // 0 = no staging
  int n_remote;                     // peers to push to, in visiting order
  int units_per_src;
  int mode;                         // 1: units are 128-row M-blocks of A, 2: units are 64-row blocks of a column shard of B
  int epoch;                        // value that marks "this call" in every flag
  int my_unit0;                     // index of this rank's first unit in everybody's `ready` numbering
  long long bytes_per_unit;
  unsigned long long wait_ns;       // budget of every flag wait
  const unsigned char* src;         // this rank's shard (local)
  unsigned char* dst[kMaxPeers];    // where it lands in peer j's buffer (peer-mapped)
  int* peer_ready[kMaxPeers];       // peer j's `ready` array (peer-mapped)
  int* ready;                       // this rank's `ready` array: one int per unit, >= epoch once the unit has landed
};

// A is [M,K]; a_major 0: stored row-major [M,K] (K contiguous), 1: stored row-major [K,M].
// B is [N,K]; b_major 0: stored row-major [N,K] (K contiguous), 1: stored row-major [K,N].
// lda / ldb are the row strides of the stored matrices, in elements.
// Returns cudaSuccess or the launch error; device-side problems land in args.status.
cudaError_t launch_gemm_bf16(const __nv_bfloat16* A, int64_t lda, int a_major, const __nv_bfloat16* B, int64_t ldb,
                             int b_major, const GemmArgs& args, cudaStream_t stream);

// All-gather -> GEMM with the staged gather above. peer_gather[s] is rank s's gather buffer [n_src * rows_per_src, K]
// (K contiguous) as mapped here, peer_ready[s] its ready array (int[n_src * rows_per_src / 128]); entry `rank` of
// both is this rank's own. Block `rank` of the local buffer must already hold the local rows.
cudaError_t launch_gemm_bf16_gathered_a_staged(__nv_bfloat16* const* peer_gather, int* const* peer_ready, int n_src,
                                               int rows_per_src, int rank, const __nv_bfloat16* B, int64_t ldb,
                                               int b_major, const GemmArgs& args, int epoch, double wait_seconds,
                                               cudaStream_t stream);

// FSDP weight gather fused into the GEMM with the staged gather. W [K, N] is sharded by COLUMNS: rank s owns
// W[:, s * N / n : (s + 1) * N / n] as a contiguous [K, N / n] matrix. peer_w[s] is rank s's gather buffer (n such
// matrices back to back) as mapped here; matrix `rank` of the local one must already hold the local shard;
// peer_ready[s] is its ready array (int[n * K / 64]). Tiles of the local shard are computed first.
cudaError_t launch_gemm_bf16_sharded_b_staged(const __nv_bfloat16* A, int64_t lda, __nv_bfloat16* const* peer_w,
                                              int* const* peer_ready, int n_src, int rank, const GemmArgs& args,
                                              int epoch, double wait_seconds, cudaStream_t stream);

// GEMM -> reduce-scatter in one kernel (args.out_mode == kOutBf16PeerPush, see GemmArgs): A [M, K] K-major with
// M = n_peers * rows_per_peer, every rank holding a K-slice; bf16 partial tiles are stored into the row owner's
// receive slot over NVLink, the owner sums its slots into args.rs_out after its own tiles.
cudaError_t launch_gemm_bf16_reduce_scatter_push(const __nv_bfloat16* A, int64_t lda, const __nv_bfloat16* B, int64_t ldb,
                                                 int b_major, const GemmArgs& args, cudaStream_t stream);

// CTA-pair variant (gemm_pair_sm100.cu): 256 x 256 tiles computed by two CTAs of a cluster with
// tcgen05.mma.cta_group::2. launch_gemm_bf16 forwards to it when gemm_pair_wanted() says so
// (environment B200_GEMM_PAIR: 0 never, 1 whenever M, N >= 256, unset: when the 256 x 256 tiles occupy at least 3/4 of the CTA pairs).
cudaError_t launch_gemm_bf16_pair(const __nv_bfloat16* A, int64_t lda, int a_major, const __nv_bfloat16* B, int64_t ldb,
                                  int b_major, const GemmArgs& args, cudaStream_t stream);
bool gemm_pair_wanted(const GemmArgs& args);

int gemm_sm_count();

}  // namespace b200
