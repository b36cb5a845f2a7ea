// Kernels that communicate over NVLink peer memory from inside the kernel (see comm_kernels.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int kCommMaxRanks = 8;

// Per-rank control block in symmetric memory (one per communicator, 4 KB):
//   flags[slot][src]  int32 epochs written by rank `src` (slot 0: grads ready, 1: norm
//                     exchanged, 2: parameters pushed, 3: generic barrier)
//   norm_slots[src]   partial sum of squared gradients contributed by rank `src`
struct CommCtrl {
  int flags[8][kCommMaxRanks];
  float norm_slots[kCommMaxRanks];
  int epoch;        // local launch counter, advanced by the kernel itself (CUDA-graph safe)
  int bar_epoch;    // launch counter of the stand-alone barrier kernel
  float sq_local;   // this rank's partial sum of squares for the step in flight
  float sq_total;   // global sum of squares of the step that completed last
  int abort_flag;
};

struct ShardedAdamWArgs {
  int world, rank;
  int64_t n_total;           // elements of the flat parameter vector (multiple of world * 8)
  int64_t n_decay;           // elements [0, n_decay) are weight-decayed
  float* peer_grad[kCommMaxRanks];           // every rank's full fp32 gradient buffer
  __nv_bfloat16* peer_param[kCommMaxRanks];  // every rank's full bf16 compute copy
  CommCtrl* peer_ctrl[kCommMaxRanks];        // every rank's control block
  const float* mc_grad;      // multicast (NVLS) alias of the gradient buffers, or nullptr
  __nv_bfloat16* mc_param;   // multicast alias of the compute copies, or nullptr
  float* master;             // this rank's fp32 master shard  [n_total / world]
  float* m;                  // moments, same shape
  float* v;
  const float* hp;           // {lr, bias_corr1, bias_corr2, grad_scale}
  float beta1, beta2, eps, wd, clip;
  uint64_t wait_budget_ns;   // bound of every cross-rank wait
  int* status;
  const float* extra_sq;     // optional: this rank's sum of squared gradients of parameters that are NOT in
                             // the flat vector (expert-parallel weights); joins the global clipping norm
  int pre_reduced;           // 1: this rank's shard of its gradient buffer already holds the sum over ranks
                             // (bucket kernels below ran during backward): skip the peer loads
};

// Reduce-scatter of ONE gradient bucket, launched on a side stream while backward still runs: publishes
// "my gradients of this bucket are final" to every peer, waits (bounded) for the peers' flags, then sums the
// peers' values of the listed ranges (this rank's shard of the bucket) into this rank's own buffer.
struct RsBucketArgs {
  int world, rank;
  float* peer_grad[kCommMaxRanks];   // every rank's full fp32 gradient buffer
  int* peer_flags[kCommMaxRanks];    // every rank's flag table [n_buckets][kCommMaxRanks]
  const int64_t* ranges;             // [n_ranges][2] (start, length) in elements, multiples of 4, inside this rank's shard
  int n_ranges;
  int bucket;
  const int* epoch;                  // device scalar: the training step; flags carry it
  uint64_t wait_budget_ns;
  int* status;
};
cudaError_t launch_rs_bucket(const RsBucketArgs& args, int blocks, cudaStream_t stream);

// Gradient reduce-scatter + global-norm clip + AdamW on the local shard + all-gather of the
// updated bf16 parameters, one cooperative launch. Leaves every rank's gradient buffer
// untouched except this rank's own shard range (which receives the reduced sum).
cudaError_t launch_sharded_adamw(const ShardedAdamWArgs& args, cudaStream_t stream);

// Cross-rank barrier over the control blocks (slot 3); bounded.
cudaError_t launch_comm_barrier(CommCtrl* const* peer_ctrl, int world, int rank, uint64_t wait_budget_ns, int* status,
                                cudaStream_t stream);

// Waits (bounded by budget_ns) until *flag >= expected. Used to test the timeout path: a flag
// that nothing sets makes the kernel record kWaitFlagTimeout in `status` and return.
cudaError_t launch_wait_flag(const int* flag, int expected, uint64_t budget_ns, int* status, cudaStream_t stream);

// Vocabulary-parallel cross-entropy: every rank holds the logits of its vocabulary shard only,
// [M, ldl] bf16 with columns [0, v_local) valid = global ids [v0, v0 + v_local). One cooperative kernel:
// per-row (max, sum-exp, target logit) of the shard, pushed to every peer's statistics buffer over
// NVLink, a flag barrier, then the global loss and, in place, this shard's gradient
// scale * (softmax - onehot). The full (M, V) logits are never gathered.
struct VocabCeArgs {
  int world, rank;
  int M, v_local, v0;
  int64_t ldl;
  __nv_bfloat16* logits;                   // this rank's shard; overwritten with its gradient when write_grad
  const int* targets;                      // [M] global ids; < 0 = ignored row (loss 0, zero gradient)
  float* peer_stats[kCommMaxRanks];        // every rank's buffer [2][world][M][4] fp32 (double-buffered by launch parity)
  CommCtrl* peer_ctrl[kCommMaxRanks];
  float* loss;                             // [M] per-row loss (identical on every rank)
  float scale;
  int write_grad;
  uint64_t wait_budget_ns;
  int* status;
};
cudaError_t launch_vocab_parallel_ce(const VocabCeArgs& args, cudaStream_t stream);

}  // namespace b200
