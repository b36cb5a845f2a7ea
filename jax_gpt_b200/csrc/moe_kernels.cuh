// Expert-parallel MoE: token dispatch, grouped SwiGLU GEMMs and weighted combine in one kernel
// per rank (see moe_kernels.cu).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm_kernels.cuh"

namespace b200 {

constexpr int kMoeMaxLocalExperts = 512;
constexpr int kMoeMaxExperts = 512;

struct EpMoeArgs {
  int world, rank;
  int tokens;    // tokens owned by this rank
  int top_k;
  int d_model;   // multiple of 256
  int inter;     // expert intermediate size, multiple of 128
  int e_local;   // experts per rank; global expert e lives on rank e / e_local
  int cap_rows;  // rows the receive buffers of every rank can hold
  // local inputs
  const __nv_bfloat16* x;  // [tokens, d_model]
  const int* idx;          // [tokens * top_k] global expert id of each (token, choice) pair
  const float* w;          // [tokens * top_k] routing weight of the pair
  const int* pos;          // [tokens * top_k] index of the pair among this rank's pairs for that expert
  const int* my_counts;    // [world * e_local] pairs per global expert from this rank
  // symmetric (peer-visible) buffers, one pointer per rank
  __nv_bfloat16* peer_recv_x[kCommMaxRanks];  // [cap_rows, d_model] rows sorted by local expert, then by source rank
  int* peer_recv_meta[kCommMaxRanks];         // [cap_rows] (source rank << 24) | source token
  float* peer_recv_w[kCommMaxRanks];          // [cap_rows] routing weight of the row
  int* peer_counts[kCommMaxRanks];            // [world][world * e_local] every rank's my_counts
  unsigned* peer_arrive[kCommMaxRanks];       // [e_local] rows delivered so far, cumulative over launches
  float* peer_out[kCommMaxRanks];             // [tokens of that rank, d_model] fp32 combine target (zeroed by owner)
  CommCtrl* peer_ctrl[kCommMaxRanks];
  // local scratch / state
  __nv_bfloat16* act;       // [cap_rows, inter] SwiGLU output
  __nv_bfloat16* gu;        // [cap_rows, 2 * inter] gate | up pre-activations saved for backward, or nullptr
  unsigned* arrive_target;  // [e_local] arrivals expected once this launch's rows are in (cumulative)
  int* act_ready;           // [cap_rows / 128 + e_local + 1] per m-tile count of finished GEMM1 epilogue warps, then the
                            // forward launch's tile counter
  int* slot_out;            // [tokens * top_k] bf16 forward: scratch, this rank's pair ids sorted by expert (the dispatch
                            // order); FP8 forward: row of each pair in its destination's receive buffer
  int* rows_out;            // [e_local] rows received per local expert (for the caller / backward)
  // ---- backward only ----
  const __nv_bfloat16* dout;                   // [tokens, d_model] gradient of the routed output
  __nv_bfloat16* peer_recv_dy[kCommMaxRanks];  // [cap_rows, d_model] routing-weighted output-gradient rows
  float* peer_dx[kCommMaxRanks];               // [tokens of that rank, d_model] fp32 input-gradient target (zeroed by owner)
  float* peer_dw[kCommMaxRanks];               // [tokens * top_k of that rank] gradient of the routing weights
  __nv_bfloat16* dgu;                          // [cap_rows, 2 * inter] gradient of gate | up
  float* dw_rows;                              // [cap_rows] <dAct, act> per received row
  int* gu_ready;                               // [cap_rows / 128 + e_local + 1] per m-tile count of finished dAct epilogue
                                               // warps, then the backward launch's tile counter
  int* expert_done;                            // [e_local] same, per expert
  float* d_gate;                               // [e_local, d_model, inter] fp32, accumulated
  float* d_up;                                 // [e_local, d_model, inter]
  float* d_down;                               // [e_local, inter, d_model]
  uint64_t wait_budget_ns;
  int* status;
  long long* prof;  // set by the launchers: per-CTA phase timeline of this launch (kMoeProfFields per CTA), or nullptr
};

// Phase timeline of the bf16 forward (which = 0) / backward (which = 1) kernel, recorded when the environment
// variable B200_MOE_PROFILE=1 is set before the first launch. Per CTA: [0] start, [1] tables built, [2] own
// dispatch done, [3] last tile's loads issued, [4] end (all globaltimer ns), [5] SM cycles the load warp waited on
// dependencies (arrivals, earlier tiles), [6] cycles the MMA warp waited for operands, [7] cycles it waited for a
// free accumulator, [8] ns when the epilogue finished its last tile, [9] SM cycles from [0] to [4].
constexpr int kMoeProfCtas = 160, kMoeProfFields = 10;
cudaError_t moe_profile_read(int which, long long* host_out);  // host_out[kMoeProfCtas * kMoeProfFields]

// Host walk of the static tile order the bf16 kernels build on the device (same code, compiled for the host), for
// tests: given the rows every local expert receives, writes (expert, phase, m, n) of every tile in order and
// returns their number (-1 for shapes the kernels reject). Forward phases: 0 gate|up GEMM, 1 down GEMM; backward:
// 0 dAct, 1 dX, 2 dW_down, 3 dW_gate|up. tiles_out holds 4 * max_tiles ints.
int moe_tile_order_host(const int* rows, int e_local, int d_model, int inter, int grid_ctas, bool backward,
                        int* tiles_out, int max_tiles, int* lag_out);

// counts[e] = number of pairs routed to global expert e; pos[p] = rank of pair p within its expert.
cudaError_t launch_moe_prepare(const int* idx, int n_pairs, int n_experts, int* counts, int* pos, cudaStream_t st);

// gate/up: [e_local, d_model, inter] bf16 (in,out); down: [e_local, inter, d_model]. The kernel reads the
// receive buffer and `act` of THIS rank through TMA (pointers args.peer_recv_x[rank], args.act).
cudaError_t launch_ep_moe_forward(const EpMoeArgs& args, const __nv_bfloat16* gate, const __nv_bfloat16* up,
                                  const __nv_bfloat16* down, cudaStream_t st);

// Backward of the LAST forward launch: dispatches the w * dout rows to the slots that launch used (x rows,
// routing metadata, act and pre-activations stay in place), computes the expert-side gradients
// (dAct with the SwiGLU backward, dX pushed to the token owners, the three weight gradients with
// ragged K, the routing-weight gradients) in one cooperative kernel. Needs `act` and `gu` of the
// forward call with the same routing.
cudaError_t launch_ep_moe_backward(const EpMoeArgs& args, const __nv_bfloat16* gate, const __nv_bfloat16* up,
                                   const __nv_bfloat16* down, cudaStream_t st);

// ------------------------------------------------------------------------------------------------
// FP8 forward (moe_fp8_kernels.cu): token rows are quantised to e4m3 with power-of-two 1 x 128 scales
// once, pushed as bytes (half the NVLink traffic of bf16) together with their UE8M0 scale bytes, the
// grouped GEMMs run on the block-scaled tensor-core path (scales in TMEM), and the SwiGLU epilogue
// re-quantises the activation for the down projection. Weights are quantised ahead of time with
// power-of-two 128 x 128 scales and stored K-major:
//   gate_q / up_q [E_local, I, D] bytes, down_q [E_local, D, I] bytes,
//   sfb1 [E_local, I/128, D/128, 512]: packed scale chunk of GEMM 1's B tile (rows 0-63 gate, 64-127 up),
//   sfb2 [E_local, D/128, I/128, 512]: packed scale chunks of down_q.
// Packed chunk layout: byte (r % 32) * 16 + (r / 32) * 4 + j = exponent of row r, K block j.
struct EpMoeFp8Args {
  int world, rank;
  int tokens, top_k, d_model, inter, e_local, cap_rows;  // expert regions are padded to 128 rows
  const __nv_bfloat16* x;
  const int* idx;
  const float* w;
  const int* pos;
  const int* my_counts;
  uint8_t* xq;                              // [tokens, d_model] local staging of the quantised rows
  uint8_t* xe;                              // [tokens, d_model / 128] their scale exponents
  uint8_t* peer_recv_q[kCommMaxRanks];      // [cap_rows, d_model]
  uint8_t* peer_recv_sf[kCommMaxRanks];     // [cap_rows / 128, d_model / 128, 512]
  int* peer_recv_meta[kCommMaxRanks];
  float* peer_recv_w[kCommMaxRanks];
  int* peer_counts[kCommMaxRanks];
  unsigned* peer_arrive[kCommMaxRanks];
  float* peer_out[kCommMaxRanks];
  CommCtrl* peer_ctrl[kCommMaxRanks];
  uint8_t* act_q;                           // [cap_rows, inter]
  uint8_t* act_sf;                          // [cap_rows / 128, inter / 128, 512]
  const uint8_t* sfb1;
  const uint8_t* sfb2;
  unsigned* arrive_target;
  int* act_ready;
  int* slot_out;
  int* rows_out;
  uint64_t wait_budget_ns;
  int* status;
};

cudaError_t launch_ep_moe_forward_fp8(const EpMoeFp8Args& args, const uint8_t* gate_q, const uint8_t* up_q,
                                      const uint8_t* down_q, cudaStream_t st);

}  // namespace b200
