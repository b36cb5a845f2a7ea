// Expert-parallel MoE forward as ONE cooperative kernel per rank.
//
//   1. every rank publishes its per-expert pair counts to all peers (tiny all-gather through peer
//      stores + a flag barrier); from the full count table each CTA derives, in shared memory,
//      where its rows go in every destination's receive buffer and how many rows each local
//      expert receives - no host round trip, no separate exchange kernel;
//   2. dispatch: four warps per CTA copy the token rows, in expert order (the pairs are sorted on the fly), straight
//      into the destination rank's expert-sorted receive buffer over NVLink, with source id and routing weight,
//      and bump that expert's arrival counter on the destination after a fence per few rows - WHILE the other
//      warps of the CTA already run the tiles of the experts whose rows are complete;
//   3. grouped GEMM 1 (tcgen05, TMA, TMEM): for each local expert, as soon as its rows have
//      arrived, [gate | up] = X_e [W_gate_e | W_up_e] with SiLU(gate) * up in the epilogue;
//   4. grouped GEMM 2: Y_e = act_e W_down_e; the epilogue multiplies each row by its routing
//      weight and adds it into the OWNER rank's fp32 output row with vectorised red.add over
//      NVLink - combine and top-k reduction happen in flight, nothing is sent back as rows.
//
// A static tile order (expert by expert, GEMM 1 tiles before GEMM 2 tiles) makes every
// dependency point backwards, so the persistent CTAs cannot deadlock; every wait (arrival
// counters of remote ranks, per-m-tile readiness of `act`, mbarriers) is bounded and reports
// through the status word. No TMA multicast; remote data is pushed into local memory first and
// read with ordinary TMA tile loads.
//
// Replaces the replicated-token expert parallelism of the reference (every rank computes all
// rows, one psum; jax_gpt/models/qwen35/moe.py:117-222) and its three ragged_dot calls
// (jax_gpt/models/qwen35/moe.py:83-87).
#include "moe_kernels.cuh"

#include <cooperative_groups.h>

#include <cstdlib>

#include "comm_device.cuh"
#include "common.cuh"
#include "moe_common.cuh"
#include "tma_host.h"

namespace cg = cooperative_groups;

namespace b200 {

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2, kBBytes = BN * BK * 2, kStageBytes = kABytes + kBBytes;
// warp 0 loads, 1 issues MMAs, 2-5 run the epilogue, 6 schedules tiles, 7-10 dispatch rows (in the forward they do
// so WHILE the other warps already work on the experts whose rows are in; in the backward all warps dispatch first)
constexpr int kThreads = 352;
constexpr int kTileWarps = 7, kDispatchWarps = kThreads / 32 - kTileWarps;
constexpr int kCopyBatch = 8;  // 16-byte loads a lane keeps in flight while it copies a token row

// per-CTA phase timelines of the last profiled launch: [0] forward, [1] backward
__device__ long long g_moe_prof[2][kMoeProfCtas * kMoeProfFields];

constexpr int kTileQ = 16;      // ring of claimed tile ids read by the load, MMA and epilogue warps
constexpr int kSchedAhead = 2;  // tiles the scheduler warp may hold ready ahead of the load warp
struct MoeBars {
  uint64_t full[kStages], empty[kStages], tmem_full[2], tmem_empty[2];
  uint64_t sched_full[kSchedAhead], sched_empty[kSchedAhead];
  uint32_t tmem_base;
  int abort_flag;
  // Entry i % kTileQ holds the i-th tile this CTA claimed, or -1 after the last one. The scheduler warp writes it
  // once the tile's dependencies are met and arrives on sched_full; the load warp reads it after that wait, the
  // MMA warp after the tile's first operand wait and the epilogue after the accumulator wait. The scheduler runs
  // at most kSchedAhead tiles ahead of the load warp, which runs at most kStages tiles ahead of the MMA warp,
  // which runs at most two accumulators ahead of the epilogue: an entry is overwritten kTileQ claims later,
  // after its last reader.
  volatile int tile_q[kTileQ];
};

// The persistent CTAs take tiles in the static order from a counter of the launch (a CTA that finishes a cheap tile
// takes the next one instead of idling beside a CTA on an expensive tile). A scheduler warp per CTA claims the tile,
// waits for its dependencies (arrival counters, earlier tiles) and only then hands it to the load warp: the claim's
// and the flags' round trips to L2 stay off the path that feeds the tensor cores. The counter is the element after
// the per-m-tile flags in the layer's own act_ready (forward) / gu_ready (backward) buffer, so launches of different
// layers never share one; block 0 zeroes it before the grid barrier that precedes the tiles.

constexpr int kStageBufBytes = 4 * 32 * 33 * 4;  // per-epilogue-warp transposition buffers
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + sizeof(MoeTables) + sizeof(MoeBars) + 64 + kStageBufBytes;

__global__ void moe_prepare_kernel(const int* __restrict__ idx, int n_pairs, int* __restrict__ counts,
                                   int* __restrict__ pos) {
  for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < n_pairs; p += gridDim.x * blockDim.x)
    pos[p] = atomicAdd(&counts[idx[p]], 1);
}

}  // namespace

namespace {

__global__ void __launch_bounds__(kThreads, 1)
ep_moe_forward_kernel(const __grid_constant__ CUtensorMap t_recv, const __grid_constant__ CUtensorMap t_act,
                      const __grid_constant__ CUtensorMap t_gate, const __grid_constant__ CUtensorMap t_up,
                      const __grid_constant__ CUtensorMap t_down, const __grid_constant__ EpMoeArgs a) {
  cg::grid_group grid = cg::this_grid();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  MoeTables* tb = reinterpret_cast<MoeTables*>(smem + kStages * kStageBytes);
  MoeBars* bars = reinterpret_cast<MoeBars*>(reinterpret_cast<uint8_t*>(tb) + ((sizeof(MoeTables) + 15) & ~size_t(15)));
  volatile int* abort_flag = &bars->abort_flag;
  float* stage_buf = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + ((sizeof(MoeBars) + 15) & ~size_t(15)));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int W = a.world, EL = a.e_local, ET = W * EL, D = a.d_model, I = a.inter;
  CommCtrl* my = a.peer_ctrl[a.rank];
  const int epoch = my->epoch + 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->tmem_full[i], 1);
      mbar_init(&bars->tmem_empty[i], 4);
    }
    for (int i = 0; i < kSchedAhead; ++i) {
      mbar_init(&bars->sched_full[i], 1);
      mbar_init(&bars->sched_empty[i], 1);
    }
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  // waits that sit behind a tile's dependencies (ready tile, its operands, its accumulator) may legitimately last as
  // long as the arrival of a late peer's rows: the caller's budget on top of the pipeline's own
  const uint64_t pipe_budget = a.wait_budget_ns + kWaitBudgetNs;
  long long* prof = (a.prof != nullptr && blockIdx.x < kMoeProfCtas) ? a.prof + blockIdx.x * kMoeProfFields : nullptr;
  long long prof_clk0 = 0;
  if (prof && threadIdx.x == 0) {
    prof[0] = static_cast<long long>(globaltimer_ns());
    prof_clk0 = clock64();
  }

  // ---- 0. this rank's pairs sorted by expert: order[first pair of e + pos[p]] = p (a.slot_out holds the order).
  //         Rows are dispatched in this order, so the experts complete one after the other on every rank and the
  //         tiles of the first experts run while the rows of the later ones are still on their way. ----
  {
    // Sort key of global expert e = (dst, el): el * W + dst, so that the first local expert of EVERY destination
    // comes first and all ranks can start their tiles together (in plain expert order the last rank would receive
    // nothing until the others' experts had been served).
    if (warp == 0) {  // exclusive scan of my_counts in key order into tb->send_off (free until build_tables)
      const int per = (ET + 31) / 32;
      int sum = 0;
      for (int i = 0; i < per; ++i) {
        const int q = lane * per + i;
        if (q < ET) sum += a.my_counts[(q % W) * EL + q / W];
      }
      int incl = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      int run = incl - sum;
      for (int i = 0; i < per; ++i) {
        const int q = lane * per + i;
        if (q < ET) {
          const int e = (q % W) * EL + q / W;
          tb->send_off[e] = run;
          run += a.my_counts[e];
        }
      }
    }
    __syncthreads();
    const int n_pairs = a.tokens * a.top_k;
    for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < n_pairs; p += gridDim.x * blockDim.x) {
      const int e = a.idx[p];
      if (e >= 0 && e < ET) {
        const int at = tb->send_off[e] + a.pos[p];
        if (at >= 0 && at < n_pairs) a.slot_out[at] = p;
      }
    }
  }

  // ---- 1. publish this rank's counts, wait for everybody's ----
  {
    const int max_mt = a.cap_rows / BM + EL;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i <= max_mt; i += gridDim.x * blockDim.x) a.act_ready[i] = 0;
  }
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) {
      my->abort_flag = 0;
    }
    for (int i = threadIdx.x; i < ET; i += blockDim.x) {
      const int c = a.my_counts[i];
      for (int p = 0; p < W; ++p) a.peer_counts[p][a.rank * ET + i] = c;
    }
    const bool ok = flag_barrier(a.peer_ctrl, W, a.rank, 4, epoch, a.wait_budget_ns, a.status);
    if (!ok && threadIdx.x == 0) my->abort_flag = 1;
  }
  __threadfence();
  grid.sync();
  bool alive = (*reinterpret_cast<volatile int*>(&my->abort_flag) == 0);
  build_tables(a, a.peer_counts[a.rank], tb, /*backward=*/false, /*pad=*/64, /*claim_ahead=*/kSchedAhead);
  if (tb->overflow) {
    if (alive && blockIdx.x == 0 && threadIdx.x == 0) report_status(a.status, kBadArgument, 40, a.cap_rows, 0);
    alive = false;
  }

  if (prof && threadIdx.x == 0) prof[1] = static_cast<long long>(globaltimer_ns());

  // ---- 3./4. grouped GEMMs over the local experts ----
  const int num_tiles = alive ? tb->tile0[tb->n_slots] : 0;
  const int n1 = I / 128;
  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long dep_clk = 0;
      for (int iter = 0; ok; ++iter) {
        const int sl = iter & (kSchedAhead - 1);
        const long long c_dep = prof ? clock64() : 0;
        if (!mbar_wait(&bars->sched_full[sl], (iter / kSchedAhead) & 1, abort_flag, pipe_budget)) break;
        if (prof) dep_clk += clock64() - c_dep;
        const int t = bars->tile_q[iter & (kTileQ - 1)];
        mbar_arrive(&bars->sched_empty[sl]);
        if (t < 0) {  // end mark through the same pipeline
          if (mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag)) mbar_arrive(&bars->full[stage]);
          break;
        }
        const TileInfo ti = decode_tile(a, tb, t);
        fence_proxy_async_global();
        const int row0 = tb->base[ti.el] + ti.m * BM;
        const int nkb = (ti.phase == 0 ? D : I) / BK;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag)) {
            report_status(a.status, kWaitEmptyTimeout, 43, blockIdx.x, t);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          mbar_arrive_expect_tx(&bars->full[stage], kStageBytes);
          if (ti.phase == 0) {
            tma_load_2d(sa, &t_recv, &bars->full[stage], kb * BK, row0);
            const int ky = ti.el * D + kb * BK;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              tma_load_2d(sb + i * 8192, &t_gate, &bars->full[stage], ti.n * 128 + 64 * i, ky);
              tma_load_2d(sb + (2 + i) * 8192, &t_up, &bars->full[stage], ti.n * 128 + 64 * i, ky);
            }
          } else {
            tma_load_2d(sa, &t_act, &bars->full[stage], kb * BK, row0);
            const int ky = ti.el * I + kb * BK;
#pragma unroll
            for (int i = 0; i < 4; ++i) tma_load_2d(sb + i * 8192, &t_down, &bars->full[stage], ti.n * BN + 64 * i, ky);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (prof) {
        prof[3] = static_cast<long long>(globaltimer_ns());
        prof[5] = dep_clk;
      }
      if (!ok || *abort_flag) {
        for (int s = 0; s < kStages; ++s) {
          const uint32_t armed = (s < stage) ? phase : (phase ^ 1);
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&bars->full[s], armed)) {
            if (globaltimer_ns() - t0 > 2000000ull) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc = make_idesc(BM, BN, 0, 1, 1);
    int stage = 0, iter = 0;
    uint32_t phase = 0;
    bool ok = true;
    long long full_clk = 0, tmem_clk = 0;
    for (; ok; ++iter) {
      const int acc = iter & 1;
      // the first operands of the next tile (or the end mark) are in; its id was written before them
      const long long c_f0 = prof ? clock64() : 0;
      if (!mbar_wait(&bars->full[stage], phase, abort_flag, pipe_budget)) {
        if (lane == 0) report_status(a.status, kWaitFullTimeout, 45, blockIdx.x, iter);
        break;
      }
      if (prof) full_clk += clock64() - c_f0;
      const int t = bars->tile_q[iter & (kTileQ - 1)];
      const long long c_t = prof ? clock64() : 0;
      if (!mbar_wait(&bars->tmem_empty[acc], ((iter >> 1) & 1) ^ 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitTmemEmptyTimeout, 44, blockIdx.x, t);
        break;
      }
      if (prof) tmem_clk += clock64() - c_t;
      if (t < 0) {  // hand the end mark on to the epilogue warps
        if (lane == 0) mbar_arrive(&bars->tmem_full[acc]);
        break;
      }
      const TileInfo ti = decode_tile(a, tb, t);
      tc_fence_after();
      const int nkb = (ti.phase == 0 ? D : I) / BK;
      for (int kb = 0; kb < nkb; ++kb) {
        if (kb > 0) {
          const long long c_f = prof ? clock64() : 0;
          if (!mbar_wait(&bars->full[stage], phase, abort_flag, pipe_budget)) {
            if (lane == 0) report_status(a.status, kWaitFullTimeout, 45, blockIdx.x, t);
            ok = false;
            break;
          }
          if (prof) full_clk += clock64() - c_f;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sa = smem_u32(smem + stage * kStageBytes), sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16(tmem_base + acc * BN, make_smem_desc(sa + k * 32, 16, 1024),
                      make_smem_desc(sb + k * 2048, 8192, 1024), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit(&bars->empty[stage]);
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok && lane == 0) tc_commit(&bars->tmem_full[acc]);
      __syncwarp();
    }
    if (prof && lane == 0) {
      prof[6] = full_clk;
      prof[7] = tmem_clk;
    }
  } else if (warp == 6) {
    if (lane == 0) {
      int ready_el = -1;
      for (int i = 0;; ++i) {
        const int sl = i & (kSchedAhead - 1);
        if (!mbar_wait(&bars->sched_empty[sl], ((i / kSchedAhead) & 1) ^ 1, abort_flag)) break;
        const int t = atomicAdd(a.act_ready + a.cap_rows / BM + EL, 1);
        if (t >= num_tiles) {
          bars->tile_q[i & (kTileQ - 1)] = -1;
          mbar_arrive(&bars->sched_full[sl]);
          break;
        }
        const TileInfo ti = decode_tile(a, tb, t);
        if (ti.phase == 0) {
          if (ti.el != ready_el) {
            const unsigned target = a.arrive_target[ti.el] + static_cast<unsigned>(tb->rows[ti.el]);
            if (!wait_counter_ge<true>(a.peer_arrive[a.rank] + ti.el, target, a.wait_budget_ns, abort_flag)) {
              report_status(a.status, kWaitFlagTimeout, 41, ti.el, t);
              break;
            }
            ready_el = ti.el;
          }
        } else {
          const unsigned* ready = reinterpret_cast<const unsigned*>(a.act_ready) + tb->mt0[ti.el] + ti.m;
          if (!wait_counter_ge<false>(ready, 4u * n1, a.wait_budget_ns, abort_flag)) {
            report_status(a.status, kWaitFlagTimeout, 42, ti.el, t);
            break;
          }
        }
        bars->tile_q[i & (kTileQ - 1)] = t;
        mbar_arrive(&bars->sched_full[sl]);
      }
    }
  } else if (warp < kTileWarps) {
    const int q = warp & 3;
    int iter = 0;
    for (;; ++iter) {
      const int acc = iter & 1;
      if (!mbar_wait(&bars->tmem_full[acc], (iter >> 1) & 1, abort_flag, pipe_budget)) {
        if (lane == 0) report_status(a.status, kWaitTmemFullTimeout, 46, blockIdx.x, iter);
        break;
      }
      const int t = bars->tile_q[iter & (kTileQ - 1)];
      if (t < 0) break;
      const TileInfo ti = decode_tile(a, tb, t);
      tc_fence_after();
      const int r = ti.m * BM + q * 32 + lane;            // row within the expert
      const bool row_ok = r < tb->rows[ti.el];
      const bool pad_row = !row_ok && r < ((tb->rows[ti.el] + 63) & ~63);  // padding rows are written as zeros
      const int64_t row = tb->base[ti.el] + r;            // row in the receive buffer
      const uint32_t tacc = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      if (ti.phase == 0) {
        __nv_bfloat16* dst = a.act + row * I + ti.n * 128;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t g[32], u[32];
          tmem_ld_32x32(tacc + c * 32, g);
          tmem_ld_32x32(tacc + 128 + c * 32, u);
          tmem_ld_wait();
          if (row_ok || pad_row) {
            const float keep = row_ok ? 1.f : 0.f;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint32_t pk[4], pg[4], pu[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float g0 = __uint_as_float(g[j + 2 * e]) * keep, g1 = __uint_as_float(g[j + 2 * e + 1]) * keep;
                const float u0 = __uint_as_float(u[j + 2 * e]) * keep, u1 = __uint_as_float(u[j + 2 * e + 1]) * keep;
                pk[e] = pack_bf16x2(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
                pg[e] = pack_bf16x2(g0, g1);
                pu[e] = pack_bf16x2(u0, u1);
              }
              *reinterpret_cast<uint4*>(dst + c * 32 + j) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              if (a.gu != nullptr) {  // pre-activations kept for the backward pass: [row, gate | up]
                __nv_bfloat16* gp = a.gu + row * (2 * I) + ti.n * 128 + c * 32 + j;
                *reinterpret_cast<uint4*>(gp) = make_uint4(pg[0], pg[1], pg[2], pg[3]);
                *reinterpret_cast<uint4*>(gp + I) = make_uint4(pu[0], pu[1], pu[2], pu[3]);
              }
            }
          }
        }
      } else {
        // Weighted combine. Each lane owns one row of the tile, but a row-per-lane reduction would
        // put 32 scattered 16-byte pieces on NVLink per instruction; the chunk is transposed through
        // shared memory so that eight lanes cover 128 contiguous bytes of one destination row.
        float wgt = 0.f;
        float* dst = nullptr;
        if (row_ok) {
          wgt = a.peer_recv_w[a.rank][row];
          const int meta = a.peer_recv_meta[a.rank][row];
          if (bounds_ok(meta >> 24, W, a.status, 203) && bounds_ok(meta & 0xFFFFFF, a.tokens * a.top_k, a.status, 204))
            dst = a.peer_out[meta >> 24] + static_cast<int64_t>((meta & 0xFFFFFF) / a.top_k) * D + ti.n * BN;
        }
        float* stg = stage_buf + (warp - 2) * (32 * 33);
        const unsigned long long dst_bits = reinterpret_cast<unsigned long long>(dst);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tacc + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) stg[lane * 33 + j] = __uint_as_float(v[j]) * wgt;
          __syncwarp();
#pragma unroll
          for (int rr = 0; rr < 32; rr += 4) {
            const int r2 = rr + (lane >> 3), c2 = (lane & 7) * 4;
            const unsigned long long db = __shfl_sync(0xffffffffu, dst_bits, r2);
            if (db != 0ull) {
              float* d2 = reinterpret_cast<float*>(db) + c * 32 + c2;
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d2), "f"(stg[r2 * 33 + c2]),
                           "f"(stg[r2 * 33 + c2 + 1]), "f"(stg[r2 * 33 + c2 + 2]), "f"(stg[r2 * 33 + c2 + 3])
                           : "memory");
            }
          }
          __syncwarp();
        }
      }
      tc_fence_before();
      if (ti.phase == 0) {
        __threadfence();
        fence_proxy_async_global();
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bars->tmem_empty[acc]);
        if (ti.phase == 0) atomicAdd(a.act_ready + tb->mt0[ti.el] + ti.m, 1);
      }
    }
    if (prof && warp == 2 && lane == 0) prof[8] = static_cast<long long>(globaltimer_ns());
  } else if (alive) {
    // ---- dispatch warps: rows in expert order, two per pass, 16-byte loads batched; the routing entries of the
    //      next pass and the order entries of the one after are fetched ahead of the copy ----
    const int n_pairs = a.tokens * a.top_k, nv = D / 8;
    const int g0 = blockIdx.x * kDispatchWarps + (warp - kTileWarps), gs = gridDim.x * kDispatchWarps;
    const int* order = a.slot_out;
    int p_nx[2], e_nx[2], pos_nx[2], p_n2[2];
    float w_nx[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int s0 = g0 + h * gs, s1 = g0 + (2 + h) * gs;
      p_nx[h] = s0 < n_pairs ? order[s0] : -1;
      p_n2[h] = s1 < n_pairs ? order[s1] : -1;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      e_nx[h] = p_nx[h] >= 0 ? a.idx[p_nx[h]] : 0;
      pos_nx[h] = p_nx[h] >= 0 ? a.pos[p_nx[h]] : 0;
      w_nx[h] = p_nx[h] >= 0 ? a.w[p_nx[h]] : 0.f;
    }
    int pend_e = -1;  // lane 2 * (pass % 4) + h remembers the expert of a delivered row until the next flush
    for (int k = 0, s = g0; s < n_pairs; ++k, s += 2 * gs) {
      const uint4* src[2] = {nullptr, nullptr};
      uint4* out[2] = {nullptr, nullptr};
      int p_cur[2], e_cur[2], pos_cur[2];
      float w_cur[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        p_cur[h] = p_nx[h];
        e_cur[h] = e_nx[h];
        pos_cur[h] = pos_nx[h];
        w_cur[h] = w_nx[h];
        p_nx[h] = p_n2[h];
        e_nx[h] = p_nx[h] >= 0 ? a.idx[p_nx[h]] : 0;
        pos_nx[h] = p_nx[h] >= 0 ? a.pos[p_nx[h]] : 0;
        w_nx[h] = p_nx[h] >= 0 ? a.w[p_nx[h]] : 0.f;
        const int s2 = s + (4 + h) * gs;
        p_n2[h] = s2 < n_pairs ? order[s2] : -1;
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int pp = p_cur[h];
        if (pp < 0) continue;
        const int e = e_cur[h];
        if (!bounds_ok(pp, n_pairs, a.status, 200) || !bounds_ok(e, ET, a.status, 201)) continue;
        const int dst = e / EL;
        const int slot = tb->send_off[e] + pos_cur[h];
        if (!bounds_ok(slot, a.cap_rows, a.status, 202)) continue;
        src[h] = reinterpret_cast<const uint4*>(a.x + static_cast<int64_t>(pp / a.top_k) * D);
        out[h] = reinterpret_cast<uint4*>(a.peer_recv_x[dst] + static_cast<int64_t>(slot) * D);
        if (lane == 0) {
          a.peer_recv_meta[dst][slot] = (a.rank << 24) | pp;  // source rank and (token, choice) pair
          a.peer_recv_w[dst][slot] = w_cur[h];
        }
        if (lane == 2 * (k & 3) + h) pend_e = e;
      }
      for (int i0 = lane; i0 < nv; i0 += 32 * kCopyBatch) {  // all loads of a batch in flight before the first store
        uint4 v[2][kCopyBatch];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int u = 0; u < kCopyBatch; ++u)
            if (src[h] != nullptr && i0 + 32 * u < nv) v[h][u] = __ldg(src[h] + i0 + 32 * u);
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int u = 0; u < kCopyBatch; ++u)
            if (src[h] != nullptr && i0 + 32 * u < nv) out[h][i0 + 32 * u] = v[h][u];
      }
      // Arrivals of up to four passes with one fence (the first two passes signal at once so that the first
      // experts start early): barrier -> fence -> relaxed reduction is a release sequence over every lane's stores.
      if (k < 2 || (k & 3) == 3 || s + 2 * gs >= n_pairs) {
        __syncwarp();
        __threadfence_system();
        if (pend_e >= 0) red_relaxed_sys_add_u32(a.peer_arrive[pend_e / EL] + (pend_e % EL), 1u);
        pend_e = -1;
        __syncwarp();
      }
    }
    if (prof && warp == kTileWarps && lane == 0) prof[2] = static_cast<long long>(globaltimer_ns());
  }

  // ---- 5. every rank's contributions have landed before anybody returns ----
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
  __threadfence_system();
  grid.sync();
  if (blockIdx.x == 0) {
    flag_barrier(a.peer_ctrl, W, a.rank, 5, epoch, a.wait_budget_ns, a.status);
    if (alive) {
      for (int el = threadIdx.x; el < EL; el += blockDim.x) {
        a.arrive_target[el] += static_cast<unsigned>(tb->rows[el]);
        a.rows_out[el] = tb->rows[el];
      }
    }
    if (threadIdx.x == 0) my->epoch = epoch;
  }
  if (prof && threadIdx.x == 0) {
    prof[4] = static_cast<long long>(globaltimer_ns());
    prof[9] = clock64() - prof_clk0;
  }
}


// ------------------------------------------------------------------------------------------------
// Backward. Tiles of a local expert (rows > 0):
//   Q0  dAct = dYw W_down^T  (+ SwiGLU backward -> dGU, <dAct, act> per row)      mt x I/256 tiles
//   Q2  dW_down += act^T dYw          (ragged K = the expert's rows, 64-row blocks)  I/128 x D/256
//   Q1  dX   = dGU [W_gate | W_up]^T, pushed to the token owners                     mt x D/256
//   Q3  dW_gate | dW_up += X^T dGU    (ragged K)                                     D/128 x 2I/256
// Q1 waits for the Q0 tiles of its m-tile, Q3 for all Q0 tiles of its expert. Slot s of the static order holds
// Q0 and Q2 of expert s, then Q1 and Q3 of expert s - lag: the dependencies point backwards by about two rounds
// of the grid, so a CTA rarely reaches a dependent tile before the tiles it needs are done.
struct BwdTile {
  int el, phase, m, n;
};

__host__ __device__ __forceinline__ BwdTile decode_bwd_tile(const EpMoeArgs& a, const MoeTables* tb, int t) {
  int sl = 0, hi = tb->n_slots - 1;  // first slot whose tile range ends after t
  while (sl < hi) {
    const int mid = (sl + hi) >> 1;
    if (tb->tile0[mid + 1] > t) hi = mid;
    else sl = mid + 1;
  }
  int r = t - tb->tile0[sl];
  const int n2 = a.d_model / BN;
  BwdTile ti;
  int front = 0;
  if (sl < a.e_local) {
    const int mt = (tb->rows[sl] + BM - 1) / BM;
    if (mt > 0) {
      const int c0 = mt * (a.inter / BN);
      front = c0 + (a.inter / BM) * n2;
      if (r < c0) {
        ti.el = sl; ti.phase = 0; ti.m = r % mt; ti.n = r / mt;
        return ti;
      }
      if (r < front) {
        r -= c0;
        ti.el = sl; ti.phase = 2; ti.m = r % (a.inter / BM); ti.n = r / (a.inter / BM);
        return ti;
      }
    }
  }
  r -= front;
  ti.el = sl - tb->lag;
  const int mt = (tb->rows[ti.el] + BM - 1) / BM;
  const int c1 = mt * n2;
  if (r < c1) {
    ti.phase = 1; ti.m = r % mt; ti.n = r / mt;
  } else {
    r -= c1; ti.phase = 3; ti.m = r % (a.d_model / BM); ti.n = r / (a.d_model / BM);
  }
  return ti;
}

struct BwdMaps {
  CUtensorMap dy_k, dgu_k, down_k, gate_k, up_k;  // K-major views: box {64, 128} for activations, {64, 256} for weights
  CUtensorMap act_mn, dy_mn, x_mn, dgu_mn;        // MN-major views of the row buffers: box {64, 64}
};

__global__ void __launch_bounds__(kThreads, 1)
ep_moe_backward_kernel(const __grid_constant__ BwdMaps tm, const __grid_constant__ EpMoeArgs a) {
  cg::grid_group grid = cg::this_grid();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  MoeTables* tb = reinterpret_cast<MoeTables*>(smem + kStages * kStageBytes);
  MoeBars* bars = reinterpret_cast<MoeBars*>(reinterpret_cast<uint8_t*>(tb) + ((sizeof(MoeTables) + 15) & ~size_t(15)));
  volatile int* abort_flag = &bars->abort_flag;
  float* stage_buf = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + ((sizeof(MoeBars) + 15) & ~size_t(15)));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int W = a.world, EL = a.e_local, ET = W * EL, D = a.d_model, I = a.inter;
  CommCtrl* my = a.peer_ctrl[a.rank];
  const int epoch = my->epoch + 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->tmem_full[i], 1);
      mbar_init(&bars->tmem_empty[i], 4);
    }
    for (int i = 0; i < kSchedAhead; ++i) {
      mbar_init(&bars->sched_full[i], 1);
      mbar_init(&bars->sched_empty[i], 1);
    }
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  // waits that sit behind a tile's dependencies (ready tile, its operands, its accumulator) may legitimately last as
  // long as the arrival of a late peer's rows: the caller's budget on top of the pipeline's own
  const uint64_t pipe_budget = a.wait_budget_ns + kWaitBudgetNs;
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x, gthreads = gridDim.x * blockDim.x;
  long long* prof = (a.prof != nullptr && blockIdx.x < kMoeProfCtas) ? a.prof + blockIdx.x * kMoeProfFields : nullptr;
  long long prof_clk0 = 0;
  if (prof && threadIdx.x == 0) {
    prof[0] = static_cast<long long>(globaltimer_ns());
    prof_clk0 = clock64();
  }

  // ---- 1. counts exchange (same protocol as forward), zero the per-launch counters ----
  {
    const int max_mt = a.cap_rows / BM + EL;
    for (int i = gtid; i <= max_mt; i += gthreads) a.gu_ready[i] = 0;
    for (int i = gtid; i < EL; i += gthreads) a.expert_done[i] = 0;
    for (int i = gtid; i < a.cap_rows; i += gthreads) a.dw_rows[i] = 0.f;
  }
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) {
      my->abort_flag = 0;
    }
    for (int i = threadIdx.x; i < ET; i += blockDim.x) {
      const int c = a.my_counts[i];
      for (int p = 0; p < W; ++p) a.peer_counts[p][a.rank * ET + i] = c;
    }
    const bool ok = flag_barrier(a.peer_ctrl, W, a.rank, 4, epoch, a.wait_budget_ns, a.status);
    if (!ok && threadIdx.x == 0) my->abort_flag = 1;
  }
  __threadfence();
  grid.sync();
  bool alive = (*reinterpret_cast<volatile int*>(&my->abort_flag) == 0);
  build_tables(a, a.peer_counts[a.rank], tb, /*backward=*/true, /*pad=*/64, /*claim_ahead=*/kSchedAhead);
  if (tb->overflow) {
    if (alive && blockIdx.x == 0 && threadIdx.x == 0) report_status(a.status, kBadArgument, 50, a.cap_rows, 0);
    alive = false;
  }
  if (prof && threadIdx.x == 0) prof[1] = static_cast<long long>(globaltimer_ns());

  // ---- 2. keep the padding rows of the receive buffers zero (nobody else writes them) ----
  if (alive) {
    const int vec_per_row = D / 8;
    for (int el = 0; el < EL; ++el) {
      const int r0 = tb->base[el] + tb->rows[el], r1 = tb->base[el] + ((tb->rows[el] + 63) & ~63);
      const int64_t n = static_cast<int64_t>(r1 - r0) * vec_per_row;
      uint4* px = reinterpret_cast<uint4*>(a.peer_recv_x[a.rank] + static_cast<int64_t>(r0) * D);
      uint4* py = reinterpret_cast<uint4*>(a.peer_recv_dy[a.rank] + static_cast<int64_t>(r0) * D);
      for (int64_t i = gtid; i < n; i += gthreads) {
        px[i] = make_uint4(0, 0, 0, 0);
        py[i] = make_uint4(0, 0, 0, 0);
      }
    }
  }

  // ---- 3. dispatch the routing-weighted dout rows to the slots the forward pass used (the x rows, the
  //         routing metadata, act and the pre-activations are still in place from the forward launch) ----
  if (alive) {
    const int n_pairs = a.tokens * a.top_k, nv = D / 8;
    const int w0 = blockIdx.x * (kThreads / 32) + warp, wstep = gridDim.x * (kThreads / 32);
    // two rows per pass (twice the loads in flight); the routing entries of the next pass are fetched before
    // this pass's rows so that their latency hides behind the copy
    int e_nx[2], pos_nx[2];
    float w_nx[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int pp = w0 + h * wstep;
      e_nx[h] = pp < n_pairs ? a.idx[pp] : 0;
      pos_nx[h] = pp < n_pairs ? a.pos[pp] : 0;
      w_nx[h] = pp < n_pairs ? a.w[pp] : 0.f;
    }
    for (int p = w0; p < n_pairs; p += 2 * wstep) {
      const uint4* sy[2] = {nullptr, nullptr};
      uint4* oy[2] = {nullptr, nullptr};
      float wp[2] = {0.f, 0.f};
      int e_cur[2], pos_cur[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        e_cur[h] = e_nx[h];
        pos_cur[h] = pos_nx[h];
        wp[h] = w_nx[h];
        const int pn = p + (2 + h) * wstep;
        e_nx[h] = pn < n_pairs ? a.idx[pn] : 0;
        pos_nx[h] = pn < n_pairs ? a.pos[pn] : 0;
        w_nx[h] = pn < n_pairs ? a.w[pn] : 0.f;
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int pp = p + h * wstep;
        if (pp >= n_pairs) continue;
        const int e = e_cur[h];
        const int slot = tb->send_off[e] + pos_cur[h];
        sy[h] = reinterpret_cast<const uint4*>(a.dout + static_cast<int64_t>(pp / a.top_k) * D);
        oy[h] = reinterpret_cast<uint4*>(a.peer_recv_dy[e / EL] + static_cast<int64_t>(slot) * D);
      }
      for (int i0 = lane; i0 < nv; i0 += 32 * kCopyBatch) {  // all loads of a batch in flight before the first store
        uint4 v[2][kCopyBatch];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int u = 0; u < kCopyBatch; ++u)
            if (sy[h] != nullptr && i0 + 32 * u < nv) v[h][u] = __ldg(sy[h] + i0 + 32 * u);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int u = 0; u < kCopyBatch; ++u) {
            if (sy[h] != nullptr && i0 + 32 * u < nv) {
              const uint4 x4 = v[h][u];
              const float2 f0 = unpack_bf16x2(x4.x), f1 = unpack_bf16x2(x4.y), f2 = unpack_bf16x2(x4.z), f3 = unpack_bf16x2(x4.w);
              oy[h][i0 + 32 * u] = make_uint4(pack_bf16x2(f0.x * wp[h], f0.y * wp[h]), pack_bf16x2(f1.x * wp[h], f1.y * wp[h]),
                                              pack_bf16x2(f2.x * wp[h], f2.y * wp[h]), pack_bf16x2(f3.x * wp[h], f3.y * wp[h]));
            }
          }
        }
      }
    }
    // one fence for all rows this warp delivered, then their arrival counts (lane l signs for the warp's pairs
    // l, l + 32, ...): barrier -> fence -> relaxed reduction is a release sequence over every lane's stores
    __syncwarp();
    __threadfence_system();
    int j = 0;
    for (int p = w0; p < n_pairs; p += wstep, ++j) {
      if ((j & 31) != lane) continue;
      const int e = a.idx[p];
      red_relaxed_sys_add_u32(a.peer_arrive[e / EL] + (e % EL), 1u);
    }
  }
  if (prof && threadIdx.x == 0) prof[2] = static_cast<long long>(globaltimer_ns());
  __threadfence();  // the zeroed padding rows are visible before any tile reads them
  grid.sync();

  const int num_tiles = alive ? tb->tile0[tb->n_slots] : 0;
  const unsigned q0_per_mtile = 4u * (I / BN);
  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long dep_clk = 0;
      for (int iter = 0; ok; ++iter) {
        const int sl = iter & (kSchedAhead - 1);
        const long long c_dep = prof ? clock64() : 0;
        if (!mbar_wait(&bars->sched_full[sl], (iter / kSchedAhead) & 1, abort_flag, pipe_budget)) break;
        if (prof) dep_clk += clock64() - c_dep;
        const int t = bars->tile_q[iter & (kTileQ - 1)];
        mbar_arrive(&bars->sched_empty[sl]);
        if (t < 0) {  // end mark through the same pipeline
          if (mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag)) mbar_arrive(&bars->full[stage]);
          break;
        }
        const BwdTile ti = decode_bwd_tile(a, tb, t);
        const int rows = tb->rows[ti.el], base = tb->base[ti.el];
        fence_proxy_async_global();
        const int nkb = ti.phase == 0 ? D / BK : (ti.phase == 1 ? 2 * I / BK : ((rows + 63) & ~63) / BK);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag)) {
            report_status(a.status, kWaitEmptyTimeout, 54, blockIdx.x, t);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          uint64_t* fb = &bars->full[stage];
          mbar_arrive_expect_tx(fb, kStageBytes);
          if (ti.phase == 0) {
            tma_load_2d(sa, &tm.dy_k, fb, kb * BK, base + ti.m * BM);
            tma_load_2d(sb, &tm.down_k, fb, kb * BK, ti.el * I + ti.n * BN);
          } else if (ti.phase == 1) {
            tma_load_2d(sa, &tm.dgu_k, fb, kb * BK, base + ti.m * BM);
            const int kh = I / BK;
            tma_load_2d(sb, kb < kh ? &tm.gate_k : &tm.up_k, fb, (kb % kh) * BK, ti.el * D + ti.n * BN);
          } else {
            const CUtensorMap* ma = ti.phase == 2 ? &tm.act_mn : &tm.x_mn;
            const CUtensorMap* mb = ti.phase == 2 ? &tm.dy_mn : &tm.dgu_mn;
            const int ky = base + kb * BK;
#pragma unroll
            for (int i = 0; i < 2; ++i) tma_load_2d(sa + i * 8192, ma, fb, ti.m * BM + 64 * i, ky);
#pragma unroll
            for (int i = 0; i < 4; ++i) tma_load_2d(sb + i * 8192, mb, fb, ti.n * BN + 64 * i, ky);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (prof) {
        prof[3] = static_cast<long long>(globaltimer_ns());
        prof[5] = dep_clk;
      }
      if (!ok || *abort_flag) {
        for (int s = 0; s < kStages; ++s) {
          const uint32_t armed = (s < stage) ? phase : (phase ^ 1);
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&bars->full[s], armed)) {
            if (globaltimer_ns() - t0 > 2000000ull) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc_kk = make_idesc(BM, BN, 0, 0, 1);
    constexpr uint32_t idesc_nn = make_idesc(BM, BN, 1, 1, 1);
    int stage = 0, iter = 0;
    uint32_t phase = 0;
    bool ok = true;
    long long full_clk = 0, tmem_clk = 0;
    for (; ok; ++iter) {
      const int acc = iter & 1;
      // the first operands of the next tile (or the end mark) are in; its id was written before them
      const long long c_f0 = prof ? clock64() : 0;
      if (!mbar_wait(&bars->full[stage], phase, abort_flag, pipe_budget)) {
        if (lane == 0) report_status(a.status, kWaitFullTimeout, 56, blockIdx.x, iter);
        break;
      }
      if (prof) full_clk += clock64() - c_f0;
      const int t = bars->tile_q[iter & (kTileQ - 1)];
      const long long c_t = prof ? clock64() : 0;
      if (!mbar_wait(&bars->tmem_empty[acc], ((iter >> 1) & 1) ^ 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitTmemEmptyTimeout, 55, blockIdx.x, t);
        break;
      }
      if (prof) tmem_clk += clock64() - c_t;
      if (t < 0) {  // hand the end mark on to the epilogue warps
        if (lane == 0) mbar_arrive(&bars->tmem_full[acc]);
        break;
      }
      const BwdTile ti = decode_bwd_tile(a, tb, t);
      tc_fence_after();
      const int rows = tb->rows[ti.el];
      const int nkb = ti.phase == 0 ? D / BK : (ti.phase == 1 ? 2 * I / BK : ((rows + 63) & ~63) / BK);
      const bool mn = ti.phase >= 2;
      for (int kb = 0; kb < nkb; ++kb) {
        if (kb > 0) {
          const long long c_f = prof ? clock64() : 0;
          if (!mbar_wait(&bars->full[stage], phase, abort_flag, pipe_budget)) {
            if (lane == 0) report_status(a.status, kWaitFullTimeout, 56, blockIdx.x, t);
            ok = false;
            break;
          }
          if (prof) full_clk += clock64() - c_f;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sa = smem_u32(smem + stage * kStageBytes), sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = mn ? make_smem_desc(sa + k * 2048, 8192, 1024) : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t bd = mn ? make_smem_desc(sb + k * 2048, 8192, 1024) : make_smem_desc(sb + k * 32, 16, 1024);
            umma_bf16(tmem_base + acc * BN, ad, bd, mn ? idesc_nn : idesc_kk, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&bars->empty[stage]);
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok && lane == 0) tc_commit(&bars->tmem_full[acc]);
      __syncwarp();
    }
    if (prof && lane == 0) {
      prof[6] = full_clk;
      prof[7] = tmem_clk;
    }
  } else if (warp == 6) {
    if (lane == 0) {
      int ready_el = -1;
      for (int i = 0;; ++i) {
        const int sl = i & (kSchedAhead - 1);
        if (!mbar_wait(&bars->sched_empty[sl], ((i / kSchedAhead) & 1) ^ 1, abort_flag)) break;
        const int t = atomicAdd(a.gu_ready + a.cap_rows / BM + EL, 1);
        if (t >= num_tiles) {
          bars->tile_q[i & (kTileQ - 1)] = -1;
          mbar_arrive(&bars->sched_full[sl]);
          break;
        }
        const BwdTile ti = decode_bwd_tile(a, tb, t);
        const int rows = tb->rows[ti.el];
        const int mt = (rows + BM - 1) / BM;
        if ((ti.phase == 0 || ti.phase == 2) && ti.el != ready_el) {
          // the dy rows of this expert have arrived (Q1 / Q3 read only what the Q0 tiles they wait for produced,
          // and the x rows of the forward launch)
          const unsigned target = a.arrive_target[ti.el] + static_cast<unsigned>(rows);
          if (!wait_counter_ge<true>(a.peer_arrive[a.rank] + ti.el, target, a.wait_budget_ns, abort_flag)) {
            report_status(a.status, kWaitFlagTimeout, 51, ti.el, t);
            break;
          }
          ready_el = ti.el;
        }
        if (ti.phase == 1) {
          const unsigned* ready = reinterpret_cast<const unsigned*>(a.gu_ready) + tb->mt0[ti.el] + ti.m;
          if (!wait_counter_ge<false>(ready, q0_per_mtile, a.wait_budget_ns, abort_flag)) {
            report_status(a.status, kWaitFlagTimeout, 52, ti.el, t);
            break;
          }
        } else if (ti.phase == 3) {
          const unsigned* done = reinterpret_cast<const unsigned*>(a.expert_done) + ti.el;
          if (!wait_counter_ge<false>(done, q0_per_mtile * mt, a.wait_budget_ns, abort_flag)) {
            report_status(a.status, kWaitFlagTimeout, 53, ti.el, t);
            break;
          }
        }
        bars->tile_q[i & (kTileQ - 1)] = t;
        mbar_arrive(&bars->sched_full[sl]);
      }
    }
  } else if (warp < kTileWarps) {
    const int q = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    float* stg = stage_buf + (warp - 2) * (32 * 33);
    int iter = 0;
    for (;; ++iter) {
      const int acc = iter & 1;
      if (!mbar_wait(&bars->tmem_full[acc], (iter >> 1) & 1, abort_flag, pipe_budget)) {
        if (lane == 0) report_status(a.status, kWaitTmemFullTimeout, 57, blockIdx.x, iter);
        break;
      }
      const int t = bars->tile_q[iter & (kTileQ - 1)];
      if (t < 0) break;
      const BwdTile ti = decode_bwd_tile(a, tb, t);
      tc_fence_after();
      const uint32_t tacc = tmem_base + acc * BN + lane_off;
      const int rows = tb->rows[ti.el], base = tb->base[ti.el];
      if (ti.phase == 0) {
        // dAct tile -> SwiGLU backward. act = silu(g) * u is recomputed from the saved pre-activations.
        const int r = ti.m * BM + q * 32 + lane;
        const bool row_ok = r < rows;
        const bool pad_row = !row_ok && r < ((rows + 63) & ~63);
        const int64_t row = base + r;
        float dwp = 0.f;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tacc + c * 32, v);
          tmem_ld_wait();
          const int col = ti.n * BN + c * 32;
          if (row_ok) {
            const __nv_bfloat16* gp = a.gu + row * (2 * I) + col;
            __nv_bfloat16* op = a.dgu + row * (2 * I) + col;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              const uint4 gr = *reinterpret_cast<const uint4*>(gp + j);
              const uint4 ur = *reinterpret_cast<const uint4*>(gp + I + j);
              const uint32_t gw[4] = {gr.x, gr.y, gr.z, gr.w}, uw[4] = {ur.x, ur.y, ur.z, ur.w};
              uint32_t og[4], ou[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 g2 = unpack_bf16x2(gw[e]), u2 = unpack_bf16x2(uw[e]);
                const float d0 = __uint_as_float(v[j + 2 * e]), d1 = __uint_as_float(v[j + 2 * e + 1]);
                const float s0 = 1.f / (1.f + __expf(-g2.x)), s1 = 1.f / (1.f + __expf(-g2.y));
                const float l0 = g2.x * s0, l1 = g2.y * s1;  // silu
                dwp += d0 * l0 * u2.x + d1 * l1 * u2.y;
                ou[e] = pack_bf16x2(d0 * l0, d1 * l1);
                og[e] = pack_bf16x2(d0 * u2.x * s0 * (1.f + g2.x * (1.f - s0)), d1 * u2.y * s1 * (1.f + g2.y * (1.f - s1)));
              }
              *reinterpret_cast<uint4*>(op + j) = make_uint4(og[0], og[1], og[2], og[3]);
              *reinterpret_cast<uint4*>(op + I + j) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
            }
          } else if (pad_row) {
            __nv_bfloat16* op = a.dgu + row * (2 * I) + col;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              *reinterpret_cast<uint4*>(op + j) = make_uint4(0, 0, 0, 0);
              *reinterpret_cast<uint4*>(op + I + j) = make_uint4(0, 0, 0, 0);
            }
          }
        }
        if (row_ok) atomicAdd(a.dw_rows + row, dwp);
      } else if (ti.phase == 1) {
        // dX rows go to the token owners with coalesced fp32 reductions (see the forward combine)
        const int r = ti.m * BM + q * 32 + lane;
        float* dst = nullptr;
        if (r < rows) {
          const int meta = a.peer_recv_meta[a.rank][base + r];
          if (bounds_ok(meta >> 24, W, a.status, 205) && bounds_ok(meta & 0xFFFFFF, a.tokens * a.top_k, a.status, 206))
            dst = a.peer_dx[meta >> 24] + static_cast<int64_t>((meta & 0xFFFFFF) / a.top_k) * D + ti.n * BN;
        }
        const unsigned long long dst_bits = reinterpret_cast<unsigned long long>(dst);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tacc + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) stg[lane * 33 + j] = __uint_as_float(v[j]);
          __syncwarp();
#pragma unroll
          for (int rr = 0; rr < 32; rr += 4) {
            const int r2 = rr + (lane >> 3), c2 = (lane & 7) * 4;
            const unsigned long long db = __shfl_sync(0xffffffffu, dst_bits, r2);
            if (db != 0ull) {
              float* d2 = reinterpret_cast<float*>(db) + c * 32 + c2;
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d2), "f"(stg[r2 * 33 + c2]),
                           "f"(stg[r2 * 33 + c2 + 1]), "f"(stg[r2 * 33 + c2 + 2]), "f"(stg[r2 * 33 + c2 + 3])
                           : "memory");
            }
          }
          __syncwarp();
        }
      } else {
        // weight-gradient tiles: every row of the tile is a real weight row; accumulate in fp32. Each lane holds
        // one row of the accumulator; the chunk is transposed through shared memory so that eight lanes add
        // 128 contiguous bytes of one weight row (whole sectors per reduction instead of 16-byte pieces).
        float* dst;
        int64_t ld;
        if (ti.phase == 2) {
          ld = D;
          dst = a.d_down + (static_cast<int64_t>(ti.el) * I + ti.m * BM + q * 32) * D + ti.n * BN;
        } else {
          const int col0 = ti.n * BN;
          ld = I;
          dst = (col0 < I ? a.d_gate : a.d_up) + (static_cast<int64_t>(ti.el) * D + ti.m * BM + q * 32) * I +
                (col0 < I ? col0 : col0 - I);
        }
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tacc + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) stg[lane * 33 + j] = __uint_as_float(v[j]);
          __syncwarp();
#pragma unroll
          for (int rr = 0; rr < 32; rr += 4) {
            const int r2 = rr + (lane >> 3), c2 = (lane & 7) * 4;
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + r2 * ld + c * 32 + c2),
                         "f"(stg[r2 * 33 + c2]), "f"(stg[r2 * 33 + c2 + 1]), "f"(stg[r2 * 33 + c2 + 2]),
                         "f"(stg[r2 * 33 + c2 + 3])
                         : "memory");
          }
          __syncwarp();
        }
      }
      tc_fence_before();
      if (ti.phase == 0) {
        __threadfence();
        fence_proxy_async_global();
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bars->tmem_empty[acc]);
        if (ti.phase == 0) {
          atomicAdd(a.gu_ready + tb->mt0[ti.el] + ti.m, 1);
          atomicAdd(a.expert_done + ti.el, 1);
        }
      }
    }
    if (prof && warp == 2 && lane == 0) prof[8] = static_cast<long long>(globaltimer_ns());
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
  __threadfence();
  grid.sync();
  // ---- routing-weight gradients back to the pair owners: dw = <dAct_weighted, act> / w ----
  if (alive) {
    const int total = tb->base[EL - 1] + tb->rows[EL - 1];
    for (int row = gtid; row < total; row += gthreads) {
      int el = 0;
      while (el + 1 < EL && row >= tb->base[el + 1]) ++el;
      if (row - tb->base[el] < tb->rows[el]) {
        const int meta = a.peer_recv_meta[a.rank][row];
        const float wv = a.peer_recv_w[a.rank][row];
        if (!bounds_ok(meta >> 24, W, a.status, 207) || !bounds_ok(meta & 0xFFFFFF, a.tokens * a.top_k, a.status, 208)) continue;
        a.peer_dw[meta >> 24][meta & 0xFFFFFF] = (wv != 0.f) ? __ldcg(a.dw_rows + row) / wv : 0.f;
      }
    }
  }
  __threadfence_system();
  grid.sync();
  if (blockIdx.x == 0) {
    flag_barrier(a.peer_ctrl, W, a.rank, 5, epoch, a.wait_budget_ns, a.status);
    if (alive) {
      for (int el = threadIdx.x; el < EL; el += blockDim.x) {
        a.arrive_target[el] += static_cast<unsigned>(tb->rows[el]);
        a.rows_out[el] = tb->rows[el];
      }
    }
    if (threadIdx.x == 0) my->epoch = epoch;
  }
  if (prof && threadIdx.x == 0) {
    prof[4] = static_cast<long long>(globaltimer_ns());
    prof[9] = clock64() - prof_clk0;
  }
}

}  // namespace

namespace {
// Address of the timeline buffer when B200_MOE_PROFILE=1 was set before the first launch, else nullptr.
long long* moe_prof_buffer(int which) {
  static int enabled = -1;
  static long long* base = nullptr;
  if (enabled < 0) {
    const char* env = getenv("B200_MOE_PROFILE");
    enabled = (env != nullptr && env[0] == '1') ? 1 : 0;
    if (enabled && cudaGetSymbolAddress(reinterpret_cast<void**>(&base), g_moe_prof) != cudaSuccess) enabled = 0;
  }
  return enabled ? base + which * kMoeProfCtas * kMoeProfFields : nullptr;
}
}  // namespace

int moe_tile_order_host(const int* rows, int e_local, int d_model, int inter, int grid_ctas, bool backward,
                        int* tiles_out, int max_tiles, int* lag_out) {
  if (e_local < 1 || e_local > kMoeMaxLocalExperts || d_model % 256 != 0 || inter % 256 != 0 || grid_ctas < 1) return -1;
  MoeTables* tb = new MoeTables();
  EpMoeArgs a{};
  a.world = 1;
  a.e_local = e_local;
  a.d_model = d_model;
  a.inter = inter;
  for (int el = 0; el < e_local; ++el) tb->rows[el] = rows[el];
  build_tile_order(a, tb, backward, /*pad=*/64, /*claim_ahead=*/kSchedAhead, grid_ctas);
  const int n = tb->tile0[tb->n_slots];
  if (lag_out != nullptr) *lag_out = tb->lag;
  for (int t = 0; t < n && t < max_tiles; ++t) {
    int el, phase, m, nn;
    if (backward) {
      const BwdTile ti = decode_bwd_tile(a, tb, t);
      el = ti.el; phase = ti.phase; m = ti.m; nn = ti.n;
    } else {
      const TileInfo ti = decode_tile(a, tb, t);
      el = ti.el; phase = ti.phase; m = ti.m; nn = ti.n;
    }
    tiles_out[4 * t] = el;
    tiles_out[4 * t + 1] = phase;
    tiles_out[4 * t + 2] = m;
    tiles_out[4 * t + 3] = nn;
  }
  delete tb;
  return n;
}

cudaError_t moe_profile_read(int which, long long* host_out) {
  if (which < 0 || which > 1) return cudaErrorInvalidValue;
  return cudaMemcpyFromSymbol(host_out, g_moe_prof, sizeof(long long) * kMoeProfCtas * kMoeProfFields,
                              sizeof(long long) * which * kMoeProfCtas * kMoeProfFields, cudaMemcpyDeviceToHost);
}

cudaError_t launch_moe_prepare(const int* idx, int n_pairs, int n_experts, int* counts, int* pos, cudaStream_t st) {
  cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int) * n_experts, st);
  if (e != cudaSuccess) return e;
  const int grid = (n_pairs + 255) / 256 < 1184 ? (n_pairs + 255) / 256 : 1184;
  moe_prepare_kernel<<<grid > 0 ? grid : 1, 256, 0, st>>>(idx, n_pairs, counts, pos);
  return cudaGetLastError();
}

cudaError_t launch_ep_moe_forward(const EpMoeArgs& args, const __nv_bfloat16* gate, const __nv_bfloat16* up,
                                  const __nv_bfloat16* down, cudaStream_t st) {
  const EpMoeArgs& a = args;
  if (a.world < 1 || a.world > kCommMaxRanks || a.e_local < 1 || a.e_local > kMoeMaxLocalExperts ||
      a.world * a.e_local > kMoeMaxExperts || a.d_model % 256 != 0 || a.inter % 128 != 0 || a.cap_rows % BM != 0 ||
      static_cast<int64_t>(a.tokens) * a.top_k >= (1 << 24))
    return cudaErrorInvalidValue;
  CUtensorMap t_recv, t_act, t_gate, t_up, t_down;
  cudaError_t e;
  if ((e = encode_tma_2d(&t_recv, a.peer_recv_x[a.rank], 2, a.d_model, a.cap_rows, a.d_model * 2ull, 64, BM)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&t_act, a.act, 2, a.inter, a.cap_rows, a.inter * 2ull, 64, BM)) != cudaSuccess) return e;
  const uint64_t gate_rows = static_cast<uint64_t>(a.e_local) * a.d_model, down_rows = static_cast<uint64_t>(a.e_local) * a.inter;
  if ((e = encode_tma_2d(&t_gate, gate, 2, a.inter, gate_rows, a.inter * 2ull, 64, 64)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&t_up, up, 2, a.inter, gate_rows, a.inter * 2ull, 64, 64)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&t_down, down, 2, a.d_model, down_rows, a.d_model * 2ull, 64, 64)) != cudaSuccess) return e;
  static bool configured = false;
  if (!configured) {
    if ((e = cudaFuncSetAttribute(ep_moe_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes)) != cudaSuccess)
      return e;
    configured = true;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  EpMoeArgs args_copy = args;
  args_copy.prof = moe_prof_buffer(0);
  void* params[] = {&t_recv, &t_act, &t_gate, &t_up, &t_down, &args_copy};
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(ep_moe_forward_kernel), dim3(sms), dim3(kThreads), params,
                                     kSmemBytes, st);
}

cudaError_t launch_ep_moe_backward(const EpMoeArgs& args, const __nv_bfloat16* gate, const __nv_bfloat16* up,
                                   const __nv_bfloat16* down, cudaStream_t st) {
  const EpMoeArgs& a = args;
  if (a.world < 1 || a.world > kCommMaxRanks || a.e_local < 1 || a.e_local > kMoeMaxLocalExperts ||
      a.world * a.e_local > kMoeMaxExperts || a.d_model % 256 != 0 || a.inter % 256 != 0 || a.cap_rows % BM != 0 ||
      static_cast<int64_t>(a.tokens) * a.top_k >= (1 << 24) || a.gu == nullptr || a.dgu == nullptr)
    return cudaErrorInvalidValue;
  BwdMaps tm;
  cudaError_t e;
  const uint64_t cap = a.cap_rows, D = a.d_model, I = a.inter, EL = a.e_local;
  if ((e = encode_tma_2d(&tm.dy_k, a.peer_recv_dy[a.rank], 2, D, cap, D * 2, 64, BM)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tm.dgu_k, a.dgu, 2, 2 * I, cap, 2 * I * 2, 64, BM)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tm.down_k, down, 2, D, EL * I, D * 2, 64, BN)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tm.gate_k, gate, 2, I, EL * D, I * 2, 64, BN)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tm.up_k, up, 2, I, EL * D, I * 2, 64, BN)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tm.act_mn, a.act, 2, I, cap, I * 2, 64, 64)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tm.dy_mn, a.peer_recv_dy[a.rank], 2, D, cap, D * 2, 64, 64)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tm.x_mn, a.peer_recv_x[a.rank], 2, D, cap, D * 2, 64, 64)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tm.dgu_mn, a.dgu, 2, 2 * I, cap, 2 * I * 2, 64, 64)) != cudaSuccess) return e;
  static bool configured = false;
  if (!configured) {
    if ((e = cudaFuncSetAttribute(ep_moe_backward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes)) != cudaSuccess)
      return e;
    configured = true;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  EpMoeArgs args_copy = args;
  args_copy.prof = moe_prof_buffer(1);
  void* params[] = {&tm, &args_copy};
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(ep_moe_backward_kernel), dim3(sms), dim3(kThreads), params,
                                     kSmemBytes, st);
}

}  // namespace b200
