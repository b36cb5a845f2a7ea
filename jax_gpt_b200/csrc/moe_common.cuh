// Pieces shared by the expert-parallel MoE kernels (moe_kernels.cu, moe_fp8_kernels.cu): the
// shared-memory routing tables built from the all-gathered pair counts, the static tile order,
// bounded counter waits and the release/acquire helpers of the arrival protocol.
#pragma once
#include "common.cuh"
#include "moe_kernels.cuh"

namespace b200 {

namespace {

constexpr int kMoeBM = 128, kMoeBN = 256;

struct MoeTables {
  int send_off[kMoeMaxExperts];      // first row of MY pairs for global expert e in its destination buffer
  int rows[kMoeMaxLocalExperts];     // rows received per local expert
  int base[kMoeMaxLocalExperts];     // first row of the local expert in this rank's receive buffer
  // Static tile order, cut into n_slots = EL + lag slots; tile0[s] is the first tile of slot s. Forward: slot s
  // holds the GEMM1 (gate|up) tiles of expert s followed by the GEMM2 (down) tiles of expert s - lag. Backward:
  // slot s holds the dAct and dW_down tiles of expert s followed by the dX and dW_gate|up tiles of expert s - lag
  // (the ones that wait for that expert's dAct tiles). The lag keeps about two rounds of tiles between producer
  // and consumer tiles, so that CTAs working side by side in the order do not stall on one another.
  int tile0[2 * kMoeMaxLocalExperts + 1];
  int lag, n_slots;
  int mt0[kMoeMaxLocalExperts + 1];    // first m-tile index of the local expert
  int overflow;                      // some rank would receive more rows than cap_rows
};


__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add_u32(unsigned* p, unsigned v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_relaxed_sys_add_u32(unsigned* p, unsigned v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait until *p (cumulative counter) has reached `target` (wrap-safe signed difference).
template <bool kSystem>
__device__ __forceinline__ bool wait_counter_ge(const unsigned* p, unsigned target, uint64_t budget_ns,
                                                volatile int* abort_flag) {
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    const unsigned v = kSystem ? ld_acquire_sys_u32(p) : ld_acquire_gpu_u32(p);
    if (static_cast<int>(v - target) >= 0) return true;
    if (*abort_flag) return false;
    if (globaltimer_ns() - t0 > budget_ns) {
      *abort_flag = 1;
      return false;
    }
    __nanosleep(32);
  }
}


// From tb->rows: the regions of the local experts in the receive buffer (base), their m-tile numbering (mt0) and the
// static tile order (lag, n_slots, tile0). One thread; also compiled for the host, where the tests walk the order.
template <class Args>
__host__ __device__ inline void build_tile_order(const Args& a, MoeTables* tb, bool backward, int pad, int claim_ahead,
                                                 int grid_ctas) {
  const int EL = a.e_local;
  const int n1 = a.inter / 128, n2 = a.d_model / kMoeBN;
  // Cost of a tile in 64-deep K blocks, plus a few blocks' worth of epilogue: the tiles other tiles wait for
  // (GEMM1 / dAct, full-depth K) take longer than the average tile, and the lag has to cover their duration.
  const float c_over = 6.f;
  const float c_prod = a.d_model / 64 + c_over + (backward ? 4.f : 0.f);
  float cost = 0.f;
  int b = 0, t = 0, m = 0;
  for (int el = 0; el < EL; ++el) {
    tb->base[el] = b;
    tb->mt0[el] = m;
    const int mt = (tb->rows[el] + kMoeBM - 1) / kMoeBM;
    const int padded = (tb->rows[el] + pad - 1) / pad * pad;
    b += padded;
    if (!backward) {
      t += mt * (n1 + n2);
      cost += mt * (n1 * c_prod + n2 * (a.inter / 64 + c_over));
    } else if (mt > 0) {
      // dAct tiles, dX tiles, dW_down tiles, dW_gate|up tiles
      const int q0 = mt * (a.inter / kMoeBN), q1 = mt * n2;
      const int q23 = (a.inter / kMoeBM) * n2 + (a.d_model / kMoeBM) * (2 * a.inter / kMoeBN);
      t += q0 + q1 + q23;
      cost += q0 * c_prod + q1 * (2 * a.inter / 64 + c_over) + q23 * (padded / 64 + c_over);
    }
    m += mt;
  }
  tb->mt0[EL] = m;
  // Lag in experts: while one producer tile runs, the grid claims about gridDim.x * (its cost / average cost)
  // tiles; three times that, plus the tiles the CTAs claim ahead of their load warps, at the average number
  // of tiles per expert.
  int lag = 1;
  if (t > 0) {
    const float lag_tiles = static_cast<float>(grid_ctas) * (3.f * c_prod * t / cost + claim_ahead);
    lag = static_cast<int>(lag_tiles * EL / t) + 1;
  }
  lag = lag < 1 ? 1 : (lag > EL ? EL : lag);
  const int n_slots = EL + lag;
  int u = 0;
  for (int sl = 0; sl < n_slots; ++sl) {
    tb->tile0[sl] = u;
    if (sl < EL) {
      const int mt = (tb->rows[sl] + kMoeBM - 1) / kMoeBM;
      if (!backward) u += mt * n1;
      else if (mt > 0) u += mt * (a.inter / kMoeBN) + (a.inter / kMoeBM) * n2;
    }
    if (sl >= lag) {
      const int mt = (tb->rows[sl - lag] + kMoeBM - 1) / kMoeBM;
      if (!backward) u += mt * n2;
      else if (mt > 0) u += mt * n2 + (a.d_model / kMoeBM) * (2 * a.inter / kMoeBN);
    }
  }
  tb->tile0[n_slots] = u;
  tb->lag = lag;
  tb->n_slots = n_slots;
}

// Fills the shared-memory tables from the all-gathered count matrix counts[src][e].
template <class Args>
__device__ void build_tables(const Args& a, const int* counts_all, MoeTables* tb, bool backward = false, int pad = 64,
                             int claim_ahead = 0) {
  const int W = a.world, EL = a.e_local, ET = W * EL;
  if (threadIdx.x == 0) tb->overflow = 0;
  __syncthreads();
  // Three passes, linear in the number of experts: padded totals per global expert (every expert's region starts
  // on a `pad`-row boundary; ragged-K weight gradients read whole blocks and the padding rows are kept zero), an
  // exclusive scan inside every destination rank's segment (one thread per destination), then the rows of the
  // sources placed before this rank.
  for (int e = threadIdx.x; e < ET; e += blockDim.x) {
    int n = 0;
    for (int s = 0; s < W; ++s) n += __ldcg(counts_all + s * ET + e);
    tb->send_off[e] = (n + pad - 1) / pad * pad;
  }
  __syncthreads();
  if (threadIdx.x < W) {
    int run = 0;
    for (int e = threadIdx.x * EL; e < (threadIdx.x + 1) * EL; ++e) {
      const int v = tb->send_off[e];
      tb->send_off[e] = run;
      run += v;
    }
    if (run > a.cap_rows) tb->overflow = 1;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < ET; e += blockDim.x) {
    int before = 0;
    for (int s = 0; s < a.rank; ++s) before += __ldcg(counts_all + s * ET + e);
    tb->send_off[e] += before;
  }
  for (int el = threadIdx.x; el < EL; el += blockDim.x) {
    int n = 0;
    for (int s = 0; s < W; ++s) n += __ldcg(counts_all + s * ET + a.rank * EL + el);
    tb->rows[el] = n;
  }
  __syncthreads();
  if (threadIdx.x == 0) build_tile_order(a, tb, backward, pad, claim_ahead, static_cast<int>(gridDim.x));
  __syncthreads();
}

struct TileInfo {
  int el, m, n, phase;  // phase 0: GEMM1 (gate|up), 1: GEMM2 (down)
};

template <class Args>
__host__ __device__ __forceinline__ TileInfo decode_tile(const Args& a, const MoeTables* tb, int t) {
  const int n1 = a.inter / 128, n2 = a.d_model / kMoeBN;
  // first slot whose tile range ends after t (slots without tiles have empty ranges): binary search
  int sl = 0, hi = tb->n_slots - 1;
  while (sl < hi) {
    const int mid = (sl + hi) >> 1;
    if (tb->tile0[mid + 1] > t) hi = mid;
    else sl = mid + 1;
  }
  int r = t - tb->tile0[sl];
  const int g1 = (sl < a.e_local) ? ((tb->rows[sl] + kMoeBM - 1) / kMoeBM) * n1 : 0;
  TileInfo ti;
  if (r < g1) {
    const int mt = (tb->rows[sl] + kMoeBM - 1) / kMoeBM;
    ti.el = sl;
    ti.phase = 0;
    ti.m = r % mt;
    ti.n = r / mt;
  } else {
    r -= g1;
    ti.el = sl - tb->lag;
    const int mt = (tb->rows[ti.el] + kMoeBM - 1) / kMoeBM;
    ti.phase = 1;
    ti.m = r % mt;
    ti.n = r / mt;
  }
  return ti;
}


}  // namespace

}  // namespace b200
