// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   warp 0      : TMA producer  (cp.async.bulk.tensor tiles -> 128B-swizzled shared memory)
//   warp 1      : MMA issuer    (one lane issues tcgen05.mma, accumulators live in TMEM)
//   warps 2..9  : epilogue      (tcgen05.ld -> registers -> fused bias / GELU / residual ->
//                                global, or fp32 atomics into local or peer buffers)
//
// The tile is 128 x BN x 64 with a multi-stage shared-memory ring and two TMEM
// accumulators, so the epilogue of tile i overlaps the main loop of tile i+1. Both
// operands may be K-major or MN-major, which covers forward (x @ W), dgrad (dy @ W^T)
// and wgrad (x^T @ dy) without transposing anything in memory.
//
// Takes the place of the XLA dot lowering the reference relies on for every linear layer
// (jax_gpt/models/gpt2/model.py:95-102,145,180 and jax_gpt/models/qwen35/fp8.py:137-150).
#include "gemm_sm100.cuh"

#include <cstdlib>
#include <mutex>

#include "comm_device.cuh"
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "tma_host.h"

namespace b200 {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kNumThreads = 320;   // TMA warp, MMA warp, 8 epilogue warps (two per TMEM lane quarter)

struct TmaSet {
  CUtensorMap m[kMaxPeers];
};

struct GatherInfo {
  int n_src;           // number of A sources (1 = plain GEMM)
  int blocks_per_src;  // M-blocks per source
  int first_src;       // source visited first
  // B (an MN-major weight [K, N]) split by COLUMNS across b_n_src sources of b_nb_per_src n-blocks each (FSDP
  // parameter shards, each stored as its own [K, N / b_n_src] matrix): the tiles of source b_first_src (the
  // local shard) are visited first, then the next source's, so compute overlaps the arrival of the others.
  int b_n_src;
  int b_nb_per_src;
  int b_first_src;
};

template <int BN>
struct Cfg {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kTmemCols = 2 * BN;  // two accumulators
  static constexpr int kEpiBytes = 8 * kEpiStageBytesPerWarp;  // store staging of the eight epilogue warps
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 /*align*/ + 256 /*barriers*/ + 256 /*seen*/;
};

struct Barriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(Barriers) <= 256, "barrier block");
constexpr int kMaxStageUnits = 2048;     // bits of the producer's "unit seen ready" mask (256 bytes behind the barriers)

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void bulk_store_1d(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Copier CTA of the staged gather, bulk-copy half (one thread works): for its share of the (peer, unit) pairs it
// streams the unit local -> shared-memory ring -> peer memory with bulk copies (up to kLag chunks of loads in
// flight) and publishes the unit in the peer's `ready` array once its stores have completed. Every wait is bounded;
// on expiry the status word is set, loads in flight are given time to land, and the thread returns.
__device__ void stage_copier(const StageCopy& sc, uint8_t* ring, int ring_bytes, Barriers* bars, int* status, int idx,
                             int n_workers) {
  constexpr int kSlots = 8, kLag = 6;     // kSlots == the number of `full` barriers the kernel initialises
  const uint32_t slot_bytes = static_cast<uint32_t>((ring_bytes / kSlots) & ~1023);
  volatile int* abort_flag = &bars->abort_flag;
  uint8_t* pend_dst[kSlots] = {};
  uint32_t pend_n[kSlots] = {};
  int issued = 0, stored = 0;
  bool ok = true;
  auto store_one = [&]() {
    const int slot = stored % kSlots;
    if (!mbar_wait(&bars->full[slot], (stored / kSlots) & 1, abort_flag)) {
      report_status(status, kWaitFullTimeout, 1000 + idx, stored, issued);
      ok = false;
      return;
    }
    bulk_store_1d(pend_dst[slot], ring + slot * slot_bytes, pend_n[slot]);
    bulk_commit();
    ++stored;
  };
  const int n_units = sc.n_remote * sc.units_per_src;
  for (int u = idx; u < n_units && ok; u += n_workers) {
    // peer-major: the whole shard goes to the peer that needs it first (the rank before this one, whose compute
    // CTAs visit this rank's rows right after their own), then to the one before that, and so on: every consumer
    // receives from one source at a time, in the order in which it consumes
    const int j = u / sc.units_per_src, i = u % sc.units_per_src;
    const unsigned char* src = sc.src + static_cast<long long>(i) * sc.bytes_per_unit;
    unsigned char* dst = sc.dst[j] + static_cast<long long>(i) * sc.bytes_per_unit;
    for (long long off = 0; off < sc.bytes_per_unit && ok; off += slot_bytes) {
      const long long left = sc.bytes_per_unit - off;
      const uint32_t n = left < slot_bytes ? static_cast<uint32_t>(left) : slot_bytes;
      const int slot = issued % kSlots;
      if (issued >= kSlots) bulk_wait_read<kSlots - kLag - 1>();   // the store that last used this slot has read it
      mbar_arrive_expect_tx(&bars->full[slot], n);
      bulk_load_1d(ring + slot * slot_bytes, src + off, n, &bars->full[slot]);
      pend_dst[slot] = dst + off;
      pend_n[slot] = n;
      ++issued;
      if (issued - stored > kLag) store_one();
    }
    while (ok && stored < issued) store_one();
    if (!ok) break;
    bulk_wait_all();             // the unit's stores have completed
    fence_proxy_async_all();
    __threadfence_system();
    st_release_sys(sc.peer_ready[j] + sc.my_unit0 + i, sc.epoch);
  }
  if (!ok) {
    *abort_flag = 1;
    for (int c = stored; c < issued; ++c) {       // loads still in flight: bounded time to land before the CTA exits
      const uint64_t t0 = globaltimer_ns();
      while (!mbar_try_wait(&bars->full[c % kSlots], (c / kSlots) & 1)) {
        if (globaltimer_ns() - t0 > 2000000ull) break;
      }
    }
  }
  bulk_wait_all();
}

// The other copier of a copier CTA: warps 1..9 push their (peer, unit) pairs with ordinary 16-byte loads (local) and
// stores (peer), eight in flight per thread; a named barrier (id 1) joins the 288 threads before thread 32 publishes
// the unit in the peer's `ready` array.
__device__ void stage_copier_ldst(const StageCopy& sc, int idx, int n_workers) {
  constexpr int kThreadsLs = kNumThreads - 32;
  const int t = threadIdx.x - 32;
  const int n_units = sc.n_remote * sc.units_per_src;
  const long long n16 = sc.bytes_per_unit / 16;
  for (int u = idx; u < n_units; u += n_workers) {
    const int j = u / sc.units_per_src, i = u % sc.units_per_src;
    const uint4* src = reinterpret_cast<const uint4*>(sc.src + static_cast<long long>(i) * sc.bytes_per_unit);
    uint4* dst = reinterpret_cast<uint4*>(sc.dst[j] + static_cast<long long>(i) * sc.bytes_per_unit);
    long long k = t;
    for (; k + 7 * kThreadsLs < n16; k += 8 * kThreadsLs) {
      uint4 v[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] = __ldg(src + k + q * kThreadsLs);
#pragma unroll
      for (int q = 0; q < 8; ++q) dst[k + q * kThreadsLs] = v[q];
    }
    for (; k < n16; k += kThreadsLs) dst[k] = __ldg(src + k);
    __threadfence_system();
    asm volatile("bar.sync 1, %0;" ::"n"(kThreadsLs) : "memory");
    if (t == 0) st_release_sys(sc.peer_ready[j] + sc.my_unit0 + i, sc.epoch);
  }
}

template <int BN, int A_MAJOR, int B_MAJOR>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_bf16_kernel(const __grid_constant__ TmaSet tma_a, const __grid_constant__ TmaSet tma_b,
                 const __grid_constant__ GemmArgs args, const __grid_constant__ GatherInfo gi,
                 const __grid_constant__ StageCopy sc) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  // 128B swizzle needs the tile bases on 1024-byte boundaries.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = smem + C::kStages * C::kStageBytes;
  Barriers* bars = reinterpret_cast<Barriers*>(epi_stage + C::kEpiBytes);
  uint32_t* seen_bits = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(bars) + 256);   // producer thread only
  volatile int* abort_flag = &bars->abort_flag;
  // staged gather: the last sc.n_copy_ctas CTAs of the grid copy, the others compute and wait for them unit by unit
  const int gemm_ctas = static_cast<int>(gridDim.x) - sc.n_copy_ctas;
  const bool is_copier = static_cast<int>(blockIdx.x) >= gemm_ctas;
  const uint64_t wait_budget = sc.n_copy_ctas > 0 ? sc.wait_ns + kWaitBudgetNs : kWaitBudgetNs;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int m_blocks = (args.M + BM - 1) / BM;
  const int n_blocks = (args.N + BN - 1) / BN;
  const int split_k = args.split_k < 1 ? 1 : args.split_k;
  const int total_kb = (args.K + BK - 1) / BK;
  const int kb_per_split = (total_kb + split_k - 1) / split_k;
  const int num_tiles = m_blocks * n_blocks * split_k;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 8; ++s) {        // all eight: a copier CTA uses every `full` barrier for its ring of eight slots
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], 8);
    }
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (is_copier) {
    __syncthreads();
    // two copiers per copier CTA: thread 0 drives the bulk-copy ring, warps 1..9 copy with loads and stores
    const int cidx = static_cast<int>(blockIdx.x) - gemm_ctas;
    if (threadIdx.x == 0)
      stage_copier(sc, smem, C::kStages * C::kStageBytes, bars, args.status, 2 * cidx, 2 * sc.n_copy_ctas);
    else if (threadIdx.x >= 32)
      stage_copier_ldst(sc, 2 * cidx + 1, 2 * sc.n_copy_ctas);
    return;
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  // Maps a linear tile index to (m block, n block, k split). Consecutive tiles share the
  // B tile so the CTAs running together re-use it out of L2. With gathered A the m blocks
  // are rotated so that the locally resident rows come first.
  auto decode_tile = [&](int t, int& m_blk, int& n_blk, int& ks) {
    ks = t % split_k;
    int mn = t / split_k;
    if (gi.n_src > 1) {
      // source-major: every tile of the local rows first (all n blocks), then the next source's, so that the
      // remote rows are needed as late as possible; inside a source consecutive tiles share the B tile
      const int per_src = gi.blocks_per_src * n_blocks;
      const int si = mn / per_src, r = mn - si * per_src;
      n_blk = r / gi.blocks_per_src;
      m_blk = ((gi.first_src + si) % gi.n_src) * gi.blocks_per_src + r % gi.blocks_per_src;
      return;
    }
    if (gi.b_n_src > 1) {
      // weight-shard-major: all tiles of the local column shard first; inside a shard consecutive tiles share B
      const int per_src = gi.b_nb_per_src * m_blocks;
      const int si = mn / per_src, r = mn - si * per_src;
      m_blk = r % m_blocks;
      n_blk = ((gi.b_first_src + si) % gi.b_n_src) * gi.b_nb_per_src + r / m_blocks;
      return;
    }
    if (args.out_mode == kOutBf16PeerPush) {
      // owner-major, the rank after this one first and this rank's own rows last: what has to cross NVLink
      // leaves early, and the reduction phase of every owner finds its remote partials complete sooner
      const int bpp = args.rows_per_peer / BM, per_peer = bpp * n_blocks;
      const int pi = mn / per_peer, r = mn - pi * per_peer;
      n_blk = r / bpp;
      m_blk = ((args.self_rank + 1 + pi) % args.n_peers) * bpp + r % bpp;
      return;
    }
    // bands of 16 m-blocks: one wave of CTAs then touches ~16 x 9 tiles instead of a whole column of A
    constexpr int kBand = 16;
    const int per_band = kBand * n_blocks;
    const int band = mn / per_band, r = mn - band * per_band;
    const int rows = min(kBand, m_blocks - band * kBand);
    m_blk = band * kBand + r % rows;
    n_blk = r / rows;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tma_b.m[0]);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      if (sc.n_copy_ctas > 0)
        for (int i = 0; i < kMaxStageUnits / 32; ++i) seen_bits[i] = 0u;
      // staged gather: has the copier published this unit? (cached per CTA; a bounded poll otherwise)
      auto unit_ready = [&](int unit) -> bool {
        if (seen_bits[unit >> 5] & (1u << (unit & 31))) return true;
        const uint64_t t0 = globaltimer_ns();
        while (ld_acquire_sys(sc.ready + unit) < sc.epoch) {      // written by the peer that pushed the unit
          if (*abort_flag || globaltimer_ns() - t0 > sc.wait_ns) return false;
          __nanosleep(100);
        }
        fence_proxy_async_all();     // the TMA reads below must observe the peer's stores
        seen_bits[unit >> 5] |= 1u << (unit & 31);
        return true;
      };
      for (int t = blockIdx.x; t < num_tiles && ok; t += gemm_ctas) {
        int m_blk, n_blk, ks;
        decode_tile(t, m_blk, n_blk, ks);
        const int src = (gi.n_src > 1) ? (m_blk / gi.blocks_per_src) : 0;
        if (sc.mode == 1 && sc.n_copy_ctas > 0 && src != gi.first_src && !unit_ready(m_blk)) {
          report_status(args.status, kWaitFlagTimeout, 2000 + blockIdx.x, t, m_blk);
          *abort_flag = 1;
          ok = false;
          break;
        }
        const int m0 = (gi.n_src > 1) ? (m_blk % gi.blocks_per_src) * BM : m_blk * BM;
        // column-sharded B: the tile's columns live in source b_src's own [K, N / b_n_src] matrix
        const int b_src = (gi.b_n_src > 1) ? n_blk / gi.b_nb_per_src : 0;
        const int n0 = (gi.b_n_src > 1) ? (n_blk % gi.b_nb_per_src) * BN : n_blk * BN;
        const CUtensorMap* tbp = &tma_b.m[b_src];
        if (sc.mode == 2 && b_src != gi.b_first_src) {
          // the whole shard of that source must have landed (its units are K-row blocks); cached per unit
          bool all = true;
          for (int i = 0; i < sc.units_per_src && all; ++i) all = unit_ready(b_src * sc.units_per_src + i);
          if (!all) {
            report_status(args.status, kWaitFlagTimeout, 3000 + blockIdx.x, t, b_src);
            *abort_flag = 1;
            ok = false;
            break;
          }
        }
        const CUtensorMap* ta = &tma_a.m[src];
        const int kb0 = ks * kb_per_split;
        const int kb1 = min(total_kb, kb0 + kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag, wait_budget)) {
            report_status(args.status, kWaitEmptyTimeout, blockIdx.x, t, kb);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * C::kStageBytes;
          uint8_t* sb = sa + C::kABytes;
          mbar_arrive_expect_tx(&bars->full[stage], C::kStageBytes);
          const int k0 = kb * BK;
          const int kb_row = k0;
          if (A_MAJOR == 0) {
            tma_load_2d(sa, ta, &bars->full[stage], k0, m0);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d(sa + i * 8192, ta, &bars->full[stage], m0 + 64 * i, k0);
          }
          if (B_MAJOR == 0) {
            tma_load_2d(sb, tbp, &bars->full[stage], k0, n0);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_2d(sb + i * 8192, tbp, &bars->full[stage], n0 + 64 * i, kb_row);
          }
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok || *abort_flag) {
        // Unwinding: give copies that are still in flight a bounded time to land so that
        // nothing writes into this CTA's shared memory after it has exited.
        // Stages below `stage` were last armed in the current lap, the others one lap earlier.
        for (int s = 0; s < C::kStages; ++s) {
          const uint32_t armed_parity = (s < stage) ? phase : (phase ^ 1);
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&bars->full[s], armed_parity)) {
            if (globaltimer_ns() - t0 > 2000000ull) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    constexpr uint32_t idesc = make_idesc(BM, BN, A_MAJOR, B_MAJOR, /*bf16*/ 1);
    int stage = 0;
    uint32_t phase = 0;
    int iter = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gemm_ctas, ++iter) {
      int m_blk, n_blk, ks;
      decode_tile(t, m_blk, n_blk, ks);
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      if (!mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1, abort_flag, wait_budget)) {
        if (lane == 0) report_status(args.status, kWaitTmemEmptyTimeout, blockIdx.x, t, iter);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + acc * BN;
      const int kb0 = ks * kb_per_split;
      const int kb1 = min(total_kb, kb0 + kb_per_split);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&bars->full[stage], phase, abort_flag, wait_budget)) {
          if (lane == 0) report_status(args.status, kWaitFullTimeout, blockIdx.x, t, kb);
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sa = smem_u32(smem + stage * C::kStageBytes);
          const uint32_t sb = sa + C::kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = (A_MAJOR == 0) ? make_smem_desc(sa + k * 32, 16, 1024)
                                                  : make_smem_desc(sa + k * 2048, 8192, 1024);
            const uint64_t bdesc = (B_MAJOR == 0) ? make_smem_desc(sb + k * 32, 16, 1024)
                                                  : make_smem_desc(sb + k * 2048, 8192, 1024);
            umma_bf16(tmem_d, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&bars->empty[stage]);  // frees the stage once these MMAs have read it
        }
        __syncwarp();
        if (++stage == C::kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok && lane == 0) tc_commit(&bars->tmem_full[acc]);
      __syncwarp();
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;  // which half of the tile's columns this warp converts and stores
    int iter = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gemm_ctas, ++iter) {
      int m_blk, n_blk, ks;
      decode_tile(t, m_blk, n_blk, ks);
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      if (!mbar_wait(&bars->tmem_full[acc], acc_phase, abort_flag, wait_budget)) {
        if (lane == 0) report_status(args.status, kWaitTmemFullTimeout, blockIdx.x, t, iter);
        ok = false;
        break;
      }
      tc_fence_after();
      // Empty K range (possible only for trailing splits): nothing was accumulated.
      const bool has_k = ks * kb_per_split < total_kb;
      gemm_epilogue_columns(args, tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16),
                            epi_stage + (warp - 2) * kEpiStageBytesPerWarp, m_blk * BM + q * 32, n_blk * BN,
                            half * (BN / 2), (half + 1) * (BN / 2), lane, ks, has_k);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty[acc]);
      if (args.out_mode == kOutBf16PeerPush && lane == 0) {
        // this warp's part of the tile is stored (the __syncwarp above orders the other lanes' stores before
        // this release): one arrival on the owner's counter of the 128-row block
        const int peer = (m_blk * BM) / args.rows_per_peer;
        int* cnt = args.peer_cnt[peer] + (m_blk - peer * (args.rows_per_peer / BM));
        // counted in 64-column groups, so that the total does not depend on the tile width the launcher picked
        const int c_lo = n_blk * BN + half * (BN / 2), c_hi = min(args.N, c_lo + BN / 2);
        __threadfence_system();
        if (c_hi > c_lo)
          asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(cnt), "r"((c_hi - c_lo) / 64) : "memory");
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
  if (args.out_mode == kOutBf16PeerPush) {
    // second phase of GEMM -> reduce-scatter: sum the n_peers bf16 partials of this rank's rows. A unit is one
    // 128-row block x 1024 columns; its block must be complete (every source, every n block, every epilogue warp).
    // Nothing in the first phase waits for another rank, so these waits cannot be part of a cycle.
    __shared__ int s_ok;
    const int bpp = args.rows_per_peer / BM;
    const int col_units = (args.N + 1023) / 1024;
    const __nv_bfloat16* recv = reinterpret_cast<const __nv_bfloat16*>(args.peer_out[args.self_rank]);
    const int64_t slot = static_cast<int64_t>(args.rows_per_peer) * args.ldo;
    for (int u = blockIdx.x; u < bpp * col_units; u += gemm_ctas) {
      const int mb = u / col_units, c0 = (u % col_units) * 1024;
      if (threadIdx.x == 0) {
        s_ok = wait_flag_ge(args.peer_cnt[args.self_rank] + mb, args.cnt_expected, args.rs_wait_ns) ? 1 : 0;
        if (!s_ok) report_status(args.status, kWaitFlagTimeout, 4000 + blockIdx.x, mb, args.cnt_expected);
      }
      __syncthreads();
      const bool ok = s_ok != 0;
      __syncthreads();
      if (!ok) break;
      const int cols8 = (min(args.N, c0 + 1024) - c0) / 8;
      for (int it = threadIdx.x; it < BM * cols8; it += kNumThreads) {
        const int r = mb * BM + it / cols8, c = c0 + (it % cols8) * 8;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int sidx = 0; sidx < args.n_peers; ++sidx) {
          const uint4 pk = *reinterpret_cast<const uint4*>(recv + sidx * slot + static_cast<int64_t>(r) * args.ldo + c);
          const float2 a0 = unpack_bf16x2(pk.x), a1 = unpack_bf16x2(pk.y), a2 = unpack_bf16x2(pk.z), a3 = unpack_bf16x2(pk.w);
          acc[0] += a0.x; acc[1] += a0.y; acc[2] += a1.x; acc[3] += a1.y;
          acc[4] += a2.x; acc[5] += a2.y; acc[6] += a3.x; acc[7] += a3.y;
        }
        *reinterpret_cast<uint4*>(args.rs_out + static_cast<int64_t>(r) * args.ldo + c) =
            make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                       pack_bf16x2(acc[6], acc[7]));
      }
    }
  }
}

template <int BN, int A_MAJOR, int B_MAJOR>
cudaError_t launch_variant(const TmaSet& ta, const TmaSet& tb, const GemmArgs& args, const GatherInfo& gi,
                           const StageCopy& sc, cudaStream_t stream) {
  using C = Cfg<BN>;
  auto kernel = gemm_bf16_kernel<BN, A_MAJOR, B_MAJOR>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const int m_blocks = (args.M + BM - 1) / BM;
  const int n_blocks = (args.N + BN - 1) / BN;
  const int tiles = m_blocks * n_blocks * (args.split_k < 1 ? 1 : args.split_k);
  // copier CTAs must be resident together with the compute CTAs that wait for them: the grid never exceeds the
  // SM count (one CTA per SM by shared memory)
  const int room = gemm_sm_count() - sc.n_copy_ctas;
  if (room < 1) return cudaErrorInvalidValue;
  const int grid = (tiles < room ? tiles : room) + sc.n_copy_ctas;
  kernel<<<grid, kNumThreads, C::kSmemBytes, stream>>>(ta, tb, args, gi, sc);
  return cudaGetLastError();
}

cudaError_t make_operand_map(CUtensorMap* map, const __nv_bfloat16* p, int64_t ld, int major, int rows_mn, int K,
                             int box_mn) {
  // K-major: stored [rows_mn, K], box {64 (k), box_mn}. MN-major: stored [K, rows_mn], box {64 (mn), 64 (k)}.
  if (major == 0) return encode_tma_2d(map, p, /*elem*/ 2, /*inner*/ K, /*outer*/ rows_mn, ld * 2, 64, box_mn);
  return encode_tma_2d(map, p, 2, rows_mn, K, ld * 2, 64, 64);
}

cudaError_t launch_common(const __nv_bfloat16* const* a_src, int n_src, int rows_per_src, int first_src, int64_t lda,
                          int a_major, const __nv_bfloat16* B, int64_t ldb, int b_major, const GemmArgs& args_in,
                          cudaStream_t stream, const __nv_bfloat16* const* b_src = nullptr, int b_n_src = 1,
                          int b_first_src = 0, const StageCopy* stage_copy = nullptr) {
  GemmArgs args = args_in;
  if (args.M <= 0 || args.N <= 0 || args.K <= 0) return cudaErrorInvalidValue;
  if (n_src < 1 || n_src > kMaxPeers) return cudaErrorInvalidValue;
  if (n_src > 1 && (rows_per_src % BM != 0 || rows_per_src * n_src != args.M)) return cudaErrorInvalidValue;
  if (args.split_k > 1 && args.out_mode != kOutF32Atomic && args.out_mode != kOutBf16PeerRed)
    return cudaErrorInvalidValue;
  if (args.out_mode == kOutBf16PeerPush &&
      (args.n_peers < 1 || args.n_peers > kMaxPeers || args.rows_per_peer % BM != 0 ||
       args.rows_per_peer * args.n_peers != args.M || args.N % 64 != 0 || (args.ldo & 7) != 0 || args.split_k > 1 ||
       args.rs_out == nullptr))
    return cudaErrorInvalidValue;
  if (args.alpha == 0.f) args.alpha = 1.f;
  // Narrow outputs get the 128-wide tile so that more CTAs have work.
  const int m_blocks = (args.M + BM - 1) / BM;
  const bool wide = (args.N >= 256) && (m_blocks * ((args.N + 255) / 256) * (args.split_k < 1 ? 1 : args.split_k) >=
                                        gemm_sm_count());
  int BN = wide ? 256 : 128;
  if (b_n_src > 1 && (args.N / b_n_src) % BN != 0) BN = 128;     // a tile must not straddle two weight shards

  TmaSet ta;
  for (int s = 0; s < n_src; ++s) {
    cudaError_t e = make_operand_map(&ta.m[s], a_src[s], lda, a_major, n_src > 1 ? rows_per_src : args.M, args.K, BM);
    if (e != cudaSuccess) return e;
  }
  for (int s = n_src; s < kMaxPeers; ++s) ta.m[s] = ta.m[0];
  TmaSet tb;
  cudaError_t e;
  int b_nb_per_src = 0;
  if (b_n_src > 1) {
    // column-sharded MN-major B: source s holds columns [s * N / b_n_src, (s + 1) * N / b_n_src) as a [K, N / b_n_src]
    // matrix of its own (row stride ldb = N / b_n_src)
    if (b_major != 1 || b_n_src > kMaxPeers || args.N % (b_n_src * BN) != 0 || args.split_k > 1) return cudaErrorInvalidValue;
    const int n_per = args.N / b_n_src;
    b_nb_per_src = n_per / BN;
    for (int s = 0; s < b_n_src; ++s)
      if ((e = make_operand_map(&tb.m[s], b_src[s], ldb, 1, n_per, args.K, BN)) != cudaSuccess) return e;
    for (int s = b_n_src; s < kMaxPeers; ++s) tb.m[s] = tb.m[0];
  } else {
    if ((e = make_operand_map(&tb.m[0], B, ldb, b_major, args.N, args.K, BN)) != cudaSuccess) return e;
    for (int s = 1; s < kMaxPeers; ++s) tb.m[s] = tb.m[0];
  }
  GatherInfo gi{n_src, n_src > 1 ? rows_per_src / BM : 0, first_src, b_n_src, b_nb_per_src, b_first_src};
  StageCopy sc{};
  if (stage_copy != nullptr) sc = *stage_copy;

#define B200_GEMM_CASE(bn, am, bm) \
  if (BN == bn && a_major == am && b_major == bm) return launch_variant<bn, am, bm>(ta, tb, args, gi, sc, stream);
  B200_GEMM_CASE(256, 0, 0)
  B200_GEMM_CASE(256, 0, 1)
  B200_GEMM_CASE(256, 1, 0)
  B200_GEMM_CASE(256, 1, 1)
  B200_GEMM_CASE(128, 0, 0)
  B200_GEMM_CASE(128, 0, 1)
  B200_GEMM_CASE(128, 1, 0)
  B200_GEMM_CASE(128, 1, 1)
#undef B200_GEMM_CASE
  return cudaErrorInvalidValue;
}

}  // namespace

int gemm_sm_count() {
  static int count = 0;
  if (count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
    if (count <= 0) count = 148;
  }
  return count;
}

cudaError_t launch_gemm_bf16(const __nv_bfloat16* A, int64_t lda, int a_major, const __nv_bfloat16* B, int64_t ldb,
                             int b_major, const GemmArgs& args, cudaStream_t stream) {
  if (gemm_pair_wanted(args)) return launch_gemm_bf16_pair(A, lda, a_major, B, ldb, b_major, args, stream);
  const __nv_bfloat16* srcs[1] = {A};
  return launch_common(srcs, 1, 0, 0, lda, a_major, B, ldb, b_major, args, stream);
}

namespace {

// Common part of the two staged launchers.
void fill_stage_copy(StageCopy* sc, int n_src, int rank, int epoch, double wait_seconds, int* const* peer_ready) {
  sc->n_remote = n_src - 1;
  // a copier CTA pushes about 25 GB/s (bulk-copy ring + load/store warps); the shard goes to n_src - 1 peers while
  // the compute CTAs work through one rank's share of the tiles. Measured at 2 ranks: 8 copiers hide the gather.
  int copiers = n_src <= 2 ? 8 : (n_src <= 4 ? 16 : 24);
  if (const char* e = getenv("B200_STAGE_COPIERS")) copiers = atoi(e) > 0 && atoi(e) < 100 ? atoi(e) : copiers;
  sc->n_copy_ctas = n_src > 1 ? copiers : 0;
  sc->epoch = epoch;
  sc->wait_ns = static_cast<unsigned long long>((wait_seconds > 0 ? wait_seconds : 20.0) * 1e9);
  sc->ready = peer_ready[rank];
  for (int j = 0; j < n_src - 1; ++j) sc->peer_ready[j] = peer_ready[(rank + n_src - 1 - j) % n_src];   // see stage_copier
}

}  // namespace

cudaError_t launch_gemm_bf16_gathered_a_staged(__nv_bfloat16* const* peer_gather, int* const* peer_ready, int n_src,
                                               int rows_per_src, int rank, const __nv_bfloat16* B, int64_t ldb,
                                               int b_major, const GemmArgs& args, int epoch, double wait_seconds,
                                               cudaStream_t stream) {
  if (n_src < 1 || n_src > kMaxPeers || rank < 0 || rank >= n_src || rows_per_src % BM != 0) return cudaErrorInvalidValue;
  if (n_src * (rows_per_src / BM) > kMaxStageUnits) return cudaErrorInvalidValue;
  const int64_t K = args.K, slice = static_cast<int64_t>(rows_per_src) * K;
  const __nv_bfloat16* srcs[kMaxPeers];
  for (int s = 0; s < n_src; ++s) srcs[s] = peer_gather[rank] + s * slice;     // the LOCAL buffer, block by block
  StageCopy sc{};
  fill_stage_copy(&sc, n_src, rank, epoch, wait_seconds, peer_ready);
  sc.mode = 1;
  sc.units_per_src = rows_per_src / BM;
  sc.bytes_per_unit = static_cast<long long>(BM) * K * 2;
  sc.my_unit0 = rank * sc.units_per_src;
  sc.src = reinterpret_cast<const unsigned char*>(peer_gather[rank] + rank * slice);
  for (int j = 0; j < n_src - 1; ++j)
    sc.dst[j] = reinterpret_cast<unsigned char*>(peer_gather[(rank + n_src - 1 - j) % n_src] + rank * slice);
  return launch_common(srcs, n_src, rows_per_src, rank, K, 0, B, ldb, b_major, args, stream, nullptr, 1, 0, &sc);
}

cudaError_t launch_gemm_bf16_reduce_scatter_push(const __nv_bfloat16* A, int64_t lda, const __nv_bfloat16* B, int64_t ldb,
                                                 int b_major, const GemmArgs& args, cudaStream_t stream) {
  if (args.out_mode != kOutBf16PeerPush) return cudaErrorInvalidValue;
  const __nv_bfloat16* srcs[1] = {A};
  return launch_common(srcs, 1, 0, 0, lda, 0, B, ldb, b_major, args, stream);
}

cudaError_t launch_gemm_bf16_sharded_b_staged(const __nv_bfloat16* A, int64_t lda, __nv_bfloat16* const* peer_w,
                                              int* const* peer_ready, int n_src, int rank, const GemmArgs& args,
                                              int epoch, double wait_seconds, cudaStream_t stream) {
  if (n_src < 1 || n_src > kMaxPeers || rank < 0 || rank >= n_src || args.N % (n_src * 128) != 0 || args.K % BK != 0)
    return cudaErrorInvalidValue;
  if (n_src * (args.K / BK) > kMaxStageUnits) return cudaErrorInvalidValue;
  const int64_t n_per = args.N / n_src, shard = static_cast<int64_t>(args.K) * n_per;
  const __nv_bfloat16* b_srcs[kMaxPeers];
  for (int s = 0; s < n_src; ++s) b_srcs[s] = peer_w[rank] + s * shard;        // the LOCAL buffer, shard by shard
  StageCopy sc{};
  fill_stage_copy(&sc, n_src, rank, epoch, wait_seconds, peer_ready);
  sc.mode = 2;
  sc.units_per_src = args.K / BK;
  sc.bytes_per_unit = static_cast<long long>(BK) * n_per * 2;
  sc.my_unit0 = rank * sc.units_per_src;
  sc.src = reinterpret_cast<const unsigned char*>(peer_w[rank] + rank * shard);
  for (int j = 0; j < n_src - 1; ++j)
    sc.dst[j] = reinterpret_cast<unsigned char*>(peer_w[(rank + n_src - 1 - j) % n_src] + rank * shard);
  const __nv_bfloat16* srcs[1] = {A};
  return launch_common(srcs, 1, 0, 0, lda, 0, nullptr, n_per, 1, args, stream, b_srcs, n_src, rank, &sc);
}

}  // namespace b200
