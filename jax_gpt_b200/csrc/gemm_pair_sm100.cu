// CTA-pair bf16 GEMM for sm_100a: two CTAs of a cluster (one SM each) share one 256 x 256 output
// tile through tcgen05.mma.cta_group::2.
//
// The single-CTA kernel (gemm_sm100.cu) reads 16 KB of A and 32 KB of B from shared memory and
// receives the same 48 KB from TMA for every 128 x 256 x 64 block, which is more than the shared
// memory of one SM delivers in the 512 cycles the tensor pipe needs for it. Here each CTA stages its
// own 128 rows of A and only HALF of the tile's B columns (128 of 256): the pair's MMA reads both
// halves, so the per-SM shared-memory traffic of a k-block drops from 96 KB to 64 KB.
//
//   warp 0      : TMA producer in BOTH CTAs (own A rows, own B half; completion bytes are counted
//                 on the LEADER's full barrier; every CTA fetches its own tiles)
//   warp 1      : MMA issuer in the leader CTA (rank 0 of the cluster); TMEM alloc / free in both
//   warps 2..9  : epilogue in both CTAs: each drains the 128 accumulator rows in its own TMEM
//
// Barriers: full[] lives in the leader (one expect_tx arrival for the bytes of both CTAs);
// empty[] and tmem_full[] exist in both CTAs and are signalled together by a multicast
// tcgen05.commit; tmem_empty[] lives in the leader and collects the 16 epilogue warps of the pair.
// Every wait is bounded; after a time-out the CTA raises its abort flag, records a status word and
// walks to the common exit, where both CTAs meet at a cluster barrier before TMEM is freed.
//
// Same role as the single-CTA kernel: the dot products behind every linear layer of the reference
// (jax_gpt/models/gpt2/model.py:95-102,145,180).
#include "gemm_sm100.cuh"

#include <cstdlib>

#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "tma_host.h"

namespace b200 {

namespace {

constexpr int BM = 128;    // accumulator rows per CTA (the pair covers 256)
constexpr int BN = 256;    // tile columns
constexpr int BNH = 128;   // B rows staged by each CTA
constexpr int BK = 64;
constexpr int kStages = 6;
constexpr int kABytes = BM * BK * 2;
constexpr int kBBytes = BNH * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = 2 * BN;
constexpr int kEpiBytes = 8 * kEpiStageBytesPerWarp;  // store staging of the eight epilogue warps
constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 + 256;
constexpr int kNumThreads = 320;
constexpr int kBand = 8;   // 256-row blocks per band of the tile order

struct PairBarriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory offset in CTA `rank` of the cluster (shared::cluster window).
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Tile load into this CTA's shared memory; the completion bytes go to the barrier at the cluster
// address `bar_cluster` (the leader's), which the cta_group::2 form of the copy permits.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster, int c0,
                                                 int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrives once on the barrier at this offset in BOTH CTAs when the pair's MMAs issued so far are done.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(static_cast<uint16_t>(3))
      : "memory");
}
// D[tmem of both CTAs] (+)= A[256 x 16: 128 rows from each CTA] * B[256 x 16: 128 rows from each CTA].
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int A_MAJOR, int B_MAJOR>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNumThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                      const __grid_constant__ GemmArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = smem + kStages * kStageBytes;
  PairBarriers* bars = reinterpret_cast<PairBarriers*>(epi_stage + kEpiBytes);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;

  const int m_blocks = (args.M + 2 * BM - 1) / (2 * BM);
  const int n_blocks = (args.N + BN - 1) / BN;
  const int split_k = args.split_k < 1 ? 1 : args.split_k;
  const int total_kb = (args.K + BK - 1) / BK;
  const int kb_per_split = (total_kb + split_k - 1) / split_k;
  const int num_tiles = m_blocks * n_blocks * split_k;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], 16);
    }
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(&bars->tmem_base, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  // Linear pair-tile index -> (256-row block, 256-column block, k split); bands of kBand row blocks
  // keep the tiles that run together inside a small set of A and B panels (L2 reuse).
  auto decode_tile = [&](int t, int& m_blk, int& n_blk, int& ks) {
    ks = t % split_k;
    const int mn = t / split_k;
    const int per_band = kBand * n_blocks;
    const int band = mn / per_band, r = mn - band * per_band;
    const int rows = min(kBand, m_blocks - band * kBand);
    m_blk = band * kBand + r % rows;
    n_blk = r / rows;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      const uint32_t full_leader = mapa_u32(smem_u32(&bars->full[0]), 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += n_pairs) {
        int m_blk, n_blk, ks;
        decode_tile(t, m_blk, n_blk, ks);
        const int m0 = m_blk * 2 * BM + static_cast<int>(rank) * BM;
        const int n0 = n_blk * BN + static_cast<int>(rank) * BNH;
        const int kb0 = ks * kb_per_split;
        const int kb1 = min(total_kb, kb0 + kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag)) {
            report_status(args.status, kWaitEmptyTimeout, blockIdx.x, t, kb);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          if (rank == 0) mbar_arrive_expect_tx(&bars->full[stage], 2 * kStageBytes);
          const uint32_t fb = full_leader + stage * 8;
          const int k0 = kb * BK;
          if (A_MAJOR == 0) {
            tma_load_2d_pair(sa, &tma_a, fb, k0, m0);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d_pair(sa + i * 8192, &tma_a, fb, m0 + 64 * i, k0);
          }
          if (B_MAJOR == 0) {
            tma_load_2d_pair(sb, &tma_b, fb, k0, n0);
          } else {
#pragma unroll
            for (int i = 0; i < BNH / 64; ++i) tma_load_2d_pair(sb + i * 8192, &tma_b, fb, n0 + 64 * i, k0);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if ((!ok || *abort_flag) && rank == 0) {
        // Unwinding: give the copies of both CTAs that are still in flight a bounded time to land
        // (they are counted on this CTA's full barriers) before the pair meets at the exit barrier.
        for (int s = 0; s < kStages; ++s) {
          const uint32_t armed_parity = (s < stage) ? phase : (phase ^ 1);
          const uint64_t t0 = globaltimer_ns();
          while (!mbar_try_wait(&bars->full[s], armed_parity)) {
            if (globaltimer_ns() - t0 > 2000000ull) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA) ------------------------------
    if (rank == 0) {
      constexpr uint32_t idesc = make_idesc(2 * BM, BN, A_MAJOR, B_MAJOR, /*bf16*/ 1);
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += n_pairs, ++iter) {
        int m_blk, n_blk, ks;
        decode_tile(t, m_blk, n_blk, ks);
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1;
        if (!mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1, abort_flag)) {
          if (lane == 0) report_status(args.status, kWaitTmemEmptyTimeout, blockIdx.x, t, iter);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        const int kb0 = ks * kb_per_split;
        const int kb1 = min(total_kb, kb0 + kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&bars->full[stage], phase, abort_flag)) {
            if (lane == 0) report_status(args.status, kWaitFullTimeout, blockIdx.x, t, kb);
            ok = false;
            break;
          }
          tc_fence_after();
          if (lane == 0) {
            const uint32_t sa = smem_u32(smem + stage * kStageBytes);
            const uint32_t sb = sa + kABytes;
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              const uint64_t adesc = (A_MAJOR == 0) ? make_smem_desc(sa + k * 32, 16, 1024)
                                                    : make_smem_desc(sa + k * 2048, 8192, 1024);
              const uint64_t bdesc = (B_MAJOR == 0) ? make_smem_desc(sb + k * 32, 16, 1024)
                                                    : make_smem_desc(sb + k * 2048, 8192, 1024);
              umma_bf16_pair(tmem_d, adesc, bdesc, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            }
            tc_commit_pair(&bars->empty[stage]);  // frees the stage in both CTAs
          }
          __syncwarp();
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok && lane == 0) tc_commit_pair(&bars->tmem_full[acc]);
        __syncwarp();
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ------------------------------
    const int q = warp & 3;            // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;  // which half of the tile's columns this warp converts and stores
    const uint32_t empty_leader = mapa_u32(smem_u32(&bars->tmem_empty[0]), 0);
    int iter = 0;
    bool ok = true;
    for (int t = pair; t < num_tiles && ok; t += n_pairs, ++iter) {
      int m_blk, n_blk, ks;
      decode_tile(t, m_blk, n_blk, ks);
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      if (!mbar_wait(&bars->tmem_full[acc], acc_phase, abort_flag)) {
        if (lane == 0) report_status(args.status, kWaitTmemFullTimeout, blockIdx.x, t, iter);
        ok = false;
        break;
      }
      tc_fence_after();
      const bool has_k = ks * kb_per_split < total_kb;
      gemm_epilogue_columns(args, tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16),
                            epi_stage + (warp - 2) * kEpiStageBytesPerWarp,
                            m_blk * 2 * BM + static_cast<int>(rank) * BM + q * 32, n_blk * BN, half * (BN / 2),
                            (half + 1) * (BN / 2), lane, ks, has_k);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(empty_leader + acc * 8);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves (or frees TMEM) while the other may still read its memory
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <int A_MAJOR, int B_MAJOR>
cudaError_t launch_pair_variant(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& args, int tiles,
                                cudaStream_t stream) {
  auto kernel = gemm_bf16_pair_kernel<A_MAJOR, B_MAJOR>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const int max_pairs = gemm_sm_count() / 2;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  kernel<<<2 * pairs, kNumThreads, kSmemBytes, stream>>>(ta, tb, args);
  return cudaGetLastError();
}

}  // namespace

int gemm_pair_mode() {
  static int mode = -1;
  if (mode < 0) {
    const char* e = std::getenv("B200_GEMM_PAIR");
    mode = (e == nullptr) ? 2 : std::atoi(e);  // 0: never, 1: whenever the shape allows, 2: by tile count
  }
  return mode;
}

bool gemm_pair_wanted(const GemmArgs& args) {
  const int mode = gemm_pair_mode();
  if (mode == 0 || args.N < 256 || args.M < 256) return false;
  if (mode == 1) return true;
  const int64_t tiles = static_cast<int64_t>((args.M + 255) / 256) * ((args.N + 255) / 256) *
                        (args.split_k < 1 ? 1 : args.split_k);
  return 4 * tiles >= 3 * (gemm_sm_count() / 2);  // at least three quarters of the CTA pairs get a tile
}

cudaError_t launch_gemm_bf16_pair(const __nv_bfloat16* A, int64_t lda, int a_major, const __nv_bfloat16* B, int64_t ldb,
                                  int b_major, const GemmArgs& args_in, cudaStream_t stream) {
  GemmArgs args = args_in;
  if (args.M <= 0 || args.N <= 0 || args.K <= 0) return cudaErrorInvalidValue;
  if (args.split_k > 1 && args.out_mode != kOutF32Atomic && args.out_mode != kOutBf16PeerRed)
    return cudaErrorInvalidValue;
  if (args.alpha == 0.f) args.alpha = 1.f;
  CUtensorMap ta, tb;
  cudaError_t e;
  // K-major: stored [rows, K], box {64 (k), 128}. MN-major: stored [K, rows], box {64 (mn), 64 (k)}.
  if (a_major == 0) e = encode_tma_2d(&ta, A, 2, args.K, args.M, lda * 2, 64, BM);
  else e = encode_tma_2d(&ta, A, 2, args.M, args.K, lda * 2, 64, 64);
  if (e != cudaSuccess) return e;
  if (b_major == 0) e = encode_tma_2d(&tb, B, 2, args.K, args.N, ldb * 2, 64, BNH);
  else e = encode_tma_2d(&tb, B, 2, args.N, args.K, ldb * 2, 64, 64);
  if (e != cudaSuccess) return e;
  const int tiles = ((args.M + 2 * BM - 1) / (2 * BM)) * ((args.N + BN - 1) / BN) * (args.split_k < 1 ? 1 : args.split_k);
  if (a_major == 0 && b_major == 0) return launch_pair_variant<0, 0>(ta, tb, args, tiles, stream);
  if (a_major == 0 && b_major == 1) return launch_pair_variant<0, 1>(ta, tb, args, tiles, stream);
  if (a_major == 1 && b_major == 0) return launch_pair_variant<1, 0>(ta, tb, args, tiles, stream);
  return launch_pair_variant<1, 1>(ta, tb, args, tiles, stream);
}

}  // namespace b200
