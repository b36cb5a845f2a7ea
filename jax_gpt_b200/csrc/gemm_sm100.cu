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

#include <mutex>

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
  // B (an MN-major weight [K, N]) split by rows across b_n_src sources of b_kb_per_src K-blocks
  // each (FSDP parameter shards): K-blocks are visited starting with source b_first_src.
  int b_n_src;
  int b_kb_per_src;
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
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 /*align*/ + 256 /*barriers*/;
};

struct Barriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

template <int BN, int A_MAJOR, int B_MAJOR>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_bf16_kernel(const __grid_constant__ TmaSet tma_a, const __grid_constant__ TmaSet tma_b,
                 const __grid_constant__ GemmArgs args, const __grid_constant__ GatherInfo gi) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  // 128B swizzle needs the tile bases on 1024-byte boundaries.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = smem + C::kStages * C::kStageBytes;
  Barriers* bars = reinterpret_cast<Barriers*>(epi_stage + C::kEpiBytes);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int m_blocks = (args.M + BM - 1) / BM;
  const int n_blocks = (args.N + BN - 1) / BN;
  const int split_k = args.split_k < 1 ? 1 : args.split_k;
  const int total_kb = (args.K + BK - 1) / BK;
  const int kb_per_split = (total_kb + split_k - 1) / split_k;
  const int num_tiles = m_blocks * n_blocks * split_k;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
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
      int mi = mn % m_blocks;
      n_blk = mn / m_blocks;
      m_blk = (mi + gi.first_src * gi.blocks_per_src) % m_blocks;
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
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m_blk, n_blk, ks;
        decode_tile(t, m_blk, n_blk, ks);
        const int src = (gi.n_src > 1) ? (m_blk / gi.blocks_per_src) : 0;
        const int m0 = (gi.n_src > 1) ? (m_blk % gi.blocks_per_src) * BM : m_blk * BM;
        const int n0 = n_blk * BN;
        const CUtensorMap* ta = &tma_a.m[src];
        const int kb0 = ks * kb_per_split;
        const int kb1 = min(total_kb, kb0 + kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag)) {
            report_status(args.status, kWaitEmptyTimeout, blockIdx.x, t, kb);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * C::kStageBytes;
          uint8_t* sb = sa + C::kABytes;
          mbar_arrive_expect_tx(&bars->full[stage], C::kStageBytes);
          // with row-sharded B the K-blocks are rotated so that the local shard is consumed first
          const int kbe = (gi.b_n_src > 1) ? (kb + gi.b_first_src * gi.b_kb_per_src) % total_kb : kb;
          const int k0 = kbe * BK;
          const CUtensorMap* tbp = &tma_b.m[(gi.b_n_src > 1) ? kbe / gi.b_kb_per_src : 0];
          const int kb_row = (gi.b_n_src > 1) ? (kbe % gi.b_kb_per_src) * BK : k0;
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
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++iter) {
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
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++iter) {
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
      // Empty K range (possible only for trailing splits): nothing was accumulated.
      const bool has_k = ks * kb_per_split < total_kb;
      gemm_epilogue_columns(args, tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16),
                            epi_stage + (warp - 2) * kEpiStageBytesPerWarp, m_blk * BM + q * 32, n_blk * BN,
                            half * (BN / 2), (half + 1) * (BN / 2), lane, ks, has_k);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int BN, int A_MAJOR, int B_MAJOR>
cudaError_t launch_variant(const TmaSet& ta, const TmaSet& tb, const GemmArgs& args, const GatherInfo& gi,
                           cudaStream_t stream) {
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
  const int grid = tiles < gemm_sm_count() ? tiles : gemm_sm_count();
  kernel<<<grid, kNumThreads, C::kSmemBytes, stream>>>(ta, tb, args, gi);
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
                          int b_first_src = 0) {
  GemmArgs args = args_in;
  if (args.M <= 0 || args.N <= 0 || args.K <= 0) return cudaErrorInvalidValue;
  if (n_src < 1 || n_src > kMaxPeers) return cudaErrorInvalidValue;
  if (n_src > 1 && (rows_per_src % BM != 0 || rows_per_src * n_src != args.M)) return cudaErrorInvalidValue;
  if (args.split_k > 1 && args.out_mode != kOutF32Atomic && args.out_mode != kOutBf16PeerRed)
    return cudaErrorInvalidValue;
  if (args.alpha == 0.f) args.alpha = 1.f;
  // Narrow outputs get the 128-wide tile so that more CTAs have work.
  const int m_blocks = (args.M + BM - 1) / BM;
  const bool wide = (args.N >= 256) && (m_blocks * ((args.N + 255) / 256) * (args.split_k < 1 ? 1 : args.split_k) >=
                                        gemm_sm_count());
  const int BN = wide ? 256 : 128;

  TmaSet ta;
  for (int s = 0; s < n_src; ++s) {
    cudaError_t e = make_operand_map(&ta.m[s], a_src[s], lda, a_major, n_src > 1 ? rows_per_src : args.M, args.K, BM);
    if (e != cudaSuccess) return e;
  }
  for (int s = n_src; s < kMaxPeers; ++s) ta.m[s] = ta.m[0];
  TmaSet tb;
  cudaError_t e;
  int b_kb_per_src = 0;
  if (b_n_src > 1) {
    // row-sharded MN-major B: source s holds rows [s * K / b_n_src, (s + 1) * K / b_n_src)
    if (b_major != 1 || b_n_src > kMaxPeers || args.K % (b_n_src * BK) != 0 || args.split_k > 1) return cudaErrorInvalidValue;
    const int k_per = args.K / b_n_src;
    b_kb_per_src = k_per / BK;
    for (int s = 0; s < b_n_src; ++s)
      if ((e = make_operand_map(&tb.m[s], b_src[s], ldb, 1, args.N, k_per, BN)) != cudaSuccess) return e;
    for (int s = b_n_src; s < kMaxPeers; ++s) tb.m[s] = tb.m[0];
  } else {
    if ((e = make_operand_map(&tb.m[0], B, ldb, b_major, args.N, args.K, BN)) != cudaSuccess) return e;
    for (int s = 1; s < kMaxPeers; ++s) tb.m[s] = tb.m[0];
  }
  GatherInfo gi{n_src, n_src > 1 ? rows_per_src / BM : 0, first_src, b_n_src, b_kb_per_src, b_first_src};

#define B200_GEMM_CASE(bn, am, bm) \
  if (BN == bn && a_major == am && b_major == bm) return launch_variant<bn, am, bm>(ta, tb, args, gi, stream);
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

cudaError_t launch_gemm_bf16_sharded_b(const __nv_bfloat16* A, int64_t lda, const __nv_bfloat16* const* b_src,
                                       int b_n_src, int b_first_src, int64_t ldb, const GemmArgs& args,
                                       cudaStream_t stream) {
  const __nv_bfloat16* srcs[1] = {A};
  return launch_common(srcs, 1, 0, 0, lda, 0, nullptr, ldb, 1, args, stream, b_src, b_n_src, b_first_src);
}

cudaError_t launch_gemm_bf16_gathered_a(const __nv_bfloat16* const* a_src, int n_src, int rows_per_src,
                                        int first_src, int64_t lda, const __nv_bfloat16* B, int64_t ldb, int b_major,
                                        const GemmArgs& args, cudaStream_t stream) {
  return launch_common(a_src, n_src, rows_per_src, first_src, lda, 0, B, ldb, b_major, args, stream);
}

}  // namespace b200
