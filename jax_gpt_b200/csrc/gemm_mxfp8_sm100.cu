// FP8 (e4m3) GEMM with the block scales applied BY THE TENSOR CORE: tcgen05.mma kind::mxf8f6f4
// .block_scale multiplies every 32-element K block of A and B by a UE8M0 (power-of-two) scale
// held in TMEM, so 1 x 128 activation scales and 128 x 128 weight scales that are powers of two
// cost nothing in the main loop (each scale is simply repeated for the four 32-blocks of its
// 128-wide slab). C[M,N] (bf16) = (A_q * sfa) . (B_q * sfb)^T with fp32 accumulation.
//
// Scale layout in global memory ("packed"): for every 128-row block and every 128-wide K slab one
// 512-byte chunk; byte (r % 32) * 16 + (r / 32) * 4 + j is the scale exponent of row r for K block
// j of the slab. That chunk is what one tcgen05.cp 32x128b.warpx4 moves from shared memory into
// four TMEM columns in the arrangement the MMA reads (lane r % 32, column r / 32, byte j).
//
// Pipeline: warp 0 TMA producer (A 128 x 128 B, B 256 x 128 B, three 512-byte scale chunks per
// stage), warp 1 issues tcgen05.cp + four K=32 MMAs per stage into ONE 128 x 256 fp32
// accumulator, eight epilogue warps pull it into registers (128 columns each), release it at
// once and convert / store while the next tile's main loop runs.
//
// The reference has no block-scaled path: its FP8 is per-row scaled W8A8 with de-quantisation of
// expert weights before the matmul (jax_gpt/models/qwen35/fp8.py:70-91,137-150).
#include "gemm_fp8_sm100.cuh"

#include "common.cuh"
#include "tma_host.h"

namespace b200 {

namespace {

constexpr int BM = 128, BN = 256, BK = 128;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK, kBBytes = BN * BK;
constexpr int kSfBytes = 512;
constexpr int kStageBytes = kABytes + kBBytes;       // 48 KB of operand tiles
constexpr int kStageSf = 3 * kSfBytes;               // SFA + two SFB chunks
constexpr int kThreads = 320;                        // producer, MMA, 8 epilogue warps
constexpr int kSfCol0 = 256;                         // TMEM: accumulator 0..255, scales from 256 (12 columns per stage)
constexpr int kSmem = 1024 + kStages * (kStageBytes + kStageSf) + 256;

struct Bars {
  uint64_t full[kStages], empty[kStages], tmem_full, tmem_empty;
  uint32_t tmem_base;
  int abort_flag;
};

struct MxArgs {
  int M, N, K;
  const uint8_t* sfa;  // [ceil(M/128), K/128, 512]
  const uint8_t* sfb;  // [ceil(N/128), K/128, 512]
  __nv_bfloat16* out;
  int64_t ldo;
  int* status;
};

// Tile order: bands of 16 m-blocks, n-blocks inside a band, so that one wave of 148 CTAs touches about
// 16 x 9 tiles (16 MB of A + 18 MB of B at K = 8192) instead of a full column of A per n-block.
constexpr int kBand = 16;
__device__ __forceinline__ void tile_coords(int t, int m_blocks, int n_blocks, int* mb, int* nb) {
  const int per_band = kBand * n_blocks;
  const int band = t / per_band, r = t - band * per_band;
  const int rows = min(kBand, m_blocks - band * kBand);
  *mb = band * kBand + r % rows;
  *nb = r / rows;
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap ta, const __grid_constant__ CUtensorMap tb,
                  const __grid_constant__ MxArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sf_smem = smem + kStages * kStageBytes;
  Bars* bars = reinterpret_cast<Bars*>(sf_smem + kStages * kStageSf);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_blocks = (a.M + BM - 1) / BM, n_blocks = (a.N + BN - 1) / BN;
  const int slabs = a.K / BK;
  const int num_tiles = m_blocks * n_blocks;
  const int sfb_rows = (a.N + 127) / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->tmem_full, 1);
    mbar_init(&bars->tmem_empty, 8);
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mb, nb;
        tile_coords(t, m_blocks, n_blocks, &mb, &nb);
        for (int s = 0; s < slabs; ++s) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag)) {
            report_status(a.status, kWaitEmptyTimeout, 80, blockIdx.x, t);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sf = sf_smem + stage * kStageSf;
          const int nb1 = 2 * nb + 1 < sfb_rows ? 2 * nb + 1 : 2 * nb;  // odd tail: the second half is out of range anyway
          mbar_arrive_expect_tx(&bars->full[stage], kStageBytes + kStageSf);
          tma_load_2d(sa, &ta, &bars->full[stage], s * BK, mb * BM);
          tma_load_2d(sa + kABytes, &tb, &bars->full[stage], s * BK, nb * BN);
          bulk_load_1d(sf, a.sfa + (static_cast<int64_t>(mb) * slabs + s) * kSfBytes, kSfBytes, &bars->full[stage]);
          bulk_load_1d(sf + kSfBytes, a.sfb + (static_cast<int64_t>(2 * nb) * slabs + s) * kSfBytes, kSfBytes,
                       &bars->full[stage]);
          bulk_load_1d(sf + 2 * kSfBytes, a.sfb + (static_cast<int64_t>(nb1) * slabs + s) * kSfBytes, kSfBytes,
                       &bars->full[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
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
    int stage = 0, iter = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++iter) {
      if (!mbar_wait(&bars->tmem_empty, (iter & 1) ^ 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitTmemEmptyTimeout, 81, blockIdx.x, t);
        break;
      }
      tc_fence_after();
      for (int s = 0; s < slabs; ++s) {
        if (!mbar_wait(&bars->full[stage], phase, abort_flag)) {
          if (lane == 0) report_status(a.status, kWaitFullTimeout, 82, blockIdx.x, t);
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sa = smem_u32(smem + stage * kStageBytes), sb = sa + kABytes;
          const uint32_t sf = smem_u32(sf_smem + stage * kStageSf);
          const uint32_t tsf = tmem_base + kSfCol0 + stage * 12;
          tmem_cp_sf(tsf, make_sf_desc(sf));
          tmem_cp_sf(tsf + 4, make_sf_desc(sf + kSfBytes));
          tmem_cp_sf(tsf + 8, make_sf_desc(sf + 2 * kSfBytes));
#pragma unroll
          for (int k = 0; k < BK / 32; ++k)
            umma_mxf8(tmem_base, make_smem_desc(sa + k * 32, 16, 1024), make_smem_desc(sb + k * 32, 16, 1024),
                      make_idesc_mx(BM, BN, k), tsf, tsf + 4, (s > 0 || k > 0) ? 1u : 0u);
          tc_commit(&bars->empty[stage]);
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok && lane == 0) tc_commit(&bars->tmem_full);
      __syncwarp();
    }
  } else {
    const int ew = warp - 2;            // 0..7
    const int q = warp & 3;             // TMEM lane quarter this warp may read
    const int half = ew >> 2;           // which 128 accumulator columns
    int iter = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++iter) {
      int mb, nb;
      tile_coords(t, m_blocks, n_blocks, &mb, &nb);
      if (!mbar_wait(&bars->tmem_full, iter & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitTmemFullTimeout, 83, blockIdx.x, t);
        break;
      }
      tc_fence_after();
      uint32_t v[4][32];
      const uint32_t taddr = tmem_base + half * 128 + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(taddr + c * 32, v[c]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty);   // the accumulator is in registers: the next tile may start
      const int row = mb * BM + q * 32 + lane;
      const int n0 = nb * BN + half * 128;
      if (row < a.M) {
        __nv_bfloat16* o = a.out + static_cast<int64_t>(row) * a.ldo + n0;
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int j = 0; j < 32; j += 8)
            if (n0 + c * 32 + j + 8 <= a.N)
              *reinterpret_cast<uint4*>(o + c * 32 + j) = make_uint4(
                  pack_bf16x2(__uint_as_float(v[c][j]), __uint_as_float(v[c][j + 1])),
                  pack_bf16x2(__uint_as_float(v[c][j + 2]), __uint_as_float(v[c][j + 3])),
                  pack_bf16x2(__uint_as_float(v[c][j + 4]), __uint_as_float(v[c][j + 5])),
                  pack_bf16x2(__uint_as_float(v[c][j + 6]), __uint_as_float(v[c][j + 7])));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace

cudaError_t launch_gemm_mxfp8(const uint8_t* a_q, const uint8_t* sfa_packed, const uint8_t* b_q,
                              const uint8_t* sfb_packed, __nv_bfloat16* out, int64_t ldo, int M, int N, int K, int* status,
                              cudaStream_t stream) {
  if (K % BK != 0 || N % 8 != 0 || M <= 0 || N <= 0 || ldo % 8 != 0) return cudaErrorInvalidValue;
  CUtensorMap ta, tb;
  cudaError_t e;
  if ((e = encode_tma_2d(&ta, a_q, 1, K, M, K, 128, BM)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tb, b_q, 1, K, N, K, 128, BN)) != cudaSuccess) return e;
  static bool configured = false;
  if (!configured) {
    if ((e = cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem)) != cudaSuccess) return e;
    configured = true;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  MxArgs args{M, N, K, sfa_packed, sfb_packed, out, ldo, status};
  gemm_mxfp8_kernel<<<tiles < sms ? tiles : sms, kThreads, kSmem, stream>>>(ta, tb, args);
  return cudaGetLastError();
}

}  // namespace b200
