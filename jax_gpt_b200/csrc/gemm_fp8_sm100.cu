// Block-scaled FP8 (e4m3) GEMM for sm_100a: C[M,N] = sum over 128-wide K slabs of
//   (A_q[:, slab] . B_q[:, slab]^T) * sa[m, slab] * sb[n / 128, slab]
// with 1 x 128 activation scales and 128 x 128 weight scales, fp32 accumulation, bf16 output.
//
// tcgen05.mma kind::f8f6f4 accumulates ONE slab at a time into a TMEM buffer; the two buffers
// ping-pong so that the tensor core works on slab s+1 while the four epilogue warps read slab s
// back with tcgen05.ld, apply the two scales with one FMA per element and add into fp32
// register accumulators (the scales are arbitrary fp32 numbers, so they cannot ride on the
// hardware's power-of-two block-scale path). TMA feeds a 6-stage ring of 128 x 128-byte tiles.
//
// The reference only has per-row scales and de-quantises expert weights to bf16 before the
// matmul (jax_gpt/models/qwen35/fp8.py:70-91,137-150); this is the block-scaled scheme instead.
#include "gemm_fp8_sm100.cuh"

#include "common.cuh"
#include "tma_host.h"

namespace b200 {

namespace {

constexpr int BM = 128, BN = 128, BK = 128;  // BK in elements == bytes
constexpr int kStages = 6;
constexpr int kTile = BM * BK;               // 16 KB
constexpr int kStageBytes = 2 * kTile;
constexpr int kThreads = 192;
constexpr int kSmem = kStages * kStageBytes + 1024 + 256;

struct Bars {
  uint64_t full[kStages], empty[kStages], tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

struct Fp8Args {
  int M, N, K;
  const float* sa;  // [M, K/128]
  const float* sb;  // [N/128 (ceil), K/128]
  void* out;
  int64_t ldo;
  int out_f32;
  int* status;
};

__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap ta, const __grid_constant__ CUtensorMap tb,
                const __grid_constant__ Fp8Args a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Bars* bars = reinterpret_cast<Bars*>(smem + kStages * kStageBytes);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_blocks = (a.M + BM - 1) / BM, n_blocks = (a.N + BN - 1) / BN;
  const int slabs = a.K / BK;
  const int num_tiles = m_blocks * n_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->tmem_full[i], 1);
      mbar_init(&bars->tmem_empty[i], 4);
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

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m0 = (t % m_blocks) * BM, n0 = (t / m_blocks) * BN;
        for (int s = 0; s < slabs; ++s) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag)) {
            report_status(a.status, kWaitEmptyTimeout, 60, blockIdx.x, t);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kStageBytes;
          mbar_arrive_expect_tx(&bars->full[stage], kStageBytes);
          tma_load_2d(sa, &ta, &bars->full[stage], s * BK, m0);
          tma_load_2d(sa + kTile, &tb, &bars->full[stage], s * BK, n0);
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
    constexpr uint32_t idesc = make_idesc(BM, BN, 0, 0, /*e4m3*/ 0);
    int stage = 0;
    uint32_t phase = 0;
    int slab_iter = 0;  // global slab counter: buffer = slab_iter & 1
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      for (int s = 0; s < slabs && ok; ++s, ++slab_iter) {
        const int buf = slab_iter & 1;
        if (!mbar_wait(&bars->tmem_empty[buf], ((slab_iter >> 1) & 1) ^ 1, abort_flag) ||
            !mbar_wait(&bars->full[stage], phase, abort_flag)) {
          if (lane == 0) report_status(a.status, kWaitFullTimeout, 61, blockIdx.x, t);
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sa = smem_u32(smem + stage * kStageBytes), sb = sa + kTile;
#pragma unroll
          for (int k = 0; k < BK / 32; ++k)
            umma_f8(tmem_base + buf * BN, make_smem_desc(sa + k * 32, 16, 1024), make_smem_desc(sb + k * 32, 16, 1024),
                    idesc, k > 0 ? 1u : 0u);
          tc_commit(&bars->empty[stage]);
          tc_commit(&bars->tmem_full[buf]);
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int kslabs = slabs;
    int slab_iter = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const int m0 = (t % m_blocks) * BM, n_blk = t / m_blocks;
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < a.M;
      const float* sa_row = a.sa + static_cast<int64_t>(row_ok ? row : 0) * kslabs;
      const float* sb_row = a.sb + static_cast<int64_t>(n_blk) * kslabs;
      float acc[BN];
#pragma unroll
      for (int j = 0; j < BN; ++j) acc[j] = 0.f;
      for (int s = 0; s < slabs; ++s, ++slab_iter) {
        const int buf = slab_iter & 1;
        if (!mbar_wait(&bars->tmem_full[buf], (slab_iter >> 1) & 1, abort_flag)) {
          if (lane == 0) report_status(a.status, kWaitTmemFullTimeout, 62, blockIdx.x, t);
          ok = false;
          break;
        }
        tc_fence_after();
        const float sc = sa_row[s] * sb_row[s];
        const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(taddr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c * 32 + j] = fmaf(__uint_as_float(v[j]), sc, acc[c * 32 + j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->tmem_empty[buf]);
      }
      if (ok && row_ok) {
        const int n0 = n_blk * BN;
        if (a.out_f32) {
          float* o = static_cast<float*>(a.out) + static_cast<int64_t>(row) * a.ldo + n0;
#pragma unroll
          for (int j = 0; j < BN; j += 4)
            if (n0 + j + 4 <= a.N) *reinterpret_cast<float4*>(o + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
        } else {
          __nv_bfloat16* o = static_cast<__nv_bfloat16*>(a.out) + static_cast<int64_t>(row) * a.ldo + n0;
#pragma unroll
          for (int j = 0; j < BN; j += 8)
            if (n0 + j + 8 <= a.N)
              *reinterpret_cast<uint4*>(o + j) =
                  make_uint4(pack_bf16x2(acc[j], acc[j + 1]), pack_bf16x2(acc[j + 2], acc[j + 3]),
                             pack_bf16x2(acc[j + 4], acc[j + 5]), pack_bf16x2(acc[j + 6], acc[j + 7]));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

}  // namespace

cudaError_t launch_gemm_fp8_blockscaled(const uint8_t* a_q, const float* a_scales, const uint8_t* b_q,
                                        const float* b_scales, void* out, int64_t ldo, int out_f32, int M, int N, int K,
                                        int* status, cudaStream_t stream) {
  if (K % BK != 0 || N % 8 != 0 || M <= 0 || N <= 0 || (out_f32 ? ldo % 4 : ldo % 8) != 0) return cudaErrorInvalidValue;
  CUtensorMap ta, tb;
  cudaError_t e;
  if ((e = encode_tma_2d(&ta, a_q, 1, K, M, K, 128, BM)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tb, b_q, 1, K, N, K, 128, BN)) != cudaSuccess) return e;
  static bool configured = false;
  if (!configured) {
    if ((e = cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem)) != cudaSuccess) return e;
    configured = true;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  Fp8Args args{M, N, K, a_scales, b_scales, out, ldo, out_f32, status};
  gemm_fp8_kernel<<<tiles < sms ? tiles : sms, kThreads, kSmem, stream>>>(ta, tb, args);
  return cudaGetLastError();
}

}  // namespace b200
