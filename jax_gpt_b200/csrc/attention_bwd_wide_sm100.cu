// Flash attention backward on tcgen05 for the WIDE heads: width 256 (gated attention of the hybrid model:
// jax_gpt/models/qwen35/gqa.py:103-119 is the dense forward this differentiates) and the MLA prefill shape
// (q/k heads 192 wide, v heads 128 wide).
//
// One CTA per (128-key block, kv head [, half of the head width], batch) loops over 64-query tiles and works on
// the transposed score tile, so that a thread owns a key row:
//
//   S^T  [128 keys x 64 q] = K Q^T          dP^T [128 x 64] = V dO^T          (TMEM columns [0,64) and [64,128))
//   P^T = exp2(scale * S^T - lse),  dS^T = P^T * (dP^T - delta) * scale       (compute warps -> shared memory)
//   dV  [128 x NV] += P^T dO        dK [128 x NK] += dS^T Q                  (accumulate in TMEM over the loop)
//   dQ^T [d x 64 q] = K^T dS^T                                                 (fp32 reductions into dq_accum)
//
// The accumulators are what limits the tile: dV and dK of a 128-key block at width 256 are 512 TMEM columns by
// themselves. Width 256 therefore runs TWO CTAs per key block; each computes the full scores (they need the whole
// head width) but only 128 of the 256 columns of dV, dK and dQ. The MLA shape fits in one CTA (dV 128, dK 192
// columns) with dQ^T re-using the score columns: two overlapping 128-row blocks (d 0..127 and 64..191), of which
// the second contributes rows 128..191.
//
// Q and dO tiles are 64 rows high so that K, V, one Q / dO stage, P^T and dS^T fit in shared memory (224 KB at
// width 256, single stage; two stages at the MLA shape).
#include "attention_sm100.cuh"

#include "common.cuh"
#include "tma_host.h"

namespace b200 {

namespace {

constexpr int kWThreads = 320;  // TMA warp, MMA warp, 8 compute warps
constexpr float kLog2eW = 1.4426950408889634f;

struct WArgs {
  int B, T, H, Hkv;
  float scale, scale_log2;
  int causal;
  const float* lse;
  const float* delta;
  float* dq_accum;  // [B*T, H*DQK] fp32
  __nv_bfloat16* dk;
  int64_t lddk;
  __nv_bfloat16* dv;
  int64_t lddv;
  int* status;
};

template <int DQK, int DV, int NSPLIT>
struct WCfg {
  static constexpr int NK = DQK / NSPLIT;            // dK / dQ columns of one CTA
  static constexpr int NV = DV / NSPLIT;             // dV columns of one CTA
  static constexpr int kKTile = 128 * DQK * 2;
  static constexpr int kVTile = 128 * DV * 2;
  static constexpr int kQTile = 64 * DQK * 2;
  static constexpr int kDOTile = 64 * DV * 2;
  static constexpr int kStageBytes = kQTile + kDOTile;
  static constexpr int kFixed = kKTile + kVTile + 2 * 16384 + 1024 + 256;
  static constexpr int kStages = (kFixed + 2 * kStageBytes <= 232448) ? 2 : 1;
  static constexpr int kOffK = 0;
  static constexpr int kOffV = kKTile;
  static constexpr int kOffRing = kKTile + kVTile;
  static constexpr int kOffPT = kOffRing + kStages * kStageBytes;   // P^T  128 x 64 bf16
  static constexpr int kOffDST = kOffPT + 16384;                    // dS^T 128 x 64 bf16
  static constexpr int kOffStats = kOffDST + 16384;                 // [2][2][64] fp32
  static constexpr int kOffBar = kOffStats + 1024;
  static constexpr int kSmem = kOffBar + 256;
  static constexpr uint32_t kColST = 0, kColDP = 64, kColDV = 128, kColDK = 256;
  static constexpr int kQBlks = (NK + 127) / 128;                   // 128-row blocks of dQ^T
  static constexpr bool kAliasDq = (256 + NK + 64 * kQBlks > 512);
  static constexpr uint32_t kColDQ = kAliasDq ? 0u : 256u + NK;
  static_assert(kSmem <= 232448, "shared memory");
  static_assert(NK % 16 == 0 && NV % 16 == 0 && NK <= 256 && NV <= 128, "tile widths");
  static_assert(kQBlks <= 2 && NK >= 128, "dQ^T blocks");
};

struct WBars {
  uint64_t kv_full, qdo_full[2], qdo_empty[2], st_full, p_ready, dq_full, dq_read, stats_ready;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* m, int c0, int c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(m)),
               "r"(c0), "r"(c1)
               : "memory");
}

// 32 bf16 values of row r, columns [c0, c0+32) of a 128-row x 64-column K-major 128B-swizzled tile.
__device__ __forceinline__ void store_chunk64(uint8_t* tile, int r, int c0, const uint32_t (&pk)[16]) {
  uint8_t* base = tile + r * 128;
  const int chunk0 = c0 >> 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int phys = (chunk0 + i) ^ (r & 7);
    *reinterpret_cast<uint4*>(base + phys * 16) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
  }
}

template <int DQK, int DV, int NSPLIT>
__global__ void __launch_bounds__(kWThreads, 1)
attn_bwd_wide_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                     const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                     const __grid_constant__ WArgs a) {
  using C = WCfg<DQK, DV, NSPLIT>;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) report_status(a.status, kBadArgument, 13, 0, 0);
    return;
  }
  WBars* bars = reinterpret_cast<WBars*>(smem + C::kOffBar);
  volatile int* abort_flag = &bars->abort_flag;
  float* stats = reinterpret_cast<float*>(smem + C::kOffStats);  // [buf][0: lse, 1: delta * scale][64]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jb = blockIdx.z;                 // key block
  const int hkv = blockIdx.x / NSPLIT, split = blockIdx.x % NSPLIT, b = blockIdx.y;
  const int group = a.H / a.Hkv;
  const int n_q64 = (a.T + 63) / 64;
  const int i0 = a.causal ? jb * 2 : 0;      // first 64-query tile that sees this key block
  const int nqi = max(n_q64 - i0, 0);
  const int n_iters = group * nqi;
  const int ck0 = split * C::NK, cv0 = split * C::NV;   // first dK / dQ and dV column of this CTA

  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->qdo_full[s], 1);
      mbar_init(&bars->qdo_empty[s], 1);
    }
    mbar_init(&bars->st_full, 1);
    mbar_init(&bars->p_ready, 256);
    mbar_init(&bars->dq_full, 1);
    mbar_init(&bars->dq_read, 256);
    mbar_init(&bars->stats_ready, 256);
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
  const uint32_t tmem = bars->tmem_base;
  const int kv_row0 = b * a.T + jb * 128;

  if (warp == 0) {
    if (lane == 0 && n_iters > 0) {
      tma_prefetch_desc(&tq);
      tma_prefetch_desc(&tdo);
      mbar_arrive_expect_tx(&bars->kv_full, C::kKTile + C::kVTile);
#pragma unroll
      for (int c = 0; c < DQK / 64; ++c)
        tma_load_2d(smem + C::kOffK + c * 16384, &tk, &bars->kv_full, hkv * DQK + c * 64, kv_row0);
#pragma unroll
      for (int c = 0; c < DV / 64; ++c)
        tma_load_2d(smem + C::kOffV + c * 16384, &tv, &bars->kv_full, hkv * DV + c * 64, kv_row0);
      for (int it = 0; it < n_iters; ++it) {
        const int s = it % C::kStages;
        const uint32_t ph = (it / C::kStages) & 1;
        if (!mbar_wait(&bars->qdo_empty[s], ph ^ 1, abort_flag)) {
          report_status(a.status, kWaitEmptyTimeout, 240, jb, it);
          break;
        }
        const int hq = hkv * group + it / nqi;
        const int qrow0 = b * a.T + (i0 + it % nqi) * 64;
        uint8_t* st = smem + C::kOffRing + s * C::kStageBytes;
        mbar_arrive_expect_tx(&bars->qdo_full[s], C::kStageBytes);
#pragma unroll
        for (int c = 0; c < DQK / 64; ++c)
          tma_load_2d(st + c * 8192, &tq, &bars->qdo_full[s], hq * DQK + c * 64, qrow0);
#pragma unroll
        for (int c = 0; c < DV / 64; ++c)
          tma_load_2d(st + C::kQTile + c * 8192, &tdo, &bars->qdo_full[s], hq * DV + c * 64, qrow0);
        if (C::kStages == 1 && it + 1 < n_iters) {
          // single stage: pull the next tile into L2 so that its load after the release is short
          const int hq1 = hkv * group + (it + 1) / nqi;
          const int qrow1 = b * a.T + (i0 + (it + 1) % nqi) * 64;
#pragma unroll
          for (int c = 0; c < DQK / 64; ++c) tma_prefetch_2d(&tq, hq1 * DQK + c * 64, qrow1);
#pragma unroll
          for (int c = 0; c < DV / 64; ++c) tma_prefetch_2d(&tdo, hq1 * DV + c * 64, qrow1);
        }
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc_st = make_idesc(128, 64, 0, 0, 1);        // K-major x K-major, 64 queries
    constexpr uint32_t idesc_dv = make_idesc(128, C::NV, 0, 1, 1);     // A K-major, B MN-major
    constexpr uint32_t idesc_dk = make_idesc(128, C::NK, 0, 1, 1);
    constexpr uint32_t idesc_dq = make_idesc(128, 64, 1, 1, 1);        // A MN-major (K^T), B MN-major (dS^T)
    bool ok = n_iters > 0 && mbar_wait(&bars->kv_full, 0, abort_flag);
    if (n_iters > 0 && !ok && lane == 0) report_status(a.status, kWaitFullTimeout, 241, jb, 0);
    const uint32_t aK = smem_u32(smem + C::kOffK), aV = smem_u32(smem + C::kOffV);
    const uint32_t aPT = smem_u32(smem + C::kOffPT), aDST = smem_u32(smem + C::kOffDST);
    auto issue_scores = [&](int it) -> bool {
      const int s = it % C::kStages;
      if (!mbar_wait(&bars->qdo_full[s], (it / C::kStages) & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitFullTimeout, 242, jb, it);
        return false;
      }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t aQ = smem_u32(smem + C::kOffRing + s * C::kStageBytes);
        const uint32_t aDO = aQ + C::kQTile;
#pragma unroll
        for (int kk = 0; kk < DQK / 16; ++kk)
          umma_bf16(tmem + C::kColST, make_smem_desc(aK + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                    make_smem_desc(aQ + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024), idesc_st, kk > 0);
#pragma unroll
        for (int kk = 0; kk < DV / 16; ++kk)
          umma_bf16(tmem + C::kColDP, make_smem_desc(aV + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                    make_smem_desc(aDO + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024), idesc_st, kk > 0);
        tc_commit(&bars->st_full);
      }
      __syncwarp();
      return true;
    };
    if (ok) ok = issue_scores(0);
    for (int it = 0; it < n_iters && ok; ++it) {
      const int s = it % C::kStages;
      if (!mbar_wait(&bars->p_ready, it & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitAttnTimeout, 244, jb, it);
        break;
      }
      if (!C::kAliasDq && it > 0 && !mbar_wait(&bars->dq_read, (it - 1) & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitAttnTimeout, 243, jb, it);
        break;
      }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t aQ = smem_u32(smem + C::kOffRing + s * C::kStageBytes);
        const uint32_t aDO = aQ + C::kQTile;
        // contraction over the 64 queries of the tile: four 16-query steps
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)
          umma_bf16(tmem + C::kColDV, make_smem_desc(aPT + k4 * 32, 16, 1024),
                    make_smem_desc(aDO + (cv0 / 64) * 8192 + k4 * 2048, 8192, 1024), idesc_dv, (it > 0 || k4 > 0));
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)
          umma_bf16(tmem + C::kColDK, make_smem_desc(aDST + k4 * 32, 16, 1024),
                    make_smem_desc(aQ + (ck0 / 64) * 8192 + k4 * 2048, 8192, 1024), idesc_dk, (it > 0 || k4 > 0));
        // dQ^T block(s): rows d0 .. d0+127 of this CTA's columns, contraction over the 128 keys
#pragma unroll
        for (int qb = 0; qb < C::kQBlks; ++qb) {
          const int d0 = ck0 + (qb == 0 ? 0 : C::NK - 128);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_bf16(tmem + C::kColDQ + qb * 64, make_smem_desc(aK + (d0 / 64) * 16384 + kk * 2048, 16384, 1024),
                      make_smem_desc(aDST + kk * 2048, 16384, 1024), idesc_dq, kk > 0);
        }
        tc_commit(&bars->dq_full);
        tc_commit(&bars->qdo_empty[s]);
      }
      __syncwarp();
      if (it + 1 < n_iters) {
        if (C::kAliasDq && !mbar_wait(&bars->dq_read, it & 1, abort_flag)) {
          if (lane == 0) report_status(a.status, kWaitAttnTimeout, 245, jb, it);
          break;
        }
        ok = issue_scores(it + 1);
      }
    }
  } else {
    const int q4 = warp & 3;
    const int half = (warp - 2) >> 2;    // which 32 of the 64 query columns this thread owns
    const int r = q4 * 32 + lane;        // key row inside the block; head-dim row when reading dQ^T
    const int tid = threadIdx.x - 64;    // 0..255
    const int kvpos = jb * 128 + r;
    const int c0 = half * 32;
    const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
    bool ok = true;
    auto stage_stats = [&](int jt) {
      const int hq_j = hkv * group + jt / nqi;
      const int q0_j = (i0 + jt % nqi) * 64;
      float* dst = stats + (jt & 1) * 128;
      if (tid < 128) {
        const int qi = tid & 63;
        const int qp = q0_j + qi;
        const int64_t si = (static_cast<int64_t>(b) * a.H + hq_j) * a.T + qp;
        if (tid < 64) dst[qi] = (qp < a.T) ? a.lse[si] : 0.f;
        else dst[64 + qi] = (qp < a.T) ? a.delta[si] * a.scale : 0.f;
      }
      mbar_arrive(&bars->stats_ready);
    };
    if (n_iters > 0) stage_stats(0);
    for (int it = 0; it < n_iters; ++it) {
      const int hq = hkv * group + it / nqi;
      const int q0 = (i0 + it % nqi) * 64;
      const float* st_lse = stats + (it & 1) * 128;
      const float* st_del = st_lse + 64;
      if (!mbar_wait(&bars->stats_ready, it & 1, abort_flag) || !mbar_wait(&bars->st_full, it & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitAttnTimeout, 246, jb, it);
        ok = false;
        break;
      }
      tc_fence_after();
      const bool need_mask = (a.causal && q0 < jb * 128 + 127) || (q0 + 64 > a.T) || ((jb + 1) * 128 > a.T);
      {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(tmem + C::kColST + c0 + lane_off, sv);
        tmem_ld_32x32(tmem + C::kColDP + c0 + lane_off, dv);
        tmem_ld_wait();
        uint32_t pp[16], dd[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(&st_lse[c0 + i]);
          const float4 d4 = *reinterpret_cast<const float4*>(&st_del[c0 + i]);
          const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, de[4] = {d4.x, d4.y, d4.z, d4.w};
          float p[4], ds[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            p[e] = exp2f(fmaf(__uint_as_float(sv[i + e]), a.scale_log2, -ls[e]));
            ds[e] = p[e] * fmaf(__uint_as_float(dv[i + e]), a.scale, -de[e]);
          }
          if (need_mask) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int qp = q0 + c0 + i + e;
              if (qp >= a.T || kvpos >= a.T || (a.causal && qp < kvpos)) {
                p[e] = 0.f;
                ds[e] = 0.f;
              }
            }
          }
          pp[i >> 1] = pack_bf16x2(p[0], p[1]);
          pp[(i >> 1) + 1] = pack_bf16x2(p[2], p[3]);
          dd[i >> 1] = pack_bf16x2(ds[0], ds[1]);
          dd[(i >> 1) + 1] = pack_bf16x2(ds[2], ds[3]);
        }
        store_chunk64(smem + C::kOffPT, r, c0, pp);
        store_chunk64(smem + C::kOffDST, r, c0, dd);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bars->p_ready);
      if (it + 1 < n_iters) stage_stats(it + 1);
      if (!mbar_wait(&bars->dq_full, it & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitAttnTimeout, 247, jb, it);
        ok = false;
        break;
      }
      tc_fence_after();
      // dQ^T: this thread holds head-dim row d of 32 queries; a warp's lanes are 32 consecutive d of one query,
      // so every reduction instruction covers one 128-byte line.
#pragma unroll
      for (int qb = 0; qb < C::kQBlks; ++qb) {
        const int d = ck0 + (qb == 0 ? 0 : C::NK - 128) + r;
        const bool mine = (qb == 0) || (r >= 256 - C::NK);   // second block: only rows past the first 128
        uint32_t v[32];
        tmem_ld_32x32(tmem + C::kColDQ + qb * 64 + c0 + lane_off, v);
        tmem_ld_wait();
        if (mine) {
          float* dq = a.dq_accum + (static_cast<int64_t>(b) * a.T + q0 + c0) * (static_cast<int64_t>(a.H) * DQK) +
                      hq * DQK + d;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (q0 + c0 + i < a.T)
              asm volatile("red.global.add.f32 [%0], %1;" ::"l"(dq + static_cast<int64_t>(i) * a.H * DQK),
                           "f"(__uint_as_float(v[i]))
                           : "memory");
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&bars->dq_read);
    }
    if (ok && n_iters > 0) {
      // The last dq_full commit also covered every dV / dK accumulation.
      tc_fence_after();
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* base = which == 0 ? a.dv : a.dk;
        const int64_t ld = which == 0 ? a.lddv : a.lddk;
        const uint32_t col = which == 0 ? C::kColDV : C::kColDK;
        const int width = which == 0 ? C::NV : C::NK;          // columns of this CTA
        const int hw = which == 0 ? DV : DQK;                  // head width in the output
        const int cfirst = which == 0 ? cv0 : ck0;
        const int per = width / 2;                             // columns per thread (two threads per key row)
#pragma unroll 1
        for (int cc = 0; cc < per / 32; ++cc) {
          const int c = half * per + cc * 32;
          uint32_t v[32];
          tmem_ld_32x32(tmem + col + c + lane_off, v);
          tmem_ld_wait();
          if (kvpos < a.T) {
            __nv_bfloat16* dst = base + static_cast<int64_t>(b * a.T + kvpos) * ld + hkv * hw + cfirst + c;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 pk = make_uint4(pack_bf16x2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])),
                                    pack_bf16x2(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3])),
                                    pack_bf16x2(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5])),
                                    pack_bf16x2(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7])));
              *reinterpret_cast<uint4*>(dst + i) = pk;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

template <int DQK, int DV, int NSPLIT>
cudaError_t wide_launch(const AttnTensors& t, const AttnShape& s, const __nv_bfloat16* dout, int64_t lddo,
                        const float* lse, const float* delta, float* dq_accum, __nv_bfloat16* dk, int64_t lddk,
                        __nv_bfloat16* dv, int64_t lddv, int* status, cudaStream_t stream) {
  using C = WCfg<DQK, DV, NSPLIT>;
  CUtensorMap tq, tk, tv, tdo;
  const uint64_t rows = static_cast<uint64_t>(s.B) * s.T;
  cudaError_t e;
  if ((e = encode_tma_2d(&tq, t.q, 2, static_cast<uint64_t>(s.H) * DQK, rows, t.ldq * 2, 64, 64)) != cudaSuccess)
    return e;
  if ((e = encode_tma_2d(&tk, t.k, 2, static_cast<uint64_t>(s.Hkv) * DQK, rows, t.ldk * 2, 64, 128)) != cudaSuccess)
    return e;
  if ((e = encode_tma_2d(&tv, t.v, 2, static_cast<uint64_t>(s.Hkv) * DV, rows, t.ldv * 2, 64, 128)) != cudaSuccess)
    return e;
  if ((e = encode_tma_2d(&tdo, dout, 2, static_cast<uint64_t>(s.H) * DV, rows, lddo * 2, 64, 64)) != cudaSuccess)
    return e;
  auto kernel = attn_bwd_wide_kernel<DQK, DV, NSPLIT>;
  static bool configured = false;
  if (!configured) {
    if ((e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem)) != cudaSuccess)
      return e;
    configured = true;
  }
  WArgs a{s.B, s.T, s.H, s.Hkv, s.scale, s.scale * kLog2eW, s.causal, lse, delta, dq_accum, dk, lddk, dv, lddv, status};
  dim3 grid(s.Hkv * NSPLIT, s.B, (s.T + 127) / 128);
  kernel<<<grid, kWThreads, C::kSmem, stream>>>(tq, tk, tv, tdo, a);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_attn_bwd_wide(const AttnTensors& t, const AttnShape& s, const __nv_bfloat16* dout, int64_t lddo,
                                 const float* lse, const float* delta, float* dq_accum, __nv_bfloat16* dk,
                                 int64_t lddk, __nv_bfloat16* dv, int64_t lddv, int* status, cudaStream_t stream) {
  if (s.H % s.Hkv != 0) return cudaErrorInvalidValue;
  const int dvw = s.Dv > 0 ? s.Dv : s.D;
  if (s.D == 256 && dvw == 256)
    return wide_launch<256, 256, 2>(t, s, dout, lddo, lse, delta, dq_accum, dk, lddk, dv, lddv, status, stream);
  if (s.D == 192 && dvw == 128)
    return wide_launch<192, 128, 1>(t, s, dout, lddo, lse, delta, dq_accum, dk, lddk, dv, lddv, status, stream);
  return cudaErrorInvalidValue;
}

}  // namespace b200
