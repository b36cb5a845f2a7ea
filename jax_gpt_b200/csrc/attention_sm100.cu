// Flash attention for sm_100a on tcgen05 tensor cores with TMEM accumulators.
//
// Forward: one CTA per (128-query block, head, batch). Warp 0 streams K/V tiles with TMA,
// warp 1 issues S = Q K^T and O_j = P V into TMEM, warps 2..5 own one query row per thread:
// they read S from TMEM, do the online softmax without any cross-thread traffic, hand P back
// through 128B-swizzled shared memory and keep the running output in registers. Two CTAs fit
// on an SM (112 KB shared memory, 256 TMEM columns each), so one CTA's softmax overlaps the
// other's MMAs.
//
// Backward: one CTA per (128-key block, kv head, batch) looping over the query blocks that
// see it. It works on the TRANSPOSED score tile S^T = K Q^T so that each thread owns a key
// row; P^T and dS^T go to shared memory once and serve three MMAs each through K-major and
// MN-major descriptors (dV += P^T dO, dK += dS^T Q, dQ = dS K) with no transposes in memory.
// dK/dV accumulate in TMEM across the whole loop; dQ tiles leave through fp32 reductions.
//
// Replaces the dense (B,H,T,S) score materialisation of the reference
// (jax_gpt/models/gpt2/model.py:167-176, jax_gpt/models/qwen35/gqa.py:103-119) and applies
// the causal rule q_pos >= k_pos on true positions.
#include "attention_sm100.cuh"

#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "tma_host.h"

namespace b200 {

namespace {

constexpr int kThreads = 320;  // TMA warp, MMA warp, 8 softmax warps
constexpr float kLog2e = 1.4426950408889634f;

struct FwdArgs {
  int B, T, Tk, H, Hkv;     // T queries and Tk keys per sequence
  int q_pos0;               // position of query 0 (causal rule: key position <= q_pos0 + query index)
  int kv_rows_b, kv_rows_h; // row of key 0 of (b, hkv) in the K / V matrices = b * kv_rows_b + hkv * kv_rows_h
  int k_col_h, v_col_h;     // first column of kv head hkv in K / V = hkv * {k,v}_col_h
  float scale_log2;
  int causal;
  __nv_bfloat16* out;
  int64_t ldo;
  float* lse;
  int* status;
};

// D: width of q and k heads; DV: width of v heads (MLA prefill uses 192 / 128).
template <int D, int DV>
struct FwdCfg {
  static constexpr int kQTile = 128 * D * 2;     // bytes of a 128 x D bf16 tile (Q and K)
  static constexpr int kVTile = 128 * DV * 2;
  static constexpr int kStageBytes = kQTile + kVTile;
  static constexpr int kPBytes = 128 * 128 * 2;
  static constexpr int kStages = (D + DV <= 256) ? 2 : 1;
  static constexpr int kOffK = kQTile;
  static constexpr int kOffP = kQTile + kStages * kStageBytes;
  static constexpr int kOffXchg = kOffP + kPBytes;  // bf16 [2][128] running-max exchange
  static constexpr int kOffBar = kOffXchg + 512;
  static constexpr int kSmem = kOffBar + 128;       // D = 64: 115328 B, two CTAs per SM
  static constexpr int kTmemCols = (128 + DV <= 256) ? 256 : 512;  // S [0,128), O [128, 128+DV)
};

struct FwdBars {
  uint64_t q_full, kv_full[2], kv_empty[2], s_full, p_ready, o_full, x_ready;
  uint32_t tmem_base;
  int abort_flag;
};

// Writes 32 consecutive bf16 values of row `r`, columns [c0, c0+32) of a 128 x 128 tile laid
// out as two K-major 128B-swizzled halves of 64 columns (the layout TMA would produce).
__device__ __forceinline__ void store_row_chunk_sw128(uint8_t* tile, int r, int c0, const uint32_t (&pk)[16]) {
  uint8_t* base = tile + (c0 >> 6) * 16384 + r * 128;
  const int chunk0 = (c0 & 63) >> 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int phys = (chunk0 + i) ^ (r & 7);
    *reinterpret_cast<uint4*>(base + phys * 16) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
  }
}

template <int D>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* m, uint64_t* bar, int col0, int row0) {
#pragma unroll
  for (int h = 0; h < D / 64; ++h) tma_load_2d(dst + h * 16384, m, bar, col0 + h * 64, row0);
}

template <int D, int DV>
__global__ void __launch_bounds__(kThreads, (D == 64) ? 2 : 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, const __grid_constant__ FwdArgs a) {
  using C = FwdCfg<D, DV>;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) report_status(a.status, kBadArgument, 1, 0, 0);
    return;
  }
  FwdBars* bars = reinterpret_cast<FwdBars*>(smem + C::kOffBar);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The query block is the slowest grid dimension and runs backwards: with a causal mask the CTAs with the most
  // key tiles are dispatched first over all heads and sequences, the short ones fill the tail of the launch.
  const int q_blk = gridDim.z - 1 - blockIdx.z;
  const int h = blockIdx.x, b = blockIdx.y;
  const int hkv = h / (a.H / a.Hkv);
  const int n_kv_all = (a.Tk + 127) / 128;
  const int n_kv = a.causal ? min((a.q_pos0 + q_blk * 128 + 127) / 128 + 1, n_kv_all) : n_kv_all;
  const int row0 = b * a.T + q_blk * 128;
  const int kv_row0 = b * a.kv_rows_b + hkv * a.kv_rows_h;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->kv_empty[s], 1);
    }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->p_ready, 256);
    mbar_init(&bars->o_full, 1);
    mbar_init(&bars->x_ready, 256);
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
  const uint32_t tmem = bars->tmem_base;
  uint8_t* sQ = smem;
  uint8_t* sP = smem + C::kOffP;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(&bars->q_full, C::kQTile);
      load_tile<D>(sQ, &tq, &bars->q_full, h * D, row0);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j % C::kStages;
        const uint32_t ph = (j / C::kStages) & 1;
        if (!mbar_wait(&bars->kv_empty[s], ph ^ 1, abort_flag)) {
          report_status(a.status, kWaitEmptyTimeout, 100, blockIdx.z, j);
          break;
        }
        uint8_t* sK = smem + C::kOffK + s * C::kStageBytes;
        mbar_arrive_expect_tx(&bars->kv_full[s], C::kStageBytes);
        load_tile<D>(sK, &tk, &bars->kv_full[s], hkv * a.k_col_h, kv_row0 + j * 128);
        load_tile<DV>(sK + C::kQTile, &tv, &bars->kv_full[s], hkv * a.v_col_h, kv_row0 + j * 128);
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc_s = make_idesc(128, 128, 0, 0, 1);
    constexpr uint32_t idesc_o = make_idesc(128, DV, 0, 1, 1);
    bool ok = mbar_wait(&bars->q_full, 0, abort_flag);
    if (!ok && lane == 0) report_status(a.status, kWaitFullTimeout, 101, blockIdx.z, 0);
    for (int j = 0; j < n_kv && ok; ++j) {
      const int s = j % C::kStages;
      const uint32_t ph = (j / C::kStages) & 1;
      if (!mbar_wait(&bars->kv_full[s], ph, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitFullTimeout, 102, blockIdx.z, j);
        break;
      }
      tc_fence_after();
      const uint32_t aQ = smem_u32(sQ);
      const uint32_t aK = smem_u32(smem + C::kOffK + s * C::kStageBytes);
      const uint32_t aV = aK + C::kQTile;
      if (lane == 0) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tmem, make_smem_desc(aQ + off, 16, 1024), make_smem_desc(aK + off, 16, 1024), idesc_s, kk > 0);
        }
        tc_commit(&bars->s_full);
      }
      __syncwarp();
      if (!mbar_wait(&bars->p_ready, j & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitAttnTimeout, 103, blockIdx.z, j);
        break;
      }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t aP = smem_u32(sP);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tmem + 128, make_smem_desc(aP + off, 16, 1024), make_smem_desc(aV + kk * 2048, 16384, 1024),
                    idesc_o, kk > 0);
        }
        tc_commit(&bars->o_full);
        tc_commit(&bars->kv_empty[s]);
      }
      __syncwarp();
    }
  } else {
    // Eight softmax warps: warps w and w+4 share a TMEM lane quarter (the same 32 query rows)
    // and split the 128 score columns and the D output columns in halves. The two threads of a
    // row agree on the running maximum through a bf16 value in shared memory (any common
    // reference works for the online softmax as long as both use the same one).
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = q * 32 + lane;  // query row inside the block == TMEM lane
    const int qi = q_blk * 128 + r;      // query index inside the sequence
    const int qpos = a.q_pos0 + qi;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    __nv_bfloat16* xchg = reinterpret_cast<__nv_bfloat16*>(smem + C::kOffXchg);  // [2][128]
    constexpr int DH = DV / 2;
    float m = -INFINITY, l = 0.f;
    float o[DH];
#pragma unroll
    for (int i = 0; i < DH; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait(&bars->s_full, j & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitAttnTimeout, 104, blockIdx.z, j);
        ok = false;
        break;
      }
      tc_fence_after();
      const bool need_mask = (a.causal && j * 128 + 127 > a.q_pos0 + q_blk * 128) || ((j + 1) * 128 > a.Tk);
      const int kv0 = j * 128 + half * 64;
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem + half * 64 + c * 32 + lane_off, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = __uint_as_float(v[i]);   // the (positive) softmax scale is applied to the maximum once, below
          if (need_mask) {
            const int kvpos = kv0 + c * 32 + i;
            if (kvpos >= a.Tk || (a.causal && kvpos > qpos)) s = -INFINITY;
          }
          mx = fmaxf(mx, s);
        }
      }
      mx *= a.scale_log2;
      const __nv_bfloat16 mine = __float2bfloat16(mx);
      xchg[half * 128 + r] = mine;
      mbar_arrive(&bars->x_ready);
      if (!mbar_wait(&bars->x_ready, j & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitAttnTimeout, 106, blockIdx.z, j);
        ok = false;
        break;
      }
      const float other = __bfloat162float(xchg[(half ^ 1) * 128 + r]);
      mx = fmaxf(fmaxf(__bfloat162float(mine), other), m);
      const float mref = (mx == -INFINITY) ? 0.f : mx;
      const float alpha = exp2f(m - mref);  // m == -inf -> 0
      float rs = 0.f;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem + half * 64 + c * 32 + lane_off, v);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float s0 = fmaf(__uint_as_float(v[i]), a.scale_log2, -mref), s1 = fmaf(__uint_as_float(v[i + 1]), a.scale_log2, -mref);
          if (need_mask) {
            const int kvpos = kv0 + c * 32 + i;
            if (kvpos >= a.Tk || (a.causal && kvpos > qpos)) s0 = -INFINITY;
            if (kvpos + 1 >= a.Tk || (a.causal && kvpos + 1 > qpos)) s1 = -INFINITY;
          }
          const float p0 = exp2f(s0), p1 = exp2f(s1);
          rs += p0 + p1;
          pk[i >> 1] = pack_bf16x2(p0, p1);
        }
        store_row_chunk_sw128(sP, r, half * 64 + c * 32, pk);
      }
      l = l * alpha + rs;
      m = mx;
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bars->p_ready);
      if (!mbar_wait(&bars->o_full, j & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitAttnTimeout, 105, blockIdx.z, j);
        ok = false;
        break;
      }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem + 128 + half * DH + c * 32 + lane_off, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = o[c * 32 + i] * alpha + __uint_as_float(v[i]);
      }
      tc_fence_before();
    }
    if (ok) {
      // total row sum = sum of the two halves; the P tile is free after the last o_full
      float* lsum = reinterpret_cast<float*>(sP);
      lsum[half * 128 + r] = l;
      mbar_arrive(&bars->x_ready);
      if (!mbar_wait(&bars->x_ready, n_kv & 1, abort_flag)) ok = false;
      if (ok) l += lsum[(half ^ 1) * 128 + r];
    }
    if (ok && qi < a.T) {
      const float inv = (l > 0.f) ? 1.f / l : 0.f;
      __nv_bfloat16* orow = a.out + static_cast<int64_t>(b * a.T + qi) * a.ldo + h * DV + half * DH;
#pragma unroll
      for (int i = 0; i < DH; i += 8) {
        uint4 pk = make_uint4(pack_bf16x2(o[i] * inv, o[i + 1] * inv), pack_bf16x2(o[i + 2] * inv, o[i + 3] * inv),
                              pack_bf16x2(o[i + 4] * inv, o[i + 5] * inv), pack_bf16x2(o[i + 6] * inv, o[i + 7] * inv));
        *reinterpret_cast<uint4*>(orow + i) = pk;
      }
      if (a.lse != nullptr && half == 0) a.lse[(static_cast<int64_t>(b) * a.H + h) * a.T + qi] = m + log2f(l);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, C::kTmemCols);
  }
}

// ------------------------------------ backward ------------------------------------------
struct BwdArgs {
  int B, T, H, Hkv;
  float scale, scale_log2;
  int causal;
  const float* lse;
  const float* delta;
  float* dq_accum;  // [B*T, H*D] fp32
  __nv_bfloat16* dk;
  int64_t lddk;
  __nv_bfloat16* dv;
  int64_t lddv;
  int* status;
};

template <int D>
struct BwdCfg {
  static constexpr int kTile = 128 * D * 2;
  static constexpr int kStages = (D == 64) ? 2 : 1;
  static constexpr int kOffK = 0;
  static constexpr int kOffV = kTile;
  static constexpr int kOffRing = 2 * kTile;                      // stages of {Q_i, dO_i}
  static constexpr int kOffPT = kOffRing + kStages * 2 * kTile;   // P^T  128 x 128 bf16
  static constexpr int kOffDST = kOffPT + 32768;                  // dS^T 128 x 128 bf16
  static constexpr int kOffStats = kOffDST + 32768;               // lse / delta, 2 x 2 x 128 fp32
  static constexpr int kOffBar = kOffStats + 2048;
  static constexpr int kSmem = kOffBar + 256;
  static constexpr int kTmemCols = 512;  // S^T [0,128), dP^T [128,256), dV [256,256+D), dK [384,384+D), dQ [448,512) or on S^T
};

struct BwdBars {
  uint64_t kv_full, qdo_full[2], qdo_empty[2], st_full, p_ready, dq_full, dq_read, stats_ready;
  uint32_t tmem_base;
  int abort_flag;
};

constexpr int kBwdThreads = 320;  // TMA warp, MMA warp, 8 compute warps (two per TMEM lane quarter)

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                const __grid_constant__ BwdArgs a) {
  using C = BwdCfg<D>;
  // D == 64 leaves room for a private dQ accumulator, so the next score tile can be issued
  // while this one's dQ is still being drained; D == 128 re-uses the score columns for dQ.
  constexpr bool kAliasDq = (D != 64);
  constexpr uint32_t kColDq = kAliasDq ? 0u : 448u;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) report_status(a.status, kBadArgument, 2, 0, 0);
    return;
  }
  BwdBars* bars = reinterpret_cast<BwdBars*>(smem + C::kOffBar);
  volatile int* abort_flag = &bars->abort_flag;
  float* stats = reinterpret_cast<float*>(smem + C::kOffStats);  // [buf][0: lse, 1: delta][128]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jb = blockIdx.z;  // key block, slowest grid dimension: block 0 (seen by every query block) goes first
  const int hkv = blockIdx.x, b = blockIdx.y;
  const int group = a.H / a.Hkv;
  const int n_q = (a.T + 127) / 128;
  const int i0 = a.causal ? jb : 0;
  const int nqi = n_q - i0;
  const int n_iters = group * nqi;

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
    tmem_alloc(&bars->tmem_base, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  const int kv_row0 = b * a.T + jb * 128;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(&bars->kv_full, 2 * C::kTile);
      load_tile<D>(smem + C::kOffK, &tk, &bars->kv_full, hkv * D, kv_row0);
      load_tile<D>(smem + C::kOffV, &tv, &bars->kv_full, hkv * D, kv_row0);
      for (int it = 0; it < n_iters; ++it) {
        const int s = it % C::kStages;
        const uint32_t ph = (it / C::kStages) & 1;
        if (!mbar_wait(&bars->qdo_empty[s], ph ^ 1, abort_flag)) {
          report_status(a.status, kWaitEmptyTimeout, 200, blockIdx.z, it);
          break;
        }
        const int hq = hkv * group + it / nqi;
        const int qrow0 = b * a.T + (i0 + it % nqi) * 128;
        uint8_t* st = smem + C::kOffRing + s * 2 * C::kTile;
        mbar_arrive_expect_tx(&bars->qdo_full[s], 2 * C::kTile);
        load_tile<D>(st, &tq, &bars->qdo_full[s], hq * D, qrow0);
        load_tile<D>(st + C::kTile, &tdo, &bars->qdo_full[s], hq * D, qrow0);
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc_st = make_idesc(128, 128, 0, 0, 1);  // K-major x K-major
    constexpr uint32_t idesc_kn = make_idesc(128, D, 0, 1, 1);    // A K-major, B MN-major
    constexpr uint32_t idesc_nn = make_idesc(128, D, 1, 1, 1);    // A MN-major, B MN-major
    bool ok = mbar_wait(&bars->kv_full, 0, abort_flag);
    if (!ok && lane == 0) report_status(a.status, kWaitFullTimeout, 201, blockIdx.z, 0);
    const uint32_t aK = smem_u32(smem + C::kOffK), aV = smem_u32(smem + C::kOffV);
    const uint32_t aPT = smem_u32(smem + C::kOffPT), aDST = smem_u32(smem + C::kOffDST);
    // S^T = K Q^T and dP^T = V dO^T of iteration `it` (its Q / dO stage must have landed).
    auto issue_scores = [&](int it) -> bool {
      const int s = it % C::kStages;
      const uint32_t ph = (it / C::kStages) & 1;
      if (!mbar_wait(&bars->qdo_full[s], ph, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitFullTimeout, 202, blockIdx.z, it);
        return false;
      }
      tc_fence_after();
      const uint32_t aQ = smem_u32(smem + C::kOffRing + s * 2 * C::kTile);
      const uint32_t aDO = aQ + C::kTile;
      if (lane == 0) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tmem, make_smem_desc(aK + off, 16, 1024), make_smem_desc(aQ + off, 16, 1024), idesc_st, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tmem + 128, make_smem_desc(aV + off, 16, 1024), make_smem_desc(aDO + off, 16, 1024), idesc_st,
                    kk > 0);
        }
        tc_commit(&bars->st_full);
      }
      __syncwarp();
      return true;
    };
    if (ok && n_iters > 0) ok = issue_scores(0);
    for (int it = 0; it < n_iters && ok; ++it) {
      const int s = it % C::kStages;
      if (!mbar_wait(&bars->p_ready, it & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitAttnTimeout, 204, blockIdx.z, it);
        break;
      }
      tc_fence_after();
      const uint32_t aQ = smem_u32(smem + C::kOffRing + s * 2 * C::kTile);
      const uint32_t aDO = aQ + C::kTile;
      if (lane == 0) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {  // contraction over the 128 query rows
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tmem + 256, make_smem_desc(aPT + off, 16, 1024), make_smem_desc(aDO + kk * 2048, 16384, 1024),
                    idesc_kn, (it > 0 || kk > 0));
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tmem + 384, make_smem_desc(aDST + off, 16, 1024), make_smem_desc(aQ + kk * 2048, 16384, 1024),
                    idesc_kn, (it > 0 || kk > 0));
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {  // contraction over the 128 key rows: dQ = dS K
          umma_bf16(tmem + kColDq, make_smem_desc(aDST + kk * 2048, 16384, 1024),
                    make_smem_desc(aK + kk * 2048, 16384, 1024), idesc_nn, kk > 0);
        }
        tc_commit(&bars->dq_full);
        tc_commit(&bars->qdo_empty[s]);
      }
      __syncwarp();
      if (it + 1 < n_iters) {
        if (kAliasDq && !mbar_wait(&bars->dq_read, it & 1, abort_flag)) {
          if (lane == 0) report_status(a.status, kWaitAttnTimeout, 203, blockIdx.z, it);
          break;
        }
        // P^T / dS^T of `it` are only re-written after the compute warps have seen dq_full(it),
        // i.e. after the MMAs above have finished reading them.
        ok = issue_scores(it + 1);
      }
    }
  } else {
    const int q4 = warp & 3;
    const int half = (warp - 2) >> 2;    // which 64 score columns (and which half of D) this thread owns
    const int r = q4 * 32 + lane;        // key row inside the block (and query row when reading dQ)
    const int tid = threadIdx.x - 64;    // 0..255
    const int kvpos = jb * 128 + r;
    const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
    bool ok = true;
    // Per-query statistics (lse, delta) of iteration `jt` go to the shared buffer jt & 1. They are staged one
    // iteration ahead (right after the element-wise part of the previous iteration), so their global-load
    // latency is off the critical path; a thread only stages jt + 1 after it has seen stats_ready(jt), i.e.
    // after every thread has finished reading buffer (jt - 1) & 1.
    auto stage_stats = [&](int jt) {
      const int hq_j = hkv * group + jt / nqi;
      const int q0_j = (i0 + jt % nqi) * 128;
      float* dst = stats + (jt & 1) * 256;
      const int qi = tid & 127;
      const int qp = q0_j + qi;
      const int64_t si = (static_cast<int64_t>(b) * a.H + hq_j) * a.T + qp;
      if (tid < 128) dst[qi] = (qp < a.T) ? a.lse[si] : 0.f;
      else dst[128 + qi] = (qp < a.T) ? a.delta[si] : 0.f;
      mbar_arrive(&bars->stats_ready);
    };
    if (n_iters > 0) stage_stats(0);
    for (int it = 0; it < n_iters; ++it) {
      const int hq = hkv * group + it / nqi;
      const int iq = i0 + it % nqi;
      const int q0 = iq * 128;
      float* st_lse = stats + (it & 1) * 256;
      float* st_del = st_lse + 128;
      // bounded rendezvous of the 256 compute threads on the per-query statistics
      if (!mbar_wait(&bars->stats_ready, it & 1, abort_flag) || !mbar_wait(&bars->st_full, it & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitAttnTimeout, 205, blockIdx.z, it);
        ok = false;
        break;
      }
      tc_fence_after();
      const bool need_mask = (a.causal && iq == jb) || ((iq + 1) * 128 > a.T) || ((jb + 1) * 128 > a.T);
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(tmem + c * 32 + lane_off, sv);
        tmem_ld_32x32(tmem + 128 + c * 32 + lane_off, dv);
        tmem_ld_wait();
        uint32_t pp[16], dd[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          // per-query statistics of four consecutive columns with one 16-byte shared-memory load each
          const float4 l4 = *reinterpret_cast<const float4*>(&st_lse[c * 32 + i]);
          const float4 d4 = *reinterpret_cast<const float4*>(&st_del[c * 32 + i]);
          const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, de[4] = {d4.x, d4.y, d4.z, d4.w};
          float p[4], ds[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int qi = c * 32 + i + e;
            bool valid = true;
            if (need_mask) {
              const int qp = q0 + qi;
              valid = !(qp >= a.T || kvpos >= a.T || (a.causal && qp < kvpos));
            }
            const float pe = valid ? exp2f(fmaf(__uint_as_float(sv[i + e]), a.scale_log2, -ls[e])) : 0.f;
            p[e] = pe;
            ds[e] = valid ? (pe * a.scale) * (__uint_as_float(dv[i + e]) - de[e]) : 0.f;
          }
          pp[i >> 1] = pack_bf16x2(p[0], p[1]);
          pp[(i >> 1) + 1] = pack_bf16x2(p[2], p[3]);
          dd[i >> 1] = pack_bf16x2(ds[0], ds[1]);
          dd[(i >> 1) + 1] = pack_bf16x2(ds[2], ds[3]);
        }
        store_row_chunk_sw128(smem + C::kOffPT, r, c * 32, pp);
        store_row_chunk_sw128(smem + C::kOffDST, r, c * 32, dd);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bars->p_ready);
      if (it + 1 < n_iters) stage_stats(it + 1);
      if (!mbar_wait(&bars->dq_full, it & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitAttnTimeout, 206, blockIdx.z, it);
        ok = false;
        break;
      }
      tc_fence_after();
      {
        const int qp = q0 + r;
        float* dq = a.dq_accum + (static_cast<int64_t>(b) * a.T + qp) * (static_cast<int64_t>(a.H) * D) + hq * D;
#pragma unroll 1
        for (int cc = 0; cc < D / 64; ++cc) {
          const int c = half * (D / 64) + cc;
          uint32_t v[32];
          tmem_ld_32x32(tmem + kColDq + c * 32 + lane_off, v);
          tmem_ld_wait();
          if (qp < a.T) {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dq + c * 32 + i),
                           "f"(__uint_as_float(v[i])), "f"(__uint_as_float(v[i + 1])), "f"(__uint_as_float(v[i + 2])),
                           "f"(__uint_as_float(v[i + 3]))
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
        const uint32_t col = which == 0 ? 256 : 384;
#pragma unroll 1
        for (int cc = 0; cc < D / 64; ++cc) {
          const int c = half * (D / 64) + cc;
          uint32_t v[32];
          tmem_ld_32x32(tmem + col + c * 32 + lane_off, v);
          tmem_ld_wait();
          if (kvpos < a.T) {
            __nv_bfloat16* dst = base + static_cast<int64_t>(b * a.T + kvpos) * ld + hkv * D + c * 32;
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
    tmem_dealloc(tmem, C::kTmemCols);
  }
}

// delta[b, h, t] = sum_d dO[b, t, h, d] * O[b, t, h, d]; one warp per token row, 16-byte loads, the D / 8 lanes
// that cover one head reduce among themselves.
template <int D>
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, int64_t ldo,
                                  const __nv_bfloat16* __restrict__ dout, int64_t lddo, float* __restrict__ delta,
                                  int B, int T, int H) {
  constexpr int kLanesPerHead = D / 8;   // 8 (D = 64) or 16 (D = 128): divides 32
  const int64_t row = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= static_cast<int64_t>(B) * T) return;
  const uint4* po = reinterpret_cast<const uint4*>(o + row * ldo);
  const uint4* pd = reinterpret_cast<const uint4*>(dout + row * lddo);
  const int nvec = H * kLanesPerHead;
  const int64_t bidx = row / T, t = row % T;
  for (int i0 = 0; i0 < nvec; i0 += 32) {
    const int i = i0 + lane;
    float s = 0.f;
    if (i < nvec) {
      const uint4 x = po[i], y = pd[i];
      const float2 x0 = unpack_bf16x2(x.x), x1 = unpack_bf16x2(x.y), x2 = unpack_bf16x2(x.z), x3 = unpack_bf16x2(x.w);
      const float2 y0 = unpack_bf16x2(y.x), y1 = unpack_bf16x2(y.y), y2 = unpack_bf16x2(y.z), y3 = unpack_bf16x2(y.w);
      s = x0.x * y0.x + x0.y * y0.y + x1.x * y1.x + x1.y * y1.y + x2.x * y2.x + x2.y * y2.y + x3.x * y3.x + x3.y * y3.y;
    }
#pragma unroll
    for (int off = kLanesPerHead / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (i < nvec && (lane % kLanesPerHead) == 0) delta[(bidx * H + i / kLanesPerHead) * T + t] = s;
  }
}

__global__ void cast_rows_kernel(const float* __restrict__ src, int64_t lds, __nv_bfloat16* __restrict__ dst,
                                 int64_t ldd, int M, int N) {
  const int n4 = N / 4;
  const int64_t total = static_cast<int64_t>(M) * n4;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / n4;
    const int c = static_cast<int>(i % n4) * 4;
    const float4 v = *reinterpret_cast<const float4*>(src + r * lds + c);
    uint2 pk = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
    *reinterpret_cast<uint2*>(dst + r * ldd + c) = pk;
  }
}

// Elementwise core of the recomputed attention backward (head widths without a tensor-core backward kernel):
// scores and dP = dO V^T come from batched library matmuls as bf16 [rows, kv]; this pass turns them IN PLACE into
// P = exp2(scale_log2 * s - lse) (zero above the causal diagonal) and dS = P * (dP - delta) * scale, eight columns
// per thread. Row r holds query position q0 + r % c (c positions per head, heads one after the other).
__global__ void attn_bwd_probs_kernel(__nv_bfloat16* __restrict__ s, __nv_bfloat16* __restrict__ dp,
                                      const float* __restrict__ lse, const float* __restrict__ delta, int64_t rows,
                                      int kv, int c, int q0, float scale_log2, float scale, int causal) {
  const int vec = kv >> 3;
  const int64_t total = rows * vec;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec;
    const int col0 = static_cast<int>(i - r * vec) << 3;
    const float l = lse[r], d = delta[r];
    const int qpos = q0 + static_cast<int>(r % c);
    uint4* sp = reinterpret_cast<uint4*>(s + r * kv + col0);
    uint4* dpp = reinterpret_cast<uint4*>(dp + r * kv + col0);
    const uint4 sv = *sp, dv = *dpp;
    const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w}, dw[4] = {dv.x, dv.y, dv.z, dv.w};
    uint32_t po[4], dso[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = unpack_bf16x2(sw[e]), g = unpack_bf16x2(dw[e]);
      float p0 = exp2f(fmaf(a.x, scale_log2, -l)), p1 = exp2f(fmaf(a.y, scale_log2, -l));
      if (causal) {
        if (col0 + 2 * e > qpos) p0 = 0.f;
        if (col0 + 2 * e + 1 > qpos) p1 = 0.f;
      }
      po[e] = pack_bf16x2(p0, p1);
      dso[e] = pack_bf16x2(p0 * (g.x - d) * scale, p1 * (g.y - d) * scale);
    }
    *sp = make_uint4(po[0], po[1], po[2], po[3]);
    *dpp = make_uint4(dso[0], dso[1], dso[2], dso[3]);
  }
}

cudaError_t make_map(CUtensorMap* m, const __nv_bfloat16* p, int64_t ld, int rows, int cols) {
  return encode_tma_2d(m, p, 2, cols, rows, ld * 2, 64, 128);
}

template <int D, int DV>
cudaError_t fwd_launch(const AttnTensors& t, const AttnShape& s, const AttnKvLayout& kv, __nv_bfloat16* out,
                       int64_t ldo, float* lse, int* status, cudaStream_t stream) {
  using C = FwdCfg<D, DV>;
  CUtensorMap tq, tk, tv;
  const int rows = s.B * s.T;
  cudaError_t e;
  if ((e = make_map(&tq, t.q, t.ldq, rows, s.H * D)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tk, t.k, 2, kv.k_cols, kv.rows, t.ldk * 2, 64, 128)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tv, t.v, 2, kv.v_cols, kv.rows, t.ldv * 2, 64, 128)) != cudaSuccess) return e;
  auto kernel = attn_fwd_kernel<D, DV>;
  static bool configured = false;
  if (!configured) {
    if ((e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem)) != cudaSuccess)
      return e;
    configured = true;
  }
  FwdArgs a{s.B, s.T, kv.Tk, s.H, s.Hkv, kv.q_pos0, kv.rows_b, kv.rows_h, kv.k_col_h, kv.v_col_h,
            s.scale * kLog2e, s.causal, out, ldo, lse, status};
  dim3 grid(s.H, s.B, (s.T + 127) / 128);
  kernel<<<grid, kThreads, C::kSmem, stream>>>(tq, tk, tv, a);
  return cudaGetLastError();
}

template <int D>
cudaError_t bwd_launch(const AttnTensors& t, const AttnShape& s, const __nv_bfloat16* out, int64_t ldo,
                       const __nv_bfloat16* dout, int64_t lddo, const float* lse, float* delta, float* dq_accum,
                       __nv_bfloat16* dk, int64_t lddk, __nv_bfloat16* dv, int64_t lddv, int* status,
                       cudaStream_t stream) {
  using C = BwdCfg<D>;
  CUtensorMap tq, tk, tv, tdo;
  const int rows = s.B * s.T;
  cudaError_t e;
  if ((e = make_map(&tq, t.q, t.ldq, rows, s.H * D)) != cudaSuccess) return e;
  if ((e = make_map(&tk, t.k, t.ldk, rows, s.Hkv * D)) != cudaSuccess) return e;
  if ((e = make_map(&tv, t.v, t.ldv, rows, s.Hkv * D)) != cudaSuccess) return e;
  if ((e = make_map(&tdo, dout, lddo, rows, s.H * D)) != cudaSuccess) return e;
  {
    const int64_t warps = static_cast<int64_t>(rows);
    const int blocks = static_cast<int>((warps * 32 + 255) / 256);
    attn_delta_kernel<D><<<blocks, 256, 0, stream>>>(out, ldo, dout, lddo, delta, s.B, s.T, s.H);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
  }
  if (D == 64) {
    // pipelined half-tile kernel unless the single-stage one is asked for (B200_ATTN_BWD=1stage)
    static const bool one_stage = [] {
      const char* ev = getenv("B200_ATTN_BWD");
      return ev != nullptr && ev[0] == '1';
    }();
    if (!one_stage)
      return launch_attn_bwd2_d64(t, s, dout, lddo, lse, delta, dq_accum, dk, lddk, dv, lddv, status, stream);
  }
  auto kernel = attn_bwd_kernel<D>;
  static bool configured = false;
  if (!configured) {
    if ((e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem)) != cudaSuccess)
      return e;
    configured = true;
  }
  BwdArgs a{s.B, s.T, s.H, s.Hkv, s.scale, s.scale * kLog2e, s.causal, lse, delta, dq_accum, dk, lddk, dv, lddv, status};
  dim3 grid(s.Hkv, s.B, (s.T + 127) / 128);
  kernel<<<grid, kBwdThreads, C::kSmem, stream>>>(tq, tk, tv, tdo, a);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_attn_fwd_kv(const AttnTensors& t, const AttnShape& s, const AttnKvLayout& kv, __nv_bfloat16* out,
                               int64_t ldo, float* lse, int* status, cudaStream_t stream) {
  if (s.H % s.Hkv != 0) return cudaErrorInvalidValue;
  const int dv = s.Dv > 0 ? s.Dv : s.D;
  if (s.D == 64 && dv == 64) {
    // two-tile kernel unless the single-tile one is asked for (B200_ATTN_FWD=1tile: comparisons, fallback)
    static const bool one_tile = [] {
      const char* e = getenv("B200_ATTN_FWD");
      return e != nullptr && e[0] == '1';
    }();
    if (!one_tile) return launch_attn_fwd2_d64(t, s, kv, out, ldo, lse, status, stream);
    return fwd_launch<64, 64>(t, s, kv, out, ldo, lse, status, stream);
  }
  if (s.D == 128 && dv == 128) return fwd_launch<128, 128>(t, s, kv, out, ldo, lse, status, stream);
  if (s.D == 256 && dv == 256) return fwd_launch<256, 256>(t, s, kv, out, ldo, lse, status, stream);
  if (s.D == 192 && dv == 128) return fwd_launch<192, 128>(t, s, kv, out, ldo, lse, status, stream);
  return cudaErrorInvalidValue;
}

cudaError_t launch_attn_fwd(const AttnTensors& t, const AttnShape& s, __nv_bfloat16* out, int64_t ldo, float* lse,
                            int* status, cudaStream_t stream) {
  const int dv = s.Dv > 0 ? s.Dv : s.D;
  AttnKvLayout kv;
  kv.Tk = s.T;
  kv.q_pos0 = 0;
  kv.rows_b = s.T;
  kv.rows_h = 0;
  kv.k_col_h = s.D;
  kv.v_col_h = dv;
  kv.rows = static_cast<uint64_t>(s.B) * s.T;
  kv.k_cols = static_cast<uint64_t>(s.Hkv) * s.D;
  kv.v_cols = static_cast<uint64_t>(s.Hkv) * dv;
  return launch_attn_fwd_kv(t, s, kv, out, ldo, lse, status, stream);
}

cudaError_t launch_attn_bwd(const AttnTensors& t, const AttnShape& s, const __nv_bfloat16* out, int64_t ldo,
                            const __nv_bfloat16* dout, int64_t lddo, const float* lse, float* delta, float* dq_accum,
                            __nv_bfloat16* dk, int64_t lddk, __nv_bfloat16* dv, int64_t lddv, int* status,
                            cudaStream_t stream) {
  if (s.H % s.Hkv != 0) return cudaErrorInvalidValue;
  if (s.D == 64)
    return bwd_launch<64>(t, s, out, ldo, dout, lddo, lse, delta, dq_accum, dk, lddk, dv, lddv, status, stream);
  if (s.D == 128)
    return bwd_launch<128>(t, s, out, ldo, dout, lddo, lse, delta, dq_accum, dk, lddk, dv, lddv, status, stream);
  return cudaErrorInvalidValue;
}

cudaError_t launch_attn_delta(const __nv_bfloat16* out, int64_t ldo, const __nv_bfloat16* dout, int64_t lddo,
                              float* delta, int B, int T, int H, int Dv, cudaStream_t stream) {
  const int64_t rows = static_cast<int64_t>(B) * T;
  const int blocks = static_cast<int>((rows * 32 + 255) / 256);
  switch (Dv) {
    case 64: attn_delta_kernel<64><<<blocks, 256, 0, stream>>>(out, ldo, dout, lddo, delta, B, T, H); break;
    case 128: attn_delta_kernel<128><<<blocks, 256, 0, stream>>>(out, ldo, dout, lddo, delta, B, T, H); break;
    case 256: attn_delta_kernel<256><<<blocks, 256, 0, stream>>>(out, ldo, dout, lddo, delta, B, T, H); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_cast_rows_f32_bf16(const float* src, int64_t lds, __nv_bfloat16* dst, int64_t ldd, int M, int N,
                                      cudaStream_t stream) {
  if (N % 4 != 0) return cudaErrorInvalidValue;
  const int64_t total = static_cast<int64_t>(M) * (N / 4);
  const int grid = static_cast<int>(std::min<int64_t>((total + 255) / 256, 148 * 16));
  cast_rows_kernel<<<grid, 256, 0, stream>>>(src, lds, dst, ldd, M, N);
  return cudaGetLastError();
}

cudaError_t launch_attn_bwd_probs(__nv_bfloat16* s, __nv_bfloat16* dp, const float* lse, const float* delta,
                                  int64_t rows, int kv, int c, int q0, float scale, int causal, cudaStream_t stream) {
  if (kv % 8 != 0 || rows <= 0 || c <= 0) return cudaErrorInvalidValue;
  const int64_t total = rows * (kv / 8);
  const int grid = static_cast<int>(std::min<int64_t>((total + 255) / 256, 148 * 32));
  attn_bwd_probs_kernel<<<grid, 256, 0, stream>>>(s, dp, lse, delta, rows, kv, c, q0, scale * kLog2e, scale, causal);
  return cudaGetLastError();
}

}  // namespace b200
