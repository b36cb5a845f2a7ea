// Flash attention forward for head width 64 on tcgen05: TWO 128-row query tiles per CTA that take turns on the
// tensor core and on the exponential unit.
//
// One CTA owns 256 consecutive queries of one (batch, head). Warp 0 streams K and V tiles with TMA through two
// independent three-deep rings, warp 1 issues every MMA, warps 2..5 are the softmax group of query tile 0 and
// warps 6..9 the group of query tile 1. A softmax thread owns one whole score row (128 columns of TMEM), so the
// running maximum and sum never leave its registers and no two threads have to agree on anything. The MMA warp
// interleaves the two tiles (S0, S1, P0 V, S0', P1 V, S1', ...): while one group turns its scores into
// probabilities, the tensor core works on the other tile, and the K / V tiles in shared memory are read for 256
// queries instead of 128.
//
// Keys and values may come from a token-major activation ([B*Tk, Hkv*D]) or straight from a cache laid out as
// (B, Hkv, max_len, D); queries sit at positions q_pos0 + i, which makes the same kernel the prefill-with-cache
// path (the reference attends over the whole zero-padded cache and masks: jax_gpt/models/qwen35/gqa.py:88-119).
#include "attention_sm100.cuh"

#include "common.cuh"
#include "tma_host.h"

namespace b200 {

namespace {

constexpr int kThreads2 = 320;  // TMA warp, MMA warp, 2 x 4 softmax warps
constexpr float kLog2e2 = 1.4426950408889634f;
constexpr int kRing = 3;

struct Fwd2Args {
  int B, Tq, Tk, H, Hkv;
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

template <int D>
struct Fwd2Cfg {
  static constexpr int kTile = 128 * D * 2;          // one 128 x D bf16 tile
  static constexpr int kPBytes = 128 * 128 * 2;
  static constexpr int kOffQ = 0;                    // Q0, Q1
  static constexpr int kOffK = 2 * kTile;            // ring of K tiles
  static constexpr int kOffV = kOffK + kRing * kTile;
  static constexpr int kOffP = kOffV + kRing * kTile;  // P0, P1
  static constexpr int kOffBar = kOffP + 2 * kPBytes;
  static constexpr int kSmem = kOffBar + 256;
  static constexpr int kColS = 0;                    // S0 [0,128), S1 [128,256)
  static constexpr int kColO = 256;                  // O0 [256,256+D), O1 [256+D, 256+2D)
};

struct Fwd2Bars {
  uint64_t q_full, k_full[kRing], k_empty[kRing], v_full[kRing], v_empty[kRing];
  uint64_t s_full[2], p_ready[2], o_full[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void store_p_chunk(uint8_t* tile, int r, int c0, const uint32_t (&pk)[16]) {
  uint8_t* base = tile + (c0 >> 6) * 16384 + r * 128;
  const int chunk0 = (c0 & 63) >> 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int phys = (chunk0 + i) ^ (r & 7);
    *reinterpret_cast<uint4*>(base + phys * 16) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
  }
}

// Bounded wait that parks the thread in the barrier's own time-limited suspend instead of spinning on the issue
// port, which the softmax warps of the other query tile need.
__device__ __forceinline__ bool mbar_wait_parked(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  uint32_t done = 0;
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity), "r"(1000u)
        : "memory");
    if (done) return true;
    if ((it & 31) == 31) {
      if (*abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > kWaitBudgetNs) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

template <int D>
__global__ void __launch_bounds__(kThreads2, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                 const __grid_constant__ CUtensorMap tv, const __grid_constant__ Fwd2Args a) {
  using C = Fwd2Cfg<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) report_status(a.status, kBadArgument, 11, 0, 0);
    return;
  }
  Fwd2Bars* bars = reinterpret_cast<Fwd2Bars*>(smem + C::kOffBar);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Pairs of query tiles, the ones with the most key tiles first (slowest grid dimension, reversed).
  const int pair = gridDim.z - 1 - blockIdx.z;
  const int h = blockIdx.x, b = blockIdx.y;
  const int hkv = h / (a.H / a.Hkv);
  const int n_kv_all = (a.Tk + 127) / 128;
  const int n_q_tiles = (a.Tq + 127) / 128;
  int nkv[2];
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    const int t = 2 * pair + g;
    if (t >= n_q_tiles) {
      nkv[g] = 0;
    } else if (a.causal) {
      // last key any query of the tile may see: q_pos0 + t*128 + 127
      const int last = a.q_pos0 + t * 128 + 127;
      nkv[g] = min(last / 128 + 1, n_kv_all);
    } else {
      nkv[g] = n_kv_all;
    }
  }
  const int n_max = max(nkv[0], nkv[1]);
  const int q_row0 = b * a.Tq + pair * 256;
  const int kv_row0 = b * a.kv_rows_b + hkv * a.kv_rows_h;
  const int k_col0 = hkv * a.k_col_h, v_col0 = hkv * a.v_col_h;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < kRing; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(&bars->s_full[g], 1);
      mbar_init(&bars->p_ready[g], 128);
      mbar_init(&bars->o_full[g], 1);
    }
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

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tq);
      tma_prefetch_desc(&tk);
      tma_prefetch_desc(&tv);
      mbar_arrive_expect_tx(&bars->q_full, 2 * C::kTile);
      tma_load_2d(smem + C::kOffQ, &tq, &bars->q_full, h * D, q_row0);
      tma_load_2d(smem + C::kOffQ + C::kTile, &tq, &bars->q_full, h * D, q_row0 + 128);
      for (int j = 0; j < n_max; ++j) {
        const int s = j % kRing;
        const uint32_t ph = (j / kRing) & 1;
        if (!mbar_wait(&bars->k_empty[s], ph ^ 1, abort_flag)) {
          report_status(a.status, kWaitEmptyTimeout, 110, pair, j);
          break;
        }
        mbar_arrive_expect_tx(&bars->k_full[s], C::kTile);
        tma_load_2d(smem + C::kOffK + s * C::kTile, &tk, &bars->k_full[s], k_col0, kv_row0 + j * 128);
        if (!mbar_wait(&bars->v_empty[s], ph ^ 1, abort_flag)) {
          report_status(a.status, kWaitEmptyTimeout, 111, pair, j);
          break;
        }
        mbar_arrive_expect_tx(&bars->v_full[s], C::kTile);
        tma_load_2d(smem + C::kOffV + s * C::kTile, &tv, &bars->v_full[s], v_col0, kv_row0 + j * 128);
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc_s = make_idesc(128, 128, 0, 0, 1);
    constexpr uint32_t idesc_o = make_idesc(128, D, 0, 1, 1);
    bool ok = mbar_wait(&bars->q_full, 0, abort_flag);
    if (!ok && lane == 0) report_status(a.status, kWaitFullTimeout, 112, pair, 0);
    // S_g(j) = Q_g K_j^T; the K stage is released by the last tile that reads it.
    auto issue_s = [&](int g, int j) -> bool {
      const int s = j % kRing;
      if (!mbar_wait(&bars->k_full[s], (j / kRing) & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitFullTimeout, 113, pair, j);
        return false;
      }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t aQ = smem_u32(smem + C::kOffQ + g * C::kTile);
        const uint32_t aK = smem_u32(smem + C::kOffK + s * C::kTile);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_bf16(tmem + C::kColS + g * 128, make_smem_desc(aQ + kk * 32, 16, 1024),
                    make_smem_desc(aK + kk * 32, 16, 1024), idesc_s, kk > 0);
        tc_commit(&bars->s_full[g]);
        const bool last_user = (g == 1) || (j >= nkv[1]);
        if (last_user) tc_commit(&bars->k_empty[s]);
      }
      __syncwarp();
      return true;
    };
    for (int g = 0; g < 2 && ok; ++g)
      if (nkv[g] > 0) ok = issue_s(g, 0);
    for (int j = 0; j < n_max && ok; ++j) {
      const int s = j % kRing;
      for (int g = 0; g < 2 && ok; ++g) {
        if (j >= nkv[g]) continue;
        if (!mbar_wait(&bars->v_full[s], (j / kRing) & 1, abort_flag) ||
            !mbar_wait(&bars->p_ready[g], j & 1, abort_flag)) {
          if (lane == 0) report_status(a.status, kWaitAttnTimeout, 114, pair, j);
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t aP = smem_u32(smem + C::kOffP + g * C::kPBytes);
          const uint32_t aV = smem_u32(smem + C::kOffV + s * C::kTile);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
            umma_bf16(tmem + C::kColO + g * D, make_smem_desc(aP + off, 16, 1024),
                      make_smem_desc(aV + kk * 2048, 16384, 1024), idesc_o, kk > 0);
          }
          tc_commit(&bars->o_full[g]);
          const bool last_user = (g == 1) || (j >= nkv[1]);
          if (last_user) tc_commit(&bars->v_empty[s]);
        }
        __syncwarp();
        if (j + 1 < nkv[g]) ok = issue_s(g, j + 1);
      }
    }
  } else {
    const int g = (warp - 2) >> 2;       // query tile of this softmax group
    const int q4 = warp & 3;             // TMEM lane quarter this warp may touch
    const int r = q4 * 32 + lane;        // row inside the tile == TMEM lane
    const int qi = (2 * pair + g) * 128 + r;   // query index inside the sequence
    const int qpos = a.q_pos0 + qi;
    const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
    const uint32_t tS = tmem + C::kColS + g * 128 + lane_off;
    const uint32_t tO = tmem + C::kColO + g * D + lane_off;
    uint8_t* sP = smem + C::kOffP + g * C::kPBytes;
    const int n_mine = nkv[g];
    float m = -INFINITY, l = 0.f;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < n_mine; ++j) {
      if (!mbar_wait_parked(&bars->s_full[g], j & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitAttnTimeout, 115, pair, j);
        ok = false;
        break;
      }
      tc_fence_after();
      const int kv0 = j * 128;
      const bool need_mask = (a.causal && kv0 + 127 > a.q_pos0 + (2 * pair + g) * 128) || (kv0 + 128 > a.Tk);
      // pass 1: row maximum of the raw scores (the positive scale is applied to the maximum once)
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(tS + c * 64, v0);
        tmem_ld_32x32(tS + c * 64 + 32, v1);
        tmem_ld_wait();
        if (!need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(__uint_as_float(v0[i]), __uint_as_float(v1[i])));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int k0 = kv0 + c * 64 + i, k1 = k0 + 32;
            const bool ok0 = k0 < a.Tk && !(a.causal && k0 > qpos);
            const bool ok1 = k1 < a.Tk && !(a.causal && k1 > qpos);
            if (ok0) mx = fmaxf(mx, __uint_as_float(v0[i]));
            if (ok1) mx = fmaxf(mx, __uint_as_float(v1[i]));
          }
        }
      }
      mx = fmaxf(mx * a.scale_log2, m);
      const float mref = (mx == -INFINITY) ? 0.f : mx;
      const float alpha = exp2f(m - mref);  // m == -inf -> 0
      float rs0 = 0.f, rs1 = 0.f;
      // pass 2: probabilities, row sum, bf16 P into the swizzled shared tile
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tS + c * 32, v);
        tmem_ld_wait();
        uint32_t pk[16];
        if (!need_mask) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = exp2f(fmaf(__uint_as_float(v[i]), a.scale_log2, -mref));
            const float p1 = exp2f(fmaf(__uint_as_float(v[i + 1]), a.scale_log2, -mref));
            rs0 += p0;
            rs1 += p1;
            pk[i >> 1] = pack_bf16x2(p0, p1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int k0 = kv0 + c * 32 + i, k1 = k0 + 1;
            float p0 = exp2f(fmaf(__uint_as_float(v[i]), a.scale_log2, -mref));
            float p1 = exp2f(fmaf(__uint_as_float(v[i + 1]), a.scale_log2, -mref));
            if (k0 >= a.Tk || (a.causal && k0 > qpos)) p0 = 0.f;
            if (k1 >= a.Tk || (a.causal && k1 > qpos)) p1 = 0.f;
            rs0 += p0;
            rs1 += p1;
            pk[i >> 1] = pack_bf16x2(p0, p1);
          }
        }
        store_p_chunk(sP, r, c * 32, pk);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bars->p_ready[g]);
      l = l * alpha + (rs0 + rs1);
      m = mx;
      if (!mbar_wait_parked(&bars->o_full[g], j & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitAttnTimeout, 116, pair, j);
        ok = false;
        break;
      }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tO + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], alpha, __uint_as_float(v[i]));
      }
      tc_fence_before();
    }
    if (ok && n_mine > 0 && qi < a.Tq) {
      const float inv = (l > 0.f) ? 1.f / l : 0.f;
      __nv_bfloat16* orow = a.out + static_cast<int64_t>(b * a.Tq + qi) * a.ldo + h * D;
#pragma unroll
      for (int i = 0; i < D; i += 8) {
        uint4 pk = make_uint4(pack_bf16x2(o[i] * inv, o[i + 1] * inv), pack_bf16x2(o[i + 2] * inv, o[i + 3] * inv),
                              pack_bf16x2(o[i + 4] * inv, o[i + 5] * inv), pack_bf16x2(o[i + 6] * inv, o[i + 7] * inv));
        *reinterpret_cast<uint4*>(orow + i) = pk;
      }
      if (a.lse != nullptr) a.lse[(static_cast<int64_t>(b) * a.H + h) * a.Tq + qi] = m + log2f(l);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace

cudaError_t launch_attn_fwd2_d64(const AttnTensors& t, const AttnShape& s, const AttnKvLayout& kv,
                                 __nv_bfloat16* out, int64_t ldo, float* lse, int* status, cudaStream_t stream) {
  constexpr int D = 64;
  using C = Fwd2Cfg<D>;
  if (s.H % s.Hkv != 0 || s.D != D || (s.Dv != 0 && s.Dv != D)) return cudaErrorInvalidValue;
  CUtensorMap tq, tk, tv;
  cudaError_t e;
  if ((e = encode_tma_2d(&tq, t.q, 2, s.H * D, static_cast<uint64_t>(s.B) * s.T, t.ldq * 2, 64, 128)) != cudaSuccess)
    return e;
  if ((e = encode_tma_2d(&tk, t.k, 2, kv.k_cols, kv.rows, t.ldk * 2, 64, 128)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tv, t.v, 2, kv.v_cols, kv.rows, t.ldv * 2, 64, 128)) != cudaSuccess) return e;
  auto kernel = attn_fwd2_kernel<D>;
  static bool configured = false;
  if (!configured) {
    if ((e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem)) != cudaSuccess)
      return e;
    configured = true;
  }
  Fwd2Args a{s.B, s.T, kv.Tk, s.H, s.Hkv, kv.q_pos0, kv.rows_b, kv.rows_h, kv.k_col_h, kv.v_col_h,
             s.scale * kLog2e2, s.causal, out, ldo, lse, status};
  const int n_pairs = ((s.T + 127) / 128 + 1) / 2;
  dim3 grid(s.H, s.B, n_pairs);
  kernel<<<grid, kThreads2, C::kSmem, stream>>>(tq, tk, tv, a);
  return cudaGetLastError();
}

}  // namespace b200
