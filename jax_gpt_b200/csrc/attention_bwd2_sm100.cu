// Flash attention backward for head width 64 on tcgen05, software-pipelined over HALF score tiles.
//
// One CTA per (128-key block, kv head, batch) loops over the query blocks that see it and works on the transposed
// tile S^T = K Q^T, so a thread owns a key row (see attention_sm100.cu for the data flow shared with the
// single-stage kernel). Here every 128-query block is handled as two halves of 64 queries:
//
//   MMA warp:      S^T_a dP^T_a | S^T_b dP^T_b | (P_a ready) dV+=, dK+= from half a, S^T_a' dP^T_a' of the NEXT block
//                  | (P_b ready) dV+=, dK+= from half b, dQ = dS K, S^T_b' dP^T_b'
//   compute warps: half a -> P^T_a, dS^T_a | drain dQ of the previous block | half b -> P^T_b, dS^T_b
//
// so the tensor core always has the other half (or the next block's scores) to work on while the eight compute
// warps run exponentials, and the compute warps find their next scores waiting in TMEM. dQ has its own TMEM
// columns and leaves through fp32 reductions one block late. dS^T is double-buffered in shared memory: dQ of block
// i reads all of dS^T(i) after the scores of half a of block i+1 were already handed to the compute warps, so
// block i+1 writes the other buffer; a buffer is re-used only after the compute warps have seen dq_full of the
// block that read it.
#include "attention_sm100.cuh"

#include "common.cuh"
#include "tma_host.h"

namespace b200 {

namespace {

constexpr int kD = 64;
constexpr int kTile = 128 * kD * 2;  // 16 KB
constexpr int kOffK = 0;
constexpr int kOffV = kTile;
constexpr int kOffRing = 2 * kTile;              // 2 stages of {Q_i, dO_i}
constexpr int kOffPT = kOffRing + 4 * kTile;     // P^T  128 x 128 bf16 (two 64-query halves of 16 KB)
constexpr int kOffDST = kOffPT + 32768;          // dS^T 128 x 128 bf16, one buffer per block parity (see below)
constexpr int kOffStats = kOffDST + 65536;       // lse / delta*scale, 2 x 2 x 128 fp32
constexpr int kOffBar = kOffStats + 2048;
constexpr int kSmem = kOffBar + 256;
// TMEM columns: S^T [0,128), dP^T [128,256), dV [256,320), dK [320,384), dQ [384,448)
constexpr uint32_t kColST = 0, kColDP = 128, kColDV = 256, kColDK = 320, kColDQ = 384;
constexpr int kBwd2Threads = 320;

struct Bwd2Args {
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

struct Bwd2Bars {
  uint64_t kv_full, qdo_full[2], qdo_empty[2], st_full[2], p_ready[2], dq_full, dq_read, stats_ready;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void store_chunk_sw128(uint8_t* tile, int r, int c0, const uint32_t (&pk)[16]) {
  uint8_t* base = tile + (c0 >> 6) * 16384 + r * 128;
  const int chunk0 = (c0 & 63) >> 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int phys = (chunk0 + i) ^ (r & 7);
    *reinterpret_cast<uint4*>(base + phys * 16) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
  }
}

__global__ void __launch_bounds__(kBwd2Threads, 1)
attn_bwd2_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                 const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                 const __grid_constant__ Bwd2Args a) {
  constexpr int D = kD;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) report_status(a.status, kBadArgument, 12, 0, 0);
    return;
  }
  Bwd2Bars* bars = reinterpret_cast<Bwd2Bars*>(smem + kOffBar);
  volatile int* abort_flag = &bars->abort_flag;
  float* stats = reinterpret_cast<float*>(smem + kOffStats);  // [buf][0: lse, 1: delta * scale][128]
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
      mbar_init(&bars->st_full[s], 1);
      mbar_init(&bars->p_ready[s], 256);
    }
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
    if (lane == 0) {
      tma_prefetch_desc(&tq);
      tma_prefetch_desc(&tdo);
      mbar_arrive_expect_tx(&bars->kv_full, 2 * kTile);
      tma_load_2d(smem + kOffK, &tk, &bars->kv_full, hkv * D, kv_row0);
      tma_load_2d(smem + kOffV, &tv, &bars->kv_full, hkv * D, kv_row0);
      for (int it = 0; it < n_iters; ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&bars->qdo_empty[s], ph ^ 1, abort_flag)) {
          report_status(a.status, kWaitEmptyTimeout, 220, jb, it);
          break;
        }
        const int hq = hkv * group + it / nqi;
        const int qrow0 = b * a.T + (i0 + it % nqi) * 128;
        uint8_t* st = smem + kOffRing + s * 2 * kTile;
        mbar_arrive_expect_tx(&bars->qdo_full[s], 2 * kTile);
        tma_load_2d(st, &tq, &bars->qdo_full[s], hq * D, qrow0);
        tma_load_2d(st + kTile, &tdo, &bars->qdo_full[s], hq * D, qrow0);
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc_st = make_idesc(128, 64, 0, 0, 1);   // K-major x K-major, 64 queries
    constexpr uint32_t idesc_kn = make_idesc(128, D, 0, 1, 1);    // A K-major, B MN-major
    constexpr uint32_t idesc_nn = make_idesc(128, D, 1, 1, 1);    // A MN-major, B MN-major
    bool ok = mbar_wait(&bars->kv_full, 0, abort_flag);
    if (!ok && lane == 0) report_status(a.status, kWaitFullTimeout, 221, jb, 0);
    const uint32_t aK = smem_u32(smem + kOffK), aV = smem_u32(smem + kOffV);
    const uint32_t aPT = smem_u32(smem + kOffPT);
    // S^T and dP^T of query half `hf` (64 queries) of block `it`.
    auto issue_scores = [&](int it, int hf) -> bool {
      const int s = it & 1;
      if (!mbar_wait(&bars->qdo_full[s], (it >> 1) & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitFullTimeout, 222, jb, it);
        return false;
      }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t aQ = smem_u32(smem + kOffRing + s * 2 * kTile) + hf * 8192;  // rows 64*hf.. of the tile
        const uint32_t aDO = aQ + kTile;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_bf16(tmem + kColST + hf * 64, make_smem_desc(aK + kk * 32, 16, 1024),
                    make_smem_desc(aQ + kk * 32, 16, 1024), idesc_st, kk > 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_bf16(tmem + kColDP + hf * 64, make_smem_desc(aV + kk * 32, 16, 1024),
                    make_smem_desc(aDO + kk * 32, 16, 1024), idesc_st, kk > 0);
        tc_commit(&bars->st_full[hf]);
      }
      __syncwarp();
      return true;
    };
    if (ok && n_iters > 0) ok = issue_scores(0, 0) && issue_scores(0, 1);
    for (int it = 0; it < n_iters && ok; ++it) {
      const int s = it & 1;
      const uint32_t aQ = smem_u32(smem + kOffRing + s * 2 * kTile);
      const uint32_t aDO = aQ + kTile;
      const uint32_t aDST = smem_u32(smem + kOffDST + (it & 1) * 32768);
      for (int hf = 0; hf < 2 && ok; ++hf) {
        if (!mbar_wait(&bars->p_ready[hf], it & 1, abort_flag)) {
          if (lane == 0) report_status(a.status, kWaitAttnTimeout, 224, jb, it);
          ok = false;
          break;
        }
        if (hf == 1 && it > 0 && !mbar_wait(&bars->dq_read, (it - 1) & 1, abort_flag)) {
          if (lane == 0) report_status(a.status, kWaitAttnTimeout, 223, jb, it);
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          // contraction over the 64 queries of this half: four 16-query steps
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const int kk = hf * 4 + k4;
            umma_bf16(tmem + kColDV, make_smem_desc(aPT + hf * 16384 + k4 * 32, 16, 1024),
                      make_smem_desc(aDO + kk * 2048, 16384, 1024), idesc_kn, (it > 0 || kk > 0));
          }
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const int kk = hf * 4 + k4;
            umma_bf16(tmem + kColDK, make_smem_desc(aDST + hf * 16384 + k4 * 32, 16, 1024),
                      make_smem_desc(aQ + kk * 2048, 16384, 1024), idesc_kn, (it > 0 || kk > 0));
          }
          if (hf == 1) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)  // contraction over the 128 key rows: dQ = dS K
              umma_bf16(tmem + kColDQ, make_smem_desc(aDST + kk * 2048, 16384, 1024),
                        make_smem_desc(aK + kk * 2048, 16384, 1024), idesc_nn, kk > 0);
            tc_commit(&bars->dq_full);
            tc_commit(&bars->qdo_empty[s]);
          }
        }
        __syncwarp();
        if (it + 1 < n_iters) ok = issue_scores(it + 1, hf);
      }
    }
  } else {
    const int q4 = warp & 3;
    const int half = (warp - 2) >> 2;    // which 32 of the 64 score columns of a half this thread owns
    const int r = q4 * 32 + lane;        // key row inside the block (and query row when reading dQ)
    const int tid = threadIdx.x - 64;    // 0..255
    const int kvpos = jb * 128 + r;
    const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
    bool ok = true;
    // (lse, delta * scale) of block `jt` go to the shared buffer jt & 1, staged one block ahead; a thread stages
    // jt + 1 only after it has seen stats_ready(jt), i.e. after every thread is done with buffer (jt - 1) & 1.
    auto stage_stats = [&](int jt) {
      const int hq_j = hkv * group + jt / nqi;
      const int q0_j = (i0 + jt % nqi) * 128;
      float* dst = stats + (jt & 1) * 256;
      const int qi = tid & 127;
      const int qp = q0_j + qi;
      const int64_t si = (static_cast<int64_t>(b) * a.H + hq_j) * a.T + qp;
      if (tid < 128) dst[qi] = (qp < a.T) ? a.lse[si] : 0.f;
      else dst[128 + qi] = (qp < a.T) ? a.delta[si] * a.scale : 0.f;
      mbar_arrive(&bars->stats_ready);
    };
    auto drain_dq = [&](int it) -> bool {
      if (!mbar_wait(&bars->dq_full, it & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitAttnTimeout, 226, jb, it);
        return false;
      }
      tc_fence_after();
      const int hq = hkv * group + it / nqi;
      const int qp = (i0 + it % nqi) * 128 + r;
      float* dq = a.dq_accum + (static_cast<int64_t>(b) * a.T + qp) * (static_cast<int64_t>(a.H) * D) + hq * D;
      uint32_t v[32];
      tmem_ld_32x32(tmem + kColDQ + half * 32 + lane_off, v);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&bars->dq_read);
      if (qp < a.T) {
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dq + half * 32 + i),
                       "f"(__uint_as_float(v[i])), "f"(__uint_as_float(v[i + 1])), "f"(__uint_as_float(v[i + 2])),
                       "f"(__uint_as_float(v[i + 3]))
                       : "memory");
      }
      return true;
    };
    if (n_iters > 0) stage_stats(0);
    for (int it = 0; it < n_iters && ok; ++it) {
      const int iq = i0 + it % nqi;
      const int q0 = iq * 128;
      const float* st_lse = stats + (it & 1) * 256;
      const float* st_del = st_lse + 128;
      if (!mbar_wait(&bars->stats_ready, it & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitAttnTimeout, 225, jb, it);
        ok = false;
        break;
      }
      const bool need_mask = (a.causal && iq == jb) || ((iq + 1) * 128 > a.T) || ((jb + 1) * 128 > a.T);
#pragma unroll 1
      for (int hf = 0; hf < 2; ++hf) {
        if (!mbar_wait(&bars->st_full[hf], it & 1, abort_flag)) {
          if (lane == 0) report_status(a.status, kWaitAttnTimeout, 227, jb, it);
          ok = false;
          break;
        }
        tc_fence_after();
        const int c0 = hf * 64 + half * 32;   // first of this thread's 32 query columns
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(tmem + kColST + c0 + lane_off, sv);
        tmem_ld_32x32(tmem + kColDP + c0 + lane_off, dv);
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
            // p = exp2(s * scale_log2 - lse); dS = p * (dP * scale - delta * scale)
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
        store_chunk_sw128(smem + kOffPT, r, c0, pp);
        store_chunk_sw128(smem + kOffDST + (it & 1) * 32768, r, c0, dd);
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(&bars->p_ready[hf]);
        if (hf == 0 && it > 0) ok = drain_dq(it - 1);
        if (!ok) break;
      }
      if (ok && it + 1 < n_iters) stage_stats(it + 1);
    }
    if (ok && n_iters > 0) ok = drain_dq(n_iters - 1);
    if (ok && n_iters > 0) {
      // The last dq_full commit also covered every dV / dK accumulation.
      tc_fence_after();
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* base = which == 0 ? a.dv : a.dk;
        const int64_t ld = which == 0 ? a.lddv : a.lddk;
        const uint32_t col = which == 0 ? kColDV : kColDK;
        uint32_t v[32];
        tmem_ld_32x32(tmem + col + half * 32 + lane_off, v);
        tmem_ld_wait();
        if (kvpos < a.T) {
          __nv_bfloat16* dst = base + static_cast<int64_t>(b * a.T + kvpos) * ld + hkv * D + half * 32;
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

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace

cudaError_t launch_attn_bwd2_d64(const AttnTensors& t, const AttnShape& s, const __nv_bfloat16* dout, int64_t lddo,
                                 const float* lse, const float* delta, float* dq_accum, __nv_bfloat16* dk,
                                 int64_t lddk, __nv_bfloat16* dv, int64_t lddv, int* status, cudaStream_t stream) {
  constexpr int D = kD;
  if (s.D != D || s.H % s.Hkv != 0) return cudaErrorInvalidValue;
  CUtensorMap tq, tk, tv, tdo;
  const uint64_t rows = static_cast<uint64_t>(s.B) * s.T;
  cudaError_t e;
  if ((e = encode_tma_2d(&tq, t.q, 2, s.H * D, rows, t.ldq * 2, 64, 128)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tk, t.k, 2, s.Hkv * D, rows, t.ldk * 2, 64, 128)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tv, t.v, 2, s.Hkv * D, rows, t.ldv * 2, 64, 128)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tdo, dout, 2, s.H * D, rows, lddo * 2, 64, 128)) != cudaSuccess) return e;
  static bool configured = false;
  if (!configured) {
    if ((e = cudaFuncSetAttribute(attn_bwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem)) !=
        cudaSuccess)
      return e;
    configured = true;
  }
  Bwd2Args a{s.B, s.T, s.H, s.Hkv, s.scale, s.scale * 1.4426950408889634f, s.causal, lse, delta, dq_accum,
             dk, lddk, dv, lddv, status};
  dim3 grid(s.Hkv, s.B, (s.T + 127) / 128);
  attn_bwd2_kernel<<<grid, kBwd2Threads, kSmem, stream>>>(tq, tk, tv, tdo, a);
  return cudaGetLastError();
}

}  // namespace b200
