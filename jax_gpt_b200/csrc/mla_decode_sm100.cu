// Paged MLA decode for sm_100a: one query token per sequence attends over its latent cache
// (576 values per token: 512 compressed KV + 64 rotary key) kept in 64-token pages.
//
// With the up-projections absorbed into the query and the output, all heads of a sequence share
// ONE key/value stream, so the kernel is written "transposed": the cached tokens are the M side
// of the score product and the (few) heads the N side,
//     S^T [64 tokens x heads]   = C[64 x 576] . Q^T              (M = 64; A, B K-major)
//     O^T [512 latent x heads]  = C[:, :512]^T . P^T             (M = 128 x 4; A MN-major from the SAME smem tile)
// One page is one tile: nine 64-column chunks fetched by TMA (128B swizzle) into one of two
// buffers, feeding both products. Two softmax groups of four warps work on alternating tiles
// (group g owns buffer g, its own score / output columns in TMEM and its own running max and sum),
// so while one group is in its softmax the tensor core already runs the other tile's score product
// and the TMA engine refills the free buffer. Softmax runs over the token (lane) axis: column
// maxima by `redux.sync` + shared memory, probabilities into a K-major smem tile, O accumulated in
// registers with the running-max correction. The KV range of a sequence is split over grid.x CTAs;
// every (split, group) writes a normalised partial and a second kernel merges them.
//
// The reference has neither MLA nor a paged cache (project_plan.md:58); its decode attends over a
// dense zero-padded buffer (jax_gpt/models/qwen35/gqa.py:96-130).
#include "mla_decode_sm100.cuh"

#include <math.h>

#include "common.cuh"
#include "tma_host.h"

namespace b200 {

namespace {

constexpr int kTile = kMlaPage;                  // 64 tokens
constexpr int kChunks = kMlaWidth / 64;          // 9 chunks of 64 columns
constexpr int kChunkBytes = kTile * 128;         // 8 KB: 64 tokens x 64 bf16
constexpr int kKvBytes = kChunks * kChunkBytes;  // 72 KB per buffer
constexpr int kThreads = 320;                    // producer, MMA issuer, 2 x 4 softmax warps

template <int kHeads>
struct DecodeCfg {
  static constexpr int kQChunkBytes = kHeads * 128;
  static constexpr int kQBytes = kChunks * kQChunkBytes;
  static constexpr int kPBytes = kHeads * 128;   // [heads x 64 tokens] K-major, per group
  static constexpr int kColS = 0;                // S^T of group g at g * kHeads
  static constexpr int kColO = 2 * kHeads;       // O^T of group g at kColO + g * 4 * kHeads
  static constexpr int kTmemCols = 10 * kHeads <= 256 ? 256 : 512;
};

template <int kHeads>
struct DecodeSmem {
  uint64_t full[2], kv_free[2], s_full[2], p_ready[2], pv_full[2], q_full;
  uint32_t tmem_base;
  int abort_flag;
  float wmax[2][4][kHeads];
  float m_run[2][2][kHeads];
  float l_run[2][kHeads];
  float alpha[2][kHeads];
};

template <int kHeads>
constexpr int decode_smem_bytes() {
  return 1024 + 2 * kKvBytes + DecodeCfg<kHeads>::kQBytes + 2 * DecodeCfg<kHeads>::kPBytes + sizeof(DecodeSmem<kHeads>);
}

__device__ __forceinline__ int float_key(float x) {
  const int b = __float_as_int(x);
  return b >= 0 ? b : (b ^ 0x7fffffff);
}
__device__ __forceinline__ float key_float(int k) { return __int_as_float(k >= 0 ? k : (k ^ 0x7fffffff)); }

__device__ __forceinline__ void bar_sync_group(int g) { asm volatile("bar.sync %0, 128;" ::"r"(1 + g) : "memory"); }

// TMEM -> registers, 32 lanes x 16 columns
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
// Asks the TMA engine to bring a tile into L2 (no shared-memory destination, no barrier).
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* m, int c0, int c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(reinterpret_cast<uint64_t>(m)),
               "r"(c0), "r"(c1)
               : "memory");
}

constexpr int kPrefetchTiles = 4;   // pages requested into L2 ahead of the shared-memory fill

template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&v)[N]) {
  if constexpr (N == 32) {
    tmem_ld_32x32(taddr, v);
  } else {
    tmem_ld_32x16(taddr, v);
  }
}

template <int kHeads>
__global__ void __launch_bounds__(kThreads, 1)
mla_decode_kernel(const __grid_constant__ CUtensorMap t_pool, const __grid_constant__ CUtensorMap t_q,
                  const __grid_constant__ MlaDecodeArgs a) {
  using Cfg = DecodeCfg<kHeads>;
  using Smem = DecodeSmem<kHeads>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* kv = smem;                       // two buffers of kKvBytes
  uint8_t* qs = kv + 2 * kKvBytes;
  uint8_t* ps = qs + Cfg::kQBytes;          // two P tiles
  Smem* sh = reinterpret_cast<Smem*>(ps + 2 * Cfg::kPBytes);
  volatile int* abort_flag = &sh->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, hb = blockIdx.y, b = blockIdx.z;
  const int sid = a.seq_ids[b];
  const int len = a.seq_lens[sid];
  const int n_tiles = (len + kTile - 1) / kTile;
  const int t0 = static_cast<int>(static_cast<int64_t>(n_tiles) * split / a.n_splits);
  const int t1 = static_cast<int>(static_cast<int64_t>(n_tiles) * (split + 1) / a.n_splits);
  const int n_it = t1 - t0;
  const int h0 = hb * kHeads;

  if (threadIdx.x == 0) {
    for (int g = 0; g < 2; ++g) {
      mbar_init(&sh->full[g], 1);
      mbar_init(&sh->kv_free[g], 1);
      mbar_init(&sh->s_full[g], 1);
      mbar_init(&sh->p_ready[g], 128);
      mbar_init(&sh->pv_full[g], 1);
    }
    mbar_init(&sh->q_full, 1);
    sh->abort_flag = 0;
    fence_mbar_init();
  }
  if (threadIdx.x < 2 * kHeads) {
    const int g = threadIdx.x / kHeads, h = threadIdx.x % kHeads;
    sh->m_run[g][0][h] = -INFINITY;
    sh->m_run[g][1][h] = -INFINITY;
    sh->l_run[g][h] = 0.f;
    sh->alpha[g][h] = 0.f;
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0 && n_it > 0) {
      bool ok = true;
      mbar_arrive_expect_tx(&sh->q_full, Cfg::kQBytes);
      for (int c = 0; c < kChunks; ++c)
        tma_load_2d(qs + c * Cfg::kQChunkBytes, &t_q, &sh->q_full, c * 64, b * a.heads + h0);
      const int* bt = a.block_table + static_cast<int64_t>(sid) * a.max_pages;
      // The two shared-memory buffers cap the bytes in flight per SM far below what HBM latency needs, so
      // the pages of the next few tiles are pulled into L2 first; the buffer fills then hit L2.
      auto prefetch = [&](int pit) {
        const int t = t0 + pit;
        if (pit < n_it && t < a.max_pages) {
          const int pg = bt[t];
          if (pg >= 0)
            for (int c = 0; c < kChunks; ++c) tma_prefetch_l2_2d(&t_pool, c * 64, pg * kMlaPage);
        }
      };
      for (int pit = 2; pit < 2 + kPrefetchTiles; ++pit) prefetch(pit);
      int it = 0;
      for (; it < n_it && ok; ++it) {
        const int g = it & 1, u = it >> 1;
        prefetch(it + 2 + kPrefetchTiles);
        if (u > 0 && !mbar_wait(&sh->kv_free[g], (u - 1) & 1, abort_flag)) {
          report_status(a.status, kWaitEmptyTimeout, 70, b, it);
          ok = false;
          break;
        }
        const int t = t0 + it;
        const int page = t < a.max_pages ? bt[t] : -1;
        if (page < 0 || !bounds_ok(page, a.n_pages, a.status, 221)) {  // a sequence longer than its page list: give up cleanly
          report_status(a.status, kBadArgument, 71, b, t);
          *abort_flag = 1;
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&sh->full[g], kKvBytes);
        for (int c = 0; c < kChunks; ++c)
          tma_load_2d(kv + g * kKvBytes + c * kChunkBytes, &t_pool, &sh->full[g], c * 64, page * kMlaPage);
      }
      if (!ok || *abort_flag) {
        // leave no bulk copy in flight: the last fill of each buffer completes its barrier when the bytes land
        const uint64_t tw = globaltimer_ns();
        for (int g = 0; g < 2; ++g) {
          const int uses = (it + 1 - g) / 2;
          if (uses > 0)
            while (!mbar_try_wait(&sh->full[g], (uses - 1) & 1) && globaltimer_ns() - tw < 2000000ull) {
            }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (score product of tile i before the output product of tile i-1) ----------------
    constexpr uint32_t idesc_s = make_idesc(kTile, kHeads, 0, 0, 1);
    constexpr uint32_t idesc_pv = make_idesc(128, kHeads, 1, 0, 1);
    const uint32_t a_kv = smem_u32(kv), a_q = smem_u32(qs), a_p = smem_u32(ps);
    bool ok = n_it > 0;
    if (ok && !mbar_wait(&sh->q_full, 0, abort_flag)) {
      if (lane == 0) report_status(a.status, kWaitFullTimeout, 72, b, 0);
      ok = false;
    }
    for (int it = 0; it <= n_it && ok; ++it) {
      if (it < n_it) {
        const int g = it & 1, u = it >> 1;
        if (!mbar_wait(&sh->full[g], u & 1, abort_flag)) {
          if (lane == 0) report_status(a.status, kWaitFullTimeout, 73, b, it);
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t kvb = a_kv + g * kKvBytes;
#pragma unroll
          for (int c = 0; c < kChunks; ++c)
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_bf16(tmem + Cfg::kColS + g * kHeads, make_smem_desc(kvb + c * kChunkBytes + k * 32, 16, 1024),
                        make_smem_desc(a_q + c * Cfg::kQChunkBytes + k * 32, 16, 1024), idesc_s, (c > 0 || k > 0) ? 1u : 0u);
          tc_commit(&sh->s_full[g]);
        }
        __syncwarp();
      }
      if (it > 0) {
        const int g = (it - 1) & 1, u = (it - 1) >> 1;
        if (!mbar_wait(&sh->p_ready[g], u & 1, abort_flag)) {
          if (lane == 0) report_status(a.status, kWaitFullTimeout, 74, b, it);
          break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t kvb = a_kv + g * kKvBytes;
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_bf16(tmem + Cfg::kColO + (g * 4 + i) * kHeads,
                        make_smem_desc(kvb + 2 * i * kChunkBytes + kk * 2048, kChunkBytes, 1024),
                        make_smem_desc(a_p + g * Cfg::kPBytes + kk * 32, 16, 1024), idesc_pv, kk > 0 ? 1u : 0u);
          tc_commit(&sh->kv_free[g]);
          tc_commit(&sh->pv_full[g]);
        }
        __syncwarp();
      }
    }
  } else {
    // ---------------- two softmax groups; group g works on tiles g, g + 2, ... ----------------
    const int g = (warp - 2) >> 2;
    const int q = warp & 3;
    const int st = ((warp - 2) & 3) * 32 + lane;        // 0 .. 127 inside the group
    const int row = q * 16 + lane;                      // token row of the tile (lanes 0..15 of each quarter hold S^T)
    const int lrow = q * 32 + lane;                     // latent row of O^T owned by this thread
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    uint8_t* pg = ps + g * Cfg::kPBytes;
    float o[4][kHeads];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int h = 0; h < kHeads; ++h) o[i][h] = 0.f;
    bool ok = true;
    int u = 0;
    for (int it = g; it < n_it; it += 2, ++u) {
      float s[kHeads];
      if (ok && !mbar_wait(&sh->s_full[g], u & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitTmemFullTimeout, 75, b, it);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);  // warp-uniform from here on (shuffles and TMEM loads below)
      if (ok) {
        tc_fence_after();
        uint32_t v[kHeads];
        tmem_ld_cols<kHeads>(tmem + Cfg::kColS + g * kHeads + lane_off, v);
        tmem_ld_wait();
        const bool valid = lane < 16 && (t0 + it) * kTile + row < len;
#pragma unroll
        for (int h = 0; h < kHeads; ++h) s[h] = valid ? __uint_as_float(v[h]) * a.scale_log2 : -INFINITY;
        float mine = -INFINITY;
#pragma unroll
        for (int h = 0; h < kHeads; ++h) {
          const float r = key_float(__reduce_max_sync(0xffffffffu, float_key(s[h])));
          if (lane == h) mine = r;
        }
        if (lane < kHeads) sh->wmax[g][q][lane] = mine;
      }
      bar_sync_group(g);
      const int pp = u & 1;
      if (ok) {
        uint8_t* prow = pg + (row & 7) * 2;
        const int c16 = row >> 3;
#pragma unroll
        for (int h = 0; h < kHeads; ++h) {
          float m = fmaxf(fmaxf(sh->wmax[g][0][h], sh->wmax[g][1][h]), fmaxf(sh->wmax[g][2][h], sh->wmax[g][3][h]));
          m = fmaxf(m, sh->m_run[g][pp][h]);
          const float mref = (m == -INFINITY) ? 0.f : m;
          if (lane < 16)
            *reinterpret_cast<__nv_bfloat16*>(prow + h * 128 + ((c16 ^ (h & 7)) << 4)) = __float2bfloat16(exp2f(s[h] - mref));
          if (st == h) {
            sh->alpha[g][h] = exp2f(sh->m_run[g][pp][h] - mref);
            sh->m_run[g][pp ^ 1][h] = m;
          }
        }
        fence_proxy_async_smem();
      }
      bar_sync_group(g);
      if (ok) {
        // running denominators from the bf16 probabilities the tensor core will use
        constexpr int kLph = 128 / kHeads;              // lanes per head: 4 (32 heads) or 8 (16 heads)
        constexpr int kU4 = 8 / kLph;                   // 16-byte pieces per lane of the head's 128-byte row
        const int h = q * (kHeads / 4) + lane / kLph, part = lane % kLph;
        const uint4* rowp = reinterpret_cast<const uint4*>(pg + h * 128) + part * kU4;
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < kU4; ++j) {
          const uint4 w4 = rowp[j];
          const float2 f0 = unpack_bf16x2(w4.x), f1 = unpack_bf16x2(w4.y), f2 = unpack_bf16x2(w4.z), f3 = unpack_bf16x2(w4.w);
          sum += (f0.x + f0.y) + (f1.x + f1.y) + (f2.x + f2.y) + (f3.x + f3.y);
        }
#pragma unroll
        for (int ofs = 1; ofs < kLph; ofs <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, ofs);
        if (part == 0) sh->l_run[g][h] = sh->l_run[g][h] * sh->alpha[g][h] + sum;
        tc_fence_before();
        mbar_arrive(&sh->p_ready[g]);
        if (!mbar_wait(&sh->pv_full[g], u & 1, abort_flag)) {
          if (lane == 0) report_status(a.status, kWaitTmemFullTimeout, 76, b, it);
          ok = false;
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t v[kHeads];
          tmem_ld_cols<kHeads>(tmem + Cfg::kColO + (g * 4 + i) * kHeads + lane_off, v);
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < kHeads; ++h) o[i][h] = o[i][h] * sh->alpha[g][h] + __uint_as_float(v[h]);
        }
        tc_fence_before();
      }
    }
    bar_sync_group(g);  // l_run of the group's last tile is complete
    // ---- normalised partial output of this (split, group) and its log2-sum-exp ----
    const int64_t pbase = (static_cast<int64_t>(b) * (2 * a.n_splits) + 2 * split + g) * a.heads;
    const int pfin = u & 1;
#pragma unroll
    for (int h = 0; h < kHeads; ++h) {
      if (h0 + h < a.heads) {
        const float l = sh->l_run[g][h];
        const float inv = (ok && l > 0.f) ? 1.f / l : 0.f;
        float* dst = a.part_out + (pbase + h0 + h) * kMlaLatent;
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i * 128 + lrow] = o[i][h] * inv;
      }
    }
    if (st < kHeads && h0 + st < a.heads) {
      const float l = sh->l_run[g][st];
      a.part_lse[pbase + h0 + st] = (ok && l > 0.f) ? sh->m_run[g][pfin][st] + log2f(l) : -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, Cfg::kTmemCols);
  }
}

// out[b, h, :] = sum_s w_s part[b, s, h, :] / sum_s w_s,  w_s = 2^(lse_s - max lse)
__global__ void mla_merge_kernel(const float* __restrict__ part_out, const float* __restrict__ part_lse,
                                 __nv_bfloat16* __restrict__ out, int heads, int n_splits) {
  const int bh = blockIdx.x;  // b * heads + h
  const int b = bh / heads, h = bh % heads;
  float mx = -INFINITY;
  for (int s = 0; s < n_splits; ++s) mx = fmaxf(mx, part_lse[(static_cast<int64_t>(b) * n_splits + s) * heads + h]);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float wsum = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const int64_t idx = (static_cast<int64_t>(b) * n_splits + s) * heads + h;
    const float lse = part_lse[idx];
    if (lse == -INFINITY) continue;
    const float w = exp2f(lse - mx);
    wsum += w;
    const float4 v = reinterpret_cast<const float4*>(part_out + idx * kMlaLatent)[threadIdx.x];
    acc[0] += w * v.x; acc[1] += w * v.y; acc[2] += w * v.z; acc[3] += w * v.w;
  }
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  uint2 pk;
  pk.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
  pk.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
  reinterpret_cast<uint2*>(out + static_cast<int64_t>(bh) * kMlaLatent)[threadIdx.x] = pk;
}

__global__ void paged_kv_write_kernel(const __nv_bfloat16* __restrict__ rows, __nv_bfloat16* __restrict__ pool,
                                      const int* __restrict__ block_table, const int* __restrict__ seq_ids,
                                      const int* __restrict__ start, int T, int width, int page_size, int max_pages,
                                      int n_pages, int* status) {
  const int b = blockIdx.y, t = blockIdx.x;
  const int sid = seq_ids[b];
  const int pos = start[b] + t;
  const int pi = pos / page_size;
  const int page = pi < max_pages ? block_table[static_cast<int64_t>(sid) * max_pages + pi] : -1;
  if (page < 0 || page >= n_pages) {
    if (threadIdx.x == 0) report_status(status, kBadArgument, 77, b, pos);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(rows + (static_cast<int64_t>(b) * T + t) * width);
  uint4* dst = reinterpret_cast<uint4*>(pool + (static_cast<int64_t>(page) * page_size + pos % page_size) * width);
  for (int i = threadIdx.x; i < width / 8; i += blockDim.x) dst[i] = src[i];
}



template <int kHeads>
cudaError_t launch_decode_t(const CUtensorMap& t_pool, const CUtensorMap& t_q, const MlaDecodeArgs& args, cudaStream_t stream) {
  static bool configured = false;
  constexpr int smem = decode_smem_bytes<kHeads>();
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(mla_decode_kernel<kHeads>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const dim3 grid(args.n_splits, (args.heads + kHeads - 1) / kHeads, args.batch);
  mla_decode_kernel<kHeads><<<grid, kThreads, smem, stream>>>(t_pool, t_q, args);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_mla_paged_decode(const __nv_bfloat16* q, const __nv_bfloat16* pool, int n_pages,
                                    const MlaDecodeArgs& args, __nv_bfloat16* out, cudaStream_t stream) {
  if (args.batch < 1 || args.heads < 1 || args.n_splits < 1 || args.max_pages < 1 || n_pages < 1) return cudaErrorInvalidValue;
  const int hpc = args.heads <= 16 ? 16 : 32;   // head columns per CTA
  CUtensorMap t_pool, t_q;
  cudaError_t e;
  if ((e = encode_tma_2d(&t_pool, pool, 2, kMlaWidth, static_cast<uint64_t>(n_pages) * kMlaPage, kMlaWidth * 2ull, 64,
                         kMlaPage)) != cudaSuccess)
    return e;
  if ((e = encode_tma_2d(&t_q, q, 2, kMlaWidth, static_cast<uint64_t>(args.batch) * args.heads, kMlaWidth * 2ull, 64,
                         hpc)) != cudaSuccess)
    return e;
  MlaDecodeArgs a2 = args;
  a2.n_pages = n_pages;
  e = hpc == 16 ? launch_decode_t<16>(t_pool, t_q, a2, stream) : launch_decode_t<32>(t_pool, t_q, a2, stream);
  if (e != cudaSuccess) return e;
  mla_merge_kernel<<<args.batch * args.heads, kMlaLatent / 4, 0, stream>>>(args.part_out, args.part_lse, out, args.heads,
                                                                          2 * args.n_splits);
  return cudaGetLastError();
}

cudaError_t launch_paged_kv_write(const __nv_bfloat16* rows, __nv_bfloat16* pool, const int* block_table,
                                  const int* seq_ids, const int* start, int batch, int T, int width, int page_size,
                                  int max_pages, int n_pages, int* status, cudaStream_t stream) {
  if (width % 8 != 0 || batch < 1 || T < 1) return cudaErrorInvalidValue;
  paged_kv_write_kernel<<<dim3(T, batch), 64, 0, stream>>>(rows, pool, block_table, seq_ids, start, T, width, page_size,
                                                           max_pages, n_pages, status);
  return cudaGetLastError();
}

}  // namespace b200
