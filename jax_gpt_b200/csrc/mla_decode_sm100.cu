// Paged MLA decode for sm_100a: one query token per sequence attends over its latent cache
// (576 values per token: 512 compressed KV + 64 rotary key) kept in 64-token pages.
//
// With the up-projections absorbed into the query and the output, all heads of a sequence share
// ONE key/value stream, so the kernel is written "transposed": the cached tokens are the M side
// of both tensor-core products and the (few) heads the N side,
//     S^T [128 tokens x 32 heads]  = C[128 x 576] . Q^T            (A, B K-major)
//     O^T [512 latent x 32 heads]  = C[:, :512]^T . P^T            (A MN-major from the SAME smem tile)
// A tile of two pages is fetched once by TMA (nine 64-column chunks, 128B swizzle) and feeds
// both products; heads beyond the real count are padding columns. Softmax runs over the token
// axis: column maxima by warp reductions + shared memory, probabilities written to a K-major
// smem tile, O accumulated in registers with the usual running-max correction. The KV range of a
// sequence is split over grid.x CTAs; a second kernel merges the splits.
//
// The reference has neither MLA nor a paged cache (project_plan.md:58); its decode attends over a
// dense zero-padded buffer (jax_gpt/models/qwen35/gqa.py:96-130).
#include "mla_decode_sm100.cuh"

#include <math.h>

#include "common.cuh"
#include "tma_host.h"

namespace b200 {

namespace {

constexpr int kTileTokens = 128;               // two pages
constexpr int kHeads = 32;                     // head columns per CTA
constexpr int kChunks = kMlaWidth / 64;        // 9 chunks of 64 columns
constexpr int kChunkBytes = kTileTokens * 128; // 16 KB: 128 tokens x 64 bf16
constexpr int kQChunkBytes = kHeads * 128;     // 4 KB
constexpr int kKvBytes = kChunks * kChunkBytes;   // 144 KB
constexpr int kQBytes = kChunks * kQChunkBytes;   // 36 KB
constexpr int kPBytes = 2 * kHeads * 128;         // 8 KB: two K-major sub-tiles of 64 tokens
constexpr int kThreads = 192;
constexpr int kTmemCols = 256;                 // S^T at column 0 (32), O^T at 32 .. 159

struct DecodeSmem {
  uint64_t full[kChunks], q_full, kv_free, s_full, p_ready, pv_full;
  uint32_t tmem_base;
  int abort_flag;
  float wmax[4][kHeads];
  float m_run[2][kHeads];
  float l_run[kHeads];
  float alpha[kHeads];
};
constexpr int kSmemBytes = 1024 + kKvBytes + kQBytes + kPBytes + sizeof(DecodeSmem);

__device__ __forceinline__ int float_key(float x) {
  const int b = __float_as_int(x);
  return b >= 0 ? b : (b ^ 0x7fffffff);
}
__device__ __forceinline__ float key_float(int k) { return __int_as_float(k >= 0 ? k : (k ^ 0x7fffffff)); }

__device__ __forceinline__ void bar_sync_softmax() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__global__ void __launch_bounds__(kThreads, 1)
mla_decode_kernel(const __grid_constant__ CUtensorMap t_pool, const __grid_constant__ CUtensorMap t_q,
                  const __grid_constant__ MlaDecodeArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* kv = smem;
  uint8_t* qs = kv + kKvBytes;
  uint8_t* ps = qs + kQBytes;
  DecodeSmem* sh = reinterpret_cast<DecodeSmem*>(ps + kPBytes);
  volatile int* abort_flag = &sh->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, hb = blockIdx.y, b = blockIdx.z;
  const int sid = a.seq_ids[b];
  const int len = a.seq_lens[sid];
  const int n_tiles = (len + kTileTokens - 1) / kTileTokens;
  const int t0 = static_cast<int>(static_cast<int64_t>(n_tiles) * split / a.n_splits);
  const int t1 = static_cast<int>(static_cast<int64_t>(n_tiles) * (split + 1) / a.n_splits);
  const int h0 = hb * kHeads;

  if (threadIdx.x == 0) {
    for (int c = 0; c < kChunks; ++c) mbar_init(&sh->full[c], 1);
    mbar_init(&sh->q_full, 1);
    mbar_init(&sh->kv_free, 1);
    mbar_init(&sh->s_full, 1);
    mbar_init(&sh->p_ready, 128);
    mbar_init(&sh->pv_full, 1);
    sh->abort_flag = 0;
    fence_mbar_init();
  }
  if (threadIdx.x < kHeads) {
    sh->m_run[0][threadIdx.x] = -INFINITY;
    sh->m_run[1][threadIdx.x] = -INFINITY;
    sh->l_run[threadIdx.x] = 0.f;
    sh->alpha[threadIdx.x] = 0.f;
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0 && t1 > t0) {
      bool ok = true;
      mbar_arrive_expect_tx(&sh->q_full, kQBytes);
      for (int c = 0; c < kChunks; ++c) tma_load_2d(qs + c * kQChunkBytes, &t_q, &sh->q_full, c * 64, b * a.heads + h0);
      const int n_pages_seq = (len + kMlaPage - 1) / kMlaPage;
      const int* bt = a.block_table + static_cast<int64_t>(sid) * a.max_pages;
      int it = 0;
      for (int t = t0; t < t1 && ok; ++t, ++it) {
        if (it > 0 && !mbar_wait(&sh->kv_free, (it - 1) & 1, abort_flag)) {
          report_status(a.status, kWaitEmptyTimeout, 70, b, t);
          ok = false;
          break;
        }
        const int p0 = bt[2 * t];
        int p1 = (2 * t + 1 < n_pages_seq && 2 * t + 1 < a.max_pages) ? bt[2 * t + 1] : p0;
        if (p1 < 0) p1 = p0;
        if (p0 < 0) {  // a sequence longer than its page list: give up cleanly
          report_status(a.status, kBadArgument, 71, b, t);
          *abort_flag = 1;
          ok = false;
          break;
        }
        for (int c = 0; c < kChunks; ++c) {
          mbar_arrive_expect_tx(&sh->full[c], kChunkBytes);
          tma_load_2d(kv + c * kChunkBytes, &t_pool, &sh->full[c], c * 64, p0 * kMlaPage);
          tma_load_2d(kv + c * kChunkBytes + kChunkBytes / 2, &t_pool, &sh->full[c], c * 64, p1 * kMlaPage);
        }
      }
      if (!ok || *abort_flag) {
        // leave no bulk copy in flight: every armed barrier completes once its bytes have landed
        const uint64_t tw = globaltimer_ns();
        for (int c = 0; c < kChunks; ++c)
          while (!mbar_try_wait(&sh->full[c], (it > 0 ? (it - 1) : 0) & 1) && globaltimer_ns() - tw < 2000000ull) {
          }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t idesc_s = make_idesc(kTileTokens, kHeads, 0, 0, 1);
    constexpr uint32_t idesc_pv = make_idesc(128, kHeads, 1, 0, 1);
    const uint32_t a_kv = smem_u32(kv), a_q = smem_u32(qs), a_p = smem_u32(ps);
    bool ok = t1 > t0;
    if (ok && !mbar_wait(&sh->q_full, 0, abort_flag)) {
      if (lane == 0) report_status(a.status, kWaitFullTimeout, 72, b, 0);
      ok = false;
    }
    int it = 0;
    for (int t = t0; t < t1 && ok; ++t, ++it) {
      for (int c = 0; c < kChunks && ok; ++c) {
        if (!mbar_wait(&sh->full[c], it & 1, abort_flag)) {
          if (lane == 0) report_status(a.status, kWaitFullTimeout, 73, b, t);
          ok = false;
          break;
        }
        tc_fence_after();
        if (lane == 0) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem, make_smem_desc(a_kv + c * kChunkBytes + k * 32, 16, 1024),
                      make_smem_desc(a_q + c * kQChunkBytes + k * 32, 16, 1024), idesc_s, (c > 0 || k > 0) ? 1u : 0u);
        }
        __syncwarp();
      }
      if (!ok) break;
      if (lane == 0) tc_commit(&sh->s_full);
      __syncwarp();
      if (!mbar_wait(&sh->p_ready, it & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitFullTimeout, 74, b, t);
        break;
      }
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_bf16(tmem + 32 + 32 * i, make_smem_desc(a_kv + 2 * i * kChunkBytes + kk * 2048, kChunkBytes, 1024),
                      make_smem_desc(a_p + (kk >> 2) * (kHeads * 128) + (kk & 3) * 32, 16, 1024), idesc_pv,
                      kk > 0 ? 1u : 0u);
        }
        tc_commit(&sh->kv_free);
        tc_commit(&sh->pv_full);
      }
      __syncwarp();
    }
  } else {
    // ---------------- softmax / accumulation warps: thread = token row (S^T) = latent row (O^T) ----------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int st = threadIdx.x - 64;  // 0 .. 127
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    float o[4][kHeads];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int h = 0; h < kHeads; ++h) o[i][h] = 0.f;
    bool ok = true;
    int it = 0;
    for (int t = t0; t < t1; ++t, ++it) {
      float s[kHeads];
      if (ok && !mbar_wait(&sh->s_full, it & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitTmemFullTimeout, 75, b, t);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);  // warp-uniform from here on (shuffles and TMEM loads below)
      if (ok) {
        tc_fence_after();
        uint32_t v[32];
        tmem_ld_32x32(tmem + lane_off, v);
        tmem_ld_wait();
        const bool valid = t * kTileTokens + row < len;
#pragma unroll
        for (int h = 0; h < kHeads; ++h) s[h] = valid ? __uint_as_float(v[h]) * a.scale_log2 : -INFINITY;
        float mine = -INFINITY;
#pragma unroll
        for (int h = 0; h < kHeads; ++h) {
          const float r = key_float(__reduce_max_sync(0xffffffffu, float_key(s[h])));
          if (lane == h) mine = r;
        }
        sh->wmax[q][lane] = mine;
      }
      bar_sync_softmax();
      const int pp = it & 1;
      if (ok) {
        const int sub = row >> 6, tt = row & 63;
        uint8_t* prow = ps + sub * (kHeads * 128) + (tt & 7) * 2;
        const int c16 = tt >> 3;
#pragma unroll
        for (int h = 0; h < kHeads; ++h) {
          float m = fmaxf(fmaxf(sh->wmax[0][h], sh->wmax[1][h]), fmaxf(sh->wmax[2][h], sh->wmax[3][h]));
          m = fmaxf(m, sh->m_run[pp][h]);
          const float mref = (m == -INFINITY) ? 0.f : m;
          const float p = exp2f(s[h] - mref);
          *reinterpret_cast<__nv_bfloat16*>(prow + h * 128 + ((c16 ^ (h & 7)) << 4)) = __float2bfloat16(p);
          if (st == h) {
            sh->alpha[h] = exp2f(sh->m_run[pp][h] - mref);
            sh->m_run[pp ^ 1][h] = m;
          }
        }
        fence_proxy_async_smem();
      }
      bar_sync_softmax();
      if (ok) {
        // running denominators from the bf16 probabilities the tensor core will use:
        // 4 lanes per head, each sums 32 of the 128 tokens of the head's row
        const int h = q * 8 + (lane >> 2), part = lane & 3;
        const uint4* rowp = reinterpret_cast<const uint4*>(ps + (part >> 1) * (kHeads * 128) + h * 128) + (part & 1) * 4;
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 u = rowp[j];
          const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
          sum += (f0.x + f0.y) + (f1.x + f1.y) + (f2.x + f2.y) + (f3.x + f3.y);
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (part == 0) sh->l_run[h] = sh->l_run[h] * sh->alpha[h] + sum;
        tc_fence_before();
        mbar_arrive(&sh->p_ready);
        if (!mbar_wait(&sh->pv_full, it & 1, abort_flag)) {
          if (lane == 0) report_status(a.status, kWaitTmemFullTimeout, 76, b, t);
          ok = false;
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t v[32];
          tmem_ld_32x32(tmem + 32 + 32 * i + lane_off, v);
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < kHeads; ++h) o[i][h] = o[i][h] * sh->alpha[h] + __uint_as_float(v[h]);
        }
        tc_fence_before();
      }
    }
    bar_sync_softmax();  // l_run of the last tile is complete
    // ---- normalised partial output and its log2-sum-exp ----
    const int64_t pbase = (static_cast<int64_t>(b) * a.n_splits + split) * a.heads;
    const int pfin = it & 1;
#pragma unroll
    for (int h = 0; h < kHeads; ++h) {
      if (h0 + h < a.heads) {
        const float l = sh->l_run[h];
        const float inv = (ok && l > 0.f) ? 1.f / l : 0.f;
        float* dst = a.part_out + (pbase + h0 + h) * kMlaLatent;
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i * 128 + row] = o[i][h] * inv;
      }
    }
    if (st < kHeads && h0 + st < a.heads) {
      const float l = sh->l_run[st];
      a.part_lse[pbase + h0 + st] = (ok && l > 0.f) ? sh->m_run[pfin][st] + log2f(l) : -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
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

}  // namespace

cudaError_t launch_mla_paged_decode(const __nv_bfloat16* q, const __nv_bfloat16* pool, int n_pages,
                                    const MlaDecodeArgs& args, __nv_bfloat16* out, cudaStream_t stream) {
  if (args.batch < 1 || args.heads < 1 || args.n_splits < 1 || args.max_pages < 1 || n_pages < 1) return cudaErrorInvalidValue;
  CUtensorMap t_pool, t_q;
  cudaError_t e;
  if ((e = encode_tma_2d(&t_pool, pool, 2, kMlaWidth, static_cast<uint64_t>(n_pages) * kMlaPage, kMlaWidth * 2ull, 64,
                         kMlaPage)) != cudaSuccess)
    return e;
  if ((e = encode_tma_2d(&t_q, q, 2, kMlaWidth, static_cast<uint64_t>(args.batch) * args.heads, kMlaWidth * 2ull, 64,
                         kHeads)) != cudaSuccess)
    return e;
  static bool configured = false;
  if (!configured) {
    if ((e = cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes)) != cudaSuccess)
      return e;
    configured = true;
  }
  const dim3 grid(args.n_splits, (args.heads + kHeads - 1) / kHeads, args.batch);
  mla_decode_kernel<<<grid, kThreads, kSmemBytes, stream>>>(t_pool, t_q, args);
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  mla_merge_kernel<<<args.batch * args.heads, kMlaLatent / 4, 0, stream>>>(args.part_out, args.part_lse, out, args.heads,
                                                                          args.n_splits);
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
