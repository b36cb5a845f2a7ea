// Gated-DeltaNet prefill kernels for sm_100a: the causal depthwise conv + SiLU, and the
// inter-chunk scan of the chunked gated delta rule on tcgen05 tensor cores.
//
// The chunked algorithm splits every head's sequence into chunks of 64 tokens. What does not depend
// on the running state S (cumulative decays, the unit-lower-triangular solve giving the corrected
// values v_eff and the decayed keys k_cum, the masked intra-chunk scores) is computed for all chunks
// at once with batched library calls. What does depend on it is a strictly sequential recurrence,
//     v_new = v_eff - k_cum S
//     o     = (q * exp(G)) S + intra v_new
//     S     = exp(g_end) S + (k * exp(g_end - G))^T v_new
// which the reference runs as a `lax.scan` over chunks (jax_gpt/models/qwen35/deltanet.py:300-360).
// Here one CTA per (batch, head) walks the chunks with S resident on chip: fp32 in the registers of
// 128 threads (one row of the 128 x 128 state each), a bf16 copy in shared memory as tensor-core
// operand. Per chunk three MMAs:
//   1. D[128 x 128] = [k_cum ; q exp(G)] S      (the two 64-row operands stacked to M = 128)
//   2. D[64:128]   += [0 ; intra] v_new         (A tile with a zero upper half)
//   3. P[128 x 128] = (k exp(g_end - G))^T v_new
// with v_new produced between 1 and 2 by the threads that own rows 0..63 of D. TMA double-buffers
// the per-chunk operand tiles.
#include "seq_kernels.cuh"

#include "common.cuh"
#include "tma_host.h"

namespace b200 {

namespace {

constexpr int kC = 64, kDk = 128, kDv = 128;
constexpr int kStages = 2;
constexpr int kA1Bytes = 128 * kDk * 2;      // 32 KB  [k_cum ; qg], two 64-column K blocks of 16 KB
constexpr int kA2Bytes = 128 * kC * 2;       // 16 KB  [0 ; intra]
constexpr int kKdBytes = kC * kDk * 2;       // 16 KB  k_dec, two 64-column blocks of 8 KB
constexpr int kStageBytes = kA1Bytes + kA2Bytes + kKdBytes;   // 64 KB
constexpr int kSbBytes = kDk * kDv * 2;      // 32 KB  S as bf16, two 64-column blocks of 16 KB
constexpr int kVnBytes = kC * kDv * 2;       // 16 KB  v_new, two 64-column blocks of 8 KB
constexpr int kThreads = 192;
constexpr int kSmem = 1024 + kStages * kStageBytes + kSbBytes + kVnBytes + 256;

struct ScanBars {
  uint64_t full[kStages], empty[kStages], d_full, vn_ready, p_full, s_ready;
  uint32_t tmem_base;
  int abort_flag;
};

struct ScanArgs {
  int n_chunks;
  const __nv_bfloat16* veff;   // [BH, N, 64, dv]
  const float* e;              // [BH, N]
  const float* s0;             // [BH, dk, dv] or nullptr
  __nv_bfloat16* o;            // [BH, N, 64, dv]
  float* s_out;                // [BH, dk, dv]
  __nv_bfloat16* s_save;       // optional [BH, N, dk, dv]: the state every chunk STARTS from (for the backward scan)
  __nv_bfloat16* vn_save;      // optional [BH, N, 64, dv]: v_new of every chunk
  int* status;
};

// byte offset of (row r, column c) in a bf16 tile made of 64-column blocks with 128-byte swizzled rows
__device__ __forceinline__ uint32_t swz(int r, int c, int block_bytes) {
  return (c >> 6) * block_bytes + r * 128 + ((((c & 63) >> 3) ^ (r & 7)) << 4) + (c & 7) * 2;
}

__global__ void __launch_bounds__(kThreads, 1)
gdn_scan_kernel(const __grid_constant__ CUtensorMap t_kq, const __grid_constant__ CUtensorMap t_intra,
                const __grid_constant__ CUtensorMap t_kdec, const __grid_constant__ ScanArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sb = smem + kStages * kStageBytes;
  uint8_t* vn = sb + kSbBytes;
  ScanBars* bars = reinterpret_cast<ScanBars*>(vn + kVnBytes);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x;
  const int N = a.n_chunks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->d_full, 1);
    mbar_init(&bars->vn_ready, 128);
    mbar_init(&bars->p_full, 1);
    mbar_init(&bars->s_ready, 128);
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  // the upper half of every [0 ; intra] tile stays zero for the whole kernel
  for (int i = threadIdx.x; i < kStages * (kA2Bytes / 2) / 16; i += kThreads) {
    const int s = i / ((kA2Bytes / 2) / 16), j = i % ((kA2Bytes / 2) / 16);
    reinterpret_cast<uint4*>(smem + s * kStageBytes + kA1Bytes)[j] = make_uint4(0, 0, 0, 0);
  }
  fence_proxy_async_smem();
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      int issued = 0;
      for (int n = 0; n < N; ++n, ++issued) {
        const int st = n & 1;
        if (n >= kStages && !mbar_wait(&bars->empty[st], ((n >> 1) - 1) & 1, abort_flag)) {
          report_status(a.status, kWaitEmptyTimeout, 100, bh, n);
          ok = false;
          break;
        }
        uint8_t* base = smem + st * kStageBytes;
        const int chunk = bh * N + n;
        mbar_arrive_expect_tx(&bars->full[st], kA1Bytes + kA2Bytes / 2 + kKdBytes);
        tma_load_2d(base, &t_kq, &bars->full[st], 0, chunk * 128);
        tma_load_2d(base + 16384, &t_kq, &bars->full[st], 64, chunk * 128);
        tma_load_2d(base + kA1Bytes + kA2Bytes / 2, &t_intra, &bars->full[st], 0, chunk * 64);
        tma_load_2d(base + kA1Bytes + kA2Bytes, &t_kdec, &bars->full[st], 0, chunk * 64);
        tma_load_2d(base + kA1Bytes + kA2Bytes + 8192, &t_kdec, &bars->full[st], 64, chunk * 64);
      }
      if (!ok || *abort_flag) {
        // leave no bulk copy in flight: wait (bounded) for the last fill of each stage to land
        const uint64_t tw = globaltimer_ns();
        for (int s = 0; s < kStages; ++s) {
          const int uses = (issued + 1 - s) / 2;
          if (uses > 0)
            while (!mbar_try_wait(&bars->full[s], (uses - 1) & 1) && globaltimer_ns() - tw < 2000000ull) {
            }
        }
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc_kn = make_idesc(128, 128, 0, 1, 1);   // A K-major, B MN-major
    constexpr uint32_t idesc_nn = make_idesc(128, 128, 1, 1, 1);   // both MN-major
    const uint32_t a_sb = smem_u32(sb), a_vn = smem_u32(vn);
    for (int n = 0; n < N; ++n) {
      const int st = n & 1;
      const uint32_t a1 = smem_u32(smem + st * kStageBytes), a2 = a1 + kA1Bytes, kd = a2 + kA2Bytes;
      if (!mbar_wait(&bars->s_ready, n & 1, abort_flag) || !mbar_wait(&bars->full[st], (n >> 1) & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitFullTimeout, 101, bh, n);
        break;
      }
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < 8; ++k)   // K = dk = 128: block k / 4, 32 bytes per step
          umma_bf16(tmem, make_smem_desc(a1 + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                    make_smem_desc(a_sb + k * 2048, 16384, 1024), idesc_kn, k > 0 ? 1u : 0u);
        tc_commit(&bars->d_full);
      }
      __syncwarp();
      if (!mbar_wait(&bars->vn_ready, n & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitFullTimeout, 102, bh, n);
        break;
      }
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < 4; ++k)   // K = 64 tokens
          umma_bf16(tmem, make_smem_desc(a2 + k * 32, 16, 1024), make_smem_desc(a_vn + k * 2048, 8192, 1024), idesc_kn, 1u);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16(tmem + 128, make_smem_desc(kd + k * 2048, 8192, 1024), make_smem_desc(a_vn + k * 2048, 8192, 1024),
                    idesc_nn, k > 0 ? 1u : 0u);
        tc_commit(&bars->empty[st]);
        tc_commit(&bars->p_full);
      }
      __syncwarp();
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;                     // row of D / P / S owned by this thread
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    float S[kDv];
    if (a.s0 != nullptr) {
      const float4* sp = reinterpret_cast<const float4*>(a.s0 + (static_cast<int64_t>(bh) * kDk + r) * kDv);
#pragma unroll
      for (int j = 0; j < kDv / 4; ++j) {
        const float4 f = sp[j];
        S[4 * j] = f.x; S[4 * j + 1] = f.y; S[4 * j + 2] = f.z; S[4 * j + 3] = f.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < kDv; ++j) S[j] = 0.f;
    }
    bool ok = true;
    for (int n = 0; n <= N; ++n) {
      // ---- publish S (bf16) for the next chunk's first product ----
      if (n < N) {
        uint4* ssave = a.s_save != nullptr
                           ? reinterpret_cast<uint4*>(a.s_save + ((static_cast<int64_t>(bh) * N + n) * kDk + r) * kDv)
                           : nullptr;
#pragma unroll
        for (int c = 0; c < kDv; c += 8) {
          const uint4 pk = make_uint4(pack_bf16x2(S[c], S[c + 1]), pack_bf16x2(S[c + 2], S[c + 3]),
                                      pack_bf16x2(S[c + 4], S[c + 5]), pack_bf16x2(S[c + 6], S[c + 7]));
          *reinterpret_cast<uint4*>(sb + swz(r, c, 16384)) = pk;
          if (ssave != nullptr) ssave[c >> 3] = pk;
        }
        fence_proxy_async_smem();
        mbar_arrive(&bars->s_ready);
      } else {
        break;
      }
      const int64_t chunk = static_cast<int64_t>(bh) * N + n;
      // rows 0..63 own a token of the chunk: fetch its corrected value early
      uint4 ve[16];
      if (r < kC) {
        const uint4* vp = reinterpret_cast<const uint4*>(a.veff + (chunk * kC + r) * kDv);
#pragma unroll
        for (int j = 0; j < 16; ++j) ve[j] = __ldg(vp + j);
      }
      const float e = a.e[chunk];
      if (ok && !mbar_wait(&bars->d_full, n & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitTmemFullTimeout, 103, bh, n);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (ok && r < kC) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tmem + c * 32 + lane_off, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            const uint4 u = ve[c * 4 + (j >> 3)];
            const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
            const uint4 pk = make_uint4(
                pack_bf16x2(f0.x - __uint_as_float(v[j]), f0.y - __uint_as_float(v[j + 1])),
                pack_bf16x2(f1.x - __uint_as_float(v[j + 2]), f1.y - __uint_as_float(v[j + 3])),
                pack_bf16x2(f2.x - __uint_as_float(v[j + 4]), f2.y - __uint_as_float(v[j + 5])),
                pack_bf16x2(f3.x - __uint_as_float(v[j + 6]), f3.y - __uint_as_float(v[j + 7])));
            *reinterpret_cast<uint4*>(vn + swz(r, c * 32 + j, 8192)) = pk;
            if (a.vn_save != nullptr)
              reinterpret_cast<uint4*>(a.vn_save + (chunk * kC + r) * kDv)[c * 4 + (j >> 3)] = pk;
          }
        }
        tc_fence_before();
        fence_proxy_async_smem();
      }
      mbar_arrive(&bars->vn_ready);
      if (ok && !mbar_wait(&bars->p_full, n & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitTmemFullTimeout, 104, bh, n);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) continue;
      tc_fence_after();
      if (r >= kC) {   // rows 64..127 of D are the chunk's outputs
        uint4* op = reinterpret_cast<uint4*>(a.o + (chunk * kC + (r - kC)) * kDv);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tmem + c * 32 + lane_off, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j += 8)
            op[c * 4 + (j >> 3)] = make_uint4(pack_bf16x2(__uint_as_float(v[j]), __uint_as_float(v[j + 1])),
                                               pack_bf16x2(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])),
                                               pack_bf16x2(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5])),
                                               pack_bf16x2(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7])));
        }
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem + 128 + c * 32 + lane_off, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) S[c * 32 + j] = S[c * 32 + j] * e + __uint_as_float(v[j]);
      }
      tc_fence_before();
    }
    if (ok) {
      float4* sp = reinterpret_cast<float4*>(a.s_out + (static_cast<int64_t>(bh) * kDk + r) * kDv);
#pragma unroll
      for (int j = 0; j < kDv / 4; ++j) sp[j] = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

// y[b, t, c] = silu(sum_j w[c, j] x[b, t - (K-1) + j, c]); state[b, c, :] = the last K raw inputs (zero padded).
// One thread owns 8 channels and a strip of kStrip consecutive tokens: the K-wide window slides through registers,
// so every input is read once (plus K - 1 rows of overlap per strip) and the weights once per strip.
template <int K, int kStrip>
__global__ void gdn_conv_silu_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                     __nv_bfloat16* __restrict__ y, float* __restrict__ state, int T, int C) {
  static_assert(K == 4, "the weight rows are read as one 8-byte vector");
  const int b = blockIdx.z, t0 = blockIdx.y * kStrip;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c0 >= C) return;
  float wv[8][K];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint2 u = *reinterpret_cast<const uint2*>(w + (c0 + i) * K);
    const float2 lo = unpack_bf16x2(u.x), hi = unpack_bf16x2(u.y);
    wv[i][0] = lo.x; wv[i][1] = lo.y; wv[i][2] = hi.x; wv[i][3] = hi.y;
  }
  const __nv_bfloat16* xb = x + static_cast<int64_t>(b) * T * C + c0;
  float win[K][8];                      // win[j] = the input row at t - (K-1) + j
#pragma unroll
  for (int j = 0; j < K; ++j) {
    const int tt = t0 - K + j;          // rows t0-K .. t0-1; the loop shifts before it uses them
    uint4 u = make_uint4(0u, 0u, 0u, 0u);
    if (tt >= 0 && j > 0) u = *reinterpret_cast<const uint4*>(xb + static_cast<int64_t>(tt) * C);   // row 0 is shifted out unused
    const uint32_t in[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf16x2(in[e]);
      win[j][2 * e] = f.x;
      win[j][2 * e + 1] = f.y;
    }
  }
#pragma unroll
  for (int s = 0; s < kStrip; ++s) {
    const int t = t0 + s;
    if (t >= T) break;
    const uint4 u = *reinterpret_cast<const uint4*>(xb + static_cast<int64_t>(t) * C);
    const uint32_t in[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int j = 0; j + 1 < K; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) win[j][i] = win[j + 1][i];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf16x2(in[e]);
      win[K - 1][2 * e] = f.x;
      win[K - 1][2 * e + 1] = f.y;
    }
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) {
        a0 += wv[2 * e][j] * win[j][2 * e];
        a1 += wv[2 * e + 1][j] * win[j][2 * e + 1];
      }
      o[e] = pack_bf16x2(a0 / (1.f + __expf(-a0)), a1 / (1.f + __expf(-a1)));
    }
    *reinterpret_cast<uint4*>(y + (static_cast<int64_t>(b) * T + t) * C + c0) = make_uint4(o[0], o[1], o[2], o[3]);
    if (state != nullptr && t == T - 1) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < K; ++j) state[(static_cast<int64_t>(b) * C + c0 + i) * K + j] = win[j][i];
    }
  }
}


// Backward of the depthwise causal FIR + SiLU above. One thread owns eight channels and a strip of kStrip time
// steps: it walks the strip (plus K-1 steps past its end, for the taps that reach back into it) with the last K
// inputs and the last K pre-activation gradients in registers, so x and dy are read once and dx written once.
//   pre[t] = sum_j w[j] x[t-(K-1)+j];  dpre[t] = dy[t] * sigmoid(pre) * (1 + pre * (1 - sigmoid(pre)))
//   dx[t]  = sum_j w[j] dpre[t+(K-1)-j];  dw[j] += sum_t dpre[t] x[t-(K-1)+j]   (fp32 atomics, one per strip)
template <int K, int kStrip>
__global__ void gdn_conv_silu_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                         const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx,
                                         float* __restrict__ dw, int T, int C) {
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * kStrip;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c0 >= C || t0 >= T) return;
  const int t1 = min(T, t0 + kStrip);
  float wv[8][K], dwa[8][K], xw[8][K], dp[8][K];  // xw / dp: sliding windows, newest in slot K-1
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < K; ++j) {
      wv[i][j] = __bfloat162float(w[(c0 + i) * K + j]);
      dwa[i][j] = 0.f;
      xw[i][j] = 0.f;
      dp[i][j] = 0.f;
    }
  auto load8 = [&](const __nv_bfloat16* base, int t, float (&f)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(base + (static_cast<int64_t>(b) * T + t) * C + c0);
    const float2 a = unpack_bf16x2(u.x), bb = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    f[0] = a.x; f[1] = a.y; f[2] = bb.x; f[3] = bb.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
  };
  // inputs before the strip (zeros before the sequence start)
#pragma unroll
  for (int j = 0; j < K - 1; ++j) {
    const int tt = t0 - (K - 1) + j;
    if (tt >= 0) {
      float f[8];
      load8(x, tt, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) xw[i][j + 1] = f[i];
    }
  }
  const int t_end = min(T, t1 + K - 1);
  for (int t = t0; t < t1 + K - 1; ++t) {
    // shift the windows; positions past the end of the sequence contribute zero gradients
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < K - 1; ++j) {
        xw[i][j] = xw[i][j + 1];
        dp[i][j] = dp[i][j + 1];
      }
    if (t < t_end) {
      float xv[8], dv[8];
      load8(x, t, xv);
      load8(dy, t, dv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        xw[i][K - 1] = xv[i];
        float pre = 0.f;
#pragma unroll
        for (int j = 0; j < K; ++j) pre = fmaf(wv[i][j], xw[i][j], pre);
        const float sg = 1.f / (1.f + __expf(-pre));
        const float g = dv[i] * sg * fmaf(pre, 1.f - sg, 1.f);
        dp[i][K - 1] = g;
        if (t < t1) {
#pragma unroll
          for (int j = 0; j < K; ++j) dwa[i][j] = fmaf(g, xw[i][j], dwa[i][j]);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        xw[i][K - 1] = 0.f;
        dp[i][K - 1] = 0.f;
      }
    }
    const int to = t - (K - 1);  // dx[to] = sum_j w[j] dpre[to + K-1 - j] = sum_j w[j] dp[K-1-j]
    if (to >= t0) {
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < K; ++j) acc = fmaf(wv[i][j], dp[i][K - 1 - j], acc);
        o[i] = acc;
      }
      *reinterpret_cast<uint4*>(dx + (static_cast<int64_t>(b) * T + to) * C + c0) =
          make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]), pack_bf16x2(o[4], o[5]), pack_bf16x2(o[6], o[7]));
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < K; ++j) atomicAdd(dw + (c0 + i) * K + j, dwa[i][j]);
}

// Gated RMSNorm of the scan output fused with the head-major -> token-major transpose:
//   y[b, t, h, :] = w * o[b, h, t, :] * rsqrt(mean(o^2) + eps) * silu(z[b, t, h, :])
// o is [B*Hv, Tpad, 128] bf16 (the scan kernel's layout), z and y are [B, T, Hv * 128] bf16. One warp per row.
__global__ void gdn_gated_norm_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ z,
                                      const float* __restrict__ w, __nv_bfloat16* __restrict__ y, int rows, int T,
                                      int Tpad, int Hv, float eps) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int h = row % Hv, bt = row / Hv, t = bt % T, b = bt / T;
  const uint2 uo = *reinterpret_cast<const uint2*>(o + ((static_cast<int64_t>(b) * Hv + h) * Tpad + t) * 128 + lane * 4);
  const uint2 uz = *reinterpret_cast<const uint2*>(z + static_cast<int64_t>(row) * 128 + lane * 4);
  const float4 wv = *reinterpret_cast<const float4*>(w + lane * 4);
  const float2 o0 = unpack_bf16x2(uo.x), o1 = unpack_bf16x2(uo.y), z0 = unpack_bf16x2(uz.x), z1 = unpack_bf16x2(uz.y);
  float ss = o0.x * o0.x + o0.y * o0.y + o1.x * o1.x + o1.y * o1.y;
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
  const float r = rsqrtf(ss * (1.f / 128.f) + eps);
  auto silu = [](float v) { return v / (1.f + __expf(-v)); };
  uint2 out;
  out.x = pack_bf16x2(wv.x * o0.x * r * silu(z0.x), wv.y * o0.y * r * silu(z0.y));
  out.y = pack_bf16x2(wv.z * o1.x * r * silu(z1.x), wv.w * o1.y * r * silu(z1.y));
  *reinterpret_cast<uint2*>(y + static_cast<int64_t>(row) * 128 + lane * 4) = out;
}

// Backward: with n = o r, s = silu(z):  dn = dy w s;  do = r (dn - n mean(dn n));  dz = dy w n silu'(z);
// dw += sum_rows dy n s (per-warp partial sums over a grid-stride loop, then one atomic per column and CTA).
__global__ void gdn_gated_norm_bwd_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ z,
                                          const float* __restrict__ w, const __nv_bfloat16* __restrict__ dy,
                                          __nv_bfloat16* __restrict__ d_o, __nv_bfloat16* __restrict__ dz,
                                          float* __restrict__ dw, int rows, int T, int Tpad, int Hv, float eps) {
  __shared__ float s_dw[8][128];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
  const float4 wv = *reinterpret_cast<const float4*>(w + lane * 4);
  const float wl[4] = {wv.x, wv.y, wv.z, wv.w};
  float dwa[4] = {0.f, 0.f, 0.f, 0.f};
  for (int row = blockIdx.x * wpb + warp; row < rows; row += gridDim.x * wpb) {
    const int h = row % Hv, bt = row / Hv, t = bt % T, b = bt / T;
    const int64_t o_off = ((static_cast<int64_t>(b) * Hv + h) * Tpad + t) * 128 + lane * 4;
    const int64_t r_off = static_cast<int64_t>(row) * 128 + lane * 4;
    const uint2 uo = *reinterpret_cast<const uint2*>(o + o_off);
    const uint2 uz = *reinterpret_cast<const uint2*>(z + r_off);
    const uint2 ud = *reinterpret_cast<const uint2*>(dy + r_off);
    const float2 a0 = unpack_bf16x2(uo.x), a1 = unpack_bf16x2(uo.y), b0 = unpack_bf16x2(uz.x), b1 = unpack_bf16x2(uz.y);
    const float2 c0 = unpack_bf16x2(ud.x), c1 = unpack_bf16x2(ud.y);
    const float ov[4] = {a0.x, a0.y, a1.x, a1.y}, zv[4] = {b0.x, b0.y, b1.x, b1.y}, dv[4] = {c0.x, c0.y, c1.x, c1.y};
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) ss += ov[i] * ov[i];
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
    const float r = rsqrtf(ss * (1.f / 128.f) + eps);
    float nv[4], dn[4], dzv[4], dot = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float sg = 1.f / (1.f + __expf(-zv[i]));
      const float sl = zv[i] * sg;
      nv[i] = ov[i] * r;
      dn[i] = dv[i] * wl[i] * sl;
      dzv[i] = dv[i] * wl[i] * nv[i] * sg * (1.f + zv[i] * (1.f - sg));
      dwa[i] += dv[i] * nv[i] * sl;
      dot += dn[i] * nv[i];
    }
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, m);
    dot *= (1.f / 128.f);
    uint2 uo_out, uz_out;
    uo_out.x = pack_bf16x2(r * (dn[0] - nv[0] * dot), r * (dn[1] - nv[1] * dot));
    uo_out.y = pack_bf16x2(r * (dn[2] - nv[2] * dot), r * (dn[3] - nv[3] * dot));
    uz_out.x = pack_bf16x2(dzv[0], dzv[1]);
    uz_out.y = pack_bf16x2(dzv[2], dzv[3]);
    *reinterpret_cast<uint2*>(d_o + o_off) = uo_out;
    *reinterpret_cast<uint2*>(dz + r_off) = uz_out;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) s_dw[warp][lane * 4 + i] = dwa[i];
  __syncthreads();
  if (threadIdx.x < 128) {
    float acc = 0.f;
    for (int q = 0; q < wpb; ++q) acc += s_dw[q][threadIdx.x];
    atomicAdd(dw + threadIdx.x, acc);
  }
}

}  // namespace

cudaError_t launch_gdn_scan(const __nv_bfloat16* kq, const __nv_bfloat16* intra, const __nv_bfloat16* kdec,
                            const __nv_bfloat16* veff, const float* e, const float* s0, __nv_bfloat16* o, float* s_out,
                            __nv_bfloat16* s_save, __nv_bfloat16* vn_save, int bh, int n_chunks, int* status,
                            cudaStream_t stream) {
  if (bh < 1 || n_chunks < 1) return cudaErrorInvalidValue;
  CUtensorMap t_kq, t_intra, t_kdec;
  cudaError_t err;
  const uint64_t chunks = static_cast<uint64_t>(bh) * n_chunks;
  if ((err = encode_tma_2d(&t_kq, kq, 2, kDk, chunks * 128, kDk * 2ull, 64, 128)) != cudaSuccess) return err;
  if ((err = encode_tma_2d(&t_intra, intra, 2, kC, chunks * kC, kC * 2ull, 64, 64)) != cudaSuccess) return err;
  if ((err = encode_tma_2d(&t_kdec, kdec, 2, kDk, chunks * kC, kDk * 2ull, 64, 64)) != cudaSuccess) return err;
  static bool configured = false;
  if (!configured) {
    if ((err = cudaFuncSetAttribute(gdn_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem)) != cudaSuccess) return err;
    configured = true;
  }
  ScanArgs args{n_chunks, veff, e, s0, o, s_out, s_save, vn_save, status};
  gdn_scan_kernel<<<bh, kThreads, kSmem, stream>>>(t_kq, t_intra, t_kdec, args);
  return cudaGetLastError();
}

cudaError_t launch_gdn_conv_silu(const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* y, float* state, int B,
                                 int T, int C, int K, cudaStream_t stream) {
  if (K != 4 || C % 8 != 0 || B < 1 || T < 1) return cudaErrorInvalidValue;
  constexpr int kStrip = 16;
  const int threads = 128;
  const dim3 grid((C / 8 + threads - 1) / threads, (T + kStrip - 1) / kStrip, B);
  gdn_conv_silu_kernel<4, kStrip><<<grid, threads, 0, stream>>>(x, w, y, state, T, C);
  return cudaGetLastError();
}

cudaError_t launch_gdn_conv_silu_bwd(const __nv_bfloat16* x, const __nv_bfloat16* w, const __nv_bfloat16* dy,
                                     __nv_bfloat16* dx, float* dw, int B, int T, int C, int K, cudaStream_t stream) {
  if (K != 4 || C % 8 != 0 || B < 1 || T < 1) return cudaErrorInvalidValue;
  constexpr int kStrip = 32;
  const int threads = 128;
  const dim3 grid((C / 8 + threads - 1) / threads, (T + kStrip - 1) / kStrip, B);
  gdn_conv_silu_bwd_kernel<4, kStrip><<<grid, threads, 0, stream>>>(x, w, dy, dx, dw, T, C);
  return cudaGetLastError();
}


// ------------------------------------------------------------------------------------------------
// Backward of the inter-chunk scan: one CTA per (batch, head) walks the chunks in REVERSE with the state
// gradient dS (128 x 128 fp32) in the registers of 128 threads and a bf16 copy in shared memory. With
// S = the state the chunk started from, Vn = its v_new (both saved by the forward kernel) and
// W = -dVn:
//   phase 1   T1 = [kdec ; 0] dS + [intra^T ; 0] dO            -> dVn (rows 0..63) = d v_eff
//   phase 2   T2 = [dO ; W] S^T      rows 0..63 d(q exp G), rows 64..127 d k_cum
//             T3 = [dO ; W] Vn^T     rows 0..63 d intra
//             T4 = [Vn ; 0] dS^T     rows 0..63 d kdec
//             T5 = (q exp G)^T dO + k_cum^T W                  -> dS <- e dS + T5,  d e = <dS, S>
// 64-row operands are stacked in pairs (or padded with a zero half) to fill M = 128.
namespace {

constexpr int kBwdThreads = 192;
constexpr int kTileKq = 0;                         // [k_cum ; qg]   128 x dk, 32 KB
constexpr int kTileKd = kTileKq + 32768;           // [kdec ; 0]     128 x dk, 32 KB
constexpr int kTileIn = kTileKd + 32768;           // intra | zeros  64 x 128, 16 KB (two 64-column blocks of 8 KB)
constexpr int kTileDw = kTileIn + 16384;           // [dO ; W]       128 x dv, 32 KB
constexpr int kTileS = kTileDw + 32768;            // S              dk x dv, 32 KB
constexpr int kTileVn = kTileS + 32768;            // [Vn ; 0]       128 x dv, 32 KB
constexpr int kTileDs = kTileVn + 32768;           // dS (bf16)      dk x dv, 32 KB
constexpr int kBwdTiles = kTileDs + 32768;         // 208 KB
constexpr int kBwdSmem = 1024 + kBwdTiles + 256;
constexpr int kBwdLoadBytes = 32768 + 16384 + 8192 + 16384 + 32768 + 16384;   // TMA bytes per chunk

struct BwdBars {
  uint64_t full, inputs_free, t1_full, w_ready, t2_full, ds_ready;
  uint32_t tmem_base;
  int abort_flag;
};

struct BwdArgs {
  int n_chunks;
  const float* e;
  const float* ds_final;
  __nv_bfloat16* d_kq;
  __nv_bfloat16* d_intra;
  __nv_bfloat16* d_kdec;
  __nv_bfloat16* d_veff;
  float* d_e;
  float* ds0;
  int* status;
};

struct BwdMaps {
  CUtensorMap kq, intra, kdec, d_o, s, vn;
};

__device__ __forceinline__ uint4 pack8(const uint32_t* v, float sign) {
  return make_uint4(pack_bf16x2(sign * __uint_as_float(v[0]), sign * __uint_as_float(v[1])),
                    pack_bf16x2(sign * __uint_as_float(v[2]), sign * __uint_as_float(v[3])),
                    pack_bf16x2(sign * __uint_as_float(v[4]), sign * __uint_as_float(v[5])),
                    pack_bf16x2(sign * __uint_as_float(v[6]), sign * __uint_as_float(v[7])));
}

__global__ void __launch_bounds__(kBwdThreads, 1)
gdn_scan_bwd_kernel(const __grid_constant__ BwdMaps tm, const __grid_constant__ BwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  BwdBars* bars = reinterpret_cast<BwdBars*>(smem + kBwdTiles);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x;
  const int N = a.n_chunks;

  if (threadIdx.x == 0) {
    mbar_init(&bars->full, 1);
    mbar_init(&bars->inputs_free, 1);
    mbar_init(&bars->t1_full, 1);
    mbar_init(&bars->w_ready, 128);
    mbar_init(&bars->t2_full, 1);
    mbar_init(&bars->ds_ready, 128);
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  // zero halves that stay zero: rows 64..127 of [kdec ; 0] and [Vn ; 0], the second column block of the intra tile
  for (int i = threadIdx.x; i < 512; i += kBwdThreads) {   // 8 KB = 512 x 16 B per zero region
    const uint4 z = make_uint4(0, 0, 0, 0);
    reinterpret_cast<uint4*>(smem + kTileKd + 8192)[i] = z;            // block 0, rows 64..127
    reinterpret_cast<uint4*>(smem + kTileKd + 16384 + 8192)[i] = z;    // block 1, rows 64..127
    reinterpret_cast<uint4*>(smem + kTileVn + 8192)[i] = z;
    reinterpret_cast<uint4*>(smem + kTileVn + 16384 + 8192)[i] = z;
    reinterpret_cast<uint4*>(smem + kTileIn + 8192)[i] = z;            // second 64-column block
  }
  fence_proxy_async_smem();
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  constexpr uint32_t kT1 = 0, kT2 = 128, kT3 = 256, kT4 = 320;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      for (int n = N - 1; n >= 0; --n, ++it) {
        // the previous chunk's products are done with the tiles (inputs_free) AND its epilogue has finished
        // reading S for d e (it then publishes dS for this chunk: ds_ready)
        if (it > 0 && (!mbar_wait(&bars->inputs_free, (it - 1) & 1, abort_flag) ||
                       !mbar_wait(&bars->ds_ready, it & 1, abort_flag))) {
          report_status(a.status, kWaitEmptyTimeout, 120, bh, n);
          break;
        }
        const int chunk = bh * N + n;
        mbar_arrive_expect_tx(&bars->full, kBwdLoadBytes);
        tma_load_2d(smem + kTileKq, &tm.kq, &bars->full, 0, chunk * 128);
        tma_load_2d(smem + kTileKq + 16384, &tm.kq, &bars->full, 64, chunk * 128);
        tma_load_2d(smem + kTileKd, &tm.kdec, &bars->full, 0, chunk * 64);
        tma_load_2d(smem + kTileKd + 16384, &tm.kdec, &bars->full, 64, chunk * 64);
        tma_load_2d(smem + kTileIn, &tm.intra, &bars->full, 0, chunk * 64);
        tma_load_2d(smem + kTileDw, &tm.d_o, &bars->full, 0, chunk * 64);
        tma_load_2d(smem + kTileDw + 16384, &tm.d_o, &bars->full, 64, chunk * 64);
        tma_load_2d(smem + kTileS, &tm.s, &bars->full, 0, chunk * 128);
        tma_load_2d(smem + kTileS + 16384, &tm.s, &bars->full, 64, chunk * 128);
        tma_load_2d(smem + kTileVn, &tm.vn, &bars->full, 0, chunk * 64);
        tma_load_2d(smem + kTileVn + 16384, &tm.vn, &bars->full, 64, chunk * 64);
      }
      if (*abort_flag && it > 0) {
        const uint64_t tw = globaltimer_ns();
        while (!mbar_try_wait(&bars->full, (it - 1) & 1) && globaltimer_ns() - tw < 2000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t i_kn = make_idesc(128, 128, 0, 1, 1);   // A K-major, B MN-major
    constexpr uint32_t i_nn = make_idesc(128, 128, 1, 1, 1);   // both MN-major
    constexpr uint32_t i_kk = make_idesc(128, 128, 0, 0, 1);   // both K-major
    constexpr uint32_t i_kk64 = make_idesc(128, 64, 0, 0, 1);
    const uint32_t b0 = smem_u32(smem);
    const uint32_t kq = b0 + kTileKq, kd = b0 + kTileKd, in = b0 + kTileIn, dw = b0 + kTileDw, ss = b0 + kTileS,
                   vn = b0 + kTileVn, ds = b0 + kTileDs;
    int it = 0;
    for (int n = N - 1; n >= 0; --n, ++it) {
      if (!mbar_wait(&bars->ds_ready, it & 1, abort_flag) || !mbar_wait(&bars->full, it & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitFullTimeout, 121, bh, n);
        break;
      }
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < 8; ++k)   // T1 = [kdec ; 0] dS      (K = dk)
          umma_bf16(tmem + kT1, make_smem_desc(kd + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                    make_smem_desc(ds + k * 2048, 16384, 1024), i_kn, k > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; ++k)   // T1 += [intra^T ; 0] dO  (K = 64 tokens)
          umma_bf16(tmem + kT1, make_smem_desc(in + k * 2048, 8192, 1024), make_smem_desc(dw + k * 2048, 16384, 1024),
                    i_nn, 1u);
        tc_commit(&bars->t1_full);
      }
      __syncwarp();
      if (!mbar_wait(&bars->w_ready, it & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitFullTimeout, 122, bh, n);
        break;
      }
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {   // K = dv
          const uint64_t a_dw = make_smem_desc(dw + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
          umma_bf16(tmem + kT2, a_dw, make_smem_desc(ss + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024), i_kk, k > 0 ? 1u : 0u);
          umma_bf16(tmem + kT3, a_dw, make_smem_desc(vn + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024), i_kk64, k > 0 ? 1u : 0u);
          umma_bf16(tmem + kT4, make_smem_desc(vn + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                    make_smem_desc(ds + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024), i_kk, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k)   // T5 = qg^T dO   (qg = rows 64..127 of the kq tile, K = tokens)
          umma_bf16(tmem + kT1, make_smem_desc(kq + 8192 + k * 2048, 16384, 1024), make_smem_desc(dw + k * 2048, 16384, 1024),
                    i_nn, k > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; ++k)   // T5 += k_cum^T W (W = rows 64..127 of the [dO ; W] tile)
          umma_bf16(tmem + kT1, make_smem_desc(kq + k * 2048, 16384, 1024),
                    make_smem_desc(dw + 8192 + k * 2048, 16384, 1024), i_nn, 1u);
        tc_commit(&bars->inputs_free);
        tc_commit(&bars->t2_full);
      }
      __syncwarp();
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    uint8_t* t_ds = smem + kTileDs;
    float dS[kDv];
    if (a.ds_final != nullptr) {
      const float4* sp = reinterpret_cast<const float4*>(a.ds_final + (static_cast<int64_t>(bh) * kDk + r) * kDv);
#pragma unroll
      for (int j = 0; j < kDv / 4; ++j) {
        const float4 f = sp[j];
        dS[4 * j] = f.x; dS[4 * j + 1] = f.y; dS[4 * j + 2] = f.z; dS[4 * j + 3] = f.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < kDv; ++j) dS[j] = 0.f;
    }
    bool ok = true;
    int it = 0;
    for (int n = N - 1; n >= -1; --n, ++it) {
      // ---- publish dS (bf16) for the chunk's products ----
#pragma unroll
      for (int c = 0; c < kDv; c += 8)
        *reinterpret_cast<uint4*>(t_ds + swz(r, c, 16384)) =
            make_uint4(pack_bf16x2(dS[c], dS[c + 1]), pack_bf16x2(dS[c + 2], dS[c + 3]), pack_bf16x2(dS[c + 4], dS[c + 5]),
                       pack_bf16x2(dS[c + 6], dS[c + 7]));
      fence_proxy_async_smem();
      if (n < 0) break;
      mbar_arrive(&bars->ds_ready);
      const int64_t chunk = static_cast<int64_t>(bh) * N + n;
      const float e = a.e[chunk];
      if (ok && !mbar_wait(&bars->t1_full, it & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitTmemFullTimeout, 123, bh, n);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (ok && r < kC) {
        tc_fence_after();
        uint4* dve = reinterpret_cast<uint4*>(a.d_veff + (chunk * kC + r) * kDv);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tmem + kT1 + c * 32 + lane_off, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            dve[c * 4 + (j >> 3)] = pack8(v + j, 1.f);
            *reinterpret_cast<uint4*>(smem + kTileDw + swz(64 + r, c * 32 + j, 16384)) = pack8(v + j, -1.f);
          }
        }
        tc_fence_before();
        fence_proxy_async_smem();
      }
      mbar_arrive(&bars->w_ready);
      if (ok && !mbar_wait(&bars->t2_full, it & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitTmemFullTimeout, 124, bh, n);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) continue;
      tc_fence_after();
      // T2: rows 0..63 -> d qg (stored at rows 64..127 of d_kq), rows 64..127 -> d k_cum (rows 0..63)
      {
        uint4* dst = reinterpret_cast<uint4*>(a.d_kq + (chunk * 128 + (r < kC ? r + kC : r - kC)) * kDk);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tmem + kT2 + c * 32 + lane_off, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j += 8) dst[c * 4 + (j >> 3)] = pack8(v + j, 1.f);
        }
      }
      if (r < kC) {
        uint4* di = reinterpret_cast<uint4*>(a.d_intra + (chunk * kC + r) * kC);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tmem + kT3 + c * 32 + lane_off, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j += 8) di[c * 4 + (j >> 3)] = pack8(v + j, 1.f);
        }
        uint4* dk = reinterpret_cast<uint4*>(a.d_kdec + (chunk * kC + r) * kDk);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tmem + kT4 + c * 32 + lane_off, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j += 8) dk[c * 4 + (j >> 3)] = pack8(v + j, 1.f);
        }
      }
      // d e = <dS, S> with the dS that entered the chunk; then dS <- e dS + T5
      float de = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tmem + kT1 + c * 32 + lane_off, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          const uint4 sv = *reinterpret_cast<const uint4*>(smem + kTileS + swz(r, c * 32 + j, 16384));
          const float2 s0 = unpack_bf16x2(sv.x), s1 = unpack_bf16x2(sv.y), s2 = unpack_bf16x2(sv.z), s3 = unpack_bf16x2(sv.w);
          const float sf[8] = {s0.x, s0.y, s1.x, s1.y, s2.x, s2.y, s3.x, s3.y};
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            const int col = c * 32 + j + t;
            de += dS[col] * sf[t];
            dS[col] = dS[col] * e + __uint_as_float(v[j + t]);
          }
        }
      }
      tc_fence_before();
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) de += __shfl_xor_sync(0xffffffffu, de, o);
      if (lane == 0) atomicAdd(a.d_e + chunk, de);
    }
    if (ok) {
      float4* sp = reinterpret_cast<float4*>(a.ds0 + (static_cast<int64_t>(bh) * kDk + r) * kDv);
#pragma unroll
      for (int j = 0; j < kDv / 4; ++j) sp[j] = make_float4(dS[4 * j], dS[4 * j + 1], dS[4 * j + 2], dS[4 * j + 3]);
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

cudaError_t launch_gdn_scan_bwd(const __nv_bfloat16* kq, const __nv_bfloat16* intra, const __nv_bfloat16* kdec,
                                const __nv_bfloat16* s_save, const __nv_bfloat16* vn_save, const float* e,
                                const __nv_bfloat16* d_o, const float* ds_final, __nv_bfloat16* d_kq,
                                __nv_bfloat16* d_intra, __nv_bfloat16* d_kdec, __nv_bfloat16* d_veff, float* d_e, float* ds0,
                                int bh, int n_chunks, int* status, cudaStream_t stream) {
  if (bh < 1 || n_chunks < 1) return cudaErrorInvalidValue;
  BwdMaps tm;
  cudaError_t err;
  const uint64_t chunks = static_cast<uint64_t>(bh) * n_chunks;
  if ((err = encode_tma_2d(&tm.kq, kq, 2, kDk, chunks * 128, kDk * 2ull, 64, 128)) != cudaSuccess) return err;
  if ((err = encode_tma_2d(&tm.intra, intra, 2, kC, chunks * kC, kC * 2ull, 64, 64)) != cudaSuccess) return err;
  if ((err = encode_tma_2d(&tm.kdec, kdec, 2, kDk, chunks * kC, kDk * 2ull, 64, 64)) != cudaSuccess) return err;
  if ((err = encode_tma_2d(&tm.d_o, d_o, 2, kDv, chunks * kC, kDv * 2ull, 64, 64)) != cudaSuccess) return err;
  if ((err = encode_tma_2d(&tm.s, s_save, 2, kDv, chunks * kDk, kDv * 2ull, 64, 128)) != cudaSuccess) return err;
  if ((err = encode_tma_2d(&tm.vn, vn_save, 2, kDv, chunks * kC, kDv * 2ull, 64, 64)) != cudaSuccess) return err;
  static bool configured = false;
  if (!configured) {
    if ((err = cudaFuncSetAttribute(gdn_scan_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem)) != cudaSuccess)
      return err;
    configured = true;
  }
  BwdArgs args{n_chunks, e, ds_final, d_kq, d_intra, d_kdec, d_veff, d_e, ds0, status};
  gdn_scan_bwd_kernel<<<bh, kBwdThreads, kBwdSmem, stream>>>(tm, args);
  return cudaGetLastError();
}

}  // namespace b200

namespace b200 {

cudaError_t launch_gdn_gated_norm(const __nv_bfloat16* o, const __nv_bfloat16* z, const float* w, __nv_bfloat16* y, int B,
                                  int T, int Tpad, int Hv, float eps, cudaStream_t stream) {
  if (B < 1 || T < 1 || Tpad < T || Hv < 1) return cudaErrorInvalidValue;
  const int rows = B * T * Hv;
  gdn_gated_norm_kernel<<<(rows + 7) / 8, 256, 0, stream>>>(o, z, w, y, rows, T, Tpad, Hv, eps);
  return cudaGetLastError();
}

cudaError_t launch_gdn_gated_norm_bwd(const __nv_bfloat16* o, const __nv_bfloat16* z, const float* w,
                                      const __nv_bfloat16* dy, __nv_bfloat16* d_o, __nv_bfloat16* dz, float* dw, int B,
                                      int T, int Tpad, int Hv, float eps, cudaStream_t stream) {
  if (B < 1 || T < 1 || Tpad < T || Hv < 1) return cudaErrorInvalidValue;
  const int rows = B * T * Hv;
  const int blocks = (rows + 7) / 8 < 148 * 8 ? (rows + 7) / 8 : 148 * 8;
  gdn_gated_norm_bwd_kernel<<<blocks, 256, 0, stream>>>(o, z, w, dy, d_o, dz, dw, rows, T, Tpad, Hv, eps);
  return cudaGetLastError();
}

}  // namespace b200
