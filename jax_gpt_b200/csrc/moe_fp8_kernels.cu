// Expert-parallel MoE forward in FP8 with tensor-core block scaling, ONE cooperative kernel per rank.
//
// Same protocol as the bf16 kernel (moe_kernels.cu: count exchange, push dispatch, arrival counters,
// static tile order, in-flight weighted combine) with the data path of the block-scaled GEMM
// (gemm_mxfp8_sm100.cu):
//   0. every token row is quantised ONCE to e4m3 with power-of-two 1 x 128 scales into local staging;
//   1. dispatch pushes the byte rows (half the bf16 traffic) and, per row and 128-wide slab, one 32-bit
//      word of UE8M0 exponents straight into the destination's packed scale chunks;
//   2. GEMM 1: tcgen05 kind::mxf8f6f4.block_scale over [gate | up] tiles; the eight epilogue warps drain
//      the accumulator into registers, apply SiLU(gate) * up, find the 1 x 128 amax of the row, and write
//      the e4m3 activation with its exponent word;
//   3. GEMM 2 on the quantised activation; the epilogue scales rows by their routing weight and adds
//      them into the owner's fp32 output with coalesced red.add over NVLink.
// B tile of GEMM 1 (256 rows of [E, I, D] weights): rows 0-63 gate[n*128 .. +64], 64-127 up[same],
// 128-191 gate[n*128+64 ..], 192-255 up[same], so that each half of the accumulator holds matching
// gate / up columns for one epilogue warp; both halves share one packed scale chunk.
#include "moe_kernels.cuh"

#include <cooperative_groups.h>

#include "comm_device.cuh"
#include "common.cuh"
#include "moe_common.cuh"
#include "tma_host.h"

namespace cg = cooperative_groups;

namespace b200 {

namespace {

constexpr int BM = 128, BN = 256, BK = 128;         // BK in bytes == e4m3 elements
constexpr int kStages = 3;
constexpr int kABytes = BM * BK, kBBytes = BN * BK;
constexpr int kSfBytes = 512;
constexpr int kStageBytes = kABytes + kBBytes;      // 48 KB
constexpr int kStageSf = 3 * kSfBytes;
constexpr int kThreads = 320;                       // producer, MMA, 8 epilogue warps
constexpr int kSfCol0 = 256;
constexpr int kPad = 128;                           // expert regions start on scale-chunk boundaries

struct Fp8Bars {
  uint64_t full[kStages], empty[kStages], tmem_full, tmem_empty, pair[4];
  uint32_t tmem_base;
  int abort_flag;
  float amax[2][4][2][32];                          // [tile parity][lane quarter][accumulator half][row]
};

constexpr int kStageBufBytes = 8 * 32 * 33 * 4;
constexpr int kSmemBytes = 1024 + kStages * (kStageBytes + kStageSf) + sizeof(MoeTables) + sizeof(Fp8Bars) + 64 + kStageBufBytes;

// 2^ceil(log2(amax / 448)) as (scale, biased exponent byte); amax == 0 -> scale 1.
__device__ __forceinline__ float pow2_scale(float amax, uint32_t* exp_byte) {
  if (!(amax > 0.f)) {
    *exp_byte = 127u;
    return 1.f;
  }
  const float s = amax * (1.f / 448.f);
  uint32_t bits = __float_as_uint(s);
  uint32_t e = (bits >> 23) & 0xff;
  if (bits & 0x7fffff) ++e;          // round the scale up to the next power of two
  e = e < 1u ? 1u : (e > 254u ? 254u : e);
  *exp_byte = e;
  return __uint_as_float(e << 23);
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

struct Fp8Maps {
  CUtensorMap recv, act, gate, up, down;
};

__global__ void __launch_bounds__(kThreads, 1)
ep_moe_forward_fp8_kernel(const __grid_constant__ Fp8Maps tm, const __grid_constant__ EpMoeFp8Args a) {
  cg::grid_group grid = cg::this_grid();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sf_smem = smem + kStages * kStageBytes;
  MoeTables* tb = reinterpret_cast<MoeTables*>(sf_smem + kStages * kStageSf);
  Fp8Bars* bars = reinterpret_cast<Fp8Bars*>(reinterpret_cast<uint8_t*>(tb) + ((sizeof(MoeTables) + 15) & ~size_t(15)));
  volatile int* abort_flag = &bars->abort_flag;
  float* stage_buf = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + ((sizeof(Fp8Bars) + 15) & ~size_t(15)));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int W = a.world, EL = a.e_local, ET = W * EL, D = a.d_model, I = a.inter;
  const int dslabs = D / 128, islabs = I / 128;
  CommCtrl* my = a.peer_ctrl[a.rank];
  const int epoch = my->epoch + 1;
  const int gwarp = blockIdx.x * (kThreads / 32) + warp, gwarps = gridDim.x * (kThreads / 32);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->tmem_full, 1);
    mbar_init(&bars->tmem_empty, 8);
    for (int i = 0; i < 4; ++i) mbar_init(&bars->pair[i], 64);
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

  // ---- 0. quantise this rank's token rows once (one warp per row, one 128-group per step) ----
  for (int tok = gwarp; tok < a.tokens; tok += gwarps) {
    const uint2* src = reinterpret_cast<const uint2*>(a.x + static_cast<int64_t>(tok) * D);
    uint32_t* dst = reinterpret_cast<uint32_t*>(a.xq + static_cast<int64_t>(tok) * D);
    for (int g = 0; g < dslabs; ++g) {
      const uint2 u = src[g * 32 + lane];
      const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y);
      float m = fmaxf(fmaxf(fabsf(f0.x), fabsf(f0.y)), fmaxf(fabsf(f1.x), fabsf(f1.y)));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      uint32_t eb;
      const float inv = 1.f / pow2_scale(m, &eb);
      dst[g * 32 + lane] = pack_e4m3x4(f0.x * inv, f0.y * inv, f1.x * inv, f1.y * inv);
      if (lane == 0) a.xe[static_cast<int64_t>(tok) * dslabs + g] = static_cast<uint8_t>(eb);
    }
  }

  // ---- 1. publish this rank's counts, wait for everybody's ----
  {
    const int max_mt = a.cap_rows / BM + EL;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < max_mt; i += gridDim.x * blockDim.x) a.act_ready[i] = 0;
  }
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) my->abort_flag = 0;
    for (int i = threadIdx.x; i < ET; i += blockDim.x) {
      const int c = a.my_counts[i];
      for (int p = 0; p < W; ++p) a.peer_counts[p][a.rank * ET + i] = c;
    }
    const bool ok = flag_barrier(a.peer_ctrl, W, a.rank, 4, epoch, a.wait_budget_ns, a.status);
    if (!ok && threadIdx.x == 0) my->abort_flag = 1;
  }
  __threadfence();
  grid.sync();   // also orders the staging rows of step 0 before the dispatch reads them
  bool alive = (*reinterpret_cast<volatile int*>(&my->abort_flag) == 0);
  build_tables(a, a.peer_counts[a.rank], tb, false, kPad);
  if (tb->overflow) {
    if (alive && blockIdx.x == 0 && threadIdx.x == 0) report_status(a.status, kBadArgument, 90, a.cap_rows, 0);
    alive = false;
  }

  // ---- 2. dispatch: one warp per (token, expert) pair: byte row + exponent words. Two rows per pass with eight
  //         16-byte loads per lane and row in flight before the first store; one fence per warp after all its rows,
  //         then their arrival counts (barrier -> fence -> relaxed reduction is a release sequence over every
  //         lane's stores). ----
  if (alive) {
    const int n_pairs = a.tokens * a.top_k, nv = D / 16;
    constexpr int kBatch = 8;
    for (int p = gwarp; p < n_pairs; p += 2 * gwarps) {
      const uint4* src[2] = {nullptr, nullptr};
      uint4* out[2] = {nullptr, nullptr};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int pp = p + h * gwarps;
        if (pp >= n_pairs) continue;
        const int e = a.idx[pp];
        if (!bounds_ok(e, ET, a.status, 211)) continue;
        const int dst = e / EL;
        const int slot = tb->send_off[e] + a.pos[pp];
        if (!bounds_ok(slot, a.cap_rows, a.status, 212)) continue;
        const int tok = pp / a.top_k;
        src[h] = reinterpret_cast<const uint4*>(a.xq + static_cast<int64_t>(tok) * D);
        out[h] = reinterpret_cast<uint4*>(a.peer_recv_q[dst] + static_cast<int64_t>(slot) * D);
        // scale exponents: chunk (slot / 128, g), word at (r % 32) * 16 + (r / 32) * 4 with r = slot % 128
        const int r = slot & 127;
        uint8_t* sfrow = a.peer_recv_sf[dst] + static_cast<int64_t>(slot >> 7) * dslabs * kSfBytes + (r & 31) * 16 + (r >> 5) * 4;
        const uint8_t* xe = a.xe + static_cast<int64_t>(tok) * dslabs;
        for (int g = lane; g < dslabs; g += 32) {
          const uint32_t eb = __ldcg(xe + g);
          *reinterpret_cast<uint32_t*>(sfrow + static_cast<int64_t>(g) * kSfBytes) = eb * 0x01010101u;
        }
        if (lane == 0) {
          a.peer_recv_meta[dst][slot] = (a.rank << 24) | pp;
          a.peer_recv_w[dst][slot] = a.w[pp];
          a.slot_out[pp] = slot;
        }
      }
      for (int i0 = lane; i0 < nv; i0 += 32 * kBatch) {
        uint4 v[2][kBatch];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int u = 0; u < kBatch; ++u)
            if (src[h] != nullptr && i0 + 32 * u < nv) v[h][u] = __ldcg(src[h] + i0 + 32 * u);
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int u = 0; u < kBatch; ++u)
            if (src[h] != nullptr && i0 + 32 * u < nv) out[h][i0 + 32 * u] = v[h][u];
      }
    }
    __syncwarp();
    __threadfence_system();
    int j = 0;
    for (int p = gwarp; p < n_pairs; p += gwarps, ++j) {
      if ((j & 31) != lane) continue;
      const int e = a.idx[p];
      if (e < 0 || e >= ET || tb->send_off[e] + a.pos[p] >= a.cap_rows) continue;  // skipped (and reported) above
      red_relaxed_sys_add_u32(a.peer_arrive[e / EL] + (e % EL), 1u);
    }
  }

  // ---- 3./4. grouped GEMMs over the local experts ----
  const int num_tiles = alive ? tb->tile0[tb->n_slots] : 0;
  const int n1 = I / 128;
  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int ready_el = -1;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const TileInfo ti = decode_tile(a, tb, t);
        if (ti.phase == 0) {
          if (ti.el != ready_el) {
            const unsigned target = a.arrive_target[ti.el] + static_cast<unsigned>(tb->rows[ti.el]);
            if (!wait_counter_ge<true>(a.peer_arrive[a.rank] + ti.el, target, a.wait_budget_ns, abort_flag)) {
              report_status(a.status, kWaitFlagTimeout, 91, ti.el, t);
              break;
            }
            ready_el = ti.el;
          }
        } else {
          const unsigned* ready = reinterpret_cast<const unsigned*>(a.act_ready) + tb->mt0[ti.el] + ti.m;
          if (!wait_counter_ge<false>(ready, 8u * n1, a.wait_budget_ns, abort_flag)) {
            report_status(a.status, kWaitFlagTimeout, 92, ti.el, t);
            break;
          }
        }
        fence_proxy_async_global();
        const int row0 = tb->base[ti.el] + ti.m * BM;
        const int chunk_row = row0 >> 7;
        const int nslab = ti.phase == 0 ? dslabs : islabs;
        for (int s = 0; s < nslab; ++s) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag)) {
            report_status(a.status, kWaitEmptyTimeout, 93, blockIdx.x, t);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          uint8_t* sf = sf_smem + stage * kStageSf;
          uint64_t* fb = &bars->full[stage];
          if (ti.phase == 0) {
            mbar_arrive_expect_tx(fb, kStageBytes + 2 * kSfBytes);
            tma_load_2d(sa, &tm.recv, fb, s * BK, row0);
            const int wr = ti.el * I + ti.n * 128;
            tma_load_2d(sb, &tm.gate, fb, s * BK, wr);
            tma_load_2d(sb + 8192, &tm.up, fb, s * BK, wr);
            tma_load_2d(sb + 16384, &tm.gate, fb, s * BK, wr + 64);
            tma_load_2d(sb + 24576, &tm.up, fb, s * BK, wr + 64);
            bulk_load_1d(sf, a.peer_recv_sf[a.rank] + (static_cast<int64_t>(chunk_row) * dslabs + s) * kSfBytes, kSfBytes, fb);
            bulk_load_1d(sf + kSfBytes,
                         a.sfb1 + ((static_cast<int64_t>(ti.el) * n1 + ti.n) * dslabs + s) * kSfBytes, kSfBytes, fb);
          } else {
            mbar_arrive_expect_tx(fb, kStageBytes + 3 * kSfBytes);
            tma_load_2d(sa, &tm.act, fb, s * BK, row0);
            const int wr = ti.el * D + ti.n * BN;
#pragma unroll
            for (int i = 0; i < 4; ++i) tma_load_2d(sb + i * 8192, &tm.down, fb, s * BK, wr + 64 * i);
            bulk_load_1d(sf, a.act_sf + (static_cast<int64_t>(chunk_row) * islabs + s) * kSfBytes, kSfBytes, fb);
            const int64_t nb = static_cast<int64_t>(ti.el) * (D / 128) + 2 * ti.n;
            bulk_load_1d(sf + kSfBytes, a.sfb2 + (nb * islabs + s) * kSfBytes, kSfBytes, fb);
            bulk_load_1d(sf + 2 * kSfBytes, a.sfb2 + ((nb + 1) * islabs + s) * kSfBytes, kSfBytes, fb);
          }
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
      const TileInfo ti = decode_tile(a, tb, t);
      if (!mbar_wait(&bars->tmem_empty, (iter & 1) ^ 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitTmemEmptyTimeout, 94, blockIdx.x, t);
        break;
      }
      tc_fence_after();
      const int nslab = ti.phase == 0 ? dslabs : islabs;
      for (int s = 0; s < nslab; ++s) {
        if (!mbar_wait(&bars->full[stage], phase, abort_flag)) {
          if (lane == 0) report_status(a.status, kWaitFullTimeout, 95, blockIdx.x, t);
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
          // GEMM 1: both halves of the B tile share one chunk; GEMM 2: the second 128 weight rows have their own
          tmem_cp_sf(tsf + 8, make_sf_desc(sf + (ti.phase == 0 ? kSfBytes : 2 * kSfBytes)));
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
    // ---------------- eight epilogue warps: (lane quarter q, accumulator half) ----------------
    const int ew = warp - 2;
    const int q = warp & 3;
    const int half = ew >> 2;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    float* stg = stage_buf + ew * (32 * 33);
    int iter = 0, g1_iter = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++iter) {
      const TileInfo ti = decode_tile(a, tb, t);
      if (!mbar_wait(&bars->tmem_full, iter & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitTmemFullTimeout, 96, blockIdx.x, t);
        break;
      }
      tc_fence_after();
      uint32_t v[4][32];
      const uint32_t taddr = tmem_base + half * 128 + lane_off;
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(taddr + c * 32, v[c]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty);   // accumulator drained: the next tile's main loop may start
      const int r = ti.m * BM + q * 32 + lane;            // row within the expert
      const bool row_ok = r < tb->rows[ti.el];
      const int64_t row = tb->base[ti.el] + r;            // row in the receive buffer
      if (ti.phase == 0) {
        // v[0..1] = 64 gate columns, v[2..3] = the matching 64 up columns
        float m = 0.f;
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float g = __uint_as_float(v[c][j]), u = __uint_as_float(v[c + 2][j]);
            const float act = g / (1.f + __expf(-g)) * u;
            v[c][j] = __float_as_uint(act);
            m = fmaxf(m, fabsf(act));
          }
        // the 1 x 128 quantisation group spans both halves: exchange the row maxima with the partner warp
        const int par = g1_iter & 1;
        float* slot = &bars->amax[par][0][0][0];
        slot[(q * 2 + half) * 32 + lane] = m;
        mbar_arrive(&bars->pair[q]);
        if (!mbar_wait(&bars->pair[q], g1_iter & 1, abort_flag)) {
          if (lane == 0) report_status(a.status, kWaitFlagTimeout, 97, blockIdx.x, t);
          break;
        }
        ++g1_iter;
        m = fmaxf(m, slot[(q * 2 + (half ^ 1)) * 32 + lane]);
        uint32_t eb;
        const float inv = 1.f / pow2_scale(m, &eb);
        if (row_ok) {
          uint4* dst = reinterpret_cast<uint4*>(a.act_q + row * I + ti.n * 128 + half * 64);
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int j = 0; j < 32; j += 16) {
              uint32_t w4[4];
#pragma unroll
              for (int k = 0; k < 4; ++k)
                w4[k] = pack_e4m3x4(__uint_as_float(v[c][j + 4 * k]) * inv, __uint_as_float(v[c][j + 4 * k + 1]) * inv,
                                    __uint_as_float(v[c][j + 4 * k + 2]) * inv, __uint_as_float(v[c][j + 4 * k + 3]) * inv);
              dst[c * 2 + (j >> 4)] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
            }
          if (half == 0) {
            const int rr = static_cast<int>(row & 127);
            uint8_t* sfp = a.act_sf + (static_cast<int64_t>(row >> 7) * islabs + ti.n) * kSfBytes + (rr & 31) * 16 + (rr >> 5) * 4;
            *reinterpret_cast<uint32_t*>(sfp) = eb * 0x01010101u;
          }
        }
        __threadfence();
        fence_proxy_async_global();
        __syncwarp();
        if (lane == 0) atomicAdd(a.act_ready + tb->mt0[ti.el] + ti.m, 1);
      } else {
        // weighted combine with coalesced fp32 reductions into the token owners' rows
        float wgt = 0.f;
        float* dst = nullptr;
        if (row_ok) {
          wgt = a.peer_recv_w[a.rank][row];
          const int meta = a.peer_recv_meta[a.rank][row];
          if (bounds_ok(meta >> 24, W, a.status, 213) && bounds_ok(meta & 0xFFFFFF, a.tokens * a.top_k, a.status, 214))
            dst = a.peer_out[meta >> 24] + static_cast<int64_t>((meta & 0xFFFFFF) / a.top_k) * D + ti.n * BN + half * 128;
        }
        const unsigned long long dst_bits = reinterpret_cast<unsigned long long>(dst);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int j = 0; j < 32; ++j) stg[lane * 33 + j] = __uint_as_float(v[c][j]) * wgt;
          __syncwarp();
#pragma unroll
          for (int rr = 0; rr < 32; rr += 4) {
            const int r2 = rr + (lane >> 3), c2 = (lane & 7) * 4;
            const unsigned long long db = __shfl_sync(0xffffffffu, dst_bits, r2);
            if (db != 0ull) {
              float* d2 = reinterpret_cast<float*>(db) + c * 32 + c2;
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d2), "f"(stg[r2 * 33 + c2]),
                           "f"(stg[r2 * 33 + c2 + 1]), "f"(stg[r2 * 33 + c2 + 2]), "f"(stg[r2 * 33 + c2 + 3])
                           : "memory");
            }
          }
          __syncwarp();
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  __threadfence_system();
  grid.sync();
  if (blockIdx.x == 0) {
    flag_barrier(a.peer_ctrl, W, a.rank, 5, epoch, a.wait_budget_ns, a.status);
    if (alive) {
      for (int el = threadIdx.x; el < EL; el += blockDim.x) {
        a.arrive_target[el] += static_cast<unsigned>(tb->rows[el]);
        a.rows_out[el] = tb->rows[el];
      }
    }
    if (threadIdx.x == 0) my->epoch = epoch;
  }
}

}  // namespace

cudaError_t launch_ep_moe_forward_fp8(const EpMoeFp8Args& args, const uint8_t* gate_q, const uint8_t* up_q,
                                      const uint8_t* down_q, cudaStream_t st) {
  const EpMoeFp8Args& a = args;
  if (a.world < 1 || a.world > kCommMaxRanks || a.e_local < 1 || a.e_local > kMoeMaxLocalExperts ||
      a.world * a.e_local > kMoeMaxExperts || a.d_model % 256 != 0 || a.inter % 128 != 0 || a.cap_rows % BM != 0 ||
      static_cast<int64_t>(a.tokens) * a.top_k >= (1 << 24))
    return cudaErrorInvalidValue;
  Fp8Maps tm;
  cudaError_t e;
  const uint64_t D = a.d_model, I = a.inter, EL = a.e_local, cap = a.cap_rows;
  if ((e = encode_tma_2d(&tm.recv, a.peer_recv_q[a.rank], 1, D, cap, D, 128, BM)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tm.act, a.act_q, 1, I, cap, I, 128, BM)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tm.gate, gate_q, 1, D, EL * I, D, 128, 64)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tm.up, up_q, 1, D, EL * I, D, 128, 64)) != cudaSuccess) return e;
  if ((e = encode_tma_2d(&tm.down, down_q, 1, I, EL * D, I, 128, 64)) != cudaSuccess) return e;
  static bool configured = false;
  if (!configured) {
    if ((e = cudaFuncSetAttribute(ep_moe_forward_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes)) != cudaSuccess)
      return e;
    configured = true;
  }
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  EpMoeFp8Args args_copy = args;
  void* params[] = {&tm, &args_copy};
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(ep_moe_forward_fp8_kernel), dim3(sms), dim3(kThreads), params,
                                     kSmemBytes, st);
}

}  // namespace b200
