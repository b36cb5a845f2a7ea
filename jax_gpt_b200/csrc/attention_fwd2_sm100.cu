// Flash attention forward for head width 64 on tcgen05: a PERSISTENT kernel with two 128-row query tiles per
// work item that take turns on the tensor core and on the exponential unit.
//
// A work item is 256 consecutive queries of one (batch, head). Each CTA (one per SM) walks a static list of
// items, heaviest first, without draining between them. One warp streams Q (two slots), K and V (two independent
// three-deep rings) with TMA and runs ahead into the next item; one warp issues every MMA; warps 0..3 are the
// softmax group of query tile 0 and warps 4..7 the group of query tile 1.
//
// A softmax thread owns one whole score row. It pulls the 128 scores of a tile into registers with one wait,
// frees the score columns at once (so S of the NEXT key tile is computed while this one is exponentiated), and
// hands P back through 128B-swizzled shared memory. The output tile stays in TMEM across key tiles: P V
// accumulates there, and the stale-maximum trick keeps it exact: a row's reference maximum is only raised when
// the true maximum grew by more than 2^8, in which case that warp rescales its 32 rows of O in TMEM (rare after
// the first tiles); otherwise probabilities are formed against the old reference, at most 256, and the row sum
// uses the same reference. Each tile's MMA warp runs one key tile ahead with the scores (S' before P V).
// The two groups alternate strictly on the exponential phase (a pair of "turn" barriers): left alone they fall
// into lockstep, both waiting on the MUFU at the same time and both leaving it idle while they load and reduce.
//
// Keys and values may come from a token-major activation ([B*Tk, Hkv*D]) or straight from a cache laid out as
// (B, Hkv, max_len, D); queries sit at positions q_pos0 + i, which makes the same kernel the prefill-with-cache
// path (the reference attends over the whole zero-padded cache and masks: jax_gpt/models/qwen35/gqa.py:88-119).
#include "attention_sm100.cuh"

#include "common.cuh"
#include "tma_host.h"

namespace b200 {

namespace {

// Warps 0..3: softmax group of query tile 0; 4..7: group of tile 1; 8: TMA; 9 and 10: the MMA warps of query
// tile 0 and 1; 11 idle. The groups are whole warpgroups so that they can take registers from the third one
// (setmaxnreg): a softmax thread keeps a 128-column score row in registers. Each query tile has its OWN MMA
// warp: a thread that issues a burst of tcgen05.mma is held for the burst (about 170 cycles until the first one
// is accepted, then the execution time of the others), so one issuing thread for both tiles would serialise them.
constexpr int kThreads2 = 384;
constexpr int kWarpTma = 8, kWarpMma = 9;   // MMA warps: kWarpMma + group
constexpr float kLog2e2 = 1.4426950408889634f;
constexpr int kRing = 3;
constexpr float kRescaleGap = 8.f;   // log2 units a row maximum may lag behind before O is rescaled

struct Fwd2Args {
  int B, Tq, Tk, H, Hkv;
  int q_pos0;               // position of query 0 (causal rule: key position <= q_pos0 + query index)
  int kv_rows_b, kv_rows_h; // row of key 0 of (b, hkv) in the K / V matrices = b * kv_rows_b + hkv * kv_rows_h
  int k_col_h, v_col_h;     // first column of kv head hkv in K / V = hkv * {k,v}_col_h
  int n_pairs, n_items;     // query-tile pairs per sequence; work items = n_pairs * H * B
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
  static constexpr int kOffQ = 0;                    // two slots of {Q0, Q1}
  static constexpr int kOffK = 4 * kTile;            // ring of K tiles
  static constexpr int kOffV = kOffK + kRing * kTile;
  static constexpr int kOffP = kOffV + kRing * kTile;  // P0, P1
  static constexpr int kOffBar = kOffP + 2 * kPBytes;
  static constexpr int kSmem = kOffBar + 512;
  static constexpr int kColS = 0;                    // S0 [0,128), S1 [128,256)
  static constexpr int kColO = 256;                  // O0 [256,256+D), O1 [256+D, 256+2D)
  static_assert(kSmem <= 232448, "shared memory");
};

struct Fwd2Bars {
  uint64_t q_full[2], q_empty[2], k_full[kRing], k_empty[kRing], v_full[kRing], v_empty[kRing];
  uint64_t s_full[2], s_free[2], p_ready[2], o_full[2], o_free[2];
  uint64_t turn[2];   // the two softmax groups take turns on the exponential unit
  uint32_t tmem_base;
  int abort_flag;
};

struct Item {
  int pair, h, b, hkv;
  int nkv[2];
  int n_max;
};

// Work item of CTA `cta` in round `round`. Items are sorted heaviest first and dealt out in snake order (left to
// right, then right to left), which keeps the per-CTA sums of key tiles within a few tiles of each other.
__device__ __forceinline__ int item_index(int round, int cta, int n_ctas) {
  return round * n_ctas + ((round & 1) ? n_ctas - 1 - cta : cta);
}

__device__ __forceinline__ Item decode_item(const Fwd2Args& a, int idx) {
  Item it;
  const int hb = a.H * a.B;
  it.pair = a.n_pairs - 1 - idx / hb;       // heaviest pairs first
  const int r = idx % hb;
  it.h = r % a.H;
  it.b = r / a.H;
  it.hkv = it.h / (a.H / a.Hkv);
  const int n_kv_all = (a.Tk + 127) / 128;
  const int n_q_tiles = (a.Tq + 127) / 128;
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    const int t = 2 * it.pair + g;
    if (t >= n_q_tiles) it.nkv[g] = 0;
    else if (a.causal) it.nkv[g] = min((a.q_pos0 + t * 128 + 127) / 128 + 1, n_kv_all);
    else it.nkv[g] = n_kv_all;
  }
  it.n_max = max(it.nkv[0], it.nkv[1]);
  return it;
}

__device__ __forceinline__ void store_p_chunk(uint8_t* tile, int r, int c0, const uint32_t (&pk)[16]) {
  uint8_t* base = tile + (c0 >> 6) * 16384 + r * 128;
  const int chunk0 = (c0 & 63) >> 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int phys = (chunk0 + i) ^ (r & 7);
    *reinterpret_cast<uint4*>(base + phys * 16) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
  }
}

template <int D>
struct MmaCtx {
  Fwd2Bars* bars;
  volatile int* abort_flag;
  int* status;
  uint32_t tmem;
  int lane;
  uint64_t dK0, dV0, dP[2];   // descriptors of ring stage 0 / of the two P tiles
};

// S_G = Q_G K^T for the key tile in ring stage `st` into the group's score columns. The columns are free once the
// group has pulled the previous tile into registers (s_free). Releases the K stage (one of two arrivals) and, with
// the item's last score tile of this group, the Q slot.
template <int D, int G>
__device__ __forceinline__ bool mma_issue_s(const MmaCtx<D>& c, uint64_t dQ, uint32_t st, uint32_t ph, uint32_t& ns,
                                            uint64_t* q_empty) {
  using C = Fwd2Cfg<D>;
  if (!mbar_wait(&c.bars->k_full[st], ph, c.abort_flag) ||
      (ns > 0 && !mbar_wait(&c.bars->s_free[G], (ns - 1) & 1, c.abort_flag))) {
    if (c.lane == 0) report_status(c.status, kWaitFullTimeout, 113, G, static_cast<int>(ns));
    return false;
  }
  tc_fence_after();
  if (c.lane == 0) {
    constexpr uint32_t idesc_s = make_idesc(128, 128, 0, 0, 1);
    const uint64_t dK = c.dK0 + static_cast<uint64_t>(st) * (C::kTile >> 4);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
      umma_bf16(c.tmem + C::kColS + G * 128, dQ + 2 * kk, dK + 2 * kk, idesc_s, kk > 0);
    tc_commit(&c.bars->s_full[G]);
    tc_commit(&c.bars->k_empty[st]);
    if (q_empty != nullptr) tc_commit(q_empty);
  }
  __syncwarp();
  ++ns;
  return true;
}

// O_G (+)= P_G V for the key tile in ring stage `st`. The first product of an item overwrites O, which the group
// must have read out for the previous item (o_free).
template <int D, int G>
__device__ __forceinline__ bool mma_issue_pv(const MmaCtx<D>& c, uint32_t st, uint32_t ph, uint32_t& npv,
                                             bool accumulate, bool wait_o_free, uint32_t n_items_done) {
  using C = Fwd2Cfg<D>;
  if (!mbar_wait(&c.bars->v_full[st], ph, c.abort_flag) || !mbar_wait(&c.bars->p_ready[G], npv & 1, c.abort_flag) ||
      (wait_o_free && !mbar_wait(&c.bars->o_free[G], (n_items_done - 1) & 1, c.abort_flag))) {
    if (c.lane == 0) report_status(c.status, kWaitAttnTimeout, 114, G, static_cast<int>(npv));
    return false;
  }
  tc_fence_after();
  if (c.lane == 0) {
    constexpr uint32_t idesc_o = make_idesc(128, D, 0, 1, 1);
    const uint64_t dV = c.dV0 + static_cast<uint64_t>(st) * (C::kTile >> 4);
    const uint64_t dP = c.dP[G];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk)
      umma_bf16(c.tmem + C::kColO + G * D, dP + ((kk >> 2) * 1024 + (kk & 3) * 2), dV + kk * 128, idesc_o,
                accumulate || kk > 0);
    tc_commit(&c.bars->o_full[G]);
    tc_commit(&c.bars->v_empty[st]);
  }
  __syncwarp();
  ++npv;
  return true;
}

// A key tile this group does not use (past its causal range) still needs its share of the stage's two releases.
// The arrival waits for the tile to have landed, so it can never run a ring cycle ahead of the loads.
template <int D>
__device__ __forceinline__ bool mma_skip_stage(const MmaCtx<D>& c, uint64_t* full, uint64_t* empty, uint32_t ph) {
  if (!mbar_wait(full, ph, c.abort_flag)) return false;
  if (c.lane == 0) mbar_arrive(empty);
  __syncwarp();
  return true;
}

// The MMA warp of query tile G: every item, every key tile, one tile ahead with the scores.
template <int D, int G>
__device__ __forceinline__ void mma_loop(MmaCtx<D>& c, const Fwd2Args& a, uint32_t sb) {
  using C = Fwd2Cfg<D>;
  Fwd2Bars* bars = c.bars;
  uint32_t ns = 0, npv = 0, nit = 0;   // running counts of this group
  uint32_t st = 0, ph = 0;             // ring stage / phase of the current key tile
  int li = 0;
  bool ok = true;
  for (int idx = item_index(li, blockIdx.x, gridDim.x); idx < a.n_items && ok; idx = item_index(++li, blockIdx.x, gridDim.x)) {
    const Item it = decode_item(a, idx);
    const int n_g = it.nkv[G], n_max = it.n_max;
    const int slot = li & 1;
    if (!mbar_wait(&bars->q_full[slot], (li >> 1) & 1, c.abort_flag)) {
      if (c.lane == 0) report_status(c.status, kWaitFullTimeout, 112, idx, G);
      break;
    }
    const uint64_t dQ = make_smem_desc(sb + C::kOffQ + (slot * 2 + G) * C::kTile, 16, 1024);
    uint64_t* q_empty = &bars->q_empty[slot];
    if (n_g > 0) {
      ok = mma_issue_s<D, G>(c, dQ, st, ph, ns, n_g == 1 ? q_empty : nullptr);
    } else {
      if (c.lane == 0) mbar_arrive(q_empty);
      __syncwarp();
      ok = mma_skip_stage<D>(c, &bars->k_full[st], &bars->k_empty[st], ph);
    }
    for (int j = 0; j < n_max && ok; ++j) {
      uint32_t st1 = st + 1, ph1 = ph;
      if (st1 == kRing) {
        st1 = 0;
        ph1 ^= 1;
      }
      if (j + 1 < n_g) ok = mma_issue_s<D, G>(c, dQ, st1, ph1, ns, j + 2 == n_g ? q_empty : nullptr);
      else if (j + 1 < n_max) ok = mma_skip_stage<D>(c, &bars->k_full[st1], &bars->k_empty[st1], ph1);
      if (ok) {
        if (j < n_g) ok = mma_issue_pv<D, G>(c, st, ph, npv, j > 0, j == 0 && nit > 0, nit);
        else ok = mma_skip_stage<D>(c, &bars->v_full[st], &bars->v_empty[st], ph);
      }
      st = st1;
      ph = ph1;
    }
    if (n_g > 0) ++nit;
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

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->q_full[s], 1);
      mbar_init(&bars->q_empty[s], 2);     // released by both MMA warps
    }
    for (int s = 0; s < kRing; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 2);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 2);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(&bars->s_full[g], 1);
      mbar_init(&bars->s_free[g], 4);
      mbar_init(&bars->p_ready[g], 4);
      mbar_init(&bars->o_full[g], 1);
      mbar_init(&bars->o_free[g], 4);
      mbar_init(&bars->turn[g], 4);
    }
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kWarpMma) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp >= 8) {
  // One instruction for the whole third warpgroup (setmaxnreg is warpgroup-aligned): it gives registers up ...
  asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
  if (warp == kWarpTma) {
    if (lane == 0) {
      tma_prefetch_desc(&tq);
      tma_prefetch_desc(&tk);
      tma_prefetch_desc(&tv);
      uint32_t tile = 0;   // key tiles loaded so far (ring position)
      int li = 0;
      bool ok = true;
      for (int idx = item_index(li, blockIdx.x, gridDim.x); idx < a.n_items && ok; idx = item_index(++li, blockIdx.x, gridDim.x)) {
        const Item it = decode_item(a, idx);
        const int slot = li & 1;
        if (!mbar_wait(&bars->q_empty[slot], ((li >> 1) & 1) ^ 1, abort_flag)) {
          report_status(a.status, kWaitEmptyTimeout, 109, idx, 0);
          break;
        }
        const int q_row0 = it.b * a.Tq + it.pair * 256;
        uint8_t* sQ = smem + C::kOffQ + slot * 2 * C::kTile;
        mbar_arrive_expect_tx(&bars->q_full[slot], 2 * C::kTile);
        tma_load_2d(sQ, &tq, &bars->q_full[slot], it.h * D, q_row0);
        tma_load_2d(sQ + C::kTile, &tq, &bars->q_full[slot], it.h * D, q_row0 + 128);
        const int kv_row0 = it.b * a.kv_rows_b + it.hkv * a.kv_rows_h;
        const int k_col0 = it.hkv * a.k_col_h, v_col0 = it.hkv * a.v_col_h;
        for (int j = 0; j < it.n_max; ++j, ++tile) {
          const int s = tile % kRing;
          const uint32_t ph = (tile / kRing) & 1;
          if (!mbar_wait(&bars->k_empty[s], ph ^ 1, abort_flag)) {
            report_status(a.status, kWaitEmptyTimeout, 110, idx, j);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&bars->k_full[s], C::kTile);
          tma_load_2d(smem + C::kOffK + s * C::kTile, &tk, &bars->k_full[s], k_col0, kv_row0 + j * 128);
          if (!mbar_wait(&bars->v_empty[s], ph ^ 1, abort_flag)) {
            report_status(a.status, kWaitEmptyTimeout, 111, idx, j);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&bars->v_full[s], C::kTile);
          tma_load_2d(smem + C::kOffV + s * C::kTile, &tv, &bars->v_full[s], v_col0, kv_row0 + j * 128);
        }
      }
    }
  } else if (warp == kWarpMma || warp == kWarpMma + 1) {
    // Issue streams are kept short: descriptors are built once and advanced by constants, ring stages and barrier
    // phases are running scalars (no division, no runtime-indexed arrays), the two groups are template instances.
    MmaCtx<D> c;
    c.bars = bars;
    c.abort_flag = abort_flag;
    c.status = a.status;
    c.tmem = tmem;
    c.lane = lane;
    const uint32_t sb = smem_u32(smem);
    c.dK0 = make_smem_desc(sb + C::kOffK, 16, 1024);
    c.dV0 = make_smem_desc(sb + C::kOffV, 16384, 1024);
    c.dP[0] = make_smem_desc(sb + C::kOffP, 16, 1024);
    c.dP[1] = make_smem_desc(sb + C::kOffP + C::kPBytes, 16, 1024);
    if (warp == kWarpMma) mma_loop<D, 0>(c, a, sb);
    else mma_loop<D, 1>(c, a, sb);
  }
  } else {
    // ... and the two softmax warpgroups take them.
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    const int g = warp >> 2;             // query tile of this softmax group
    const int q4 = warp & 3;             // TMEM lane quarter this warp may touch
    const int r = q4 * 32 + lane;        // row inside the tile == TMEM lane
    const uint32_t lane_off = static_cast<uint32_t>(q4 * 32) << 16;
    const uint32_t tS = tmem + C::kColS + g * 128 + lane_off;
    const uint32_t tO = tmem + C::kColO + g * D + lane_off;
    uint8_t* sP = smem + C::kOffP + g * C::kPBytes;
    uint32_t n = 0;                      // key tiles this group has processed (running over all items)
    uint32_t turn = 0;                   // exponential-phase turns taken or passed on (same count in both groups)
    bool ok = true;
    // Group 0 goes first: its wait looks at the phase BEFORE the current one, group 1 waits for group 0's arrival.
    auto take_turn = [&]() -> bool {
      return mbar_wait(&bars->turn[g], (turn & 1) ^ (g == 0 ? 1u : 0u), abort_flag);
    };
    auto pass_turn = [&]() {
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->turn[g ^ 1]);
      ++turn;
    };
    int li = 0;
    for (int idx = item_index(li, blockIdx.x, gridDim.x); idx < a.n_items && ok;
         idx = item_index(++li, blockIdx.x, gridDim.x)) {
      const Item it = decode_item(a, idx);
      const int n_mine = it.nkv[g];
      const int q_tile0 = (2 * it.pair + g) * 128;
      const int qi = q_tile0 + r;          // query index inside the sequence
      const int qpos = a.q_pos0 + qi;
      float m = -INFINITY, l = 0.f;        // m: the reference the probabilities are formed against
      for (int j = 0; j < it.n_max; ++j) {
        if (j >= n_mine) {
          // a key tile only the other group sees: hand the turn straight on
          if (!take_turn()) {
            ok = false;
            break;
          }
          pass_turn();
          continue;
        }
        if (!mbar_wait(&bars->s_full[g], n & 1, abort_flag)) {
          if (lane == 0) report_status(a.status, kWaitAttnTimeout, 115, idx, j);
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t s[128];
        tmem_ld_32x32(tS, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
        tmem_ld_32x32(tS + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
        tmem_ld_32x32(tS + 64, *reinterpret_cast<uint32_t(*)[32]>(&s[64]));
        tmem_ld_32x32(tS + 96, *reinterpret_cast<uint32_t(*)[32]>(&s[96]));
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->s_free[g]);   // one arrival per warp: 128 arrivals would serialise
        const int kv0 = j * 128;
        const bool need_mask = (a.causal && kv0 + 127 > a.q_pos0 + q_tile0) || (kv0 + 128 > a.Tk);
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 128; ++i) {
            const int kp = kv0 + i;
            if (kp >= a.Tk || (a.causal && kp > qpos)) s[i] = 0xff800000u;  // -inf
          }
        }
        float mx8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) mx8[i] = __uint_as_float(s[i]);
#pragma unroll
        for (int i = 8; i < 128; ++i) mx8[i & 7] = fmaxf(mx8[i & 7], __uint_as_float(s[i]));
        const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])),
                               fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7]))) * a.scale_log2;   // scale > 0
        if (j == 0) {
          m = mx;
        } else {
          const bool grow = mx > m + kRescaleGap;          // also true when m is still -inf and mx is finite
          if (__any_sync(0xffffffffu, grow)) {
            // the warp rescales its 32 rows of O (rows that did not grow keep factor 1)
            const float alpha = grow ? exp2f(m - mx) : 1.f;
            if (!mbar_wait(&bars->o_full[g], (n - 1) & 1, abort_flag)) {
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
              for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
              tmem_st_32x32(tO + c * 32, v);
            }
            tmem_st_wait();
            l *= alpha;
            if (grow) m = mx;
          }
        }
        const float mref = (m == -INFINITY) ? 0.f : m;
        const float nmref = -mref;
        float rs[4] = {0.f, 0.f, 0.f, 0.f};
        if (j > 0 && !mbar_wait(&bars->o_full[g], (n - 1) & 1, abort_flag)) {   // P V of tile j-1 has read sP
          ok = false;
          break;
        }
        if (!take_turn()) {
          ok = false;
          break;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float p0 = exp2f(fmaf(__uint_as_float(s[c * 32 + i]), a.scale_log2, nmref));
            const float p1 = exp2f(fmaf(__uint_as_float(s[c * 32 + i + 1]), a.scale_log2, nmref));
            const float p2 = exp2f(fmaf(__uint_as_float(s[c * 32 + i + 2]), a.scale_log2, nmref));
            const float p3 = exp2f(fmaf(__uint_as_float(s[c * 32 + i + 3]), a.scale_log2, nmref));
            rs[0] += p0;
            rs[1] += p1;
            rs[2] += p2;
            rs[3] += p3;
            pk[i >> 1] = pack_bf16x2(p0, p1);
            pk[(i >> 1) + 1] = pack_bf16x2(p2, p3);
          }
          store_p_chunk(sP, r, c * 32, pk);
        }
        pass_turn();
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_ready[g]);
        l += (rs[0] + rs[1]) + (rs[2] + rs[3]);
        ++n;
      }
      if (!ok) break;
      if (n_mine == 0) continue;
      if (!ok) break;
      // final O of the item: wait for the last P V, pull it out and release the columns for the next item
      if (!mbar_wait(&bars->o_full[g], (n - 1) & 1, abort_flag)) {
        if (lane == 0) report_status(a.status, kWaitAttnTimeout, 116, idx, 0);
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t o[D];
#pragma unroll
      for (int c = 0; c < D / 32; ++c) tmem_ld_32x32(tO + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&o[c * 32]));
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->o_free[g]);
      if (qi < a.Tq) {
        const float inv = (l > 0.f) ? 1.f / l : 0.f;
        __nv_bfloat16* orow = a.out + static_cast<int64_t>(it.b * a.Tq + qi) * a.ldo + it.h * D;
#pragma unroll
        for (int i = 0; i < D; i += 8) {
          uint4 pk = make_uint4(
              pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv),
              pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv),
              pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv),
              pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv));
          *reinterpret_cast<uint4*>(orow + i) = pk;
        }
        if (a.lse != nullptr)
          a.lse[(static_cast<int64_t>(it.b) * a.H + it.h) * a.Tq + qi] = ((m == -INFINITY) ? 0.f : m) + log2f(l);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kWarpMma) {
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
  static int n_sms = 0;
  if (!configured) {
    if ((e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem)) != cudaSuccess)
      return e;
    int dev = 0;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
    if ((e = cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
    configured = true;
  }
  const int n_pairs = ((s.T + 127) / 128 + 1) / 2;
  const int n_items = n_pairs * s.H * s.B;
  Fwd2Args a{s.B, s.T, kv.Tk, s.H, s.Hkv, kv.q_pos0, kv.rows_b, kv.rows_h, kv.k_col_h, kv.v_col_h, n_pairs, n_items,
             s.scale * kLog2e2, s.causal, out, ldo, lse, status};
  const int grid = n_items < n_sms ? n_items : n_sms;
  kernel<<<grid, kThreads2, C::kSmem, stream>>>(tq, tk, tv, a);
  return cudaGetLastError();
}

}  // namespace b200
