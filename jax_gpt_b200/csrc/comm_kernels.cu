// Communication fused into compute over NVLink peer memory.
//
// sharded_adamw_kernel is the FSDP / ZeRO optimizer step as ONE cooperative kernel per rank:
//
//   flag barrier (all ranks' gradients are final)
//   A: reduce-scatter  - this rank sums its 1/W slice of every rank's fp32 gradient buffer with
//      plain peer loads (or one multimem.ld_reduce through the NVSwitch when a multicast
//      alias is given), keeps the reduced slice locally and accumulates sum(g^2)
//   exchange of the W partial sums of squares through the control blocks (same summation
//      order on every rank, so every rank applies the same clip coefficient)
//   B: clip -> Adam -> decoupled weight decay -> lr on the local fp32 master shard, then
//      all-gather - the updated bf16 values are pushed straight into every rank's compute
//      buffer (peer stores, or one multimem.st)
//   flag barrier (every rank's pushes have landed; nobody reads gradients any more)
//
// Every cross-rank wait is bounded; on expiry the kernel records kWaitFlagTimeout, skips
// the remaining work, still passes every grid-wide sync and returns normally.
//
// The optimizer math is the chain of jax_gpt/trainer/optimizer.py:48-63; the reference
// leaves gradient reduction to XLA (jax_gpt/trainer/train_step.py:63-67) and has no FSDP
// (jax_gpt/trainer/sharding.py:58-69 declares the axis only).
#include "comm_kernels.cuh"

#include <cooperative_groups.h>

#include "comm_device.cuh"
#include "common.cuh"

namespace cg = cooperative_groups;

namespace b200 {

namespace {

__device__ __forceinline__ float block_sum(float v) {
  __shared__ float red[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  }
  return s;  // valid in thread 0
}

__global__ void __launch_bounds__(512, 2) sharded_adamw_kernel(const __grid_constant__ ShardedAdamWArgs a) {
  cg::grid_group grid = cg::this_grid();
  CommCtrl* my = a.peer_ctrl[a.rank];
  const int epoch = my->epoch + 1;
  const int W = a.world;
  const int64_t S = a.n_total / W;  // shard length
  const int64_t base = S * a.rank;
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;

  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) {
      my->sq_local = a.extra_sq != nullptr ? __ldcg(a.extra_sq) : 0.f;
      my->abort_flag = 0;
    }
    if (!flag_barrier(a.peer_ctrl, W, a.rank, 0, epoch, a.wait_budget_ns, a.status) && threadIdx.x == 0)
      my->abort_flag = 1;
  }
  __threadfence();
  grid.sync();
  bool alive = (*reinterpret_cast<volatile int*>(&my->abort_flag) == 0);

  // ---- A: reduce-scatter of this rank's slice + partial sum of squares ----
  float sq = 0.f;
  if (alive) {
    float* mine = a.peer_grad[a.rank] + base;
    for (int64_t i = tid * 4; i < S; i += nthreads * 4) {
      float4 acc;
      if (a.pre_reduced) {
        acc = *reinterpret_cast<const float4*>(mine + i);
      } else if (a.mc_grad != nullptr) {
        acc = multimem_ld_reduce_f32x4(a.mc_grad + base + i);
      } else {
        acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int p = 0; p < kCommMaxRanks; ++p) {
          if (p < W) {
            const int src = (a.rank + p) % W;  // start local, spread the peers across ranks
            const float4 g = __ldcg(reinterpret_cast<const float4*>(a.peer_grad[src] + base + i));
            acc.x += g.x; acc.y += g.y; acc.z += g.z; acc.w += g.w;
          }
        }
      }
      if (!a.pre_reduced) *reinterpret_cast<float4*>(mine + i) = acc;
      sq += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    }
  }
  sq = block_sum(sq);
  if (threadIdx.x == 0 && alive) atomicAdd(&my->sq_local, sq);
  __threadfence();
  grid.sync();

  // ---- exchange of the partial norms ----
  if (blockIdx.x == 0) {
    if (alive && threadIdx.x < W)
      st_relaxed_sys_f32(&a.peer_ctrl[threadIdx.x]->norm_slots[a.rank], *reinterpret_cast<volatile float*>(&my->sq_local));
    const bool ok = flag_barrier(a.peer_ctrl, W, a.rank, 1, epoch, a.wait_budget_ns, a.status);
    if (threadIdx.x == 0) {
      if (!ok) my->abort_flag = 1;
      float tot = 0.f;
      for (int p = 0; p < W; ++p) tot += *reinterpret_cast<volatile float*>(&my->norm_slots[p]);
      my->sq_total = tot;
    }
  }
  __threadfence();
  grid.sync();
  alive = (*reinterpret_cast<volatile int*>(&my->abort_flag) == 0);

  // ---- B: AdamW on the shard, push bf16 parameters to every rank ----
  if (alive) {
    const float lr = a.hp[0], bc1 = a.hp[1], bc2 = a.hp[2], gscale = a.hp[3];
    float coef = gscale;
    if (a.clip > 0.f) {
      const float norm = sqrtf(*reinterpret_cast<volatile float*>(&my->sq_total)) * gscale;
      coef *= fminf(1.f, a.clip / (norm + 1e-6f));
    }
    const float* gsh = a.peer_grad[a.rank] + base;
    for (int64_t i = tid * 8; i < S; i += nthreads * 8) {
      float g[8], p[8], m[8], v[8];
      *reinterpret_cast<float4*>(g) = *reinterpret_cast<const float4*>(gsh + i);
      *reinterpret_cast<float4*>(g + 4) = *reinterpret_cast<const float4*>(gsh + i + 4);
      *reinterpret_cast<float4*>(p) = *reinterpret_cast<const float4*>(a.master + i);
      *reinterpret_cast<float4*>(p + 4) = *reinterpret_cast<const float4*>(a.master + i + 4);
      *reinterpret_cast<float4*>(m) = *reinterpret_cast<const float4*>(a.m + i);
      *reinterpret_cast<float4*>(m + 4) = *reinterpret_cast<const float4*>(a.m + i + 4);
      *reinterpret_cast<float4*>(v) = *reinterpret_cast<const float4*>(a.v + i);
      *reinterpret_cast<float4*>(v + 4) = *reinterpret_cast<const float4*>(a.v + i + 4);
      const float wd = (base + i < a.n_decay) ? a.wd : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gi = g[j] * coef;
        m[j] = a.beta1 * m[j] + (1.f - a.beta1) * gi;
        v[j] = a.beta2 * v[j] + (1.f - a.beta2) * gi * gi;
        const float u = (m[j] / bc1) / (sqrtf(v[j] / bc2) + a.eps) + wd * p[j];
        p[j] -= lr * u;
      }
      *reinterpret_cast<float4*>(a.master + i) = *reinterpret_cast<float4*>(p);
      *reinterpret_cast<float4*>(a.master + i + 4) = *reinterpret_cast<float4*>(p + 4);
      *reinterpret_cast<float4*>(a.m + i) = *reinterpret_cast<float4*>(m);
      *reinterpret_cast<float4*>(a.m + i + 4) = *reinterpret_cast<float4*>(m + 4);
      *reinterpret_cast<float4*>(a.v + i) = *reinterpret_cast<float4*>(v);
      *reinterpret_cast<float4*>(a.v + i + 4) = *reinterpret_cast<float4*>(v + 4);
      const uint4 pk = make_uint4(pack_bf16x2(p[0], p[1]), pack_bf16x2(p[2], p[3]), pack_bf16x2(p[4], p[5]),
                                  pack_bf16x2(p[6], p[7]));
      if (a.mc_param != nullptr) {
        multimem_st_b128(a.mc_param + base + i, pk);
      } else {
#pragma unroll
        for (int q = 0; q < kCommMaxRanks; ++q) {
          if (q < W) {
            const int dst = (a.rank + q) % W;
            *reinterpret_cast<uint4*>(a.peer_param[dst] + base + i) = pk;
          }
        }
      }
    }
  }
  __threadfence_system();
  grid.sync();
  if (blockIdx.x == 0) {
    flag_barrier(a.peer_ctrl, W, a.rank, 2, epoch, a.wait_budget_ns, a.status);
    if (threadIdx.x == 0) my->epoch = epoch;
  }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(256, 1) vocab_parallel_ce_kernel(const __grid_constant__ VocabCeArgs a) {
  cg::grid_group grid = cg::this_grid();
  CommCtrl* my = a.peer_ctrl[a.rank];
  const int epoch = my->epoch + 1;
  const int W = a.world;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gwarp = blockIdx.x * (blockDim.x >> 5) + warp, gwarps = gridDim.x * (blockDim.x >> 5);
  const int64_t buf = static_cast<int64_t>(epoch & 1) * W * a.M * 4;
  const int nvec = a.v_local / 8;  // 16-byte vectors; the tail is read element-wise

  // ---- phase 1: statistics of this shard, pushed to every rank ----
  for (int row = gwarp; row < a.M; row += gwarps) {
    const __nv_bfloat16* lp = a.logits + static_cast<int64_t>(row) * a.ldl;
    const uint4* lv = reinterpret_cast<const uint4*>(lp);
    float mx = -INFINITY;
    for (int i = lane; i < nvec; i += 32) {
      const uint4 u = lv[i];
      const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
      mx = fmaxf(mx, fmaxf(fmaxf(fmaxf(f0.x, f0.y), fmaxf(f1.x, f1.y)), fmaxf(fmaxf(f2.x, f2.y), fmaxf(f3.x, f3.y))));
    }
    for (int i = nvec * 8 + lane; i < a.v_local; i += 32) mx = fmaxf(mx, __bfloat162float(lp[i]));
    mx = warp_max(mx);
    float se = 0.f;
    for (int i = lane; i < nvec; i += 32) {
      const uint4 u = lv[i];
      const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z), f3 = unpack_bf16x2(u.w);
      se += __expf(f0.x - mx) + __expf(f0.y - mx) + __expf(f1.x - mx) + __expf(f1.y - mx) + __expf(f2.x - mx) +
            __expf(f2.y - mx) + __expf(f3.x - mx) + __expf(f3.y - mx);
    }
    for (int i = nvec * 8 + lane; i < a.v_local; i += 32) se += __expf(__bfloat162float(lp[i]) - mx);
    se = warp_sum(se);
    const int tg = a.targets[row] - a.v0;
    const float tl = (tg >= 0 && tg < a.v_local) ? __bfloat162float(lp[tg]) : 0.f;
    if (lane < W) {
      float4* dst = reinterpret_cast<float4*>(a.peer_stats[lane] + buf + (static_cast<int64_t>(a.rank) * a.M + row) * 4);
      *dst = make_float4(mx, se, tl, 0.f);
    }
  }
  __threadfence_system();
  grid.sync();
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) my->abort_flag = 0;
    __syncthreads();
    const bool ok = flag_barrier(a.peer_ctrl, W, a.rank, 6, epoch, a.wait_budget_ns, a.status);
    if (!ok && threadIdx.x == 0) my->abort_flag = 1;
    if (threadIdx.x == 0) my->epoch = epoch;
  }
  __threadfence();
  grid.sync();
  if (*reinterpret_cast<volatile int*>(&my->abort_flag) != 0) return;

  // ---- phase 2: global loss; this shard's gradient in place ----
  const float* st = a.peer_stats[a.rank] + buf;
  for (int row = gwarp; row < a.M; row += gwarps) {
    float gm = -INFINITY;
    for (int r = 0; r < W; ++r) gm = fmaxf(gm, __ldcg(st + (static_cast<int64_t>(r) * a.M + row) * 4));
    float gs = 0.f, tl = 0.f;
    for (int r = 0; r < W; ++r) {
      const float4 s4 = __ldcg(reinterpret_cast<const float4*>(st + (static_cast<int64_t>(r) * a.M + row) * 4));
      gs += s4.y * __expf(s4.x - gm);
      tl += s4.z;
    }
    const int target = a.targets[row];
    const bool valid = target >= 0;
    if (lane == 0) a.loss[row] = valid ? (__logf(gs) + gm - tl) : 0.f;
    if (!a.write_grad) continue;
    const float inv = valid ? a.scale / gs : 0.f;
    const int tg = target - a.v0;
    __nv_bfloat16* lp = a.logits + static_cast<int64_t>(row) * a.ldl;
    uint4* lv = reinterpret_cast<uint4*>(lp);
    for (int i = lane; i < nvec; i += 32) {
      const uint4 u = lv[i];
      const uint32_t in[4] = {u.x, u.y, u.z, u.w};
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16x2(in[e]);
        const int c = i * 8 + 2 * e;
        float p0 = __expf(f.x - gm) * inv, p1 = __expf(f.y - gm) * inv;
        if (valid && c == tg) p0 -= a.scale;
        if (valid && c + 1 == tg) p1 -= a.scale;
        o[e] = pack_bf16x2(p0, p1);
      }
      lv[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    for (int i = nvec * 8 + lane; i < a.v_local; i += 32) {
      float p = __expf(__bfloat162float(lp[i]) - gm) * inv;
      if (valid && i == tg) p -= a.scale;
      lp[i] = __float2bfloat16(p);
    }
  }
}

__global__ void __launch_bounds__(256) rs_bucket_kernel(const __grid_constant__ RsBucketArgs a) {
  __shared__ int ok_s;
  const int epoch = *a.epoch;
  const int W = a.world;
  if (threadIdx.x == 0) ok_s = 1;
  if (blockIdx.x == 0 && threadIdx.x < W) {
    __threadfence_system();
    st_release_sys(a.peer_flags[threadIdx.x] + a.bucket * kCommMaxRanks + a.rank, epoch);
  }
  __syncthreads();
  if (threadIdx.x < W) {
    if (!wait_flag_ge(a.peer_flags[a.rank] + a.bucket * kCommMaxRanks + threadIdx.x, epoch, a.wait_budget_ns)) {
      report_status(a.status, kWaitFlagTimeout, 110, a.bucket, threadIdx.x);
      ok_s = 0;
    }
  }
  __syncthreads();
  if (!ok_s) return;
  const int64_t tid = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) * 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x * 4;
  float* mine = a.peer_grad[a.rank];
  for (int r = 0; r < a.n_ranges; ++r) {
    const int64_t start = a.ranges[2 * r], len = a.ranges[2 * r + 1];
    for (int64_t i = tid; i < len; i += stride) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int p = 0; p < kCommMaxRanks; ++p) {
        if (p < W) {
          const int src = (a.rank + p) % W;
          const float4 g = __ldcg(reinterpret_cast<const float4*>(a.peer_grad[src] + start + i));
          acc.x += g.x; acc.y += g.y; acc.z += g.z; acc.w += g.w;
        }
      }
      *reinterpret_cast<float4*>(mine + start + i) = acc;
    }
  }
}

__global__ void comm_barrier_kernel(CommCtrl* const* peer_ctrl_dev, int world, int rank, uint64_t budget_ns,
                                    int* status) {
  __shared__ CommCtrl* peers[kCommMaxRanks];
  if (threadIdx.x < world) peers[threadIdx.x] = peer_ctrl_dev[threadIdx.x];
  __syncthreads();
  CommCtrl* my = peers[rank];
  const int epoch = my->bar_epoch + 1;
  flag_barrier(peers, world, rank, 3, epoch, budget_ns, status);
  if (threadIdx.x == 0) my->bar_epoch = epoch;
}

__global__ void wait_flag_kernel(const int* flag, int expected, uint64_t budget_ns, int* status) {
  if (threadIdx.x == 0 && !wait_flag_ge(flag, expected, budget_ns))
    report_status(status, kWaitFlagTimeout, 99, expected, 0);
}

}  // namespace

cudaError_t launch_sharded_adamw(const ShardedAdamWArgs& args, cudaStream_t stream) {
  if (args.world < 1 || args.world > kCommMaxRanks || args.n_total % (static_cast<int64_t>(args.world) * 8) != 0)
    return cudaErrorInvalidValue;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int per_sm = 0;
  cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sharded_adamw_kernel, 512, 0);
  if (e != cudaSuccess) return e;
  if (per_sm < 1) return cudaErrorLaunchOutOfResources;
  const int grid = sms * (per_sm > 2 ? 2 : per_sm);
  ShardedAdamWArgs a = args;
  void* params[] = {&a};
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(sharded_adamw_kernel), dim3(grid), dim3(512), params, 0,
                                     stream);
}

cudaError_t launch_rs_bucket(const RsBucketArgs& args, int blocks, cudaStream_t stream) {
  if (args.world < 1 || args.world > kCommMaxRanks || args.n_ranges < 0 || blocks < 1) return cudaErrorInvalidValue;
  rs_bucket_kernel<<<blocks, 256, 0, stream>>>(args);
  return cudaGetLastError();
}

cudaError_t launch_vocab_parallel_ce(const VocabCeArgs& args, cudaStream_t stream) {
  if (args.world < 1 || args.world > kCommMaxRanks || args.M < 1 || args.v_local < 1 || args.ldl % 8 != 0)
    return cudaErrorInvalidValue;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int want = (args.M + 7) / 8;
  VocabCeArgs a = args;
  void* params[] = {&a};
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(vocab_parallel_ce_kernel), dim3(want < sms ? want : sms),
                                     dim3(256), params, 0, stream);
}

cudaError_t launch_comm_barrier(CommCtrl* const* peer_ctrl_dev, int world, int rank, uint64_t wait_budget_ns,
                                int* status, cudaStream_t stream) {
  comm_barrier_kernel<<<1, 32, 0, stream>>>(peer_ctrl_dev, world, rank, wait_budget_ns, status);
  return cudaGetLastError();
}

cudaError_t launch_wait_flag(const int* flag, int expected, uint64_t budget_ns, int* status, cudaStream_t stream) {
  wait_flag_kernel<<<1, 32, 0, stream>>>(flag, expected, budget_ns, status);
  return cudaGetLastError();
}

}  // namespace b200
