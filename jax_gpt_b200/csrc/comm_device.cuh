// Device-side primitives for cross-rank signalling over peer-mapped memory: system-scope
// release / acquire flag accesses, NVLS multimem accesses, bounded flag waits and an
// all-to-all flag barrier. Shared by the kernels that communicate from inside the kernel.
#pragma once
#include "comm_kernels.cuh"
#include "common.cuh"

namespace b200 {

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys_f32(float* p, float v) {
  asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(mc)
               : "memory");
  return r;
}
__device__ __forceinline__ void multimem_st_b128(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// Bounded wait until *flag >= expected (system scope). Returns false on expiry.
__device__ __forceinline__ bool wait_flag_ge(const int* flag, int expected, uint64_t budget_ns) {
  if (ld_acquire_sys(flag) >= expected) return true;
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    if (ld_acquire_sys(flag) >= expected) return true;
    if (globaltimer_ns() - t0 > budget_ns) return false;
    __nanosleep(64);
  }
}

// All-to-all flag barrier run by the first `world` threads of ONE block. Thread p tells rank p
// "I reached `epoch` on `slot`" and waits for rank p to say the same. Returns false on expiry.
static __device__ __noinline__ bool flag_barrier(CommCtrl* const* peer_ctrl, int world, int rank, int slot, int epoch,
                             uint64_t budget_ns, int* status) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const int p = threadIdx.x;
    __threadfence_system();
    st_release_sys(&peer_ctrl[p]->flags[slot][rank], epoch);
    if (!wait_flag_ge(&peer_ctrl[rank]->flags[slot][p], epoch, budget_ns)) {
      report_status(status, kWaitFlagTimeout, slot, p, epoch);
      ok_s = 0;
    }
  }
  __syncthreads();
  return ok_s != 0;
}

}  // namespace b200
