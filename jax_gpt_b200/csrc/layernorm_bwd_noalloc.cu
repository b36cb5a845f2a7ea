// Allocation-free LayerNorm backward: see layernorm_bwd_noalloc.h for the contract.
//
// Same two-kernel scheme as the regular norm backward (per-block partial sums of the scale and
// bias gradients, then a column reduction), specialised to LayerNorm with rows of at most 1024
// elements handled one warp per row, and with the partial sums in a library-resident array
// instead of caller-provided scratch.
#include "layernorm_bwd_noalloc.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

namespace {

constexpr int kMaxD = B200_LN_BWD_NOALLOC_MAX_D;
constexpr int kMaxBlocks = B200_LN_BWD_NOALLOC_MAX_BLOCKS;
constexpr int kRows = B200_LN_BWD_NOALLOC_ROWS_PER_BLOCK;  // warps (= rows in flight) per block
constexpr size_t kScratchFloats = static_cast<size_t>(kMaxBlocks) * kRows * 2 * kMaxD;

// Partial sums: [block * kRows + warp][0: dgamma, 1: dbeta][D]. Lives in every GPU's copy of the
// library image. On the host this name is only a handle for cudaGetSymbolAddress; the address
// the kernels use is looked up per device in scratch_for_current_device().
static __device__ __align__(256) float g_ln_bwd_scratch[kScratchFloats];

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
    const float2 t = __bfloat1622float2(h);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// One warp per row, NV vectors of 8 elements per lane (D <= NV * 256).
template <int NV>
__global__ void ln_bwd_partial_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                      const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean,
                                      const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ dres,
                                      __nv_bfloat16* __restrict__ dx, float* __restrict__ partials, int M, int D) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float dg_acc[NV][8], db_acc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dg_acc[i][j] = db_acc[i][j] = 0.f;
  const int groups = (M + kRows - 1) / kRows;
  for (int grp = blockIdx.x; grp < groups; grp += gridDim.x) {
    const int row = grp * kRows + warp;
    if (row >= M) continue;  // warp-uniform; no block-wide barrier in this loop
    const float mu = mean[row], rs = rstd[row];
    float xh[NV][8], dg[NV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int col = (i * 32 + lane) * 8;
      if (col < D) {
        float xv[8], dv[8], g[8];
        load8(x + static_cast<int64_t>(row) * D + col, xv);
        load8(dy + static_cast<int64_t>(row) * D + col, dv);
        load8(gamma + col, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xv[j] - mu) * rs;
          dg[i][j] = dv[j] * g[j];
          s1 += dg[i][j];
          s2 += dg[i][j] * xh[i][j];
          dg_acc[i][j] += dv[j] * xh[i][j];
          db_acc[i][j] += dv[j];
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) xh[i][j] = dg[i][j] = 0.f;
      }
    }
    s1 = warp_sum(s1) / D;
    s2 = warp_sum(s2) / D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int col = (i * 32 + lane) * 8;
      if (col < D) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (dg[i][j] - s1 - xh[i][j] * s2);
        if (dres != nullptr) {
          float r[8];
          load8(dres + static_cast<int64_t>(row) * D + col, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        store8(dx + static_cast<int64_t>(row) * D + col, o);
      }
    }
  }
  // Every (block, warp) slot that the reduction will read is written here, zeros included.
  float* part = partials + static_cast<int64_t>(blockIdx.x * kRows + warp) * 2 * D;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (i * 32 + lane) * 8;
    if (col < D) {
      *reinterpret_cast<float4*>(part + col) = make_float4(dg_acc[i][0], dg_acc[i][1], dg_acc[i][2], dg_acc[i][3]);
      *reinterpret_cast<float4*>(part + col + 4) = make_float4(dg_acc[i][4], dg_acc[i][5], dg_acc[i][6], dg_acc[i][7]);
      *reinterpret_cast<float4*>(part + D + col) = make_float4(db_acc[i][0], db_acc[i][1], db_acc[i][2], db_acc[i][3]);
      *reinterpret_cast<float4*>(part + D + col + 4) =
          make_float4(db_acc[i][4], db_acc[i][5], db_acc[i][6], db_acc[i][7]);
    }
  }
}

// Column sums of the partial rows, added to dgamma | dbeta. Block (32, 32).
__global__ void ln_bwd_reduce_kernel(const float* __restrict__ partials, int n_rows, int D, float* __restrict__ dgamma,
                                     float* __restrict__ dbeta) {
  __shared__ float red[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;  // column of the concatenated [dgamma | dbeta] row
  float s = 0.f;
  if (c < 2 * D)
    for (int r = threadIdx.y; r < n_rows; r += 32) s += partials[static_cast<int64_t>(r) * 2 * D + c];
  red[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < 2 * D) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) t += red[k][threadIdx.x];
    if (c < D) dgamma[c] += t;
    else dbeta[c - D] += t;
  }
}

// Device address of g_ln_bwd_scratch on the current device, resolved once per device.
cudaError_t scratch_for_current_device(float** out) {
  constexpr int kMaxDevices = 64;
  static float* table[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (table[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_ln_bwd_scratch);
    if (e != cudaSuccess) return e;
    table[dev] = p;
  }
  *out = table[dev];
  return cudaSuccess;
}

bool misaligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }

}  // namespace

extern "C" int b200_layernorm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* mean,
                                          const float* rstd, const void* dres, void* dx, float* dgamma, float* dbeta,
                                          int M, int D, void* cuda_stream) {
  if (D > kMaxD) return B200_NOALLOC_ERR_TOO_LARGE;
  if (M < 1 || D < 8 || (D % 8) != 0) return B200_NOALLOC_ERR_BAD_SHAPE;
  if (!dy || !x || !gamma || !mean || !rstd || !dx || !dgamma || !dbeta) return B200_NOALLOC_ERR_NULL_PTR;
  if (misaligned(dy) || misaligned(x) || misaligned(gamma) || misaligned(dx) || (dres && misaligned(dres)) ||
      misaligned(dgamma) || misaligned(dbeta))
    return B200_NOALLOC_ERR_ALIGNMENT;
  float* scratch = nullptr;
  cudaError_t e = scratch_for_current_device(&scratch);
  if (e != cudaSuccess) return static_cast<int>(e);
  cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
  const int groups = (M + kRows - 1) / kRows;
  const int grid = groups < kMaxBlocks ? groups : kMaxBlocks;
  auto* dy_ = static_cast<const __nv_bfloat16*>(dy);
  auto* x_ = static_cast<const __nv_bfloat16*>(x);
  auto* g_ = static_cast<const __nv_bfloat16*>(gamma);
  auto* dr_ = static_cast<const __nv_bfloat16*>(dres);
  auto* dx_ = static_cast<__nv_bfloat16*>(dx);
  if (D <= 256) ln_bwd_partial_kernel<1><<<grid, kRows * 32, 0, st>>>(dy_, x_, g_, mean, rstd, dr_, dx_, scratch, M, D);
  else if (D <= 512) ln_bwd_partial_kernel<2><<<grid, kRows * 32, 0, st>>>(dy_, x_, g_, mean, rstd, dr_, dx_, scratch, M, D);
  else if (D <= 768) ln_bwd_partial_kernel<3><<<grid, kRows * 32, 0, st>>>(dy_, x_, g_, mean, rstd, dr_, dx_, scratch, M, D);
  else ln_bwd_partial_kernel<4><<<grid, kRows * 32, 0, st>>>(dy_, x_, g_, mean, rstd, dr_, dx_, scratch, M, D);
  e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  ln_bwd_reduce_kernel<<<(2 * D + 31) / 32, dim3(32, 32), 0, st>>>(scratch, grid * kRows, D, dgamma, dbeta);
  return static_cast<int>(cudaGetLastError());
}

extern "C" const char* b200_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "success";
    case B200_NOALLOC_ERR_TOO_LARGE:
      return "row width D exceeds B200_LN_BWD_NOALLOC_MAX_D (1024): the built-in scratch cannot hold the partial sums";
    case B200_NOALLOC_ERR_BAD_SHAPE: return "M must be >= 1 and D a multiple of 8 that is >= 8";
    case B200_NOALLOC_ERR_NULL_PTR: return "a required pointer is NULL";
    case B200_NOALLOC_ERR_ALIGNMENT: return "a pointer is not 16-byte aligned";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown error code";
  }
}
