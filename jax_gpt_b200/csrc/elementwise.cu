// Bandwidth-bound kernels: LayerNorm / RMSNorm (forward + backward), token+position
// embedding, fused softmax cross-entropy (loss and dlogits in one pass), bias gradient,
// the AdamW chain with global-norm clipping, and small helpers. All take bf16 activations,
// keep statistics in fp32 and move 16 bytes per thread per access.
//
// Semantics follow the reference: LayerNorm eps 1e-5 with scale and bias
// (jax_gpt/models/gpt2/model.py:60-65), RMSNorm x/sqrt(mean x^2 + eps)*(1+w)
// (jax_gpt/models/qwen35/primitives.py:29-32), mean softmax-CE in fp32
// (jax_gpt/trainer/train_step.py:56-60), clip -> Adam -> decoupled decay -> lr
// (jax_gpt/trainer/optimizer.py:48-63).
#include "elementwise.cuh"

#include <algorithm>

#include "common.cuh"

namespace b200 {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the WPR warps that share one row (WPR == 1: warp shuffle only).
template <int WPR>
__device__ __forceinline__ float row_sum(float v, float* scratch, int row_in_block, int warp_in_row) {
  v = warp_sum(v);
  if (WPR == 1) return v;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[row_in_block * WPR + warp_in_row] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < WPR; ++w) s += scratch[row_in_block * WPR + w];
  return s;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                       pack_bf16x2(f[6], f[7]));
  *reinterpret_cast<uint4*>(p) = u;
}

// ------------------------------- norm forward ---------------------------------------
// MODE 0: LayerNorm (gamma, beta). MODE 1: RMSNorm with weight w. MODE 2: RMSNorm with (1+w).
// One row is handled by WPR warps; each lane keeps NV vectors of 8 elements in registers.
template <int NV, int WPR, int MODE>
__global__ void norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                                const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                                float* __restrict__ mean_out, float* __restrict__ rstd_out, int M, int D, float eps) {
  constexpr int ROWS = 4 / WPR > 0 ? 4 / WPR : 1;  // rows per block (128 or 32*WPR threads)
  __shared__ float scratch[ROWS * WPR + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_in_block = warp / WPR, warp_in_row = warp % WPR;
  const int row = blockIdx.x * ROWS + row_in_block;
  const bool active = row < M;
  const int rr = active ? row : 0;
  const __nv_bfloat16* xr = x + static_cast<int64_t>(rr) * D;
  float v[NV][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (i * WPR * 32 + warp_in_row * 32 + lane) * 8;
    if (col < D) {
      load8(xr + col, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[i][j];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
    }
  }
  float mean = 0.f;
  if (MODE == 0) mean = row_sum<WPR>(s, scratch, row_in_block, warp_in_row) / D;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (i * WPR * 32 + warp_in_row * 32 + lane) * 8;
    if (col < D) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float d = v[i][j] - mean;
        q += d * d;
      }
    }
  }
  const float var = row_sum<WPR>(q, scratch, row_in_block, warp_in_row) / D;
  const float rstd = rsqrtf(var + eps);
  if (active && lane == 0 && warp_in_row == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  if (!active) return;
  __nv_bfloat16* yr = y + static_cast<int64_t>(row) * D;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (i * WPR * 32 + warp_in_row * 32 + lane) * 8;
    if (col < D) {
      float g[8], b[8], o[8];
      load8(gamma + col, g);
      if (MODE == 0) load8(beta + col, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float n = (v[i][j] - mean) * rstd;
        if (MODE == 0) o[j] = n * g[j] + b[j];
        else if (MODE == 1) o[j] = n * g[j];
        else o[j] = n * (1.f + g[j]);
      }
      store8(yr + col, o);
    }
  }
}

// ------------------------------- norm backward --------------------------------------
// dx = rstd * (dyg - mean(dyg) - xhat * mean(dyg * xhat))   (LayerNorm)
// dx = rstd * (dyg - xhat * mean(dyg * xhat))               (RMSNorm)
// with dyg = dy * gamma (or dy * (1+w)). dgamma/dbeta are accumulated per thread over the
// rows a block visits and flushed once with fp32 atomics. `dres` (optional) is added to dx,
// which folds the residual-branch gradient into the same pass.
template <int NV, int WPR, int MODE>
__global__ void __launch_bounds__((4 / WPR > 0 ? 4 / WPR : 1) * WPR * 32, NV <= 3 ? 4 : 1)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                                const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                                __nv_bfloat16* __restrict__ dx, float* __restrict__ partials, int M, int D) {
  constexpr int ROWS = 4 / WPR > 0 ? 4 / WPR : 1;
  __shared__ float scratch[ROWS * WPR + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_in_block = warp / WPR, warp_in_row = warp % WPR;
  float dg_acc[NV][8], db_acc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dg_acc[i][j] = db_acc[i][j] = 0.f;

  const int row_groups = (M + ROWS - 1) / ROWS;
  for (int rg = blockIdx.x; rg < row_groups; rg += gridDim.x) {
    const int row = rg * ROWS + row_in_block;
    const bool active = row < M;
    const int rr = active ? row : 0;
    const float mean = (MODE == 0) ? mean_in[rr] : 0.f;
    const float rstd = rstd_in[rr];
    float xh[NV][8], dg[NV][8];
    uint4 res_raw[NV];  // the residual-branch gradient is fetched with the other operands, not after the row sums
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int col = (i * WPR * 32 + warp_in_row * 32 + lane) * 8;
      res_raw[i] = make_uint4(0u, 0u, 0u, 0u);
      if (col < D && active) {
        float xv[8], dv[8], g[8];
        if (dres != nullptr) res_raw[i] = *reinterpret_cast<const uint4*>(dres + static_cast<int64_t>(rr) * D + col);
        load8(x + static_cast<int64_t>(rr) * D + col, xv);
        load8(dy + static_cast<int64_t>(rr) * D + col, dv);
        load8(gamma + col, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xv[j] - mean) * rstd;
          const float gg = (MODE == 2) ? (1.f + g[j]) : g[j];
          dg[i][j] = dv[j] * gg;
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
    if (MODE == 0) s1 = row_sum<WPR>(s1, scratch, row_in_block, warp_in_row) / D; else s1 = 0.f;
    s2 = row_sum<WPR>(s2, scratch, row_in_block, warp_in_row) / D;
    if (active) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int col = (i * WPR * 32 + warp_in_row * 32 + lane) * 8;
        if (col < D) {
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = rstd * (dg[i][j] - s1 - xh[i][j] * s2);
          if (dres != nullptr) {
            const float2 a = unpack_bf16x2(res_raw[i].x), b = unpack_bf16x2(res_raw[i].y),
                         c = unpack_bf16x2(res_raw[i].z), d = unpack_bf16x2(res_raw[i].w);
            o[0] += a.x; o[1] += a.y; o[2] += b.x; o[3] += b.y; o[4] += c.x; o[5] += c.y; o[6] += d.x; o[7] += d.y;
          }
          store8(dx + static_cast<int64_t>(row) * D + col, o);
        }
      }
    }
  }
  // One partial row per (block, row slot): plain stores, reduced by norm_bwd_reduce_kernel.
  float* part = partials + static_cast<int64_t>(blockIdx.x * ROWS + row_in_block) * 2 * D;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int col = (i * WPR * 32 + warp_in_row * 32 + lane) * 8;
    if (col < D) {
      *reinterpret_cast<float4*>(part + col) = make_float4(dg_acc[i][0], dg_acc[i][1], dg_acc[i][2], dg_acc[i][3]);
      *reinterpret_cast<float4*>(part + col + 4) = make_float4(dg_acc[i][4], dg_acc[i][5], dg_acc[i][6], dg_acc[i][7]);
      if (MODE == 0) {
        *reinterpret_cast<float4*>(part + D + col) = make_float4(db_acc[i][0], db_acc[i][1], db_acc[i][2], db_acc[i][3]);
        *reinterpret_cast<float4*>(part + D + col + 4) =
            make_float4(db_acc[i][4], db_acc[i][5], db_acc[i][6], db_acc[i][7]);
      }
    }
  }
}

// dgamma[c] += sum_r partials[r][0][c]; dbeta[c] += sum_r partials[r][1][c]. Block (32, 32):
// threadIdx.x walks columns (coalesced), threadIdx.y strides over the partial rows of the block's
// slice (blockIdx.y of gridDim.y slices; the slices meet in one fp32 atomic per column).
constexpr int kNormReduceSlices = 8;
__global__ void norm_bwd_reduce_kernel(const float* __restrict__ partials, int n_rows, int D, int with_beta,
                                       float* __restrict__ dgamma, float* __restrict__ dbeta) {
  __shared__ float red[32][33];
  const int width = with_beta ? 2 * D : D;
  const int c = blockIdx.x * 32 + threadIdx.x;  // column in the concatenated [dgamma | dbeta] row
  const int per = (n_rows + gridDim.y - 1) / gridDim.y;
  const int r0 = blockIdx.y * per, r1 = min(n_rows, r0 + per);
  float s = 0.f;
  if (c < width) {
#pragma unroll 4
    for (int r = r0 + threadIdx.y; r < r1; r += 32) s += partials[static_cast<int64_t>(r) * 2 * D + c];
  }
  red[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < width) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) t += red[k][threadIdx.x];
    if (c < D) atomicAdd(dgamma + c, t);
    else if (dbeta != nullptr) atomicAdd(dbeta + (c - D), t);
  }
}

template <int MODE>
cudaError_t norm_fwd_dispatch(const __nv_bfloat16* x, const __nv_bfloat16* g, const __nv_bfloat16* b,
                              __nv_bfloat16* y, float* mean, float* rstd, int M, int D, float eps, cudaStream_t st) {
  if (D % 8 != 0 || D > 8192) return cudaErrorInvalidValue;
#define LAUNCH(NV, WPR)                                                                                   \
  {                                                                                                       \
    constexpr int ROWS = 4 / WPR > 0 ? 4 / WPR : 1;                                                       \
    norm_fwd_kernel<NV, WPR, MODE><<<(M + ROWS - 1) / ROWS, ROWS * WPR * 32, 0, st>>>(x, g, b, y, mean,   \
                                                                                     rstd, M, D, eps);   \
    return cudaGetLastError();                                                                            \
  }
  if (D <= 256) LAUNCH(1, 1)
  if (D <= 512) LAUNCH(2, 1)
  if (D <= 768) LAUNCH(3, 1)
  if (D <= 1024) LAUNCH(4, 1)
  if (D <= 2048) LAUNCH(2, 4)
  if (D <= 4096) LAUNCH(4, 4)
  LAUNCH(8, 4)
#undef LAUNCH
}

template <int MODE>
cudaError_t norm_bwd_dispatch(const __nv_bfloat16* dy, const __nv_bfloat16* x, const __nv_bfloat16* g,
                              const float* mean, const float* rstd, const __nv_bfloat16* dres, __nv_bfloat16* dx,
                              float* dgamma, float* dbeta, float* partials, int M, int D, cudaStream_t st) {
  if (D % 8 != 0 || D > 8192) return cudaErrorInvalidValue;
#define LAUNCH(NV, WPR)                                                                                    \
  {                                                                                                        \
    constexpr int ROWS = 4 / WPR > 0 ? 4 / WPR : 1;                                                        \
    int groups = (M + ROWS - 1) / ROWS;                                                                    \
    int grid = groups < kNormBwdMaxBlocks ? groups : kNormBwdMaxBlocks;                                    \
    norm_bwd_kernel<NV, WPR, MODE><<<grid, ROWS * WPR * 32, 0, st>>>(dy, x, g, mean, rstd, dres, dx,       \
                                                                    partials, M, D);                       \
    cudaError_t e_ = cudaGetLastError();                                                                   \
    if (e_ != cudaSuccess) return e_;                                                                      \
    const int width_ = (MODE == 0) ? 2 * D : D;                                                            \
    norm_bwd_reduce_kernel<<<dim3((width_ + 31) / 32, kNormReduceSlices), dim3(32, 32), 0, st>>>(partials, grid * ROWS, D, \
                                                                       MODE == 0 ? 1 : 0, dgamma, dbeta); \
    return cudaGetLastError();                                                                             \
  }
  if (D <= 256) LAUNCH(1, 1)
  if (D <= 512) LAUNCH(2, 1)
  if (D <= 768) LAUNCH(3, 1)
  if (D <= 1024) LAUNCH(4, 1)
  if (D <= 2048) LAUNCH(2, 4)
  if (D <= 4096) LAUNCH(4, 4)
  LAUNCH(8, 4)
#undef LAUNCH
}

// ------------------------------- embedding ------------------------------------------
__global__ void embed_fwd_kernel(const int32_t* __restrict__ idx, const __nv_bfloat16* __restrict__ wte,
                                 const __nv_bfloat16* __restrict__ wpe, __nv_bfloat16* __restrict__ out, int n_tok,
                                 int T, int D, int pos0) {
  const int vecs = D / 8;
  const int64_t total = static_cast<int64_t>(n_tok) * vecs;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int tok = static_cast<int>(i / vecs), c = static_cast<int>(i % vecs) * 8;
    float a[8];
    load8(wte + static_cast<int64_t>(idx[tok]) * D + c, a);
    if (wpe != nullptr) {
      float p[8];
      load8(wpe + static_cast<int64_t>(pos0 + tok % T) * D + c, p);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += p[j];
    }
    store8(out + static_cast<int64_t>(tok) * D + c, a);
  }
}

__global__ void embed_bwd_kernel(const int32_t* __restrict__ idx, const __nv_bfloat16* __restrict__ dout,
                                 float* __restrict__ dwte, float* __restrict__ dwpe, int n_tok, int T, int D,
                                 int pos0) {
  const int vecs = D / 8;
  const int64_t total = static_cast<int64_t>(n_tok) * vecs;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int tok = static_cast<int>(i / vecs), c = static_cast<int>(i % vecs) * 8;
    float g[8];
    load8(dout + static_cast<int64_t>(tok) * D + c, g);
    float* wt = dwte + static_cast<int64_t>(idx[tok]) * D + c;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(wt + j, g[j]);
    if (dwpe != nullptr) {
      float* wp = dwpe + static_cast<int64_t>(pos0 + tok % T) * D + c;
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(wp + j, g[j]);
    }
  }
}

// ------------------------------- cross entropy --------------------------------------
// One block per row. logits [M, ldl] bf16 (only the first V columns are real vocabulary).
// Writes loss[row] = logsumexp - logit[target] and, in place, dlogits = (softmax - onehot)
// * scale as bf16; padded columns get 0. A target < 0 marks an ignored row (loss 0, grad 0).
__global__ void __launch_bounds__(512)
ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const int32_t* __restrict__ targets,
                  float* __restrict__ loss, int V, int ldl, float scale, int write_grad) {
  __shared__ float red[32];
  __shared__ float bcast[2];
  const int row = blockIdx.x;
  __nv_bfloat16* lr = logits + static_cast<int64_t>(row) * ldl;
  const int tgt = targets[row];
  const int nvec = V / 8;  // full vectors; the tail is handled scalar
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8];
    load8(lr + i * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) mx = fmaxf(mx, f[j]);
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += blockDim.x) mx = fmaxf(mx, __bfloat162float(lr[c]));
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : -INFINITY;
    v = warp_max(v);
    if (threadIdx.x == 0) bcast[0] = v;
  }
  __syncthreads();
  mx = bcast[0];
  float se = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8];
    load8(lr + i * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) se += __expf(f[j] - mx);
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += blockDim.x) se += __expf(__bfloat162float(lr[c]) - mx);
  se = warp_sum(se);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = se;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) bcast[1] = v;
  }
  __syncthreads();
  se = bcast[1];
  const float lse = mx + logf(se);
  if (threadIdx.x == 0) loss[row] = (tgt >= 0) ? (lse - __bfloat162float(lr[tgt])) : 0.f;
  if (!write_grad) return;
  const float inv = (tgt >= 0) ? scale / se : 0.f;
  const int nvec_all = ldl / 8;
  for (int i = threadIdx.x; i < nvec_all; i += blockDim.x) {
    float f[8];
    load8(lr + i * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = i * 8 + j;
      float g = (c < V) ? __expf(f[j] - mx) * inv : 0.f;
      if (c == tgt) g -= scale;
      f[j] = g;
    }
    store8(lr + i * 8, f);
  }
}

// ------------------------------- bias gradient --------------------------------------
// dbias[c] += sum_rows dy[r, c]. Block = 32 x 8 threads handling a 256-column strip.
__global__ void bias_grad_kernel(const __nv_bfloat16* __restrict__ dy, float* __restrict__ dbias, int M, int N,
                                 int rows_per_block) {
  __shared__ float acc[8][256 + 8];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int col = blockIdx.x * 256 + tx * 8;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(M, r0 + rows_per_block);
  float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col < N) {
    for (int r = r0 + ty; r < r1; r += 8) {
      float f[8];
      load8(dy + static_cast<int64_t>(r) * N + col, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j] += f[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[ty][tx * 8 + j] = s[j];
  __syncthreads();
  const int t = ty * 32 + tx;  // 0..255 -> one column each
  float v = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) v += acc[k][t];
  const int c = blockIdx.x * 256 + t;
  if (c < N) atomicAdd(dbias + c, v);
}

// ------------------------------- optimizer ------------------------------------------
__global__ void sumsq_kernel(const float* __restrict__ g, int64_t n, float* __restrict__ out) {
  float s = 0.f;
  const int64_t n4 = n / 4;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float4 v = g4[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  for (int64_t i = n4 * 4 + blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    s += g[i] * g[i];
  __shared__ float red[32];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) atomicAdd(out, v);
  }
}

// One AdamW step over a flat range. Hyper-parameters that change every step live in a small
// device array so a captured CUDA graph can be replayed: hp = {lr, bias_corr1, bias_corr2,
// grad_scale}. gnorm_sq (optional) holds sum g^2 of the UNSCALED gradient over all ranges;
// the clip coefficient min(1, clip / (sqrt(gnorm_sq) * grad_scale)) is applied on the fly.
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, __nv_bfloat16* __restrict__ p_bf16, int64_t n,
                             const float* __restrict__ hp, const float* __restrict__ gnorm_sq, float beta1,
                             float beta2, float eps, float wd, float clip, int zero_grad) {
  const float lr = hp[0], bc1 = hp[1], bc2 = hp[2], gscale = hp[3];
  float coef = gscale;
  if (gnorm_sq != nullptr && clip > 0.f) {
    const float norm = sqrtf(*gnorm_sq) * gscale;
    coef *= fminf(1.f, clip / (norm + 1e-6f));
  }
  auto update = [&](float gi, float& mi, float& vi, float& pi) {
    gi *= coef;
    mi = beta1 * mi + (1.f - beta1) * gi;
    vi = beta2 * vi + (1.f - beta2) * gi * gi;
    const float u = (mi / bc1) / (sqrtf(vi / bc2) + eps) + wd * pi;
    pi -= lr * u;
  };
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t nth = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
                     reinterpret_cast<uintptr_t>(v)) & 15) == 0 &&
                   (p_bf16 == nullptr || (reinterpret_cast<uintptr_t>(p_bf16) & 7) == 0);
  const int64_t n4 = vec ? n / 4 : 0;
  for (int64_t i = tid; i < n4; i += nth) {
    float4 gv = reinterpret_cast<float4*>(g)[i], mv = reinterpret_cast<float4*>(m)[i],
           vv = reinterpret_cast<float4*>(v)[i], pv = reinterpret_cast<float4*>(p)[i];
    update(gv.x, mv.x, vv.x, pv.x);
    update(gv.y, mv.y, vv.y, pv.y);
    update(gv.z, mv.z, vv.z, pv.z);
    update(gv.w, mv.w, vv.w, pv.w);
    reinterpret_cast<float4*>(m)[i] = mv;
    reinterpret_cast<float4*>(v)[i] = vv;
    reinterpret_cast<float4*>(p)[i] = pv;
    if (p_bf16 != nullptr)
      reinterpret_cast<uint2*>(p_bf16)[i] = make_uint2(pack_bf16x2(pv.x, pv.y), pack_bf16x2(pv.z, pv.w));
    if (zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int64_t i = n4 * 4 + tid; i < n; i += nth) {
    float mi = m[i], vi = v[i], pi = p[i];
    update(g[i], mi, vi, pi);
    m[i] = mi;
    v[i] = vi;
    p[i] = pi;
    if (p_bf16 != nullptr) p_bf16[i] = __float2bfloat16(pi);
    if (zero_grad) g[i] = 0.f;
  }
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, int64_t n) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    out[i] = __float2bfloat16(in[i]);
}

}  // namespace

cudaError_t launch_norm_fwd(int mode, const __nv_bfloat16* x, const __nv_bfloat16* gamma, const __nv_bfloat16* beta,
                            __nv_bfloat16* y, float* mean, float* rstd, int M, int D, float eps, cudaStream_t st) {
  if (M <= 0) return cudaSuccess;
  if (mode == 0) return norm_fwd_dispatch<0>(x, gamma, beta, y, mean, rstd, M, D, eps, st);
  if (mode == 1) return norm_fwd_dispatch<1>(x, gamma, beta, y, mean, rstd, M, D, eps, st);
  return norm_fwd_dispatch<2>(x, gamma, beta, y, mean, rstd, M, D, eps, st);
}

cudaError_t launch_norm_bwd(int mode, const __nv_bfloat16* dy, const __nv_bfloat16* x, const __nv_bfloat16* gamma,
                            const float* mean, const float* rstd, const __nv_bfloat16* dres, __nv_bfloat16* dx,
                            float* dgamma, float* dbeta, float* partials, int M, int D, cudaStream_t st) {
  if (M <= 0) return cudaSuccess;
  if (mode == 0) return norm_bwd_dispatch<0>(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, partials, M, D, st);
  if (mode == 1) return norm_bwd_dispatch<1>(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, partials, M, D, st);
  return norm_bwd_dispatch<2>(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, partials, M, D, st);
}

cudaError_t launch_embed_fwd(const int32_t* idx, const __nv_bfloat16* wte, const __nv_bfloat16* wpe,
                             __nv_bfloat16* out, int n_tok, int T, int D, int pos0, cudaStream_t st) {
  if (D % 8 != 0) return cudaErrorInvalidValue;
  const int64_t total = static_cast<int64_t>(n_tok) * (D / 8);
  const int grid = static_cast<int>(std::min<int64_t>((total + 255) / 256, 148 * 16));
  embed_fwd_kernel<<<grid, 256, 0, st>>>(idx, wte, wpe, out, n_tok, T, D, pos0);
  return cudaGetLastError();
}

cudaError_t launch_embed_bwd(const int32_t* idx, const __nv_bfloat16* dout, float* dwte, float* dwpe, int n_tok,
                             int T, int D, int pos0, cudaStream_t st) {
  if (D % 8 != 0) return cudaErrorInvalidValue;
  const int64_t total = static_cast<int64_t>(n_tok) * (D / 8);
  const int grid = static_cast<int>(std::min<int64_t>((total + 255) / 256, 148 * 16));
  embed_bwd_kernel<<<grid, 256, 0, st>>>(idx, dout, dwte, dwpe, n_tok, T, D, pos0);
  return cudaGetLastError();
}

cudaError_t launch_ce_fwd_bwd(__nv_bfloat16* logits, const int32_t* targets, float* loss, int M, int V, int ldl,
                              float scale, int write_grad, cudaStream_t st) {
  if (ldl % 8 != 0 || V > ldl) return cudaErrorInvalidValue;
  ce_fwd_bwd_kernel<<<M, 512, 0, st>>>(logits, targets, loss, V, ldl, scale, write_grad);
  return cudaGetLastError();
}

cudaError_t launch_bias_grad(const __nv_bfloat16* dy, float* dbias, int M, int N, cudaStream_t st) {
  if (N % 8 != 0) return cudaErrorInvalidValue;
  const int col_blocks = (N + 255) / 256;
  int row_blocks = (148 * 4 + col_blocks - 1) / col_blocks;
  int rows_per_block = (M + row_blocks - 1) / row_blocks;
  rows_per_block = ((rows_per_block + 7) / 8) * 8;
  row_blocks = (M + rows_per_block - 1) / rows_per_block;
  bias_grad_kernel<<<dim3(col_blocks, row_blocks), dim3(32, 8), 0, st>>>(dy, dbias, M, N, rows_per_block);
  return cudaGetLastError();
}

cudaError_t launch_sumsq(const float* g, int64_t n, float* out, cudaStream_t st) {
  const int grid = static_cast<int>(std::min<int64_t>((n / 4 + 255) / 256 + 1, 148 * 8));
  sumsq_kernel<<<grid, 256, 0, st>>>(g, n, out);
  return cudaGetLastError();
}

// AdamW with ALL state in bf16: the weights themselves are the master copy and both moments are bf16, 6 bytes of
// state per parameter instead of 16 (the 77 B-parameter expert banks of the MoE benchmark shapes do not fit
// otherwise). Every bf16 store is rounded stochastically (a per-element hash of index and step supplies the lower
// 16 bits), so updates smaller than half a bf16 ulp still move the weight in expectation instead of being lost.
__device__ __forceinline__ uint32_t hash32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352dU;
  x ^= x >> 15;
  x *= 0x846ca68bU;
  x ^= x >> 16;
  return x;
}
__device__ __forceinline__ uint32_t sr_bf16_bits(float x, uint32_t rnd16) {
  uint32_t b = __float_as_uint(x);
  if ((b & 0x7f800000u) != 0x7f800000u) b += rnd16;   // leave inf / nan alone
  return b >> 16;
}

__global__ void adamw_bf16_state_kernel(__nv_bfloat16* __restrict__ p, float* __restrict__ g,
                                        __nv_bfloat16* __restrict__ m, __nv_bfloat16* __restrict__ v, int64_t n,
                                        const float* __restrict__ hp, const float* __restrict__ gnorm_sq, float beta1,
                                        float beta2, float eps, float wd, float clip, int zero_grad, uint32_t seed) {
  const float lr = hp[0], bc1 = hp[1], bc2 = hp[2], gscale = hp[3];
  float coef = gscale;
  if (gnorm_sq != nullptr && clip > 0.f) {
    const float norm = sqrtf(*gnorm_sq) * gscale;
    coef *= fminf(1.f, clip / (norm + 1e-6f));
  }
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t nth = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = tid; i < n; i += nth) {
    float gi = g[i] * coef;
    float mi = __bfloat162float(m[i]), vi = __bfloat162float(v[i]), pi = __bfloat162float(p[i]);
    mi = beta1 * mi + (1.f - beta1) * gi;
    vi = beta2 * vi + (1.f - beta2) * gi * gi;
    pi -= lr * ((mi / bc1) / (sqrtf(vi / bc2) + eps) + wd * pi);
    const uint32_t r = hash32(static_cast<uint32_t>(i) * 0x9e3779b9u + static_cast<uint32_t>(i >> 32) + seed);
    const uint32_t r2 = hash32(r ^ 0x85ebca6bu);
    reinterpret_cast<uint16_t*>(p)[i] = static_cast<uint16_t>(sr_bf16_bits(pi, r & 0xffffu));
    reinterpret_cast<uint16_t*>(m)[i] = static_cast<uint16_t>(sr_bf16_bits(mi, r >> 16));
    reinterpret_cast<uint16_t*>(v)[i] = static_cast<uint16_t>(sr_bf16_bits(vi, r2 & 0xffffu));
    if (zero_grad) g[i] = 0.f;
  }
}

cudaError_t launch_adamw_bf16_state(__nv_bfloat16* p, float* g, __nv_bfloat16* m, __nv_bfloat16* v, int64_t n,
                                    const float* hp, const float* gnorm_sq, float beta1, float beta2, float eps,
                                    float wd, float clip, int zero_grad, uint32_t seed, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  const int grid = static_cast<int>(std::min<int64_t>((n + 255) / 256, 148 * 16));
  adamw_bf16_state_kernel<<<grid, 256, 0, st>>>(p, g, m, v, n, hp, gnorm_sq, beta1, beta2, eps, wd, clip, zero_grad,
                                                seed);
  return cudaGetLastError();
}

cudaError_t launch_adamw(float* p, float* g, float* m, float* v, __nv_bfloat16* p_bf16, int64_t n, const float* hp,
                         const float* gnorm_sq, float beta1, float beta2, float eps, float wd, float clip,
                         int zero_grad, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  const int grid = static_cast<int>(std::min<int64_t>((n + 255) / 256, 148 * 16));
  adamw_kernel<<<grid, 256, 0, st>>>(p, g, m, v, p_bf16, n, hp, gnorm_sq, beta1, beta2, eps, wd, clip, zero_grad);
  return cudaGetLastError();
}

cudaError_t launch_cast_f32_bf16(const float* in, __nv_bfloat16* out, int64_t n, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  const int grid = static_cast<int>(std::min<int64_t>((n + 255) / 256, 148 * 16));
  cast_f32_bf16_kernel<<<grid, 256, 0, st>>>(in, out, n);
  return cudaGetLastError();
}

}  // namespace b200
