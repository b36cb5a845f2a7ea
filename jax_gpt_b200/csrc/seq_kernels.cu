// Routing, rotary, FP8 quantisation and Gated-DeltaNet decode kernels.
//
// Semantics: softmax top-k router with renormalisation (jax_gpt/models/qwen35/moe.py:50-55);
// DeepSeek-V3 group-limited sigmoid router (HF deepseek_v3 `route_tokens_to_experts`); per-head
// RMSNorm with (1 + w) and half-split partial rotary (jax_gpt/models/qwen35/primitives.py:29-32,
// 79-109, jax_gpt/models/qwen35/gqa.py:67-85); the gated delta-rule decode step with its conv
// window update and gated RMSNorm (jax_gpt/models/qwen35/deltanet.py:51-56,129-203,437-443).
#include "seq_kernels.cuh"

#include <cuda_fp8.h>

#include "common.cuh"

namespace b200 {

namespace {

constexpr int kMaxPerLane = 16;  // E <= 512

__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Warp-wide argmax over (value, index) pairs; the smaller index wins ties.
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) {
      v = ov;
      i = oi;
    }
  }
}

// One warp per token. Lane l holds experts [l * per, (l + 1) * per).
__global__ void router_kernel(int mode, const float* __restrict__ logits, const float* __restrict__ bias, int M, int E,
                              int k, int n_group, int topk_group, float scale, float* __restrict__ weights,
                              int* __restrict__ ids, int* __restrict__ counts) {
  const int tok = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (tok >= M) return;
  const int per = E / 32;
  float s[kMaxPerLane], c[kMaxPerLane];
  const float* row = logits + static_cast<int64_t>(tok) * E + lane * per;
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    if (j < per) {
      const float x = row[j];
      if (mode == 1) {
        s[j] = 1.f / (1.f + __expf(-x));
        c[j] = s[j] + (bias != nullptr ? bias[lane * per + j] : 0.f);
      } else {
        s[j] = x;
        c[j] = x;
      }
    } else {
      s[j] = 0.f;
      c[j] = -INFINITY;
    }
  }
  if (mode == 1 && n_group > 1) {
    // group score = sum of the two largest selection scores of the group
    float t1 = -INFINITY, t2 = -INFINITY;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      if (j < per) {
        if (c[j] > t1) { t2 = t1; t1 = c[j]; }
        else if (c[j] > t2) t2 = c[j];
      }
    }
    const int lanes_per_group = 32 / n_group;
    for (int o = 1; o < lanes_per_group; o <<= 1) {
      const float b1 = __shfl_xor_sync(0xffffffffu, t1, o), b2 = __shfl_xor_sync(0xffffffffu, t2, o);
      const float n1 = fmaxf(t1, b1);
      const float n2 = fmaxf(fminf(t1, b1), fmaxf(t2, b2));
      t1 = n1;
      t2 = n2;
    }
    const int my_group = lane / lanes_per_group;
    const bool leader = (lane % lanes_per_group) == 0;
    float gscore = t1 + t2;
    unsigned kept = 0;
    for (int r = 0; r < topk_group; ++r) {
      float v = (leader && !((kept >> my_group) & 1u)) ? gscore : -INFINITY;
      int gi = my_group;
      warp_argmax(v, gi);
      kept |= 1u << gi;
    }
    if (!((kept >> my_group) & 1u)) {
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j)
        if (j < per) c[j] = 0.f;  // masked-out experts compete with score 0, as in the HF implementation
    }
  }
  float mx = 0.f, denom = 1.f;
  if (mode == 0) {
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (j < per) m = fmaxf(m, s[j]);
    mx = warp_max_f(m);
  }
  // top-k by repeated warp argmax
  float wsel = 0.f;   // lane r keeps the r-th selected weight
  int isel = 0;
  float wsum = 0.f;
  for (int r = 0; r < k; ++r) {
    float bv = -INFINITY;
    int bj = 0;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (j < per && c[j] > bv) { bv = c[j]; bj = j; }
    float v = bv;
    int gi = lane * per + bj;
    warp_argmax(v, gi);
    const int owner = gi / per, oj = gi - owner * per;
    float sv = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (j == oj) sv = s[j];
    sv = __shfl_sync(0xffffffffu, sv, owner);
    if (lane == owner) {
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j)
        if (j == oj) c[j] = -INFINITY;
    }
    const float wv = (mode == 0) ? __expf(sv - mx) : sv;
    wsum += wv;
    if (lane == r) { wsel = wv; isel = gi; }
  }
  denom = (mode == 0) ? wsum : (wsum + 1e-20f);
  if (lane < k) {
    const float out = (mode == 0) ? wsel / denom : wsel / denom * scale;
    weights[static_cast<int64_t>(tok) * k + lane] = out;
    ids[static_cast<int64_t>(tok) * k + lane] = isel;
    if (counts != nullptr) atomicAdd(counts + isel, 1);
  }
}

// One warp per (row, head).
__global__ void rmsnorm_rope_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ norm_w,
                                    const float* __restrict__ freqs, __nv_bfloat16* __restrict__ y, int rows, int T,
                                    int H, int dh, int rope_dim, int pos0, float eps, int one_plus) {
  const int64_t gw = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= static_cast<int64_t>(rows) * H) return;
  const int64_t row = gw / H;
  const int per = dh / 32;
  const __nv_bfloat16* xp = x + gw * dh + lane * per;
  float v[8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    v[j] = (j < per) ? __bfloat162float(xp[j]) : 0.f;
    ss += v[j] * v[j];
  }
  if (norm_w != nullptr) {
    const float r = rsqrtf(warp_sum_f(ss) / dh + eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j < per) {
        const float w = __bfloat162float(norm_w[lane * per + j]);
        v[j] = v[j] * r * (one_plus ? 1.f + w : w);
      }
    }
  }
  if (rope_dim > 0) {
    const int half = rope_dim / 2;
    const int dl = half / per;  // partner lane distance
    const int pos = pos0 + static_cast<int>(row % T);
    const float* fr = freqs + static_cast<int64_t>(pos) * half * 2;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j < per) {
        const int i = lane * per + j;
        const float lo = __shfl_sync(0xffffffffu, v[j], (lane + 32 - dl) & 31);  // partner below (i - half)
        const float hi = __shfl_sync(0xffffffffu, v[j], (lane + dl) & 31);       // partner above (i + half)
        if (i < half) {
          v[j] = v[j] * fr[i * 2] - hi * fr[i * 2 + 1];
        } else if (i < rope_dim) {
          v[j] = v[j] * fr[(i - half) * 2] + lo * fr[(i - half) * 2 + 1];
        }
      }
    }
  }
  __nv_bfloat16* yp = y + gw * dh + lane * per;
#pragma unroll
  for (int j = 0; j < 8; ++j)
    if (j < per) yp[j] = __float2bfloat16(v[j]);
}

// Backward of rmsnorm_rope_kernel: persistent blocks, one warp per (row, head) item; the weight gradient is
// accumulated per lane over the block's items, reduced through shared memory and flushed once per block.
__global__ void rmsnorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                        const __nv_bfloat16* __restrict__ norm_w, const float* __restrict__ freqs,
                                        __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, int rows, int T, int H,
                                        int dh, int rope_dim, int pos0, float eps, int one_plus) {
  __shared__ float red[8][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per = dh / 32;
  const int64_t items = static_cast<int64_t>(rows) * H;
  float dw_acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int64_t gw = blockIdx.x * 8 + warp; gw < items; gw += static_cast<int64_t>(gridDim.x) * 8) {
    const int64_t row = gw / H;
    const __nv_bfloat16* xp = x + gw * dh + lane * per;
    const __nv_bfloat16* gp = dy + gw * dh + lane * per;
    float xv[8], dv[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      xv[j] = (j < per) ? __bfloat162float(xp[j]) : 0.f;
      dv[j] = (j < per) ? __bfloat162float(gp[j]) : 0.f;
      ss += xv[j] * xv[j];
    }
    if (rope_dim > 0) {   // transpose of the rotation
      const int half = rope_dim / 2;
      const int dl = half / per;
      const int pos = pos0 + static_cast<int>(row % T);
      const float* fr = freqs + static_cast<int64_t>(pos) * half * 2;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (j < per) {
          const int i = lane * per + j;
          const float lo = __shfl_sync(0xffffffffu, dv[j], (lane + 32 - dl) & 31);
          const float hi = __shfl_sync(0xffffffffu, dv[j], (lane + dl) & 31);
          if (i < half) {
            dv[j] = dv[j] * fr[i * 2] + hi * fr[i * 2 + 1];
          } else if (i < rope_dim) {
            dv[j] = dv[j] * fr[(i - half) * 2] - lo * fr[(i - half) * 2 + 1];
          }
        }
      }
    }
    if (norm_w != nullptr) {
      const float r = rsqrtf(warp_sum_f(ss) / dh + eps);
      float dot = 0.f;
      float dxh[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (j < per) {
          const float w = __bfloat162float(norm_w[lane * per + j]);
          const float xh = xv[j] * r;
          dw_acc[j] += dv[j] * xh;
          dxh[j] = dv[j] * (one_plus ? 1.f + w : w);
          dot += dxh[j] * xh;
          xv[j] = xh;
        } else {
          dxh[j] = 0.f;
        }
      }
      dot = warp_sum_f(dot) / dh;
#pragma unroll
      for (int j = 0; j < 8; ++j) dv[j] = r * (dxh[j] - xv[j] * dot);
    }
    __nv_bfloat16* op = dx + gw * dh + lane * per;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < per) op[j] = __float2bfloat16(dv[j]);
  }
  if (norm_w != nullptr && dw != nullptr) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < per) red[warp][lane * per + j] = dw_acc[j];
    __syncthreads();
    for (int i = threadIdx.x; i < dh; i += blockDim.x) {
      float t = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < 8; ++w8) t += red[w8][i];
      atomicAdd(dw + i, t);
    }
  }
}

__device__ __forceinline__ float pow2_ceil(float s) {
  // smallest power of two >= s (s > 0)
  int e;
  const float m = frexpf(s, &e);  // s = m * 2^e, m in [0.5, 1)
  return (m == 0.5f) ? ldexpf(1.f, e - 1) : ldexpf(1.f, e);
}

__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

// One warp per 1 x 128 block.
__global__ void fp8_quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                       float* __restrict__ scales, int M, int K, int pow2) {
  const int64_t gw = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int kb = K / 128;
  if (gw >= static_cast<int64_t>(M) * kb) return;
  const int64_t row = gw / kb;
  const int blk = static_cast<int>(gw % kb);
  const __nv_bfloat16* p = x + row * K + blk * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
  amax = warp_max_f(amax);
  float sc = fmaxf(amax, 1e-12f) / 448.f;
  if (pow2) sc = pow2_ceil(sc);
  const float inv = 1.f / sc;
  const uint32_t pk = to_e4m3(a.x * inv) | (to_e4m3(a.y * inv) << 8) | (to_e4m3(b.x * inv) << 16) |
                      (static_cast<uint32_t>(to_e4m3(b.y * inv)) << 24);
  *reinterpret_cast<uint32_t*>(q + row * K + blk * 128 + lane * 4) = pk;
  if (lane == 0) scales[row * kb + blk] = sc;
}

// Block-scaled e4m3 quantisation for the hardware-scaled GEMM, one CTA (256 threads) per 128 x 128 tile of x
// [R, C] bf16, optionally TRANSPOSING: the output is q [R, C] (contraction along C) or q^T [C, R] (contraction
// along R) with one power-of-two scale per 1 x 128 block of an output row (kBlock = false) or per 128 x 128 tile
// (kBlock = true). The scales are written twice: as fp32 ([rows, Kc/128] or [rows/128, Kc/128]) and as exponent
// bytes in the packed layout the GEMM copies into tensor memory: [rows/128, Kc/128, 512] bytes, the word at byte
// (r % 32) * 16 + ((r % 128) / 32) * 4 of a chunk holding the exponent of output row r four times.
// The tile passes through shared memory, so both the reads of x and the writes of q move whole lines also
// when transposing (the weight-gradient operands of an FP8 layer are x^T and dy^T).
template <bool kTranspose, bool kBlock>
__global__ void __launch_bounds__(256)
fp8_quant_mx_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scales,
                    uint8_t* __restrict__ sf_packed, int R, int C) {
  constexpr int kLd = 136;  // padded row of the staged tile, in elements (272 bytes: keeps 16-byte alignment)
  __shared__ __align__(16) __nv_bfloat16 tile[128 * kLd];
  __shared__ float red[8];
  const int cb = C / 128;
  const int tr = blockIdx.x / cb, tc = blockIdx.x % cb;
  const int r0 = tr * 128, c0 = tc * 128;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int idx = it * 256 + threadIdx.x;
    const int row = idx >> 4, cv = idx & 15;
    const uint4 v = *reinterpret_cast<const uint4*>(x + static_cast<int64_t>(r0 + row) * C + c0 + cv * 8);
    *reinterpret_cast<uint4*>(tile + row * kLd + cv * 8) = v;
  }
  __syncthreads();
  const int line = threadIdx.x >> 1, half = threadIdx.x & 1;  // output row inside the tile, which 64 of its elements
  float f[64];
  float amax = 0.f;
  if (!kTranspose) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 v = *reinterpret_cast<const uint4*>(tile + line * kLd + half * 64 + i * 8);
      const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
      f[8 * i] = a.x; f[8 * i + 1] = a.y; f[8 * i + 2] = b.x; f[8 * i + 3] = b.y;
      f[8 * i + 4] = c.x; f[8 * i + 5] = c.y; f[8 * i + 6] = d.x; f[8 * i + 7] = d.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 64; ++i) f[i] = __bfloat162float(tile[(half * 64 + i) * kLd + line]);
  }
#pragma unroll
  for (int i = 0; i < 64; ++i) amax = fmaxf(amax, fabsf(f[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));  // the two halves of a line sit in adjacent lanes
  if (kBlock) {
    amax = warp_max_f(amax);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  }
  const float sc = pow2_ceil(fmaxf(amax, 1e-12f) / 448.f);
  const float inv = 1.f / sc;
  // output geometry: row of q this line becomes, and the 128-wide block along the contraction dimension
  const int out_row = kTranspose ? (c0 + line) : (r0 + line);
  const int kblk = kTranspose ? tr : tc;
  const int64_t ldq = kTranspose ? R : C;
  const int n_kblk = static_cast<int>(ldq / 128);
  uint8_t* qp = q + static_cast<int64_t>(out_row) * ldq + kblk * 128 + half * 64;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float* g = f + i * 16 + j * 4;
      w[j] = to_e4m3(g[0] * inv) | (to_e4m3(g[1] * inv) << 8) | (to_e4m3(g[2] * inv) << 16) |
             (static_cast<uint32_t>(to_e4m3(g[3] * inv)) << 24);
    }
    *reinterpret_cast<uint4*>(qp + i * 16) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  if (half == 0) {
    int e;
    frexpf(sc, &e);                                   // sc = 0.5 * 2^e exactly
    const uint32_t byte = static_cast<uint32_t>(min(254, max(0, e - 1 + 127)));
    uint8_t* chunk = sf_packed + (static_cast<int64_t>(out_row >> 7) * n_kblk + kblk) * 512;
    *reinterpret_cast<uint32_t*>(chunk + (out_row & 31) * 16 + ((out_row & 127) >> 5) * 4) = byte * 0x01010101u;
    if (scales != nullptr) {
      if (!kBlock) scales[static_cast<int64_t>(out_row) * n_kblk + kblk] = sc;
      else if (line == 0) scales[static_cast<int64_t>(out_row >> 7) * n_kblk + kblk] = sc;
    }
  }
}

// One block of 256 threads per 128 x 128 tile.
__global__ void fp8_quant_128x128_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q,
                                         float* __restrict__ scales, int R, int C, int pow2) {
  __shared__ float red[8];
  __shared__ float sc_s;
  const int cb = C / 128;
  const int tr = blockIdx.x / cb, tc = blockIdx.x % cb;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float amax = 0.f;
  for (int r = warp; r < 128; r += 8) {
    const uint2 raw = *reinterpret_cast<const uint2*>(w + static_cast<int64_t>(tr * 128 + r) * C + tc * 128 + lane * 4);
    const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))));
  }
  amax = warp_max_f(amax);
  if (lane == 0) red[warp] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.f;
    for (int i = 0; i < 8; ++i) m = fmaxf(m, red[i]);
    float sc = fmaxf(m, 1e-12f) / 448.f;
    if (pow2) sc = pow2_ceil(sc);
    sc_s = sc;
    scales[tr * cb + tc] = sc;
  }
  __syncthreads();
  const float inv = 1.f / sc_s;
  for (int r = warp; r < 128; r += 8) {
    const int64_t off = static_cast<int64_t>(tr * 128 + r) * C + tc * 128 + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(w + off);
    const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
    const uint32_t pk = to_e4m3(a.x * inv) | (to_e4m3(a.y * inv) << 8) | (to_e4m3(b.x * inv) << 16) |
                        (static_cast<uint32_t>(to_e4m3(b.y * inv)) << 24);
    *reinterpret_cast<uint32_t*>(q + off) = pk;
  }
}

}  // namespace

namespace {

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }

// Block-wide sum for blockDim.x <= 256 (scratch: 8 floats).
__device__ __forceinline__ float block_sum_256(float v, float* scratch) {
  v = warp_sum_f(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
  for (int i = 0; i < (blockDim.x + 31) / 32; ++i) s += scratch[i];
  return s;
}

// Shifts the conv window of `channel` left, appends x_new, returns silu(sum_k w[k] * window[k]).
__device__ __forceinline__ float conv_step(float* state, const __nv_bfloat16* w, int Kc, float x_new) {
  float acc = 0.f;
  for (int k = 0; k < Kc - 1; ++k) {
    const float s = state[k + 1];
    state[k] = s;
    acc += s * __bfloat162float(w[k]);
  }
  state[Kc - 1] = x_new;
  acc += x_new * __bfloat162float(w[Kc - 1]);
  return silu_f(acc);
}

// One block per (sequence, qk head); it serves the Hv / Hqk value heads that share the qk head.
// Thread t owns q/k feature t (t < dk) and output feature t (t < dv): blockDim.x = max(dk, dv).
__global__ void gdn_decode_kernel(const __nv_bfloat16* __restrict__ mixed, const __nv_bfloat16* __restrict__ z,
                                  const __nv_bfloat16* __restrict__ bproj, const __nv_bfloat16* __restrict__ aproj,
                                  float* __restrict__ conv_state, const __nv_bfloat16* __restrict__ conv_w,
                                  const __nv_bfloat16* __restrict__ A_log, const __nv_bfloat16* __restrict__ dt_bias,
                                  const __nv_bfloat16* __restrict__ norm_w, float* __restrict__ state,
                                  __nv_bfloat16* __restrict__ out, int Hqk, int Hv, int dk, int dv, int Kc, float eps,
                                  int ld_mixed, int ld_z, int ld_b, int ld_a) {
  extern __shared__ float sm[];
  float* qs = sm;            // [dk]
  float* ks = sm + dk;       // [dk]
  float* scratch = sm + 2 * dk;
  const int b = blockIdx.x / Hqk, hq = blockIdx.x % Hqk;
  const int rep = Hv / Hqk;
  const int Kd = Hqk * dk, Vd = Hv * dv, C = 2 * Kd + Vd;
  const int t = threadIdx.x;
  const __nv_bfloat16* mx = mixed + static_cast<int64_t>(b) * ld_mixed;   // the inputs may be column slices of one GEMM output
  float* cs = conv_state + static_cast<int64_t>(b) * C * Kc;
  float qv = 0.f, kv_ = 0.f;
  if (t < dk) {
    const int cq = hq * dk + t, ck = Kd + hq * dk + t;
    qv = conv_step(cs + static_cast<int64_t>(cq) * Kc, conv_w + static_cast<int64_t>(cq) * Kc, Kc, __bfloat162float(mx[cq]));
    kv_ = conv_step(cs + static_cast<int64_t>(ck) * Kc, conv_w + static_cast<int64_t>(ck) * Kc, Kc, __bfloat162float(mx[ck]));
  }
  const float qn = block_sum_256(qv * qv, scratch);
  const float kn = block_sum_256(kv_ * kv_, scratch);
  if (t < dk) {
    qs[t] = qv * rsqrtf(qn + 1e-6f) * rsqrtf(static_cast<float>(dk));
    ks[t] = kv_ * rsqrtf(kn + 1e-6f);
  }
  __syncthreads();
  for (int r = 0; r < rep; ++r) {
    const int hv = hq * rep + r;
    float o = 0.f, zv = 0.f;
    if (t < dv) {
      const int cv = 2 * Kd + hv * dv + t;
      const float vv = conv_step(cs + static_cast<int64_t>(cv) * Kc, conv_w + static_cast<int64_t>(cv) * Kc, Kc,
                                 __bfloat162float(mx[cv]));
      const float beta = 1.f / (1.f + __expf(-__bfloat162float(bproj[static_cast<int64_t>(b) * ld_b + hv])));
      const float xa = __bfloat162float(aproj[static_cast<int64_t>(b) * ld_a + hv]) + __bfloat162float(dt_bias[hv]);
      const float sp = (xa > 20.f) ? xa : log1pf(__expf(xa));
      const float eg = __expf(-__expf(__bfloat162float(A_log[hv])) * sp);
      float* S = state + (static_cast<int64_t>(b) * Hv + hv) * dk * dv + t;  // column t, stride dv
      float kvm = 0.f;
      for (int i = 0; i < dk; ++i) kvm += S[static_cast<int64_t>(i) * dv] * eg * ks[i];
      const float delta = (vv - kvm) * beta;
      for (int i = 0; i < dk; ++i) {
        const float s = S[static_cast<int64_t>(i) * dv] * eg + ks[i] * delta;
        S[static_cast<int64_t>(i) * dv] = s;
        o += s * qs[i];
      }
      zv = __bfloat162float(z[static_cast<int64_t>(b) * ld_z + hv * dv + t]);
    }
    const float ms = block_sum_256((t < dv) ? o * o : 0.f, scratch) / dv;
    if (t < dv)
      out[static_cast<int64_t>(b) * Vd + hv * dv + t] =
          __float2bfloat16(__bfloat162float(norm_w[t]) * o * rsqrtf(ms + eps) * silu_f(zv));
  }
}

}  // namespace

cudaError_t launch_router(int mode, const float* logits, const float* bias, int M, int E, int k, int n_group,
                          int topk_group, float scale, float* weights, int* ids, int* counts, cudaStream_t st) {
  if (E % 32 != 0 || E > 32 * kMaxPerLane || k > 32 || k < 1) return cudaErrorInvalidValue;
  if (mode == 1 && n_group > 1 && (32 % n_group != 0 || E % n_group != 0 || topk_group > n_group))
    return cudaErrorInvalidValue;
  if (M <= 0) return cudaSuccess;
  router_kernel<<<(M + 7) / 8, 256, 0, st>>>(mode, logits, bias, M, E, k, n_group, topk_group, scale, weights, ids,
                                             counts);
  return cudaGetLastError();
}

cudaError_t launch_rmsnorm_rope(const __nv_bfloat16* x, const __nv_bfloat16* norm_w, const float* freqs,
                                __nv_bfloat16* y, int rows, int T, int H, int dh, int rope_dim, int pos0, float eps,
                                int one_plus, cudaStream_t st) {
  if (dh % 32 != 0 || dh > 256) return cudaErrorInvalidValue;
  const int per = dh / 32;
  if (rope_dim > 0 && (rope_dim % 2 != 0 || (rope_dim / 2) % per != 0 || rope_dim > dh)) return cudaErrorInvalidValue;
  const int64_t warps = static_cast<int64_t>(rows) * H;
  if (warps <= 0) return cudaSuccess;
  rmsnorm_rope_kernel<<<static_cast<int>((warps + 7) / 8), 256, 0, st>>>(x, norm_w, freqs, y, rows, T, H, dh, rope_dim,
                                                                       pos0, eps, one_plus);
  return cudaGetLastError();
}

cudaError_t launch_rmsnorm_rope_bwd(const __nv_bfloat16* x, const __nv_bfloat16* dy, const __nv_bfloat16* norm_w,
                                    const float* freqs, __nv_bfloat16* dx, float* dw, int rows, int T, int H, int dh,
                                    int rope_dim, int pos0, float eps, int one_plus, cudaStream_t st) {
  if (dh % 32 != 0 || dh > 256) return cudaErrorInvalidValue;
  const int per = dh / 32;
  if (rope_dim > 0 && (rope_dim % 2 != 0 || (rope_dim / 2) % per != 0 || rope_dim > dh)) return cudaErrorInvalidValue;
  const int64_t warps = static_cast<int64_t>(rows) * H;
  if (warps <= 0) return cudaSuccess;
  const int64_t want = (warps + 7) / 8;
  rmsnorm_rope_bwd_kernel<<<static_cast<int>(want < 1184 ? want : 1184), 256, 0, st>>>(
      x, dy, norm_w, freqs, dx, dw, rows, T, H, dh, rope_dim, pos0, eps, one_plus);
  return cudaGetLastError();
}

cudaError_t launch_fp8_quant_1x128(const __nv_bfloat16* x, uint8_t* q, float* scales, int M, int K, int pow2,
                                   cudaStream_t st) {
  if (K % 128 != 0) return cudaErrorInvalidValue;
  const int64_t warps = static_cast<int64_t>(M) * (K / 128);
  if (warps <= 0) return cudaSuccess;
  fp8_quant_1x128_kernel<<<static_cast<int>((warps + 7) / 8), 256, 0, st>>>(x, q, scales, M, K, pow2);
  return cudaGetLastError();
}

cudaError_t launch_fp8_quant_128x128(const __nv_bfloat16* w, uint8_t* q, float* scales, int R, int C, int pow2,
                                     cudaStream_t st) {
  if (R % 128 != 0 || C % 128 != 0) return cudaErrorInvalidValue;
  fp8_quant_128x128_kernel<<<(R / 128) * (C / 128), 256, 0, st>>>(w, q, scales, R, C, pow2);
  return cudaGetLastError();
}

cudaError_t launch_fp8_quant_mx(const __nv_bfloat16* x, uint8_t* q, float* scales, uint8_t* sf_packed, int R, int C,
                                int transpose, int block, cudaStream_t st) {
  if (R % 128 != 0 || C % 128 != 0 || R <= 0 || C <= 0) return cudaErrorInvalidValue;
  const int grid = (R / 128) * (C / 128);
  if (transpose) {
    if (block) fp8_quant_mx_kernel<true, true><<<grid, 256, 0, st>>>(x, q, scales, sf_packed, R, C);
    else fp8_quant_mx_kernel<true, false><<<grid, 256, 0, st>>>(x, q, scales, sf_packed, R, C);
  } else {
    if (block) fp8_quant_mx_kernel<false, true><<<grid, 256, 0, st>>>(x, q, scales, sf_packed, R, C);
    else fp8_quant_mx_kernel<false, false><<<grid, 256, 0, st>>>(x, q, scales, sf_packed, R, C);
  }
  return cudaGetLastError();
}

cudaError_t launch_gdn_decode_step(const __nv_bfloat16* mixed, const __nv_bfloat16* z, const __nv_bfloat16* bproj,
                                   const __nv_bfloat16* aproj, float* conv_state, const __nv_bfloat16* conv_w,
                                   const __nv_bfloat16* A_log, const __nv_bfloat16* dt_bias,
                                   const __nv_bfloat16* norm_w, float* state, __nv_bfloat16* out, int B, int Hqk, int Hv,
                                   int dk, int dv, int Kc, float eps, int ld_mixed, int ld_z, int ld_b, int ld_a,
                                   cudaStream_t st) {
  const int threads = ((dk > dv ? dk : dv) + 31) / 32 * 32;
  if (threads > 256 || Hv % Hqk != 0 || Kc < 1) return cudaErrorInvalidValue;
  gdn_decode_kernel<<<B * Hqk, threads, (2 * dk + 8) * sizeof(float), st>>>(mixed, z, bproj, aproj, conv_state, conv_w,
                                                                          A_log, dt_bias, norm_w, state, out, Hqk, Hv,
                                                                          dk, dv, Kc, eps, ld_mixed, ld_z, ld_b, ld_a);
  return cudaGetLastError();
}

}  // namespace b200
