// Gated-DeltaNet prefill: everything of the chunked gated delta rule that does NOT depend on the running state,
// forward and backward, as one kernel each (fp32 on the CUDA cores, no library call).
//
// Per chunk of 64 tokens and per value head the chunked algorithm needs (jax_gpt/models/qwen35/deltanet.py:214-300,
// which computes them with batched einsums and a triangular solve):
//     beta = sigmoid(b)            g = -exp(A_log) softplus(a + dt_bias)        G = cumsum(g) inside the chunk
//     q^ = l2norm(q) dk^-1/2       k^ = l2norm(k)
//     A     = strict_lower(beta_i (k^_i . k^_j) exp(G_i - G_j))
//     X     = (I + A)^-1 [beta v | beta exp(G) k^]            ->  v_eff (64 x 128), k_cum (64 x 128)
//     intra = lower(q^_i . k^_j exp(G_i - G_j))               k_dec = k^ exp(G_end - G)      q_e = q^ exp(G)
// and the inter-chunk scan (gdn_kernels.cu) consumes [k_cum ; q_e], intra, k_dec, v_eff, exp(G_end).
//
// One CTA of 256 threads owns one (batch, q/k head, chunk) and loops over the value heads that share the q/k head:
// the normalised q and k tiles stay in shared memory as fp32, the 64 x 64 Gram matrices are computed by a 16 x 16
// thread grid (4 x 4 interleaved entries each), and the unit-lower-triangular solve is a forward substitution with
// one right-hand-side COLUMN per thread held in 64 registers (256 columns = 256 threads), so it needs no barriers.
//
// The backward kernel recomputes the forward quantities from the same inputs, solves the transposed system
// Y = (I + A)^-T dX by backward substitution (again one column per thread), forms dA = -strict_lower(Y X^T), and
// pushes the gradients through the decays, the gates, the Gram matrices and the two L2 norms down to d(mixed),
// d(b), d(a), d(A_log) and d(dt_bias). Gradients of q and k are summed over the value heads on chip, so the kernel
// has no global atomics except the two per-head scalars. Those 2 x 64 x 128 fp32 sums are thread-private (64 values
// per thread) but must survive the substitution phases, which need every register for the 64-entry columns; shared
// memory is full, so they are parked in tensor memory (tcgen05.st / tcgen05.ld, 128 columns) between the phases.
#include "seq_kernels.cuh"

#include "common.cuh"

namespace b200 {

namespace {

constexpr int kC = 64;            // chunk length
constexpr int kD = 128;           // dk = dv
constexpr int kLd = kD + 4;       // row stride (floats) of the 64 x 128 fp32 tiles in shared memory
constexpr int kThreads = 256;
constexpr float kQScale = 0.08838834764831845f;   // 128^-1/2

struct PrepGeom {
  int T, N, Hqk, Hv, conv_dim;
};

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float bf2f(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ float2 bf2f2(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ float dot4(const float4& a, const float4& b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }

// Loads the chunk's q and k rows (bf16, 128 wide each) as fp32 into sq / sk, L2-normalises every row (q is also
// scaled by dk^-1/2) and leaves the reciprocal norms in s_rq / s_rk. Rows at or beyond T become zero.
__device__ void load_qk_normalised(const __nv_bfloat16* mixed_b, const PrepGeom& gm, int n, int hq, float* sq, float* sk,
                                   float* s_rq, float* s_rk) {
  const int tid = threadIdx.x;
  for (int idx = tid; idx < 2 * kC * 16; idx += kThreads) {
    const int which = idx / (kC * 16), rem = idx % (kC * 16);
    const int i = rem / 16, v8 = rem % 16;
    const int t = n * kC + i;
    float* dst = (which ? sk : sq) + i * kLd + v8 * 8;
    if (t < gm.T) {
      const uint4 raw = *reinterpret_cast<const uint4*>(mixed_b + static_cast<size_t>(t) * gm.conv_dim +
                                                        which * gm.Hqk * kD + hq * kD + v8 * 8);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(p[e]);
        dst[2 * e] = f.x;
        dst[2 * e + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) dst[e] = 0.f;
    }
  }
  __syncthreads();
  const int i = tid >> 2, qd = tid & 3;
  float ssq = 0.f, ssk = 0.f;
#pragma unroll
  for (int m = 0; m < 16; ++m) {
    const float2 a = *reinterpret_cast<const float2*>(sq + i * kLd + 2 * (qd + 4 * m));
    const float2 b = *reinterpret_cast<const float2*>(sk + i * kLd + 2 * (qd + 4 * m));
    ssq += a.x * a.x + a.y * a.y;
    ssk += b.x * b.x + b.y * b.y;
  }
  ssq += __shfl_xor_sync(0xffffffffu, ssq, 1);
  ssq += __shfl_xor_sync(0xffffffffu, ssq, 2);
  ssk += __shfl_xor_sync(0xffffffffu, ssk, 1);
  ssk += __shfl_xor_sync(0xffffffffu, ssk, 2);
  const float rq = rsqrtf(ssq + 1e-6f), rk = rsqrtf(ssk + 1e-6f);
#pragma unroll
  for (int m = 0; m < 16; ++m) {
    float2* a = reinterpret_cast<float2*>(sq + i * kLd + 2 * (qd + 4 * m));
    float2* b = reinterpret_cast<float2*>(sk + i * kLd + 2 * (qd + 4 * m));
    a->x *= rq * kQScale;
    a->y *= rq * kQScale;
    b->x *= rk;
    b->y *= rk;
  }
  if (qd == 0) {
    s_rq[i] = rq;
    s_rk[i] = rk;
  }
  __syncthreads();
}

// Thread (ti, tj) of the 16 x 16 grid owns entries (ti + 16 a, tj + 16 b): s = k^ k^T, w = q^ k^T. Entries above
// the diagonal are never used, so block columns b > a are skipped.
__device__ __forceinline__ void gram_blocks(const float* sq, const float* sk, int ti, int tj, float (&s)[4][4],
                                            float (&w)[4][4]) {
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) s[a][b] = w[a][b] = 0.f;
#pragma unroll 2
  for (int c = 0; c < kD; c += 4) {
    float4 ki[4], qi[4], kj[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      ki[a] = *reinterpret_cast<const float4*>(sk + (ti + 16 * a) * kLd + c);
      qi[a] = *reinterpret_cast<const float4*>(sq + (ti + 16 * a) * kLd + c);
      kj[a] = *reinterpret_cast<const float4*>(sk + (tj + 16 * a) * kLd + c);
    }
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b)
        if (b <= a) {
          s[a][b] += dot4(ki[a], kj[b]);
          w[a][b] += dot4(qi[a], kj[b]);
        }
  }
}

// Gates of one value head for the 64 rows of the chunk (threads 0..63 compute, everybody leaves synchronised):
// s_beta, s_g (raw log-decay), s_G (inclusive cumulative sum), s_eg = exp(G), s_ed = exp(G_end - G), s_asig =
// sigmoid(a + dt_bias) (the derivative of the softplus). Rows at or beyond T have beta = g = 0.
__device__ void chunk_gates(const __nv_bfloat16* b_in, const __nv_bfloat16* a_in, float a_neg, float dtb,
                            const PrepGeom& gm, int batch, int n, int hv, float* s_beta, float* s_g, float* s_G,
                            float* s_eg, float* s_ed, float* s_asig) {
  const int tid = threadIdx.x;
  if (tid < kC) {
    const int t = n * kC + tid;
    float beta = 0.f, g = 0.f, asig = 0.f;
    if (t < gm.T) {
      const size_t off = (static_cast<size_t>(batch) * gm.T + t) * gm.Hv + hv;
      beta = sigmoid_f(bf2f(b_in + off));
      const float x = bf2f(a_in + off) + dtb;
      g = a_neg * softplus_f(x);
      asig = sigmoid_f(x);
    }
    s_beta[tid] = beta;
    s_g[tid] = g;
    s_asig[tid] = asig;
  }
  __syncthreads();
  if (tid < kC) {
    float G = 0.f;
    for (int j = 0; j <= tid; ++j) G += s_g[j];
    s_G[tid] = G;
  }
  __syncthreads();
  if (tid < kC) {
    s_eg[tid] = expf(s_G[tid]);
    s_ed[tid] = expf(s_G[kC - 1] - s_G[tid]);
  }
  __syncthreads();
}

struct PrepFwdArgs {
  const __nv_bfloat16* mixed;   // [B, T, conv_dim]: q | k | v after conv + SiLU
  const __nv_bfloat16* b_in;    // [B, T, Hv]
  const __nv_bfloat16* a_in;    // [B, T, Hv]
  const float* A_log;           // [Hv]
  const float* dt_bias;         // [Hv]
  __nv_bfloat16* kq;            // [B*Hv, N, 128, 128]
  __nv_bfloat16* intra;         // [B*Hv, N, 64, 64]
  __nv_bfloat16* kdec;          // [B*Hv, N, 64, 128]
  __nv_bfloat16* veff;          // [B*Hv, N, 64, 128]
  float* e;                     // [B*Hv, N]
  PrepGeom gm;
};

constexpr int kFwdSmemFloats = 2 * kC * kLd + kC * kC + 8 * kC;

__global__ void __launch_bounds__(kThreads) gdn_chunk_prep_fwd_kernel(const PrepFwdArgs p) {
  extern __shared__ __align__(16) float smem[];
  float* sq = smem;
  float* sk = sq + kC * kLd;
  float* sA = sk + kC * kLd;
  float* s_beta = sA + kC * kC;
  float* s_g = s_beta + kC;
  float* s_G = s_g + kC;
  float* s_eg = s_G + kC;
  float* s_ed = s_eg + kC;
  float* s_asig = s_ed + kC;
  float* s_rq = s_asig + kC;
  float* s_rk = s_rq + kC;
  const PrepGeom gm = p.gm;
  const int tid = threadIdx.x, n = blockIdx.x, hq = blockIdx.y, batch = blockIdx.z;
  const int rep = gm.Hv / gm.Hqk;
  const __nv_bfloat16* mixed_b = p.mixed + static_cast<size_t>(batch) * gm.T * gm.conv_dim;
  load_qk_normalised(mixed_b, gm, n, hq, sq, sk, s_rq, s_rk);
  const int ti = tid >> 4, tj = tid & 15;
  float s[4][4], w[4][4];
  gram_blocks(sq, sk, ti, tj, s, w);
  for (int r = 0; r < rep; ++r) {
    const int hv = hq * rep + r;
    const size_t chunk = (static_cast<size_t>(batch) * gm.Hv + hv) * gm.N + n;
    chunk_gates(p.b_in, p.a_in, -expf(p.A_log[hv]), p.dt_bias[hv], gm, batch, n, hv, s_beta, s_g, s_G, s_eg, s_ed, s_asig);
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int i = ti + 16 * a, j = tj + 16 * b;
        const float D = j <= i ? expf(s_G[i] - s_G[j]) : 0.f;
        sA[i * kC + j] = j < i ? s_beta[i] * s[a][b] * D : 0.f;
        p.intra[(chunk * kC + i) * kC + j] = __float2bfloat16(j <= i ? w[a][b] * D : 0.f);
      }
    __syncthreads();
    {
      // forward substitution, one column of [beta v | beta exp(G) k^] per thread
      const int c = tid & 127;
      const bool vhalf = tid < 128;
      float x[kC];
      if (vhalf) {
        const __nv_bfloat16* vp = mixed_b + 2 * gm.Hqk * kD + hv * kD + c;
#pragma unroll
        for (int i = 0; i < kC; ++i) {
          const int t = n * kC + i;
          x[i] = t < gm.T ? s_beta[i] * bf2f(vp + static_cast<size_t>(t) * gm.conv_dim) : 0.f;
        }
      } else {
#pragma unroll
        for (int i = 0; i < kC; ++i) x[i] = s_beta[i] * s_eg[i] * sk[i * kLd + c];
      }
#pragma unroll
      for (int i = 1; i < kC; ++i) {
        float acc = 0.f;
#pragma unroll
        for (int j4 = 0; j4 * 4 < i; ++j4) {
          const float4 m = *reinterpret_cast<const float4*>(sA + i * kC + 4 * j4);   // entries at or right of the diagonal are 0
          acc += m.x * x[4 * j4] + m.y * x[4 * j4 + 1] + m.z * x[4 * j4 + 2] + m.w * x[4 * j4 + 3];
        }
        x[i] -= acc;
      }
      __nv_bfloat16* out = vhalf ? p.veff + chunk * kC * kD + c : p.kq + chunk * 2 * kC * kD + c;
#pragma unroll
      for (int i = 0; i < kC; ++i) out[i * kD] = __float2bfloat16(x[i]);
    }
    for (int idx = tid; idx < kC * (kD / 2); idx += kThreads) {
      const int i = idx >> 6, c2 = idx & 63;
      const float2 q2 = *reinterpret_cast<const float2*>(sq + i * kLd + 2 * c2);
      const float2 k2 = *reinterpret_cast<const float2*>(sk + i * kLd + 2 * c2);
      const float eg = s_eg[i], ed = s_ed[i];
      *reinterpret_cast<__nv_bfloat162*>(p.kq + (chunk * 2 * kC + kC + i) * kD + 2 * c2) =
          __floats2bfloat162_rn(q2.x * eg, q2.y * eg);
      *reinterpret_cast<__nv_bfloat162*>(p.kdec + (chunk * kC + i) * kD + 2 * c2) =
          __floats2bfloat162_rn(k2.x * ed, k2.y * ed);
    }
    if (tid == 0) p.e[chunk] = s_eg[kC - 1];
    __syncthreads();
  }
}

struct PrepBwdArgs {
  const __nv_bfloat16* mixed;
  const __nv_bfloat16* b_in;
  const __nv_bfloat16* a_in;
  const float* A_log;
  const float* dt_bias;
  const __nv_bfloat16* d_kq;      // [B*Hv, N, 128, 128]: rows 0-63 d k_cum, rows 64-127 d q_e
  const __nv_bfloat16* d_intra;   // [B*Hv, N, 64, 64]
  const __nv_bfloat16* d_kdec;    // [B*Hv, N, 64, 128]
  const __nv_bfloat16* d_veff;    // [B*Hv, N, 64, 128]
  const float* d_e;               // [B*Hv, N]
  __nv_bfloat16* d_mixed;         // [B, T, conv_dim]
  float* d_b;                     // [B, T, Hv]
  float* d_a;                     // [B, T, Hv]
  float* d_A_log;                 // [Hv], accumulated
  float* d_dt_bias;               // [Hv], accumulated
  PrepGeom gm;
};

constexpr int kBwdSmemFloats = 4 * kC * kLd + 3 * kC * kC + 10 * kC + 4;

__global__ void __launch_bounds__(kThreads, 1) gdn_chunk_prep_bwd_kernel(const PrepBwdArgs p) {
  extern __shared__ __align__(16) float smem[];
  float* sq = smem;
  float* sk = sq + kC * kLd;
  float* sX = sk + kC * kLd;
  float* sY = sX + kC * kLd;
  float* sM0 = sY + kC * kLd;        // k^ k^T * decay (strict lower), later dS + dS^T
  float* sM1 = sM0 + kC * kC;        // q^ k^T * decay (lower), later dW
  float* sM2 = sM1 + kC * kC;        // dW^T
  float* s_beta = sM2 + kC * kC;
  float* s_g = s_beta + kC;
  float* s_G = s_g + kC;
  float* s_eg = s_G + kC;
  float* s_ed = s_eg + kC;
  float* s_asig = s_ed + kC;
  float* s_rq = s_asig + kC;
  float* s_rk = s_rq + kC;
  float* s_dG = s_rk + kC;
  float* s_dbeta = s_dG + kC;
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(s_dbeta + kC);
  const PrepGeom gm = p.gm;
  const int tid = threadIdx.x, n = blockIdx.x, hq = blockIdx.y, batch = blockIdx.z;
  const int rep = gm.Hv / gm.Hqk;
  const size_t tok0 = static_cast<size_t>(batch) * gm.T;
  const __nv_bfloat16* mixed_b = p.mixed + tok0 * gm.conv_dim;
  __nv_bfloat16* d_mixed_b = p.d_mixed + tok0 * gm.conv_dim;
  load_qk_normalised(mixed_b, gm, n, hq, sq, sk, s_rq, s_rk);
  const int ti = tid >> 4, tj = tid & 15;     // Gram-matrix mapping
  const int ri = tid >> 2, rqd = tid & 3;     // row mapping: row ri, column pairs rqd + 4 m
  const int cc = tid & 127, hb = tid >> 7;    // column mapping: column cc, rows 2 m + hb
  // gradients of the scaled q^ and of k^, summed over the value heads: parked in tensor memory, this thread's lane
  // (warp % 4 selects the lane quadrant) and 64 columns (dq: 0-31, dk: 32-63 of the warp's column group)
  if (tid < 32) {
    tmem_alloc(s_tmem, 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t park = *s_tmem + ((static_cast<uint32_t>((tid >> 5) & 3) * 32u) << 16) + static_cast<uint32_t>(tid >> 7) * 64u;
  {
    uint32_t z[32];
#pragma unroll
    for (int m = 0; m < 32; ++m) z[m] = 0u;
    tmem_st_32x32(park, z);
    tmem_st_32x32(park + 32, z);
    tmem_st_wait();
  }

  for (int r = 0; r < rep; ++r) {
    const int hv = hq * rep + r;
    const size_t chunk = (static_cast<size_t>(batch) * gm.Hv + hv) * gm.N + n;
    const float a_neg = -expf(p.A_log[hv]);
    chunk_gates(p.b_in, p.a_in, a_neg, p.dt_bias[hv], gm, batch, n, hv, s_beta, s_g, s_G, s_eg, s_ed, s_asig);
    if (tid < kC) s_dG[tid] = s_dbeta[tid] = 0.f;
    {
      float s[4][4], w[4][4];
      gram_blocks(sq, sk, ti, tj, s, w);
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int i = ti + 16 * a, j = tj + 16 * b;
          const float D = j <= i ? expf(s_G[i] - s_G[j]) : 0.f;
          sM0[i * kC + j] = j < i ? s[a][b] * D : 0.f;
          sM1[i * kC + j] = j <= i ? w[a][b] * D : 0.f;
        }
    }
    __syncthreads();

    float da[4][4];                            // dA of this thread's Gram entries
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) da[a][b] = 0.f;

#pragma unroll 1
    for (int h = 0; h < 2; ++h) {              // h = 0: the value columns, h = 1: the key columns of the solve
      // The two substitutions of a pass are independent (X needs the right-hand side, Y the incoming gradient):
      // threads 0-127 solve the columns of X while threads 128-255 solve the columns of Y.
      if (tid < 128) {
        const int c = tid;
        float x[kC];
        if (h == 0) {
          const __nv_bfloat16* vp = mixed_b + 2 * gm.Hqk * kD + hv * kD + c;
#pragma unroll
          for (int i = 0; i < kC; ++i) {
            const int t = n * kC + i;
            x[i] = t < gm.T ? s_beta[i] * bf2f(vp + static_cast<size_t>(t) * gm.conv_dim) : 0.f;
          }
        } else {
#pragma unroll
          for (int i = 0; i < kC; ++i) x[i] = s_beta[i] * s_eg[i] * sk[i * kLd + c];
        }
        // X = (I + A)^-1 R with A_ij = beta_i M0_ij
#pragma unroll
        for (int i = 1; i < kC; ++i) {
          float acc = 0.f;
#pragma unroll
          for (int j4 = 0; j4 * 4 < i; ++j4) {
            const float4 m = *reinterpret_cast<const float4*>(sM0 + i * kC + 4 * j4);
            acc += m.x * x[4 * j4] + m.y * x[4 * j4 + 1] + m.z * x[4 * j4 + 2] + m.w * x[4 * j4 + 3];
          }
          x[i] -= s_beta[i] * acc;
        }
#pragma unroll
        for (int i = 0; i < kC; ++i) sX[i * kLd + c] = x[i];
      } else {
        const int c = tid - 128;
        float x[kC];
        // Y = (I + A)^-T dX, right-looking: once y_j is final, y_i -= A_ji y_j for every i < j
        const __nv_bfloat16* dxp = h == 0 ? p.d_veff + chunk * kC * kD + c : p.d_kq + chunk * 2 * kC * kD + c;
#pragma unroll
        for (int i = 0; i < kC; ++i) x[i] = bf2f(dxp + i * kD);
#pragma unroll
        for (int j = kC - 1; j >= 1; --j) {
          const float t = s_beta[j] * x[j];
#pragma unroll
          for (int i4 = 0; i4 * 4 < j; ++i4) {
            const float4 m = *reinterpret_cast<const float4*>(sM0 + j * kC + 4 * i4);
            x[4 * i4] -= m.x * t;
            x[4 * i4 + 1] -= m.y * t;
            x[4 * i4 + 2] -= m.z * t;
            x[4 * i4 + 3] -= m.w * t;
          }
        }
#pragma unroll
        for (int i = 0; i < kC; ++i) sY[i * kLd + c] = x[i];
        if (h == 0) {
          __nv_bfloat16* dvp = d_mixed_b + 2 * gm.Hqk * kD + hv * kD + c;
#pragma unroll
          for (int i = 0; i < kC; ++i) {
            const int t = n * kC + i;
            if (t < gm.T) dvp[static_cast<size_t>(t) * gm.conv_dim] = __float2bfloat16(s_beta[i] * x[i]);
          }
        }
      }
      __syncthreads();
      // dA -= Y X^T on this thread's entries
#pragma unroll 2
      for (int c = 0; c < kD; c += 4) {
        float4 yi[4], xj[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          yi[a] = *reinterpret_cast<const float4*>(sY + (ti + 16 * a) * kLd + c);
          xj[a] = *reinterpret_cast<const float4*>(sX + (tj + 16 * a) * kLd + c);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int b = 0; b < 4; ++b)
            if (b <= a) da[a][b] -= dot4(yi[a], xj[b]);
      }
      // per-row dot products of Y with the right-hand side's own factor (v, or k^)
      {
        float u = 0.f;
        const int t = n * kC + ri;
        if (h == 0) {
          if (t < gm.T) {
            const __nv_bfloat16* vp = mixed_b + static_cast<size_t>(t) * gm.conv_dim + 2 * gm.Hqk * kD + hv * kD;
#pragma unroll
            for (int m = 0; m < 16; ++m) {
              const float2 y2 = *reinterpret_cast<const float2*>(sY + ri * kLd + 2 * (rqd + 4 * m));
              const float2 v2 = bf2f2(vp + 2 * (rqd + 4 * m));
              u += y2.x * v2.x + y2.y * v2.y;
            }
          }
        } else {
#pragma unroll
          for (int m = 0; m < 16; ++m) {
            const float2 y2 = *reinterpret_cast<const float2*>(sY + ri * kLd + 2 * (rqd + 4 * m));
            const float2 k2 = *reinterpret_cast<const float2*>(sk + ri * kLd + 2 * (rqd + 4 * m));
            u += y2.x * k2.x + y2.y * k2.y;
          }
        }
        u += __shfl_xor_sync(0xffffffffu, u, 1);
        u += __shfl_xor_sync(0xffffffffu, u, 2);
        if (rqd == 0) {
          if (h == 0) {
            atomicAdd(s_dbeta + ri, u);
          } else {
            atomicAdd(s_dbeta + ri, s_eg[ri] * u);
            atomicAdd(s_dG + ri, s_beta[ri] * s_eg[ri] * u);
          }
        }
      }
      __syncthreads();
    }

    // through the decayed Gram matrices: E = dA * A + d_intra * intra feeds dG (row sums minus column sums);
    // dS = dA beta D and dW = d_intra D go to q^ and k^ through three 64 x 64 x 128 products
    {
      float m0[4][4], m1[4][4], di[4][4];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int i = ti + 16 * a, j = tj + 16 * b;
          m0[a][b] = sM0[i * kC + j];
          m1[a][b] = sM1[i * kC + j];
          di[a][b] = j <= i ? bf2f(p.d_intra + (chunk * kC + i) * kC + j) : 0.f;
        }
      __syncthreads();      // every entry is in registers before the mirrored writes start
      float row_e[4], row_b[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        row_e[a] = row_b[a] = 0.f;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int i = ti + 16 * a, j = tj + 16 * b;
          if (j > i) continue;               // the mirror entry's owner writes this position
          const float D = expf(s_G[i] - s_G[j]);
          const float dA = j < i ? da[a][b] : 0.f;
          const float E = dA * s_beta[i] * m0[a][b] + di[a][b] * m1[a][b];
          row_e[a] += E;
          atomicAdd(s_dG + j, -E);
          row_b[a] += dA * m0[a][b];
          const float dS = dA * s_beta[i] * D;
          const float dW = di[a][b] * D;
          sM0[i * kC + j] = dS;
          sM0[j * kC + i] = dS;
          sM1[i * kC + j] = dW;
          sM2[j * kC + i] = dW;
          if (j < i) {
            sM1[j * kC + i] = 0.f;
            sM2[i * kC + j] = 0.f;
          }
        }
      }
#pragma unroll
      for (int a = 0; a < 4; ++a) {
#pragma unroll
        for (int o = 8; o >= 1; o >>= 1) {
          row_e[a] += __shfl_xor_sync(0xffffffffu, row_e[a], o);
          row_b[a] += __shfl_xor_sync(0xffffffffu, row_b[a], o);
        }
        if (tj == 0) {
          atomicAdd(s_dG + ti + 16 * a, row_e[a]);
          atomicAdd(s_dbeta + ti + 16 * a, row_b[a]);
        }
      }
    }
    __syncthreads();
    float dq[32], dk[32];
    {
      uint32_t v[32];
      tmem_ld_32x32(park, v);
      tmem_ld_wait();
#pragma unroll
      for (int m = 0; m < 32; ++m) dq[m] = __uint_as_float(v[m]);
      tmem_ld_32x32(park + 32, v);
      tmem_ld_wait();
#pragma unroll
      for (int m = 0; m < 32; ++m) {
        const int i = 2 * m + hb;
        dk[m] = __uint_as_float(v[m]) + s_beta[i] * s_eg[i] * sY[i * kLd + cc];   // sY: the key half of Y
      }
    }
    {
      float col[kC];
#pragma unroll
      for (int j = 0; j < kC; ++j) col[j] = sk[j * kLd + cc];
#pragma unroll
      for (int m = 0; m < 32; ++m) {
        const int i = 2 * m + hb;
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int j4 = 0; j4 < 16; ++j4) {
          const float4 s4 = *reinterpret_cast<const float4*>(sM0 + i * kC + 4 * j4);
          const float4 w4 = *reinterpret_cast<const float4*>(sM1 + i * kC + 4 * j4);
          a0 += s4.x * col[4 * j4] + s4.y * col[4 * j4 + 1] + s4.z * col[4 * j4 + 2] + s4.w * col[4 * j4 + 3];
          a1 += w4.x * col[4 * j4] + w4.y * col[4 * j4 + 1] + w4.z * col[4 * j4 + 2] + w4.w * col[4 * j4 + 3];
        }
        dk[m] += a0;
        dq[m] += a1;
      }
#pragma unroll
      for (int j = 0; j < kC; ++j) col[j] = sq[j * kLd + cc];
#pragma unroll
      for (int m = 0; m < 32; ++m) {
        const int i = 2 * m + hb;
        float a0 = 0.f;
#pragma unroll
        for (int j4 = 0; j4 < 16; ++j4) {
          const float4 t4 = *reinterpret_cast<const float4*>(sM2 + i * kC + 4 * j4);
          a0 += t4.x * col[4 * j4] + t4.y * col[4 * j4 + 1] + t4.z * col[4 * j4 + 2] + t4.w * col[4 * j4 + 3];
        }
        dk[m] += a0;
      }
    }
    // q_e = q^ exp(G), k_dec = k^ exp(G_end - G), e = exp(G_end)
    {
      const __nv_bfloat16* dqe = p.d_kq + (chunk * 2 * kC + kC) * kD;
      const __nv_bfloat16* dkd = p.d_kdec + chunk * kC * kD;
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int m = 0; m < 16; ++m) {
        const int c2 = 2 * (rqd + 4 * m);
        const float2 g1 = bf2f2(dqe + ri * kD + c2), g2 = bf2f2(dkd + ri * kD + c2);
        const float2 q2 = *reinterpret_cast<const float2*>(sq + ri * kLd + c2);
        const float2 k2 = *reinterpret_cast<const float2*>(sk + ri * kLd + c2);
        s1 += g1.x * q2.x + g1.y * q2.y;
        s2 += g2.x * k2.x + g2.y * k2.y;
      }
      s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
      s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
      s2 += __shfl_xor_sync(0xffffffffu, s2, 1);
      s2 += __shfl_xor_sync(0xffffffffu, s2, 2);
      if (rqd == 0) {
        const float t = s_ed[ri] * s2;
        atomicAdd(s_dG + ri, s_eg[ri] * s1 - t);
        atomicAdd(s_dG + kC - 1, t);
      }
      if (tid == 0) atomicAdd(s_dG + kC - 1, p.d_e[chunk] * s_eg[kC - 1]);
#pragma unroll
      for (int m = 0; m < 32; ++m) {
        const int i = 2 * m + hb;
        dq[m] += s_eg[i] * bf2f(dqe + i * kD + cc);
        dk[m] += s_ed[i] * bf2f(dkd + i * kD + cc);
      }
    }
    if (r + 1 < rep) {
      uint32_t v[32];
#pragma unroll
      for (int m = 0; m < 32; ++m) v[m] = __float_as_uint(dq[m]);
      tmem_st_32x32(park, v);
#pragma unroll
      for (int m = 0; m < 32; ++m) v[m] = __float_as_uint(dk[m]);
      tmem_st_32x32(park + 32, v);
      tmem_st_wait();
    } else {
      // last value head: straight to shared memory for the L2-norm backward (sX is free; sY still feeds nothing)
#pragma unroll
      for (int m = 0; m < 32; ++m) sX[(2 * m + hb) * kLd + cc] = dq[m];
      __syncthreads();      // every thread has read the key half of Y out of sY
#pragma unroll
      for (int m = 0; m < 32; ++m) sY[(2 * m + hb) * kLd + cc] = dk[m];
    }
    __syncthreads();
    // gates: dg = reverse cumulative sum of dG; g = -exp(A_log) softplus(a + dt_bias); beta = sigmoid(b)
    if (tid < kC) {
      float dg = 0.f;
      for (int m = tid; m < kC; ++m) dg += s_dG[m];
      const int t = n * kC + tid;
      float d_alog = 0.f, d_dtb = 0.f;
      if (t < gm.T) {
        const size_t off = (tok0 + t) * gm.Hv + hv;
        const float d_a = dg * a_neg * s_asig[tid];
        const float beta = s_beta[tid];
        p.d_a[off] = d_a;
        p.d_b[off] = s_dbeta[tid] * beta * (1.f - beta);
        d_alog = dg * s_g[tid];
        d_dtb = d_a;
      }
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) {
        d_alog += __shfl_xor_sync(0xffffffffu, d_alog, o);
        d_dtb += __shfl_xor_sync(0xffffffffu, d_dtb, o);
      }
      if ((tid & 31) == 0) {
        atomicAdd(p.d_A_log + hv, d_alog);
        atomicAdd(p.d_dt_bias + hv, d_dtb);
      }
    }
    __syncthreads();
  }

  // through the L2 norms: y = x r, r = rsqrt(sum x^2 + eps)  =>  dx = r (dy - y (y . dy))
  {
    float dotq = 0.f, dotk = 0.f;
#pragma unroll
    for (int m = 0; m < 16; ++m) {
      const int c2 = 2 * (rqd + 4 * m);
      const float2 gq = *reinterpret_cast<const float2*>(sX + ri * kLd + c2);
      const float2 gk = *reinterpret_cast<const float2*>(sY + ri * kLd + c2);
      const float2 q2 = *reinterpret_cast<const float2*>(sq + ri * kLd + c2);
      const float2 k2 = *reinterpret_cast<const float2*>(sk + ri * kLd + c2);
      dotq += gq.x * q2.x + gq.y * q2.y;
      dotk += gk.x * k2.x + gk.y * k2.y;
    }
    dotq += __shfl_xor_sync(0xffffffffu, dotq, 1);
    dotq += __shfl_xor_sync(0xffffffffu, dotq, 2);
    dotk += __shfl_xor_sync(0xffffffffu, dotk, 1);
    dotk += __shfl_xor_sync(0xffffffffu, dotk, 2);
    const int t = n * kC + ri;
    if (t < gm.T) {
      const float rq = s_rq[ri], rk = s_rk[ri];
      __nv_bfloat16* oq = d_mixed_b + static_cast<size_t>(t) * gm.conv_dim + hq * kD;
      __nv_bfloat16* ok = oq + gm.Hqk * kD;
      // sq holds q^ s (s = dk^-1/2): d q^ = s dQ, q^ (q^ . d q^) = sq (sq . dQ) / s
#pragma unroll
      for (int m = 0; m < 16; ++m) {
        const int c2 = 2 * (rqd + 4 * m);
        const float2 gq = *reinterpret_cast<const float2*>(sX + ri * kLd + c2);
        const float2 gk = *reinterpret_cast<const float2*>(sY + ri * kLd + c2);
        const float2 q2 = *reinterpret_cast<const float2*>(sq + ri * kLd + c2);
        const float2 k2 = *reinterpret_cast<const float2*>(sk + ri * kLd + c2);
        *reinterpret_cast<__nv_bfloat162*>(oq + c2) = __floats2bfloat162_rn(
            rq * (kQScale * gq.x - q2.x * dotq / kQScale), rq * (kQScale * gq.y - q2.y * dotq / kQScale));
        *reinterpret_cast<__nv_bfloat162*>(ok + c2) =
            __floats2bfloat162_rn(rk * (gk.x - k2.x * dotk), rk * (gk.y - k2.y * dotk));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid < 32) tmem_dealloc(*s_tmem, 128);
}

bool prep_geom_ok(int B, int T, int Hqk, int Hv) { return B >= 1 && T >= 1 && Hqk >= 1 && Hv >= Hqk && Hv % Hqk == 0; }

}  // namespace

cudaError_t launch_gdn_chunk_prep(const __nv_bfloat16* mixed, const __nv_bfloat16* b_in, const __nv_bfloat16* a_in,
                                  const float* A_log, const float* dt_bias, __nv_bfloat16* kq, __nv_bfloat16* intra,
                                  __nv_bfloat16* kdec, __nv_bfloat16* veff, float* e, int B, int T, int Hqk, int Hv,
                                  cudaStream_t stream) {
  if (!prep_geom_ok(B, T, Hqk, Hv)) return cudaErrorInvalidValue;
  const int N = (T + kC - 1) / kC;
  constexpr int smem = kFwdSmemFloats * 4;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(gdn_chunk_prep_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return err;
    configured = true;
  }
  PrepFwdArgs args{mixed, b_in, a_in, A_log, dt_bias, kq, intra, kdec, veff, e, {T, N, Hqk, Hv, (2 * Hqk + Hv) * kD}};
  gdn_chunk_prep_fwd_kernel<<<dim3(N, Hqk, B), kThreads, smem, stream>>>(args);
  return cudaGetLastError();
}

cudaError_t launch_gdn_chunk_prep_bwd(const __nv_bfloat16* mixed, const __nv_bfloat16* b_in, const __nv_bfloat16* a_in,
                                      const float* A_log, const float* dt_bias, const __nv_bfloat16* d_kq,
                                      const __nv_bfloat16* d_intra, const __nv_bfloat16* d_kdec,
                                      const __nv_bfloat16* d_veff, const float* d_e, __nv_bfloat16* d_mixed, float* d_b,
                                      float* d_a, float* d_A_log, float* d_dt_bias, int B, int T, int Hqk, int Hv,
                                      cudaStream_t stream) {
  if (!prep_geom_ok(B, T, Hqk, Hv)) return cudaErrorInvalidValue;
  const int N = (T + kC - 1) / kC;
  constexpr int smem = kBwdSmemFloats * 4;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(gdn_chunk_prep_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return err;
    configured = true;
  }
  PrepBwdArgs args{mixed, b_in, a_in, A_log, dt_bias, d_kq, d_intra, d_kdec, d_veff, d_e,
                   d_mixed, d_b, d_a, d_A_log, d_dt_bias, {T, N, Hqk, Hv, (2 * Hqk + Hv) * kD}};
  gdn_chunk_prep_bwd_kernel<<<dim3(N, Hqk, B), kThreads, smem, stream>>>(args);
  return cudaGetLastError();
}

}  // namespace b200
