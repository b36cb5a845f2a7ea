// Single-token (decode) attention over a dense KV cache laid out as (B, Hkv, max_len, D), split over the keys.
//
// Decode attention is a stream over the cache: every key and value row is read once for the G = H / Hkv query
// heads that share it, and there are at most eight query rows per kv head, far too few for a tensor-core tile. So
// this is a bandwidth kernel: a CTA takes one (key range, kv head, sequence); D/8 lanes share a key row with one
// 16-byte load each, dot it with the G queries held in registers, reduce across those lanes with shuffles and run
// an online softmax per lane group; groups, warps and finally key ranges are merged by their (max, sum) pairs.
// The number of valid keys may come from a device counter, so a CUDA-graph decode loop needs no host value.
//
// Replaces the dense masked attention over the whole cache buffer of the reference's cached paths
// (jax_gpt/models/qwen35/gqa.py:88-119, jax_gpt/models/gpt2/model.py:159-176).
#include "attention_sm100.cuh"

#include "common.cuh"

namespace b200 {

namespace {

constexpr int kDecWarps = 4;

struct DecArgs {
  const __nv_bfloat16* q;   // [B, H*D], row stride ldq
  int64_t ldq;
  const __nv_bfloat16* k;   // cache (B, Hkv, max_len, D): strides in elements
  const __nv_bfloat16* v;
  int64_t kv_stride_b, kv_stride_h, kv_stride_t;
  const int* pos_ptr;       // device: number of valid keys = pos_ptr[0] + len_add (nullptr: len)
  int len, len_add;
  int H, Hkv;
  float scale_log2;
  float* part_o;            // [B, H, n_splits, D] un-normalised partial outputs
  float* part_ml;           // [B, H, n_splits, 2] (running max in log2 units, sum)
  // paged cache (table != nullptr): k / v point at the K and V halves of a page pool [n_pages, page_size, width];
  // key t of sequence seq_ids[b] sits in row table[seq, t / page_size] * page_size + t % page_size, kv_stride_t is the
  // pool's row width, the number of valid keys is lens[seq] + len_add
  const int* table;
  const int* seq_ids;
  const int* lens;
  int page_size, max_pages;
};

template <int D, int G>
__global__ void __launch_bounds__(kDecWarps * 32)
attn_decode_split_kernel(const DecArgs a) {
  constexpr int LPK = D / 8;          // lanes that share one key row
  constexpr int KPW = 32 / LPK;       // keys per warp step
  constexpr int KPS = KPW * kDecWarps;
  __shared__ float sm_o[kDecWarps][G][D];
  __shared__ float sm_m[kDecWarps][G], sm_l[kDecWarps][G];
  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int n_splits = gridDim.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % LPK, grp = lane / LPK;
  const int seq = a.table != nullptr ? a.seq_ids[b] : b;
  const int len = a.table != nullptr ? a.lens[seq] + a.len_add : (a.pos_ptr != nullptr ? a.pos_ptr[0] + a.len_add : a.len);
  const int* pages = a.table != nullptr ? a.table + static_cast<int64_t>(seq) * a.max_pages : nullptr;
  // cache row of key t: the key index itself for a dense cache, page * page_size + offset for a paged one
  auto key_row = [&](int t) -> int64_t {
    if (pages == nullptr) return t;
    return static_cast<int64_t>(pages[t / a.page_size]) * a.page_size + t % a.page_size;
  };
  const int per = ((len + n_splits - 1) / n_splits + KPS - 1) / KPS * KPS;
  const int k0 = split * per, k1 = min(len, k0 + per);

  float qf[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const uint4 u = *reinterpret_cast<const uint4*>(a.q + static_cast<int64_t>(b) * a.ldq + (hkv * G + g) * D + sub * 8);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf16x2(w[e]);
      qf[g][2 * e] = f.x * a.scale_log2;
      qf[g][2 * e + 1] = f.y * a.scale_log2;
    }
  }
  float m[G], l[G], o[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) o[g][e] = 0.f;
  }
  const __nv_bfloat16* kb = a.k + b * a.kv_stride_b + hkv * a.kv_stride_h + sub * 8;
  const __nv_bfloat16* vb = a.v + b * a.kv_stride_b + hkv * a.kv_stride_h + sub * 8;
  // Two keys per lane group in flight. The trip count is uniform over the warp (the shuffles below need every
  // lane); a lane group whose key is past the range loads nothing and skips the update.
  for (int base = k0 + warp * KPW; base < k1; base += 2 * KPS) {
    const int ka = base + grp, kc = ka + KPS;
    const bool has_a = ka < k1, has_c = kc < k1;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const int64_t ra = has_a ? key_row(ka) * a.kv_stride_t : 0, rc = has_c ? key_row(kc) * a.kv_stride_t : 0;
    const uint4 kua = has_a ? *reinterpret_cast<const uint4*>(kb + ra) : zero;
    const uint4 vua = has_a ? *reinterpret_cast<const uint4*>(vb + ra) : zero;
    const uint4 kuc = has_c ? *reinterpret_cast<const uint4*>(kb + rc) : zero;
    const uint4 vuc = has_c ? *reinterpret_cast<const uint4*>(vb + rc) : zero;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      const uint4 ku = which == 0 ? kua : kuc;
      const uint4 vu = which == 0 ? vua : vuc;
      const bool valid = which == 0 ? has_a : has_c;
      const uint32_t kw[4] = {ku.x, ku.y, ku.z, ku.w}, vw[4] = {vu.x, vu.y, vu.z, vu.w};
      float kf[8], vf[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf16x2(kw[e]), h = unpack_bf16x2(vw[e]);
        kf[2 * e] = f.x;
        kf[2 * e + 1] = f.y;
        vf[2 * e] = h.x;
        vf[2 * e + 1] = h.y;
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) s = fmaf(qf[g][e], kf[e], s);
#pragma unroll
        for (int off = LPK / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (valid) {
          const float mn = fmaxf(m[g], s);
          const float alpha = exp2f(m[g] - mn), p = exp2f(s - mn);
          l[g] = fmaf(l[g], alpha, p);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[g][e] = fmaf(o[g][e], alpha, p * vf[e]);
          m[g] = mn;
        }
      }
    }
  }
  // merge the lane groups of a warp (same columns, different keys)
#pragma unroll
  for (int off = LPK; off < 32; off <<= 1) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[g], off);
      const float lo = __shfl_xor_sync(0xffffffffu, l[g], off);
      const float mn = fmaxf(m[g], mo);
      const float wa = (m[g] == -INFINITY) ? 0.f : exp2f(m[g] - mn);
      const float wb = (mo == -INFINITY) ? 0.f : exp2f(mo - mn);
      l[g] = l[g] * wa + lo * wb;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float oo = __shfl_xor_sync(0xffffffffu, o[g][e], off);
        o[g][e] = o[g][e] * wa + oo * wb;
      }
      m[g] = mn;
    }
  }
  if (grp == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int e = 0; e < 8; ++e) sm_o[warp][g][sub * 8 + e] = o[g][e];
      if (sub == 0) {
        sm_m[warp][g] = m[g];
        sm_l[warp][g] = l[g];
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += kDecWarps * 32) {
    const int g = i / D, c = i % D;
    float mn = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) mn = fmaxf(mn, sm_m[w][g]);
    float acc = 0.f, ls = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float wt = (sm_m[w][g] == -INFINITY) ? 0.f : exp2f(sm_m[w][g] - mn);
      acc = fmaf(sm_o[w][g][c], wt, acc);
      ls = fmaf(sm_l[w][g], wt, ls);
    }
    const int64_t row = (static_cast<int64_t>(b) * a.H + hkv * G + g) * n_splits + split;
    a.part_o[row * D + c] = acc;
    if (c == 0) {
      a.part_ml[row * 2] = mn;
      a.part_ml[row * 2 + 1] = ls;
    }
  }
}

// out[b, h, :] = sum_s part_o[s] 2^(m_s - M) / sum_s l_s 2^(m_s - M); one CTA per (head, sequence), D threads.
template <int D>
__global__ void attn_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         int n_splits, __nv_bfloat16* __restrict__ out, int64_t ldo, int H) {
  const int h = blockIdx.x, b = blockIdx.y, c = threadIdx.x;
  const int64_t row0 = (static_cast<int64_t>(b) * H + h) * n_splits;
  float mn = -INFINITY;
  for (int s = 0; s < n_splits; ++s) mn = fmaxf(mn, part_ml[(row0 + s) * 2]);
  float acc = 0.f, ls = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = part_ml[(row0 + s) * 2];
    const float wt = (ms == -INFINITY) ? 0.f : exp2f(ms - mn);
    acc = fmaf(part_o[(row0 + s) * D + c], wt, acc);
    ls = fmaf(part_ml[(row0 + s) * 2 + 1], wt, ls);
  }
  out[static_cast<int64_t>(b) * ldo + h * D + c] = __float2bfloat16(ls > 0.f ? acc / ls : 0.f);
}

template <int D, int G>
cudaError_t decode_launch(const DecArgs& a, int B, int n_splits, __nv_bfloat16* out, int64_t ldo,
                          cudaStream_t stream) {
  dim3 grid(n_splits, a.Hkv, B);
  attn_decode_split_kernel<D, G><<<grid, kDecWarps * 32, 0, stream>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  attn_decode_merge_kernel<D><<<dim3(a.H, B), D, 0, stream>>>(a.part_o, a.part_ml, n_splits, out, ldo, a.H);
  return cudaGetLastError();
}

template <int D>
cudaError_t decode_dispatch_g(const DecArgs& a, int B, int n_splits, __nv_bfloat16* out, int64_t ldo,
                              cudaStream_t stream) {
  switch (a.H / a.Hkv) {
    case 1: return decode_launch<D, 1>(a, B, n_splits, out, ldo, stream);
    case 2: return decode_launch<D, 2>(a, B, n_splits, out, ldo, stream);
    case 4: return decode_launch<D, 4>(a, B, n_splits, out, ldo, stream);
    case 8: return decode_launch<D, 8>(a, B, n_splits, out, ldo, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

cudaError_t launch_attn_decode(const __nv_bfloat16* q, int64_t ldq, const __nv_bfloat16* k, const __nv_bfloat16* v,
                               int64_t kv_stride_b, int64_t kv_stride_h, int64_t kv_stride_t, const int* pos_ptr,
                               int len, int len_add, int B, int H, int Hkv, int D, float scale, int n_splits,
                               float* part_o, float* part_ml, __nv_bfloat16* out, int64_t ldo, cudaStream_t stream) {
  if (H % Hkv != 0 || n_splits < 1 || kv_stride_t % 8 != 0 || kv_stride_h % 8 != 0 || kv_stride_b % 8 != 0 ||
      ldq % 8 != 0)
    return cudaErrorInvalidValue;
  DecArgs a{q, ldq, k, v, kv_stride_b, kv_stride_h, kv_stride_t, pos_ptr, len, len_add, H, Hkv,
            scale * 1.4426950408889634f, part_o, part_ml, nullptr, nullptr, nullptr, 0, 0};
  switch (D) {
    case 64: return decode_dispatch_g<64>(a, B, n_splits, out, ldo, stream);
    case 128: return decode_dispatch_g<128>(a, B, n_splits, out, ldo, stream);
    case 256: return decode_dispatch_g<256>(a, B, n_splits, out, ldo, stream);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_attn_decode_paged(const __nv_bfloat16* q, int64_t ldq, const __nv_bfloat16* pool, int width,
                                     const int* block_table, const int* seq_ids, const int* seq_lens, int len_add,
                                     int page_size, int max_pages, int B, int H, int Hkv, int D, float scale, int n_splits,
                                     float* part_o, float* part_ml, __nv_bfloat16* out, int64_t ldo, cudaStream_t stream) {
  if (H % Hkv != 0 || n_splits < 1 || width != 2 * Hkv * D || width % 8 != 0 || ldq % 8 != 0 || page_size < 1)
    return cudaErrorInvalidValue;
  // a pool row holds K of every kv head, then V of every kv head
  DecArgs a{q, ldq, pool, pool + Hkv * D, 0, D, width, nullptr, 0, len_add, H, Hkv,
            scale * 1.4426950408889634f, part_o, part_ml, block_table, seq_ids, seq_lens, page_size, max_pages};
  switch (D) {
    case 64: return decode_dispatch_g<64>(a, B, n_splits, out, ldo, stream);
    case 128: return decode_dispatch_g<128>(a, B, n_splits, out, ldo, stream);
    case 256: return decode_dispatch_g<256>(a, B, n_splits, out, ldo, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace b200
