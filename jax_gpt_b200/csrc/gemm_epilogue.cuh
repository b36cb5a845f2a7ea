// Epilogue of the tcgen05 GEMM kernels: one 32-column chunk of one accumulator row per thread
// (alpha, bias, GELU / GELU' with the saved pre-activation, residual, then a bf16 / fp32 store or an
// fp32 reduction into a local or peer buffer). Shared by the single-CTA and the CTA-pair kernels.
#pragma once
#include "common.cuh"
#include "gemm_sm100.cuh"

namespace b200 {

// v: the 32 fp32 accumulator values of row `row`, columns [col0, col0 + 32); ks: the tile's K split
// (bias and residual are added by split 0 only).
__device__ __forceinline__ void gemm_epilogue_chunk(const GemmArgs& args, const uint32_t (&v)[32], int row, int col0,
                                                    int ks) {
  float f[32];
  if (args.alpha == 1.f) {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) * args.alpha;
  }
  const bool full = (col0 + 32 <= args.N);
  if (args.bias != nullptr && ks == 0) {
    if (full && (reinterpret_cast<uintptr_t>(args.bias) & 15) == 0) {
      const uint4* bp = reinterpret_cast<const uint4*>(args.bias + col0);  // col0 is a multiple of 32
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        const uint4 pk = __ldg(bp + (j >> 3));
        const float2 a0 = unpack_bf16x2(pk.x), a1 = unpack_bf16x2(pk.y), a2 = unpack_bf16x2(pk.z),
                     a3 = unpack_bf16x2(pk.w);
        f[j] += a0.x;
        f[j + 1] += a0.y;
        f[j + 2] += a1.x;
        f[j + 3] += a1.y;
        f[j + 4] += a2.x;
        f[j + 5] += a2.y;
        f[j + 6] += a3.x;
        f[j + 7] += a3.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (full || col0 + j < args.N) f[j] += __bfloat162float(args.bias[col0 + j]);
    }
  }
  if (args.epilogue == kEpiGelu) {
    __nv_bfloat16* aux = args.aux_out + static_cast<int64_t>(row) * args.ldaux + col0;
    if (full && (args.ldaux & 7) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        // the activation is taken of the ROUNDED pre-activation, which is what the backward pass reads
        const uint4 pk = make_uint4(pack_bf16x2(f[j], f[j + 1]), pack_bf16x2(f[j + 2], f[j + 3]),
                                    pack_bf16x2(f[j + 4], f[j + 5]), pack_bf16x2(f[j + 6], f[j + 7]));
        *reinterpret_cast<uint4*>(aux + j) = pk;
        const float2 a0 = unpack_bf16x2(pk.x), a1 = unpack_bf16x2(pk.y), a2 = unpack_bf16x2(pk.z),
                     a3 = unpack_bf16x2(pk.w);
        f[j] = gelu_tanh(a0.x);
        f[j + 1] = gelu_tanh(a0.y);
        f[j + 2] = gelu_tanh(a1.x);
        f[j + 3] = gelu_tanh(a1.y);
        f[j + 4] = gelu_tanh(a2.x);
        f[j + 5] = gelu_tanh(a2.y);
        f[j + 6] = gelu_tanh(a3.x);
        f[j + 7] = gelu_tanh(a3.y);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const __nv_bfloat16 r = __float2bfloat16(f[j]);
        if (col0 + j < args.N) aux[j] = r;
        f[j] = gelu_tanh(__bfloat162float(r));
      }
    }
  } else if (args.epilogue == kEpiGeluGrad) {
    const __nv_bfloat16* aux = args.aux_in + static_cast<int64_t>(row) * args.ldaux + col0;
    if (full && (args.ldaux & 7) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 pk = *reinterpret_cast<const uint4*>(aux + j);
        float2 a0 = unpack_bf16x2(pk.x), a1 = unpack_bf16x2(pk.y), a2 = unpack_bf16x2(pk.z),
               a3 = unpack_bf16x2(pk.w);
        f[j] *= gelu_tanh_grad(a0.x);
        f[j + 1] *= gelu_tanh_grad(a0.y);
        f[j + 2] *= gelu_tanh_grad(a1.x);
        f[j + 3] *= gelu_tanh_grad(a1.y);
        f[j + 4] *= gelu_tanh_grad(a2.x);
        f[j + 5] *= gelu_tanh_grad(a2.y);
        f[j + 6] *= gelu_tanh_grad(a3.x);
        f[j + 7] *= gelu_tanh_grad(a3.y);
      }
    } else {
      {
_Pragma("unroll") for (int j = 0; j < 32; ++j)
        if (col0 + j < args.N) f[j] *= gelu_tanh_grad(__bfloat162float(aux[j]));
      }
    }
  }
  if (args.residual != nullptr && ks == 0) {
    const __nv_bfloat16* res = args.residual + static_cast<int64_t>(row) * args.ldr + col0;
    if (full && (args.ldr & 7) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 pk = *reinterpret_cast<const uint4*>(res + j);
        float2 a0 = unpack_bf16x2(pk.x), a1 = unpack_bf16x2(pk.y), a2 = unpack_bf16x2(pk.z),
               a3 = unpack_bf16x2(pk.w);
        f[j] += a0.x;
        f[j + 1] += a0.y;
        f[j + 2] += a1.x;
        f[j + 3] += a1.y;
        f[j + 4] += a2.x;
        f[j + 5] += a2.y;
        f[j + 6] += a3.x;
        f[j + 7] += a3.y;
      }
    } else {
      {
_Pragma("unroll") for (int j = 0; j < 32; ++j)
        if (col0 + j < args.N) f[j] += __bfloat162float(res[j]);
      }
    }
  }
  if (args.out_mode == kOutBf16) {
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(args.out) + static_cast<int64_t>(row) * args.ldo + col0;
    if (full && (args.ldo & 7) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 pk = make_uint4(pack_bf16x2(f[j], f[j + 1]), pack_bf16x2(f[j + 2], f[j + 3]),
                              pack_bf16x2(f[j + 4], f[j + 5]), pack_bf16x2(f[j + 6], f[j + 7]));
        *reinterpret_cast<uint4*>(o + j) = pk;
      }
    } else {
      {
_Pragma("unroll") for (int j = 0; j < 32; ++j)
        if (col0 + j < args.N) o[j] = __float2bfloat16(f[j]);
      }
    }
  } else if (args.out_mode == kOutF32) {
    float* o = static_cast<float*>(args.out) + static_cast<int64_t>(row) * args.ldo + col0;
    if (full && (args.ldo & 3) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(o + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
    } else {
      {
_Pragma("unroll") for (int j = 0; j < 32; ++j)
        if (col0 + j < args.N) o[j] = f[j];
      }
    }
  } else {
    float* o;
    if (args.out_mode == kOutBf16PeerRed) {
      const int peer = row / args.rows_per_peer;
      o = args.peer_out[peer] + static_cast<int64_t>(row - peer * args.rows_per_peer) * args.ldo + col0;
    } else {
      o = static_cast<float*>(args.out) + static_cast<int64_t>(row) * args.ldo + col0;
    }
    if (full && (args.ldo & 3) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        // vectorised fp32 reduction; also valid on peer-mapped (NVLink) addresses
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o + j), "f"(f[j]), "f"(f[j + 1]),
                     "f"(f[j + 2]), "f"(f[j + 3])
                     : "memory");
      }
    } else {
      {
_Pragma("unroll") for (int j = 0; j < 32; ++j)
        if (col0 + j < args.N) atomicAdd(o + j, f[j]);
      }
    }
  }
}

constexpr int kEpiStageBytesPerWarp = 4096;  // 32 rows x 128 bytes (64 bf16 columns)

// True when a 64-column group can take the staged path below (warp-uniform).
__device__ __forceinline__ bool gemm_epilogue_staged_ok(const GemmArgs& args, int col0, int ks) {
  if ((args.out_mode != kOutBf16 && args.out_mode != kOutBf16PeerPush) || col0 + 64 > args.N || (args.ldo & 7) != 0)
    return false;
  const bool has_res = args.residual != nullptr && ks == 0;
  if (has_res && (args.epilogue == kEpiGeluGrad || (args.ldr & 7) != 0)) return false;
  if (args.epilogue != kEpiNone && (args.ldaux & 7) != 0) return false;
  if (args.bias != nullptr && (reinterpret_cast<uintptr_t>(args.bias) & 15) != 0) return false;
  return true;
}

// One warp converts 32 accumulator rows x 64 columns and writes them as bf16. The values pass through a
// 4 KB shared-memory tile of the warp (rows of 128 bytes, 16-byte chunks XOR-swizzled by the row so that
// both the row-per-lane accesses and the transposed ones are free of bank conflicts): global loads of the
// residual / saved pre-activation and the global stores then move whole 128-byte lines (eight lanes per
// row, four rows per instruction) instead of 32 scattered 16-byte pieces.
//   tmem_addr: TMEM address of the warp's lane quarter at the first of the 64 columns
//   row0: global row of lane 0; col0: first global column (multiple of 64)
__device__ __forceinline__ void gemm_epilogue_group64(const GemmArgs& args, uint32_t tmem_addr, uint8_t* stage,
                                                      int row0, int col0, int lane, int ks) {
  const bool has_res = args.residual != nullptr && ks == 0;
  const bool gelu_grad = args.epilogue == kEpiGeluGrad;
  const int tr = lane >> 3, tc = lane & 7;  // transposed role: row within a group of four, 16-byte chunk
  auto chunk_ptr = [&](int r, int c) { return reinterpret_cast<uint4*>(stage + r * 128 + ((c ^ (r & 7)) << 4)); };
  auto stage_load = [&](const __nv_bfloat16* src, int64_t ld) {
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int r = it * 4 + tr;
      uint4 val = make_uint4(0u, 0u, 0u, 0u);
      if (row0 + r < args.M)
        val = __ldg(reinterpret_cast<const uint4*>(src + static_cast<int64_t>(row0 + r) * ld + col0 + tc * 8));
      *chunk_ptr(r, tc) = val;
    }
    __syncwarp();
  };
  auto stage_store = [&](__nv_bfloat16* dst, int64_t ld) {
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int r = it * 4 + tr;
      if (row0 + r < args.M)
        *reinterpret_cast<uint4*>(dst + static_cast<int64_t>(row0 + r) * ld + col0 + tc * 8) = *chunk_ptr(r, tc);
    }
    __syncwarp();
  };

  if (has_res) stage_load(args.residual, args.ldr);
  else if (gelu_grad) stage_load(args.aux_in, args.ldaux);

#pragma unroll 1
  for (int h = 0; h < 2; ++h) {
    uint32_t v[32];
    tmem_ld_32x32(tmem_addr + h * 32, v);
    tmem_ld_wait();
    float f[32];
    if (args.alpha == 1.f) {
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) * args.alpha;
    }
    if (args.bias != nullptr && ks == 0) {
      const uint4* bp = reinterpret_cast<const uint4*>(args.bias + col0 + h * 32);
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        const uint4 pk = __ldg(bp + (j >> 3));
        const float2 a0 = unpack_bf16x2(pk.x), a1 = unpack_bf16x2(pk.y), a2 = unpack_bf16x2(pk.z),
                     a3 = unpack_bf16x2(pk.w);
        f[j] += a0.x;
        f[j + 1] += a0.y;
        f[j + 2] += a1.x;
        f[j + 3] += a1.y;
        f[j + 4] += a2.x;
        f[j + 5] += a2.y;
        f[j + 6] += a3.x;
        f[j + 7] += a3.y;
      }
    }
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      uint4* sp = chunk_ptr(lane, h * 4 + (j >> 3));
      if (has_res || gelu_grad) {
        const uint4 pk = *sp;
        const float2 a0 = unpack_bf16x2(pk.x), a1 = unpack_bf16x2(pk.y), a2 = unpack_bf16x2(pk.z),
                     a3 = unpack_bf16x2(pk.w);
        if (gelu_grad) {
          f[j] *= gelu_tanh_grad(a0.x);
          f[j + 1] *= gelu_tanh_grad(a0.y);
          f[j + 2] *= gelu_tanh_grad(a1.x);
          f[j + 3] *= gelu_tanh_grad(a1.y);
          f[j + 4] *= gelu_tanh_grad(a2.x);
          f[j + 5] *= gelu_tanh_grad(a2.y);
          f[j + 6] *= gelu_tanh_grad(a3.x);
          f[j + 7] *= gelu_tanh_grad(a3.y);
        } else {
          f[j] += a0.x;
          f[j + 1] += a0.y;
          f[j + 2] += a1.x;
          f[j + 3] += a1.y;
          f[j + 4] += a2.x;
          f[j + 5] += a2.y;
          f[j + 6] += a3.x;
          f[j + 7] += a3.y;
        }
      }
      *sp = make_uint4(pack_bf16x2(f[j], f[j + 1]), pack_bf16x2(f[j + 2], f[j + 3]), pack_bf16x2(f[j + 4], f[j + 5]),
                       pack_bf16x2(f[j + 6], f[j + 7]));
    }
  }
  if (args.epilogue == kEpiGelu) {
    // the staged values are the rounded pre-activations: store them, then overwrite them with the activation
    stage_store(args.aux_out, args.ldaux);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint4* sp = chunk_ptr(lane, c);
      const uint4 pk = *sp;
      const float2 a0 = unpack_bf16x2(pk.x), a1 = unpack_bf16x2(pk.y), a2 = unpack_bf16x2(pk.z),
                   a3 = unpack_bf16x2(pk.w);
      *sp = make_uint4(pack_bf16x2(gelu_tanh(a0.x), gelu_tanh(a0.y)), pack_bf16x2(gelu_tanh(a1.x), gelu_tanh(a1.y)),
                       pack_bf16x2(gelu_tanh(a2.x), gelu_tanh(a2.y)), pack_bf16x2(gelu_tanh(a3.x), gelu_tanh(a3.y)));
    }
  }
  if (args.out_mode == kOutBf16PeerPush) {
    // the 32 rows belong to one owner: they go into this rank's slot of the owner's receive buffer
    const int peer = row0 / args.rows_per_peer;
    __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(args.peer_out[peer]) +
                          (static_cast<int64_t>(args.self_rank) - peer) * args.rows_per_peer * args.ldo;
    stage_store(base, args.ldo);
  } else {
    stage_store(static_cast<__nv_bfloat16*>(args.out), args.ldo);
  }
}

// fp32 outputs (plain store or reduction into a local buffer), 32 rows x 32 columns per call: the same staging
// tile holds 128-byte rows of four-float chunks, so that every store / red.add instruction covers four whole lines.
__device__ __forceinline__ bool gemm_epilogue_staged_f32_ok(const GemmArgs& args, int col0, int ks) {
  if (args.out_mode != kOutF32 && args.out_mode != kOutF32Atomic) return false;
  if (col0 + 32 > args.N || (args.ldo & 3) != 0 || args.epilogue != kEpiNone) return false;
  if (ks == 0 && (args.bias != nullptr || args.residual != nullptr)) return false;
  return true;
}
__device__ __forceinline__ void gemm_epilogue_group32_f32(const GemmArgs& args, uint32_t tmem_addr, uint8_t* stage,
                                                          int row0, int col0, int lane) {
  const int tr = lane >> 3, tc = lane & 7;
  auto chunk_ptr = [&](int r, int c) { return reinterpret_cast<float4*>(stage + r * 128 + ((c ^ (r & 7)) << 4)); };
  uint32_t v[32];
  tmem_ld_32x32(tmem_addr, v);
  tmem_ld_wait();
#pragma unroll
  for (int c = 0; c < 8; ++c)
    *chunk_ptr(lane, c) = make_float4(__uint_as_float(v[4 * c]) * args.alpha, __uint_as_float(v[4 * c + 1]) * args.alpha,
                                      __uint_as_float(v[4 * c + 2]) * args.alpha,
                                      __uint_as_float(v[4 * c + 3]) * args.alpha);
  __syncwarp();
  float* out = static_cast<float*>(args.out);
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = it * 4 + tr;
    if (row0 + r < args.M) {
      const float4 val = *chunk_ptr(r, tc);
      float* o = out + static_cast<int64_t>(row0 + r) * args.ldo + col0 + tc * 4;
      if (args.out_mode == kOutF32) {
        *reinterpret_cast<float4*>(o) = val;
      } else {
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o), "f"(val.x), "f"(val.y), "f"(val.z),
                     "f"(val.w)
                     : "memory");
      }
    }
  }
  __syncwarp();
}

// The columns [col_begin, col_end) of one accumulator (multiples of 64 within the tile) for one epilogue warp:
// staged 64-column groups where possible, 32-column chunks otherwise.
//   tmem_acc: TMEM address of the accumulator's column 0 in the warp's lane quarter; n0: the tile's first column
__device__ __forceinline__ void gemm_epilogue_columns(const GemmArgs& args, uint32_t tmem_acc, uint8_t* stage, int row0,
                                                      int n0, int col_begin, int col_end, int lane, int ks,
                                                      bool has_k) {
  const int row = row0 + lane;
#pragma unroll 1
  for (int cc = col_begin; cc < col_end; cc += 64) {
    const int col0 = n0 + cc;
    if (col0 >= args.N) break;  // uniform across the warp
    if (!has_k) continue;
    if (gemm_epilogue_staged_ok(args, col0, ks)) {
      gemm_epilogue_group64(args, tmem_acc + cc, stage, row0, col0, lane, ks);
      continue;
    }
#pragma unroll 1
    for (int h = 0; h < 2; ++h) {
      if (col0 + h * 32 >= args.N) break;
      if (gemm_epilogue_staged_f32_ok(args, col0 + h * 32, ks)) {
        gemm_epilogue_group32_f32(args, tmem_acc + cc + h * 32, stage, row0, col0 + h * 32, lane);
        continue;
      }
      uint32_t v[32];
      tmem_ld_32x32(tmem_acc + cc + h * 32, v);
      tmem_ld_wait();
      if (row < args.M) gemm_epilogue_chunk(args, v, row, col0 + h * 32, ks);
    }
  }
}

}  // namespace b200
