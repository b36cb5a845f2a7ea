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

}  // namespace b200
