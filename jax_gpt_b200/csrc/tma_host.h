// Host-side construction of TMA tensor maps. The driver entry point is resolved at run
// time through the CUDA runtime so the library links without libcuda.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// 2-D tiled map with 128-byte swizzle. `inner` / `outer` are extents in elements, the row
// stride is in bytes (multiple of 16), the box is `box_inner` x `box_outer` elements and
// box_inner * elem_bytes must equal 128.
cudaError_t encode_tma_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                          uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);

// 3-D variant: dims (inner, mid, outer) with byte strides for mid and outer.
cudaError_t encode_tma_3d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t inner, uint64_t mid,
                          uint64_t outer, uint64_t mid_stride_bytes, uint64_t outer_stride_bytes, uint32_t box_inner,
                          uint32_t box_mid, uint32_t box_outer);

}  // namespace b200
