#include "tma_host.h"

#include <cudaTypedefs.h>

namespace b200 {

namespace {

PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

// cuTensorMapEncodeTiled is a driver call and needs a current context on the calling thread.
// Threads that have only used the runtime lazily (e.g. an autograd worker) may not have one
// yet; a no-op runtime call binds the primary context.
void ensure_context() {
  thread_local bool ready = false;
  if (!ready) {
    cudaFree(nullptr);
    ready = true;
  }
}

CUtensorMapDataType dtype_for(int elem_bytes) {
  return elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                         : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
}

}  // namespace

cudaError_t encode_tma_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                          uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  auto fn = get_encode();
  if (fn == nullptr) return cudaErrorNotSupported;
  ensure_context();
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_stride_bytes & 15) != 0) return cudaErrorMisalignedAddress;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dtype_for(elem_bytes), 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

cudaError_t encode_tma_3d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t inner, uint64_t mid,
                          uint64_t outer, uint64_t mid_stride_bytes, uint64_t outer_stride_bytes, uint32_t box_inner,
                          uint32_t box_mid, uint32_t box_outer) {
  auto fn = get_encode();
  if (fn == nullptr) return cudaErrorNotSupported;
  ensure_context();
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (mid_stride_bytes & 15) != 0 || (outer_stride_bytes & 15) != 0)
    return cudaErrorMisalignedAddress;
  cuuint64_t dims[3] = {inner, mid, outer};
  cuuint64_t strides[2] = {mid_stride_bytes, outer_stride_bytes};
  cuuint32_t box[3] = {box_inner, box_mid, box_outer};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dtype_for(elem_bytes), 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

}  // namespace b200
