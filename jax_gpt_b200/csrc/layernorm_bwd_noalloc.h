/* LayerNorm backward for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference project. It exists for hosts that embed
 * this library but cannot call cudaMalloc themselves or let a library do it for them: for
 * example an inference server whose own memory manager has already claimed the whole device
 * and hands out sub-ranges, or a plug-in that runs under a framework which accounts for every
 * byte of device memory and forbids allocations outside its pool. Such callers still own their
 * inputs and outputs, but they have nowhere to put the kernel's scratch.
 *
 * The regular launcher (b200::launch_norm_bwd) takes that scratch, a buffer of per-block
 * partial sums of the scale and bias gradients, from the caller. This variant keeps it in a
 * fixed array that is part of the library image, so every GPU that loads the library holds
 * B200_LN_BWD_NOALLOC_SCRATCH_BYTES (about 9.3 MiB) from load until exit, used or not. The
 * price of the fixed size is a limit on the row width:
 *
 *     D % 8 == 0  and  8 <= D <= B200_LN_BWD_NOALLOC_MAX_D (1024)
 *
 * Wider rows are rejected with B200_NOALLOC_ERR_TOO_LARGE; nothing is launched.
 *
 * Semantics are those of the regular entry point in LayerNorm mode:
 *     dx     = layer_norm_backward(dy; x, gamma, mean, rstd)  (+ dres when dres != NULL)
 *     dgamma += sum_rows dy * xhat          (accumulated into what is there)
 *     dbeta  += sum_rows dy
 * dy, x, dres, dx are [M, D] bf16 row-major; gamma is [D] bf16; mean, rstd are [M] fp32 as
 * written by the forward kernel; dgamma, dbeta are [D] fp32. All pointers are device pointers
 * on the current device, 16-byte aligned. The stream must belong to the current device as well
 * (the scratch address is looked up for the device that is current at the call).
 *
 * Things a caller has to know:
 *  - The first call on each device looks up the device address of the scratch array
 *    (cudaGetSymbolAddress) and remembers it. Make that first call during start-up, with the
 *    device current, before any stream capture begins on that device.
 *  - The function calls no cudaMalloc, cudaFree or other allocating routine, on any call.
 *  - All calls on a device share the one scratch array. Two calls whose kernels can overlap on
 *    the GPU (different streams without an ordering between them, or host threads launching
 *    concurrently) race on it and produce wrong gradients. Calls on one stream are safe.
 *  - The array keeps the previous call's partial sums. That is harmless: every row of it that a
 *    call reads is written by the same call first, so nothing has to start at zero.
 *
 * Returns 0 on success, a negative B200_NOALLOC_ERR_* code for a rejected argument, or the
 * positive cudaError_t of a failed CUDA call. b200_noalloc_strerror() turns any of them into text.
 */
#ifndef B200_LAYERNORM_BWD_NOALLOC_H_
#define B200_LAYERNORM_BWD_NOALLOC_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_LN_BWD_NOALLOC_MAX_D 1024
#define B200_LN_BWD_NOALLOC_MAX_BLOCKS 296
#define B200_LN_BWD_NOALLOC_ROWS_PER_BLOCK 4
#define B200_LN_BWD_NOALLOC_SCRATCH_BYTES \
  ((size_t)B200_LN_BWD_NOALLOC_MAX_BLOCKS * B200_LN_BWD_NOALLOC_ROWS_PER_BLOCK * 2 * B200_LN_BWD_NOALLOC_MAX_D * 4)

#define B200_NOALLOC_ERR_TOO_LARGE (-1)  /* D beyond B200_LN_BWD_NOALLOC_MAX_D */
#define B200_NOALLOC_ERR_BAD_SHAPE (-2)  /* M < 1, D < 8 or D not a multiple of 8 */
#define B200_NOALLOC_ERR_NULL_PTR (-3)   /* a required pointer is NULL */
#define B200_NOALLOC_ERR_ALIGNMENT (-4)  /* a pointer is not 16-byte aligned */

int b200_layernorm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* mean,
                               const float* rstd, const void* dres, void* dx, float* dgamma, float* dbeta, int M,
                               int D, void* cuda_stream);

const char* b200_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif

#endif /* B200_LAYERNORM_BWD_NOALLOC_H_ */
