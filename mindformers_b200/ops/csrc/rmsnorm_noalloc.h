// RMSNorm backward for callers that are not allowed to allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for embedders of this library.
//
// Who needs it: code that runs where cudaMalloc is off limits. Examples are a plug-in whose host application
// owns all device memory and hands out fixed buffers, a real-time or serving loop that has promised not to touch
// the allocator after start-up (an allocation may synchronise the device or fail under fragmentation), and code
// on a stream that is being recorded, where allocation calls are not permitted. The regular entry point,
// mfb_rmsnorm_bwd, asks such a caller for a scratch buffer of mfb_rmsnorm_bwd_parts(T) * H floats; this variant
// brings its own.
//
// What it computes: exactly what mfb_rmsnorm_bwd computes (dx, and dw summed over the T rows), with the partial
// column sums kept in an array that is compiled into the library instead of in caller memory. The caller still
// passes every input and output pointer.
//
// Limits and rules:
//   * H must be a multiple of 8 and at most 8192; larger H is rejected with an error (return code 1,
//     text from mfb_last_error()). T is not limited: rows are spread over at most 148 thread blocks.
//   * The built-in array is 148 * 8192 floats (4.6 MiB). Each GPU that loads the library holds one copy until
//     the process ends, whether or not this function is ever called.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device
//     current) and remembers it. Make that first call during start-up, before any stream capture begins.
//   * All calls on a device share the one array, and it keeps whatever the last call left in it. A call
//     overwrites every element it later reads, so no clearing is needed between calls; but two calls that
//     overlap on the GPU (different streams without an ordering between them) race on it. Serialise them.
//   * Nothing here calls cudaMalloc, cudaFree or any other allocating routine.
//
// Returns 0 on success; 1 bad argument, 2 launch failure, 3/4 set-up failure.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

int mfb_rmsnorm_bwd_noalloc(const void* dy,      // [T, H] bf16 gradient of the normalised output
                            const void* h,       // [T, H] bf16 input of the norm (after the residual add)
                            const void* w,       // [H] bf16 norm weight
                            const float* rstd,   // [T] reciprocal RMS saved by the forward pass
                            const void* dres,    // [T, H] bf16 gradient arriving through the residual, or null
                            void* dx,            // [T, H] bf16 out
                            float* dw_f32,       // [H] fp32 out (or null)
                            void* dw_bf16,       // [H] bf16 out (or null); one of the two must be given
                            int accumulate,      // 0: dw = sum, 1: dw += sum
                            int T, int H, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
