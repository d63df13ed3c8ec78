// Allocation-free entry point of the uttt_b200 extension.
//
// This entry point has no counterpart in the reference implementation.  It exists for callers that are not
// allowed to allocate device memory while they run: code executing inside a memory-pool-restricted serving
// process, a host thread that must never take the allocator lock, or a plugin whose host application owns
// every byte of the device heap.  Such callers cannot use the regular RMSNorm backward of this library,
// because that one asks torch for a temporary [blocks, d] buffer to hold per-CTA partial sums of the weight
// gradient.
//
// uttt_rms_norm_bwd_noalloc computes the same result (dx and dw of y = x * rsqrt(mean(x^2) + eps) * w) but keeps
// the partial sums in a fixed array that lives inside the library image: 128 x 4096 floats = 2 MiB per GPU that
// loads the library, held until the process exits.  It calls no cudaMalloc / cudaFree and no allocating
// library routine (torch's included); the caller passes every input and output buffer.
//
// Limits and rules:
//   * d must be a multiple of 8 and at most 4096; rows >= 1.  Larger sizes are rejected (return code 2), never
//     truncated.
//   * dtype: 0 = bfloat16, 1 = float32 (dy, x, w, dx share it; rstd and dw are float32).  w may be NULL
//     (parameter-free norm): then dw is not written.
//   * The first call on each device looks up the device address of the internal array (with that device
//     current).  Make that first call before starting any stream capture on the device.
//   * All calls share the one array per device and it keeps the previous call's contents.  Nothing in it needs
//     to start at zero (every slot that is read is written first by the same call), but two calls whose
//     kernels overlap on the GPU (different streams, no ordering) would overwrite each other's partial sums:
//     serialise them.
//
// Return value: 0 on success; 1 bad argument; 2 size beyond the built-in maximum; 3 a CUDA call failed
// (cudaGetLastError() has the detail).
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

int uttt_rms_norm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                              int rows, int d, int dtype, void* cuda_stream);

#ifdef __cplusplus
}
#endif
