// Allocation-free entry point of the elementwise library (built from elementwise.cu).
//
// This entry point has no counterpart in the reference project: it exists for callers of this library that are
// not allowed to allocate device memory at the point where they need an RMSNorm backward pass.  Typical cases:
//   * a serving or training process whose device-memory budget is fixed at start-up, where a later cudaMalloc can
//     fail, or stalls the whole device because cudaMalloc / cudaFree synchronise;
//   * a plug-in called from another runtime (a C, C++ or Fortran host, or a language binding without PyTorch) that
//     has no caching allocator to ask for workspace and must not touch the owner's memory pool;
//   * a latency-critical step that has been audited to perform no allocator calls at all.
// The ordinary entry point `ts_rmsnorm_bwd` needs a caller-provided fp32 workspace of [parts][H] floats for the
// per-CTA partial sums of the weight gradient.  Here that workspace is a fixed array inside the library image.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest row width (elements) and number of partial rows the built-in workspace holds.
// The array is TS_NOALLOC_MAX_PARTS * TS_NOALLOC_MAX_H floats = 4.625 MiB; every GPU that loads the library keeps
// that much reserved until the process exits.
#define TS_NOALLOC_MAX_H 8192
#define TS_NOALLOC_MAX_PARTS 148

// RMSNorm backward without any allocation.  Same mathematics and argument meaning as `ts_rmsnorm_bwd`, minus the
// workspace argument:
//   dx[rows][H]  = rstd * (dy * (w + w_offset) - xhat * mean(dy * (w + w_offset) * xhat)) (+ dres if given)
//   dw[H]        = sum over rows of dy * xhat   (written to dw_f32 and / or dw_bf16; added to them if accumulate_dw)
// Inputs and outputs are still the caller's buffers.  All pointers are device pointers on the current device;
// dy / x / w / dres / dx / dw_bf16 are bf16, rstd / dw_f32 fp32.  H must be a multiple of 8.
//
// Returns 0 on success.  Returns -20 (and prints one line to stderr) when H > TS_NOALLOC_MAX_H, H % 8 != 0 or
// rows <= 0 or rows >= 2^31; the workspace is never exceeded.  Returns a positive cudaError_t value if the CUDA runtime refuses
// the set-up or a launch.
//
// Set-up: the first call on each device looks up the device address of the built-in workspace
// (cudaGetSymbolAddress) with that device current and caches it.  Make that first call before any stream capture
// begins; later calls only launch kernels.
//
// Sharing: every call on a device uses the same workspace and leaves its last contents in it.  Each call
// overwrites every element it later reads, so nothing needs clearing between calls; but two calls that can run
// at the same time on one GPU (different streams, or different host threads on different streams) race on it.
// Serialise them on one stream or with events.
//
// The function calls no cudaMalloc, cudaFree, or any other allocating routine (PyTorch's included).
int ts_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                           float* dw_f32, void* dw_bf16, int accumulate_dw, long long rows, int H, float w_offset,
                           void* stream);

#ifdef __cplusplus
}
#endif
