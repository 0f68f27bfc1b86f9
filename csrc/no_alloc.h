// Entry point for callers that must not allocate device memory.
//
// This has no counterpart in the reference implementation (which is pure Python on PyTorch and lets
// the caching allocator provide every temporary).  It exists for embedders of this library that run
// where an allocation is not allowed or not possible: code executing inside someone else's memory
// budget (a serving process whose whole device pool was reserved up front), code running between the
// begin and end of a CUDA stream capture started by the host application, plugins called from a
// runtime that forbids cudaMalloc in its callbacks, and real-time loops that cannot afford the
// implicit device synchronisation cudaFree performs.  Such callers own their inputs and outputs but
// have nowhere to get the kernel's temporary storage from.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the built-in scratch area covers: hidden size (columns) and the number of per-CTA
// partial rows the kernel may use.  Scratch held per GPU: B2_NOALLOC_MAX_PARTIALS * B2_NOALLOC_MAX_H * 4 bytes
// (= 2 MiB), resident from the moment the library is loaded on that GPU until the process exits.
#define B2_NOALLOC_MAX_H 2048
#define B2_NOALLOC_MAX_PARTIALS 256

// RMSNorm backward without any allocation.  Same mathematics and kernels as b2_rmsnorm_bwd, but the
// fp32 partial-sum buffer for the weight gradient lives in a static device array inside the library
// instead of being passed in.
//
//   dy, x [M, H] bf16; w [H] bf16; rstd [M] fp32 (saved by the forward); dx [M, H] bf16 (output);
//   dw [H] (output; bf16, or fp32 when dw_fp32 != 0; accumulate_dw != 0 adds to it).
//   H must be a multiple of 8, at most B2_NOALLOC_MAX_H, and 256 must be divisible by H / 8.
//
// Returns 0 on success; a non-zero code with a message in b2_last_error() when the size exceeds the
// built-in scratch, an argument is malformed, or a CUDA call fails.
//
// The first call on each device looks up the device address of the scratch array, and the first call
// from each host thread makes the library's device current on that thread (cudaSetDevice, or an empty
// cudaFree when no device was announced): make the first call of every (thread, device) pair outside of
// any stream capture.  Null data pointers, a negative M and an H outside the limits above are rejected
// with code 10 before anything is launched; M == 0 is a successful no-op.  All calls on a device share the one scratch array: the kernel
// overwrites the part it uses before reading it, so nothing has to be cleared between calls, but two
// calls whose kernels overlap in time on the same device (different streams) would corrupt each
// other's partial sums — issue them on one stream or order them with events.
int b2_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                           void* dw, int M, int H, int add_to_dx, int accumulate_dw, int dw_fp32,
                           void* stream);

#ifdef __cplusplus
}
#endif
