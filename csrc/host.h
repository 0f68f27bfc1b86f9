// Host-side helpers shared by the launchers: status word access and TMA tensor-map encoding.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define B2_EXPORT extern "C" __attribute__((visibility("default")))

namespace b2 {

// Makes the process's device (b2_set_device) current on the calling thread.  Launchers call this
// first: autograd runs backward passes on worker threads that this library's runtime has never
// seen, and driver entry points such as the tensor-map encoder need a current context.
void ensure_thread_context();

// Device address of this device's status word (one int; 0 = no error).
int* status_ptr();

// Last host-side error text (argument checks, CUDA runtime failures).
void set_error(const char* fmt, ...);

// Encode (and cache) a 2-D tiled tensor map over a row-major [rows, cols] matrix of 2-byte
// elements with row stride `ld` elements; box = [box_rows, box_cols], 128-byte swizzle.
// box_cols * 2 must be 128.  Returns nullptr on failure.
const CUtensorMap* tensor_map_2d_bf16(const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                                      uint32_t box_rows, uint32_t box_cols);

// Generic N-D (<=4) tiled tensor map for 2-byte elements.  dims/strides innermost first; strides in
// bytes for dims 1..n-1.  swizzle: 0 none, 1 32B, 2 64B, 3 128B.
const CUtensorMap* tensor_map_nd_bf16(const void* base, int rank, const uint64_t* dims,
                                      const uint64_t* strides_bytes, const uint32_t* box,
                                      int swizzle);

inline int num_sms() {
  static int n[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (n[dev] == 0) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
  return n[dev];
}

}  // namespace b2
