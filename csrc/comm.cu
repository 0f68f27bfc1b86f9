// Kernels that move data between GPUs through peer pointers (NVLink / NVSwitch), fused with the
// arithmetic around the transfer:
//
//   peer_write          trainer -> engine weight sync: cast (fp32/bf16 -> bf16/fp32), optional in-place
//                       add (LoRA delta), position-weighted checksum of the payload, one launch per chunk
//   words_checksum      receiver-side checksum of a staging buffer
//   zero_reduce_shard   ZeRO gradient reduce-scatter by peer loads: this rank's shard of every peer's
//                       bucket is summed, scaled, written as fp32 and its squared norm accumulated
//   zero_adamw_publish  clip + AdamW on the shard, updated bf16 parameters stored into every peer's
//                       parameter bucket (the all-gather), all in one pass
//   flag_signal / flag_wait  system-scope release / bounded acquire on a flag word
//
// A destination or source pointer may belong to this GPU or to a peer; the kernels do not care.  No
// TMA and no thread-block clusters are used here: plain (vectorised) loads and stores only.
#include "common.cuh"
#include "host.h"

namespace b2 {

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <typename T>
__device__ __forceinline__ float cvt_in(T v);
template <>
__device__ __forceinline__ float cvt_in<float>(float v) { return v; }
template <>
__device__ __forceinline__ float cvt_in<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T cvt_out(float v);
template <>
__device__ __forceinline__ float cvt_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 cvt_out<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <typename T>
__device__ __forceinline__ unsigned long long bits_of(T v);
template <>
__device__ __forceinline__ unsigned long long bits_of<float>(float v) { return __float_as_uint(v); }
template <>
__device__ __forceinline__ unsigned long long bits_of<__nv_bfloat16>(__nv_bfloat16 v) {
  return *reinterpret_cast<unsigned short*>(&v);
}

// dst[off + i] = (add ? dst[off + i] : 0) + src[i]; checksum[0] += bits(dst_i), checksum[1] += bits * (off+i+1)
template <typename T>
__device__ __forceinline__ void load8_as_float(const T* p, float* f);
template <>
__device__ __forceinline__ void load8_as_float<float>(const float* p, float* f) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <>
__device__ __forceinline__ void load8_as_float<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
  const uint4 q = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = unpack_bf16x2(w[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const T* v);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float* v) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const __nv_bfloat16* v) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(v);
}

template <typename S, typename D>
__global__ void peer_write_kernel(const S* __restrict__ src, D* __restrict__ dst, long long n,
                                  long long elem_offset, int add, unsigned long long* __restrict__ checksum) {
  unsigned long long c0 = 0, c1 = 0;
  // Vector body: 8 elements per thread step (16- or 32-byte accesses, so a warp's peer store is one or two
  // full 512-byte runs instead of 64 bytes); used when source and destination are 16-byte aligned.
  long long nvec = 0;
  if ((reinterpret_cast<uintptr_t>(src) % 16 == 0) &&
      (reinterpret_cast<uintptr_t>(dst + elem_offset) % 16 == 0))
    nvec = n / 8;
  for (long long vi = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; vi < nvec;
       vi += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long i0 = vi * 8;
    float f[8];
    load8_as_float<S>(src + i0, f);
    if (add) {
      float d[8];
      load8_as_float<D>(dst + elem_offset + i0, d);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += d[j];
    }
    alignas(16) D o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o[j] = cvt_out<D>(f[j]);
      const unsigned long long b = bits_of<D>(o[j]);
      c0 += b;
      c1 += b * static_cast<unsigned long long>(elem_offset + i0 + j + 1);
    }
    store8<D>(dst + elem_offset + i0, o);
  }
  for (long long i = nvec * 8 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float v = cvt_in<S>(src[i]);
    if (add) v += cvt_in<D>(dst[elem_offset + i]);
    const D o = cvt_out<D>(v);
    dst[elem_offset + i] = o;
    const unsigned long long b = bits_of<D>(o);
    c0 += b;
    c1 += b * static_cast<unsigned long long>(elem_offset + i + 1);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    c0 += __shfl_xor_sync(0xffffffffu, c0, o);
    c1 += __shfl_xor_sync(0xffffffffu, c1, o);
  }
  if ((threadIdx.x & 31) == 0 && checksum) {
    atomicAdd(checksum, c0);
    atomicAdd(checksum + 1, c1);
  }
  __threadfence_system();
}

template <typename D>
__global__ void words_checksum_kernel(const D* __restrict__ buf, long long n,
                                      unsigned long long* __restrict__ checksum) {
  unsigned long long c0 = 0, c1 = 0;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const unsigned long long b = bits_of<D>(buf[i]);
    c0 += b;
    c1 += b * static_cast<unsigned long long>(i + 1);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    c0 += __shfl_xor_sync(0xffffffffu, c0, o);
    c1 += __shfl_xor_sync(0xffffffffu, c1, o);
  }
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(checksum, c0);
    atomicAdd(checksum + 1, c1);
  }
}

// One unit of a batched copy: n elements from src (element index 0) to dst + dst_off.  A tensor larger than the unit
// size is cut into several units, so that one launch spreads a whole weight image evenly over the grid.
struct CopyUnit {
  const void* src;
  long long dst_off;
  long long n;
};

template <typename S, typename D>
__device__ __forceinline__ void peer_write_span(const S* __restrict__ src, D* __restrict__ dst, long long n,
                                                long long elem_offset, int add, unsigned long long& c0,
                                                unsigned long long& c1, int tid, int nthreads) {
  long long nvec = 0;
  if ((reinterpret_cast<uintptr_t>(src) % 16 == 0) && (reinterpret_cast<uintptr_t>(dst + elem_offset) % 16 == 0))
    nvec = n / 8;
  for (long long vi = tid; vi < nvec; vi += nthreads) {
    const long long i0 = vi * 8;
    float f[8];
    load8_as_float<S>(src + i0, f);
    if (add) {
      float d[8];
      load8_as_float<D>(dst + elem_offset + i0, d);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += d[j];
    }
    alignas(16) D o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o[j] = cvt_out<D>(f[j]);
      const unsigned long long b = bits_of<D>(o[j]);
      c0 += b;
      c1 += b * static_cast<unsigned long long>(elem_offset + i0 + j + 1);
    }
    store8<D>(dst + elem_offset + i0, o);
  }
  for (long long i = nvec * 8 + tid; i < n; i += nthreads) {
    float v = cvt_in<S>(src[i]);
    if (add) v += cvt_in<D>(dst[elem_offset + i]);
    const D o = cvt_out<D>(v);
    dst[elem_offset + i] = o;
    const unsigned long long b = bits_of<D>(o);
    c0 += b;
    c1 += b * static_cast<unsigned long long>(elem_offset + i + 1);
  }
}

// The whole image in one launch: block b handles units b, b + grid, ...; cast, optional add and the
// position-weighted checksum as in peer_write_kernel (positions are offsets into the destination image).
template <typename S, typename D>
__global__ void peer_write_batch_kernel(const CopyUnit* __restrict__ units, int nunits, D* __restrict__ dst, int add,
                                        unsigned long long* __restrict__ checksum) {
  unsigned long long c0 = 0, c1 = 0;
  for (int u = blockIdx.x; u < nunits; u += gridDim.x) {
    const CopyUnit cu = units[u];
    peer_write_span<S, D>(static_cast<const S*>(cu.src), dst, cu.n, cu.dst_off, add, c0, c1, threadIdx.x, blockDim.x);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    c0 += __shfl_xor_sync(0xffffffffu, c0, o);
    c1 += __shfl_xor_sync(0xffffffffu, c1, o);
  }
  if ((threadIdx.x & 31) == 0 && checksum) {
    atomicAdd(checksum, c0);
    atomicAdd(checksum + 1, c1);
  }
  __threadfence_system();
}

// Checksum of the same spans on the receiving side (src is ignored): only what a delta touched is summed.
template <typename D>
__global__ void spans_checksum_kernel(const CopyUnit* __restrict__ units, int nunits, const D* __restrict__ buf,
                                      unsigned long long* __restrict__ checksum) {
  unsigned long long c0 = 0, c1 = 0;
  for (int u = blockIdx.x; u < nunits; u += gridDim.x) {
    const CopyUnit cu = units[u];
    for (long long i = threadIdx.x; i < cu.n; i += blockDim.x) {
      const unsigned long long b = bits_of<D>(buf[cu.dst_off + i]);
      c0 += b;
      c1 += b * static_cast<unsigned long long>(cu.dst_off + i + 1);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    c0 += __shfl_xor_sync(0xffffffffu, c0, o);
    c1 += __shfl_xor_sync(0xffffffffu, c1, o);
  }
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(checksum, c0);
    atomicAdd(checksum + 1, c1);
  }
}

struct PeerPtrs {
  void* p[8];
};

// out[i] = scale * sum_r peers[r][shard_start + i]  (bf16 buckets, 8 elements per thread step);
// norm_sq[0] += sum(out^2).
__global__ void zero_reduce_shard_kernel(PeerPtrs peers, int world, long long shard_start, long long n,
                                         float scale, float* __restrict__ out, int accumulate,
                                         float* __restrict__ norm_sq) {
  float ss = 0.f;
  const long long nvec = n / 8;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
      const uint4 q = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(peers.p[r]) +
                                                      shard_start + i * 8);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    float4* o = reinterpret_cast<float4*>(out + i * 8);
    float4 prev[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
    if (accumulate) {
      prev[0] = o[0];
      prev[1] = o[1];
    }
    const float pv[8] = {prev[0].x, prev[0].y, prev[0].z, prev[0].w, prev[1].x, prev[1].y, prev[1].z, prev[1].w};
    float r[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      r[j] = acc[j] * scale + pv[j];
      ss += r[j] * r[j];
    }
    o[0] = make_float4(r[0], r[1], r[2], r[3]);
    o[1] = make_float4(r[4], r[5], r[6], r[7]);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0 && norm_sq) atomicAdd(norm_sq, ss);
}

// AdamW on the fp32 shard, then the updated bf16 values are stored at [shard_start + i] of every peer's
// parameter bucket.  hyper / norm_sq as in adamw_kernel (loss_optim.cu).
__global__ void zero_adamw_publish_kernel(float* __restrict__ master, float* __restrict__ m,
                                          float* __restrict__ v, const float* __restrict__ grad, long long n,
                                          const float* __restrict__ hyper, const float* __restrict__ norm_sq,
                                          PeerPtrs params, int world, long long shard_start) {
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd = hyper[4];
  const float bc1 = hyper[5], bc2 = hyper[6], max_norm = hyper[7];
  float clip = 1.f;
  bool skip = false;
  if (norm_sq != nullptr) {
    const float ns = norm_sq[0];
    if (!isfinite(ns)) skip = true;
    else if (max_norm > 0.f) clip = fminf(1.f, max_norm / (sqrtf(ns) + 1e-6f));
  }
  const long long nvec = n / 8;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    // 8 consecutive elements per thread as two float4 per array: consecutive threads read consecutive
    // 32-byte pieces, so every warp access is fully coalesced
    float4* mp = reinterpret_cast<float4*>(master + i * 8);
    float4* mm = reinterpret_cast<float4*>(m + i * 8);
    float4* mv = reinterpret_cast<float4*>(v + i * 8);
    const float4* mg = reinterpret_cast<const float4*>(grad + i * 8);
    float4 pw[2] = {mp[0], mp[1]};
    float p[8] = {pw[0].x, pw[0].y, pw[0].z, pw[0].w, pw[1].x, pw[1].y, pw[1].z, pw[1].w};
    if (!skip) {
      const float4 gw[2] = {mg[0], mg[1]};
      float4 m4[2] = {mm[0], mm[1]};
      float4 v4[2] = {mv[0], mv[1]};
      const float gq[8] = {gw[0].x, gw[0].y, gw[0].z, gw[0].w, gw[1].x, gw[1].y, gw[1].z, gw[1].w};
      float mq[8] = {m4[0].x, m4[0].y, m4[0].z, m4[0].w, m4[1].x, m4[1].y, m4[1].z, m4[1].w};
      float vq[8] = {v4[0].x, v4[0].y, v4[0].z, v4[0].w, v4[1].x, v4[1].y, v4[1].z, v4[1].w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float g = gq[j] * clip;
        mq[j] = b1 * mq[j] + (1.f - b1) * g;
        vq[j] = b2 * vq[j] + (1.f - b2) * g * g;
        p[j] = p[j] * (1.f - lr * wd) - lr * (mq[j] / bc1) / (sqrtf(vq[j] / bc2) + eps);
      }
      mm[0] = make_float4(mq[0], mq[1], mq[2], mq[3]);
      mm[1] = make_float4(mq[4], mq[5], mq[6], mq[7]);
      mv[0] = make_float4(vq[0], vq[1], vq[2], vq[3]);
      mv[1] = make_float4(vq[4], vq[5], vq[6], vq[7]);
      mp[0] = make_float4(p[0], p[1], p[2], p[3]);
      mp[1] = make_float4(p[4], p[5], p[6], p[7]);
    }
    uint4 o;
    o.x = pack_bf16x2(p[0], p[1]);
    o.y = pack_bf16x2(p[2], p[3]);
    o.z = pack_bf16x2(p[4], p[5]);
    o.w = pack_bf16x2(p[6], p[7]);
    for (int r = 0; r < world; ++r)
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.p[r]) + shard_start + i * 8) = o;
  }
  __threadfence_system();
}

__global__ void flag_signal_kernel(int* flag, int value) {
  __threadfence_system();
  st_release_sys(flag, value);
}
// Waits until *flag >= value, at most limit_ns; result[0] = 1 on success, 0 when the wait ran out (the
// status word then also records ERR_COMM_FLAG_WAIT).
__global__ void flag_wait_kernel(const int* flag, int value, unsigned long long limit_ns, int* result,
                                 int* status) {
  const unsigned long long t0 = globaltimer_ns();
  int ok = 0;
  for (;;) {
    if (ld_acquire_sys(flag) >= value) {
      ok = 1;
      break;
    }
    if (globaltimer_ns() - t0 > limit_ns) break;
    __nanosleep(200);
  }
  result[0] = ok;
  if (!ok) atomicCAS(status, 0, ERR_COMM_FLAG_WAIT);
}

}  // namespace b2

using namespace b2;

static int grid_for(long long n, int threads, int per_sm = 8) {
  long long b = (n + threads - 1) / threads;
  const long long cap = static_cast<long long>(num_sms()) * per_sm;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}
#define B2_LAUNCH_CHECK(name)                                        \
  do {                                                               \
    cudaError_t e_ = cudaGetLastError();                             \
    if (e_ != cudaSuccess) {                                         \
      set_error(name " launch failed: %s", cudaGetErrorString(e_)); \
      return 4;                                                      \
    }                                                                \
  } while (0)

// dst may be a peer pointer.  checksum: device u64[2] (nullable), accumulated across calls.
B2_EXPORT int b2_peer_write(const void* src, int src_fp32, void* dst, int dst_fp32, long long n,
                            long long elem_offset, int add, unsigned long long* checksum, void* stream_) {
  b2::ensure_thread_context();
  if (n <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const int g = grid_for(n, 256, 4);
  if (src_fp32 && dst_fp32)
    peer_write_kernel<float, float><<<g, 256, 0, s>>>(static_cast<const float*>(src), static_cast<float*>(dst), n, elem_offset, add, checksum);
  else if (src_fp32)
    peer_write_kernel<float, __nv_bfloat16><<<g, 256, 0, s>>>(static_cast<const float*>(src), static_cast<__nv_bfloat16*>(dst), n, elem_offset, add, checksum);
  else if (dst_fp32)
    peer_write_kernel<__nv_bfloat16, float><<<g, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(src), static_cast<float*>(dst), n, elem_offset, add, checksum);
  else
    peer_write_kernel<__nv_bfloat16, __nv_bfloat16><<<g, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), n, elem_offset, add, checksum);
  B2_LAUNCH_CHECK("peer_write");
  return 0;
}

// units: device array of {src pointer, destination element offset, element count} (24 bytes each); every source has
// the same element type.  One launch writes the whole image into dst (local or peer pointer).
B2_EXPORT int b2_peer_write_batch(const void* units, int nunits, int src_fp32, void* dst, int dst_fp32, int add,
                                  unsigned long long* checksum, void* stream_) {
  b2::ensure_thread_context();
  if (nunits <= 0) return 0;
  if (units == nullptr || dst == nullptr) { set_error("peer_write_batch: null table or destination"); return 10; }
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const CopyUnit* u = static_cast<const CopyUnit*>(units);
  int g = num_sms() * 4;
  if (g > nunits) g = nunits;
  if (src_fp32 && dst_fp32)
    peer_write_batch_kernel<float, float><<<g, 256, 0, s>>>(u, nunits, static_cast<float*>(dst), add, checksum);
  else if (src_fp32)
    peer_write_batch_kernel<float, __nv_bfloat16><<<g, 256, 0, s>>>(u, nunits, static_cast<__nv_bfloat16*>(dst), add, checksum);
  else if (dst_fp32)
    peer_write_batch_kernel<__nv_bfloat16, float><<<g, 256, 0, s>>>(u, nunits, static_cast<float*>(dst), add, checksum);
  else
    peer_write_batch_kernel<__nv_bfloat16, __nv_bfloat16><<<g, 256, 0, s>>>(u, nunits, static_cast<__nv_bfloat16*>(dst), add, checksum);
  B2_LAUNCH_CHECK("peer_write_batch");
  return 0;
}

B2_EXPORT int b2_spans_checksum(const void* units, int nunits, const void* buf, int is_fp32,
                                unsigned long long* checksum, void* stream_) {
  b2::ensure_thread_context();
  if (nunits <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const CopyUnit* u = static_cast<const CopyUnit*>(units);
  int g = num_sms() * 4;
  if (g > nunits) g = nunits;
  if (is_fp32)
    spans_checksum_kernel<float><<<g, 256, 0, s>>>(u, nunits, static_cast<const float*>(buf), checksum);
  else
    spans_checksum_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(u, nunits, static_cast<const __nv_bfloat16*>(buf), checksum);
  B2_LAUNCH_CHECK("spans_checksum");
  return 0;
}

B2_EXPORT int b2_words_checksum(const void* buf, int is_fp32, long long n, unsigned long long* checksum,
                                void* stream_) {
  b2::ensure_thread_context();
  if (n <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  if (is_fp32)
    words_checksum_kernel<float><<<grid_for(n, 256, 4), 256, 0, s>>>(static_cast<const float*>(buf), n, checksum);
  else
    words_checksum_kernel<__nv_bfloat16><<<grid_for(n, 256, 4), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(buf), n, checksum);
  B2_LAUNCH_CHECK("words_checksum");
  return 0;
}

// peers: host array of `world` device pointers (bf16 gradient buckets, this rank's own included).
B2_EXPORT int b2_zero_reduce_shard(void* const* peers, int world, long long shard_start, long long n,
                                   float scale, float* out, int accumulate, float* norm_sq, void* stream_) {
  b2::ensure_thread_context();
  if (world < 1 || world > 8 || (n % 8) || (shard_start % 8)) {
    set_error("zero_reduce_shard: world in 1..8 and 8-element aligned shard required");
    return 10;
  }
  if (n <= 0) return 0;
  PeerPtrs pp;
  for (int r = 0; r < 8; ++r) pp.p[r] = r < world ? peers[r] : nullptr;
  zero_reduce_shard_kernel<<<grid_for(n / 8, 256, 4), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      pp, world, shard_start, n, scale, out, accumulate, norm_sq);
  B2_LAUNCH_CHECK("zero_reduce_shard");
  return 0;
}

B2_EXPORT int b2_zero_adamw_publish(float* master, float* m, float* v, const float* grad, long long n,
                                    const float* hyper, const float* norm_sq, void* const* params, int world,
                                    long long shard_start, void* stream_) {
  b2::ensure_thread_context();
  if (world < 1 || world > 8 || (n % 8) || (shard_start % 8)) {
    set_error("zero_adamw_publish: world in 1..8 and 8-element aligned shard required");
    return 10;
  }
  if (n <= 0) return 0;
  PeerPtrs pp;
  for (int r = 0; r < 8; ++r) pp.p[r] = r < world ? params[r] : nullptr;
  zero_adamw_publish_kernel<<<grid_for(n / 8, 256, 4), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      master, m, v, grad, n, hyper, norm_sq, pp, world, shard_start);
  B2_LAUNCH_CHECK("zero_adamw_publish");
  return 0;
}

B2_EXPORT int b2_flag_signal(int* flag, int value, void* stream_) {
  b2::ensure_thread_context();
  flag_signal_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream_)>>>(flag, value);
  B2_LAUNCH_CHECK("flag_signal");
  return 0;
}

// result: device int[1].  limit_ms bounds the wait (a second or so in normal use).
B2_EXPORT int b2_flag_wait(const int* flag, int value, int limit_ms, int* result, void* stream_) {
  b2::ensure_thread_context();
  int* status = status_ptr();
  if (!status) return 3;
  flag_wait_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream_)>>>(
      flag, value, static_cast<unsigned long long>(limit_ms) * 1000000ull, result, status);
  B2_LAUNCH_CHECK("flag_wait");
  return 0;
}

namespace b2 {

// ---- multimem (NVLS) forms: one instruction addresses every GPU bound to the multicast object --------------
// Sum over all GPUs of 8 bf16 at the same offset, accumulated in fp32 inside the switch.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
  return r;
}
// 16 bytes stored at the same offset of every GPU's buffer (this GPU's own included).
__device__ __forceinline__ void multimem_st_16B(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w) : "memory");
}

// Group barrier in one launch with the epoch kept on the device, so the launch can sit inside a CUDA graph:
// epoch = ++epochs[channel]; every peer's slot [my_rank][channel] = epoch (release, system scope); then wait,
// bounded, until every source's slot in this rank's own buffer has reached the epoch.  All ranks call it the same
// number of times per channel, so their epochs agree.  ok[0] is cleared (and stays cleared until the host resets
// it) when a wait runs out; the status word records ERR_COMM_FLAG_WAIT.
__global__ void flag_barrier_kernel(PeerPtrs flag_bufs, const int* my_flags, int* epochs, int world, int my_rank,
                                    int channels, int channel, unsigned long long limit_ns, int* ok, int* status) {
  const int lane = threadIdx.x;
  int e = 0;
  if (lane == 0) {
    e = epochs[channel] + 1;
    epochs[channel] = e;
  }
  e = __shfl_sync(0xffffffffu, e, 0);
  __threadfence_system();
  bool failed = false;
  if (lane < world) {
    st_release_sys(static_cast<int*>(flag_bufs.p[lane]) + my_rank * channels + channel, e);
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
      if (ld_acquire_sys(my_flags + lane * channels + channel) >= e) break;
      if (globaltimer_ns() - t0 > limit_ns) {
        failed = true;
        break;
      }
      __nanosleep(100);
    }
  }
  if (__any_sync(0xffffffffu, failed) && lane == 0) {
    ok[0] = 0;
    atomicCAS(status, 0, ERR_COMM_FLAG_WAIT);
  }
}

// Reduce-scatter through the switch: out[i] = scale * sum over GPUs of bucket[shard_start + i], one
// multimem.ld_reduce per 8 elements instead of one load per peer.
__global__ void zero_reduce_shard_mc_kernel(const __nv_bfloat16* __restrict__ mc_bucket, long long shard_start,
                                            long long n, float scale, float* __restrict__ out, int accumulate,
                                            float* __restrict__ norm_sq) {
  float ss = 0.f;
  const long long nvec = n / 8;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  constexpr int U = 4;    // independent reductions in flight per thread: a multimem.ld_reduce is a round trip to the switch
  for (long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
    uint4 q[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      q[u] = make_uint4(0u, 0u, 0u, 0u);
      if (i < nvec) q[u] = multimem_ld_reduce_bf16x8(mc_bucket + shard_start + i * 8);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < nvec) {
        const uint32_t w[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
        float4* o = reinterpret_cast<float4*>(out + i * 8);
        float pv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (accumulate) {
          const float4 p0 = o[0], p1 = o[1];
          pv[0] = p0.x; pv[1] = p0.y; pv[2] = p0.z; pv[3] = p0.w; pv[4] = p1.x; pv[5] = p1.y; pv[6] = p1.z; pv[7] = p1.w;
        }
        float r[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(w[j]);
          r[2 * j] = f.x * scale + pv[2 * j];
          r[2 * j + 1] = f.y * scale + pv[2 * j + 1];
          ss += r[2 * j] * r[2 * j] + r[2 * j + 1] * r[2 * j + 1];
        }
        o[0] = make_float4(r[0], r[1], r[2], r[3]);
        o[1] = make_float4(r[4], r[5], r[6], r[7]);
      }
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0 && norm_sq) atomicAdd(norm_sq, ss);
}

// All-reduce of the two squared-norm partial sums (replicated / TP-sharded parameters) of a data-parallel group in
// one launch: every rank stores its pair into every peer's slot [parity][my_rank], a barrier (as above) orders the
// stores, then each rank sums the slots.  norm_sq[0] = total; grad_norm[0] = sqrt(total), or -1 when not finite.
// Slots are double-buffered by epoch parity: a rank that is one step ahead writes the other half.
__global__ void norm_allreduce_kernel(PeerPtrs slot_bufs, const float* my_slots, PeerPtrs flag_bufs,
                                      const int* my_flags, int* epochs, int world, int my_rank, int channels,
                                      int channel, const float* parts, float* norm_sq, float* grad_norm,
                                      unsigned long long limit_ns, int* ok, int* status) {
  const int lane = threadIdx.x;
  int e = 0;
  if (lane == 0) {
    e = epochs[channel] + 1;
    epochs[channel] = e;
  }
  e = __shfl_sync(0xffffffffu, e, 0);
  const int half = (e & 1) * 16;      // [2 halves][8 ranks][2 floats]
  bool failed = false;
  if (lane < world) {
    float* dst = static_cast<float*>(slot_bufs.p[lane]) + half + my_rank * 2;
    dst[0] = parts[0];
    dst[1] = parts[1];
    __threadfence_system();
    st_release_sys(static_cast<int*>(flag_bufs.p[lane]) + my_rank * channels + channel, e);
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
      if (ld_acquire_sys(my_flags + lane * channels + channel) >= e) break;
      if (globaltimer_ns() - t0 > limit_ns) {
        failed = true;
        break;
      }
      __nanosleep(100);
    }
  }
  failed = __any_sync(0xffffffffu, failed);
  float mine = 0.f;
  if (lane < world) {
    const volatile float* src = my_slots + half + lane * 2;
    mine = src[0] + src[1];
  }
  mine = warp_sum(mine);
  if (lane == 0) {
    if (failed) {
      ok[0] = 0;
      atomicCAS(status, 0, ERR_COMM_FLAG_WAIT);
    }
    norm_sq[0] = mine;
    const float g = sqrtf(mine);
    grad_norm[0] = isfinite(g) ? g : -1.f;
  }
}

// AdamW + publish through the switch: one multimem.st writes the updated bf16 values into every GPU's bucket.
// `ok` (nullable): when it reads 0 (an earlier bounded wait of this step ran out) the update is skipped.
__global__ void zero_adamw_publish_any_kernel(float* __restrict__ master, float* __restrict__ m,
                                              float* __restrict__ v, const float* __restrict__ grad, long long n,
                                              const float* __restrict__ hyper, const float* __restrict__ norm_sq,
                                              PeerPtrs params, __nv_bfloat16* mc_params, int world,
                                              long long shard_start, const int* __restrict__ ok) {
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd = hyper[4];
  const float bc1 = hyper[5], bc2 = hyper[6], max_norm = hyper[7];
  float clip = 1.f;
  bool skip = ok != nullptr && ok[0] == 0;
  if (norm_sq != nullptr) {
    const float ns = norm_sq[0];
    if (!isfinite(ns)) skip = true;
    else if (max_norm > 0.f) clip = fminf(1.f, max_norm / (sqrtf(ns) + 1e-6f));
  }
  const long long nvec = n / 8;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4* mp = reinterpret_cast<float4*>(master + i * 8);
    float4* mm = reinterpret_cast<float4*>(m + i * 8);
    float4* mv = reinterpret_cast<float4*>(v + i * 8);
    const float4* mg = reinterpret_cast<const float4*>(grad + i * 8);
    float4 pw[2] = {mp[0], mp[1]};
    float p[8] = {pw[0].x, pw[0].y, pw[0].z, pw[0].w, pw[1].x, pw[1].y, pw[1].z, pw[1].w};
    if (!skip) {
      const float4 gw[2] = {mg[0], mg[1]};
      float4 m4[2] = {mm[0], mm[1]};
      float4 v4[2] = {mv[0], mv[1]};
      const float gq[8] = {gw[0].x, gw[0].y, gw[0].z, gw[0].w, gw[1].x, gw[1].y, gw[1].z, gw[1].w};
      float mq[8] = {m4[0].x, m4[0].y, m4[0].z, m4[0].w, m4[1].x, m4[1].y, m4[1].z, m4[1].w};
      float vq[8] = {v4[0].x, v4[0].y, v4[0].z, v4[0].w, v4[1].x, v4[1].y, v4[1].z, v4[1].w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float g = gq[j] * clip;
        mq[j] = b1 * mq[j] + (1.f - b1) * g;
        vq[j] = b2 * vq[j] + (1.f - b2) * g * g;
        p[j] = p[j] * (1.f - lr * wd) - lr * (mq[j] / bc1) / (sqrtf(vq[j] / bc2) + eps);
      }
      mm[0] = make_float4(mq[0], mq[1], mq[2], mq[3]);
      mm[1] = make_float4(mq[4], mq[5], mq[6], mq[7]);
      mv[0] = make_float4(vq[0], vq[1], vq[2], vq[3]);
      mv[1] = make_float4(vq[4], vq[5], vq[6], vq[7]);
      mp[0] = make_float4(p[0], p[1], p[2], p[3]);
      mp[1] = make_float4(p[4], p[5], p[6], p[7]);
    }
    uint4 o;
    o.x = pack_bf16x2(p[0], p[1]);
    o.y = pack_bf16x2(p[2], p[3]);
    o.z = pack_bf16x2(p[4], p[5]);
    o.w = pack_bf16x2(p[6], p[7]);
    if (mc_params != nullptr) {
      multimem_st_16B(mc_params + shard_start + i * 8, o);
    } else {
      for (int r = 0; r < world; ++r)
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.p[r]) + shard_start + i * 8) = o;
    }
  }
  __threadfence_system();
}
}  // namespace b2

static PeerPtrs peer_ptrs_of(void* const* a, int world) {
  PeerPtrs pp;
  for (int r = 0; r < 8; ++r) pp.p[r] = (a != nullptr && r < world) ? a[r] : nullptr;
  return pp;
}

// One-launch barrier over the group with a device-side epoch (see flag_barrier_kernel).  epochs: device int[channels];
// ok: device int[1], cleared on a wait that ran out.
B2_EXPORT int b2_flag_barrier(void* const* flag_bufs, const int* my_flags, int* epochs, int world, int my_rank,
                              int channels, int channel, int limit_ms, int* ok, void* stream_) {
  b2::ensure_thread_context();
  if (world < 1 || world > 8 || channel < 0 || channel >= channels) {
    set_error("flag_barrier: world in 1..8 and 0 <= channel < channels required");
    return 10;
  }
  int* status = status_ptr();
  if (!status) return 3;
  flag_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(
      peer_ptrs_of(flag_bufs, world), my_flags, epochs, world, my_rank, channels, channel,
      static_cast<unsigned long long>(limit_ms) * 1000000ull, ok, status);
  B2_LAUNCH_CHECK("flag_barrier");
  return 0;
}

// mc_bucket: multicast address of the bf16 gradient bucket (torch symmetric memory's multicast_ptr).
B2_EXPORT int b2_zero_reduce_shard_mc(const void* mc_bucket, long long shard_start, long long n, float scale,
                                      float* out, int accumulate, float* norm_sq, void* stream_) {
  b2::ensure_thread_context();
  if (mc_bucket == nullptr || (n % 8) || (shard_start % 8)) {
    set_error("zero_reduce_shard_mc: multicast pointer and 8-element aligned shard required");
    return 10;
  }
  if (n <= 0) return 0;
  zero_reduce_shard_mc_kernel<<<grid_for(n / 8, 256, 4), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const __nv_bfloat16*>(mc_bucket), shard_start, n, scale, out, accumulate, norm_sq);
  B2_LAUNCH_CHECK("zero_reduce_shard_mc");
  return 0;
}

// parts: device float[2]; slot_bufs: each rank's float[32] slot buffer; results in norm_sq[0] and grad_norm[0].
B2_EXPORT int b2_norm_allreduce(void* const* slot_bufs, const float* my_slots, void* const* flag_bufs,
                                const int* my_flags, int* epochs, int world, int my_rank, int channels, int channel,
                                const float* parts, float* norm_sq, float* grad_norm, int limit_ms, int* ok,
                                void* stream_) {
  b2::ensure_thread_context();
  if (world < 1 || world > 8 || channel < 0 || channel >= channels) {
    set_error("norm_allreduce: world in 1..8 and 0 <= channel < channels required");
    return 10;
  }
  int* status = status_ptr();
  if (!status) return 3;
  norm_allreduce_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(
      peer_ptrs_of(slot_bufs, world), my_slots, peer_ptrs_of(flag_bufs, world), my_flags, epochs, world, my_rank,
      channels, channel, parts, norm_sq, grad_norm, static_cast<unsigned long long>(limit_ms) * 1000000ull, ok, status);
  B2_LAUNCH_CHECK("norm_allreduce");
  return 0;
}

// AdamW + parameter publish; params: host array of peer pointers (plain stores) or mc_params: the bucket's multicast
// address (one store through the switch).  ok (nullable): device int, 0 skips the update.
B2_EXPORT int b2_zero_adamw_publish2(float* master, float* m, float* v, const float* grad, long long n,
                                     const float* hyper, const float* norm_sq, void* const* params, void* mc_params,
                                     int world, long long shard_start, const int* ok, void* stream_) {
  b2::ensure_thread_context();
  if (world < 1 || world > 8 || (n % 8) || (shard_start % 8) || (params == nullptr && mc_params == nullptr)) {
    set_error("zero_adamw_publish2: world in 1..8, 8-element aligned shard and a destination required");
    return 10;
  }
  if (n <= 0) return 0;
  zero_adamw_publish_any_kernel<<<grid_for(n / 8, 256, 4), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      master, m, v, grad, n, hyper, norm_sq, peer_ptrs_of(params, world), static_cast<__nv_bfloat16*>(mc_params),
      world, shard_start, ok);
  B2_LAUNCH_CHECK("zero_adamw_publish2");
  return 0;
}

namespace b2 {
// Signal every peer: flags_of_peer[r][my_rank * channels + channel] = value (system-scope release).
__global__ void flag_signal_all_kernel(PeerPtrs flag_bufs, int world, int my_rank, int channels, int channel,
                                       int value) {
  __threadfence_system();
  const int r = threadIdx.x;
  if (r < world) st_release_sys(static_cast<int*>(flag_bufs.p[r]) + my_rank * channels + channel, value);
}
// Wait until my_flags[src * channels + channel] >= value for every src, at most limit_ns.
__global__ void flag_wait_all_kernel(const int* my_flags, int world, int channels, int channel, int value,
                                     unsigned long long limit_ns, int* result, int* status) {
  const int src = threadIdx.x;
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (src < world) {
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
      if (ld_acquire_sys(my_flags + src * channels + channel) >= value) break;
      if (globaltimer_ns() - t0 > limit_ns) {
        atomicExch(&failed, 1 + src);
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (result) result[0] = failed ? 0 : 1;
    if (failed) atomicCAS(status, 0, ERR_COMM_FLAG_WAIT);
  }
}
}  // namespace b2

// flag_bufs: host array of `world` device pointers to each rank's int32 flag buffer [world * channels].
B2_EXPORT int b2_flag_signal_all(void* const* flag_bufs, int world, int my_rank, int channels, int channel,
                                 int value, void* stream_) {
  b2::ensure_thread_context();
  if (world < 1 || world > 8) { set_error("flag_signal_all: world must be 1..8"); return 10; }
  PeerPtrs pp;
  for (int r = 0; r < 8; ++r) pp.p[r] = r < world ? flag_bufs[r] : nullptr;
  flag_signal_all_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(pp, world, my_rank, channels, channel, value);
  B2_LAUNCH_CHECK("flag_signal_all");
  return 0;
}
B2_EXPORT int b2_flag_wait_all(const int* my_flags, int world, int channels, int channel, int value, int limit_ms,
                               int* result, void* stream_) {
  b2::ensure_thread_context();
  int* status = status_ptr();
  if (!status) return 3;
  flag_wait_all_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_)>>>(
      my_flags, world, channels, channel, value, static_cast<unsigned long long>(limit_ms) * 1000000ull, result, status);
  B2_LAUNCH_CHECK("flag_wait_all");
  return 0;
}
