// Batched temperature + nucleus (top-p) sampling over [B, V] logits without a sort.
//
// One CTA per row.  e_i = exp((l_i - max)/T) is a positive float, so its bit pattern orders like the
// value.  Two histogram passes over the bit pattern (12 bits each), weighted by probability mass, find
// the smallest threshold tau such that the mass of {e_i >= tau} reaches top_p * Z (24-bit resolution;
// everything inside the last sub-bin is kept).  A final pass in index order picks the token where the
// running kept mass crosses u * kept_mass.  temperature <= 0 returns the argmax.
#include "common.cuh"
#include "host.h"

namespace b2 {

constexpr int SMP_THREADS = 1024;
constexpr int SMP_BINS = 4096;

template <typename T>
__device__ __forceinline__ float ld_logit(const T* p, long long i);
template <>
__device__ __forceinline__ float ld_logit<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}

__device__ __forceinline__ float block_reduce_max(float v, float* scratch) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = threadIdx.x < 32 ? scratch[threadIdx.x] : -INFINITY;
  if (threadIdx.x < 32) t = warp_max(t);
  if (threadIdx.x == 0) scratch[0] = t;
  __syncthreads();
  t = scratch[0];
  __syncthreads();
  return t;
}
__device__ __forceinline__ float block_reduce_sum(float v, float* scratch) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = threadIdx.x < 32 ? scratch[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) t = warp_sum(t);
  if (threadIdx.x == 0) scratch[0] = t;
  __syncthreads();
  t = scratch[0];
  __syncthreads();
  return t;
}

// Walk the histogram from the top bin down until the cumulative mass reaches `target`; returns the bin
// and the mass strictly above it.  Executed by thread 0 (4096 steps worst case, shared memory).
__device__ __forceinline__ void find_bin(const float* hist, float target, int* bin_out, float* above_out) {
  float cum = 0.f;
  int b = SMP_BINS - 1;
  for (; b > 0; --b) {
    if (cum + hist[b] >= target) break;
    cum += hist[b];
  }
  *bin_out = b;
  *above_out = cum;
}

template <typename T>
__global__ void __launch_bounds__(SMP_THREADS) topp_sample_kernel(
    const T* __restrict__ logits, int V, int ld, const float* __restrict__ temperature,
    const float* __restrict__ top_p, const float* __restrict__ uniform, long long* __restrict__ out_ids,
    float* __restrict__ out_logprob) {
  __shared__ float hist[SMP_BINS];
  __shared__ float scratch[32];
  __shared__ int s_bin;
  __shared__ float s_above;
  __shared__ float s_scan[SMP_THREADS];
  __shared__ int s_pick;
  const long long row = blockIdx.x;
  const T* lr = logits + row * ld;
  const int tid = threadIdx.x;
  const float temp = temperature[row];
  const float tp = fminf(fmaxf(top_p[row], 0.f), 1.f);

  // pass 1: max (and argmax for greedy)
  float mx = -INFINITY;
  int amx = 0;
  for (int i = tid; i < V; i += SMP_THREADS) {
    const float l = ld_logit<T>(lr, i);
    if (l > mx) { mx = l; amx = i; }
  }
  const float gmax = block_reduce_max(mx, scratch);
  if (temp <= 0.f) {
    // smallest index among the maxima
    int cand = (mx == gmax) ? amx : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __shared__ int s_arg[32];
    if ((tid & 31) == 0) s_arg[tid >> 5] = cand;
    __syncthreads();
    if (tid == 0) {
      int best = s_arg[0];
      for (int w = 1; w < SMP_THREADS / 32; ++w) best = min(best, s_arg[w]);
      out_ids[row] = best;
      if (out_logprob) out_logprob[row] = 0.f;
    }
    return;
  }
  const float inv_t = 1.f / temp;
  // pass 2: Z and the coarse histogram (top 12 bits of e's pattern)
  for (int i = tid; i < SMP_BINS; i += SMP_THREADS) hist[i] = 0.f;
  __syncthreads();
  float z = 0.f;
  for (int i = tid; i < V; i += SMP_THREADS) {
    const float e = __expf((ld_logit<T>(lr, i) - gmax) * inv_t);
    z += e;
    atomicAdd(&hist[__float_as_uint(e) >> 20], e);
  }
  const float Z = block_reduce_sum(z, scratch);
  const float target = tp * Z;
  if (tid == 0) find_bin(hist, target, &s_bin, &s_above);
  __syncthreads();
  const int bin1 = s_bin;
  const float above1 = s_above;
  __syncthreads();
  // pass 3: refine inside bin1 with the next 12 bits
  for (int i = tid; i < SMP_BINS; i += SMP_THREADS) hist[i] = 0.f;
  __syncthreads();
  for (int i = tid; i < V; i += SMP_THREADS) {
    const float e = __expf((ld_logit<T>(lr, i) - gmax) * inv_t);
    const uint32_t u = __float_as_uint(e);
    if (static_cast<int>(u >> 20) == bin1) atomicAdd(&hist[(u >> 8) & 0xFFF], e);
  }
  __syncthreads();
  if (tid == 0) find_bin(hist, target - above1, &s_bin, &s_above);
  __syncthreads();
  const uint32_t tau_bits = (static_cast<uint32_t>(bin1) << 20) | (static_cast<uint32_t>(s_bin) << 8);
  __syncthreads();
  // pass 4: kept mass per thread over a contiguous index range, scan, pick
  const int per = (V + SMP_THREADS - 1) / SMP_THREADS;
  const int i0 = tid * per, i1 = min(V, i0 + per);
  float mine = 0.f;
  for (int i = i0; i < i1; ++i) {
    const float e = __expf((ld_logit<T>(lr, i) - gmax) * inv_t);
    if (__float_as_uint(e) >= tau_bits) mine += e;
  }
  s_scan[tid] = mine;
  __syncthreads();
  // inclusive scan (Hillis-Steele over 1024 entries)
  for (int o = 1; o < SMP_THREADS; o <<= 1) {
    const float add = tid >= o ? s_scan[tid - o] : 0.f;
    __syncthreads();
    s_scan[tid] += add;
    __syncthreads();
  }
  const float kept = s_scan[SMP_THREADS - 1];
  const float r = fminf(uniform[row], 0.99999994f) * kept;
  if (tid == 0) s_pick = -1;
  __syncthreads();
  const float before = s_scan[tid] - mine;
  if (mine > 0.f && r >= before && r < s_scan[tid]) {
    float run = before;
    int pick = -1, last_kept = -1;
    for (int i = i0; i < i1; ++i) {
      const float e = __expf((ld_logit<T>(lr, i) - gmax) * inv_t);
      if (__float_as_uint(e) >= tau_bits) {
        last_kept = i;
        run += e;
        if (run > r) { pick = i; break; }
      }
    }
    if (pick < 0) pick = last_kept;
    s_pick = pick;
  }
  __syncthreads();
  if (tid == 0) {
    int pick = s_pick;
    if (pick < 0) pick = amx;  // numerical corner: fall back to thread 0's best candidate
    out_ids[row] = pick;
    if (out_logprob) out_logprob[row] = (ld_logit<T>(lr, pick) - gmax) * inv_t - __logf(Z);
  }
}

}  // namespace b2

using namespace b2;

// logits [B, V] with row stride ld (fp32 or bf16); temperature / top_p / uniform: fp32 [B] on the device;
// out_ids int64 [B]; out_logprob (optional) = log-prob of the pick under the tempered full softmax.
B2_EXPORT int b2_topp_sample(const void* logits, int is_fp32, int B, int V, int ld, const float* temperature,
                             const float* top_p, const float* uniform, long long* out_ids, float* out_logprob,
                             void* stream) {
  b2::ensure_thread_context();
  if (B <= 0) return 0;
  if (is_fp32)
    topp_sample_kernel<float><<<B, SMP_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float*>(logits), V, ld, temperature, top_p, uniform, out_ids, out_logprob);
  else
    topp_sample_kernel<__nv_bfloat16><<<B, SMP_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(logits), V, ld, temperature, top_p, uniform, out_ids, out_logprob);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("topp_sample launch failed: %s", cudaGetErrorString(e));
    return 4;
  }
  return 0;
}
