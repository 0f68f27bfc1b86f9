// Batched temperature + nucleus (top-p) sampling over [B, V] logits without a sort.
//
// One CTA per row, four streaming passes over the row (served by L2 after the first), 16-byte loads
// with four in flight per thread:
//   1. online max / sum-exp of the tempered logits -> gmax, Z (greedy rows take an argmax pass and
//      return).
//   2. e_i = exp(y_i - gmax) is a positive float whose bit pattern orders like its value.  A
//      4096-bin histogram over the top 12 bits, weighted by probability mass, finds the bin in which
//      the mass of {e >= tau} reaches top_p.  Mass is accumulated as 2^40-scaled fixed point in two
//      32-bit words per bin with native integer shared-memory atomics (a float atomicAdd on shared
//      memory is a compare-and-swap loop and collapses when many lanes hit one bin); the walk over
//      the bins is a block-wide scan, not a serial loop.
//   3. the same over the next 12 bits inside that bin: 24-bit threshold tau; everything inside the
//      last sub-bin is kept.
//   4. kept mass per thread over a contiguous index range, block scan, and the thread whose range
//      contains u * kept_mass walks it to pick the token (index order, like the CPU oracle).
// temperature <= 0 returns the argmax (smallest index among equal maxima).
#include "common.cuh"
#include "host.h"

namespace b2 {

constexpr int SMP_THREADS = 1024;
constexpr int SMP_BINS = 4096;
constexpr float SMP_FIXED_ONE = 1099511627776.f;  // 2^40

template <typename T>
__device__ __forceinline__ float ld_logit(const T* p, long long i);
template <>
__device__ __forceinline__ float ld_logit<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}

template <typename T>
struct Chunk;
template <>
struct Chunk<float> {
  static constexpr int W = 4;
  __device__ static __forceinline__ void unpack(const uint4& q, float* f) {
    f[0] = __uint_as_float(q.x); f[1] = __uint_as_float(q.y);
    f[2] = __uint_as_float(q.z); f[3] = __uint_as_float(q.w);
  }
};
template <>
struct Chunk<__nv_bfloat16> {
  static constexpr int W = 8;
  __device__ static __forceinline__ void unpack(const uint4& q, float* f) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = unpack_bf16x2(w[j]);
      f[2 * j] = t.x;
      f[2 * j + 1] = t.y;
    }
  }
};

// fn(first_index, values, count): strided over the block (chunk c -> thread c % SMP_THREADS).
template <typename T, bool VEC, typename F>
__device__ __forceinline__ void scan_strided(const T* lr, int V, F&& fn) {
  if constexpr (VEC) {
    constexpr int W = Chunk<T>::W;
    const int nch = V / W;
    const uint4* p = reinterpret_cast<const uint4*>(lr);
    for (int c = threadIdx.x; c < nch; c += 4 * SMP_THREADS) {
      uint4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (c + u * SMP_THREADS < nch) q[u] = p[c + u * SMP_THREADS];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int cc = c + u * SMP_THREADS;
        if (cc < nch) {
          float f[W];
          Chunk<T>::unpack(q[u], f);
          fn(cc * W, f, W);
        }
      }
    }
  } else {
    for (int i = threadIdx.x; i < V; i += SMP_THREADS) {
      const float f = ld_logit<T>(lr, i);
      fn(i, &f, 1);
    }
  }
}
// fn over the contiguous range [i0, i1) (i0 a multiple of the chunk width when VEC).
template <typename T, bool VEC, typename F>
__device__ __forceinline__ void scan_range(const T* lr, int i0, int i1, F&& fn) {
  if constexpr (VEC) {
    constexpr int W = Chunk<T>::W;
    const uint4* p = reinterpret_cast<const uint4*>(lr);
    for (int i = i0; i < i1; i += 4 * W) {
      uint4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i + u * W < i1) q[u] = p[(i + u * W) / W];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i + u * W < i1) {
          float f[W];
          Chunk<T>::unpack(q[u], f);
          fn(i + u * W, f, W);
        }
    }
  } else {
    for (int i = i0; i < i1; ++i) {
      const float f = ld_logit<T>(lr, i);
      fn(i, &f, 1);
    }
  }
}

__device__ __forceinline__ void hist_add(uint32_t* lo, uint32_t* hi, int bin, unsigned long long x) {
  const uint32_t xl = static_cast<uint32_t>(x);
  uint32_t xh = static_cast<uint32_t>(x >> 32);
  if (xl) {
    const uint32_t old = atomicAdd(&lo[bin], xl);
    xh += (old + xl) < xl ? 1u : 0u;  // carry out of the low word
  }
  if (xh) atomicAdd(&hi[bin], xh);
}

// Walk the bins from the top down until the cumulative mass reaches `target` (>= 1): the bin where
// it does, and the mass strictly above that bin.  All SMP_THREADS threads take part; thread t owns
// bins 4095-4t .. 4092-4t.  Results land in *bin_out / *above_out (shared memory) after the final
// barrier.
__device__ __forceinline__ void find_bin(const uint32_t* lo, const uint32_t* hi, unsigned long long target,
                                         unsigned long long* wsum, int* bin_out,
                                         unsigned long long* above_out, unsigned long long* total_out) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned long long own[4], mine = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int b = SMP_BINS - 1 - 4 * tid - k;
    own[k] = (static_cast<unsigned long long>(hi[b]) << 32) + lo[b];
    mine += own[k];
  }
  unsigned long long incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) wsum[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const unsigned long long w = wsum[lane];
    unsigned long long wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    wsum[lane] = wi - w;  // exclusive prefix of the warp totals
    if (lane == 31 && total_out) *total_out = wi;
  }
  __syncthreads();
  const unsigned long long excl = wsum[warp] + incl - mine;
  if (excl < target && target <= excl + mine) {
    unsigned long long cum = excl;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (cum + own[k] >= target) {
        *bin_out = SMP_BINS - 1 - 4 * tid - k;
        *above_out = cum;
        break;
      }
      cum += own[k];
    }
  }
  __syncthreads();
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(SMP_THREADS) topp_sample_kernel(
    const T* __restrict__ logits, int V, int ld, const float* __restrict__ temperature,
    const float* __restrict__ top_p, const float* __restrict__ uniform, long long* __restrict__ out_ids,
    float* __restrict__ out_logprob) {
  __shared__ uint32_t hist_lo[SMP_BINS];
  __shared__ uint32_t hist_hi[SMP_BINS];
  __shared__ unsigned long long s_wsum[32];
  __shared__ float s_f[64];
  __shared__ int s_i[32];
  __shared__ int s_bin;
  __shared__ unsigned long long s_above, s_total;
  __shared__ int s_pick;
  const long long row = blockIdx.x;
  const T* lr = logits + row * ld;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float temp = temperature[row];
  const float tp = fminf(fmaxf(top_p[row], 0.f), 1.f);

  if (temp <= 0.f) {
    float mx = -INFINITY;
    int amx = 0x7fffffff;
    scan_strided<T, VEC>(lr, V, [&](int i0, const float* f, int n) {
      for (int i = 0; i < n; ++i)
        if (f[i] > mx) { mx = f[i]; amx = i0 + i; }
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, mx, o);
      const int oi = __shfl_xor_sync(0xffffffffu, amx, o);
      if (om > mx || (om == mx && oi < amx)) { mx = om; amx = oi; }
    }
    if (lane == 0) { s_f[warp] = mx; s_i[warp] = amx; }
    __syncthreads();
    if (tid == 0) {
      float bm = s_f[0];
      int bi = s_i[0];
      for (int w = 1; w < SMP_THREADS / 32; ++w)
        if (s_f[w] > bm || (s_f[w] == bm && s_i[w] < bi)) { bm = s_f[w]; bi = s_i[w]; }
      out_ids[row] = bi == 0x7fffffff ? 0 : bi;
      if (out_logprob) out_logprob[row] = 0.f;
    }
    return;
  }

  const float inv_t = 1.f / temp;
  // pass 1: online max and sum of exp over the tempered logits
  float m = -INFINITY, z = 0.f;
  scan_strided<T, VEC>(lr, V, [&](int, const float* f, int n) {
    float cm = f[0] * inv_t;
    for (int i = 1; i < n; ++i) cm = fmaxf(cm, f[i] * inv_t);
    const float nm = fmaxf(m, cm);
    if (nm == -INFINITY) return;
    float acc = z * __expf(m - nm);
    for (int i = 0; i < n; ++i) acc += __expf(f[i] * inv_t - nm);
    z = acc;
    m = nm;
  });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const float oz = __shfl_xor_sync(0xffffffffu, z, o);
    const float nm = fmaxf(m, om);
    z = nm == -INFINITY ? 0.f : z * __expf(m - nm) + oz * __expf(om - nm);
    m = nm;
  }
  if (lane == 0) { s_f[warp] = m; s_f[32 + warp] = z; }
  for (int i = tid; i < SMP_BINS; i += SMP_THREADS) { hist_lo[i] = 0; hist_hi[i] = 0; }
  if (tid == 0) { s_bin = 0; s_above = 0; s_pick = -1; }
  __syncthreads();
  float gmax = s_f[0];
  for (int w = 1; w < 32; ++w) gmax = fmaxf(gmax, s_f[w]);
  float Z = 0.f;
  for (int w = 0; w < 32; ++w) Z += s_f[w] == -INFINITY ? 0.f : s_f[32 + w] * __expf(s_f[w] - gmax);
  const float kscale = SMP_FIXED_ONE / Z;

  // pass 2: coarse histogram (top 12 bits of e's pattern), mass in fixed point
  scan_strided<T, VEC>(lr, V, [&](int, const float* f, int n) {
    for (int i = 0; i < n; ++i) {
      const float e = __expf(f[i] * inv_t - gmax);
      const unsigned long long x = __float2ull_rz(e * kscale);
      if (x) hist_add(hist_lo, hist_hi, __float_as_uint(e) >> 20, x);
    }
  });
  __syncthreads();
  find_bin(hist_lo, hist_hi, ~0ull, s_wsum, &s_bin, &s_above, &s_total);  // only the total (no bin reaches 2^64-1)
  const unsigned long long total = s_total;
  unsigned long long target = static_cast<unsigned long long>(static_cast<double>(tp) * static_cast<double>(total));
  target = target < 1 ? 1 : (target > total ? total : target);
  find_bin(hist_lo, hist_hi, target, s_wsum, &s_bin, &s_above, nullptr);
  const int bin1 = s_bin;
  const unsigned long long above1 = s_above;
  __syncthreads();
  // pass 3: refine inside bin1 with the next 12 bits
  for (int i = tid; i < SMP_BINS; i += SMP_THREADS) { hist_lo[i] = 0; hist_hi[i] = 0; }
  if (tid == 0) { s_bin = 0; s_above = 0; }
  __syncthreads();
  scan_strided<T, VEC>(lr, V, [&](int, const float* f, int n) {
    for (int i = 0; i < n; ++i) {
      const float e = __expf(f[i] * inv_t - gmax);
      const uint32_t u = __float_as_uint(e);
      if (static_cast<int>(u >> 20) == bin1) {
        const unsigned long long x = __float2ull_rz(e * kscale);
        if (x) hist_add(hist_lo, hist_hi, (u >> 8) & 0xFFF, x);
      }
    }
  });
  __syncthreads();
  find_bin(hist_lo, hist_hi, target - above1, s_wsum, &s_bin, &s_above, nullptr);
  const uint32_t tau_bits = (static_cast<uint32_t>(bin1) << 20) | (static_cast<uint32_t>(s_bin) << 8);

  // pass 4: kept mass per thread over a contiguous index range, block scan, pick
  constexpr int W = VEC ? Chunk<T>::W : 1;
  int per = (V + SMP_THREADS - 1) / SMP_THREADS;
  per = (per + 4 * W - 1) / (4 * W) * (4 * W);
  const int i0 = min(V, tid * per), i1 = min(V, i0 + per);
  float mine = 0.f;
  scan_range<T, VEC>(lr, i0, i1, [&](int, const float* f, int n) {
    for (int i = 0; i < n; ++i) {
      const float e = __expf(f[i] * inv_t - gmax);
      if (__float_as_uint(e) >= tau_bits) mine += e;
    }
  });
  float incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  __syncthreads();
  if (lane == 31) s_f[warp] = incl;
  __syncthreads();
  float wpre = 0.f, kept = 0.f;
  for (int w = 0; w < 32; ++w) {
    if (w < warp) wpre += s_f[w];
    kept += s_f[w];
  }
  incl += wpre;
  const float before = incl - mine;
  const float r = fminf(uniform[row], 0.99999994f) * kept;
  auto walk = [&](float limit) {
    float run = before;
    int pick = -1, last_kept = -1;
    for (int i = i0; i < i1 && pick < 0; ++i) {
      const float e = __expf(ld_logit<T>(lr, i) * inv_t - gmax);
      if (__float_as_uint(e) >= tau_bits) {
        last_kept = i;
        run += e;
        if (run > limit) pick = i;
      }
    }
    return pick >= 0 ? pick : last_kept;
  };
  if (mine > 0.f && r >= before && r < incl) atomicMax(&s_pick, walk(r));
  __syncthreads();
  // every thread takes its own copy before anyone may write again: branching on the shared word itself would
  // let a late thread see a neighbour's fallback write and skip the barrier below
  const bool need_fallback = s_pick < 0;
  __syncthreads();
  // numerical corner (r rounded up to the kept mass): the last kept token
  if (need_fallback && mine > 0.f) atomicMax(&s_pick, walk(INFINITY));
  __syncthreads();
  if (tid == 0) {
    const int pick = max(s_pick, 0);
    out_ids[row] = pick;
    if (out_logprob) out_logprob[row] = ld_logit<T>(lr, pick) * inv_t - gmax - __logf(Z);
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
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t esz = is_fp32 ? 4 : 2;
  // 16-byte loads need every row to start on a 16-byte boundary and to hold whole chunks
  const bool vec = (reinterpret_cast<uintptr_t>(logits) % 16 == 0) && ((static_cast<size_t>(ld) * esz) % 16 == 0) &&
                   ((static_cast<size_t>(V) * esz) % 16 == 0);
  if (is_fp32) {
    const float* p = static_cast<const float*>(logits);
    if (vec) topp_sample_kernel<float, true><<<B, SMP_THREADS, 0, st>>>(p, V, ld, temperature, top_p, uniform, out_ids, out_logprob);
    else topp_sample_kernel<float, false><<<B, SMP_THREADS, 0, st>>>(p, V, ld, temperature, top_p, uniform, out_ids, out_logprob);
  } else {
    const __nv_bfloat16* p = static_cast<const __nv_bfloat16*>(logits);
    if (vec) topp_sample_kernel<__nv_bfloat16, true><<<B, SMP_THREADS, 0, st>>>(p, V, ld, temperature, top_p, uniform, out_ids, out_logprob);
    else topp_sample_kernel<__nv_bfloat16, false><<<B, SMP_THREADS, 0, st>>>(p, V, ld, temperature, top_p, uniform, out_ids, out_logprob);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("topp_sample launch failed: %s", cudaGetErrorString(e));
    return 4;
  }
  return 0;
}
