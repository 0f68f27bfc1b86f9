// Vocabulary-row kernels for the fused LM-head loss (cross-entropy and token log-prob, forward and
// in-place backward over a chunk of logits), the GRPO token loss, and the flat-buffer optimizer
// kernels (sum of squares / non-finite scan, fused AdamW with clip + unscale, casts).
#include "common.cuh"
#include "host.h"

namespace b2 {

constexpr int ROW_THREADS = 1024;

struct MaxSum {
  float m, s;
};
__device__ __forceinline__ MaxSum combine(MaxSum a, MaxSum b) {
  MaxSum r;
  r.m = fmaxf(a.m, b.m);
  r.s = (a.m == -INFINITY ? 0.f : a.s * __expf(a.m - r.m)) + (b.m == -INFINITY ? 0.f : b.s * __expf(b.m - r.m));
  return r;
}
__device__ __forceinline__ MaxSum block_maxsum(MaxSum v, MaxSum* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum t;
    t.m = __shfl_xor_sync(0xffffffffu, v.m, o);
    t.s = __shfl_xor_sync(0xffffffffu, v.s, o);
    v = combine(v, t);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  MaxSum t = (lane < (blockDim.x >> 5)) ? scratch[lane] : MaxSum{-INFINITY, 0.f};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum u;
    u.m = __shfl_xor_sync(0xffffffffu, t.m, o);
    u.s = __shfl_xor_sync(0xffffffffu, t.s, o);
    t = combine(t, u);
  }
  return t;
}

// mode 0: cross-entropy forward + in-place backward.  dlogits = coef*(softmax - onehot) with
//         coef = *scale for rows whose label != ignore (else 0); loss_sum += (lse - logit[label]).
// mode 1: log-prob forward only: lse_out[row], logp_out[row] (0 for ignored rows).
// mode 2: log-prob backward in place: dlogits = g[row] * (onehot - softmax), using lse_in[row].
// mode 3: vocabulary-sharded pass 1: stats_out[row] = {max, sum exp(x - max), label logit or 0} of
//         this shard's columns [vocab_start, vocab_start + V) of a vocab_total-wide row.
// mode 4: vocabulary-sharded CE backward in place with the row's global lse given in lse_io.
// Modes 2 and 4 accept a shard (labels are global ids; the one-hot lands only in its owner).
// logits: [rows, ld] bf16, V valid columns (V % 8 == 0).  labels int64.
__global__ void __launch_bounds__(ROW_THREADS) vocab_rows_kernel(
    __nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels, int V, int ld, int mode,
    const float* __restrict__ scale, float* __restrict__ loss_sum, float* __restrict__ lse_io,
    float* __restrict__ logp_out, const float* __restrict__ g_in, long long ignore_index,
    float inv_temperature, long long vocab_start, long long vocab_total, float* __restrict__ stats_out) {
  __shared__ MaxSum scratch[32];
  const size_t row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  // labels index the whole vocabulary; this launch sees columns [vocab_start, vocab_start + V) of it
  const long long label_global = labels[row];
  const bool valid = label_global != ignore_index && label_global >= 0 && label_global < vocab_total;
  const long long label = label_global - vocab_start;
  const bool in_shard = valid && label >= 0 && label < V;
  const int nvec = V / 8;
  float lse;
  if (mode == 0 || mode == 1 || mode == 3) {
    MaxSum ms{-INFINITY, 0.f};
    for (int c = threadIdx.x; c < nvec; c += ROW_THREADS) {
      uint4 q = *reinterpret_cast<const uint4*>(lr + c * 8);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      float f[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 t = unpack_bf16x2(w[j]);
        f[2 * j] = t.x * inv_temperature;
        f[2 * j + 1] = t.y * inv_temperature;
      }
      float m = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) m = fmaxf(m, f[j]);
      const float nm = fmaxf(ms.m, m);
      float s = ms.m == -INFINITY ? 0.f : ms.s * __expf(ms.m - nm);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += __expf(f[j] - nm);
      ms.m = nm;
      ms.s = s;
    }
    ms = block_maxsum(ms, scratch);
    if (mode == 3) {
      // vocabulary-sharded pass 1: this shard's (max, sum exp(x - max), label logit or 0); the caller
      // combines the shards' triples into the row's log-sum-exp.
      if (threadIdx.x == 0) {
        stats_out[row * 3 + 0] = ms.m;
        stats_out[row * 3 + 1] = ms.s;
        stats_out[row * 3 + 2] = in_shard ? __bfloat162float(lr[label]) * inv_temperature : 0.f;
      }
      return;
    }
    lse = ms.m + __logf(ms.s);
  } else {
    lse = lse_io[row];
  }
  const float label_logit = in_shard ? __bfloat162float(lr[label]) * inv_temperature : 0.f;
  if (mode == 1) {
    if (threadIdx.x == 0) {
      lse_io[row] = lse;
      logp_out[row] = valid ? label_logit - lse : 0.f;
    }
    return;
  }
  float coef;
  if (mode == 0) {
    coef = valid ? *scale : 0.f;
    if (threadIdx.x == 0 && valid) atomicAdd(loss_sum, lse - label_logit);
  } else if (mode == 4) {
    coef = valid ? *scale : 0.f;  // sharded CE: the loss itself was summed by the caller
  } else {
    coef = valid ? -g_in[row] : 0.f;  // dlogits = g*(onehot - softmax) = (-g)*(softmax - onehot)
  }
  coef *= inv_temperature;
  __syncthreads();  // every thread has read lr[label] before anyone overwrites it
  for (int c = threadIdx.x; c < nvec; c += ROW_THREADS) {
    uint4 q = *reinterpret_cast<const uint4*>(lr + c * 8);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = unpack_bf16x2(w[j]);
      f[2 * j] = coef * __expf(t.x * inv_temperature - lse);
      f[2 * j + 1] = coef * __expf(t.y * inv_temperature - lse);
    }
    if (in_shard && label >= c * 8 && label < c * 8 + 8) f[label - c * 8] -= coef;
    uint4 o;
    o.x = pack_bf16x2(f[0], f[1]);
    o.y = pack_bf16x2(f[2], f[3]);
    o.z = pack_bf16x2(f[4], f[5]);
    o.w = pack_bf16x2(f[6], f[7]);
    *reinterpret_cast<uint4*>(lr + c * 8) = o;
  }
}

// ---------------------------------------------------------------------------------------------
// GRPO token loss (clipped surrogate + KL to a frozen reference), forward and gradient w.r.t. the
// token log-probs, same formula as the reference (src/engines/train_engine.py:1409-1433):
//   ratio = exp(lp - old); loss_tok = -min(ratio*A, clamp(ratio,1-e,1+e)*A) * mask
//   policy = sum(loss_tok)/(sum(mask)+1e-8); kl = max(0, sum((lp-ref)*mask)/(sum(mask)+1e-8))
// Pass 1 accumulates {sum loss_tok, sum mask, sum (lp-ref)*mask, sum ratio*mask, clipped count, max
// ratio, min ratio} into stats[8]; pass 2 writes g = dLoss/dlp.
// ---------------------------------------------------------------------------------------------
__global__ void grpo_stats_kernel(const float* __restrict__ lp, const float* __restrict__ old_lp,
                                  const float* __restrict__ ref_lp, const float* __restrict__ mask,
                                  const float* __restrict__ adv, int rows, int cols, float clip_eps,
                                  float* __restrict__ stats) {
  float s_loss = 0.f, s_mask = 0.f, s_kl = 0.f, s_ratio = 0.f, s_clip = 0.f;
  float rmax = -INFINITY, rmin = INFINITY;
  const long long total = static_cast<long long>(rows) * cols;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float m = mask[i];
    if (m == 0.f) continue;
    const float a = adv[i / cols];
    const float ratio = __expf(lp[i] - old_lp[i]);
    const float clipped = fminf(fmaxf(ratio, 1.f - clip_eps), 1.f + clip_eps);
    s_loss += -fminf(ratio * a, clipped * a) * m;
    s_mask += m;
    if (ref_lp) s_kl += (lp[i] - ref_lp[i]) * m;
    s_ratio += ratio * m;
    s_clip += fabsf(ratio - 1.f) > clip_eps ? 1.f : 0.f;
    rmax = fmaxf(rmax, ratio);
    rmin = fminf(rmin, ratio);
  }
  s_loss = warp_sum(s_loss);
  s_mask = warp_sum(s_mask);
  s_kl = warp_sum(s_kl);
  s_ratio = warp_sum(s_ratio);
  s_clip = warp_sum(s_clip);
  rmax = warp_max(rmax);
  rmin = -warp_max(-rmin);
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(stats + 0, s_loss);
    atomicAdd(stats + 1, s_mask);
    atomicAdd(stats + 2, s_kl);
    atomicAdd(stats + 3, s_ratio);
    atomicAdd(stats + 4, s_clip);
    // float max/min through int ordering (ratios are positive)
    if (rmax > 0.f) atomicMax(reinterpret_cast<int*>(stats + 5), __float_as_int(rmax));
    if (rmin < INFINITY) atomicMin(reinterpret_cast<int*>(stats + 6), __float_as_int(rmin));
  }
}
__global__ void grpo_grad_kernel(const float* __restrict__ lp, const float* __restrict__ old_lp,
                                 const float* __restrict__ mask, const float* __restrict__ adv, int rows,
                                 int cols, float clip_eps, float beta, int has_ref,
                                 const float* __restrict__ stats, float loss_scale,
                                 float* __restrict__ g_out) {
  const float denom = stats[1] + 1e-8f;
  const float kl_mean = stats[2] / denom;
  const float kl_coef = (has_ref && beta > 0.f && kl_mean > 0.f) ? beta / denom : 0.f;
  const long long total = static_cast<long long>(rows) * cols;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float m = mask[i];
    float g = 0.f;
    if (m != 0.f) {
      const float a = adv[i / cols];
      const float ratio = __expf(lp[i] - old_lp[i]);
      const float clipped = fminf(fmaxf(ratio, 1.f - clip_eps), 1.f + clip_eps);
      // d/dlp of -min(ratio*a, clipped*a): the unclipped branch is active when it is the smaller
      // one (ties go to the unclipped branch, as torch.min's gradient does for equal inputs split);
      // the clipped branch has zero gradient whenever the clamp is saturated.
      const float s1 = ratio * a, s2 = clipped * a;
      float d = 0.f;
      if (s1 <= s2) d = ratio * a;
      else if (clipped == ratio) d = ratio * a;
      g = (-d / denom + kl_coef) * m * loss_scale;
    }
    g_out[i] = g;
  }
}

// ---------------------------------------------------------------------------------------------
// Flat-buffer optimizer kernels.
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// out[0] += sum(x^2) (NaN/Inf propagate, so one scalar doubles as the non-finite check).
template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ x, long long n, float* __restrict__ out) {
  float s = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = to_f<T>(x[i]);
    s += v * v;
  }
  __shared__ float scratch[32];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? scratch[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) atomicAdd(out, t);
  }
}

// Fused AdamW on an fp32 master shard.
//   g = grad * grad_scale * clip,  clip = min(1, max_norm / (sqrt(norm_sq[0]) + 1e-6))  (max_norm <= 0: off)
//   skipped entirely when norm_sq[0] is not finite (the caller then also does not advance its step).
//   Writes the updated parameter as bf16 (param_out) when given.  hyper = {lr, beta1, beta2, eps,
//   weight_decay, bias_correction1, bias_correction2, max_norm} lives in device memory so that the
//   launch can be captured in a CUDA graph while the host advances the schedule.
template <typename G>
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                             const G* __restrict__ grad, __nv_bfloat16* __restrict__ param_out,
                             long long n, const float* __restrict__ hyper,
                             const float* __restrict__ norm_sq, float grad_scale) {
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd = hyper[4];
  const float bc1 = hyper[5], bc2 = hyper[6], max_norm = hyper[7];
  float clip = 1.f;
  if (norm_sq != nullptr) {
    const float ns = norm_sq[0];
    if (!isfinite(ns)) return;
    if (max_norm > 0.f) clip = fminf(1.f, max_norm / (sqrtf(ns) + 1e-6f));
  }
  const float gs = grad_scale * clip;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float g = to_f<G>(grad[i]) * gs;
    float p = master[i];
    const float mi = b1 * m[i] + (1.f - b1) * g;
    const float vi = b2 * v[i] + (1.f - b2) * g * g;
    m[i] = mi;
    v[i] = vi;
    p = p * (1.f - lr * wd) - lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    master[i] = p;
    if (param_out) param_out[i] = __float2bfloat16(p);
  }
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                        long long n, float scale) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = __float2bfloat16(src[i] * scale);
}
__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst,
                                        long long n, float scale, int accumulate) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = __bfloat162float(src[i]) * scale;
    dst[i] = accumulate ? dst[i] + v : v;
  }
}

}  // namespace b2

using namespace b2;

#define B2_LAUNCH_CHECK(name)                                        \
  do {                                                               \
    cudaError_t e_ = cudaGetLastError();                             \
    if (e_ != cudaSuccess) {                                         \
      set_error(name " launch failed: %s", cudaGetErrorString(e_)); \
      return 4;                                                      \
    }                                                                \
  } while (0)

static int grid_for(long long n, int threads) {
  long long b = (n + threads - 1) / threads;
  const long long cap = static_cast<long long>(num_sms()) * 8;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

B2_EXPORT int b2_vocab_rows(void* logits, const long long* labels, int rows, int V, int ld, int mode,
                            const float* scale, float* loss_sum, float* lse, float* logp,
                            const float* g, long long ignore_index, float inv_temperature,
                            long long vocab_start, long long vocab_total, float* stats, void* stream) {
  b2::ensure_thread_context();
  if (V % 8 || ld % 8) { set_error("vocab_rows: V and ld must be multiples of 8"); return 10; }
  if (mode < 0 || mode > 4 || (mode == 3 && !stats) || ((mode == 2 || mode == 4) && !lse)) {
    set_error("vocab_rows: bad mode or missing buffer");
    return 11;
  }
  if (rows <= 0) return 0;
  if (vocab_total <= 0) vocab_total = V;
  vocab_rows_kernel<<<rows, ROW_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(logits), labels, V, ld, mode, scale, loss_sum, lse, logp, g,
      ignore_index, inv_temperature, vocab_start, vocab_total, stats);
  B2_LAUNCH_CHECK("vocab_rows");
  return 0;
}

// stats: fp32[8], caller-zeroed except stats[6] which must start at +inf (min ratio).
B2_EXPORT int b2_grpo_loss(const float* lp, const float* old_lp, const float* ref_lp, const float* mask,
                           const float* adv, int rows, int cols, float clip_eps, float beta,
                           float loss_scale, float* stats, float* g_out, void* stream_) {
  b2::ensure_thread_context();
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long total = static_cast<long long>(rows) * cols;
  if (total <= 0) return 0;
  grpo_stats_kernel<<<grid_for(total, 256), 256, 0, stream>>>(lp, old_lp, ref_lp, mask, adv, rows, cols,
                                                             clip_eps, stats);
  B2_LAUNCH_CHECK("grpo_stats");
  if (g_out) {
    grpo_grad_kernel<<<grid_for(total, 256), 256, 0, stream>>>(lp, old_lp, mask, adv, rows, cols, clip_eps,
                                                              beta, ref_lp != nullptr, stats, loss_scale,
                                                              g_out);
    B2_LAUNCH_CHECK("grpo_grad");
  }
  return 0;
}

B2_EXPORT int b2_sumsq(const void* x, long long n, int is_fp32, float* out, void* stream) {
  b2::ensure_thread_context();
  if (n <= 0) return 0;
  if (is_fp32)
    sumsq_kernel<float><<<grid_for(n, 512), 512, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float*>(x), n, out);
  else
    sumsq_kernel<__nv_bfloat16><<<grid_for(n, 512), 512, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), n, out);
  B2_LAUNCH_CHECK("sumsq");
  return 0;
}

B2_EXPORT int b2_adamw(float* master, float* m, float* v, const void* grad, int grad_fp32, void* param_out,
                       long long n, const float* hyper, const float* norm_sq, float grad_scale,
                       void* stream) {
  b2::ensure_thread_context();
  if (n <= 0) return 0;
  if (grad_fp32)
    adamw_kernel<float><<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        master, m, v, static_cast<const float*>(grad), static_cast<__nv_bfloat16*>(param_out), n, hyper,
        norm_sq, grad_scale);
  else
    adamw_kernel<__nv_bfloat16><<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        master, m, v, static_cast<const __nv_bfloat16*>(grad), static_cast<__nv_bfloat16*>(param_out), n,
        hyper, norm_sq, grad_scale);
  B2_LAUNCH_CHECK("adamw");
  return 0;
}

B2_EXPORT int b2_cast_f32_to_bf16(const float* src, void* dst, long long n, float scale, void* stream) {
  b2::ensure_thread_context();
  if (n <= 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, static_cast<__nv_bfloat16*>(dst), n, scale);
  B2_LAUNCH_CHECK("cast_f32_to_bf16");
  return 0;
}
B2_EXPORT int b2_cast_bf16_to_f32(const void* src, float* dst, long long n, float scale, int accumulate,
                                  void* stream) {
  b2::ensure_thread_context();
  if (n <= 0) return 0;
  cast_bf16_to_f32_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), dst, n, scale, accumulate);
  B2_LAUNCH_CHECK("cast_bf16_to_f32");
  return 0;
}
