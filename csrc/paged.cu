// Paged KV-cache kernels: block-segment KV store (bf16 and fp8-e4m3 with one scale per block and kv
// head), gather / dequantise into contiguous bf16, paged decode attention with split-KV partitions
// and the exact log-sum-exp merge.
//
// Cache layout for one layer and one of {K, V}: [num_blocks, 16 tokens, Hkv, 128] (bf16 or fp8 bytes);
// scales [num_blocks, Hkv] fp32 (value = stored * scale).
#include <cuda_fp8.h>

#include "common.cuh"
#include "host.h"

namespace b2 {

constexpr int PAGE = 16;
constexpr int HD = 128;
constexpr float FP8_MAX = 448.f;

__device__ __forceinline__ float fp8_to_float(uint8_t v) {
  __nv_fp8_e4m3 t;
  t.__x = v;
  return static_cast<float>(t);
}
__device__ __forceinline__ uint8_t float_to_fp8(float v) {
  __nv_fp8_e4m3 t(v);
  return t.__x;
}

// ---------------------------------------------------------------------------------------------
// KV store.  A segment is a run of `count` consecutive new tokens (rows tok0.. of k / v) that land in
// one cache block starting at slot `off`: seg = {block, tok0, count, off}.  Grid (nseg, Hkv, 2) —
// z = 0 stores K, z = 1 stores V; 128 threads = one per head dimension.
// fp8: the block's scale only ever grows; when a new token raises it, the tokens already in the block
// are requantised by the same CTA (a block's tail is owned by one sequence, so no one else writes it).
// ---------------------------------------------------------------------------------------------
template <bool FP8>
__global__ void __launch_bounds__(128) kv_store_kernel(
    const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v, int ld_k, int ld_v,
    void* __restrict__ k_cache, void* __restrict__ v_cache, float* __restrict__ k_scale,
    float* __restrict__ v_scale, const int* __restrict__ segs, int Hkv) {
  __shared__ float red[4];
  const int seg = blockIdx.x, h = blockIdx.y, which = blockIdx.z;
  const int block = segs[seg * 4 + 0], tok0 = segs[seg * 4 + 1], count = segs[seg * 4 + 2],
            off = segs[seg * 4 + 3];
  if (block < 0 || count <= 0) return;
  const __nv_bfloat16* src = which ? v : k;
  const int ld = which ? ld_v : ld_k;
  const int d = threadIdx.x;
  const size_t base = (static_cast<size_t>(block) * PAGE) * Hkv * HD + static_cast<size_t>(h) * HD + d;
  const size_t tok_stride = static_cast<size_t>(Hkv) * HD;
  if (!FP8) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(which ? v_cache : k_cache);
    for (int t = 0; t < count; ++t)
      dst[base + (off + t) * tok_stride] = src[static_cast<size_t>(tok0 + t) * ld + h * HD + d];
    return;
  }
  uint8_t* dst = reinterpret_cast<uint8_t*>(which ? v_cache : k_cache);
  float* scale_p = (which ? v_scale : k_scale) + static_cast<size_t>(block) * Hkv + h;
  float vals[PAGE];
  float amax = 0.f;
  for (int t = 0; t < count; ++t) {
    vals[t] = __bfloat162float(src[static_cast<size_t>(tok0 + t) * ld + h * HD + d]);
    amax = fmaxf(amax, fabsf(vals[t]));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  const float old_scale = off > 0 ? *scale_p : 0.f;
  float new_scale = fmaxf(old_scale, amax / FP8_MAX);
  if (new_scale <= 0.f) new_scale = 1.f / FP8_MAX;
  if (off > 0 && new_scale > old_scale) {
    const float r = old_scale / new_scale;
    for (int t = 0; t < off; ++t) {
      const size_t a = base + t * tok_stride;
      dst[a] = float_to_fp8(fp8_to_float(dst[a]) * r);
    }
  }
  const float inv = 1.f / new_scale;
  for (int t = 0; t < count; ++t) dst[base + (off + t) * tok_stride] = float_to_fp8(vals[t] * inv);
  __syncthreads();
  if (threadIdx.x == 0) *scale_p = new_scale;
}

// ---------------------------------------------------------------------------------------------
// Gather cache rows into contiguous bf16 K / V [rows, Hkv*128]; slot[r] = block*16 + offset.
// ---------------------------------------------------------------------------------------------
template <bool FP8>
__global__ void kv_gather_kernel(const void* __restrict__ k_cache, const void* __restrict__ v_cache,
                                 const float* __restrict__ k_scale, const float* __restrict__ v_scale,
                                 const int* __restrict__ slot, __nv_bfloat16* __restrict__ k_out,
                                 __nv_bfloat16* __restrict__ v_out, int rows, int Hkv) {
  const int W = Hkv * HD;
  const long long total = static_cast<long long>(rows) * W;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / W), c = static_cast<int>(i % W);
    const int s = slot[r];
    const size_t a = static_cast<size_t>(s) * W + c;
    if (FP8) {
      const size_t sc = static_cast<size_t>(s / PAGE) * Hkv + c / HD;
      k_out[i] = __float2bfloat16(fp8_to_float(reinterpret_cast<const uint8_t*>(k_cache)[a]) * k_scale[sc]);
      v_out[i] = __float2bfloat16(fp8_to_float(reinterpret_cast<const uint8_t*>(v_cache)[a]) * v_scale[sc]);
    } else {
      k_out[i] = reinterpret_cast<const __nv_bfloat16*>(k_cache)[a];
      v_out[i] = reinterpret_cast<const __nv_bfloat16*>(v_cache)[a];
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Paged decode attention: one query token per sequence.  Grid (B, Hkv, nsplit); a CTA streams its
// partition of the sequence's pages (64 tokens per step through shared memory), scores all G = Hq/Hkv
// query heads of its kv head, and keeps an online softmax.  nsplit == 1 writes the output directly;
// otherwise unnormalised partials + (max, sum) go to a workspace for the merge kernel.
// ---------------------------------------------------------------------------------------------
constexpr int DEC_THREADS = 128;
constexpr int DEC_CHUNK = 64;
constexpr int DEC_MAX_G = 8;

template <bool FP8>
__global__ void __launch_bounds__(DEC_THREADS) paged_decode_kernel(
    const __nv_bfloat16* __restrict__ q, const void* __restrict__ k_cache, const void* __restrict__ v_cache,
    const float* __restrict__ k_scale, const float* __restrict__ v_scale,
    const int* __restrict__ block_tables, const int* __restrict__ context_lens, int max_blocks,
    __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, int Hq, int Hkv,
    int partition, float scale) {
  constexpr int ESZ = FP8 ? 1 : 2;
  constexpr int ROW = HD * ESZ + 16;  // padded row: conflict-free 16-byte reads across rows
  __shared__ __align__(16) uint8_t sK[DEC_CHUNK * ROW];
  __shared__ __align__(16) uint8_t sV[DEC_CHUNK * ROW];
  __shared__ float sQ[DEC_MAX_G][HD];
  __shared__ float sS[DEC_MAX_G][DEC_CHUNK];
  __shared__ float sM[DEC_MAX_G], sL[DEC_MAX_G], sAlpha[DEC_MAX_G];
  __shared__ float sKs[DEC_CHUNK / PAGE], sVs[DEC_CHUNK / PAGE];

  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z, nsplit = gridDim.z;
  const int G = Hq / Hkv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ctx = context_lens[b];
  const int t_begin = split * partition;
  const int t_end = min(ctx, t_begin + partition);
  const int* table = block_tables + static_cast<size_t>(b) * max_blocks;
  const size_t tok_stride = static_cast<size_t>(Hkv) * HD * ESZ;

  for (int i = tid; i < G * HD; i += DEC_THREADS)
    sQ[i / HD][i % HD] = __bfloat162float(q[(static_cast<size_t>(b) * Hq + kvh * G + i / HD) * HD + i % HD]) * scale;
  if (tid < DEC_MAX_G) {
    sM[tid] = -INFINITY;
    sL[tid] = 0.f;
  }
  float acc[DEC_MAX_G / 2][2];
#pragma unroll
  for (int i = 0; i < DEC_MAX_G / 2; ++i) acc[i][0] = acc[i][1] = 0.f;
  __syncthreads();

  for (int c0 = t_begin; c0 < t_end; c0 += DEC_CHUNK) {
    const int n = min(DEC_CHUNK, t_end - c0);
    // stage K and V rows of this chunk (16-byte pieces)
    constexpr int PIECES = HD * ESZ / 16;
    for (int i = tid; i < n * PIECES; i += DEC_THREADS) {
      const int t = i / PIECES, pc = i % PIECES;
      const int pos = c0 + t;
      const int blk = table[pos / PAGE];
      const size_t a = (static_cast<size_t>(blk) * PAGE + pos % PAGE) * tok_stride +
                       static_cast<size_t>(kvh) * HD * ESZ + pc * 16;
      *reinterpret_cast<uint4*>(sK + t * ROW + pc * 16) =
          *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(k_cache) + a);
      *reinterpret_cast<uint4*>(sV + t * ROW + pc * 16) =
          *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(v_cache) + a);
    }
    if (FP8 && tid < DEC_CHUNK / PAGE) {
      const int pos = c0 + tid * PAGE;
      if (pos < t_end) {
        const int blk = table[pos / PAGE];
        sKs[tid] = k_scale[static_cast<size_t>(blk) * Hkv + kvh];
        sVs[tid] = v_scale[static_cast<size_t>(blk) * Hkv + kvh];
      }
    }
    __syncthreads();
    // scores
    for (int i = tid; i < G * DEC_CHUNK; i += DEC_THREADS) {
      const int t = i % DEC_CHUNK, g = i / DEC_CHUNK;
      float s = -INFINITY;
      if (t < n) {
        s = 0.f;
        const uint8_t* row = sK + t * ROW;
        if (FP8) {
#pragma unroll
          for (int pc = 0; pc < 8; ++pc) {
            uint4 u = *reinterpret_cast<const uint4*>(row + pc * 16);
            const uint8_t* e = reinterpret_cast<const uint8_t*>(&u);
#pragma unroll
            for (int j = 0; j < 16; ++j) s += sQ[g][pc * 16 + j] * fp8_to_float(e[j]);
          }
          s *= sKs[t / PAGE];
        } else {
#pragma unroll
          for (int pc = 0; pc < 16; ++pc) {
            uint4 u = *reinterpret_cast<const uint4*>(row + pc * 16);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float2 f = unpack_bf16x2(w[j]);
              s += sQ[g][pc * 8 + 2 * j] * f.x + sQ[g][pc * 8 + 2 * j + 1] * f.y;
            }
          }
        }
      }
      sS[g][t] = s;
    }
    __syncthreads();
    // online softmax: warp w owns query heads w, w+4
    for (int g = warp; g < G; g += DEC_THREADS / 32) {
      const float s0 = sS[g][lane], s1 = sS[g][lane + 32];
      const float cm = warp_max(fmaxf(s0, s1));
      const float m_old = sM[g];
      const float m_new = fmaxf(m_old, cm);
      const float p0 = __expf(s0 - m_new), p1 = __expf(s1 - m_new);
      const float ps = warp_sum(p0 + p1);
      sS[g][lane] = p0;
      sS[g][lane + 32] = p1;
      if (lane == 0) {
        const float alpha = m_old == -INFINITY ? 0.f : __expf(m_old - m_new);
        sAlpha[g] = alpha;
        sL[g] = sL[g] * alpha + ps;
        sM[g] = m_new;
      }
    }
    __syncthreads();
    // P*V: thread owns (g, two dims)
#pragma unroll
    for (int it = 0; it < DEC_MAX_G / 2; ++it) {
      const int p = tid + it * DEC_THREADS;
      if (p < G * (HD / 2)) {
        const int g = p / (HD / 2), dp = (p % (HD / 2)) * 2;
        float a0 = acc[it][0] * sAlpha[g], a1 = acc[it][1] * sAlpha[g];
        for (int t = 0; t < n; ++t) {
          const float pw = sS[g][t];
          float v0, v1;
          if (FP8) {
            const uint8_t* e = sV + t * ROW + dp;
            const float vs = sVs[t / PAGE];
            v0 = fp8_to_float(e[0]) * vs;
            v1 = fp8_to_float(e[1]) * vs;
          } else {
            float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(sV + t * ROW + dp * 2));
            v0 = f.x;
            v1 = f.y;
          }
          a0 += pw * v0;
          a1 += pw * v1;
        }
        acc[it][0] = a0;
        acc[it][1] = a1;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int it = 0; it < DEC_MAX_G / 2; ++it) {
    const int p = tid + it * DEC_THREADS;
    if (p < G * (HD / 2)) {
      const int g = p / (HD / 2), dp = (p % (HD / 2)) * 2;
      const int head = kvh * G + g;
      if (nsplit == 1) {
        const float inv = sL[g] > 0.f ? 1.f / sL[g] : 0.f;
        *reinterpret_cast<uint32_t*>(out + (static_cast<size_t>(b) * Hq + head) * HD + dp) =
            pack_bf16x2(acc[it][0] * inv, acc[it][1] * inv);
      } else {
        float* po = part_o + ((static_cast<size_t>(b) * Hq + head) * nsplit + split) * HD + dp;
        po[0] = acc[it][0];
        po[1] = acc[it][1];
      }
    }
  }
  if (nsplit > 1 && tid < G) {
    float* ml = part_ml + ((static_cast<size_t>(b) * Hq + kvh * G + tid) * nsplit + split) * 2;
    ml[0] = sM[tid];
    ml[1] = sL[tid];
  }
}

// Exact merge of split-KV partials: out = sum_i acc_i e^{m_i - M} / sum_i l_i e^{m_i - M}.
__global__ void __launch_bounds__(HD) paged_merge_kernel(const float* __restrict__ part_o,
                                                        const float* __restrict__ part_ml,
                                                        __nv_bfloat16* __restrict__ out,
                                                        float* __restrict__ lse_out, int nsplit) {
  const size_t bh = blockIdx.x;
  const int d = threadIdx.x;
  float M = -INFINITY;
  for (int i = 0; i < nsplit; ++i) M = fmaxf(M, part_ml[(bh * nsplit + i) * 2]);
  float L = 0.f, o = 0.f;
  for (int i = 0; i < nsplit; ++i) {
    const float m = part_ml[(bh * nsplit + i) * 2], l = part_ml[(bh * nsplit + i) * 2 + 1];
    if (m == -INFINITY) continue;
    const float w = __expf(m - M);
    L += l * w;
    o += part_o[(bh * nsplit + i) * HD + d] * w;
  }
  out[bh * HD + d] = __float2bfloat16(L > 0.f ? o / L : 0.f);
  if (lse_out && d == 0) lse_out[bh] = M + __logf(L);
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

B2_EXPORT int b2_kv_store(const void* k, const void* v, int ld_k, int ld_v, void* k_cache, void* v_cache,
                          float* k_scale, float* v_scale, const int* segs, int nseg, int Hkv, int head_dim,
                          int fp8, void* stream) {
  b2::ensure_thread_context();
  if (head_dim != HD) { set_error("kv_store: head_dim must be 128"); return 10; }
  if (nseg <= 0) return 0;
  dim3 grid(nseg, Hkv, 2);
  if (fp8)
    kv_store_kernel<true><<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), ld_k, ld_v, k_cache, v_cache,
        k_scale, v_scale, segs, Hkv);
  else
    kv_store_kernel<false><<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), ld_k, ld_v, k_cache, v_cache,
        k_scale, v_scale, segs, Hkv);
  B2_LAUNCH_CHECK("kv_store");
  return 0;
}

B2_EXPORT int b2_kv_gather(const void* k_cache, const void* v_cache, const float* k_scale, const float* v_scale,
                           const int* slot, void* k_out, void* v_out, int rows, int Hkv, int head_dim, int fp8,
                           void* stream) {
  b2::ensure_thread_context();
  if (head_dim != HD) { set_error("kv_gather: head_dim must be 128"); return 10; }
  if (rows <= 0) return 0;
  const long long total = static_cast<long long>(rows) * Hkv * HD;
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(num_sms()) * 16;
  if (blocks > cap) blocks = cap;
  if (fp8)
    kv_gather_kernel<true><<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        k_cache, v_cache, k_scale, v_scale, slot, static_cast<__nv_bfloat16*>(k_out),
        static_cast<__nv_bfloat16*>(v_out), rows, Hkv);
  else
    kv_gather_kernel<false><<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        k_cache, v_cache, k_scale, v_scale, slot, static_cast<__nv_bfloat16*>(k_out),
        static_cast<__nv_bfloat16*>(v_out), rows, Hkv);
  B2_LAUNCH_CHECK("kv_gather");
  return 0;
}

// partition: tokens per split (multiple of 64); nsplit = ceil(max_ctx / partition) chosen by the caller.
// part_o: fp32 [B, Hq, nsplit, 128]; part_ml: fp32 [B, Hq, nsplit, 2] (only read when nsplit > 1).
B2_EXPORT int b2_paged_decode(const void* q, const void* k_cache, const void* v_cache, const float* k_scale,
                              const float* v_scale, const int* block_tables, const int* context_lens,
                              int max_blocks, void* out, float* part_o, float* part_ml, float* lse, int B,
                              int Hq, int Hkv, int head_dim, int partition, int nsplit, float scale, int fp8,
                              void* stream_) {
  b2::ensure_thread_context();
  if (head_dim != HD || Hq % Hkv != 0 || Hq / Hkv > DEC_MAX_G || partition % DEC_CHUNK != 0 || nsplit < 1) {
    set_error("paged_decode: head_dim 128, Hq/Hkv <= 8, partition %% 64 == 0 required");
    return 10;
  }
  if (B <= 0) return 0;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  dim3 grid(B, Hkv, nsplit);
  if (fp8)
    paged_decode_kernel<true><<<grid, DEC_THREADS, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(q), k_cache, v_cache, k_scale, v_scale, block_tables, context_lens,
        max_blocks, static_cast<__nv_bfloat16*>(out), part_o, part_ml, Hq, Hkv, partition, scale);
  else
    paged_decode_kernel<false><<<grid, DEC_THREADS, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(q), k_cache, v_cache, k_scale, v_scale, block_tables, context_lens,
        max_blocks, static_cast<__nv_bfloat16*>(out), part_o, part_ml, Hq, Hkv, partition, scale);
  B2_LAUNCH_CHECK("paged_decode");
  if (nsplit > 1) {
    paged_merge_kernel<<<B * Hq, HD, 0, stream>>>(part_o, part_ml, static_cast<__nv_bfloat16*>(out), lse, nsplit);
    B2_LAUNCH_CHECK("paged_merge");
  }
  return 0;
}
