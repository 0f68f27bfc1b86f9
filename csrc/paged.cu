// Paged KV-cache kernels: block-segment KV store (bf16 and fp8-e4m3 with one scale per block and kv
// head), gather / dequantise into contiguous bf16, paged decode attention with split-KV partitions
// and the exact log-sum-exp merge.
//
// Cache layout for one layer and one of {K, V}: [num_blocks, 16 tokens, Hkv, 128] (bf16 or fp8 bytes);
// scales [num_blocks, Hkv] fp32 (value = stored * scale).
#include <cuda_fp8.h>

#include <cstdlib>

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
// Paged decode attention: one query token per sequence.  Grid (B, Hkv * head groups, nsplit); a CTA streams
// its partition of the sequence's pages, scores the query heads of its kv head, and keeps an online softmax.
// nsplit == 1 writes the output directly; otherwise unnormalised partials + (max, sum) go to a workspace for
// the merge kernel.
// ---------------------------------------------------------------------------------------------
constexpr int DEC_THREADS = 128;
constexpr int DEC_CHUNK = 64;   // partitions are multiples of this many tokens
constexpr int DEC_MAX_G = 8;
constexpr int DEC_UNROLL = 4;   // cache rows in flight per lane group
constexpr int DEC_DEFAULT_MODE = 3;   // row loop of the decode kernel when B200FW_DECODE_MODE is unset
constexpr float DEC_LOG2E = 1.4426950408889634f;
constexpr float DEC_LN2 = 0.6931471805599453f;

template <bool FP8>
__device__ __forceinline__ void dec_unpack(const uint4& u, float* f);
template <>
__device__ __forceinline__ void dec_unpack<false>(const uint4& u, float* f) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = unpack_bf16x2(w[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
template <>
__device__ __forceinline__ void dec_unpack<true>(const uint4& u, float* f) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const __half2_raw r = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>((w[j] >> (16 * h)) & 0xFFFFu),
                                                       __NV_E4M3);
      const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&r));
      f[4 * j + 2 * h] = t.x;
      f[4 * j + 2 * h + 1] = t.y;
    }
  }
}

// Decode attention over the paged cache, one CTA per (sequence, kv head, head group, partition).
// A cache row (128 dims) is spread over LPT = 16 (bf16) or 8 (fp8) lanes of a warp, 16 bytes each, so one
// warp-wide access covers 2 (4) tokens and every lane handles DEC_UNROLL K and V pieces per step; no data is
// ever shared between lanes through memory.  Each lane group runs its own online softmax over the tokens it sees (running
// maximum, sum and DPL accumulator dims per head, base-2 exponent domain); groups and warps are merged
// once at the end with the exact log-sum-exp rule.  GH query heads of the kv head are handled per CTA
// (their q pieces sit in registers); larger GQA ratios use several CTAs (head groups) per kv head.
// MODE 0: plain row loop, the K and V pieces of a step are loaded into registers and consumed.
// MODE 3: every warp owns a ring of three stages in shared memory, filled by 16-byte asynchronous copies
// (cp.async.cg, no register staging); a lane reads back exactly the bytes it copied, so no barrier is needed, and
// two steps' worth of K and V rows stay in flight per warp without growing the register count.  (Measured at
// 256 x 1024: 0.194 ms against 0.231 ms for MODE 0; a four-stage ring, 0.203 ms, and a register software pipeline,
// 0.283 ms, were tried and dropped.)
template <bool FP8, int GH, int MODE>
__global__ void __launch_bounds__(DEC_THREADS) paged_decode_kernel(
    const __nv_bfloat16* __restrict__ q, const void* __restrict__ k_cache, const void* __restrict__ v_cache,
    const float* __restrict__ k_scale, const float* __restrict__ v_scale,
    const int* __restrict__ block_tables, const int* __restrict__ context_lens, int max_blocks,
    __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, int Hq, int Hkv,
    int partition, float scale) {
  constexpr int ESZ = FP8 ? 1 : 2;
  constexpr int LPT = HD * ESZ / 16;   // lanes per token row
  constexpr int TPW = 32 / LPT;        // token rows per warp-wide load
  constexpr int DPL = 16 / ESZ;        // dims per lane
  constexpr int U = DEC_UNROLL;
  static_assert(MODE == 0 || MODE == 3, "row loop: 0 (registers) or 3 (three-stage cp.async ring)");
  constexpr int STAGES = MODE >= 2 ? MODE : 1;
  __shared__ float sAcc[DEC_THREADS / 32][GH][HD];
  __shared__ float sM[DEC_THREADS / 32][GH], sL[DEC_THREADS / 32][GH];
  extern __shared__ __align__(16) uint8_t dec_ring[];   // [warp][stage][u][K | V][32 lanes x 16 B] (MODE >= 2)

  const int G = Hq / Hkv;
  const int groups_per_kv = G / GH;
  const int b = blockIdx.x, kvh = blockIdx.y / groups_per_kv, hg = blockIdx.y % groups_per_kv;
  const int split = blockIdx.z, nsplit = gridDim.z;
  const int head0 = kvh * G + hg * GH;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = lane / LPT, sub = lane % LPT;
  const int ctx = context_lens[b];
  const int t_begin = split * partition;
  const int t_end = min(ctx, t_begin + partition);
  const int* table = block_tables + static_cast<size_t>(b) * max_blocks;
  const size_t tok_stride = static_cast<size_t>(Hkv) * HD * ESZ;
  const uint8_t* kc = reinterpret_cast<const uint8_t*>(k_cache) + static_cast<size_t>(kvh) * HD * ESZ + sub * 16;
  const uint8_t* vc = reinterpret_cast<const uint8_t*>(v_cache) + static_cast<size_t>(kvh) * HD * ESZ + sub * 16;

  float qr[GH][DPL], acc[GH][DPL], m[GH], l[GH];
  const float qs = scale * DEC_LOG2E;
#pragma unroll
  for (int g = 0; g < GH; ++g) {
    const __nv_bfloat16* qp = q + (static_cast<size_t>(b) * Hq + head0 + g) * HD + sub * DPL;
#pragma unroll
    for (int d = 0; d < DPL; ++d) {
      qr[g][d] = __bfloat162float(qp[d]) * qs;
      acc[g][d] = 0.f;
    }
    m[g] = -INFINITY;
    l[g] = 0.f;
  }

  // One step of a lane group: U cache rows (their K and V pieces, the block's scales, validity).
  struct Rows {
    uint4 kq[U], vq[U];
    float ks[U], vs[U];
    bool valid[U];
  };
  auto load_rows = [&](Rows& r, int base) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int tok = base + u * TPW + group;
      r.valid[u] = tok < t_end;
      r.kq[u] = make_uint4(0, 0, 0, 0);
      r.vq[u] = make_uint4(0, 0, 0, 0);
      r.ks[u] = r.vs[u] = 1.f;
      if (r.valid[u]) {
        const int blk = table[tok / PAGE];
        const size_t a = (static_cast<size_t>(blk) * PAGE + tok % PAGE) * tok_stride;
        r.kq[u] = *reinterpret_cast<const uint4*>(kc + a);
        r.vq[u] = *reinterpret_cast<const uint4*>(vc + a);
        if (FP8) {
          r.ks[u] = k_scale[static_cast<size_t>(blk) * Hkv + kvh];
          r.vs[u] = v_scale[static_cast<size_t>(blk) * Hkv + kvh];
        }
      }
    }
  };
  auto consume = [&](const Rows& r) {
    const uint4* kq = r.kq;
    const uint4* vq = r.vq;
    const float* ks = r.ks;
    const float* vs = r.vs;
    const bool* valid = r.valid;
    float sc[U][GH];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float kf[DPL];
      dec_unpack<FP8>(kq[u], kf);
#pragma unroll
      for (int g = 0; g < GH; ++g) {
        float d0 = 0.f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) d0 = fmaf(qr[g][d], kf[d], d0);
#pragma unroll
        for (int o = LPT / 2; o > 0; o >>= 1) d0 += __shfl_xor_sync(0xffffffffu, d0, o);
        sc[u][g] = valid[u] ? d0 * ks[u] : -INFINITY;
      }
    }
#pragma unroll
    for (int g = 0; g < GH; ++g) {
      float mn = m[g];
#pragma unroll
      for (int u = 0; u < U; ++u) mn = fmaxf(mn, sc[u][g]);
      if (mn == -INFINITY) {   // this lane group has not seen a token yet: its weights are zero
#pragma unroll
        for (int u = 0; u < U; ++u) sc[u][g] = 0.f;
        continue;
      }
      const float alpha = fast_exp2(m[g] - mn);
      m[g] = mn;
      float ps = 0.f;
#pragma unroll
      for (int d = 0; d < DPL; ++d) acc[g][d] *= alpha;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float p = fast_exp2(sc[u][g] - mn);
        ps += p;
        sc[u][g] = p * vs[u];
      }
      l[g] = l[g] * alpha + ps;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float vf[DPL];
      dec_unpack<FP8>(vq[u], vf);
#pragma unroll
      for (int g = 0; g < GH; ++g)
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[g][d] = fmaf(sc[u][g], vf[d], acc[g][d]);
    }
  };
  {
    constexpr int STEP = (DEC_THREADS / 32) * TPW * U;
    int base = t_begin + warp * (TPW * U);
    if (MODE >= 2) {
      const uint32_t ring = smem_u32(dec_ring) + (warp * STAGES * U * 2 * 32 + lane) * 16;
      auto issue = [&](int stage, int at) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int tok = at + u * TPW + group;
          if (tok < t_end) {
            const int blk = table[tok / PAGE];
            const size_t a = (static_cast<size_t>(blk) * PAGE + tok % PAGE) * tok_stride;
            const uint32_t dst = ring + ((stage * U + u) * 2) * 512;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(kc + a) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 512), "l"(vc + a) : "memory");
          }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");   // one group per stage, empty ones included
      };
#pragma unroll
      for (int s = 0; s < STAGES - 1; ++s) issue(s, base + s * STEP);
      int slot = 0;
      for (; base < t_end; base += STEP) {
        issue(slot == 0 ? STAGES - 1 : slot - 1, base + (STAGES - 1) * STEP);
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 1) : "memory");
        Rows r;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int tok = base + u * TPW + group;
          r.valid[u] = tok < t_end;
          r.kq[u] = make_uint4(0, 0, 0, 0);
          r.vq[u] = make_uint4(0, 0, 0, 0);
          r.ks[u] = r.vs[u] = 1.f;
          if (r.valid[u]) {
            const uint32_t src = ring + ((slot * U + u) * 2) * 512;
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(r.kq[u].x), "=r"(r.kq[u].y), "=r"(r.kq[u].z), "=r"(r.kq[u].w)
                         : "r"(src));
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(r.vq[u].x), "=r"(r.vq[u].y), "=r"(r.vq[u].z), "=r"(r.vq[u].w)
                         : "r"(src + 512));
            if (FP8) {
              const int blk = table[tok / PAGE];
              r.ks[u] = k_scale[static_cast<size_t>(blk) * Hkv + kvh];
              r.vs[u] = v_scale[static_cast<size_t>(blk) * Hkv + kvh];
            }
          }
        }
        consume(r);
        slot = slot + 1 == STAGES ? 0 : slot + 1;
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
      for (; base < t_end; base += STEP) {
        Rows r;
        load_rows(r, base);
        consume(r);
      }
    }
  }

  // merge the lane groups of the warp, then the warps
#pragma unroll
  for (int o = LPT; o < 32; o <<= 1) {
#pragma unroll
    for (int g = 0; g < GH; ++g) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[g], o);
      const float lo = __shfl_xor_sync(0xffffffffu, l[g], o);
      const float mn = fmaxf(m[g], mo);
      const float wa = mn == -INFINITY ? 0.f : fast_exp2(m[g] - mn);
      const float wb = mn == -INFINITY ? 0.f : fast_exp2(mo - mn);
#pragma unroll
      for (int d = 0; d < DPL; ++d) {
        const float ao = __shfl_xor_sync(0xffffffffu, acc[g][d], o);
        acc[g][d] = acc[g][d] * wa + ao * wb;
      }
      l[g] = l[g] * wa + lo * wb;
      m[g] = mn;
    }
  }
  if (group == 0) {
#pragma unroll
    for (int g = 0; g < GH; ++g) {
#pragma unroll
      for (int d = 0; d < DPL; ++d) sAcc[warp][g][sub * DPL + d] = acc[g][d];
      if (sub == 0) {
        sM[warp][g] = m[g];
        sL[warp][g] = l[g];
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int g = 0; g < GH; ++g) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_THREADS / 32; ++w) M = fmaxf(M, sM[w][g]);
    float L = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_THREADS / 32; ++w) {
      const float wgt = sM[w][g] == -INFINITY ? 0.f : fast_exp2(sM[w][g] - M);
      L += sL[w][g] * wgt;
      o += sAcc[w][g][tid] * wgt;
    }
    const int head = head0 + g;
    if (nsplit == 1) {
      out[(static_cast<size_t>(b) * Hq + head) * HD + tid] = __float2bfloat16(L > 0.f ? o / L : 0.f);
    } else {
      part_o[((static_cast<size_t>(b) * Hq + head) * nsplit + split) * HD + tid] = o;
      if (tid == 0) {
        float* ml = part_ml + ((static_cast<size_t>(b) * Hq + head) * nsplit + split) * 2;
        ml[0] = M * DEC_LN2;   // natural-log domain for the merge kernel
        ml[1] = L;
      }
    }
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
  const int G = Hq / Hkv;
  // query heads per CTA (their q pieces and accumulators live in registers: fp8 rows put 16 dims on a
  // lane, so four heads would leave room for only two CTAs per SM)
  const int GH = (G % 4 == 0 && !fp8) ? 4 : (G % 2 == 0 ? 2 : 1);
  dim3 grid(B, Hkv * (G / GH), nsplit);
  // B200FW_DECODE_MODE selects the row loop: 0 registers, 3 the cp.async ring (read on every call, so that one
  // process can compare them)
  const int mode = [] {
    const char* e = std::getenv("B200FW_DECODE_MODE");
    if (e != nullptr && (e[0] == '0' || e[0] == '3')) return e[0] - '0';
    return DEC_DEFAULT_MODE;
  }();
#define B2_DECODE_LAUNCH_M(F8, GHV, MD)                                                                    \
  do {                                                                                                     \
    constexpr int ring = MD >= 2 ? (DEC_THREADS / 32) * MD * DEC_UNROLL * 2 * 512 : 0;                     \
    auto kern = paged_decode_kernel<F8, GHV, MD>;                                                          \
    if (ring > 0) {                                                                                        \
      static bool attr_set[64] = {};                                                                       \
      int dev = 0;                                                                                         \
      cudaGetDevice(&dev);                                                                                 \
      if (!attr_set[dev & 63]) {                                                                           \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ring);                     \
        attr_set[dev & 63] = true;                                                                         \
      }                                                                                                    \
    }                                                                                                      \
    kern<<<grid, DEC_THREADS, ring, stream>>>(                                                             \
        static_cast<const __nv_bfloat16*>(q), k_cache, v_cache, k_scale, v_scale, block_tables, context_lens, \
        max_blocks, static_cast<__nv_bfloat16*>(out), part_o, part_ml, Hq, Hkv, partition, scale);         \
  } while (0)
#define B2_DECODE_LAUNCH(F8, GHV)                                                                          \
  do {                                                                                                     \
    if (mode == 3) B2_DECODE_LAUNCH_M(F8, GHV, 3);                                                         \
    else B2_DECODE_LAUNCH_M(F8, GHV, 0);                                                                   \
  } while (0)
  if (fp8) {
    if (GH == 4) B2_DECODE_LAUNCH(true, 4);
    else if (GH == 2) B2_DECODE_LAUNCH(true, 2);
    else B2_DECODE_LAUNCH(true, 1);
  } else {
    if (GH == 4) B2_DECODE_LAUNCH(false, 4);
    else if (GH == 2) B2_DECODE_LAUNCH(false, 2);
    else B2_DECODE_LAUNCH(false, 1);
  }
#undef B2_DECODE_LAUNCH_M
#undef B2_DECODE_LAUNCH
  B2_LAUNCH_CHECK("paged_decode");
  if (nsplit > 1) {
    paged_merge_kernel<<<B * Hq, HD, 0, stream>>>(part_o, part_ml, static_cast<__nv_bfloat16*>(out), lse, nsplit);
    B2_LAUNCH_CHECK("paged_merge");
  }
  return 0;
}
