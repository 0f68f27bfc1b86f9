// RMSNorm forward/backward, fused per-head QK-RMSNorm + rotary embedding forward/backward, SwiGLU
// forward/backward, embedding gather / scatter-add.  All HBM-bound: 16-byte vector accesses, fp32
// math, bf16 storage.
#include <atomic>

#include "common.cuh"
#include "host.h"

namespace b2 {

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  bf16x8 r = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(r.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  bf16x8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = r;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < THREADS / 32) ? scratch[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// ---------------------------------------------------------------------------------------------
// RMSNorm forward: one CTA per row, H % 8 == 0.  y = x * rstd * w ; rstd saved for backward.
// ---------------------------------------------------------------------------------------------
constexpr int RMS_THREADS = 256;
constexpr int RMS_MAX_VEC = 4;  // up to 256*8*4 = 8192 columns kept in registers

__global__ void __launch_bounds__(RMS_THREADS) rmsnorm_fwd_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
    __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int H, float eps) {
  __shared__ float scratch[32];
  const size_t row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * H;
  __nv_bfloat16* yr = y + row * H;
  float v[RMS_MAX_VEC][8];
  float ss = 0.f;
  const int nvec = H / 8;
#pragma unroll
  for (int i = 0; i < RMS_MAX_VEC; ++i) {
    const int c = threadIdx.x + i * RMS_THREADS;
    if (c < nvec) {
      load8(xr + c * 8, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  // columns beyond the register window (H > 8192): accumulate only
  for (int c = threadIdx.x + RMS_MAX_VEC * RMS_THREADS; c < nvec; c += RMS_THREADS) {
    float t[8];
    load8(xr + c * 8, t);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += t[j] * t[j];
  }
  ss = block_sum<RMS_THREADS>(ss, scratch);
  const float rstd = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < RMS_MAX_VEC; ++i) {
    const int c = threadIdx.x + i * RMS_THREADS;
    if (c < nvec) {
      float wv[8], o[8];
      load8(w + c * 8, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rstd * wv[j];
      store8(yr + c * 8, o);
    }
  }
  for (int c = threadIdx.x + RMS_MAX_VEC * RMS_THREADS; c < nvec; c += RMS_THREADS) {
    float t[8], wv[8], o[8];
    load8(xr + c * 8, t);
    load8(w + c * 8, wv);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = t[j] * rstd * wv[j];
    store8(yr + c * 8, o);
  }
}

// RMSNorm backward.  Persistent CTAs stride over rows; each keeps a partial dw in registers and
// writes it to dw_partial[cta, H] (fp32); a second kernel reduces the partials.
//   dx = rstd * (dy*w - xhat * mean(dy*w*xhat)),  dw = sum_rows dy * xhat,  xhat = x*rstd
__global__ void __launch_bounds__(RMS_THREADS) rmsnorm_bwd_kernel(
    const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
    const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
    __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, int M, int H, int add_to_dx) {
  __shared__ float scratch[32];
  const int nvec = H / 8;
  float dwacc[RMS_MAX_VEC][8];
  float wv[RMS_MAX_VEC][8];
#pragma unroll
  for (int i = 0; i < RMS_MAX_VEC; ++i) {
    const int c = threadIdx.x + i * RMS_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
    if (c < nvec) load8(w + c * 8, wv[i]);
  }
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    const __nv_bfloat16* xr = x + static_cast<size_t>(row) * H;
    const __nv_bfloat16* dyr = dy + static_cast<size_t>(row) * H;
    __nv_bfloat16* dxr = dx + static_cast<size_t>(row) * H;
    const float rstd = rstd_in[row];
    float xh[RMS_MAX_VEC][8], g[RMS_MAX_VEC][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < RMS_MAX_VEC; ++i) {
      const int c = threadIdx.x + i * RMS_THREADS;
      if (c < nvec) {
        float xv[8], dv[8];
        load8(xr + c * 8, xv);
        load8(dyr + c * 8, dv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = xv[j] * rstd;
          dwacc[i][j] += dv[j] * xh[i][j];
          g[i][j] = dv[j] * wv[i][j];
          dot += g[i][j] * xh[i][j];
        }
      }
    }
    dot = block_sum<RMS_THREADS>(dot, scratch);
    const float mean = dot / H;
#pragma unroll
    for (int i = 0; i < RMS_MAX_VEC; ++i) {
      const int c = threadIdx.x + i * RMS_THREADS;
      if (c < nvec) {
        float o[8];
        if (add_to_dx) load8(dxr + c * 8, o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = rstd * (g[i][j] - xh[i][j] * mean);
          o[j] = add_to_dx ? o[j] + d : d;
        }
        store8(dxr + c * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < RMS_MAX_VEC; ++i) {
    const int c = threadIdx.x + i * RMS_THREADS;
    if (c < nvec) {
      float* p = dw_partial + static_cast<size_t>(blockIdx.x) * H + c * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) p[j] = dwacc[i][j];
    }
  }
}


// ---------------------------------------------------------------------------------------------
// Warp-per-row variants for H <= 2048 (NV = H/256 rounded up, <= 8 vectors of 8 per lane): no block-wide
// barriers on the critical path, rows stay in registers, 8 rows in flight per 256-thread CTA.
// ---------------------------------------------------------------------------------------------
template <int NV>
__global__ void __launch_bounds__(256) rmsnorm_fwd_warp_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
    __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int M, int H, float eps) {
  const int lane = threadIdx.x & 31;
  const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
  const int nvec = H / 8;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < M; row += warps_per_grid) {
    const __nv_bfloat16* xr = x + static_cast<size_t>(row) * H;
    float v[NV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        load8(xr + c * 8, v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
      }
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / H + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
    __nv_bfloat16* yr = y + static_cast<size_t>(row) * H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        float o[8], wv[8];
        load8(w + c * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rstd * wv[j];
        store8(yr + c * 8, o);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// RMSNorm backward split in two high-occupancy kernels (H <= 2048):
//   dx kernel: one warp per row, nothing carried across rows (few registers, many warps in flight);
//   dw kernel: column reduction dw[h] = sum_r dy[r,h] * x[r,h] * rstd[r]; a thread owns 8 columns and
//              strides over rows with four independent loads in flight; per-CTA partials.
// x and dy are read twice, the second time from L2.
// ---------------------------------------------------------------------------------------------
template <int NV>
__global__ void __launch_bounds__(256) rmsnorm_bwd_dx_kernel(
    const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
    const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
    __nv_bfloat16* __restrict__ dx, int M, int H, int add_to_dx) {
  const int lane = threadIdx.x & 31;
  const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
  const int nvec = H / 8;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < M; row += warps_per_grid) {
    const __nv_bfloat16* xr = x + static_cast<size_t>(row) * H;
    const __nv_bfloat16* dyr = dy + static_cast<size_t>(row) * H;
    __nv_bfloat16* dxr = dx + static_cast<size_t>(row) * H;
    const float rstd = rstd_in[row];
    float xh[NV][8], g[NV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        float dv[8], wv[8];
        load8(xr + c * 8, xh[i]);
        load8(dyr + c * 8, dv);
        load8(w + c * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] *= rstd;
          g[i][j] = dv[j] * wv[j];
          dot += g[i][j] * xh[i][j];
        }
      }
    }
    dot = warp_sum(dot) / H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        float o[8];
        if (add_to_dx) load8(dxr + c * 8, o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = rstd * (g[i][j] - xh[i][j] * dot);
          o[j] = add_to_dx ? o[j] + d : d;
        }
        store8(dxr + c * 8, o);
      }
    }
  }
}

__global__ void __launch_bounds__(256) rmsnorm_bwd_dw_kernel(
    const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
    const float* __restrict__ rstd_in, float* __restrict__ dw_partial, int M, int H) {
  // thread -> column vector c = threadIdx.x % nvec (nvec <= 256), row lane rl = threadIdx.x / nvec
  const int nvec = H / 8;
  const int rows_per_cta_step = blockDim.x / nvec;       // 1 for H=2048, 2 for H=1024, ...
  const int c = threadIdx.x % nvec, rl = threadIdx.x / nvec;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const int stride = gridDim.x * rows_per_cta_step;
  int row = blockIdx.x * rows_per_cta_step + rl;
  if (rl < rows_per_cta_step) {
    for (; row + 3 * stride < M; row += 4 * stride) {
      float xv[4][8], dv[4][8], rs[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const size_t o = static_cast<size_t>(row + u * stride) * H + c * 8;
        load8(x + o, xv[u]);
        load8(dy + o, dv[u]);
        rs[u] = rstd_in[row + u * stride];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += dv[u][j] * xv[u][j] * rs[u];
    }
    for (; row < M; row += stride) {
      float xv[8], dv[8];
      const size_t o = static_cast<size_t>(row) * H + c * 8;
      load8(x + o, xv);
      load8(dy + o, dv);
      const float rs = rstd_in[row];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += dv[j] * xv[j] * rs;
    }
  }
  extern __shared__ float sdw[];   // [H]
  for (int i = threadIdx.x; i < H; i += blockDim.x) sdw[i] = 0.f;
  __syncthreads();
  if (rl < rows_per_cta_step) {
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(&sdw[c * 8 + j], acc[j]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < H; i += blockDim.x) dw_partial[static_cast<size_t>(blockIdx.x) * H + i] = sdw[i];
}

// dw[h] (+)= sum_p partial[p, h]   (bf16 or fp32 destination)
// Column sums of partial[P, H].  Block = 32 columns x 8 warps: warp w sums rows w, w+8, ... with four
// independent chains, the eight warp results meet in shared memory.  (One thread per column walking all P
// rows is a single dependent chain of P L2 round trips: 9-12 us for 256 x 1024.)
__global__ void __launch_bounds__(256) reduce_partials_kernel(const float* __restrict__ partial,
                                                              void* __restrict__ dw, int P, int H,
                                                              int accumulate, int out_fp32) {
  __shared__ float part[8][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int h = blockIdx.x * 32 + lane;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (h < H) {
    int p = w;
    for (; p + 24 < P; p += 32) {
#pragma unroll
      for (int u = 0; u < 4; ++u) acc[u] += partial[static_cast<size_t>(p + 8 * u) * H + h];
    }
    for (; p < P; p += 8) acc[0] += partial[static_cast<size_t>(p) * H + h];
  }
  part[w][lane] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
  __syncthreads();
  if (w != 0 || h >= H) return;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s += part[i][lane];
  if (out_fp32) {
    float* o = reinterpret_cast<float*>(dw);
    o[h] = accumulate ? o[h] + s : s;
  } else {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(dw);
    o[h] = __float2bfloat16(accumulate ? __bfloat162float(o[h]) + s : s);
  }
}

// ---------------------------------------------------------------------------------------------
// Fused per-head RMSNorm (q_norm / k_norm) + half-rotation RoPE, head_dim = 128.
// qkv: [M, (Hq + 2*Hkv) * 128] (the fused projection output); q_out [M,Hq,128], k_out [M,Hkv,128].
// cos/sin: fp32 tables [max_pos, 64].  rstd_out: [M, Hq+Hkv] fp32 for backward.
// ---------------------------------------------------------------------------------------------
// One warp per token.  A head (128 dims) is spread over 16 lanes at 8 elements (16 bytes) each, so one
// warp-wide access covers two heads; the rotation partner (dim +- 64) sits in lane ^ 8.  The token's
// cos / sin row is loaded once and reused by all its q and k heads, and QKR_PAIRS head pairs are loaded
// before the first is processed.  (A warp per (token, head) with 8-byte accesses and a dependent
// position -> table load per unit ran at a third of the memory bandwidth.)
constexpr int QKR_PAIRS = 4;

__device__ __forceinline__ void qkr_unpack8(const uint4& q, float* f) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = unpack_bf16x2(w[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 qkr_pack8(const float* f) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]);
  o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]);
  o.w = pack_bf16x2(f[6], f[7]);
  return o;
}
__device__ __forceinline__ float sum16(float v) {   // over the 16 lanes that share a head
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// STORE: the inference form.  Token `tok` owns row slots[tok] (= block * block_size + offset; negative: padding, no
// store) of a bf16 paged cache laid out [rows, Hkv, 128]; its rotated keys and its values (copied from the projection
// output) are written there by the same warp, so the runner needs no separate store launch and K / V are not re-read.
template <bool STORE>
__global__ void __launch_bounds__(256) qknorm_rope_fwd_kernel(
    const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ qw,
    const __nv_bfloat16* __restrict__ kw, const int* __restrict__ pos,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t,
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out,
    float* __restrict__ rstd_out, int M, int Hq, int Hkv, int ld_qkv, float eps,
    const int* __restrict__ slots, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache) {
  const int heads = Hq + Hkv;
  const int lane = threadIdx.x & 31, l16 = lane & 15, sub = lane >> 4;
  const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
  const bool upper = l16 >= 8;              // this lane holds dims 64..127 of its head
  float wq[8], wk[8];
  qkr_unpack8(*reinterpret_cast<const uint4*>(qw + l16 * 8), wq);
  qkr_unpack8(*reinterpret_cast<const uint4*>(kw + l16 * 8), wk);
  const int npairs = (heads + 1) / 2;
  for (int tok = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; tok < M; tok += warps_per_grid) {
    const int p = pos[tok];
    const int fi = (l16 & 7) * 8;           // frequency index of this lane's first element
    float cs[8], sn[8];
    {
      const float4* c = reinterpret_cast<const float4*>(cos_t + static_cast<size_t>(p) * 64 + fi);
      const float4* s_ = reinterpret_cast<const float4*>(sin_t + static_cast<size_t>(p) * 64 + fi);
      const float4 c0 = c[0], c1 = c[1], s0 = s_[0], s1 = s_[1];
      cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
      sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
    }
    const __nv_bfloat16* row = qkv + static_cast<size_t>(tok) * ld_qkv + l16 * 8;
    const int slot = STORE ? slots[tok] : -1;
    if (STORE && slot >= 0) {
      // values: plain copy of the Hkv value heads, two heads per warp-wide access
      for (int hv = sub; hv < Hkv; hv += 2)
        *reinterpret_cast<uint4*>(v_cache + (static_cast<size_t>(slot) * Hkv + hv) * 128 + l16 * 8) =
            *reinterpret_cast<const uint4*>(row + (heads + hv) * 128);
    }
    for (int hp0 = 0; hp0 < npairs; hp0 += QKR_PAIRS) {
      uint4 raw[QKR_PAIRS];
#pragma unroll
      for (int u = 0; u < QKR_PAIRS; ++u) {
        const int head = min(2 * (hp0 + u) + sub, heads - 1);   // tail units repeat the last head (not stored)
        raw[u] = *reinterpret_cast<const uint4*>(row + head * 128);
      }
#pragma unroll
      for (int u = 0; u < QKR_PAIRS; ++u) {
        const int head = 2 * (hp0 + u) + sub;
        const bool is_q = head < Hq;
        float v[8];
        qkr_unpack8(raw[u], v);
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
        const float rstd = rsqrtf(sum16(ss) * (1.f / 128.f) + eps);
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float n = v[j] * rstd * (is_q ? wq[j] : wk[j]);
          const float partner = __shfl_xor_sync(0xffffffffu, n, 8);
          // first half: y = x1*c - x2*s ; second half: y = x2*c + x1*s
          o[j] = upper ? n * cs[j] + partner * sn[j] : n * cs[j] - partner * sn[j];
        }
        if (head < heads) {
          __nv_bfloat16* dst = is_q ? q_out + (static_cast<size_t>(tok) * Hq + head) * 128 + l16 * 8
                                    : k_out + (static_cast<size_t>(tok) * Hkv + (head - Hq)) * 128 + l16 * 8;
          const uint4 packed = qkr_pack8(o);
          *reinterpret_cast<uint4*>(dst) = packed;
          if (STORE && !is_q && slot >= 0)
            *reinterpret_cast<uint4*>(k_cache + (static_cast<size_t>(slot) * Hkv + (head - Hq)) * 128 + l16 * 8) = packed;
          if (l16 == 0 && rstd_out) rstd_out[static_cast<size_t>(tok) * heads + head] = rstd;
        }
      }
    }
  }
}

// Backward: dq/dk (post-RoPE grads) -> grads w.r.t. the projection output (written into dqkv's q and
// k column ranges) and partial weight grads accumulated with fp32 atomics into dqw/dkw [128].
__global__ void __launch_bounds__(256) qknorm_rope_bwd_kernel(
    const __nv_bfloat16* __restrict__ dq, const __nv_bfloat16* __restrict__ dk,
    const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ qw,
    const __nv_bfloat16* __restrict__ kw, const int* __restrict__ pos,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t,
    const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dqkv, float* __restrict__ dqw,
    float* __restrict__ dkw, int M, int Hq, int Hkv, int ld_qkv) {
  __shared__ float sdw[2][128];
  for (int i = threadIdx.x; i < 256; i += blockDim.x) (&sdw[0][0])[i] = 0.f;
  __syncthreads();
  const int heads = Hq + Hkv;
  const int lane = threadIdx.x & 31, l16 = lane & 15, sub = lane >> 4;
  const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
  const bool upper = l16 >= 8;
  // a lane always owns the same eight head dimensions: weight gradients accumulate in registers
  float dwq[8], dwk[8], wq[8], wk[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) dwq[j] = dwk[j] = 0.f;
  qkr_unpack8(*reinterpret_cast<const uint4*>(qw + l16 * 8), wq);
  qkr_unpack8(*reinterpret_cast<const uint4*>(kw + l16 * 8), wk);
  const int npairs = (heads + 1) / 2;
  for (int tok = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; tok < M; tok += warps_per_grid) {
    const int p = pos[tok];
    const int fi = (l16 & 7) * 8;
    float cs[8], sn[8];
    {
      const float4* c = reinterpret_cast<const float4*>(cos_t + static_cast<size_t>(p) * 64 + fi);
      const float4* s_ = reinterpret_cast<const float4*>(sin_t + static_cast<size_t>(p) * 64 + fi);
      const float4 c0 = c[0], c1 = c[1], s0 = s_[0], s1 = s_[1];
      cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
      sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
    }
    const size_t xoff = static_cast<size_t>(tok) * ld_qkv + l16 * 8;
    for (int hp0 = 0; hp0 < npairs; hp0 += QKR_PAIRS) {
      uint4 graw[QKR_PAIRS], xraw[QKR_PAIRS];
      float rs[QKR_PAIRS];
#pragma unroll
      for (int u = 0; u < QKR_PAIRS; ++u) {
        const int head = min(2 * (hp0 + u) + sub, heads - 1);   // tail units repeat the last head (masked below)
        const __nv_bfloat16* gsrc = head < Hq ? dq + (static_cast<size_t>(tok) * Hq + head) * 128 + l16 * 8
                                              : dk + (static_cast<size_t>(tok) * Hkv + (head - Hq)) * 128 + l16 * 8;
        graw[u] = *reinterpret_cast<const uint4*>(gsrc);
        xraw[u] = *reinterpret_cast<const uint4*>(qkv + xoff + head * 128);
        rs[u] = rstd_in[static_cast<size_t>(tok) * heads + head];
      }
#pragma unroll
      for (int u = 0; u < QKR_PAIRS; ++u) {
        const int head = 2 * (hp0 + u) + sub;
        const bool live = head < heads;
        const bool is_q = head < Hq;
        float g[8], xv[8], xh[8], gw_[8];
        qkr_unpack8(graw[u], g);
        qkr_unpack8(xraw[u], xv);
        const float rstd = rs[u];
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float partner = __shfl_xor_sync(0xffffffffu, g[j], 8);
          // inverse rotation: dx1 = dy1*c + dy2*s ; dx2 = dy2*c - dy1*s
          const float dn = upper ? g[j] * cs[j] - partner * sn[j] : g[j] * cs[j] + partner * sn[j];
          xh[j] = xv[j] * rstd;
          gw_[j] = dn * (is_q ? wq[j] : wk[j]);
          dot += gw_[j] * xh[j];
          if (live) {
            if (is_q) dwq[j] += dn * xh[j];
            else dwk[j] += dn * xh[j];
          }
        }
        dot = sum16(dot) * (1.f / 128.f);
        if (live) {
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = rstd * (gw_[j] - xh[j] * dot);
          *reinterpret_cast<uint4*>(dqkv + xoff + head * 128) = qkr_pack8(o);
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    atomicAdd(&sdw[0][l16 * 8 + j], dwq[j]);
    atomicAdd(&sdw[1][l16 * 8 + j], dwk[j]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 128; i += blockDim.x) {
    atomicAdd(dqw + i, sdw[0][i]);
    atomicAdd(dkw + i, sdw[1][i]);
  }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU on the fused gate|up projection output gu [M, 2I]: out = silu(gate) * up.
// ---------------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                  long long M, int I) {
  const int nvec = I / 8;
  const long long total = M * nvec;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / nvec;
    const int c = static_cast<int>(i % nvec) * 8;
    float g[8], u[8], o[8];
    load8(gu + row * 2 * I + c, g);
    load8(gu + row * 2 * I + I + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    store8(out + row * I + c, o);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout,
                                  const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ dgu,
                                  long long M, int I) {
  const int nvec = I / 8;
  const long long total = M * nvec;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / nvec;
    const int c = static_cast<int>(i % nvec) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + row * 2 * I + c, g);
    load8(gu + row * 2 * I + I + c, u);
    load8(dout + row * I + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * s;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * (s + silu * (1.f - s));
    }
    store8(dgu + row * 2 * I + c, dg);
    store8(dgu + row * 2 * I + I + c, du);
  }
}

// ---------------------------------------------------------------------------------------------
// Embedding gather and scatter-add (bf16 weights / grads; ids int64).
// ---------------------------------------------------------------------------------------------
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids,
                                     const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, int M, int H) {
  const int nvec = H / 8;
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    const long long id = ids[row];
    const bf16x8* src = reinterpret_cast<const bf16x8*>(table + id * H);
    bf16x8* dst = reinterpret_cast<bf16x8*>(out + static_cast<size_t>(row) * H);
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) dst[c] = src[c];
  }
}
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids,
                                     const __nv_bfloat16* __restrict__ dout,
                                     __nv_bfloat16* __restrict__ dtable, int M, int H) {
  const int npair = H / 2;
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    const long long id = ids[row];
    const __nv_bfloat162* src = reinterpret_cast<const __nv_bfloat162*>(dout + static_cast<size_t>(row) * H);
    __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(dtable + id * H);
    for (int c = threadIdx.x; c < npair; c += blockDim.x) atomicAdd(dst + c, src[c]);
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

B2_EXPORT int b2_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int M, int H, float eps,
                             void* stream) {
  b2::ensure_thread_context();
  if (H % 8) { set_error("rmsnorm: H %% 8 != 0"); return 10; }
  if (M <= 0) return 0;
  if (H <= 2048) {
    int blocks = (M + 7) / 8;
    const int cap = num_sms() * 16;
    if (blocks > cap) blocks = cap;
    auto xs = static_cast<const __nv_bfloat16*>(x);
    auto ws = static_cast<const __nv_bfloat16*>(w);
    auto ys = static_cast<__nv_bfloat16*>(y);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (H <= 1024) rmsnorm_fwd_warp_kernel<4><<<blocks, 256, 0, st>>>(xs, ws, ys, rstd, M, H, eps);
    else rmsnorm_fwd_warp_kernel<8><<<blocks, 256, 0, st>>>(xs, ws, ys, rstd, M, H, eps);
    B2_LAUNCH_CHECK("rmsnorm_fwd");
    return 0;
  }
  rmsnorm_fwd_kernel<<<M, RMS_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<__nv_bfloat16*>(y), rstd, H, eps);
  B2_LAUNCH_CHECK("rmsnorm_fwd");
  return 0;
}

// dw_partial: fp32 scratch of at least b2_rmsnorm_bwd_ctas() * H floats.
B2_EXPORT int b2_rmsnorm_bwd_ctas() {
  b2::ensure_thread_context(); return num_sms() * 2; }

B2_EXPORT int b2_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                             void* dw, float* dw_partial, int M, int H, int add_to_dx,
                             int accumulate_dw, int dw_fp32, void* stream_) {
  b2::ensure_thread_context();
  if (H % 8 || H > RMS_THREADS * 8 * RMS_MAX_VEC) { set_error("rmsnorm_bwd: H must be a multiple of 8 and <= 8192"); return 10; }
  if (M <= 0) return 0;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int ctas = num_sms() * 2;
  if (ctas > M) ctas = M;
  if (H <= 2048 && 256 % (H / 8) == 0) {
    auto dys = static_cast<const __nv_bfloat16*>(dy);
    auto xs = static_cast<const __nv_bfloat16*>(x);
    auto ws = static_cast<const __nv_bfloat16*>(w);
    auto dxs = static_cast<__nv_bfloat16*>(dx);
    int blocks = (M + 7) / 8;
    const int cap = num_sms() * 8;
    if (blocks > cap) blocks = cap;
    if (H <= 1024) rmsnorm_bwd_dx_kernel<4><<<blocks, 256, 0, stream>>>(dys, xs, ws, rstd, dxs, M, H, add_to_dx);
    else rmsnorm_bwd_dx_kernel<8><<<blocks, 256, 0, stream>>>(dys, xs, ws, rstd, dxs, M, H, add_to_dx);
    B2_LAUNCH_CHECK("rmsnorm_bwd_dx");
    const int dw_ctas = ctas > num_sms() ? num_sms() : ctas;
    rmsnorm_bwd_dw_kernel<<<dw_ctas, 256, H * static_cast<int>(sizeof(float)), stream>>>(dys, xs, rstd, dw_partial, M, H);
    B2_LAUNCH_CHECK("rmsnorm_bwd_dw");
    reduce_partials_kernel<<<(H + 31) / 32, 256, 0, stream>>>(dw_partial, dw, dw_ctas, H, accumulate_dw, dw_fp32);
    B2_LAUNCH_CHECK("rmsnorm_bwd_reduce");
    return 0;
  }
  rmsnorm_bwd_kernel<<<ctas, RMS_THREADS, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
      static_cast<const __nv_bfloat16*>(w), rstd, static_cast<__nv_bfloat16*>(dx), dw_partial, M, H,
      add_to_dx);
  B2_LAUNCH_CHECK("rmsnorm_bwd");
  reduce_partials_kernel<<<(H + 31) / 32, 256, 0, stream>>>(dw_partial, dw, ctas, H, accumulate_dw, dw_fp32);
  B2_LAUNCH_CHECK("rmsnorm_bwd_reduce");
  return 0;
}

B2_EXPORT int b2_qknorm_rope_fwd(const void* qkv, const void* qw, const void* kw, const int* pos,
                                 const float* cos_t, const float* sin_t, void* q_out, void* k_out,
                                 float* rstd, int M, int Hq, int Hkv, int head_dim, int ld_qkv, float eps,
                                 void* stream) {
  b2::ensure_thread_context();
  if (head_dim != 128) { set_error("qknorm_rope: head_dim must be 128"); return 10; }
  if (M <= 0) return 0;
  long long blocks = (static_cast<long long>(M) + 7) / 8;   // one warp per token
  const long long fcap = static_cast<long long>(num_sms()) * 16;
  if (blocks > fcap) blocks = fcap;
  qknorm_rope_fwd_kernel<false><<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(qw),
      static_cast<const __nv_bfloat16*>(kw), pos, cos_t, sin_t, static_cast<__nv_bfloat16*>(q_out),
      static_cast<__nv_bfloat16*>(k_out), rstd, M, Hq, Hkv, ld_qkv, eps, nullptr, nullptr, nullptr);
  B2_LAUNCH_CHECK("qknorm_rope_fwd");
  return 0;
}

// Inference form: QK-norm + RoPE + store of the new K / V rows into a bf16 paged cache ([rows, Hkv, 128], row =
// block * block_size + offset) in one launch.  slots: int32 [M], negative = no store (padding rows of a graph batch).
B2_EXPORT int b2_qknorm_rope_store(const void* qkv, const void* qw, const void* kw, const int* pos,
                                   const float* cos_t, const float* sin_t, void* q_out, void* k_out, int M, int Hq,
                                   int Hkv, int head_dim, int ld_qkv, float eps, const int* slots, void* k_cache,
                                   void* v_cache, void* stream) {
  b2::ensure_thread_context();
  if (head_dim != 128) { set_error("qknorm_rope_store: head_dim must be 128"); return 10; }
  if (slots == nullptr || k_cache == nullptr || v_cache == nullptr) {
    set_error("qknorm_rope_store: slots and both caches are required");
    return 10;
  }
  if (M <= 0) return 0;
  long long blocks = (static_cast<long long>(M) + 7) / 8;   // one warp per token
  const long long fcap = static_cast<long long>(num_sms()) * 16;
  if (blocks > fcap) blocks = fcap;
  qknorm_rope_fwd_kernel<true><<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(qw),
      static_cast<const __nv_bfloat16*>(kw), pos, cos_t, sin_t, static_cast<__nv_bfloat16*>(q_out),
      static_cast<__nv_bfloat16*>(k_out), nullptr, M, Hq, Hkv, ld_qkv, eps, slots,
      static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache));
  B2_LAUNCH_CHECK("qknorm_rope_store");
  return 0;
}

// dqw / dkw: fp32 [128] accumulators (caller zeroes them or accumulates across micro-batches).
B2_EXPORT int b2_qknorm_rope_bwd(const void* dq, const void* dk, const void* qkv, const void* qw,
                                 const void* kw, const int* pos, const float* cos_t, const float* sin_t,
                                 const float* rstd, void* dqkv, float* dqw, float* dkw, int M, int Hq,
                                 int Hkv, int head_dim, int ld_qkv, void* stream) {
  b2::ensure_thread_context();
  if (head_dim != 128) { set_error("qknorm_rope: head_dim must be 128"); return 10; }
  if (M <= 0) return 0;
  long long blocks = (static_cast<long long>(M) + 7) / 8;   // one warp per token
  const long long cap = static_cast<long long>(num_sms()) * 8;
  if (blocks > cap) blocks = cap;
  qknorm_rope_bwd_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dq), static_cast<const __nv_bfloat16*>(dk),
      static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(qw),
      static_cast<const __nv_bfloat16*>(kw), pos, cos_t, sin_t, rstd, static_cast<__nv_bfloat16*>(dqkv),
      dqw, dkw, M, Hq, Hkv, ld_qkv);
  B2_LAUNCH_CHECK("qknorm_rope_bwd");
  return 0;
}

B2_EXPORT int b2_swiglu_fwd(const void* gu, void* out, long long M, int I, void* stream) {
  b2::ensure_thread_context();
  if (I % 8) { set_error("swiglu: I %% 8 != 0"); return 10; }
  if (M <= 0) return 0;
  const long long total = M * (I / 8);
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(num_sms()) * 16;
  if (blocks > cap) blocks = cap;
  swiglu_fwd_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(out), M, I);
  B2_LAUNCH_CHECK("swiglu_fwd");
  return 0;
}
B2_EXPORT int b2_swiglu_bwd(const void* dout, const void* gu, void* dgu, long long M, int I, void* stream) {
  b2::ensure_thread_context();
  if (I % 8) { set_error("swiglu: I %% 8 != 0"); return 10; }
  if (M <= 0) return 0;
  const long long total = M * (I / 8);
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(num_sms()) * 16;
  if (blocks > cap) blocks = cap;
  swiglu_bwd_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(gu),
      static_cast<__nv_bfloat16*>(dgu), M, I);
  B2_LAUNCH_CHECK("swiglu_bwd");
  return 0;
}

B2_EXPORT int b2_embedding_fwd(const long long* ids, const void* table, void* out, int M, int H, void* stream) {
  b2::ensure_thread_context();
  if (H % 8) { set_error("embedding: H %% 8 != 0"); return 10; }
  if (M <= 0) return 0;
  int blocks = M < num_sms() * 8 ? M : num_sms() * 8;
  embedding_fwd_kernel<<<blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), M, H);
  B2_LAUNCH_CHECK("embedding_fwd");
  return 0;
}
B2_EXPORT int b2_embedding_bwd(const long long* ids, const void* dout, void* dtable, int M, int H, void* stream) {
  b2::ensure_thread_context();
  if (H % 8) { set_error("embedding: H %% 8 != 0"); return 10; }
  if (M <= 0) return 0;
  int blocks = M < num_sms() * 8 ? M : num_sms() * 8;
  embedding_bwd_kernel<<<blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, static_cast<const __nv_bfloat16*>(dout), static_cast<__nv_bfloat16*>(dtable), M, H);
  B2_LAUNCH_CHECK("embedding_bwd");
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the RMSNorm backward (declared and documented in no_alloc.h).
// ---------------------------------------------------------------------------------------------
#include "no_alloc.h"

// Per-CTA partial sums of the weight gradient.  In host code this name is only a handle for the
// runtime's symbol lookup, never a device address: the address is fetched once per device below.
static __device__ __align__(256) float g_noalloc_dw_partial[B2_NOALLOC_MAX_PARTIALS * B2_NOALLOC_MAX_H];

static float* noalloc_scratch_ptr() {
  static std::atomic<float*> ptrs[64];   // zero-initialised; racing first calls store the same address
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("rmsnorm_bwd_noalloc: cannot determine the current device");
    return nullptr;
  }
  float* p = ptrs[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_dw_partial);
    if (e != cudaSuccess || p == nullptr) {
      set_error("rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    ptrs[dev].store(p, std::memory_order_release);
  }
  return p;
}

B2_EXPORT int b2_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                     void* dx, void* dw, int M, int H, int add_to_dx, int accumulate_dw,
                                     int dw_fp32, void* stream_) {
  b2::ensure_thread_context();
  if (H <= 0 || H % 8 != 0 || H > B2_NOALLOC_MAX_H || 256 % (H / 8) != 0) {
    set_error("rmsnorm_bwd_noalloc: H=%d is outside the built-in scratch (multiple of 8, <= %d, 256 %% (H/8) == 0)",
              H, B2_NOALLOC_MAX_H);
    return 10;
  }
  if (M < 0) {
    set_error("rmsnorm_bwd_noalloc: M=%d is negative", M);
    return 10;
  }
  if (M == 0) return 0;
  if (!dy || !x || !w || !rstd || !dx || !dw) {
    set_error("rmsnorm_bwd_noalloc: null pointer (dy=%p x=%p w=%p rstd=%p dx=%p dw=%p)", dy, x, w,
              static_cast<const void*>(rstd), dx, dw);
    return 10;
  }
  float* partial = noalloc_scratch_ptr();   // first call per device: symbol lookup (not during capture)
  if (partial == nullptr) return 3;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int dw_ctas = num_sms();
  if (dw_ctas > B2_NOALLOC_MAX_PARTIALS) dw_ctas = B2_NOALLOC_MAX_PARTIALS;
  if (dw_ctas > M) dw_ctas = M;
  auto dys = static_cast<const __nv_bfloat16*>(dy);
  auto xs = static_cast<const __nv_bfloat16*>(x);
  auto ws = static_cast<const __nv_bfloat16*>(w);
  auto dxs = static_cast<__nv_bfloat16*>(dx);
  int blocks = (M + 7) / 8;
  const int cap = num_sms() * 8;
  if (blocks > cap) blocks = cap;
  if (H <= 1024) rmsnorm_bwd_dx_kernel<4><<<blocks, 256, 0, stream>>>(dys, xs, ws, rstd, dxs, M, H, add_to_dx);
  else rmsnorm_bwd_dx_kernel<8><<<blocks, 256, 0, stream>>>(dys, xs, ws, rstd, dxs, M, H, add_to_dx);
  B2_LAUNCH_CHECK("rmsnorm_bwd_noalloc(dx)");
  // every CTA writes its whole [H] row of partials, so stale contents of the shared array are never read
  rmsnorm_bwd_dw_kernel<<<dw_ctas, 256, H * static_cast<int>(sizeof(float)), stream>>>(dys, xs, rstd, partial, M, H);
  B2_LAUNCH_CHECK("rmsnorm_bwd_noalloc(dw)");
  reduce_partials_kernel<<<(H + 31) / 32, 256, 0, stream>>>(partial, dw, dw_ctas, H, accumulate_dw, dw_fp32);
  B2_LAUNCH_CHECK("rmsnorm_bwd_noalloc(reduce)");
  return 0;
}
