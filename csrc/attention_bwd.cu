// Causal flash-attention backward for sm_100a (head_dim 128, GQA) on tcgen05 / TMEM.
//
// Three kernels:
//   attn_bwd_prep   D[h,t] = sum_d dO*O                                   (HBM-bound)
//   attn_bwd_dkdv   one CTA per (128-row kv tile, kv head, batch); streams 64-row Q/dO tiles of every
//                   q head of the group; S^T = K Q^T and dP^T = V dO^T land in TMEM with kv on the
//                   lanes, so P^T and dS^T are written to shared memory directly as K-major A
//                   operands of dV += P^T dO and dK += dS^T Q (dO / Q tiles are re-read MN-major).
//   attn_bwd_dq     one CTA per (128-row q tile, q head, batch); streams 64-row K/V tiles;
//                   S = Q K^T, dP = dO V^T, dQ += dS K.
// S/dP accumulators are double-buffered in TMEM so the MMAs of step i+1 overlap the elementwise
// work of step i.  The elementwise work (exp2, dS, bf16 pack, swizzled shared-memory stores) is the
// critical path, so eight warps share it: warps 2..5 take columns 0..31 of every 64-column tile,
// warps 6..9 columns 32..63 (a warp may touch the TMEM lane quarter warp%4, which both groups cover).  Recomputing S and dP in both kernels costs 7 instead of 5 GEMMs per tile pair
// but needs no atomics and is deterministic.
#include "common.cuh"
#include "host.h"

namespace b2 {

constexpr int ATB_THREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2..9 elementwise (two column halves)

__device__ __forceinline__ void ew_barrier() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
constexpr float LOG2E = 1.4426950408889634f;

// ---------------------------------------------------------------------------------------------
__global__ void attn_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o,
                                     const __nv_bfloat16* __restrict__ d_o, float* __restrict__ D,
                                     long long T, int Hq) {
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= T * Hq) return;
  const long long t = gw / Hq;
  const int h = static_cast<int>(gw % Hq);
  const size_t off = (static_cast<size_t>(t) * Hq + h) * 128 + lane * 4;
  uint2 a = *reinterpret_cast<const uint2*>(o + off);
  uint2 b = *reinterpret_cast<const uint2*>(d_o + off);
  float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y);
  float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
  s = warp_sum(s);
  if (lane == 0) D[static_cast<size_t>(h) * T + t] = s;
}

// ---------------------------------------------------------------------------------------------
constexpr int ATB_STAGES = 3;   // streamed-tile ring depth: TMA latency spans about two iterations

struct DkDvSmem {
  static constexpr int K = 0;                 // 32 KiB  [128 x 128]
  static constexpr int V = K + 32768;         // 32 KiB
  static constexpr int Q = V + 32768;         // STAGES x 16 KiB [64 x 128]
  static constexpr int DO = Q + ATB_STAGES * 16384;    // STAGES x 16 KiB
  static constexpr int PT = DO + ATB_STAGES * 16384;   // 2 x 16 KiB [128 x 64]
  static constexpr int DST = PT + 2 * 16384;  // 2 x 16 KiB
  static constexpr int BARS = DST + 2 * 16384;
  static constexpr int TOTAL = BARS + 144 + 1024 /*lse, D*/ + 1024;
};

__global__ void __launch_bounds__(ATB_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ64, const __grid_constant__ CUtensorMap tmdO64,
                     const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     const float* __restrict__ lse, const float* __restrict__ Dsum,
                     __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv, int ld_dk, int ld_dv,
                     int S, int Hq, int Hkv, float scale, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DkDvSmem::BARS);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;    // [3]
  uint64_t* qdo_empty = bars + 4;   // [3]
  uint64_t* sdp_full = bars + 7;    // [2]
  uint64_t* sdp_empty = bars + 9;   // [2]
  uint64_t* pds_full = bars + 11;   // [2]
  uint64_t* pds_empty = bars + 13;  // [2]
  uint64_t* acc_done = bars + 15;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  float* s_lse = reinterpret_cast<float*>(bars + 18);   // [2][64], pre-multiplied by log2(e)
  float* s_D = s_lse + 128;                             // [2][64]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jt = blockIdx.x;  // kv tile (128 rows); light tiles (large jt) are scheduled last anyway
  const int kvh = blockIdx.y, batch = blockIdx.z;
  const int G = Hq / Hkv;
  const int T = gridDim.z * S;
  const int nq64 = (S + 63) / 64;
  const int i_begin = 2 * jt;  // first 64-row q tile that can see this kv tile
  const int per_head = nq64 - i_begin;
  const int n_it = per_head > 0 ? per_head * G : 0;
  const int kv_row0 = batch * S + jt * 128;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < ATB_STAGES; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sdp_full[i], 1);
      mbar_init(&sdp_empty[i], 256);
      mbar_init(&pds_full[i], 256);
      mbar_init(&pds_empty[i], 1);
    }
    mbar_init(acc_done, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const uint32_t tmem_ST = tmem_base;         // 2 x 64
  const uint32_t tmem_DPT = tmem_base + 128;  // 2 x 64
  const uint32_t tmem_DV = tmem_base + 256;   // 128
  const uint32_t tmem_DK = tmem_base + 384;   // 128

  if (warp == 0) {
    if (lane == 0 && n_it > 0) {
      mbar_expect_tx(kv_full, 65536);
      tma_load_2d(smem + DkDvSmem::K, &tmK, kv_full, kvh * 128, kv_row0);
      tma_load_2d(smem + DkDvSmem::K + 16384, &tmK, kv_full, kvh * 128 + 64, kv_row0);
      tma_load_2d(smem + DkDvSmem::V, &tmV, kv_full, kvh * 128, kv_row0);
      tma_load_2d(smem + DkDvSmem::V + 16384, &tmV, kv_full, kvh * 128 + 64, kv_row0);
      for (int it = 0; it < n_it; ++it) {
        const int st = it % ATB_STAGES;
        const uint32_t ph = (it / ATB_STAGES) & 1;
        const int head = kvh * G + it / per_head;
        const int qrow = batch * S + (i_begin + it % per_head) * 64;
        if (!mbar_wait(&qdo_empty[st], ph ^ 1, status, ERR_ATTN_WAIT)) break;
        uint8_t* sQ = smem + DkDvSmem::Q + st * 16384;
        uint8_t* sdO = smem + DkDvSmem::DO + st * 16384;
        mbar_expect_tx(&qdo_full[st], 32768);
        tma_load_2d(sQ, &tmQ64, &qdo_full[st], head * 128, qrow);
        tma_load_2d(sQ + 8192, &tmQ64, &qdo_full[st], head * 128 + 64, qrow);
        tma_load_2d(sdO, &tmdO64, &qdo_full[st], head * 128, qrow);
        tma_load_2d(sdO + 8192, &tmdO64, &qdo_full[st], head * 128 + 64, qrow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(1, 128, 64, 0, 0);     // [128 kv] x [64 q], K = d
      constexpr uint32_t idesc_acc = make_idesc_f16(1, 128, 128, 0, 1);  // [128 kv] x [128 d], K = q
      const uint32_t k_base = smem_u32(smem + DkDvSmem::K);
      const uint32_t v_base = smem_u32(smem + DkDvSmem::V);
      auto issue_sdp = [&](int it) {
        const int st = it & 1;
        const int ks = it % ATB_STAGES;
        const uint32_t q_base = smem_u32(smem + DkDvSmem::Q + ks * 16384);
        const uint32_t do_base = smem_u32(smem + DkDvSmem::DO + ks * 16384);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t oa = (ks >> 2) * 16384 + (ks & 3) * 32;
          const uint32_t ob = (ks >> 2) * 8192 + (ks & 3) * 32;
          umma_f16_ss(tmem_ST + st * 64, make_smem_desc_sw128(k_base + oa, 16, 1024),
                      make_smem_desc_sw128(q_base + ob, 16, 1024), idesc_s, ks != 0);
        }
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t oa = (ks >> 2) * 16384 + (ks & 3) * 32;
          const uint32_t ob = (ks >> 2) * 8192 + (ks & 3) * 32;
          umma_f16_ss(tmem_DPT + st * 64, make_smem_desc_sw128(v_base + oa, 16, 1024),
                      make_smem_desc_sw128(do_base + ob, 16, 1024), idesc_s, ks != 0);
        }
        umma_commit(&sdp_full[st]);
      };
      bool ok = mbar_wait(kv_full, 0, status, ERR_ATTN_WAIT) &&
                mbar_wait(&qdo_full[0], 0, status, ERR_ATTN_WAIT);
      if (ok) {
        tc_fence_after();
        issue_sdp(0);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        if (it + 1 < n_it) {
          const int st = (it + 1) & 1;
          const uint32_t ph = ((it + 1) >> 1) & 1;
          if (!mbar_wait(&qdo_full[(it + 1) % ATB_STAGES], ((it + 1) / ATB_STAGES) & 1, status, ERR_ATTN_WAIT) ||
              !mbar_wait(&sdp_empty[st], ph ^ 1, status, ERR_ATTN_WAIT)) {
            ok = false;
            break;
          }
          tc_fence_after();
          issue_sdp(it + 1);
        }
        const int st = it & 1;
        if (!mbar_wait(&pds_full[st], (it >> 1) & 1, status, ERR_ATTN_WAIT)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t pt_base = smem_u32(smem + DkDvSmem::PT + st * 16384);
        const uint32_t dst_base = smem_u32(smem + DkDvSmem::DST + st * 16384);
        const int kst = it % ATB_STAGES;
        const uint32_t q_base = smem_u32(smem + DkDvSmem::Q + kst * 16384);
        const uint32_t do_base = smem_u32(smem + DkDvSmem::DO + kst * 16384);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_f16_ss(tmem_DV, make_smem_desc_sw128(pt_base + ks * 32, 16, 1024),
                      make_smem_desc_sw128(do_base + ks * 2048, 8192, 1024), idesc_acc, (it | ks) != 0);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_f16_ss(tmem_DK, make_smem_desc_sw128(dst_base + ks * 32, 16, 1024),
                      make_smem_desc_sw128(q_base + ks * 2048, 8192, 1024), idesc_acc, (it | ks) != 0);
        umma_commit(&qdo_empty[kst]);
        umma_commit(&pds_empty[st]);
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;           // which 32 columns of the 64-column tile
    const int etid = (warp - 2) * 32 + lane;    // 0..255 among the elementwise threads
    const int r = quarter * 32 + lane;          // kv row in tile
    const int kv_pos = jt * 128 + r;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = scale * LOG2E;
    bool ok = n_it > 0;
    for (int it = 0; it < n_it; ++it) {
      const int st = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      const int head = kvh * G + it / per_head;
      const int q0 = (i_begin + it % per_head) * 64;  // first q position of this tile
      // stage this tile's row statistics (64 q positions) in shared memory
      if (etid < 128) {
        const int c = etid & 63;
        const int qc = min(q0 + c, S - 1);
        const size_t o = static_cast<size_t>(head) * T + batch * S + qc;
        if (etid < 64) s_lse[st * 64 + c] = lse[o] * LOG2E;
        else s_D[st * 64 + c] = Dsum[o];
      }
      ew_barrier();   // every elementwise thread reaches this each iteration, also after a failed wait
      if (ok) ok = mbar_wait(&sdp_full[st], ph, status, ERR_ATTN_WAIT);
      if (!ok) continue;
      tc_fence_after();
      uint32_t ts[32], tp[32];
      tmem_ld_32x32b_x32(tmem_ST + lane_off + st * 64 + half * 32, ts);
      tmem_ld_32x32b_x32(tmem_DPT + lane_off + st * 64 + half * 32, tp);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&sdp_empty[st]);
      const float* lse_s = s_lse + st * 64 + half * 32;
      const float* D_s = s_D + st * 64 + half * 32;
      const int qb = q0 + half * 32;
      const bool need_mask = (qb < jt * 128 + 128) || (qb + 32 > S) || (jt * 128 + 128 > S);
      float pv[32], dsv[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float p = exp2f(__uint_as_float(ts[c]) * sl2 - lse_s[c]);
        if (need_mask) {
          const int qp = qb + c;
          if (!((qp < S) && (kv_pos <= qp) && (kv_pos < S))) p = 0.f;
        }
        pv[c] = p;
        dsv[c] = p * (__uint_as_float(tp[c]) - D_s[c]) * scale;
      }
      ok = mbar_wait(&pds_empty[st], ph ^ 1, status, ERR_ATTN_WAIT);
      if (!ok) continue;
      uint8_t* sPT = smem + DkDvSmem::PT + st * 16384 + r * 128;
      uint8_t* sDST = smem + DkDvSmem::DST + st * 16384 + r * 128;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        uint4 a, b;
        a.x = pack_bf16x2(pv[c4 * 8 + 0], pv[c4 * 8 + 1]);
        a.y = pack_bf16x2(pv[c4 * 8 + 2], pv[c4 * 8 + 3]);
        a.z = pack_bf16x2(pv[c4 * 8 + 4], pv[c4 * 8 + 5]);
        a.w = pack_bf16x2(pv[c4 * 8 + 6], pv[c4 * 8 + 7]);
        b.x = pack_bf16x2(dsv[c4 * 8 + 0], dsv[c4 * 8 + 1]);
        b.y = pack_bf16x2(dsv[c4 * 8 + 2], dsv[c4 * 8 + 3]);
        b.z = pack_bf16x2(dsv[c4 * 8 + 4], dsv[c4 * 8 + 5]);
        b.w = pack_bf16x2(dsv[c4 * 8 + 6], dsv[c4 * 8 + 7]);
        const int sw = (((half * 4 + c4) ^ (r & 7)) << 4);
        *reinterpret_cast<uint4*>(sPT + sw) = a;
        *reinterpret_cast<uint4*>(sDST + sw) = b;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&pds_full[st]);
    }
    // write-out: the first column group stores dV, the second dK
    const bool in_range = kv_pos < S;
    __nv_bfloat16* orow = half ? dk + static_cast<size_t>(kv_row0 + r) * ld_dk + kvh * 128
                               : dv + static_cast<size_t>(kv_row0 + r) * ld_dv + kvh * 128;
    if (n_it == 0) {
      if (in_range) {
        const uint4 z = make_uint4(0, 0, 0, 0);
        for (int c = 0; c < 16; ++c) *reinterpret_cast<uint4*>(orow + c * 8) = z;
      }
    } else if (ok && mbar_wait(acc_done, 0, status, ERR_ATTN_WAIT)) {
      tc_fence_after();
      const uint32_t tb = (half ? tmem_DK : tmem_DV) + lane_off;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t t[32];
        tmem_ld_32x32b_x32(tb + c * 32, t);
        tmem_ld_wait();
        if (in_range) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(t[v * 8 + 0]), __uint_as_float(t[v * 8 + 1]));
            o.y = pack_bf16x2(__uint_as_float(t[v * 8 + 2]), __uint_as_float(t[v * 8 + 3]));
            o.z = pack_bf16x2(__uint_as_float(t[v * 8 + 4]), __uint_as_float(t[v * 8 + 5]));
            o.w = pack_bf16x2(__uint_as_float(t[v * 8 + 6]), __uint_as_float(t[v * 8 + 7]));
            *reinterpret_cast<uint4*>(orow + c * 32 + v * 8) = o;
          }
        }
      }
    }
  }

  if (*reinterpret_cast<volatile int*>(status) != 0) {
    unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------
struct DqSmem {
  static constexpr int Q = 0;                // 32 KiB [128 x 128]
  static constexpr int DO = Q + 32768;       // 32 KiB
  static constexpr int K = DO + 32768;       // STAGES x 16 KiB [64 x 128]
  static constexpr int V = K + ATB_STAGES * 16384;    // STAGES x 16 KiB
  static constexpr int DS = V + ATB_STAGES * 16384;   // 2 x 16 KiB [128 x 64]
  static constexpr int BARS = DS + 2 * 16384;
  static constexpr int TOTAL = BARS + 256 + 1024;
};

__global__ void __launch_bounds__(ATB_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmK64, const __grid_constant__ CUtensorMap tmV64,
                   const float* __restrict__ lse, const float* __restrict__ Dsum,
                   __nv_bfloat16* __restrict__ dq, int S, int Hq, int Hkv, float scale, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DqSmem::BARS);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;    // [3]
  uint64_t* kv_empty = bars + 4;   // [3]
  uint64_t* sdp_full = bars + 7;   // [2]
  uint64_t* sdp_empty = bars + 9;  // [2]
  uint64_t* ds_full = bars + 11;   // [2]
  uint64_t* ds_empty = bars + 13;  // [2]
  uint64_t* acc_done = bars + 15;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_q_tiles = (S + 127) / 128;
  const int qt = num_q_tiles - 1 - blockIdx.x;
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kvh = head / (Hq / Hkv);
  const int T = gridDim.z * S;
  const int nkv64 = (S + 63) / 64;
  const int n_it = min(nkv64, 2 * qt + 2);
  const int row0 = batch * S + qt * 128;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < ATB_STAGES; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sdp_full[i], 1);
      mbar_init(&sdp_empty[i], 256);
      mbar_init(&ds_full[i], 256);
      mbar_init(&ds_empty[i], 1);
    }
    mbar_init(acc_done, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const uint32_t tmem_S = tmem_base;         // 2 x 64
  const uint32_t tmem_DP = tmem_base + 128;  // 2 x 64
  const uint32_t tmem_DQ = tmem_base + 256;  // 128

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 65536);
      tma_load_2d(smem + DqSmem::Q, &tmQ, q_full, head * 128, row0);
      tma_load_2d(smem + DqSmem::Q + 16384, &tmQ, q_full, head * 128 + 64, row0);
      tma_load_2d(smem + DqSmem::DO, &tmdO, q_full, head * 128, row0);
      tma_load_2d(smem + DqSmem::DO + 16384, &tmdO, q_full, head * 128 + 64, row0);
      for (int it = 0; it < n_it; ++it) {
        const int st = it % ATB_STAGES;
        const uint32_t ph = (it / ATB_STAGES) & 1;
        const int krow = batch * S + it * 64;
        if (!mbar_wait(&kv_empty[st], ph ^ 1, status, ERR_ATTN_WAIT)) break;
        uint8_t* sK = smem + DqSmem::K + st * 16384;
        uint8_t* sV = smem + DqSmem::V + st * 16384;
        mbar_expect_tx(&kv_full[st], 32768);
        tma_load_2d(sK, &tmK64, &kv_full[st], kvh * 128, krow);
        tma_load_2d(sK + 8192, &tmK64, &kv_full[st], kvh * 128 + 64, krow);
        tma_load_2d(sV, &tmV64, &kv_full[st], kvh * 128, krow);
        tma_load_2d(sV + 8192, &tmV64, &kv_full[st], kvh * 128 + 64, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(1, 128, 64, 0, 0);     // [128 q] x [64 kv], K = d
      constexpr uint32_t idesc_acc = make_idesc_f16(1, 128, 128, 0, 1);  // [128 q] x [128 d], K = kv
      const uint32_t q_base = smem_u32(smem + DqSmem::Q);
      const uint32_t do_base = smem_u32(smem + DqSmem::DO);
      auto issue_sdp = [&](int it) {
        const int st = it & 1;
        const int ks_ = it % ATB_STAGES;
        const uint32_t k_base = smem_u32(smem + DqSmem::K + ks_ * 16384);
        const uint32_t v_base = smem_u32(smem + DqSmem::V + ks_ * 16384);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t oa = (ks >> 2) * 16384 + (ks & 3) * 32;
          const uint32_t ob = (ks >> 2) * 8192 + (ks & 3) * 32;
          umma_f16_ss(tmem_S + st * 64, make_smem_desc_sw128(q_base + oa, 16, 1024),
                      make_smem_desc_sw128(k_base + ob, 16, 1024), idesc_s, ks != 0);
        }
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t oa = (ks >> 2) * 16384 + (ks & 3) * 32;
          const uint32_t ob = (ks >> 2) * 8192 + (ks & 3) * 32;
          umma_f16_ss(tmem_DP + st * 64, make_smem_desc_sw128(do_base + oa, 16, 1024),
                      make_smem_desc_sw128(v_base + ob, 16, 1024), idesc_s, ks != 0);
        }
        umma_commit(&sdp_full[st]);
      };
      bool ok = mbar_wait(q_full, 0, status, ERR_ATTN_WAIT) &&
                mbar_wait(&kv_full[0], 0, status, ERR_ATTN_WAIT);
      if (ok) {
        tc_fence_after();
        issue_sdp(0);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        if (it + 1 < n_it) {
          const int st = (it + 1) & 1;
          const uint32_t ph = ((it + 1) >> 1) & 1;
          if (!mbar_wait(&kv_full[(it + 1) % ATB_STAGES], ((it + 1) / ATB_STAGES) & 1, status, ERR_ATTN_WAIT) ||
              !mbar_wait(&sdp_empty[st], ph ^ 1, status, ERR_ATTN_WAIT)) {
            ok = false;
            break;
          }
          tc_fence_after();
          issue_sdp(it + 1);
        }
        const int st = it & 1;
        if (!mbar_wait(&ds_full[st], (it >> 1) & 1, status, ERR_ATTN_WAIT)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const int kst = it % ATB_STAGES;
        const uint32_t ds_base = smem_u32(smem + DqSmem::DS + st * 16384);
        const uint32_t k_base = smem_u32(smem + DqSmem::K + kst * 16384);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_f16_ss(tmem_DQ, make_smem_desc_sw128(ds_base + ks * 32, 16, 1024),
                      make_smem_desc_sw128(k_base + ks * 2048, 8192, 1024), idesc_acc, (it | ks) != 0);
        umma_commit(&kv_empty[kst]);
        umma_commit(&ds_empty[st]);
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const int q_pos = qt * 128 + r;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = scale * LOG2E;
    const int qc = q_pos < S ? q_pos : S - 1;
    const float lse_r = lse[static_cast<size_t>(head) * T + batch * S + qc] * LOG2E;
    const float D_r = Dsum[static_cast<size_t>(head) * T + batch * S + qc];
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int st = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      if (!mbar_wait(&sdp_full[st], ph, status, ERR_ATTN_WAIT)) { ok = false; break; }
      tc_fence_after();
      uint32_t ts[32], tp[32];
      tmem_ld_32x32b_x32(tmem_S + lane_off + st * 64 + half * 32, ts);
      tmem_ld_32x32b_x32(tmem_DP + lane_off + st * 64 + half * 32, tp);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&sdp_empty[st]);
      const int k0 = it * 64 + half * 32;
      const bool need_mask = (k0 + 32 > qt * 128) || (k0 + 32 > S) || (qt * 128 + 128 > S);
      float dsv[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float p = exp2f(__uint_as_float(ts[c]) * sl2 - lse_r);
        if (need_mask) {
          const int kp = k0 + c;
          if (!((q_pos < S) && (kp <= q_pos) && (kp < S))) p = 0.f;
        }
        dsv[c] = p * (__uint_as_float(tp[c]) - D_r) * scale;
      }
      if (!mbar_wait(&ds_empty[st], ph ^ 1, status, ERR_ATTN_WAIT)) { ok = false; break; }
      uint8_t* sDS = smem + DqSmem::DS + st * 16384 + r * 128;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        uint4 b;
        b.x = pack_bf16x2(dsv[c4 * 8 + 0], dsv[c4 * 8 + 1]);
        b.y = pack_bf16x2(dsv[c4 * 8 + 2], dsv[c4 * 8 + 3]);
        b.z = pack_bf16x2(dsv[c4 * 8 + 4], dsv[c4 * 8 + 5]);
        b.w = pack_bf16x2(dsv[c4 * 8 + 6], dsv[c4 * 8 + 7]);
        *reinterpret_cast<uint4*>(sDS + (((half * 4 + c4) ^ (r & 7)) << 4)) = b;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&ds_full[st]);
    }
    if (ok && mbar_wait(acc_done, 0, status, ERR_ATTN_WAIT)) {
      tc_fence_after();
      const bool in_range = q_pos < S;
      __nv_bfloat16* orow = dq + (static_cast<size_t>(row0 + r) * Hq + head) * 128 + half * 64;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t t[32];
        tmem_ld_32x32b_x32(tmem_DQ + lane_off + half * 64 + c * 32, t);
        tmem_ld_wait();
        if (in_range) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(t[v * 8 + 0]), __uint_as_float(t[v * 8 + 1]));
            o.y = pack_bf16x2(__uint_as_float(t[v * 8 + 2]), __uint_as_float(t[v * 8 + 3]));
            o.z = pack_bf16x2(__uint_as_float(t[v * 8 + 4]), __uint_as_float(t[v * 8 + 5]));
            o.w = pack_bf16x2(__uint_as_float(t[v * 8 + 6]), __uint_as_float(t[v * 8 + 7]));
            *reinterpret_cast<uint4*>(orow + c * 32 + v * 8) = o;
          }
        }
      }
    }
  }

  if (*reinterpret_cast<volatile int*>(status) != 0) {
    unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace b2

using namespace b2;

// Inputs as in b2_attn_fwd plus out, d_out [T, Hq*128], lse [Hq, T].  Outputs: dq [T, Hq*128];
// dk rows with stride ld_dk, dv rows with stride ld_dv (so both can be column slices of a fused
// gradient buffer).  Dsum: fp32 scratch [Hq, T].
B2_EXPORT int b2_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* d_out,
                          const float* lse, float* Dsum, void* dq, void* dk, void* dv, int B, int S, int Hq,
                          int Hkv, int head_dim, int ld_v, int ld_dk, int ld_dv, float scale, void* stream_) {
  b2::ensure_thread_context();
  if (head_dim != 128 || Hq % Hkv != 0 || (ld_v % 8) || (ld_dk % 8) || (ld_dv % 8)) {
    set_error("attn_bwd: head_dim must be 128, Hq %% Hkv == 0, leading dims %% 8 == 0");
    return 10;
  }
  if (B <= 0 || S <= 0) return 0;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(attn_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             DkDvSmem::TOTAL) != cudaSuccess ||
        cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             DqSmem::TOTAL) != cudaSuccess) {
      set_error("attn_bwd: cannot set shared memory size");
      return 1;
    }
    configured[dev] = true;
  }
  const uint64_t T = static_cast<uint64_t>(B) * S;
  const uint64_t wq = static_cast<uint64_t>(Hq) * 128, wk = static_cast<uint64_t>(Hkv) * 128;
  const CUtensorMap* tq128 = tensor_map_2d_bf16(q, T, wq, wq, 128, 64);
  const CUtensorMap* tq64 = tensor_map_2d_bf16(q, T, wq, wq, 64, 64);
  const CUtensorMap* tdo128 = tensor_map_2d_bf16(d_out, T, wq, wq, 128, 64);
  const CUtensorMap* tdo64 = tensor_map_2d_bf16(d_out, T, wq, wq, 64, 64);
  const CUtensorMap* tk128 = tensor_map_2d_bf16(k, T, wk, wk, 128, 64);
  const CUtensorMap* tk64 = tensor_map_2d_bf16(k, T, wk, wk, 64, 64);
  const CUtensorMap* tv128 = tensor_map_2d_bf16(v, T, wk, ld_v, 128, 64);
  const CUtensorMap* tv64 = tensor_map_2d_bf16(v, T, wk, ld_v, 64, 64);
  if (!tq128 || !tq64 || !tdo128 || !tdo64 || !tk128 || !tk64 || !tv128 || !tv64) return 2;
  int* status = status_ptr();
  if (!status) return 3;
  {
    const long long warps = static_cast<long long>(T) * Hq;
    attn_bwd_prep_kernel<<<static_cast<int>((warps + 7) / 8), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(d_out), Dsum,
        static_cast<long long>(T), Hq);
  }
  const int nt = (S + 127) / 128;
  attn_bwd_dkdv_kernel<<<dim3(nt, Hkv, B), ATB_THREADS, DkDvSmem::TOTAL, stream>>>(
      *tq64, *tdo64, *tk128, *tv128, lse, Dsum, static_cast<__nv_bfloat16*>(dk),
      static_cast<__nv_bfloat16*>(dv), ld_dk, ld_dv, S, Hq, Hkv, scale, status);
  attn_bwd_dq_kernel<<<dim3(nt, Hq, B), ATB_THREADS, DqSmem::TOTAL, stream>>>(
      *tq128, *tdo128, *tk64, *tv64, lse, Dsum, static_cast<__nv_bfloat16*>(dq), S, Hq, Hkv, scale, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("attn_bwd launch failed: %s", cudaGetErrorString(e));
    return 4;
  }
  return 0;
}
