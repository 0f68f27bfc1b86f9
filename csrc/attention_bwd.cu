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

constexpr int ATB_THREADS = 352;  // warp 0 TMA, warps 1 and 10 MMA issue, warps 2..9 elementwise (two groups)

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
  static constexpr int TOTAL = BARS + 160 + 1024 /*lse, D*/ + 1024;
};

// Persistent: each CTA walks the work items (kv tile, kv head, batch) dealt in boustrophedon order,
// heaviest first (small kv tile index = most q tiles).  Barriers, TMEM and the Q/dO
// ring live across items; the K/V tiles of the next item are requested as soon as the last S^T/dP^T
// MMAs of the current one retire.
struct DkDvItem {
  int jt, kvh, batch, i_begin, per_head, n_it;
};
__device__ __forceinline__ DkDvItem dkdv_item(int w, int Hkv, int B, int nq64, int G) {
  DkDvItem it;
  const int hb = w % (Hkv * B);
  it.jt = w / (Hkv * B);
  it.kvh = hb % Hkv;
  it.batch = hb / Hkv;
  it.i_begin = 2 * it.jt;  // first 64-row q tile that can see this kv tile
  it.per_head = nq64 - it.i_begin;
  it.n_it = it.per_head > 0 ? it.per_head * G : 0;
  return it;
}

// Roles (ATB_THREADS = 352): warp 0 streams tiles with TMA; warp 1 issues the S^T / dP^T MMAs; warp 10
// issues the dV / dK MMAs; warps 2..5 (group 0) do the elementwise step of the even global iterations,
// warps 6..9 (group 1) that of the odd ones, each thread owning one kv row and all 64 q columns of its
// iteration (two passes of 32).  See the dQ kernel for why there are two groups and two issuers.
__global__ void __launch_bounds__(ATB_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ64, const __grid_constant__ CUtensorMap tmdO64,
                     const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     const float* __restrict__ lse, const float* __restrict__ Dsum,
                     __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv, int ld_dk, int ld_dv,
                     int B, int S, int Hq, int Hkv, float scale, int* status) {
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
  uint64_t* kv_empty = bars + 16;
  uint64_t* acc_free = bars + 17;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  float* s_lse = reinterpret_cast<float*>(bars + 20);   // [group][64], pre-multiplied by log2(e)
  float* s_D = s_lse + 128;                             // [group][64], pre-multiplied by the softmax scale

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = Hq / Hkv;
  const int T = B * S;
  const int nq64 = (S + 63) / 64;
  const int n_items = ((S + 127) / 128) * Hkv * B;
  // first item with work at or after w along this CTA's path (n_items if none)
  auto first_with_work = [&](int w) {
    while (w < n_items && dkdv_item(w, Hkv, B, nq64, G).n_it == 0) w = snake_next(w);
    return w;
  };

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(kv_empty, 1);
    for (int i = 0; i < ATB_STAGES; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sdp_full[i], 1);
      mbar_init(&sdp_empty[i], 4);   // one arrive per warp of the group that owns buffer i
      mbar_init(&pds_full[i], 4);
      mbar_init(&pds_empty[i], 1);
    }
    mbar_init(acc_done, 1);
    mbar_init(acc_free, 8);          // every elementwise warp, after it has read its part of dV / dK
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
    if (lane == 0) {
      int g = 0, n = 0;
      bool ok = true;
      for (int w = first_with_work(blockIdx.x); w < n_items && ok; w = first_with_work(snake_next(w)), ++n) {
        const DkDvItem item = dkdv_item(w, Hkv, B, nq64, G);
        const int kv_row0 = item.batch * S + item.jt * 128;
        if (!mbar_wait(kv_empty, (n & 1) ^ 1, status, ERR_ATTN_WAIT)) break;
        mbar_expect_tx(kv_full, 65536);
        tma_load_2d(smem + DkDvSmem::K, &tmK, kv_full, item.kvh * 128, kv_row0);
        tma_load_2d(smem + DkDvSmem::K + 16384, &tmK, kv_full, item.kvh * 128 + 64, kv_row0);
        tma_load_2d(smem + DkDvSmem::V, &tmV, kv_full, item.kvh * 128, kv_row0);
        tma_load_2d(smem + DkDvSmem::V + 16384, &tmV, kv_full, item.kvh * 128 + 64, kv_row0);
        for (int it = 0; it < item.n_it; ++it, ++g) {
          const int st = g % ATB_STAGES;
          const uint32_t ph = (g / ATB_STAGES) & 1;
          const int head = item.kvh * G + it / item.per_head;
          const int qrow = item.batch * S + (item.i_begin + it % item.per_head) * 64;
          if (!mbar_wait(&qdo_empty[st], ph ^ 1, status, ERR_ATTN_WAIT)) { ok = false; break; }
          uint8_t* sQ = smem + DkDvSmem::Q + st * 16384;
          uint8_t* sdO = smem + DkDvSmem::DO + st * 16384;
          mbar_expect_tx(&qdo_full[st], 32768);
          tma_load_2d(sQ, &tmQ64, &qdo_full[st], head * 128, qrow);
          tma_load_2d(sQ + 8192, &tmQ64, &qdo_full[st], head * 128 + 64, qrow);
          tma_load_2d(sdO, &tmdO64, &qdo_full[st], head * 128, qrow);
          tma_load_2d(sdO + 8192, &tmdO64, &qdo_full[st], head * 128 + 64, qrow);
        }
      }
    }
  } else if (warp == 1) {
    // ---- S^T = K Q^T and dP^T = V dO^T of every global iteration ------------------------------------
    const bool leader = elect_one();
    constexpr uint32_t idesc_s = make_idesc_f16(1, 128, 64, 0, 0);     // [128 kv] x [64 q], K = d
    const uint64_t d_k = make_smem_desc_sw128(smem_u32(smem + DkDvSmem::K), 16, 1024);
    const uint64_t d_v = make_smem_desc_sw128(smem_u32(smem + DkDvSmem::V), 16, 1024);
    int g = 0, n = 0;
    bool ok = true;
    for (int w = first_with_work(blockIdx.x); w < n_items && ok; w = first_with_work(snake_next(w)), ++n) {
      const DkDvItem item = dkdv_item(w, Hkv, B, nq64, G);
      if (!mbar_wait(kv_full, n & 1, status, ERR_ATTN_WAIT)) break;
      for (int it = 0; it < item.n_it; ++it, ++g) {
        const int st = g & 1;
        const int ks_ = g % ATB_STAGES;
        if (!mbar_wait(&qdo_full[ks_], (g / ATB_STAGES) & 1, status, ERR_ATTN_WAIT) ||
            !mbar_wait(&sdp_empty[st], ((g >> 1) & 1) ^ 1, status, ERR_ATTN_WAIT)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t d_q = make_smem_desc_sw128(smem_u32(smem + DkDvSmem::Q + ks_ * 16384), 16, 1024);
        const uint64_t d_do = make_smem_desc_sw128(smem_u32(smem + DkDvSmem::DO + ks_ * 16384), 16, 1024);
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t oa = (ks >> 2) * 16384 + (ks & 3) * 32;
            const uint32_t ob = (ks >> 2) * 8192 + (ks & 3) * 32;
            umma_f16_ss(tmem_ST + st * 64, desc_advance(d_k, oa), desc_advance(d_q, ob), idesc_s, ks != 0);
          }
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t oa = (ks >> 2) * 16384 + (ks & 3) * 32;
            const uint32_t ob = (ks >> 2) * 8192 + (ks & 3) * 32;
            umma_f16_ss(tmem_DPT + st * 64, desc_advance(d_v, oa), desc_advance(d_do, ob), idesc_s, ks != 0);
          }
          umma_commit(&sdp_full[st]);
          if (it + 1 == item.n_it) umma_commit(kv_empty);   // last S^T/dP^T of the item: K/V may be reloaded
        }
      }
    }
  } else if (warp == 10) {
    // ---- dV += P^T dO and dK += dS^T Q of every global iteration --------------------------------------
    const bool leader = elect_one();
    constexpr uint32_t idesc_acc = make_idesc_f16(1, 128, 128, 0, 1);  // [128 kv] x [128 d], K = q
    int g = 0, n = 0;
    bool ok = true;
    for (int w = first_with_work(blockIdx.x); w < n_items && ok; w = first_with_work(snake_next(w)), ++n) {
      const DkDvItem item = dkdv_item(w, Hkv, B, nq64, G);
      // the elementwise warps must have read the previous item's dV / dK before they are overwritten
      if (n > 0 && !mbar_wait(acc_free, (n - 1) & 1, status, ERR_ATTN_WAIT)) break;
      for (int it = 0; it < item.n_it; ++it, ++g) {
        const int st = g & 1;
        const int kst = g % ATB_STAGES;
        if (!mbar_wait(&qdo_full[kst], (g / ATB_STAGES) & 1, status, ERR_ATTN_WAIT) ||
            !mbar_wait(&pds_full[st], (g >> 1) & 1, status, ERR_ATTN_WAIT)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t d_pt = make_smem_desc_sw128(smem_u32(smem + DkDvSmem::PT + st * 16384), 16, 1024);
        const uint64_t d_dst = make_smem_desc_sw128(smem_u32(smem + DkDvSmem::DST + st * 16384), 16, 1024);
        const uint64_t d_qm = make_smem_desc_sw128(smem_u32(smem + DkDvSmem::Q + kst * 16384), 8192, 1024);
        const uint64_t d_dom = make_smem_desc_sw128(smem_u32(smem + DkDvSmem::DO + kst * 16384), 8192, 1024);
        const uint32_t acc0 = it != 0;
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_f16_ss(tmem_DV, desc_advance(d_pt, ks * 32), desc_advance(d_dom, ks * 2048), idesc_acc,
                        ks ? 1u : acc0);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_f16_ss(tmem_DK, desc_advance(d_dst, ks * 32), desc_advance(d_qm, ks * 2048), idesc_acc,
                        ks ? 1u : acc0);
          umma_commit(&qdo_empty[kst]);
          umma_commit(&pds_empty[st]);
          if (it + 1 == item.n_it) umma_commit(acc_done);
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    const int grp = (warp - 2) >> 2;            // elementwise group = parity of the iterations it handles
    const int gtid = ((warp - 2) & 3) * 32 + lane;   // 0..127 inside the group
    const int r = quarter * 32 + lane;          // kv row in tile
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = scale * LOG2E;
    bool ok = true;
    int g = 0, n = 0;
    // Row statistics (lse, D) of a 64-row q tile go through shared memory (one buffer per group).  The
    // global loads for the group's next tile (two iterations ahead, possibly in the next item) are issued
    // at the top of an iteration and stored at its end (after a second group barrier: everyone has read
    // the current ones), so their latency hides behind the elementwise work.
    auto stat_load = [&](int w, int it) -> float {   // position (item w, iteration it), may run past the item
      DkDvItem item = dkdv_item(w, Hkv, B, nq64, G);
      while (it >= item.n_it) {
        it -= item.n_it;
        w = first_with_work(snake_next(w));
        if (w >= n_items) return 0.f;
        item = dkdv_item(w, Hkv, B, nq64, G);
      }
      const int head_ = item.kvh * G + it / item.per_head;
      const int q0_ = (item.i_begin + it % item.per_head) * 64;
      const int qc = min(q0_ + (gtid & 63), S - 1);
      const size_t o = static_cast<size_t>(head_) * T + item.batch * S + qc;
      return gtid < 64 ? lse[o] * LOG2E : Dsum[o] * scale;
    };
    auto stat_store = [&](float v) {
      if (gtid < 64) s_lse[grp * 64 + gtid] = v;
      else s_D[grp * 64 + (gtid & 63)] = v;
    };
    auto group_barrier = [&]() {
      if (grp) asm volatile("bar.sync 2, 128;" ::: "memory");
      else asm volatile("bar.sync 1, 128;" ::: "memory");
    };
    bool first = true;
    for (int w = blockIdx.x; w < n_items; w = snake_next(w)) {
      const DkDvItem item = dkdv_item(w, Hkv, B, nq64, G);
      const int kv_pos = item.jt * 128 + r;
      const int kv_row0 = item.batch * S + item.jt * 128;
      const bool in_range = kv_pos < S;
      __nv_bfloat16* orow = grp ? dk + static_cast<size_t>(kv_row0 + r) * ld_dk + item.kvh * 128
                                : dv + static_cast<size_t>(kv_row0 + r) * ld_dv + item.kvh * 128;
      if (item.n_it == 0) {   // no query sees this kv tile: zero gradients
        if (in_range) {
          const uint4 z = make_uint4(0, 0, 0, 0);
          for (int c = 0; c < 16; ++c) *reinterpret_cast<uint4*>(orow + c * 8) = z;
        }
        continue;
      }
      for (int it = 0; it < item.n_it; ++it, ++g) {
        if ((g & 1) != grp) continue;
        const int st = grp;
        const uint32_t ph = (g >> 1) & 1;
        const int q0 = (item.i_begin + it % item.per_head) * 64;  // first q position of this tile
        if (first) {
          stat_store(stat_load(w, it));
          first = false;
        }
        const float next_stat = stat_load(w, it + 2);
        group_barrier();   // publishes this tile's statistics; every thread of the group reaches both
                           // barriers in each of the group's iterations, also after a failed wait
        if (ok) ok = mbar_wait_warp(&sdp_full[st], ph, status, ERR_ATTN_WAIT);
        if (!ok) {
          group_barrier();
          continue;
        }
        tc_fence_after();
        uint8_t* sPT = smem + DkDvSmem::PT + st * 16384 + r * 128;
        uint8_t* sDST = smem + DkDvSmem::DST + st * 16384 + r * 128;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t ts[32], tp[32];
          tmem_ld_32x32b_x32(tmem_ST + lane_off + st * 64 + half * 32, ts);
          tmem_ld_32x32b_x32(tmem_DPT + lane_off + st * 64 + half * 32, tp);
          tmem_ld_wait();
          if (half == 1) {
            tc_fence_before();
            mbar_arrive_warp(&sdp_empty[st]);   // both halves are in registers: the buffer may be refilled
          }
          const float* lse_s = s_lse + grp * 64 + half * 32;
          const float* D_s = s_D + grp * 64 + half * 32;
          const int qb = q0 + half * 32;
          const bool need_mask = (qb < item.jt * 128 + 128) || (qb + 32 > S) || (item.jt * 128 + 128 > S);
          float pv[32], dsv[32];
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            float p = fast_exp2(fmaf(__uint_as_float(ts[c]), sl2, -lse_s[c]));
            if (need_mask) {
              const int qp = qb + c;
              if (!((qp < S) && (kv_pos <= qp) && (kv_pos < S))) p = 0.f;
            }
            pv[c] = p;
            dsv[c] = p * fmaf(__uint_as_float(tp[c]), scale, -D_s[c]);   // D_s holds D * scale
          }
          if (half == 0) {
            ok = mbar_wait_warp(&pds_empty[st], ph ^ 1, status, ERR_ATTN_WAIT);
            if (!ok) break;
          }
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
        }
        group_barrier();          // every thread of the group has read this tile's statistics
        stat_store(next_stat);
        if (!ok) continue;
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive_warp(&pds_full[st]);
      }
      // write-out: group 0 stores dV, group 1 dK
      if (ok) ok = mbar_wait_warp(acc_done, n & 1, status, ERR_ATTN_WAIT);
      ++n;
      if (!ok) continue;
      tc_fence_after();
      const uint32_t tb = (grp ? tmem_DK : tmem_DV) + lane_off;
      // Staged through this group's P^T buffer: every MMA that read it has completed (acc_done) and the
      // group itself is its only writer.
      uint8_t* stage = smem + DkDvSmem::PT + grp * 16384 + ((warp - 2) & 3) * 4096;
      const int wrow0 = item.jt * 128 + quarter * 32;   // first kv position of this warp's 32 rows
      __nv_bfloat16* obase = grp ? dk + static_cast<size_t>(kv_row0 + quarter * 32) * ld_dk + item.kvh * 128
                                 : dv + static_cast<size_t>(kv_row0 + quarter * 32) * ld_dv + item.kvh * 128;
      const size_t ld_o = grp ? ld_dk : ld_dv;
#pragma unroll
      for (int hc = 0; hc < 2; ++hc) {   // two halves of 64 columns = 128 bytes per row each
        uint4 ov[8];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t t[32];
          tmem_ld_32x32b_x32(tb + hc * 64 + c * 32, t);
          tmem_ld_wait();
          if (hc == 1 && c == 1) {
            tc_fence_before();
            mbar_arrive_warp(acc_free);   // this warp's part of the accumulators is in registers
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            ov[c * 4 + v].x = pack_bf16x2(__uint_as_float(t[v * 8 + 0]), __uint_as_float(t[v * 8 + 1]));
            ov[c * 4 + v].y = pack_bf16x2(__uint_as_float(t[v * 8 + 2]), __uint_as_float(t[v * 8 + 3]));
            ov[c * 4 + v].z = pack_bf16x2(__uint_as_float(t[v * 8 + 4]), __uint_as_float(t[v * 8 + 5]));
            ov[c * 4 + v].w = pack_bf16x2(__uint_as_float(t[v * 8 + 6]), __uint_as_float(t[v * 8 + 7]));
          }
        }
        warp_store_rows_128B(stage, ov, [&](int row) -> uint8_t* {
          if (wrow0 + row >= S) return nullptr;
          return reinterpret_cast<uint8_t*>(obase + static_cast<size_t>(row) * ld_o + hc * 64);
        });
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
  static constexpr int EPI = DS + 2 * 16384;           // 8 warps x 4 KiB write-out staging
  static constexpr int BARS = EPI + 8 * 4096;
  static constexpr int TOTAL = BARS + 256 + 1024;
};

// Persistent: each CTA walks the work items (q tile, head, batch) dealt in boustrophedon order,
// heaviest first.  Barriers, TMEM and the K/V ring live across items, so a
// new item costs one Q/dO reload (issued as soon as the previous item's last S/dP MMAs retire, i.e.
// hidden behind its last elementwise step, dQ MMA and write-out) instead of a CTA launch, a TMEM
// allocation and a cold pipeline.
struct DqItem {
  int qt, head, batch, n_it;
};
__device__ __forceinline__ DqItem dq_item(int w, int num_q_tiles, int Hq, int B, int nkv64) {
  DqItem it;
  const int hb = w % (Hq * B);
  it.qt = num_q_tiles - 1 - w / (Hq * B);  // heaviest tiles first
  it.head = hb % Hq;
  it.batch = hb / Hq;
  it.n_it = min(nkv64, 2 * it.qt + 2);
  return it;
}

// Roles (ATB_THREADS = 352): warp 0 streams tiles with TMA; warp 1 issues the S / dP MMAs; warp 10
// issues the dQ MMAs; warps 2..5 (group 0) do the elementwise step of the even global iterations and
// warps 6..9 (group 1) that of the odd ones, each thread owning one q row and all 64 kv columns of its
// iteration (two passes of 32).  With two groups every elementwise chain (wait for S/dP, tcgen05.ld,
// exp2 / dS, swizzled stores, arrive) has two iterations of time, and with two issuing warps the 16
// S/dP instructions of iteration g+1 and the 4 dQ instructions of iteration g are issued concurrently:
// a single issuing lane and a single elementwise group each needed ~1900 cycles per iteration against
// ~800 cycles of tensor work.
__global__ void __launch_bounds__(ATB_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmK64, const __grid_constant__ CUtensorMap tmV64,
                   const float* __restrict__ lse, const float* __restrict__ Dsum,
                   __nv_bfloat16* __restrict__ dq, int B, int S, int Hq, int Hkv, float scale,
                   int* status) {
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
  uint64_t* q_empty = bars + 16;
  uint64_t* acc_free = bars + 17;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_q_tiles = (S + 127) / 128;
  const int T = B * S;
  const int nkv64 = (S + 63) / 64;
  const int n_items = num_q_tiles * Hq * B;
  const int G = Hq / Hkv;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int i = 0; i < ATB_STAGES; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sdp_full[i], 1);
      mbar_init(&sdp_empty[i], 4);   // one arrive per warp of the group that owns buffer i
      mbar_init(&ds_full[i], 4);
      mbar_init(&ds_empty[i], 1);
    }
    mbar_init(acc_done, 1);
    mbar_init(acc_free, 8);          // every elementwise warp, after it has read its part of dQ
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
      int g = 0;   // K/V tiles loaded so far (ring position, continues across items)
      int n = 0;   // items started
      bool ok = true;
      for (int w = blockIdx.x; w < n_items && ok; w = snake_next(w), ++n) {
        const DqItem item = dq_item(w, num_q_tiles, Hq, B, nkv64);
        const int row0 = item.batch * S + item.qt * 128;
        const int kvh = item.head / G;
        if (!mbar_wait(q_empty, (n & 1) ^ 1, status, ERR_ATTN_WAIT)) break;
        mbar_expect_tx(q_full, 65536);
        tma_load_2d(smem + DqSmem::Q, &tmQ, q_full, item.head * 128, row0);
        tma_load_2d(smem + DqSmem::Q + 16384, &tmQ, q_full, item.head * 128 + 64, row0);
        tma_load_2d(smem + DqSmem::DO, &tmdO, q_full, item.head * 128, row0);
        tma_load_2d(smem + DqSmem::DO + 16384, &tmdO, q_full, item.head * 128 + 64, row0);
        for (int it = 0; it < item.n_it; ++it, ++g) {
          const int st = g % ATB_STAGES;
          const uint32_t ph = (g / ATB_STAGES) & 1;
          const int krow = item.batch * S + it * 64;
          if (!mbar_wait(&kv_empty[st], ph ^ 1, status, ERR_ATTN_WAIT)) { ok = false; break; }
          uint8_t* sK = smem + DqSmem::K + st * 16384;
          uint8_t* sV = smem + DqSmem::V + st * 16384;
          mbar_expect_tx(&kv_full[st], 32768);
          tma_load_2d(sK, &tmK64, &kv_full[st], kvh * 128, krow);
          tma_load_2d(sK + 8192, &tmK64, &kv_full[st], kvh * 128 + 64, krow);
          tma_load_2d(sV, &tmV64, &kv_full[st], kvh * 128, krow);
          tma_load_2d(sV + 8192, &tmV64, &kv_full[st], kvh * 128 + 64, krow);
        }
      }
    }
  } else if (warp == 1) {
    // ---- S = Q K^T and dP = dO V^T of every global iteration (uniform control flow, one issuing lane) ----
    const bool leader = elect_one();
    constexpr uint32_t idesc_s = make_idesc_f16(1, 128, 64, 0, 0);     // [128 q] x [64 kv], K = d
    const uint64_t d_q = make_smem_desc_sw128(smem_u32(smem + DqSmem::Q), 16, 1024);
    const uint64_t d_do = make_smem_desc_sw128(smem_u32(smem + DqSmem::DO), 16, 1024);
    int g = 0, n = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < n_items && ok; w = snake_next(w), ++n) {
      const DqItem item = dq_item(w, num_q_tiles, Hq, B, nkv64);
      if (!mbar_wait(q_full, n & 1, status, ERR_ATTN_WAIT)) break;
      for (int it = 0; it < item.n_it; ++it, ++g) {
        const int st = g & 1;
        const int ks_ = g % ATB_STAGES;
        if (!mbar_wait(&kv_full[ks_], (g / ATB_STAGES) & 1, status, ERR_ATTN_WAIT) ||
            !mbar_wait(&sdp_empty[st], ((g >> 1) & 1) ^ 1, status, ERR_ATTN_WAIT)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t d_k = make_smem_desc_sw128(smem_u32(smem + DqSmem::K + ks_ * 16384), 16, 1024);
        const uint64_t d_v = make_smem_desc_sw128(smem_u32(smem + DqSmem::V + ks_ * 16384), 16, 1024);
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t oa = (ks >> 2) * 16384 + (ks & 3) * 32;
            const uint32_t ob = (ks >> 2) * 8192 + (ks & 3) * 32;
            umma_f16_ss(tmem_S + st * 64, desc_advance(d_q, oa), desc_advance(d_k, ob), idesc_s, ks != 0);
          }
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t oa = (ks >> 2) * 16384 + (ks & 3) * 32;
            const uint32_t ob = (ks >> 2) * 8192 + (ks & 3) * 32;
            umma_f16_ss(tmem_DP + st * 64, desc_advance(d_do, oa), desc_advance(d_v, ob), idesc_s, ks != 0);
          }
          umma_commit(&sdp_full[st]);
          if (it + 1 == item.n_it) umma_commit(q_empty);   // last S/dP of the item: Q/dO may be reloaded
        }
      }
    }
  } else if (warp == 10) {
    // ---- dQ += dS K of every global iteration ------------------------------------------------------
    const bool leader = elect_one();
    constexpr uint32_t idesc_acc = make_idesc_f16(1, 128, 128, 0, 1);  // [128 q] x [128 d], K = kv
    int g = 0, n = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < n_items && ok; w = snake_next(w), ++n) {
      const DqItem item = dq_item(w, num_q_tiles, Hq, B, nkv64);
      // the elementwise warps must have read the previous item's dQ before it is overwritten
      if (n > 0 && !mbar_wait(acc_free, (n - 1) & 1, status, ERR_ATTN_WAIT)) break;
      for (int it = 0; it < item.n_it; ++it, ++g) {
        const int st = g & 1;
        const int kst = g % ATB_STAGES;
        if (!mbar_wait(&kv_full[kst], (g / ATB_STAGES) & 1, status, ERR_ATTN_WAIT) ||
            !mbar_wait(&ds_full[st], (g >> 1) & 1, status, ERR_ATTN_WAIT)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t d_ds = make_smem_desc_sw128(smem_u32(smem + DqSmem::DS + st * 16384), 16, 1024);
        const uint64_t d_km = make_smem_desc_sw128(smem_u32(smem + DqSmem::K + kst * 16384), 8192, 1024);
        const uint32_t acc0 = it != 0;
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_f16_ss(tmem_DQ, desc_advance(d_ds, ks * 32), desc_advance(d_km, ks * 2048), idesc_acc,
                        ks ? 1u : acc0);
          umma_commit(&kv_empty[kst]);
          umma_commit(&ds_empty[st]);
          if (it + 1 == item.n_it) umma_commit(acc_done);
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    const int grp = (warp - 2) >> 2;            // elementwise group = parity of the iterations it handles
    const int r = quarter * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = scale * LOG2E;
    bool ok = true;
    int g = 0, n = 0;
    auto row_stats = [&](const DqItem& item, float* lse_r, float* D_r) {
      const int q_pos = item.qt * 128 + r;
      const int qc = q_pos < S ? q_pos : S - 1;
      const size_t o = static_cast<size_t>(item.head) * T + item.batch * S + qc;
      *lse_r = lse[o] * LOG2E;
      *D_r = Dsum[o] * scale;
    };
    float lse_r = 0.f, D_r = 0.f;
    if (static_cast<int>(blockIdx.x) < n_items) row_stats(dq_item(blockIdx.x, num_q_tiles, Hq, B, nkv64), &lse_r, &D_r);
    for (int w = blockIdx.x; w < n_items && ok; w = snake_next(w), ++n) {
      const DqItem item = dq_item(w, num_q_tiles, Hq, B, nkv64);
      const int qt = item.qt;
      const int q_pos = qt * 128 + r;
      const int row0 = item.batch * S + qt * 128;
      // next item's row statistics: requested now, consumed after this item's write-out
      float lse_n = 0.f, D_n = 0.f;
      if (snake_next(w) < n_items)
        row_stats(dq_item(snake_next(w), num_q_tiles, Hq, B, nkv64), &lse_n, &D_n);
      for (int it = 0; it < item.n_it; ++it, ++g) {
        if ((g & 1) != grp) continue;
        const int st = grp;
        const uint32_t ph = (g >> 1) & 1;
        if (!mbar_wait_warp(&sdp_full[st], ph, status, ERR_ATTN_WAIT)) { ok = false; break; }
        tc_fence_after();
        uint8_t* sDS = smem + DqSmem::DS + st * 16384 + r * 128;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t ts[32], tp[32];
          tmem_ld_32x32b_x32(tmem_S + lane_off + st * 64 + half * 32, ts);
          tmem_ld_32x32b_x32(tmem_DP + lane_off + st * 64 + half * 32, tp);
          tmem_ld_wait();
          if (half == 1) {
            tc_fence_before();
            mbar_arrive_warp(&sdp_empty[st]);   // both halves are in registers: S/dP buffer may be refilled
          }
          const int k0 = it * 64 + half * 32;
          const bool need_mask = (k0 + 32 > qt * 128) || (k0 + 32 > S) || (qt * 128 + 128 > S);
          float dsv[32];
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            float p = fast_exp2(fmaf(__uint_as_float(ts[c]), sl2, -lse_r));
            if (need_mask) {
              const int kp = k0 + c;
              if (!((q_pos < S) && (kp <= q_pos) && (kp < S))) p = 0.f;
            }
            dsv[c] = p * fmaf(__uint_as_float(tp[c]), scale, -D_r);   // D_r holds D * scale
          }
          if (half == 0 && !mbar_wait_warp(&ds_empty[st], ph ^ 1, status, ERR_ATTN_WAIT)) { ok = false; break; }
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            uint4 b;
            b.x = pack_bf16x2(dsv[c4 * 8 + 0], dsv[c4 * 8 + 1]);
            b.y = pack_bf16x2(dsv[c4 * 8 + 2], dsv[c4 * 8 + 3]);
            b.z = pack_bf16x2(dsv[c4 * 8 + 4], dsv[c4 * 8 + 5]);
            b.w = pack_bf16x2(dsv[c4 * 8 + 6], dsv[c4 * 8 + 7]);
            *reinterpret_cast<uint4*>(sDS + (((half * 4 + c4) ^ (r & 7)) << 4)) = b;
          }
        }
        if (!ok) break;
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive_warp(&ds_full[st]);
      }
      if (!ok || !mbar_wait_warp(acc_done, n & 1, status, ERR_ATTN_WAIT)) { ok = false; break; }
      tc_fence_after();
      // write-out: group 0 stores dQ columns 0..63, group 1 columns 64..127 (128 bytes per row and thread)
      uint4 ov[8];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t t[32];
        tmem_ld_32x32b_x32(tmem_DQ + lane_off + grp * 64 + c * 32, t);
        tmem_ld_wait();
        if (c == 1) {
          tc_fence_before();
          mbar_arrive_warp(acc_free);   // this warp's part of dQ is in registers
        }
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          ov[c * 4 + v].x = pack_bf16x2(__uint_as_float(t[v * 8 + 0]), __uint_as_float(t[v * 8 + 1]));
          ov[c * 4 + v].y = pack_bf16x2(__uint_as_float(t[v * 8 + 2]), __uint_as_float(t[v * 8 + 3]));
          ov[c * 4 + v].z = pack_bf16x2(__uint_as_float(t[v * 8 + 4]), __uint_as_float(t[v * 8 + 5]));
          ov[c * 4 + v].w = pack_bf16x2(__uint_as_float(t[v * 8 + 6]), __uint_as_float(t[v * 8 + 7]));
        }
      }
      {
        const int wrow0 = qt * 128 + quarter * 32;   // first q position of this warp's 32 rows
        __nv_bfloat16* base = dq + (static_cast<size_t>(row0 + quarter * 32) * Hq + item.head) * 128 + grp * 64;
        warp_store_rows_128B(smem + DqSmem::EPI + (warp - 2) * 4096, ov, [&](int row) -> uint8_t* {
          if (wrow0 + row >= S) return nullptr;
          return reinterpret_cast<uint8_t*>(base + static_cast<size_t>(row) * Hq * 128);
        });
      }
      lse_r = lse_n;
      D_r = D_n;
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
  const int dkdv_items = nt * Hkv * B;
  attn_bwd_dkdv_kernel<<<dkdv_items < num_sms() ? dkdv_items : num_sms(), ATB_THREADS, DkDvSmem::TOTAL, stream>>>(
      *tq64, *tdo64, *tk128, *tv128, lse, Dsum, static_cast<__nv_bfloat16*>(dk),
      static_cast<__nv_bfloat16*>(dv), ld_dk, ld_dv, B, S, Hq, Hkv, scale, status);
  const int dq_items = nt * Hq * B;
  attn_bwd_dq_kernel<<<dq_items < num_sms() ? dq_items : num_sms(), ATB_THREADS, DqSmem::TOTAL, stream>>>(
      *tq128, *tdo128, *tk64, *tv64, lse, Dsum, static_cast<__nv_bfloat16*>(dq), B, S, Hq, Hkv, scale, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("attn_bwd launch failed: %s", cudaGetErrorString(e));
    return 4;
  }
  return 0;
}
