// Causal flash-attention forward for sm_100a (head_dim 128, GQA), tcgen05 MMAs with S and O in TMEM.
//
// A work item is one 128-row query tile of one (batch, q-head); a persistent CTA per SM walks the
// items.  The softmax warps read S from TMEM, write P (bf16 pairs) back to TMEM, from where the PV MMA
// takes it as its A operand (no shared-memory round trip), and rescale the O accumulator in TMEM only when the running
// row maximum grew by more than 2^8 (the final normalisation uses the same reference maximum for
// P and for the row sum, so a stale maximum is exact as long as nothing overflows).
//
// Layouts: q [T, Hq*128], k [T, Hkv*128], v [T, ld_v] (a column slice of the fused projection output),
// out [T, Hq*128], lse [Hq, T] (natural log, scaled scores).  T = B*S; sequence b owns rows b*S..b*S+S-1.
#include "common.cuh"
#include "host.h"

namespace b2 {

constexpr int AT_THREADS = 352;  // warp 0 TMA, warps 1 and 10 MMA issue, warps 2..9 softmax (two threads per row)
constexpr int AT_TILE_BYTES = 128 * 128 * 2;  // 32 KiB: two [128 x 64] swizzled halves
constexpr int AT_HALF_BYTES = 128 * 64 * 2;

struct AttnFwdSmem {
  // offsets into the 1024-byte aligned dynamic shared memory
  static constexpr int Q = 0;                           // 2 tiles (this item's and the next item's)
  static constexpr int K = Q + 2 * AT_TILE_BYTES;       // 2 stages
  static constexpr int V = K + 2 * AT_TILE_BYTES;       // 2 stages
  static constexpr int EPI = V + 2 * AT_TILE_BYTES;     // 8 warps x 4 KiB write-out staging
  static constexpr int BARS = EPI + 8 * 4096;           // barriers (256 B), then the row exchange buffer (1 KiB)
  static constexpr int TOTAL = BARS + 256 + 1024 + 1024;   // 198912
};

// One work item: a 128-row query tile of one (batch, q head).
struct FwdItem {
  int head, kvh, qt, q_len, kv_len, kv_off, k_begin, row0, n_kv, batch;
  bool active;
};
struct FwdParams {
  int S, Hq, Hkv, B, max_tiles, total_q;
  const int* cu_q;
  const int* cu_k;
  // Paged keys / values (chunked prefill straight out of the KV cache): block_tables[b][i] is the cache block
  // that holds keys 16 i .. 16 i + 15 of sequence b; the K / V tensor maps then describe the cache as a
  // [blocks * 16, Hkv * 128] matrix with 16-row boxes, and cu_k only carries the key counts.
  const int* block_tables;
  int max_blocks;
};
// Fixed-length mode (cu_q == nullptr): every sequence has S query and S key tokens.  Variable
// length mode: sequence b owns query rows cu_q[b]..cu_q[b+1] and key rows cu_k[b]..cu_k[b+1]; its
// queries are the LAST q_len positions of its kv_len keys (chunked prefill / speculative verify), so
// query i sees keys 0..(kv_len - q_len + i).
__device__ __forceinline__ FwdItem fwd_item(int w, const FwdParams& p) {
  FwdItem it;
  const int hb = w % (p.Hq * p.B);
  const int x = w / (p.Hq * p.B);   // tile rank counted from the last (heaviest) tile
  it.head = hb % p.Hq;
  const int batch = hb / p.Hq;
  it.batch = batch;
  const int q_begin = p.cu_q ? p.cu_q[batch] : batch * p.S;
  it.q_len = p.cu_q ? p.cu_q[batch + 1] - q_begin : p.S;
  it.k_begin = p.cu_k ? p.cu_k[batch] : batch * p.S;
  it.kv_len = p.cu_k ? p.cu_k[batch + 1] - it.k_begin : p.S;
  it.kv_off = it.kv_len - it.q_len;
  const int num_q_tiles = (it.q_len + 127) / 128;
  it.qt = num_q_tiles - 1 - x;
  it.active = it.qt >= 0 && it.q_len > 0;
  it.kvh = it.head / (p.Hq / p.Hkv);
  const int last_key = min(it.kv_len, it.kv_off + (it.qt + 1) * 128);  // exclusive
  it.n_kv = it.active ? (last_key + 127) / 128 : 0;
  it.active = it.active && it.n_kv > 0;
  it.row0 = q_begin + it.qt * 128;
  return it;
}
__device__ __forceinline__ int fwd_next_active(int w, int n_items, const FwdParams& p) {
  int x = snake_next(w);
  while (x < n_items && !fwd_item(x, p).active) x = snake_next(x);
  return x;
}

// Persistent: each CTA walks its share of the items (heaviest tiles first, dealt in boustrophedon order).
// Barriers, TMEM and the K/V ring live across items; the next item's Q is requested as soon as the last
// Q*K^T of the current item retires.
//
// Roles (AT_THREADS = 352): warp 0 streams K/V with TMA, warp 1 issues the Q*K^T MMAs, warp 10 the P*V
// MMAs, warps 2..9 run the softmax.  A query row is shared by two threads (warps w and w+4 touch the same
// TMEM lane quarter): each takes 64 of the tile's 128 key columns, the pair exchanges its partial row
// maximum through shared memory and keeps partial row sums that are added at the end.  S and P are
// double-buffered in TMEM (S 2 x 128 columns, O 128, P 2 x 64 = all 512), so the softmax of tile j+1 never
// waits for P*V of tile j unless the running maximum grew enough to force a rescale of O.  Q is double-
// buffered in shared memory: the next item's Q arrives while the current item is still being processed.
__global__ void __launch_bounds__(AT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, __nv_bfloat16* __restrict__ out,
                float* __restrict__ lse_out, const FwdParams prm, float scale, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AttnFwdSmem::BARS);
  uint64_t* q_full = bars + 0;    // [2] with q_empty at bars + 17
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* v_full = bars + 3;    // [2]
  uint64_t* k_empty = bars + 5;   // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2]
  uint64_t* s_empty = bars + 11;  // [2]
  uint64_t* p_full = bars + 13;   // [2]
  uint64_t* pv_done = bars + 15;  // [2]
  uint64_t* q_empty = bars + 17;  // [2]
  uint64_t* o_free = bars + 19;
  uint64_t* q_full2 = bars + 20;  // second Q slot's full barrier
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  float* xchg = reinterpret_cast<float*>(smem + AttnFwdSmem::BARS + 256);   // [2 column halves][128 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int Hq = prm.Hq;
  const int n_items = prm.max_tiles * prm.Hq * prm.B;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_full2, 1);
    mbar_init(&q_empty[0], 1);
    mbar_init(&q_empty[1], 1);
    mbar_init(o_free, 8);            // every softmax warp, after it has read its part of O
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 8);     // one arrive per softmax warp
      mbar_init(&p_full[i], 8);
      mbar_init(&pv_done[i], 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const uint32_t tmem_S = tmem_base;        // 2 x 128 columns
  const uint32_t tmem_O = tmem_base + 256;  // 128 columns
  const uint32_t tmem_P = tmem_base + 384;  // 2 x 64 columns: P as bf16 pairs, the A operand of P*V

  int w0 = blockIdx.x;
  if (w0 < n_items && !fwd_item(w0, prm).active) w0 = fwd_next_active(w0, n_items, prm);

  if (warp == 0) {
    if (lane == 0) {
      int g = 0, n = 0;
      bool ok = true;
      for (int w = w0; w < n_items && ok; w = fwd_next_active(w, n_items, prm), ++n) {
        const FwdItem item = fwd_item(w, prm);
        // Q slot n & 1: free once the last Q*K^T of item n-2 has retired, i.e. long before item n starts
        uint64_t* qf = (n & 1) ? q_full2 : q_full;
        uint8_t* sQ = smem + AttnFwdSmem::Q + (n & 1) * AT_TILE_BYTES;
        if (!mbar_wait(&q_empty[n & 1], ((n >> 1) & 1) ^ 1, status, ERR_ATTN_WAIT)) break;
        mbar_expect_tx(qf, AT_TILE_BYTES);
        tma_load_2d(sQ, &tmQ, qf, item.head * 128, item.row0);
        tma_load_2d(sQ + AT_HALF_BYTES, &tmQ, qf, item.head * 128 + 64, item.row0);
        for (int j = 0; j < item.n_kv; ++j, ++g) {
          const int st = g & 1;
          const uint32_t ph = (g >> 1) & 1;
          const int krow = item.k_begin + j * 128;
          if (!mbar_wait(&k_empty[st], ph ^ 1, status, ERR_ATTN_WAIT)) { ok = false; break; }
          uint8_t* sK = smem + AttnFwdSmem::K + st * AT_TILE_BYTES;
          uint8_t* sV = smem + AttnFwdSmem::V + st * AT_TILE_BYTES;
          if (prm.block_tables != nullptr) {
            // a 128-key tile is eight 16-token pages: each lands as a [16 x 64] box at its row offset of the
            // swizzled tile (16 rows x 128 B = 2 KiB, a whole number of swizzle atoms).  Pages past the end of the
            // sequence repeat its last page: those keys are masked, the bytes only have to be finite.
            const int* tbl = prm.block_tables + static_cast<size_t>(item.batch) * prm.max_blocks;
            const int last_page = (item.kv_len - 1) / 16;
            int rows[8];
#pragma unroll
            for (int pg = 0; pg < 8; ++pg) rows[pg] = tbl[min(j * 8 + pg, last_page)] * 16;
            mbar_expect_tx(&k_full[st], AT_TILE_BYTES);
#pragma unroll
            for (int pg = 0; pg < 8; ++pg) {
              tma_load_2d(sK + pg * 2048, &tmK, &k_full[st], item.kvh * 128, rows[pg]);
              tma_load_2d(sK + AT_HALF_BYTES + pg * 2048, &tmK, &k_full[st], item.kvh * 128 + 64, rows[pg]);
            }
            if (!mbar_wait(&v_empty[st], ph ^ 1, status, ERR_ATTN_WAIT)) { ok = false; break; }
            mbar_expect_tx(&v_full[st], AT_TILE_BYTES);
#pragma unroll
            for (int pg = 0; pg < 8; ++pg) {
              tma_load_2d(sV + pg * 2048, &tmV, &v_full[st], item.kvh * 128, rows[pg]);
              tma_load_2d(sV + AT_HALF_BYTES + pg * 2048, &tmV, &v_full[st], item.kvh * 128 + 64, rows[pg]);
            }
            continue;
          }
          mbar_expect_tx(&k_full[st], AT_TILE_BYTES);
          tma_load_2d(sK, &tmK, &k_full[st], item.kvh * 128, krow);
          tma_load_2d(sK + AT_HALF_BYTES, &tmK, &k_full[st], item.kvh * 128 + 64, krow);
          if (!mbar_wait(&v_empty[st], ph ^ 1, status, ERR_ATTN_WAIT)) { ok = false; break; }
          mbar_expect_tx(&v_full[st], AT_TILE_BYTES);
          tma_load_2d(sV, &tmV, &v_full[st], item.kvh * 128, krow);
          tma_load_2d(sV + AT_HALF_BYTES, &tmV, &v_full[st], item.kvh * 128 + 64, krow);
        }
      }
    }
  } else if (warp == 1) {
    // ---- S = Q K^T of every global iteration (uniform control flow, one issuing lane) --------------
    const bool leader = elect_one();
    constexpr uint32_t idesc_s = make_idesc_f16(1, 128, 128, 0, 0);
    int g = 0, n = 0;
    bool ok = true;
    for (int w = w0; w < n_items && ok; w = fwd_next_active(w, n_items, prm), ++n) {
      const FwdItem item = fwd_item(w, prm);
      if (!mbar_wait((n & 1) ? q_full2 : q_full, (n >> 1) & 1, status, ERR_ATTN_WAIT)) break;
      const uint64_t d_q = make_smem_desc_sw128(smem_u32(smem + AttnFwdSmem::Q + (n & 1) * AT_TILE_BYTES), 16, 1024);
      for (int j = 0; j < item.n_kv; ++j, ++g) {
        const int st = g & 1;
        if (!mbar_wait(&k_full[st], (g >> 1) & 1, status, ERR_ATTN_WAIT) ||
            !mbar_wait(&s_empty[st], ((g >> 1) & 1) ^ 1, status, ERR_ATTN_WAIT)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t d_k = make_smem_desc_sw128(smem_u32(smem + AttnFwdSmem::K + st * AT_TILE_BYTES), 16, 1024);
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t o = (ks >> 2) * AT_HALF_BYTES + (ks & 3) * 32;
            umma_f16_ss(tmem_S + st * 128, desc_advance(d_q, o), desc_advance(d_k, o), idesc_s, ks != 0);
          }
          umma_commit(&k_empty[st]);
          umma_commit(&s_full[st]);
          if (j + 1 == item.n_kv) umma_commit(&q_empty[n & 1]);   // last Q*K^T of the item: its Q slot is free
        }
      }
    }
  } else if (warp == 10) {
    // ---- O += P V of every global iteration ------------------------------------------------------
    const bool leader = elect_one();
    constexpr uint32_t idesc_pv = make_idesc_f16(1, 128, 128, 0, 1);
    int g = 0, n = 0;
    bool ok = true;
    for (int w = w0; w < n_items && ok; w = fwd_next_active(w, n_items, prm), ++n) {
      const FwdItem item = fwd_item(w, prm);
      // the softmax warps must have read the previous item's O before it is overwritten
      if (n > 0 && !mbar_wait(o_free, (n - 1) & 1, status, ERR_ATTN_WAIT)) break;
      for (int j = 0; j < item.n_kv; ++j, ++g) {
        const int st = g & 1;
        if (!mbar_wait(&p_full[st], (g >> 1) & 1, status, ERR_ATTN_WAIT) ||
            !mbar_wait(&v_full[st], (g >> 1) & 1, status, ERR_ATTN_WAIT)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t d_v = make_smem_desc_sw128(smem_u32(smem + AttnFwdSmem::V + st * AT_TILE_BYTES),
                                                  AT_HALF_BYTES, 1024);
        const uint32_t acc0 = j != 0;
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            // A = P from TMEM: 16 bf16 of K per instruction = 8 columns
            umma_f16_ts(tmem_O, tmem_P + st * 64 + ks * 8, desc_advance(d_v, ks * 2048), idesc_pv, ks ? 1u : acc0);
          }
          umma_commit(&v_empty[st]);
          umma_commit(&pv_done[st]);
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;         // which 64 key columns of every tile this thread handles
    const int r = quarter * 32 + lane;        // query row inside the tile
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = scale * 1.4426950408889634f;
    // the two threads of a row meet at a 64-thread named barrier (one per lane quarter)
    auto pair_barrier = [&]() {
      switch (quarter) {
        case 0: asm volatile("bar.sync 1, 64;" ::: "memory"); break;
        case 1: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
        case 2: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
        default: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
      }
    };
    bool ok = true;
    int g = 0, n = 0;
    for (int w = w0; w < n_items && ok; w = fwd_next_active(w, n_items, prm), ++n) {
      const FwdItem item = fwd_item(w, prm);
      const int q_idx = item.qt * 128 + r;      // index among this sequence's queries
      const int q_pos = item.kv_off + q_idx;    // last key this query may see
      float m_used = -INFINITY, l = 0.f;        // l: this thread's 64 columns only
      for (int j = 0; j < item.n_kv; ++j, ++g) {
        const int st = g & 1;
        const uint32_t ph = (g >> 1) & 1;
        if (!mbar_wait_warp(&s_full[st], ph, status, ERR_ATTN_WAIT)) { ok = false; break; }
        tc_fence_after();
        float s[64];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t t[32];
          tmem_ld_32x32b_x32(tmem_S + lane_off + st * 128 + half * 64 + c * 32, t);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(t[i]);
        }
        tc_fence_before();
        mbar_arrive_warp(&s_empty[st]);
        const bool need_mask = ((j + 1) * 128 > item.kv_off + item.qt * 128 + 1) || ((j + 1) * 128 > item.kv_len);
        if (need_mask) {
          const int col0 = j * 128 + half * 64;
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (col0 + i > q_pos || col0 + i >= item.kv_len) s[i] = -INFINITY;
        }
        // four independent max chains, then the partner's half through shared memory
        float mx0 = s[0], mx1 = s[1], mx2 = s[2], mx3 = s[3];
#pragma unroll
        for (int i = 4; i < 64; i += 4) {
          mx0 = fmaxf(mx0, s[i]);
          mx1 = fmaxf(mx1, s[i + 1]);
          mx2 = fmaxf(mx2, s[i + 2]);
          mx3 = fmaxf(mx3, s[i + 3]);
        }
        xchg[half * 128 + r] = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        pair_barrier();
        const float mx = fmaxf(xchg[r], xchg[128 + r]);
        pair_barrier();   // both have read before either writes the next tile's value
        const float m_new = fmaxf(m_used, mx);
        if (j > 0) {
          const bool need = (m_new - m_used) * sl2 > 8.f;   // same decision in both threads of the row
          if (__any_sync(0xffffffffu, need)) {
            // rare: O is rescaled, which needs the previous P*V complete
            if (!mbar_wait_warp(&pv_done[(g - 1) & 1], ((g - 1) >> 1) & 1, status, ERR_ATTN_WAIT)) { ok = false; break; }
            tc_fence_after();
            const float alpha = need ? exp2f((m_used - m_new) * sl2) : 1.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {   // this thread's 64 columns of O
              uint32_t t[16];
              tmem_ld_32x32b_x16(tmem_O + lane_off + half * 64 + c * 16, t);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * alpha);
              tmem_st_32x32b_x16(tmem_O + lane_off + half * 64 + c * 16, t);
            }
            tmem_st_wait();
            if (need) {
              l *= alpha;
              m_used = m_new;
            }
          }
        } else {
          m_used = m_new;
        }
        // the P buffer of this tile was last read by P*V two tiles ago
        if (g >= 2 && !mbar_wait_warp(&pv_done[st], ph ^ 1, status, ERR_ATTN_WAIT)) { ok = false; break; }
        const float mb = m_used * sl2;
        const uint32_t tP = tmem_P + lane_off + st * 64 + half * 32;   // this thread's 64 keys = 32 packed columns
        float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
        for (int c16 = 0; c16 < 2; ++c16) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float p0 = fast_exp2(fmaf(s[c16 * 32 + 2 * i], sl2, -mb));
            const float p1 = fast_exp2(fmaf(s[c16 * 32 + 2 * i + 1], sl2, -mb));
            rs0 += p0;
            rs1 += p1;
            pk[i] = pack_bf16x2(p0, p1);
          }
          tmem_st_32x32b_x16(tP + c16 * 16, pk);
        }
        tmem_st_wait();
        l += rs0 + rs1;
        tc_fence_before();
        mbar_arrive_warp(&p_full[st]);
      }
      // the last P*V of the item
      if (!ok || !mbar_wait_warp(&pv_done[(g - 1) & 1], ((g - 1) >> 1) & 1, status, ERR_ATTN_WAIT)) { ok = false; break; }
      tc_fence_after();
      // row sum = both halves; write-out: each thread normalises and stores its 64 columns of O
      xchg[half * 128 + r] = l;
      pair_barrier();
      const float lsum = xchg[r] + xchg[128 + r];
      pair_barrier();
      const float inv = 1.f / lsum;
      const bool in_range = q_idx < item.q_len;
      uint4 ov[8];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t t[32];
        tmem_ld_32x32b_x32(tmem_O + lane_off + half * 64 + c * 32, t);
        tmem_ld_wait();
        if (c == 1) {
          tc_fence_before();
          mbar_arrive_warp(o_free);   // this warp's part of O is in registers
        }
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          ov[c * 4 + v].x = pack_bf16x2(__uint_as_float(t[v * 8 + 0]) * inv, __uint_as_float(t[v * 8 + 1]) * inv);
          ov[c * 4 + v].y = pack_bf16x2(__uint_as_float(t[v * 8 + 2]) * inv, __uint_as_float(t[v * 8 + 3]) * inv);
          ov[c * 4 + v].z = pack_bf16x2(__uint_as_float(t[v * 8 + 4]) * inv, __uint_as_float(t[v * 8 + 5]) * inv);
          ov[c * 4 + v].w = pack_bf16x2(__uint_as_float(t[v * 8 + 6]) * inv, __uint_as_float(t[v * 8 + 7]) * inv);
        }
      }
      {
        const int wq0 = item.qt * 128 + quarter * 32;   // index (within the sequence) of this warp's first query row
        __nv_bfloat16* base = out + (static_cast<size_t>(item.row0 + quarter * 32) * Hq + item.head) * 128 + half * 64;
        warp_store_rows_128B(smem + AttnFwdSmem::EPI + (warp - 2) * 4096, ov, [&](int row) -> uint8_t* {
          if (wq0 + row >= item.q_len) return nullptr;
          return reinterpret_cast<uint8_t*>(base + static_cast<size_t>(row) * Hq * 128);
        });
      }
      if (half == 0 && in_range && lse_out)
        lse_out[static_cast<size_t>(item.head) * prm.total_q + item.row0 + r] = m_used * scale + __logf(lsum);
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

// q [Tq, Hq*128], out [Tq, Hq*128]; k rows have stride ld_k, v rows stride ld_v elements.
// Fixed length: cu_q = cu_k = nullptr, Tq = Tk = B*S.  Variable length: cu_q / cu_k are int32 [B+1]
// device arrays of row offsets, max_q = longest query run, total_q / total_k = row counts.
B2_EXPORT int b2_attn_fwd_varlen(const void* q, const void* k, const void* v, void* out, float* lse, int B,
                                 int S, int Hq, int Hkv, int head_dim, int ld_k, int ld_v, float scale,
                                 const int* cu_q, const int* cu_k, int max_q, int total_q, int total_k,
                                 void* stream_);

B2_EXPORT int b2_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S,
                          int Hq, int Hkv, int head_dim, int ld_v, float scale, void* stream_) {
  return b2_attn_fwd_varlen(q, k, v, out, lse, B, S, Hq, Hkv, head_dim, Hkv * 128, ld_v, scale, nullptr,
                            nullptr, S, B * S, B * S, stream_);
}

B2_EXPORT int b2_attn_fwd_varlen(const void* q, const void* k, const void* v, void* out, float* lse, int B,
                                 int S, int Hq, int Hkv, int head_dim, int ld_k, int ld_v, float scale,
                                 const int* cu_q, const int* cu_k, int max_q, int total_q, int total_k,
                                 void* stream_) {
  b2::ensure_thread_context();
  if (head_dim != 128 || Hq % Hkv != 0 || (ld_v % 8) != 0 || (ld_k % 8) != 0) {
    set_error("attn_fwd: head_dim must be 128, Hq %% Hkv == 0, ld_k / ld_v %% 8 == 0");
    return 10;
  }
  if (B <= 0 || max_q <= 0 || total_q <= 0) return 0;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             AttnFwdSmem::TOTAL) != cudaSuccess) {
      set_error("attn_fwd: cannot set shared memory size");
      return 1;
    }
    configured[dev] = true;
  }
  const CUtensorMap* tq = tensor_map_2d_bf16(q, total_q, static_cast<uint64_t>(Hq) * 128, static_cast<uint64_t>(Hq) * 128, 128, 64);
  const CUtensorMap* tk = tensor_map_2d_bf16(k, total_k, static_cast<uint64_t>(Hkv) * 128, ld_k, 128, 64);
  const CUtensorMap* tv = tensor_map_2d_bf16(v, total_k, static_cast<uint64_t>(Hkv) * 128, ld_v, 128, 64);
  if (!tq || !tk || !tv) return 2;
  int* status = status_ptr();
  if (!status) return 3;
  FwdParams prm;
  prm.S = S; prm.Hq = Hq; prm.Hkv = Hkv; prm.B = B; prm.max_tiles = (max_q + 127) / 128; prm.total_q = total_q;
  prm.cu_q = cu_q; prm.cu_k = cu_k;
  prm.block_tables = nullptr; prm.max_blocks = 0;
  const long long n_items = static_cast<long long>(prm.max_tiles) * Hq * B;
  const int grid = n_items < num_sms() ? static_cast<int>(n_items) : num_sms();
  attn_fwd_kernel<<<grid, AT_THREADS, AttnFwdSmem::TOTAL, stream>>>(
      *tq, *tk, *tv, static_cast<__nv_bfloat16*>(out), lse, prm, scale, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("attn_fwd launch failed: %s", cudaGetErrorString(e));
    return 4;
  }
  return 0;
}

// Chunked prefill over the paged KV cache: the keys / values of sequence b are the first kv_len[b] tokens of the
// cache blocks block_tables[b][*] (16 tokens per block, bf16, layout [blocks, 16, Hkv, 128]); its queries are the last
// q_len[b] of them (the chunk's own K / V must already be stored).  cu_q / cu_k: int32 [B+1] prefix sums of the query
// and key counts.  No gather of the context into a contiguous buffer: the TMA producer walks the block table.
B2_EXPORT int b2_attn_fwd_paged(const void* q, const void* k_cache, const void* v_cache, void* out, float* lse, int B,
                                int Hq, int Hkv, int head_dim, int num_blocks, float scale, const int* cu_q,
                                const int* cu_k, const int* block_tables, int max_blocks, int max_q, int total_q,
                                void* stream_) {
  b2::ensure_thread_context();
  if (head_dim != 128 || Hq % Hkv != 0 || block_tables == nullptr || cu_q == nullptr || cu_k == nullptr || max_blocks <= 0) {
    set_error("attn_fwd_paged: head_dim 128, Hq %% Hkv == 0, block tables and prefix sums required");
    return 10;
  }
  if (B <= 0 || max_q <= 0 || total_q <= 0) return 0;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             AttnFwdSmem::TOTAL) != cudaSuccess) {
      set_error("attn_fwd_paged: cannot set shared memory size");
      return 1;
    }
    configured[dev] = true;
  }
  const uint64_t W = static_cast<uint64_t>(Hkv) * 128;
  const CUtensorMap* tq = tensor_map_2d_bf16(q, total_q, static_cast<uint64_t>(Hq) * 128, static_cast<uint64_t>(Hq) * 128, 128, 64);
  const CUtensorMap* tk = tensor_map_2d_bf16(k_cache, static_cast<uint64_t>(num_blocks) * 16, W, W, 16, 64);
  const CUtensorMap* tv = tensor_map_2d_bf16(v_cache, static_cast<uint64_t>(num_blocks) * 16, W, W, 16, 64);
  if (!tq || !tk || !tv) return 2;
  int* status = status_ptr();
  if (!status) return 3;
  FwdParams prm;
  prm.S = 0; prm.Hq = Hq; prm.Hkv = Hkv; prm.B = B; prm.max_tiles = (max_q + 127) / 128; prm.total_q = total_q;
  prm.cu_q = cu_q; prm.cu_k = cu_k;
  prm.block_tables = block_tables; prm.max_blocks = max_blocks;
  const long long n_items = static_cast<long long>(prm.max_tiles) * Hq * B;
  const int grid = n_items < num_sms() ? static_cast<int>(n_items) : num_sms();
  attn_fwd_kernel<<<grid, AT_THREADS, AttnFwdSmem::TOTAL, stream>>>(
      *tq, *tk, *tv, static_cast<__nv_bfloat16*>(out), lse, prm, scale, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("attn_fwd_paged launch failed: %s", cudaGetErrorString(e));
    return 4;
  }
  return 0;
}
