// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma with
// fp32 accumulators in TMEM -> tcgen05.ld epilogue.
//
//   C[M,N] (+)= A[M,K] * B[N,K]^T  (+ R[M,N])
//
// Each operand may be stored with its contraction dimension contiguous ("K-major", e.g. activations
// [M,K] and nn.Linear weights [N,K]) or with its M/N dimension contiguous ("MN-major", e.g. the weight
// as the B operand of dX = dY * W, or dY / X as operands of dW = dY^T * X), so forward, grad-input and
// grad-weight GEMMs all run without a transpose pass.
//
// CTA layout (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (one elected lane) and TMEM
// owner, warps 2..5 = epilogue (one TMEM lane quarter each).  The bf16 epilogue goes through shared
// memory: every thread converts its row of a 64-column slab and writes it in the 128-byte-swizzled
// layout, then one thread issues a TMA store of the [128 x 64] slab (two slab buffers alternate); the
// residual / accumulate operand comes in the same way by a TMA load into the slab buffer.  Direct
// per-thread global stores would touch 32 different cache lines per warp instruction and made the
// epilogue, not the MMA, the limiter for short-K GEMMs.  Two TMEM accumulators of BN columns
// let the epilogue of tile i overlap the main loop of tile i+1.  One CTA per SM (TMEM and shared
// memory are sized for that), grid = min(#tiles, #SMs), static round-robin tile schedule with
// M-grouped rasterisation for L2 reuse.
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "host.h"

namespace b2 {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_GROUP_M = 16;

// epilogue flags
constexpr int GEMM_OUT_FP32 = 1;     // C is fp32 (else bf16)
constexpr int GEMM_ACCUMULATE = 2;   // C += result
constexpr int GEMM_RESIDUAL = 4;     // result += R (bf16, same ld as C)

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int SLAB_BYTES = GEMM_BM * 64 * 2;   // one [128 x 64] bf16 epilogue slab
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * SLAB_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int TMEM_COLS = 2 * BN;  // 512 or 256: powers of two
};

struct GemmMnDesc {
  uint32_t lbo, sbo, kstep;
};

// Communication fused into the GEMM (tensor-parallel layers with sequence-parallel activations):
//   COMM 1  GEMM -> reduce-scatter: every output tile is stored straight into the receive buffer of
//           the rank that owns those rows (peer stores over NVLink), a per-tile counter on the owner
//           is bumped with a system-scope release, and after its own tiles each CTA reduces finished
//           row blocks of THIS rank's shard (sum over source ranks + residual).
//   COMM 2  all-gather -> GEMM: four extra warps per CTA PUSH this rank's activation shard, piece by piece
//           (128 rows x 256 columns), into the gather buffer of every rank: one multimem.st through the
//           switch where the buffers are bound to a multicast object, else one store per peer.  Stores need
//           no round trip, so a few warps per SM keep NVLink full (loads from a peer are latency-bound).  A
//           piece ends with a system-scope release add on every rank's counter of that row block; the TMA
//           producer waits until the counter of the block it is about to load has all its pieces, then reads
//           A tiles from the LOCAL gather buffer.  No TMA ever targets another GPU's memory, no clusters.
struct GemmComm {
  void* peer_recv[8];       // COMM 1: [world][rows_per_rank][N] bf16 receive buffer on each rank
  int* peer_cnt[8];         // COMM 1: per (row block, n block) arrival counters on each rank
  void* peer_gather[8];     // COMM 2: [M][K] bf16 gather buffer on each rank (the A operand there)
  void* mc_gather;          // COMM 2: multicast address of the gather buffers (one store reaches every rank), or null
  int* peer_flags[8];       // COMM 2: per-128-row-block arrival counters on each rank
  int* peer_ready[8];       // COMM 2: [world] "rank p has entered call c" words on each rank
  const void* local_src;    // COMM 2: this rank's [rows_per_rank][K] bf16 activation shard (ordinary local memory)
  void* gather;             // COMM 2: this rank's gather buffer
  int* gather_flags;        // COMM 2: this rank's arrival counters
  int ready_epoch;          // COMM 2: number of this call among the context's fused all-gather calls
  int pieces_per_block;     // COMM 2: column chunks a 128-row block is pushed in (arrivals per block and call)
  void* out;                // COMM 1: [rows_per_rank][N] bf16 result of the reduce
  const void* residual;     // COMM 1: optional [rows_per_rank][N] bf16 added in the reduce
  int world, rank, rows_per_rank, epoch;
};

__device__ __forceinline__ void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys_s32(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_gpu_s32(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_s32(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded spin until *p >= value (acquire).  sys: the writer is another GPU.
template <bool SYS>
__device__ __forceinline__ bool wait_flag_ge(const int* p, int value, int* status, int code) {
  unsigned long long t0 = 0;
  for (uint32_t it = 0;; ++it) {
    const int v = SYS ? ld_acquire_sys_s32(p) : ld_acquire_gpu_s32(p);
    if (v >= value) return true;
    if ((it & 63u) == 63u) {
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (*reinterpret_cast<volatile int*>(status) != 0) return false;
      if (now - t0 > (SYS ? PEER_WAIT_LIMIT_NS : WAIT_LIMIT_NS)) {
        atomicCAS(status, 0, code);
        return false;
      }
    }
    __nanosleep(100);
  }
}

// Sum ROWS rows per step over up to MAXW source ranks (all loads issued before the first add, so that
// enough requests are in flight to be bound by HBM bandwidth), add the residual, store bf16.
template <int ROWS, int MAXW, int WARPS>
__device__ __forceinline__ void reduce_rows(const __nv_bfloat16* __restrict__ recv, const GemmComm& comm, int rb,
                                            int c, int N, int ewarp) {
  for (int rr = ewarp * ROWS; rr < GEMM_BM; rr += WARPS * ROWS) {
    uint4 q[ROWS][MAXW];
    uint4 rq[ROWS];
#pragma unroll
    for (int u = 0; u < ROWS; ++u) {
      const int lrow = rb * GEMM_BM + rr + u;
#pragma unroll
      for (int s_ = 0; s_ < MAXW; ++s_)
        if (s_ < comm.world)
          q[u][s_] = __ldcg(reinterpret_cast<const uint4*>(
              recv + (static_cast<size_t>(s_) * comm.rows_per_rank + lrow) * N + c));
      if (comm.residual)
        rq[u] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(comm.residual) +
                                                static_cast<size_t>(lrow) * N + c);
    }
#pragma unroll
    for (int u = 0; u < ROWS; ++u) {
      const int lrow = rb * GEMM_BM + rr + u;
      float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s_ = 0; s_ < MAXW; ++s_) {
        if (s_ < comm.world) {
          const uint32_t w[4] = {q[u][s_].x, q[u][s_].y, q[u][s_].z, q[u][s_].w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 f = unpack_bf16x2(w[k]);
            a[2 * k] += f.x;
            a[2 * k + 1] += f.y;
          }
        }
      }
      if (comm.residual) {
        const uint32_t w[4] = {rq[u].x, rq[u].y, rq[u].z, rq[u].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = unpack_bf16x2(w[k]);
          a[2 * k] += f.x;
          a[2 * k + 1] += f.y;
        }
      }
      uint4 o;
      o.x = pack_bf16x2(a[0], a[1]);
      o.y = pack_bf16x2(a[2], a[3]);
      o.z = pack_bf16x2(a[4], a[5]);
      o.w = pack_bf16x2(a[6], a[7]);
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(comm.out) + static_cast<size_t>(lrow) * N + c) = o;
    }
  }
}

// Second operand pair appended along the contraction: C = A * B^T + A2 * B2^T in ONE accumulator pass (k-blocks of
// the first pair, then of the second).  A2 is K-major [M, K2]; B2 has the layout of B ([N, K2], or [K2, N] when B is
// MN-major).  A LoRA update rides in the base projection this way: A2 = x * A_lora^T (rank columns), B2 = scaled B_lora,
// with no second pass over the [M, N] output.  K2 = 0: no second pair.
struct GemmExt {
  CUtensorMap tmA2, tmB2;
  int K2;
};

template <int BN, bool A_MN, bool B_MN, int COMM>
__global__ void __launch_bounds__(GEMM_THREADS + (COMM == 2 ? 128 : COMM == 1 ? 64 : 0), 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmR,
                 void* __restrict__ Cout, const __nv_bfloat16* __restrict__ R, int M, int N, int K,
                 int ldc, int flags, GemmMnDesc mn, const __grid_constant__ GemmComm comm, int* status,
                 int split_k, const __grid_constant__ GemmExt ext) {
  using Cfg = GemmCfg<BN>;
  static_assert(COMM == 0 || !A_MN, "fused communication paths take a K-major A operand");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* slabs = smem + Cfg::STAGES * Cfg::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(slabs + 2 * Cfg::SLAB_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + Cfg::STAGES;
  uint64_t* tmem_full = bars + 2 * Cfg::STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint64_t* addend_bar = tmem_empty + 2;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(addend_bar + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // in the fused kernels every pipeline wait sits downstream of a wait for another GPU: same (long) bound
  constexpr unsigned long long LIM = COMM != 0 ? PEER_WAIT_LIMIT_NS : WAIT_LIMIT_NS;

  const int num_m = (M + GEMM_BM - 1) / GEMM_BM;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + GEMM_BK - 1) / GEMM_BK;
  const int num_kb2 = (COMM == 0 && !A_MN && split_k == 1) ? (ext.K2 + GEMM_BK - 1) / GEMM_BK : 0;
  // Split-K (fp32 accumulate outputs only): a work unit is (tile, K slice); unit u covers tile
  // u % num_tiles and k-blocks [ks * num_kb / split_k, (ks + 1) * num_kb / split_k) with ks = u / num_tiles,
  // and its epilogue adds into C with fp32 atomics.  Weight-gradient GEMMs have few output tiles and a
  // very long contraction (the token count): without the split, 96 tiles leave a third of the SMs idle.
  const int num_units = num_tiles * split_k;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 128);
      mbar_init(&addend_bar[a], 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  auto tile_coords = [&](int t, int& m_blk, int& n_blk) {
    const int per_group = GEMM_GROUP_M * num_n;
    const int g = t / per_group;
    const int first_m = g * GEMM_GROUP_M;
    const int gsz = min(GEMM_GROUP_M, num_m - first_m);
    const int r = t - g * per_group;
    m_blk = first_m + (r % gsz);
    n_blk = r / gsz;
    if (COMM == 1) {
      // Consecutive row blocks of the schedule belong to consecutive owners (starting with the next rank, own rows
      // last): every rank works on row block j of ALL owners before block j + 1, so block j of every shard is
      // complete on all sources after (j + 1) / blocks-per-rank of the kernel and its owner can reduce it while the
      // GEMM goes on.  (A rank-by-rank order finishes every shard only at the very end: the whole reduce is exposed.)
      const int bpr = comm.rows_per_rank / GEMM_BM;
      const int j = m_blk / comm.world, s_ = m_blk % comm.world;
      m_blk = ((s_ + comm.rank + 1) % comm.world) * bpr + j;
    } else if (COMM == 2) {
      // this rank's own row blocks first (they are read from the local shard and depend on nobody), then, since
      // every rank pushes its row block j at about the same time, block j of all other sources before block j + 1
      const int bpr = comm.rows_per_rank / GEMM_BM;
      if (m_blk < bpr || comm.world == 1) {
        m_blk = comm.rank * bpr + m_blk;
      } else {
        const int v = m_blk - bpr;
        const int j = v / (comm.world - 1), s_ = v % (comm.world - 1) + 1;
        m_blk = ((comm.rank + s_) % comm.world) * bpr + j;
      }
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
        const int t = u % num_tiles, ks = u / num_tiles;
        const int kb_begin = ks * num_kb / split_k, kb_end = (ks + 1) * num_kb / split_k;
        int m_blk, n_blk;
        tile_coords(t, m_blk, n_blk);
        const int m0 = m_blk * GEMM_BM, n0 = n_blk * BN;
        // COMM 2: own rows come straight from this rank's shard (tensor map tmR); a peer's rows must have arrived
        // in the local gather buffer
        const int own0 = COMM == 2 ? comm.rank * (comm.rows_per_rank / GEMM_BM) : 0;
        const bool own = COMM == 2 && m_blk >= own0 && m_blk < own0 + comm.rows_per_rank / GEMM_BM;
        if (COMM == 2 && !own) {
          if (!wait_flag_ge<true>(comm.gather_flags + m_blk, comm.epoch * comm.pieces_per_block, status,
                                  ERR_COMM_FLAG_WAIT)) {
            ok = false;
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        const CUtensorMap* mapA = own ? &tmR : &tmA;
        const int a_row = own ? m0 - own0 * GEMM_BM : m0;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, status, ERR_GEMM_PRODUCER_WAIT, LIM)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sB = sA + Cfg::A_BYTES;
          mbar_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          if (!A_MN) {
            tma_load_2d(sA, mapA, &full_bar[stage], kb * GEMM_BK, a_row);
          } else {
#pragma unroll
            for (int c = 0; c < GEMM_BM / 64; ++c)
              tma_load_2d(sA + c * 8192, &tmA, &full_bar[stage], m0 + c * 64, kb * GEMM_BK);
          }
          if (!B_MN) {
            tma_load_2d(sB, &tmB, &full_bar[stage], kb * GEMM_BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sB + c * 8192, &tmB, &full_bar[stage], n0 + c * 64, kb * GEMM_BK);
          }
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        // the second operand pair's k-blocks (rows past K2 are filled with zeros by the TMA unit)
        for (int kb = 0; kb < num_kb2 && ok; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, status, ERR_GEMM_PRODUCER_WAIT, LIM)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sB = sA + Cfg::A_BYTES;
          mbar_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          tma_load_2d(sA, &ext.tmA2, &full_bar[stage], kb * GEMM_BK, m0);
          if (!B_MN) {
            tma_load_2d(sB, &ext.tmB2, &full_bar[stage], kb * GEMM_BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sB + c * 8192, &ext.tmB2, &full_bar[stage], n0 + c * 64, kb * GEMM_BK);
          }
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // The whole warp runs this (uniform) control flow so that descriptors and addresses stay in the
    // uniform datapath; only the tcgen05 instructions themselves are issued by one elected lane.
    {
      const bool leader = elect_one();
      constexpr uint32_t idesc = make_idesc_f16(1, GEMM_BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
        const int ks = u / num_tiles;
        const int kb_begin = ks * num_kb / split_k, kb_end = (ks + 1) * num_kb / split_k;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, status, ERR_GEMM_MMA_WAIT_TMEM, LIM)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb_begin; kb < kb_end + num_kb2; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, status, ERR_GEMM_MMA_WAIT_FULL, LIM)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t b_base = a_base + Cfg::A_BYTES;
          const uint64_t a0 = A_MN ? make_smem_desc_sw128(a_base, mn.lbo, mn.sbo) : make_smem_desc_sw128(a_base, 16, 1024);
          const uint64_t b0 = B_MN ? make_smem_desc_sw128(b_base, mn.lbo, mn.sbo) : make_smem_desc_sw128(b_base, 16, 1024);
          const uint32_t a_step = A_MN ? mn.kstep : 32u, b_step = B_MN ? mn.kstep : 32u;
          const uint32_t acc0 = kb != kb_begin ? 1u : 0u;
          // a k-block of the second pair holds K2 - 64 * i valid columns: skip the 16-wide steps that are all zeros
          const int ksteps = kb < kb_end ? GEMM_BK / 16 : min(GEMM_BK / 16, (ext.K2 - (kb - kb_end) * GEMM_BK + 15) / 16);
          if (leader) {
#pragma unroll
            for (int k = 0; k < GEMM_BK / 16; ++k)
              if (k < ksteps)
                umma_f16_ss(d_tmem, desc_advance(a0, k * a_step), desc_advance(b0, k * b_step), idesc, k ? 1u : acc0);
            umma_commit(&empty_bar[stage]);
          }
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (leader) umma_commit(&tmem_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else if (COMM == 1 && warp >= 6) {
    // ---- reduce warps: sum this rank's row blocks over all source ranks as they complete --------------------
    // A job is (row block rb of this rank's shard, column block nb), dealt to the CTAs in the order the row blocks
    // complete (see tile_coords).  These two warps only wait and move memory (two, not four: 256 threads per CTA
    // keep the full register budget for the epilogue), so the reduction of block j runs under the MMAs and
    // epilogues of the blocks after it instead of behind the last tile.
    const int ct = threadIdx.x - 192;                 // 0..63
    const int rwarp = ct >> 5;
    const int rjobs = (comm.rows_per_rank / GEMM_BM) * num_n;
    const __nv_bfloat16* recv = static_cast<const __nv_bfloat16*>(comm.peer_recv[comm.rank]);
    const int* cnt = comm.peer_cnt[comm.rank];
    bool ok = true;
    for (int job = blockIdx.x; job < rjobs; job += gridDim.x) {
      if (ct == 0 && ok) ok = wait_flag_ge<true>(cnt + job, comm.world * comm.epoch, status, ERR_COMM_FLAG_WAIT);
      if (named_barrier_or(2, 64, !ok)) break;
      const int rb = job / num_n, nb = job % num_n;
      const int c = nb * BN + lane * 8;               // 32 lanes x 8 columns = one 256-column row segment
      if (c >= N || (BN == 128 && lane >= 16)) continue;
      if (comm.world <= 4)
        reduce_rows<4, 4, 2>(recv, comm, rb, c, N, rwarp);
      else
        reduce_rows<2, 8, 2>(recv, comm, rb, c, N, rwarp);
    }
  } else if (COMM == 2 && warp >= 6) {
    // ---- push warps: this rank's shard -> every rank's gather buffer, piece by piece ---------------------
    const int ct = threadIdx.x - 192;                 // 0..127
    const int bpr = comm.rows_per_rank / GEMM_BM;
    // Arrival: a peer that has entered this call has (in its stream order) finished every earlier kernel that
    // read the gather buffer this call overwrites.
    if (blockIdx.x == 0 && ct < comm.world) {
      __threadfence_system();
      asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(comm.peer_ready[ct] + comm.rank), "r"(comm.ready_epoch) : "memory");
    }
    bool ok = true;
    if (ct < comm.world)
      ok = wait_flag_ge<true>(comm.peer_ready[comm.rank] + ct, comm.ready_epoch, status, ERR_COMM_FLAG_WAIT);
    if (!named_barrier_or(2, 128, !ok)) {
      constexpr int CW = 256;                          // columns per piece
      const bool use_mc = comm.mc_gather != nullptr;
      const int chunks = comm.pieces_per_block;
      const int pieces = bpr * chunks;
      const __nv_bfloat16* src0 = static_cast<const __nv_bfloat16*>(comm.local_src);
      for (int p = blockIdx.x; p < pieces; p += gridDim.x) {
        const int b = p / chunks, c0 = (p % chunks) * CW;
        const int cw = min(CW, K - c0);
        const int vpr = cw >> 3;                       // 16-byte vectors per row of the piece
        const int total = GEMM_BM * vpr;
        const __nv_bfloat16* src = src0 + static_cast<size_t>(b) * GEMM_BM * K + c0;
        const size_t dst_off = (static_cast<size_t>(comm.rank) * bpr + b) * GEMM_BM * K + c0;
        for (int v = ct; v < total; v += 128 * 8) {
          uint4 t[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int vv = v + u * 128;
            t[u] = make_uint4(0u, 0u, 0u, 0u);
            if (vv < total) t[u] = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(vv / vpr) * K + (vv % vpr) * 8);
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int vv = v + u * 128;
            if (vv < total) {
              const size_t off = dst_off + static_cast<size_t>(vv / vpr) * K + (vv % vpr) * 8;
              if (use_mc) {
                asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(
                                 static_cast<__nv_bfloat16*>(comm.mc_gather) + off),
                             "r"(t[u].x), "r"(t[u].y), "r"(t[u].z), "r"(t[u].w) : "memory");
              } else {
#pragma unroll
                for (int r = 0; r < 8; ++r)
                  if (r < comm.world)
                    *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(comm.peer_gather[r]) + off) = t[u];
              }
            }
          }
        }
        // the piece's stores (all 128 threads) happen before the barrier; the release below, by one lane per
        // destination rank, is cumulative over them: no system-scope fence in every thread
        named_barrier(2, 128);
        if (ct < comm.world) red_release_sys_add(comm.peer_flags[ct] + comm.rank * bpr + b, 1);
      }
    }
  } else {
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t acc = 0, acc_phase = 0;
    const bool out_fp32 = flags & GEMM_OUT_FP32;
    const bool accumulate = flags & GEMM_ACCUMULATE;
    const bool residual = flags & GEMM_RESIDUAL;
    uint32_t slab_count = 0;
    const bool atomic_out = split_k > 1;   // several units add into the same fp32 tile
    for (int u = blockIdx.x; u < num_units; u += gridDim.x) {
      const int t = u % num_tiles;
      int m_blk, n_blk;
      tile_coords(t, m_blk, n_blk);
      const int n0 = n_blk * BN;
      const int row = m_blk * GEMM_BM + quarter * 32 + lane;
      if (COMM == 1) {
        // leave together: the epilogue threads meet at named barriers further down
        const bool got = mbar_wait(&tmem_full[acc], acc_phase, status, ERR_GEMM_EPI_WAIT, LIM);
        if (named_barrier_or(1, 128, !got)) break;
      } else if (!mbar_wait(&tmem_full[acc], acc_phase, status, ERR_GEMM_EPI_WAIT, LIM)) {
        break;
      }
      tc_fence_after();
      const uint32_t t_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      if (COMM == 1) {
        // ---- reduce-scatter: store the tile into the owner's receive slot for this source rank -------
        const int owner = (m_blk * GEMM_BM) / comm.rows_per_rank;
        const int lrow0 = m_blk * GEMM_BM - owner * comm.rows_per_rank;   // tile's first row inside the owner's shard
        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(comm.peer_recv[owner]) +
                             (static_cast<size_t>(comm.rank) * comm.rows_per_rank + lrow0) * N;
        const int r = quarter * 32 + lane;
        const int et = threadIdx.x - 64;          // 0..127
        uint8_t* sbuf = slabs;
        // Each 64-column slab goes registers -> swizzled shared memory -> full 128-byte row segments to
        // the owner (8 lanes per row), so the NVLink writes are whole lines instead of scattered 16-byte pieces.
#pragma unroll 1
        for (int sl = 0; sl < BN / 64; ++sl) {
          uint32_t v[64];
          {
            uint32_t t[32];
            tmem_ld_32x32b_x32(t_base + sl * 64, t);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = t[i];
            tmem_ld_32x32b_x32(t_base + sl * 64 + 32, t);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[32 + i] = t[i];
          }
          named_barrier(1, 128);                  // the previous slab has been read out of shared memory
          uint8_t* rowp = sbuf + r * 128;
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[c8 * 8 + 0]), __uint_as_float(v[c8 * 8 + 1]));
            o.y = pack_bf16x2(__uint_as_float(v[c8 * 8 + 2]), __uint_as_float(v[c8 * 8 + 3]));
            o.z = pack_bf16x2(__uint_as_float(v[c8 * 8 + 4]), __uint_as_float(v[c8 * 8 + 5]));
            o.w = pack_bf16x2(__uint_as_float(v[c8 * 8 + 6]), __uint_as_float(v[c8 * 8 + 7]));
            *reinterpret_cast<uint4*>(rowp + ((c8 ^ (r & 7)) << 4)) = o;
          }
          named_barrier(1, 128);
          const int col0 = n0 + sl * 64;
          const int ch = et & 7;
          if (col0 + ch * 8 < N) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rowi = (et >> 3) + 16 * i;
              const uint4 val = *reinterpret_cast<const uint4*>(sbuf + rowi * 128 + ((ch ^ (rowi & 7)) << 4));
              if (m_blk * GEMM_BM + rowi < M)
                *reinterpret_cast<uint4*>(dst + static_cast<size_t>(rowi) * N + col0 + ch * 8) = val;
            }
          }
        }
        tc_fence_before();
        mbar_arrive(&tmem_empty[acc]);
        // every thread's peer stores happen before this barrier; the system-scope release below (one lane) is
        // cumulative over them, so the other 127 threads go on to the next tile without a fence of their own
        named_barrier(1, 128);
        if (warp == 2 && lane == 0) {
          const int rb = (m_blk * GEMM_BM - owner * comm.rows_per_rank) / GEMM_BM;
          red_release_sys_add(comm.peer_cnt[owner] + rb * num_n + n_blk, 1);
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
        continue;
      }
      if (!out_fp32) {
        // ---- bf16 output: shared-memory slabs + TMA store ------------------------------------------
        const int r = quarter * 32 + lane;
        const bool issuer = (warp == 2 && lane == 0);
        const bool addend = accumulate || residual;
        const int m0 = m_blk * GEMM_BM;
        bool ok = true;
#pragma unroll 1
        for (int sl = 0; sl < BN / 64; ++sl) {
          const int buf = slab_count & 1;
          uint8_t* sbuf = slabs + buf * Cfg::SLAB_BYTES;
          const int col0 = n0 + sl * 64;
          if (issuer) tma_store_wait_read<1>();     // the store that used this buffer two slabs ago is done
          named_barrier(1, 128);
          if (addend && issuer && col0 < N) {
            mbar_expect_tx(&addend_bar[buf], Cfg::SLAB_BYTES);
            tma_load_2d(sbuf, accumulate ? &tmC : &tmR, &addend_bar[buf], col0, m0);
          }
          uint32_t v[64];
          {
            uint32_t t[32];
            tmem_ld_32x32b_x32(t_base + sl * 64, t);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = t[i];
            tmem_ld_32x32b_x32(t_base + sl * 64 + 32, t);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[32 + i] = t[i];
          }
          if (sl == BN / 64 - 1) {   // accumulator fully read: hand it back to the MMA warp
            tc_fence_before();
            mbar_arrive(&tmem_empty[acc]);
          }
          if (col0 < N) {
            uint8_t* rowp = sbuf + r * 128;
            if (addend) {
              if (ok) ok = mbar_wait(&addend_bar[buf], (slab_count >> 1) & 1, status, ERR_GEMM_EPI_WAIT);
#pragma unroll
              for (int c8 = 0; c8 < 8; ++c8) {
                const uint4 q = *reinterpret_cast<const uint4*>(rowp + ((c8 ^ (r & 7)) << 4));
                const uint32_t qq[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 f = unpack_bf16x2(qq[j]);
                  v[c8 * 8 + 2 * j] = __float_as_uint(__uint_as_float(v[c8 * 8 + 2 * j]) + f.x);
                  v[c8 * 8 + 2 * j + 1] = __float_as_uint(__uint_as_float(v[c8 * 8 + 2 * j + 1]) + f.y);
                }
              }
            }
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(v[c8 * 8 + 0]), __uint_as_float(v[c8 * 8 + 1]));
              o.y = pack_bf16x2(__uint_as_float(v[c8 * 8 + 2]), __uint_as_float(v[c8 * 8 + 3]));
              o.z = pack_bf16x2(__uint_as_float(v[c8 * 8 + 4]), __uint_as_float(v[c8 * 8 + 5]));
              o.w = pack_bf16x2(__uint_as_float(v[c8 * 8 + 6]), __uint_as_float(v[c8 * 8 + 7]));
              *reinterpret_cast<uint4*>(rowp + ((c8 ^ (r & 7)) << 4)) = o;
            }
          }
          fence_proxy_async_smem();
          named_barrier(1, 128);
          if (col0 < N) {
            if (issuer) {
              tma_store_2d(&tmC, sbuf, col0, m0);
              tma_store_commit();
            }
            ++slab_count;    // buffer parity and addend-barrier phase advance only when a slab was used
          }
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
        if (named_barrier_or(1, 128, !ok)) break;   // all 128 epilogue threads leave together
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_base + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row < M && col0 < N) {
          const size_t off = static_cast<size_t>(row) * ldc + col0;
          const bool full = (col0 + 32 <= N);
          if (residual) {
            const __nv_bfloat16* rp = R + off;
            if (full) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 q = *reinterpret_cast<const uint4*>(rp + v * 8);
                const uint32_t qq[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float2 f = unpack_bf16x2(qq[j]);
                  r[v * 8 + 2 * j] = __float_as_uint(__uint_as_float(r[v * 8 + 2 * j]) + f.x);
                  r[v * 8 + 2 * j + 1] = __float_as_uint(__uint_as_float(r[v * 8 + 2 * j + 1]) + f.y);
                }
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < N; ++j)
                r[j] = __float_as_uint(__uint_as_float(r[j]) + __bfloat162float(rp[j]));
            }
          }
          if (out_fp32) {
            float* cp = reinterpret_cast<float*>(Cout) + off;
            if (full) {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4 o = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                       __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                if (atomic_out) {
                  atomicAdd(reinterpret_cast<float4*>(cp + 4 * v), o);
                  continue;
                }
                if (accumulate) {
                  float4 p = *reinterpret_cast<float4*>(cp + 4 * v);
                  o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
                }
                *reinterpret_cast<float4*>(cp + 4 * v) = o;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < N; ++j) {
                if (atomic_out) atomicAdd(cp + j, __uint_as_float(r[j]));
                else cp[j] = __uint_as_float(r[j]) + (accumulate ? cp[j] : 0.f);
              }
            }
          } else {
            __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(Cout) + off;
            if (full) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]);
                if (accumulate) {
                  uint4 q = *reinterpret_cast<const uint4*>(cp + v * 8);
                  const uint32_t qq[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    float2 p = unpack_bf16x2(qq[j]);
                    f[2 * j] += p.x;
                    f[2 * j + 1] += p.y;
                  }
                }
                uint4 o;
                o.x = pack_bf16x2(f[0], f[1]);
                o.y = pack_bf16x2(f[2], f[3]);
                o.z = pack_bf16x2(f[4], f[5]);
                o.w = pack_bf16x2(f[6], f[7]);
                *reinterpret_cast<uint4*>(cp + v * 8) = o;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < N; ++j) {
                float f = __uint_as_float(r[j]);
                if (accumulate) f += __bfloat162float(cp[j]);
                cp[j] = __float2bfloat16(f);
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&tmem_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (warp == 2 && lane == 0) tma_store_wait_all<0>();   // shared memory stays valid until stores have read it
  }

  // Common tail: every thread arrives here, also after a wait that ran out.
  if (*reinterpret_cast<volatile int*>(status) != 0) {
    // give TMA copies and MMAs still in flight time to land before shared memory / TMEM go away
    unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

static GemmMnDesc g_mn_desc = {8192u, 1024u, 2048u};

template <int BN, bool A_MN, bool B_MN, int COMM = 0>
static int launch_gemm(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                       int lda, int ldb, int ldc, int flags, int max_ctas, cudaStream_t stream,
                       const GemmComm* comm_in = nullptr, const void* A2 = nullptr, const void* B2 = nullptr,
                       int K2 = 0, int lda2 = 0, int ldb2 = 0) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, COMM>;
  GemmComm comm;
  memset(&comm, 0, sizeof(comm));
  if (comm_in) comm = *comm_in;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) !=
        cudaSuccess) {
      set_error("gemm: cudaFuncSetAttribute(smem=%d) failed", Cfg::SMEM_BYTES);
      return 1;
    }
    configured[dev] = true;
  }
  const CUtensorMap* ta = A_MN ? tensor_map_2d_bf16(A, K, M, lda, 64, 64)
                               : tensor_map_2d_bf16(A, M, K, lda, GEMM_BM, 64);
  const CUtensorMap* tb = B_MN ? tensor_map_2d_bf16(B, K, N, ldb, 64, 64)
                               : tensor_map_2d_bf16(B, N, K, ldb, BN, 64);
  if (!ta || !tb) return 2;
  const bool out_fp32 = flags & GEMM_OUT_FP32;
  const CUtensorMap* tc = (out_fp32 || COMM == 1) ? ta : tensor_map_2d_bf16(C, M, N, ldc, GEMM_BM, 64);
  const CUtensorMap* tr = (!out_fp32 && (flags & GEMM_RESIDUAL)) ? tensor_map_2d_bf16(R, M, N, ldc, GEMM_BM, 64) : tc;
  if (COMM == 2)   // the second A map: this rank's own activation shard, read in place
    tr = tensor_map_2d_bf16(comm.local_src, comm.rows_per_rank, K, K, GEMM_BM, 64);
  if (!tc || !tr) return 2;
  int* status = status_ptr();
  if (!status) return 3;
  const int num_tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + BN - 1) / BN);
  int grid = num_sms();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  // Split-K for fp32 outputs with a long contraction: pick the split that minimises the number of
  // waves times the work per unit (ties go to the smaller split); every slice keeps >= 16 k-blocks.
  int split_k = 1;
  // B200FW_DETERMINISTIC=1 keeps one unit per output tile: split-K slices add into C with float atomics, whose
  // order changes from run to run
  static const bool deterministic = [] {
    const char* e = std::getenv("B200FW_DETERMINISTIC");
    return e != nullptr && e[0] == '1';
  }();
  if (COMM == 0 && out_fp32 && !(flags & GEMM_RESIDUAL) && !deterministic) {
    const int num_kb = (K + GEMM_BK - 1) / GEMM_BK;
    double best = static_cast<double>((num_tiles + grid - 1) / grid);
    for (int sk = 2; sk <= 4 && num_kb / sk >= 16; ++sk) {
      const double cost = static_cast<double>((num_tiles * sk + grid - 1) / grid) / sk;
      if (cost < best * 0.95) {
        best = cost;
        split_k = sk;
      }
    }
    if (split_k > 1 && !(flags & GEMM_ACCUMULATE)) {
      // the slices add into C with atomics: an overwriting GEMM starts from zero
      if (cudaMemset2DAsync(C, static_cast<size_t>(ldc) * 4, 0, static_cast<size_t>(N) * 4, M, stream) != cudaSuccess) {
        set_error("gemm: clearing the split-K output failed");
        return 5;
      }
    }
  }
  if (num_tiles * split_k < grid) grid = num_tiles * split_k;
  GemmExt ext;
  ext.tmA2 = *ta;
  ext.tmB2 = *tb;
  ext.K2 = 0;
  if (K2 > 0) {
    if (COMM != 0 || A_MN || split_k != 1) {
      set_error("gemm: a second operand pair needs a K-major A, no split-K and no fused collective");
      return 6;
    }
    const CUtensorMap* ta2 = tensor_map_2d_bf16(A2, M, K2, lda2, GEMM_BM, 64);
    const CUtensorMap* tb2 = B_MN ? tensor_map_2d_bf16(B2, K2, N, ldb2, 64, 64)
                                  : tensor_map_2d_bf16(B2, N, K2, ldb2, BN, 64);
    if (!ta2 || !tb2) return 2;
    ext.tmA2 = *ta2;
    ext.tmB2 = *tb2;
    ext.K2 = K2;
  }
  kern<<<grid, GEMM_THREADS + (COMM == 2 ? 128 : COMM == 1 ? 64 : 0), Cfg::SMEM_BYTES, stream>>>(
      *ta, *tb, *tc, *tr, C, reinterpret_cast<const __nv_bfloat16*>(R), M, N, K, ldc, flags, g_mn_desc, comm, status,
      split_k, ext);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("gemm launch failed: %s", cudaGetErrorString(e));
    return 4;
  }
  return 0;
}

}  // namespace b2

// C[M,N] (+)= A * B^T (+ R).  a_mn / b_mn: 0 = operand stored [rows, K] (K contiguous),
// 1 = operand stored [K, rows] (rows contiguous).  lda / ldb / ldc in elements.
// flags: 1 fp32 output, 2 accumulate into C, 4 add bf16 residual R.  bn: 0 = auto, else 128 / 256.
// max_ctas: 0 = all SMs; a smaller grid leaves SMs free for a concurrent kernel.
B2_EXPORT int b2_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                           int lda, int ldb, int ldc, int a_mn, int b_mn, int flags, int bn,
                           int max_ctas, void* stream_) {
  b2::ensure_thread_context();
  using namespace b2;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const bool out_fp32 = flags & GEMM_OUT_FP32;
  if ((lda % 8) || (ldb % 8) || (ldc % (out_fp32 ? 4 : 8)) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15) || ((flags & GEMM_RESIDUAL) && (R == nullptr ||
      (reinterpret_cast<uintptr_t>(R) & 15)))) {
    set_error("gemm: operands need 16-byte aligned bases and leading dimensions (lda %d ldb %d ldc %d)",
              lda, ldb, ldc);
    return 10;
  }
  if (bn == 0) {
    const int sms = num_sms();
    const int tiles256 = ((M + 127) / 128) * ((N + 255) / 256);
    bn = (tiles256 >= sms || N % 256 == 0) && tiles256 * 2 > sms ? 256 : 128;
    // fp32 accumulate outputs with a long contraction can split K instead of shrinking the tile
    if (out_fp32 && N % 256 == 0 && K >= 4096) bn = 256;
  }
#define B2_GEMM_CASE(BN_, AMN_, BMN_)                                                              \
  if (bn == BN_ && a_mn == AMN_ && b_mn == BMN_)                                                   \
    return launch_gemm<BN_, AMN_ != 0, BMN_ != 0>(A, B, C, R, M, N, K, lda, ldb, ldc, flags, max_ctas, stream);
  B2_GEMM_CASE(256, 0, 0)
  B2_GEMM_CASE(256, 0, 1)
  B2_GEMM_CASE(256, 1, 1)
  B2_GEMM_CASE(256, 1, 0)
  B2_GEMM_CASE(128, 0, 0)
  B2_GEMM_CASE(128, 0, 1)
  B2_GEMM_CASE(128, 1, 1)
  B2_GEMM_CASE(128, 1, 0)
#undef B2_GEMM_CASE
  set_error("gemm: unsupported configuration bn=%d a_mn=%d b_mn=%d", bn, a_mn, b_mn);
  return 11;
}

// C[M,N] = A * B^T + A2 * B2^T (+ R) with both products in one accumulator pass (see GemmExt).  A and A2 are K-major
// ([M, K], [M, K2]); B2 has B's layout.  K2 and both leading dimensions must be multiples of 8 elements.  Output bf16
// (flags: 2 accumulate into C, 4 add residual R) or fp32 (flag 1, no split-K).
B2_EXPORT int b2_gemm_bf16_ext(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda,
                               int ldb, int ldc, int b_mn, int flags, int bn, const void* A2, const void* B2, int K2,
                               int lda2, int ldb2, void* stream_) {
  b2::ensure_thread_context();
  using namespace b2;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const bool out_fp32 = flags & GEMM_OUT_FP32;
  if ((lda % 8) || (ldb % 8) || (ldc % (out_fp32 ? 4 : 8)) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(C) & 15) ||
      ((flags & GEMM_RESIDUAL) && (R == nullptr || (reinterpret_cast<uintptr_t>(R) & 15)))) {
    set_error("gemm_ext: operands need 16-byte aligned bases and leading dimensions (lda %d ldb %d ldc %d)", lda, ldb, ldc);
    return 10;
  }
  if (K2 <= 0 || (K2 % 8) || A2 == nullptr || B2 == nullptr || (lda2 % 8) || (ldb2 % 8) ||
      (reinterpret_cast<uintptr_t>(A2) & 15) || (reinterpret_cast<uintptr_t>(B2) & 15)) {
    set_error("gemm_ext: the second pair needs K2 %% 8 == 0 and 16-byte aligned operands (K2 %d lda2 %d ldb2 %d)", K2,
              lda2, ldb2);
    return 10;
  }
  if (out_fp32 && !(flags & GEMM_RESIDUAL)) {
    set_error("gemm_ext: fp32 outputs may split K, which the second pair does not support");
    return 10;
  }
  if (bn == 0) {
    const int sms = num_sms();
    const int tiles256 = ((M + 127) / 128) * ((N + 255) / 256);
    bn = (tiles256 >= sms || N % 256 == 0) && tiles256 * 2 > sms ? 256 : 128;
  }
#define B2_GEMM_EXT_CASE(BN_, BMN_)                                                                              \
  if (bn == BN_ && b_mn == BMN_)                                                                                 \
    return launch_gemm<BN_, false, BMN_ != 0>(A, B, C, R, M, N, K, lda, ldb, ldc, flags, 0, stream, nullptr, A2, B2, \
                                              K2, lda2, ldb2);
  B2_GEMM_EXT_CASE(256, 0)
  B2_GEMM_EXT_CASE(256, 1)
  B2_GEMM_EXT_CASE(128, 0)
  B2_GEMM_EXT_CASE(128, 1)
#undef B2_GEMM_EXT_CASE
  set_error("gemm_ext: unsupported configuration bn=%d b_mn=%d", bn, b_mn);
  return 11;
}

// Test hook: descriptor strides used for MN-major operands (bytes): distance between 64-element
// chunks along M/N, distance between 8-row groups along K, and the start-address step per UMMA_K.
B2_EXPORT void b2_gemm_set_mn_desc(unsigned lbo, unsigned sbo, unsigned kstep) {
  b2::g_mn_desc.lbo = lbo;
  b2::g_mn_desc.sbo = sbo;
  b2::g_mn_desc.kstep = kstep;
}


// Tensor-parallel GEMMs with the collective inside the kernel.  mode 1: GEMM -> reduce-scatter,
// mode 2: all-gather -> GEMM.  b_mn as in b2_gemm_bf16; A is K-major.  M = world * rows_per_rank rows in
// total, rows_per_rank a multiple of 128.  Pointer arrays have `world` entries (peer pointers of the
// symmetric buffers).  epoch: the 1-based use count of this (buffer, counter) set; counters and flags
// only ever grow, nothing is reset between calls.
//   mode 1: A [M,K] local, out [rows_per_rank, N]; recv[r]: [world, rows_per_rank, N] on rank r; cnt[r]:
//           int32 [(rows_per_rank/128) * ceil(N/bn)] on rank r.
//   mode 2: A: this rank's [rows_per_rank, K] shard (ordinary memory); gathers[r]: rank r's [M, K] gather buffer
//           (mc_gather: their multicast address or null); flags[r]: int32 [M/128] arrival counters on rank r;
//           ready[r]: int32 [world] on rank r; ready_epoch: 1-based count of mode-2 calls on this context;
//           C [M, N] local output.  The gathered activations are left in gathers[rank].
B2_EXPORT int b2_gemm_bf16_comm(int mode, const void* A, const void* B, void* C, int M, int N, int K, int ldb,
                                int b_mn, int bn, void* const* recv, void* const* cnt, void* out,
                                const void* residual, void* const* gathers, void* mc_gather, void* const* flags,
                                void* const* ready, int ready_epoch, int world, int rank, int rows_per_rank,
                                int epoch, void* stream_) {
  using namespace b2;
  b2::ensure_thread_context();
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (world < 1 || world > 8 || rows_per_rank % GEMM_BM != 0 || M != world * rows_per_rank || (K % 8) || (N % 8) ||
      (mode != 1 && mode != 2) || (bn != 128 && bn != 256)) {
    set_error("gemm_comm: need world <= 8, rows_per_rank %% 128 == 0, M == world*rows_per_rank, K,N %% 8 == 0");
    return 10;
  }
  if (mode == 1 && (N % 32) != 0) {
    set_error("gemm_comm: reduce-scatter mode needs N %% 32 == 0");
    return 10;
  }
  GemmComm comm;
  memset(&comm, 0, sizeof(comm));
  for (int r = 0; r < world; ++r) {
    if (mode == 1) {
      comm.peer_recv[r] = recv[r];
      comm.peer_cnt[r] = static_cast<int*>(cnt[r]);
    } else {
      comm.peer_gather[r] = gathers[r];
      comm.peer_flags[r] = static_cast<int*>(flags[r]);
      comm.peer_ready[r] = static_cast<int*>(ready[r]);
    }
  }
  if (mode == 2) {
    comm.gather = gathers[rank];
    comm.gather_flags = static_cast<int*>(flags[rank]);
    comm.mc_gather = mc_gather;
    comm.local_src = A;
    comm.ready_epoch = ready_epoch;
    comm.pieces_per_block = (K + 255) / 256;
  }
  comm.out = out;
  comm.residual = residual;
  comm.world = world;
  comm.rank = rank;
  comm.rows_per_rank = rows_per_rank;
  comm.epoch = epoch;
  const void* Aop = mode == 2 ? comm.gather : A;
#define B2_COMM_CASE(BN_, BMN_, MODE_)                                                                   \
  if (bn == BN_ && b_mn == BMN_ && mode == MODE_)                                                        \
    return launch_gemm<BN_, false, BMN_ != 0, MODE_>(Aop, B, C, nullptr, M, N, K, K, ldb, N, 0, 0, stream, &comm);
  B2_COMM_CASE(256, 0, 1)
  B2_COMM_CASE(256, 1, 1)
  B2_COMM_CASE(128, 0, 1)
  B2_COMM_CASE(128, 1, 1)
  B2_COMM_CASE(256, 0, 2)
  B2_COMM_CASE(256, 1, 2)
  B2_COMM_CASE(128, 0, 2)
  B2_COMM_CASE(128, 1, 2)
#undef B2_COMM_CASE
  set_error("gemm_comm: unsupported configuration");
  return 11;
}
