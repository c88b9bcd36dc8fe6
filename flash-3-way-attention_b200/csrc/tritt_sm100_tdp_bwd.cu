// Triple-dot-product trittention backward on Blackwell tensor cores (tcgen05 + TMEM + TMA).
//
// Same pair-row formulation as the forward kernel.  For one query q and a tile of 128 rows
// x of a "row" key tensor X (with its value tensor Y), against 128-row slabs of the
// "column" key/value tensors Kc / Vc:
//     A [r,h] = alpha*log2(e) * Q[q,h]  * X[x_r,h]          A'[r,h] = dO[q,h] * Y[x_r,h]
//     S  = A  Kc^T          P  = exp2(S - lse2[q])          (recomputed from the saved lse)
//     dP = A' Vc^T          dS = P * (dP - Dq),  Dq = sum_h dO[q,h] O[q,h]
//     G += dS Kc            U += P Vc                        (accumulated over the slabs in TMEM)
// and per tile   dX[x_r,h] += alpha G[r,h] Q[q,h],   dY[x_r,h] += U[r,h] dO[q,h],
//                dQ[q,h]   += alpha sum_r G[r,h] X[x_r,h].
// Role 0 takes X = K2, Y = V2, Kc = K1, Vc = SiLU(V1) and yields dQ, dK2, dV2.  Role 1 swaps
// the two key axes (the score and the gated value are symmetric under the swap): X = K1,
// Y = SiLU(V1), Kc = K2, Vc = V2, and yields dK1 and dSiLU(V1).  Four GEMM-shaped products per
// (tile, slab) and role - eight in all against the six of a minimal schedule - but every
// key-side gradient is owned by rows of a tile, so the only cross-CTA reductions are one
// 128 x D block per tile and tensor, added to fp32 accumulators by TMA reduce-add.
// (The reference runs one Triton kernel per gradient, recomputing P five times:
// triple_dot_product/kernels/bwd_dq.py, bwd_dk1.py, bwd_dk2.py, bwd_dv1.py, bwd_dv2.py.)
//
// Tensor-core usage follows what the hardware rewards: 128-column slabs, so that every
// accumulation chain is 8 instructions of 128x128x16 (an instruction below N = 128 costs the same
// ~48-64 cycles), TMEM fully used
// as S | dP | G | U (4 x 128 columns at D = 128).  P and dS are written back as 16-bit into the
// first half of the S and dP column ranges and feed the G / U products from tensor memory.
//
// CTA layout (persistent, 512 threads): warp 0 TMA producer, warp 1 tcgen05.mma issuer, warps 4-11 two
// soft-max warpgroups (64 columns of every slab each; they also form the operands), warps 12-15 the
// fold warpgroup.  The slab pipeline is split in four hand-offs so that the exponentials (the MUFU
// bound part) overlap the tensor pipe although S and dP are single-buffered:
//     MMA:      U(c) S(c+1) | G(c) dP(c+1) | U(c+1) S(c+2) | ...
//     soft-max:      [S(c+1) -> P(c+1)]  [dP(c+1), P(c+1) -> dS(c+1)]
// (At head dimension 64, where tensor memory has room, P has buffers of its own and S(c+1) goes before U(c): see
// kFreeS in the kernel.)
// The fold warpgroup drains G / U of tile t (TMEM -> registers -> shared memory -> TMA reduce-add)
// while the other warps already run tile t+1.  Work item = (query, head, role); it walks the row tiles
// x <= q and, inside, the column slabs c <= q.
// On request (TRITT_FLAG_BWD_CTA_PAIRS) the same kernel runs as clusters of two CTAs: each CTA keeps its own query,
// operand tiles, soft-max and fold, the even CTA issues every product for both (cta_group::2, 256 rows), the column
// tiles are split between the two shared memories, and hand-offs to the issuing thread cross the pair.
#include "tritt_sm100_tdp.cuh"

#include <type_traits>

namespace tritt {
namespace {
using namespace sm100;

constexpr int kBC = 128;  // key columns per slab

template <int D> struct BwdCfg {
  static constexpr int kTileA = 128 * D * 2;   // one 128-row operand / key / value tile
  // ring of column tiles Kc(c), Vc(c), Kc(c+1), Vc(c+1), ...: two slabs deep at head dimension 128 (all the shared
  // memory there is), four at 64
  static constexpr int kStages = D == 64 ? 8 : 4;
  static constexpr int kOffA = 0;              // A  (row-key pre-product)
  static constexpr int kOffA2 = kTileA;        // A' (row-value pre-product)
  static constexpr int kOffRing = 2 * kTileA;
  static constexpr int kOffStage = kOffRing + kStages * kTileA;  // fold staging: 4 warps x 2 slots x 4 KiB
  static constexpr int kStageBytes = 4 * 2 * 4096;
  static constexpr int kOffDq = kOffStage + kStageBytes;         // [D] fp32: dQ column sums of the current query
  static constexpr int kOffVec = kOffDq + D * 4;                 // [2 parities][2][D] fp32: Q[q], dO[q]
  static constexpr int kOffMisc = kOffVec + 4 * D * 4;           // [4] fp32: Dq partials
  static constexpr int kOffBars = kOffMisc + 16;                 // barriers (no static shared memory is used, so
  static constexpr int kSmem = kOffBars + 288;                   //  the dynamic region starts 1024-byte aligned)
  static constexpr int kTmemS = 0, kTmemDP = 128, kTmemG = 256, kTmemU = 256 + D;
  static constexpr int kTmemP = 384;   // head dimension 64 only: two buffers of 64 columns for P (by slab parity)
};

// NSW soft-max warpgroups (2 or 4) + 4 service warps (TMA, MMA, 2 idle) + the fold warpgroup
template <int NSW> struct BwdThreads {
  static constexpr int kSoftmax = 128 * NSW;
  static constexpr int kTotal = 128 + kSoftmax + 128;
  static constexpr int kFoldWarp0 = 4 + 4 * NSW;  // first warp of the fold warpgroup (a multiple of 4)
};

struct BwdParams {
  const void *q, *o, *d_o;
  const void* x[2];  // row key tensor per role (raw pointers, for the dQ fold)
  const float* lse;
  void* dq;
  int T, BN, nq, q_mod, q_rem, causal;
  int k1w, k2w, kkl, kkr;  // windows of the causal mask (T or more = unbounded)
  float alpha;
  int* status;
};

struct BwdBarriers {
  uint64_t ring_full[8], ring_empty[8];
  uint64_t xy_full, ax_ready, ay_ready, a_free;  // A (score operand) and A' (dP operand) become ready separately
  uint64_t s_ready, dp_ready, ds_ready;              // slab hand-offs
  // P in two column halves, a pair of barriers per slab parity: with the early score product the soft-max warps
  // can hand over P(c+1) before the issuing warp has looked at P(c) (it may be waiting for the fold at a tile's
  // first slab), and a barrier that is two phases ahead of its waiter reads as not ready for ever
  uint64_t p_ready[2][2];
  uint64_t s_free;                                   // head dimension 64: the soft-max warps hold a slab's scores in registers
  uint64_t gu_done, u_free, g_free;               // tile hand-offs with the fold warpgroup (U is drained first)
  uint64_t sm_sync, fold_sync;
  uint64_t vec_free[2];                           // fold warpgroup -> soft-max: a copy of Q[q] / dO[q] is no longer read
  uint32_t tmem_base;
  int abort_flag;
};


// fp16 only: the recomputed probabilities of a query that attends n pairs are ~1/n, which for late rows lies below
// fp16's normal range (6e-5; 1/n = 2e-7 at q = 2048).  P and dS are therefore formed times 2^e, e = min(10, log2 of
// the attended pairs' count bound), and the fold warpgroup divides it out of G and U.  2^10 keeps a probability of 1
// times a dP - Dq of up to 64 finite.  bf16 has fp32's exponent range and needs none of this (e = 0).
template <typename T16>
__device__ __forceinline__ int prob_shift(int q, int causal, int T, int k1w, int k2w) {
  if constexpr (std::is_same<T16, __half>::value) {
    const int n1 = causal ? min(q, k1w) + 1 : T, n2 = causal ? min(q, k2w) + 1 : T;
    const int e = (31 - __clz(n1)) + (31 - __clz(n2));
    return min(10, e);
  }
  return 0;
}

// The four 64-row-box maps of the key / value tensors are used by the CTA-pair variant only.
struct BwdHalfMaps {
  CUtensorMap k1, k2, sv1, v2;
};

// PAIR: the kernel runs as clusters of two CTAs that take two queries of one (head, role) in lockstep: CTA `rank`
// owns query 2 i + rank with its own operand tiles, soft-max and fold, and the even CTA issues every product for both
// with cta_group::2 (M = 256: 128 pair rows per CTA).  The column tiles are then shared: each CTA holds half of a
// tile's N extent per product (64 of its 128 rows for S / dP, 64 of its D columns for G / U), so the tensor cores
// read 128 KB of shared memory per slab and SM instead of 192 KB.
template <int D, typename T16, int NSW, bool PAIR>
__global__ void __launch_bounds__(BwdThreads<NSW>::kTotal, 1)
tdp_bwd_kernel(const __grid_constant__ CUtensorMap tmK1, const __grid_constant__ CUtensorMap tmK2,
               const __grid_constant__ CUtensorMap tmSV1, const __grid_constant__ CUtensorMap tmV2,
               const __grid_constant__ CUtensorMap tmDK1, const __grid_constant__ CUtensorMap tmDK2,
               const __grid_constant__ CUtensorMap tmDSV1, const __grid_constant__ CUtensorMap tmDV2,
               const __grid_constant__ BwdHalfMaps half, BwdParams p) {
  static_assert(!PAIR || D == 128, "the CTA-pair tile layout is written for head dimension 128");
  using Cfg = BwdCfg<D>;
  constexpr int NS = Cfg::kStages;
  constexpr int KH = D / 64;
  constexpr int kNumSoftmax = BwdThreads<NSW>::kSoftmax;
  constexpr int kFoldWarp0 = BwdThreads<NSW>::kFoldWarp0;
  constexpr int CW = kBC / NSW;  // slab columns owned by one soft-max warpgroup
  // Head dimension 64 leaves 128 columns of tensor memory free: P then goes to a buffer of its own (two, by slab
  // parity) instead of over the scores, and the next slab's score product is issued as soon as the soft-max warps hold
  // this slab's scores in registers (`s_free`) instead of after U has consumed P: the loop S -> P -> U -> S is open.
  // (U(c) is issued before S(c+2), and the pipe runs in order, so P(c) has been consumed when P(c+2) is written.)
  constexpr bool kFreeS = D == 64 && !PAIR;
  extern __shared__ __align__(1024) uint8_t smem[];
  static_assert(sizeof(BwdBarriers) <= 288, "barrier block too large");
  BwdBarriers& bars = *reinterpret_cast<BwdBarriers*>(smem + Cfg::kOffBars);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (smem_u32(smem) & 1023u) {
    // swizzled tiles need 1024-byte alignment; uniform over the CTA, so every thread leaves here
    if (tid == 0 && p.status) atomicOr(p.status, 8);
    return;
  }

  if (tid == 0) {
    bars.abort_flag = 0;
    for (int i = 0; i < NS; ++i) {
      mbar_init(&bars.ring_full[i], 1);
      mbar_init(&bars.ring_empty[i], 1);
    }
    mbar_init(&bars.xy_full, 1);
    // (hand-offs to the issuing thread: every thread arrives, or, in a pair, one lane per warp of both CTAs on the
    //  even CTA's barrier)
    constexpr uint32_t kToMmaSm = PAIR ? 2 * kNumSoftmax / 32 : kNumSoftmax, kToMmaFold = PAIR ? 2 * 4 : 128;
    mbar_init(&bars.ax_ready, kToMmaSm);
    mbar_init(&bars.ay_ready, kToMmaSm);
    mbar_init(&bars.a_free, 1);   // a commit behind the tile's last score / dP products
    mbar_init(&bars.s_ready, 1);
    mbar_init(&bars.dp_ready, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&bars.p_ready[i >> 1][i & 1], kToMmaSm);
    mbar_init(&bars.ds_ready, kToMmaSm);
    mbar_init(&bars.s_free, kToMmaSm);
    mbar_init(&bars.gu_done, 1);
    mbar_init(&bars.u_free, kToMmaFold);
    mbar_init(&bars.g_free, kToMmaFold);
    mbar_init(&bars.sm_sync, kNumSoftmax);
    mbar_init(&bars.fold_sync, 128);
    mbar_init(&bars.vec_free[0], 128);
    mbar_init(&bars.vec_free[1], 128);
    fence_barrier_init();
  }
  if (warp == 0) {
    if constexpr (PAIR) {
      tmem_alloc_pair(&bars.tmem_base, 512);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&bars.tmem_base, 512);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();  // the other CTA's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem = bars.tmem_base;
  volatile int* abort_flag = &bars.abort_flag;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  // work is dealt to CTAs, or to CTA pairs
  const long unit = PAIR ? (long)(blockIdx.x >> 1) : (long)blockIdx.x;
  const long n_units = PAIR ? (long)(gridDim.x >> 1) : (long)gridDim.x;
  // hand-off to the issuing thread (after the caller's fences)
  auto to_mma = [&](uint64_t* bar) {
    if constexpr (PAIR) {
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mbar_in_cta(bar, 0));
    } else {
      mbar_arrive(bar);
    }
  };

  const int T = p.T;
  // items: (query, head, role), or in a pair (two queries, head, role)
  const long n_items = (long)(PAIR ? p.nq / 2 : p.nq) * p.BN * 2;

  // item -> (role, head, query); late (expensive) queries first.  Items 2r and 2r + 1 are the two roles of one (head,
  // query); which of them is which alternates with r in blocks of half the grid, so that the items of one CTA
  // (gridDim.x apart) alternate between the roles: role-0 tiles cost more (their fold also forms dQ), and a CTA
  // that only ever saw one role would finish 6 % later than its neighbour.
  // In a pair `q` is this CTA's query and `qr` the later one of the two, whose tile ranges both CTAs walk (the
  // earlier query masks what lies beyond it).
  auto decode = [&](long item, int& role, int& bh, int& q, int& qr) {
    const long r = item >> 1;
    role = (int)((item ^ (r / ((n_units + 1) >> 1))) & 1);
    bh = (int)(r % p.BN);
    if constexpr (PAIR) {
      const int i_hi = p.nq - 1 - 2 * (int)(r / p.BN);
      q = p.q_rem + (i_hi - 1 + (int)rank) * p.q_mod;
      qr = p.q_rem + i_hi * p.q_mod;
    } else {
      q = p.q_rem + (p.nq - 1 - (int)(r / p.BN)) * p.q_mod;
      qr = q;
    }
  };
  // Causal mask j <= q <= j + k1w, k <= q <= k + k2w, k - kkl <= j <= k + kkr, seen from a role's rows x and
  // columns c (role 0: x = k, c = j; role 1: x = j, c = k):  x in [q - xw, q],  c in [q - cw, q],  c in [x - below, x + above].
  struct Win { int xw, cw, below, above; };
  auto role_win = [&](int role) {
    return role == 0 ? Win{p.k2w, p.k1w, p.kkl, p.kkr} : Win{p.k1w, p.k2w, p.kkr, p.kkl};
  };
  // row tiles of a query: rows [max(0, q - xw, q - cw - above), q]  (rows below the third bound see no column);
  // column slabs of row tile xt: [max(0, q - cw, x_first - below), min(q, x_last + above)], never empty
  auto x_range = [&](int q, const Win& w, int& xt0, int& nxt) {
    if (!p.causal) {
      xt0 = 0;
      nxt = (T + 127) / 128;
      return;
    }
    const int xlo = max(0, max(q - w.xw, q - w.cw - w.above));
    xt0 = xlo / 128;
    nxt = q / 128 - xt0 + 1;
  };
  auto c_range = [&](int q, const Win& w, int xt, int& c0, int& ncs) {
    if (!p.causal) {
      c0 = 0;
      ncs = (T + kBC - 1) / kBC;
      return;
    }
    const int xlo = max(0, max(q - w.xw, q - w.cw - w.above));
    const int xa = max(xt * 128, xlo), xb = min(xt * 128 + 127, q);
    const int ca = max(0, max(q - w.cw, xa - w.below)), cb = min(q, xb + w.above);
    c0 = ca / kBC;
    ncs = cb / kBC - c0 + 1;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // (like the MMA warp: the whole warp walks the schedule converged, one elected lane issues the copies)
    {
      const bool leader = elect_one();
      if (leader) {
        const CUtensorMap* maps[8] = {&tmK1, &tmK2, &tmSV1, &tmV2, &tmDK1, &tmDK2, &tmDSV1, &tmDV2};
        for (int i = 0; i < 8; ++i) tma_prefetch_desc(maps[i]);
      }
      uint32_t xt_count = 0, pos = 0;
      bool alive = true;
      // One column tile (128 rows of Kc or Vc) into the next ring stage.  In a pair each CTA fetches what its half
      // of the products reads: rows [64 rank, 64 rank + 64) of the tile (both 64-column halves, 8 KB each: the B
      // operand of S / dP) and columns [64 rank, 64 rank + 64) of all 128 rows (16 KB: the B operand of G / U); the
      // bytes of both CTAs are counted on the even CTA's barrier, where the issuing thread waits.
      auto load_stage = [&](const CUtensorMap* tm, const CUtensorMap* tm_half, int row0, int bh) -> bool {
        const int st = pos % NS;
        if (!__all_sync(0xffffffffu, mbar_wait_x<PAIR>(&bars.ring_empty[st], ((pos / NS) & 1) ^ 1, abort_flag)))
          return false;
        uint8_t* dst = smem + Cfg::kOffRing + st * Cfg::kTileA;
        if (leader) {
          if constexpr (PAIR) {
            if (rank == 0) mbar_arrive_expect_tx(&bars.ring_full[st], 2 * Cfg::kTileA);
            const uint32_t full0 = mbar_in_cta(&bars.ring_full[st], 0);
            tma_load_3d_pair(dst, tm_half, full0, 0, row0 + 64 * (int)rank, bh);
            tma_load_3d_pair(dst + 8192, tm_half, full0, 64, row0 + 64 * (int)rank, bh);
            tma_load_3d_pair(dst + 16384, tm, full0, 64 * (int)rank, row0, bh);
          } else {
            mbar_arrive_expect_tx(&bars.ring_full[st], Cfg::kTileA);
            for (int hh = 0; hh < KH; ++hh) tma_load_3d(dst + hh * 16384, tm, &bars.ring_full[st], hh * 64, row0, bh);
          }
        }
        ++pos;
        return true;
      };
      for (long item = unit; item < n_items && alive; item += n_units) {
        int role, bh, q, qr, xt0, nxt;
        decode(item, role, bh, q, qr);
        const Win win = role_win(role);
        x_range(qr, win, xt0, nxt);
        // role 0: columns K1 / SiLU(V1), rows K2 / V2;   role 1: columns K2 / V2, rows K1 / SiLU(V1)
        const CUtensorMap* tmKc = role == 0 ? &tmK1 : &tmK2;
        const CUtensorMap* tmVc = role == 0 ? &tmSV1 : &tmV2;
        const CUtensorMap* tmKcH = role == 0 ? &half.k1 : &half.k2;
        const CUtensorMap* tmVcH = role == 0 ? &half.sv1 : &half.v2;
        const CUtensorMap* tmX = role == 0 ? &tmK2 : &tmK1;
        const CUtensorMap* tmY = role == 0 ? &tmV2 : &tmSV1;
        for (int xt = xt0; xt < xt0 + nxt && alive; ++xt, ++xt_count) {
          int c0, ncs;
          c_range(qr, win, xt, c0, ncs);
          // the tile's first key / value slab does not depend on the operand buffers: fetch it before waiting for them
          alive = load_stage(tmKc, tmKcH, c0 * kBC, bh);
          if (alive) alive = load_stage(tmVc, tmVcH, c0 * kBC, bh);
          if (!alive || !__all_sync(0xffffffffu, mbar_wait_x<PAIR>(&bars.a_free, (xt_count & 1) ^ 1, abort_flag))) {
            alive = false;
            break;
          }
          if (leader) {
            mbar_arrive_expect_tx(&bars.xy_full, 2 * Cfg::kTileA);
            for (int hh = 0; hh < KH; ++hh) {
              tma_load_3d(smem + Cfg::kOffA + hh * 16384, tmX, &bars.xy_full, hh * 64, xt * 128, bh);
              tma_load_3d(smem + Cfg::kOffA2 + hh * 16384, tmY, &bars.xy_full, hh * 64, xt * 128, bh);
            }
          }
          for (int c = c0 + 1; c < c0 + ncs && alive; ++c) {
            alive = load_stage(tmKc, tmKcH, c * kBC, bh);
            if (alive) alive = load_stage(tmVc, tmVcH, c * kBC, bh);
          }
        }
      }
      if (!alive && (!PAIR || rank == 0)) {
        const uint32_t first = pos > (uint32_t)NS ? pos - NS : 0;
        for (uint32_t q2 = first; q2 < pos; ++q2) {
          const long long t0 = clock64();
          while (!mbar_try_wait(&bars.ring_full[q2 % NS], (q2 / NS) & 1) && clock64() - t0 < kWaitTicks / 8) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp walks the schedule in step and one elected lane issues: with converged control flow the
    // descriptor arithmetic stays on the uniform datapath, where a lone thread needs a register-to-uniform move
    // per operand and loses its issue slots to the busy warps of its scheduler (a stand-alone loop of these chains
    // under issue pressure: 15.3 k cycles per 32 instructions from one thread, 3.9 k from a converged warp).
    if (rank == 0) {
      const bool leader = elect_one();
      constexpr int kFmt = std::is_same<T16, __nv_bfloat16>::value ? 1 : 0;
      constexpr int kM = PAIR ? 256 : 128;   // rows of one instruction (both CTAs of a pair)
      constexpr uint32_t idesc_s = make_idesc_f16(kM, kBC, kFmt, false, false);
      constexpr uint32_t idesc_g = make_idesc_f16(kM, D, kFmt, false, true);
      // descriptor low words; per instruction only a constant (in 16-byte units) is added
      constexpr uint32_t kHi = desc_hi(1024);
      constexpr uint32_t kTile16 = Cfg::kTileA >> 4;
      const uint32_t aLo = desc_lo(smem_u32(smem + Cfg::kOffA), 16), a2Lo = desc_lo(smem_u32(smem + Cfg::kOffA2), 16);
      const uint32_t ringK = desc_lo(smem_u32(smem + Cfg::kOffRing), 16);      // K-major view of a stage
      // row-major (MN-major) view; in a pair the stage's second half: this CTA's 64 columns of all 128 rows
      const uint32_t ringMN = desc_lo(smem_u32(smem + Cfg::kOffRing + (PAIR ? 16384 : 0)), 16384);
      // K-major view: 64-column blocks of a tile are 16 KB apart, of a pair's 64-row half 8 KB
      constexpr uint32_t kBlkK = (PAIR ? 8192 : 16384) >> 4;
      auto commit = [&](uint64_t* bar) {
        if (!leader) return;
        if constexpr (PAIR) mma_commit_pair(bar); else mma_commit(bar);
      };
      auto mma_ss_any = [&](uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t acc) {
        if (!leader) return;
        if constexpr (PAIR) mma_ss_lo_pair(d, a_lo, b_lo, kHi, idesc, acc); else mma_ss_lo(d, a_lo, b_lo, kHi, idesc, acc);
      };
      auto mma_ts_any = [&](uint32_t d, uint32_t a_t, uint32_t b_lo, uint32_t idesc, uint32_t acc) {
        if (!leader) return;
        if constexpr (PAIR) mma_ts_lo_pair(d, a_t, b_lo, kHi, idesc, acc); else mma_ts_lo(d, a_t, b_lo, kHi, idesc, acc);
      };
      // (every lane waits; the vote keeps the warp converged whatever a lane's wait returned)
      auto wait_all = [&](uint64_t* bar, uint32_t parity) {
        return __all_sync(0xffffffffu, mbar_wait_x<PAIR>(bar, parity, abort_flag));
      };
      uint32_t xt_count = 0, base = 0, n = 0;
      bool alive = true;
      auto wait_full = [&](uint32_t pos) {
        return wait_all(&bars.ring_full[pos % NS], (pos / NS) & 1);
      };
      // One 8-instruction accumulation chain each (D = 128): S = A Kc^T, dP = A' Vc^T (operands in shared
      // memory, key/value tile K-major), U (+)= P Vc, G (+)= dS Kc (P / dS from tensor memory, the tile row-major).
      auto issue_s = [&](uint32_t pos) -> bool {
        if (!wait_full(pos)) return false;
        const uint32_t bLo = ringK + (pos % NS) * kTile16;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t kk = (k >> 2) * (16384 >> 4) + (k & 3) * 2, kb = (k >> 2) * kBlkK + (k & 3) * 2;
          mma_ss_any(tmem + Cfg::kTmemS, aLo + kk, bLo + kb, idesc_s, k > 0);
        }
        commit(&bars.s_ready);
        return true;
      };
      auto issue_dp = [&](uint32_t pos) -> bool {
        if (!wait_full(pos)) return false;
        const uint32_t bLo = ringK + (pos % NS) * kTile16;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t kk = (k >> 2) * (16384 >> 4) + (k & 3) * 2, kb = (k >> 2) * kBlkK + (k & 3) * 2;
          mma_ss_any(tmem + Cfg::kTmemDP, a2Lo + kk, bLo + kb, idesc_s, k > 0);
        }
        commit(&bars.dp_ready);
        return true;
      };
      // soft-max warpgroup g packed its CW columns of P into S[CW*g, CW*g + CW/2) and of dS into dP[CW*g, ...)
      constexpr int KPW = CW / 16;  // 16-deep MMA steps per warpgroup
      // U is issued in two halves: the k-steps fed by the first half of every warpgroup's columns as soon as
      // that half of P is there, the rest when the second half arrives (same accumulation chain).
      auto issue_u_half = [&](uint32_t pos, uint32_t acc, int half, uint32_t pbuf) {
        const uint32_t st = pos % NS;
        bool first = half == 0;
#pragma unroll
        for (int k = 0; k < kBC / 16; ++k) {
          if (((k % KPW) >= KPW / 2) != (half == 1)) continue;
          const uint32_t a = kFreeS ? tmem + Cfg::kTmemP + pbuf * 64 + k * 8
                                    : tmem + Cfg::kTmemS + (k / KPW) * CW + (k % KPW) * 8;
          mma_ts_any(tmem + Cfg::kTmemU, a, ringMN + st * kTile16 + k * (2048 >> 4), idesc_g, first ? acc : 1u);
          first = false;
        }
        if (half == 1) commit(&bars.ring_empty[st]);
      };
      auto issue_g = [&](uint32_t pos, uint32_t acc) {
        const uint32_t st = pos % NS;
#pragma unroll
        for (int k = 0; k < kBC / 16; ++k) {
          const uint32_t a = tmem + Cfg::kTmemDP + (k / KPW) * CW + (k % KPW) * 8;
          mma_ts_any(tmem + Cfg::kTmemG, a, ringMN + st * kTile16 + k * (2048 >> 4), idesc_g, k > 0 ? 1u : acc);
        }
        commit(&bars.ring_empty[st]);
      };

      for (long item = unit; item < n_items && alive; item += n_units) {
        int role, bh, q, qr, xt0, nxt;
        decode(item, role, bh, q, qr);
        const Win win = role_win(role);
        x_range(qr, win, xt0, nxt);
        for (int xt = xt0; xt < xt0 + nxt && alive; ++xt, ++xt_count) {
          int c0, ncs;
          c_range(qr, win, xt, c0, ncs);
          // the first score product starts while the soft-max warps still form the dP operand
          if (!wait_all(&bars.ax_ready, xt_count & 1)) { alive = false; break; }
          tc_fence_after();
          if (!issue_s(base)) { alive = false; break; }
          if (!wait_all(&bars.ay_ready, xt_count & 1)) { alive = false; break; }
          tc_fence_after();
          if (!issue_dp(base + 1)) { alive = false; break; }
          // Once the tile's last S and dP products have run, its operand tiles may be reloaded: the commit lets the
          // producer fetch the next tile's rows a slab before the soft-max warps are done with this one.
          if (ncs == 1) commit(&bars.a_free);
          for (int c = 0; c < ncs && alive; ++c, ++n) {
            const bool more = c + 1 < ncs;
            if constexpr (kFreeS) {
              if (!wait_all(&bars.s_free, n & 1)) { alive = false; break; }
              tc_fence_after();
              if (more && !issue_s(base + 2 * (c + 1))) { alive = false; break; }
            }
            if (!wait_all(&bars.p_ready[n & 1][0], (n >> 1) & 1)) { alive = false; break; }
            if (c == 0) {
              // the fold warpgroup must have drained the previous tile's U
              if (!wait_all(&bars.u_free, (xt_count & 1) ^ 1)) { alive = false; break; }
            }
            tc_fence_after();
            issue_u_half(base + 2 * c + 1, c > 0, 0, n & 1);
            if (!wait_all(&bars.p_ready[n & 1][1], (n >> 1) & 1)) { alive = false; break; }
            tc_fence_after();
            issue_u_half(base + 2 * c + 1, c > 0, 1, n & 1);
            if constexpr (!kFreeS) {
              if (more && !issue_s(base + 2 * (c + 1))) { alive = false; break; }
            }
            if (!wait_all(&bars.ds_ready, n & 1)) { alive = false; break; }
            if (c == 0) {
              // ... and the previous tile's G
              if (!wait_all(&bars.g_free, (xt_count & 1) ^ 1)) { alive = false; break; }
            }
            tc_fence_after();
            issue_g(base + 2 * c, c > 0);
            if (more && !issue_dp(base + 2 * (c + 1) + 1)) { alive = false; break; }
            if (c + 2 == ncs) commit(&bars.a_free);   // that was the tile's last dP (its last S went before it)
          }
          if (alive) commit(&bars.gu_done);
          base += 2 * ncs;
        }
      }
    }
  } else if (warp >= 4 && warp < kFoldWarp0) {
    // ------------------------------------------------------------------ soft-max warpgroups
    const int wg = (warp - 4) >> 2;            // owns columns [CW*wg, CW*wg + CW) of every slab
    const int wq = warp & 3;
    const int row = wq * 32 + lane;
    const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
    float* vec = (float*)(smem + Cfg::kOffVec);
    float* misc = (float*)(smem + Cfg::kOffMisc);
    uint32_t xt_count = 0, n = 0, sync_phase = 0, item_count = 0;
    bool alive = true;
    auto sm_sync = [&]() -> bool {
      mbar_arrive(&bars.sm_sync);
      const bool ok = mbar_wait_x<PAIR>(&bars.sm_sync, sync_phase & 1, abort_flag);
      ++sync_phase;
      return __all_sync(0xffffffffu, ok);
    };

    for (long item = unit; item < n_items && alive; item += n_units, ++item_count) {
      int role, bh, q, qr, xt0, nxt;
      decode(item, role, bh, q, qr);
      const Win win = role_win(role);
      x_range(qr, win, xt0, nxt);
      const size_t hb = (size_t)bh * T * D;
      float* qv = vec + (item_count & 1) * 2 * D;  // Q[q, :] (double-buffered by item: the fold warpgroup of the
      float* dov = qv + D;                         // dO[q, :]  previous item may still be reading its copy)
      if (!sm_sync()) { alive = false; break; }    // previous item's readers of misc are done
      // the fold warpgroup can lag two items behind: wait until it has stopped reading this copy of the vectors
      alive = __all_sync(0xffffffffu,
                         mbar_wait_x<PAIR>(&bars.vec_free[item_count & 1], ((item_count >> 1) & 1) ^ 1, abort_flag));
      if (!alive) break;
      const float scale2 = p.alpha * kLog2e;
      if (wg == 0) {
        float dq_part = 0.f;
        if (row < D) {
          const float qf = to_f(((const T16*)p.q)[hb + (size_t)q * D + row]);
          const float dof = to_f(((const T16*)p.d_o)[hb + (size_t)q * D + row]);
          qv[row] = qf * scale2;   // (pre-scaled: the score operand is scale2 * Q[q] (.) X)
          dov[row] = dof;
          dq_part = dof * to_f(((const T16*)p.o)[hb + (size_t)q * D + row]);
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) dq_part += __shfl_xor_sync(0xffffffffu, dq_part, o);
        if (lane == 0) misc[wq] = dq_part;
      }
      if (!sm_sync()) { alive = false; break; }
      const float Dq = misc[0] + misc[1] + misc[2] + misc[3];
      // (minus the fp16 range shift: P below is the probability times 2^e)
      const float lse2 = p.lse[(size_t)bh * T + q] * kLog2e - (float)prob_shift<T16>(q, p.causal, T, p.k1w, p.k2w);
      const float2 nlse = make_float2(-lse2, -lse2), ndq = make_float2(-Dq, -Dq);

      for (int xt = xt0; xt < xt0 + nxt && alive; ++xt, ++xt_count) {
        int c0, ncs;
        c_range(qr, win, xt, c0, ncs);
        // ---- operand formation (in place): A = scale2*Q[q] (.) X tile,  A' = dO[q] (.) Y tile
        alive = __all_sync(0xffffffffu, mbar_wait_x<PAIR>(&bars.xy_full, xt_count & 1, abort_flag));
        if (!alive) break;
        // (each warpgroup takes half of the columns; the eight Q / dO values of a 16-byte chunk are the same for all rows)
#pragma unroll
        for (int ci = 0; ci < D / 8 / NSW; ++ci) {
          const int cc = wg * (D / 8 / NSW) + ci;
          const uint32_t off = (cc >> 3) * 16384 + swz128(row, cc & 7);
          const uint4 xv = *reinterpret_cast<const uint4*>(smem + Cfg::kOffA + off);
          const float4 q0 = *reinterpret_cast<const float4*>(qv + cc * 8), q1 = *reinterpret_cast<const float4*>(qv + cc * 8 + 4);
          const float2 qf[4] = {make_float2(q0.x, q0.y), make_float2(q0.z, q0.w), make_float2(q1.x, q1.y),
                                make_float2(q1.z, q1.w)};
          uint32_t wx[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 a2 = __fmul2_rn(unpack2<T16>(wx[e]), qf[e]);
            wx[e] = pack2<T16>(a2.x, a2.y);
          }
          *reinterpret_cast<uint4*>(smem + Cfg::kOffA + off) = make_uint4(wx[0], wx[1], wx[2], wx[3]);
        }
        fence_async_smem();
        to_mma(&bars.ax_ready);
#pragma unroll
        for (int ci = 0; ci < D / 8 / NSW; ++ci) {
          const int cc = wg * (D / 8 / NSW) + ci;
          const uint32_t off = (cc >> 3) * 16384 + swz128(row, cc & 7);
          const uint4 yv = *reinterpret_cast<const uint4*>(smem + Cfg::kOffA2 + off);
          const float4 d0 = *reinterpret_cast<const float4*>(dov + cc * 8), d1 = *reinterpret_cast<const float4*>(dov + cc * 8 + 4);
          const float2 df[4] = {make_float2(d0.x, d0.y), make_float2(d0.z, d0.w), make_float2(d1.x, d1.y),
                                make_float2(d1.z, d1.w)};
          uint32_t wy[4] = {yv.x, yv.y, yv.z, yv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 a2 = __fmul2_rn(unpack2<T16>(wy[e]), df[e]);
            wy[e] = pack2<T16>(a2.x, a2.y);
          }
          *reinterpret_cast<uint4*>(smem + Cfg::kOffA2 + off) = make_uint4(wy[0], wy[1], wy[2], wy[3]);
        }
        fence_async_smem();
        to_mma(&bars.ay_ready);

        // columns this row sees: [c_lo, c_hi] (empty for a row outside its own range: its P is zero)
        const int x_r = xt * 128 + row;
        int c_lo = 0, c_hi = x_r < T ? T - 1 : -1;
        if (p.causal) {
          const bool row_valid = x_r <= q && q - x_r <= win.xw;
          c_lo = max(q - win.cw, x_r - win.below);
          c_hi = row_valid ? min(q, x_r + win.above) : c_lo - 1;
        }
        const uint32_t tS = tmem + lane_base + Cfg::kTmemS + wg * CW;
        const uint32_t tDP = tmem + lane_base + Cfg::kTmemDP + wg * CW;

        for (int c = 0; c < ncs; ++c, ++n) {
          const int lo = c_lo - (c0 + c) * kBC - wg * CW, hi = c_hi - (c0 + c) * kBC - wg * CW;
          uint32_t pk[CW / 2];
          // ---- S -> P
          alive = __all_sync(0xffffffffu, mbar_wait_x<PAIR>(&bars.s_ready, n & 1, abort_flag));
          if (!alive) break;
          tc_fence_after();
          static_assert(CW == 64, "the two-half hand-off of P is written for two soft-max warpgroups");
          // (the read of the second half is in flight while the first half is worked on)
          uint32_t sh[2][32];
          tmem_ld32(tS, sh[0]);
          tmem_wait_ld();
          tmem_ld32(tS + 32, sh[1]);
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            if (hf == 1) {
              tmem_wait_ld();
              if constexpr (kFreeS) {
                // both halves of the scores are in registers: the next slab's product may overwrite them
                tc_fence_before();
                to_mma(&bars.s_free);
              }
            }
            const uint32_t(&s)[32] = sh[hf];
            const int l2 = lo - hf * 32, h2 = hi - hf * 32;
            if (l2 <= 0 && h2 >= 31) {
              // (packed fp32 pairs: one subtraction per two scores)
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const float2 x = __fadd2_rn(make_float2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), nlse);
                pk[hf * 16 + (i >> 1)] = pack2<T16>(exp2f(x.x), exp2f(x.y));
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const float p0 = (i >= l2 && i <= h2) ? exp2f(__uint_as_float(s[i]) - lse2) : 0.f;
                const float p1 = (i + 1 >= l2 && i + 1 <= h2) ? exp2f(__uint_as_float(s[i + 1]) - lse2) : 0.f;
                pk[hf * 16 + (i >> 1)] = pack2<T16>(p0, p1);
              }
            }
            // P half -> S columns this thread has already read; hand it to the MMA warp right away
            tmem_st16(kFreeS ? tmem + lane_base + Cfg::kTmemP + (n & 1) * 64 + wg * 32 + hf * 16 : tS + hf * 16,
                      *reinterpret_cast<uint32_t(*)[16]>(&pk[hf * 16]));
            tmem_wait_st();
            tc_fence_before();
            to_mma(&bars.p_ready[n & 1][hf]);
          }
          // ---- dP, P -> dS
          alive = __all_sync(0xffffffffu, mbar_wait_x<PAIR>(&bars.dp_ready, n & 1, abort_flag));
          if (!alive) break;
          tc_fence_after();
          uint32_t dk[CW / 2];
          {
            uint32_t dp[CW];
#pragma unroll
            for (int sc = 0; sc < CW / 32; ++sc) tmem_ld32(tDP + sc * 32, *reinterpret_cast<uint32_t(*)[32]>(&dp[sc * 32]));
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < CW; i += 2) {
              const float2 d = __fadd2_rn(make_float2(__uint_as_float(dp[i]), __uint_as_float(dp[i + 1])), ndq);
              const float2 ds = __fmul2_rn(unpack2<T16>(pk[i >> 1]), d);
              dk[i >> 1] = pack2<T16>(ds.x, ds.y);
            }
          }
          tmem_st(tDP, dk);  // dS -> first half of this warpgroup's dP columns
          tmem_wait_st();
          tc_fence_before();
          to_mma(&bars.ds_ready);
        }
        if (!alive) break;
      }
    }
  } else if (warp >= kFoldWarp0) {
    // ------------------------------------------------------------------ fold warpgroup
    // Drains G / U of a finished tile: 32-column pieces -> registers -> scaled by Q[q] / dO[q] -> shared memory
    // (128-byte swizzle) -> TMA reduce-add into the fp32 accumulators; for role 0 also dQ[q] += sum_r G X.
    const int wq = warp & 3;
    const int row = wq * 32 + lane;
    const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
    uint8_t* slots = smem + Cfg::kOffStage + wq * 8192;  // two 4 KiB slots of this warp
    float* dq_acc = (float*)(smem + Cfg::kOffDq);
    float* vec = (float*)(smem + Cfg::kOffVec);
    uint32_t xt_count = 0, sync_phase = 0, item_count = 0, round = 0;
    bool alive = true;
    auto fold_sync = [&]() -> bool {
      mbar_arrive(&bars.fold_sync);
      const bool ok = mbar_wait_x<PAIR>(&bars.fold_sync, sync_phase & 1, abort_flag);
      ++sync_phase;
      return __all_sync(0xffffffffu, ok);
    };
    for (long item = unit; item < n_items && alive; item += n_units, ++item_count) {
      int role, bh, q, qr, xt0, nxt;
      decode(item, role, bh, q, qr);
      const Win win = role_win(role);
      x_range(qr, win, xt0, nxt);
      const size_t hb = (size_t)bh * T * D;
      const T16* Xg = (const T16*)p.x[role] + hb;
      const CUtensorMap* tmDX = role == 0 ? &tmDK2 : &tmDK1;
      const CUtensorMap* tmDY = role == 0 ? &tmDV2 : &tmDSV1;
      const float* qv = vec + (item_count & 1) * 2 * D;
      const float* dov = qv + D;
      // A query that attends a single pair has P = 1 and a score gradient of exactly zero (TdpMask::single_pair):
      // what G holds for it is P (dP - Dq) with the two terms equal only up to the 16-bit rounding of the stored
      // output, so G is dropped (dQ = 0, nothing added to dK1 / dK2) instead of being folded.
      const bool single = TdpMask{p.causal, T, p.k1w, p.k2w, p.kkl, p.kkr}.single_pair(q);
      // undoes the fp16 range shift of P and dS (1 for bf16)
      const float unshift = exp2f(-(float)prob_shift<T16>(q, p.causal, T, p.k1w, p.k2w));
      const float alpha_u = p.alpha * unshift;
      if (role == 0) {
        if (row < D) dq_acc[row] = 0.f;
        if (!fold_sync()) { alive = false; break; }
      }
      for (int xt = xt0; xt < xt0 + nxt && alive; ++xt, ++xt_count) {
        const int x_r = xt * 128 + row;
        const bool x_ok = (p.causal ? (x_r <= q && q - x_r <= win.xw) : true) && x_r < T;
        // (rows outside the query's range carry zeros: a warp whose 32 rows all are has nothing to add)
        const bool warp_rows_live = __any_sync(0xffffffffu, x_ok);
        alive = __all_sync(0xffffffffu, mbar_wait_x<PAIR>(&bars.gu_done, xt_count & 1, abort_flag));
        if (!alive) break;
        tc_fence_after();
#pragma unroll 1
        for (int pc = 0; pc < 2 * (D / 32); ++pc, ++round) {
          const bool is_u = pc < D / 32;   // U first: the next tile needs its accumulator earlier than G's
          const int h0 = (is_u ? pc : pc - D / 32) * 32;
          // role 0, G pieces: this row's X values for the dQ product (issued early to hide the latency)
          uint4 xr[4];
          const bool want_dq = !is_u && role == 0 && !single;
          if (want_dq) {
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4)
              xr[i4] = x_ok ? __ldg(reinterpret_cast<const uint4*>(Xg + (size_t)x_r * D + h0 + i4 * 8))
                            : make_uint4(0, 0, 0, 0);
          }
          uint32_t g[32];
          tmem_ld32(tmem + lane_base + (is_u ? Cfg::kTmemU : Cfg::kTmemG) + h0, g);
          tmem_wait_ld();
          // scale by Q[q] / dO[q] right away: after the hand-off below the soft-max warps may move on to a
          // later query and overwrite an older copy of these vectors
          float v[32];
          {
            const float4* mul = reinterpret_cast<const float4*>((is_u ? dov : qv) + h0);
            // (the Q copy carries the factor alpha * log2(e) of the score operand)
            const float sc = is_u ? unshift : unshift * (1.f / kLog2e);
            const float2 sc2 = make_float2(sc, sc);
#pragma unroll
            for (int i4 = 0; i4 < 8; ++i4) {
              const float4 m = mul[i4];
              const float2 lo = __fmul2_rn(__fmul2_rn(make_float2(__uint_as_float(g[i4 * 4]), __uint_as_float(g[i4 * 4 + 1])), sc2),
                                           make_float2(m.x, m.y));
              const float2 hi = __fmul2_rn(__fmul2_rn(make_float2(__uint_as_float(g[i4 * 4 + 2]), __uint_as_float(g[i4 * 4 + 3])), sc2),
                                           make_float2(m.z, m.w));
              v[i4 * 4] = lo.x;
              v[i4 * 4 + 1] = lo.y;
              v[i4 * 4 + 2] = hi.x;
              v[i4 * 4 + 3] = hi.y;
            }
          }
          if (pc == D / 32 - 1) {
            // last piece of U is in registers: that accumulator may be overwritten
            tc_fence_before();
            to_mma(&bars.u_free);
          }
          if (pc == 2 * (D / 32) - 1) {
            // likewise G
            tc_fence_before();
            to_mma(&bars.g_free);
            if (xt == xt0 + nxt - 1) mbar_arrive(&bars.vec_free[item_count & 1]);  // and this query's vectors are done with
          }
          uint8_t* slot = slots + (round & 1) * 4096;
          // the reduce-add issued two rounds ago from this slot must have finished reading it
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          __syncwarp();
#pragma unroll
          for (int i4 = 0; i4 < 8; ++i4)
            *reinterpret_cast<float4*>(slot + swz128(lane, i4)) =
                make_float4(v[i4 * 4], v[i4 * 4 + 1], v[i4 * 4 + 2], v[i4 * 4 + 3]);
          fence_async_smem();
          __syncwarp();
          // (rows beyond the query carry zeros: a warp whose 32 rows are all beyond it has nothing to add)
          if (lane == 0 && warp_rows_live && (is_u || !single)) {
            tma_reduce_add_3d(is_u ? tmDY : tmDX, slot, h0, xt * 128 + wq * 32, bh);
            bulk_commit();
          }
          if (want_dq) {
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4) {
              const uint32_t wx[4] = {xr[i4].x, xr[i4].y, xr[i4].z, xr[i4].w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 gx = __fmul2_rn(__fmul2_rn(make_float2(__uint_as_float(g[i4 * 8 + 2 * e]),
                                                                    __uint_as_float(g[i4 * 8 + 2 * e + 1])),
                                                        make_float2(alpha_u, alpha_u)),
                                             unpack2<T16>(wx[e]));
                v[i4 * 8 + 2 * e] = gx.x;
                v[i4 * 8 + 2 * e + 1] = gx.y;
              }
            }
            const float colsum = warp_transpose_sum(v, lane);
            atomicAdd(&dq_acc[h0 + lane], colsum);
          }
        }
      }
      if (!alive) break;
      if (role == 0) {
        if (!fold_sync()) { alive = false; break; }  // every warp's contribution to dq_acc has landed
        if (row < D) ((T16*)p.dq)[hb + (size_t)q * D + row] = from_f<T16>(dq_acc[row]);
        if (!fold_sync()) { alive = false; break; }  // dq_acc may be cleared for the next item
      }
    }
    bulk_wait_all();  // reduce-adds still in flight must complete before the CTA retires
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();  // neither CTA frees tensor memory or leaves while the other may still use it
  if (warp == 0) {
    if constexpr (PAIR) tmem_dealloc_pair(tmem, 512); else tmem_dealloc(tmem, 512);
  }
  if (tid == 0 && bars.abort_flag && p.status) atomicOr(p.status, 4);
}

template <int D, typename T16, int NSW>
int launch_bwd(const TdpArgs& a) {
  using Cfg = BwdCfg<D>;
  const int BN = a.B * a.N;
  const size_t n = (size_t)BN * a.T * a.D;
  float* part = (float*)a.workspace;          // dK1 | dK2 | dSiLU(V1) | dV2
  T16* sv1 = (T16*)(part + 4 * n);
  TRITT_CUDA_OK(cudaMemsetAsync(part, 0, 4 * n * sizeof(float), a.stream));
  silu_kernel<T16><<<(unsigned)((n / 8 + 255) / 256 + 1), 256, 0, a.stream>>>((const T16*)a.v1, sv1, n);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  CUtensorMap tmK1, tmK2, tmSV1, tmV2, tmDK1, tmDK2, tmDSV1, tmDV2;
  int rc;
  if ((rc = make_tmap_3d(&tmK1, a.k1, 2, D, a.T, BN, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmK2, a.k2, 2, D, a.T, BN, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmSV1, sv1, 2, D, a.T, BN, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmV2, a.v2, 2, D, a.T, BN, 64, 128))) return rc;
  if ((rc = make_tmap_3d_f32(&tmDK1, part, D, a.T, BN, 32, 32))) return rc;
  if ((rc = make_tmap_3d_f32(&tmDK2, part + n, D, a.T, BN, 32, 32))) return rc;
  if ((rc = make_tmap_3d_f32(&tmDSV1, part + 2 * n, D, a.T, BN, 32, 32))) return rc;
  if ((rc = make_tmap_3d_f32(&tmDV2, part + 3 * n, D, a.T, BN, 32, 32))) return rc;
  BwdParams p{};
  p.q = a.q; p.o = a.o; p.d_o = a.d_o; p.lse = a.lse_in; p.dq = a.dq;
  p.x[0] = a.k2; p.x[1] = a.k1;
  p.T = a.T; p.BN = BN; p.q_mod = a.q_mod; p.q_rem = a.q_rem;
  p.nq = a.q_rem < a.T ? (a.T - a.q_rem + a.q_mod - 1) / a.q_mod : 0;
  p.causal = a.mask.causal;
  p.k1w = a.mask.k1w;
  p.k2w = a.mask.k2w;
  p.kkl = a.mask.kkl;
  p.kkr = a.mask.kkr;
  p.alpha = a.alpha;
  p.status = a.status_word;
  BwdHalfMaps half{};
  // CTA pairs (on request: TRITT_FLAG_BWD_CTA_PAIRS): head dimension 128, an even number of queries, and a mask
  // whose tile ranges are the same for two neighbouring queries (no windows); everything else runs one CTA per item.
  const TdpMask& m = a.mask;
  bool pair = (a.flags & TRITT_FLAG_BWD_CTA_PAIRS) && D == 128 && p.nq >= 2 && p.nq % 2 == 0 &&
              (!m.causal || (m.k1w >= a.T && m.k2w >= a.T && m.kkl >= a.T && m.kkr >= a.T));
  if (p.nq > 0 && pair) {
    if constexpr (D == 128) {
      auto kern = tdp_bwd_kernel<D, T16, NSW, true>;
      TRITT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
      cudaLaunchConfig_t cfg{};
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.gridDim = dim3(2, 1, 1);
      cfg.blockDim = dim3(BwdThreads<NSW>::kTotal, 1, 1);
      cfg.dynamicSmemBytes = Cfg::kSmem;
      cfg.stream = a.stream;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters < 1) {
        (void)cudaGetLastError();
        pair = false;   // no room for a pair on this device: one CTA per item
      } else {
        if ((rc = make_tmap_3d(&half.k1, a.k1, 2, D, a.T, BN, 64, 64))) return rc;
        if ((rc = make_tmap_3d(&half.k2, a.k2, 2, D, a.T, BN, 64, 64))) return rc;
        if ((rc = make_tmap_3d(&half.sv1, sv1, 2, D, a.T, BN, 64, 64))) return rc;
        if ((rc = make_tmap_3d(&half.v2, a.v2, 2, D, a.T, BN, 64, 64))) return rc;
        const long items = (long)(p.nq / 2) * BN * 2;
        cfg.gridDim = dim3((unsigned)(2 * (items < clusters ? items : clusters)), 1, 1);
        TRITT_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, tmK1, tmK2, tmSV1, tmV2, tmDK1, tmDK2, tmDSV1, tmDV2, half, p));
        count_launch();
      }
    }
  }
  if (p.nq > 0 && !pair) {
    auto kern = tdp_bwd_kernel<D, T16, NSW, false>;
    TRITT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
    const long items = (long)p.nq * BN * 2;
    const int grid = (int)(items < num_sms() ? items : num_sms());
    kern<<<grid, BwdThreads<NSW>::kTotal, Cfg::kSmem, a.stream>>>(tmK1, tmK2, tmSV1, tmV2, tmDK1, tmDK2, tmDSV1, tmDV2, half, p);
    count_launch();
    TRITT_CUDA_OK(cudaGetLastError());
  }
  if (a.flags & TRITT_FLAG_BWD_PARTIAL) return 0;
  return simt_tdp_bwd_finalize(a.v1, a.dk1, a.dk2, a.dv1, a.dv2, n, a.dtype, part, a.stream);
}

template <int D, typename T16>
int launch_bwd_any(const TdpArgs& a) {
  return launch_bwd<D, T16, 2>(a);
}

}  // namespace


size_t sm100_tdp_bwd_workspace(int B, int N, int T, int D) {
  const size_t n = (size_t)B * N * T * D;
  return 4 * n * sizeof(float) + n * 2;
}

int sm100_tdp_bwd(const TdpArgs& a) {
  if (a.dtype == TRITT_BF16)
    return a.D == 128 ? launch_bwd_any<128, __nv_bfloat16>(a) : launch_bwd_any<64, __nv_bfloat16>(a);
  return a.D == 128 ? launch_bwd_any<128, __half>(a) : launch_bwd_any<64, __half>(a);
}

}  // namespace tritt
