// Triple-dot-product trittention forward on Blackwell tensor cores (tcgen05 + TMEM + TMA).
//
// Formulation.  For one query q and a tile of 128 K2 rows, the 128 "pair rows" r = (q, k)
// carry the pre-scaled operand  A[r,h] = alpha*log2(e) * Q[q,h] * K2[k,h].  With it the
// score slab is an ordinary GEMM, S[r,j] = sum_h A[r,h] K1[j,h], and the walk over j is
// exactly a flash-attention inner loop with K1 as keys and SiLU(V1) as values:
//     acc[r,h] = sum_j exp2(S[r,j] - m_r) SiLU(V1)[j,h]          (online soft-max per row)
// The V2 factor and the soft-max over k are applied when the tile is folded into the
// query's running output:  O[q,h] = sum_r w_r acc[r,h] V2[k_r,h] / sum_r w_r l_r.
// (The reference's Blackwell Triton kernel uses the same (q,k)-row arrangement,
// b200/fwd_b200.py:217-220,253,317-321, with 16x16 query/key tiles; its generic kernel
// builds K1 x K2 outer products per tile, triple_dot_product/kernels/fwd.py:160-164.)
//
// One CTA (persistent, 512 threads) processes a pair of queries (qa, qb) of the same 128-row
// block as two row tiles that share every K1 / SiLU(V1) tile and take turns on the tensor pipe:
//   warp 0       TMA producer: the K2 tile of each k-tile, then a ring of 128-row K1 / SiLU(V1) tiles
//   warp 1       issues tcgen05.mma: S_x = A_x*K1^T (128x128 fp32 slab in TMEM, one per tile) and
//                acc_x += P_x*SiLU(V1) with P_x read from TMEM (it overlays S_x) and the value tile used
//                row-major (MN-major descriptor).  128-column slabs keep every accumulation chain at
//                8 instructions of 128x128x16, the shape the pipe runs at full rate.
//   warps 4-11   two soft-max warpgroups (one row per thread); they also form A_a, A_b.  Where a head-wide bound on
//                the scores is small (per-head statistics from a small kernel before this one) every row takes its
//                own score bound as the soft-max reference and the warpgroups work on the same slab, tile a then
//                tile b, 64 of its 128 columns each: one pass, exp2, P written back to TMEM as 16-bit over the
//                first half of the columns just read.  Otherwise warpgroup x owns tile x and a thread its whole
//                row: row maximum, exp2 with lazy rescaling of the accumulator, P over the first 64 columns of S_x
//   warps 12-15  fold warpgroup: when a k-tile is finished, folds acc_x (times V2, soft-max over k) into
//                the queries' running (max, sum, output) while the other warps start the next k-tile
// Causal structure: for a fixed query the mask is "j <= q" on columns and "k <= q" on rows, so
// whole slabs above q are never visited, only the last slab is masked (by a column bound that
// is uniform over the rows), and rows with k > q get weight zero in the fold.
#include "tritt_common.cuh"
#include "tritt_sm100.cuh"
#include "tritt_sm100_tdp.cuh"

#include <type_traits>

namespace tritt {
namespace {
using namespace sm100;

constexpr int kThreads = 512;
constexpr int kBJ = 128;            // key columns per slab
constexpr float kRescaleGap = 8.f;  // rescale the accumulator only when the row max grew by more than 2^8

template <int D> struct FwdCfg {
  static constexpr int kTileA = 128 * D * 2;    // bytes of one 128-row tile (operand, K1 or SiLU(V1))
  static constexpr int kStages = 4;
  static constexpr int kOffAa = 0;
  static constexpr int kOffAb = kTileA;
  static constexpr int kOffRing = 2 * kTileA;
  static constexpr int kOffStats = kOffRing + kStages * kTileA;  // [2 parities][2 tiles][128][4] fp32: row (reference, two partial sums, -)
  static constexpr int kOffRed = kOffStats + 2 * 2 * 128 * 4 * 4;  // [2 tiles][4 warps][D] fp32 column sums
  static constexpr int kOffFstat = kOffRed + 2 * 4 * D * 4;        // [2 tiles][8] fp32 warp max / sum
  static constexpr int kOffNorm = kOffFstat + 2 * 8 * 4;            // [2 tiles][2 column halves][128] fp32: partial |A_row|^2
  static constexpr int kOffBars = kOffNorm + 2 * 2 * 128 * 4;
  static constexpr int kSmem = kOffBars + 256;
  static constexpr int kTmemO = 256;  // S_a | S_b | acc_a | acc_b
};

struct FwdParams {
  void* out;
  float* lse;
  const void *q, *v2;
  int T, BN, nq, q_mod, q_rem, causal, n_pairs;
  int k1w, k2w, kkl, kkr;  // windows of the causal mask (T or more = unbounded)
  float scale2;  // alpha * log2(e)
  const float* k1_norm2_max;  // [BN] largest squared row norm of K1 per head, or null (no score bound available)
  const float* q_norm2_max;   // [BN] largest squared row norm of Q per head (with k1_norm2_max)
  const float* k2_elem2_max;  // [BN] largest squared element of K2 per head (with k1_norm2_max)
  float bound_limit;          // rows whose score bound is below this skip the row-maximum pass
  int* status;
};

struct FwdBarriers {
  uint64_t ring_full[4], ring_empty[4];
  uint64_t k2_full, a_ready, a_free;
  uint64_t s_ready[2], p_ready[2];               // per tile, one phase per slab
  uint64_t o_done, o_free[2], stats_ready[2];    // per k-tile hand-offs with the fold warpgroup
  uint64_t fold_sync;
  uint32_t tmem_base;
  int abort_flag;
};

template <int D, typename T16>
__global__ void __launch_bounds__(kThreads, 1)
tdp_fwd_kernel(const __grid_constant__ CUtensorMap tmK1, const __grid_constant__ CUtensorMap tmK2,
               const __grid_constant__ CUtensorMap tmSV1, FwdParams p) {
  using Cfg = FwdCfg<D>;
  constexpr int NS = Cfg::kStages;
  constexpr int KH = D / 64;  // 64-column halves per row
  extern __shared__ __align__(1024) uint8_t smem[];
  static_assert(sizeof(FwdBarriers) <= 256, "barrier block too large");
  FwdBarriers& bars = *reinterpret_cast<FwdBarriers*>(smem + Cfg::kOffBars);
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
    mbar_init(&bars.k2_full, 1);
    mbar_init(&bars.a_ready, 256);
    mbar_init(&bars.a_free, 256);
    for (int x = 0; x < 2; ++x) {
      mbar_init(&bars.s_ready[x], 1);
      mbar_init(&bars.p_ready[x], 256);
      mbar_init(&bars.o_free[x], 128);
      mbar_init(&bars.stats_ready[x], 256);
    }
    mbar_init(&bars.o_done, 1);
    mbar_init(&bars.fold_sync, 128);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&bars.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars.tmem_base;
  volatile int* abort_flag = &bars.abort_flag;

  const int T = p.T;
  const long n_items = (long)p.n_pairs * p.BN;

  // Work item -> (head, query pair).  Items are ordered by decreasing cost (late queries first).
  auto decode = [&](long item, int& bh, int& qa, int& qb) {
    const int pr = p.n_pairs - 1 - (int)(item / p.BN);
    bh = (int)(item % p.BN);
    const int ia = 2 * pr, ib = min(2 * pr + 1, p.nq - 1);
    qa = p.q_rem + ia * p.q_mod;
    qb = p.q_rem + ib * p.q_mod;
  };
  // Tiles a query pair visits (qa <= qb).  Causal mask: j <= q <= j + k1w, k <= q <= k + k2w, k - kkl <= j <= k + kkr.
  // k-tiles: rows k in [max(0, qa - k2w, qa - k1w - kkr), qb]  (rows below the third bound see no column at all);
  // slabs of k-tile kt: columns j in [max(0, qa - k1w, k_first - kkl), min(qb, k_last + kkr)], never empty.
  auto k_range = [&](int qa, int qb, int& kt0, int& nkt) {
    if (!p.causal) {
      kt0 = 0;
      nkt = (T + 127) / 128;
      return;
    }
    const int klo = max(0, max(qa - p.k2w, qa - p.k1w - p.kkr));
    kt0 = klo / 128;
    nkt = qb / 128 - kt0 + 1;
  };
  auto j_range = [&](int qa, int qb, int kt, int& jt0, int& njt) {
    if (!p.causal) {
      jt0 = 0;
      njt = (T + kBJ - 1) / kBJ;
      return;
    }
    const int klo = max(0, max(qa - p.k2w, qa - p.k1w - p.kkr));
    const int ka = max(kt * 128, klo), kb = min(kt * 128 + 127, qb);
    const int ja = max(0, max(qa - p.k1w, ka - p.kkl)), jb = min(qb, kb + p.kkr);
    jt0 = ja / kBJ;
    njt = jb / kBJ - jt0 + 1;
  };
  // Attended columns of k-tile kt (union over its rows): [ja, jb].  A slab whose attended columns all lie in one
  // 64-column half (halves() = 1: the lower, 2: the upper, 0: both) runs as 128 x 64 score products and a 64-deep
  // value product.
  auto col_span = [&](int qa, int qb, int kt, int& ja, int& jb) {
    ja = 0;
    jb = T - 1;
    if (p.causal) {
      const int klo = max(0, max(qa - p.k2w, qa - p.k1w - p.kkr));
      const int ka = max(kt * 128, klo), kb = min(kt * 128 + 127, qb);
      ja = max(0, max(qa - p.k1w, ka - p.kkl));
      jb = min(qb, kb + p.kkr);
    }
  };
  auto halves = [](int ja, int jb, int j0) { return jb < j0 + 64 ? 1 : (ja >= j0 + 64 ? 2 : 0); };
  // How the soft-max warps divide a head's work.  Every score of the head is bounded by
  // |s| max_q |Q_q| max |K2 element| max_j |K1_j|  (|A_row|^2 = s^2 sum_h Q_h^2 K2_h^2 <= s^2 max_h K2_h^2 |Q_q|^2).
  // Where that is below the limit, every row can take its own score bound as soft-max reference (one pass, nothing
  // to agree on between threads) and the two warpgroups split every slab's columns; otherwise each warpgroup owns one
  // tile and a thread its whole row (maximum pass, rescaling).  Uniform over a work item, read by every role.
  auto head_split = [&](int bh) -> bool {
    if (!p.k1_norm2_max) return false;
    const float b = fabsf(p.scale2) * sqrtf(__ldg(p.q_norm2_max + bh)) * sqrtf(__ldg(p.k2_elem2_max + bh)) *
                    sqrtf(__ldg(p.k1_norm2_max + bh));
    return b <= p.bound_limit;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // (the whole warp walks the schedule converged, one elected lane issues the copies)
    {
      const bool leader = elect_one();
      if (leader) {
        tma_prefetch_desc(&tmK1);
        tma_prefetch_desc(&tmK2);
        tma_prefetch_desc(&tmSV1);
      }
      uint32_t kt_count = 0, pos = 0;
      bool alive = true;
      auto load_stage = [&](const CUtensorMap* tm, int row0, int bh) -> bool {
        const int st = pos % NS;
        if (!__all_sync(0xffffffffu, mbar_wait(&bars.ring_empty[st], ((pos / NS) & 1) ^ 1, abort_flag))) return false;
        if (leader) {
          mbar_arrive_expect_tx(&bars.ring_full[st], Cfg::kTileA);
          for (int hh = 0; hh < KH; ++hh)
            tma_load_3d(smem + Cfg::kOffRing + st * Cfg::kTileA + hh * 16384, tm, &bars.ring_full[st], hh * 64, row0, bh);
        }
        ++pos;
        return true;
      };
      for (long item = blockIdx.x; item < n_items && alive; item += gridDim.x) {
        int bh, qa, qb, kt0, nkt;
        decode(item, bh, qa, qb);
        k_range(qa, qb, kt0, nkt);
        for (int kt = kt0; kt < kt0 + nkt && alive; ++kt, ++kt_count) {
          int jt0, njt;
          j_range(qa, qb, kt, jt0, njt);
          // the first K1 tile does not depend on the previous k-tile: fetch it before waiting for the operand buffer
          alive = load_stage(&tmK1, jt0 * kBJ, bh);
          if (!alive || !__all_sync(0xffffffffu, mbar_wait(&bars.a_free, (kt_count & 1) ^ 1, abort_flag))) {
            alive = false;
            break;
          }
          if (leader) {
            mbar_arrive_expect_tx(&bars.k2_full, Cfg::kTileA);
            for (int hh = 0; hh < KH; ++hh)
              tma_load_3d(smem + Cfg::kOffAa + hh * 16384, &tmK2, &bars.k2_full, hh * 64, kt * 128, bh);
          }
          // ring order: K1(0), V(0), K1(1), V(1), ...
          for (int jt = jt0; jt < jt0 + njt && alive; ++jt) {
            alive = load_stage(&tmSV1, jt * kBJ, bh);
            if (alive && jt + 1 < jt0 + njt) alive = load_stage(&tmK1, (jt + 1) * kBJ, bh);
          }
        }
      }
      if (!alive) {
        // give copies still in flight a bounded chance to land before the CTA retires
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
    // descriptor arithmetic stays on the uniform datapath, where a lone thread needs a register-to-uniform move per
    // operand and loses its issue slots to the busy warps of its scheduler.
    {
      const bool leader = elect_one();
      // (every lane waits; the vote keeps the warp converged whatever a lane's wait returned)
      auto wait_all = [&](uint64_t* bar, uint32_t parity) {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
      };
      auto commit = [&](uint64_t* bar) {
        if (leader) mma_commit(bar);
      };
      constexpr int kFmt = std::is_same<T16, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_s = make_idesc_f16(128, kBJ, kFmt, false, false);
      constexpr uint32_t idesc_pv = make_idesc_f16(128, D, kFmt, false, true);
      // descriptor low words; per instruction only a constant (in 16-byte units) is added
      constexpr uint32_t kHi = desc_hi(1024);
      constexpr uint32_t kTile16 = Cfg::kTileA >> 4;
      const uint32_t aLo[2] = {desc_lo(smem_u32(smem + Cfg::kOffAa), 16), desc_lo(smem_u32(smem + Cfg::kOffAb), 16)};
      const uint32_t ringK = desc_lo(smem_u32(smem + Cfg::kOffRing), 16);      // K-major view of a stage
      const uint32_t ringMN = desc_lo(smem_u32(smem + Cfg::kOffRing), 16384);  // row-major (MN-major) view
      uint32_t kt_count = 0, base = 0, n = 0;  // n: slabs finished so far (same for both tiles)
      bool alive = true;
      auto wait_full = [&](uint32_t pos) {
        return wait_all(&bars.ring_full[pos % NS], (pos / NS) & 1);
      };
      auto release = [&](uint32_t pos) { commit(&bars.ring_empty[pos % NS]); };
      // S_x = A_x * K1tile^T  (one chain of D/16 instructions); hm != 0: only 64 rows of the key tile (the lower
      // or the upper ones), scores in the first 64 columns of S_x
      constexpr uint32_t idesc_s64 = make_idesc_f16(128, 64, kFmt, false, false);
      auto issue_s = [&](int x, uint32_t pos, int hm) {
        const uint32_t bLo = ringK + (pos % NS) * kTile16;
        if (hm == 0) {
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t kk = (k >> 2) * (16384 >> 4) + (k & 3) * 2;
            if (leader) mma_ss_lo(tmem + x * kBJ, aLo[x] + kk, bLo + kk, kHi, idesc_s, k > 0);
          }
        } else {
          const uint32_t bRow = bLo + (hm == 2 ? (64 * 128) >> 4 : 0);   // rows 64.. of a 128-byte-pitch block
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t kk = (k >> 2) * (16384 >> 4) + (k & 3) * 2;
            if (leader) mma_ss_lo(tmem + x * kBJ, aLo[x] + kk, bRow + kk, kHi, idesc_s64, k > 0);
          }
        }
        commit(&bars.s_ready[x]);
      };
      // acc_x (+)= P_x * SiLU(V1)tile  (one chain of 8 instructions; P_x overlays the first 64 columns of S_x);
      // hm != 0: P_x has 64 columns (4 instructions) and meets the lower or upper 64 rows of the value tile
      // (split: P of a warpgroup's columns sits over the first half of them; otherwise over the first 64 columns of S_x)
      auto issue_pv = [&](int x, uint32_t pos, uint32_t acc, int hm, bool split) {
        const uint32_t bLo = ringMN + (pos % NS) * kTile16;
        if (hm == 0) {
#pragma unroll
          for (int k = 0; k < kBJ / 16; ++k)
            if (leader)
              mma_ts_lo(tmem + Cfg::kTmemO + x * D, tmem + x * kBJ + (split ? (k >> 2) * 64 + (k & 3) * 8 : k * 8),
                      bLo + k * (2048 >> 4), kHi, idesc_pv, k > 0 ? 1u : acc);
        } else {
          const uint32_t bRow = bLo + (hm == 2 ? (4 * 2048) >> 4 : 0);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            if (leader)
              mma_ts_lo(tmem + Cfg::kTmemO + x * D, tmem + x * kBJ + (split ? (k >> 1) * 32 + (k & 1) * 8 : k * 8),
                      bRow + k * (2048 >> 4), kHi, idesc_pv, k > 0 ? 1u : acc);
        }
      };

      for (long item = blockIdx.x; item < n_items && alive; item += gridDim.x) {
        int bh, qa, qb, kt0, nkt;
        decode(item, bh, qa, qb);
        k_range(qa, qb, kt0, nkt);
        const bool split = head_split(bh);
        for (int kt = kt0; kt < kt0 + nkt && alive; ++kt, ++kt_count) {
          int jt0, njt;
          j_range(qa, qb, kt, jt0, njt);
          if (!wait_all(&bars.a_ready, kt_count & 1)) { alive = false; break; }
          tc_fence_after();
          if (!wait_full(base)) { alive = false; break; }
          int ja, jb;
          col_span(qa, qb, kt, ja, jb);
          int hm = halves(ja, jb, jt0 * kBJ);
          issue_s(0, base, hm);
          issue_s(1, base, hm);
          release(base);
          for (int jt = 0; jt < njt && alive; ++jt, ++n) {
            const uint32_t pv = base + 2 * jt + 1, pk = base + 2 * jt + 2;
            const bool more = jt + 1 < njt;
            const int hm_next = more ? halves(ja, jb, (jt0 + jt + 1) * kBJ) : 0;
            for (int x = 0; x < 2 && alive; ++x) {
              if (!wait_all(&bars.p_ready[x], n & 1)) { alive = false; break; }
              if (jt == 0) {
                // the fold warpgroup must have drained the previous k-tile's accumulator of this tile
                if (!wait_all(&bars.o_free[x], (kt_count & 1) ^ 1)) { alive = false; break; }
              }
              tc_fence_after();
              if (x == 0 && !wait_full(pv)) { alive = false; break; }
              issue_pv(x, pv, jt > 0, hm, split);
              if (x == 1) release(pv);
              if (more) {
                if (x == 0 && !wait_full(pk)) { alive = false; break; }
                issue_s(x, pk, hm_next);
                if (x == 1) release(pk);
              }
            }
            hm = hm_next;
          }
          if (alive) commit(&bars.o_done);
          base += 2 * njt;
        }
      }
    }
  } else if (warp >= 4 && warp < 12) {
    // ------------------------------------------------------------------ soft-max warpgroups
    // Both warpgroups work on the same slab, tile a first, then tile b: warpgroup `wg` takes the slab's columns
    // [wg * 64, wg * 64 + 64) (32 of a half-width slab's 64), one row per thread, and writes P over the first half of
    // the columns it has read.  While they are on one tile, the tensor pipe runs the other tile's two products.
    const int wg = (warp - 4) >> 2;         // column half of every slab
    const int wq = warp & 3;                // TMEM lane quadrant of this warp
    const int row = wq * 32 + lane;         // row of both tiles owned by this thread
    const int st = tid - 128;               // 0..255 over both warpgroups
    const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
    float* stats = (float*)(smem + Cfg::kOffStats);
    float* norms = (float*)(smem + Cfg::kOffNorm);
    uint32_t kt_count = 0, n = 0;
    bool alive = true;

    // largest score of this thread's NC columns at TMEM address tS ([lo, hi]: the columns the row may see)
    auto row_max = [&](auto nc, uint32_t tS, bool full, int lo, int hi) -> float {
      constexpr int NC = decltype(nc)::value;
      uint32_t sr[NC];
      if constexpr (NC == 64) tmem_ld64(tS, sr); else tmem_ld32(tS, sr);
      tmem_wait_ld();
      float mx = -INFINITY;
      if (full) {
        // four independent chains instead of one NC-deep dependency
        float m0 = __uint_as_float(sr[0]), m1 = __uint_as_float(sr[1]), m2 = __uint_as_float(sr[2]),
              m3 = __uint_as_float(sr[3]);
#pragma unroll
        for (int c = 4; c < NC; c += 4) {
          m0 = fmaxf(m0, __uint_as_float(sr[c]));
          m1 = fmaxf(m1, __uint_as_float(sr[c + 1]));
          m2 = fmaxf(m2, __uint_as_float(sr[c + 2]));
          m3 = fmaxf(m3, __uint_as_float(sr[c + 3]));
        }
        mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      } else {
#pragma unroll
        for (int c = 0; c < NC; ++c)
          if (c >= lo && c <= hi) mx = fmaxf(mx, __uint_as_float(sr[c]));
      }
      return mx;
    };
    // P = exp2(S - m) of this thread's NC columns, packed to 16 bits over the first NC / 2 of them; returns their sum
    // (written at tP, which lies within columns this thread has read)
    auto form_p = [&](auto nc, uint32_t tS, uint32_t tP, bool full, int lo, int hi, float m) -> float {
      constexpr int NC = decltype(nc)::value;
      uint32_t sr[NC];
      if constexpr (NC == 64) tmem_ld64(tS, sr); else tmem_ld32(tS, sr);
      tmem_wait_ld();
      uint32_t pk[NC / 2];
      float ps0 = 0.f, ps1 = 0.f;
      if (full) {
        // packed fp32 pairs: one subtraction and one addition per two scores
        const float2 nm = make_float2(-m, -m);
        float2 pa = make_float2(0.f, 0.f), pb = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < NC; c += 4) {
          const float2 x0 = __fadd2_rn(make_float2(__uint_as_float(sr[c]), __uint_as_float(sr[c + 1])), nm);
          const float2 x1 = __fadd2_rn(make_float2(__uint_as_float(sr[c + 2]), __uint_as_float(sr[c + 3])), nm);
          const float2 e0 = make_float2(exp2f(x0.x), exp2f(x0.y));
          const float2 e1 = make_float2(exp2f(x1.x), exp2f(x1.y));
          pa = __fadd2_rn(pa, e0);
          pb = __fadd2_rn(pb, e1);
          pk[c >> 1] = pack2<T16>(e0.x, e0.y);
          pk[(c >> 1) + 1] = pack2<T16>(e1.x, e1.y);
        }
        ps0 = pa.x + pb.x;
        ps1 = pa.y + pb.y;
      } else {
        // (a row with no valid column so far has m = -inf and selects 0 everywhere)
#pragma unroll
        for (int c = 0; c < NC; c += 2) {
          const float p0 = (c >= lo && c <= hi) ? exp2f(__uint_as_float(sr[c]) - m) : 0.f;
          const float p1 = (c + 1 >= lo && c + 1 <= hi) ? exp2f(__uint_as_float(sr[c + 1]) - m) : 0.f;
          ps0 += p0;
          ps1 += p1;
          pk[c >> 1] = pack2<T16>(p0, p1);
        }
      }
      tmem_st(tP, pk);
      return ps0 + ps1;
    };

    for (long item = blockIdx.x; item < n_items && alive; item += gridDim.x) {
      int bh, qa, qb, kt0, nkt;
      decode(item, bh, qa, qb);
      k_range(qa, qb, kt0, nkt);
      const T16* Qg = (const T16*)p.q + (size_t)bh * T * D;
      // largest K1 row norm of this head: with |A_row| it bounds every score of the row (Cauchy-Schwarz)
      const float k1_max = p.k1_norm2_max ? sqrtf(__ldg(p.k1_norm2_max + bh)) : INFINITY;
      const bool split = head_split(bh);

      for (int kt = kt0; kt < kt0 + nkt && alive; ++kt, ++kt_count) {
        int jt0, njt, ja, jb;
        j_range(qa, qb, kt, jt0, njt);
        col_span(qa, qb, kt, ja, jb);
        // Columns this row may see, per tile: [c_lo, c_hi].  A row outside the k range of its query (its weight in
        // the fold is zero) keeps the query's own column range so that it never sees an empty one by construction;
        // a row inside can still see none in a slab, or at all: its maximum then stays -inf and its P zero.
        int c_lo[2] = {0, 0}, c_hi[2] = {T - 1, T - 1};
        if (p.causal) {
          const int k_r = kt * 128 + row;
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            const int qx = x == 0 ? qa : qb;
            const bool in_k = k_r <= qx && qx - k_r <= p.k2w;
            c_lo[x] = max(qx - p.k1w, in_k ? k_r - p.kkl : 0);
            c_hi[x] = in_k ? min(qx, k_r + p.kkr) : qx;
          }
        }
        // ---- operand formation: A_a = s*Q[qa] (.) K2tile (in place), A_b = s*Q[qb] (.) K2tile
        alive = __all_sync(0xffffffffu, mbar_wait(&bars.k2_full, kt_count & 1, abort_flag));
        if (!alive) break;
        {
          const int r = st & 127;
          constexpr int CPT = D / 16;  // 16-byte chunks per thread
          const int c0 = (st >> 7) * CPT;
          float na = 0.f, nb = 0.f;  // this thread's share of |A_a[r]|^2 and |A_b[r]|^2
#pragma unroll
          for (int i = 0; i < CPT; ++i) {
            const int cc = c0 + i, hh = cc >> 3, c = cc & 7;
            const uint32_t off = hh * 16384 + swz128(r, c);
            const uint4 kv = *reinterpret_cast<const uint4*>(smem + Cfg::kOffAa + off);
            const uint4 qav = __ldg(reinterpret_cast<const uint4*>(Qg + (size_t)qa * D + cc * 8));
            const uint4 qbv = __ldg(reinterpret_cast<const uint4*>(Qg + (size_t)qb * D + cc * 8));
            const uint32_t w[4] = {kv.x, kv.y, kv.z, kv.w};
            const uint32_t wa[4] = {qav.x, qav.y, qav.z, qav.w};
            const uint32_t wb[4] = {qbv.x, qbv.y, qbv.z, qbv.w};
            uint32_t oa[4], ob[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = unpack2<T16>(w[e]);
              const float2 fa = unpack2<T16>(wa[e]), fb = unpack2<T16>(wb[e]);
              const float k0 = f.x * p.scale2, k1v = f.y * p.scale2;
              const float a0 = k0 * fa.x, a1 = k1v * fa.y, b0 = k0 * fb.x, b1 = k1v * fb.y;
              na = fmaf(a0, a0, fmaf(a1, a1, na));
              nb = fmaf(b0, b0, fmaf(b1, b1, nb));
              oa[e] = pack2<T16>(a0, a1);
              ob[e] = pack2<T16>(b0, b1);
            }
            *reinterpret_cast<uint4*>(smem + Cfg::kOffAa + off) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
            *reinterpret_cast<uint4*>(smem + Cfg::kOffAb + off) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
          }
          // (read by both owners of row r after their first s_ready wait of this k-tile, which this thread's
          //  a_ready arrival below precedes; rewritten only after both have passed a_free)
          norms[(0 * 2 + (st >> 7)) * 128 + r] = na;
          norms[(1 * 2 + (st >> 7)) * 128 + r] = nb;
        }
        fence_async_smem();   // generic-proxy stores above -> visible to the tensor core's reads
        mbar_arrive(&bars.a_ready);

        if (split) {
          // ---- walk over the slabs, both warpgroups on the same slab: tile a, then tile b; warpgroup `wg` takes the
          // slab's columns [wg * 64, wg * 64 + 64) (32 of a half-width slab's 64).  The reference of every row is its
          // score bound |A_row| * max_j |K1_j| (log2 units), which the head-wide bound keeps below the limit: P stays
          // within [2^-2b, 1], representable in the 16-bit type, and no row maximum is needed.
          float ref[2], l_sum[2] = {0.f, 0.f};
#pragma unroll
          for (int x = 0; x < 2; ++x) ref[x] = 0.f;
          for (int jt = 0; jt < njt && alive; ++jt, ++n) {
            // A slab with attended columns in one 64-column half only was computed for that half alone: its scores
            // are in the first 64 columns of S_x and stand for the slab's columns [coff, coff + 64).
            const int hm = halves(ja, jb, (jt0 + jt) * kBJ);
            const int nh = hm ? 1 : 2, coff = hm == 2 ? 64 : 0;
            const int cw = 32 * nh;                                  // columns of this warpgroup in this slab
            const int j0 = (jt0 + jt) * kBJ + coff + wg * cw;      // its first column
#pragma unroll
            for (int x = 0; x < 2; ++x) {
              alive = __all_sync(0xffffffffu, mbar_wait(&bars.s_ready[x], n & 1, abort_flag));
              if (!alive) break;
              tc_fence_after();
              if (jt == 0) ref[x] = sqrtf(norms[(x * 2 + 0) * 128 + row] + norms[(x * 2 + 1) * 128 + row]) * k1_max;
              // the last score product of this k-tile has read A_a and A_b
              if (x == 1 && jt == njt - 1) mbar_arrive(&bars.a_free);
              const uint32_t tS = tmem + lane_base + x * kBJ + wg * cw;
              // this row's valid columns among the warpgroup's: [lo, hi]; the warp takes the unmasked code when all
              // its rows see all of them
              const int lo = c_lo[x] - j0, hi = c_hi[x] - j0;
              const bool full = __all_sync(0xffffffffu, lo <= 0 && hi >= cw - 1);
              // P over the first half of the columns this thread has read
              l_sum[x] += nh == 2 ? form_p(std::integral_constant<int, 64>{}, tS, tS, full, lo, hi, ref[x])
                                  : form_p(std::integral_constant<int, 32>{}, tS, tS, full, lo, hi, ref[x]);
              tmem_wait_st();
              tc_fence_before();
              mbar_arrive(&bars.p_ready[x]);
            }
          }
          if (!alive) break;
          // ---- hand this k-tile's row statistics to the fold warpgroup: (reference, sum of warpgroup 0, of warpgroup 1)
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            float* srow = stats + (((kt_count & 1) * 2 + x) * 128 + row) * 4;
            if (wg == 0) {
              srow[0] = ref[x];
              srow[1] = l_sum[x];
            } else {
              srow[2] = l_sum[x];
            }
            mbar_arrive(&bars.stats_ready[x]);
          }
        } else {
          // ---- walk over the slabs, one warpgroup per tile (warpgroup 0: tile a), one whole row per thread: row
          // maximum, exp2 with lazy rescaling of the accumulator.  A warp whose rows all have a score bound below the
          // limit still uses the bound as reference and skips the maximum pass.  (Arrivals count twice: the barriers
          // expect both warpgroups.)
          const int x = wg;
          const int c_lo_x = x ? c_lo[1] : c_lo[0], c_hi_x = x ? c_hi[1] : c_hi[0];
          const uint32_t tS = tmem + lane_base + x * kBJ;
          float m_used = -INFINITY, l_sum = 0.f;
          bool fast = false;
          for (int jt = 0; jt < njt && alive; ++jt, ++n) {
            alive = __all_sync(0xffffffffu, mbar_wait(&bars.s_ready[x], n & 1, abort_flag));
            if (!alive) break;
            tc_fence_after();
            if (jt == 0) {
              const float bound = sqrtf(norms[(x * 2 + 0) * 128 + row] + norms[(x * 2 + 1) * 128 + row]) * k1_max;
              fast = __all_sync(0xffffffffu, bound <= p.bound_limit);
              if (fast) m_used = bound;
            }
            if (jt == njt - 1) mbar_arrive(&bars.a_free);  // the last score product of this k-tile has read A_x
            const int hm = halves(ja, jb, (jt0 + jt) * kBJ);
            const int nh = hm ? 1 : 2, coff = hm == 2 ? 64 : 0;
            const int j0 = (jt0 + jt) * kBJ + coff;
            const int lo = c_lo_x - j0, hi = c_hi_x - j0;
            const bool full = __all_sync(0xffffffffu, lo <= 0 && hi >= 64 * nh - 1);
            using N64 = std::integral_constant<int, 64>;
            if (!fast) {
              // pass 1: row maximum
              float mx = row_max(N64{}, tS, full, lo, hi);
              if (nh == 2) mx = fmaxf(mx, row_max(N64{}, tS + 64, full, lo - 64, hi - 64));
              if (jt == 0) {
                m_used = mx;  // nothing accumulated yet in this k-tile
              } else {
                const bool grow = mx > m_used + kRescaleGap;
                if (__any_sync(0xffffffffu, grow)) {
                  // some row of this warp moved its max up noticeably: rescale accumulator rows (factor 1 for the
                  // rows that did not move)
                  const float corr = grow ? exp2f(m_used - mx) : 1.f;
                  if (grow) {
                    m_used = mx;
                    l_sum *= corr;
                  }
                  // (s_ready of this slab was committed after the previous P*V, so that product has landed)
                  const uint32_t tO = tmem + lane_base + Cfg::kTmemO + x * D;
#pragma unroll
                  for (int ch = 0; ch < D / 32; ++ch) {
                    uint32_t o[32];
                    tmem_ld32(tO + ch * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                    tmem_st32(tO + ch * 32, o);
                  }
                }
              }
            }
            // pass 2: P = exp2(S - m), packed to 16 bits over the columns already consumed
            l_sum += form_p(N64{}, tS, tS, full, lo, hi, m_used);
            if (nh == 2) l_sum += form_p(N64{}, tS + 64, tS + 32, full, lo - 64, hi - 64, m_used);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_n(&bars.p_ready[x], 2);
          }
          if (!alive) break;
          // ---- hand this k-tile's row statistics to the fold warpgroup
          float* srow = stats + (((kt_count & 1) * 2 + x) * 128 + row) * 4;
          srow[0] = m_used;
          srow[1] = l_sum;
          srow[2] = 0.f;
          mbar_arrive_n(&bars.stats_ready[x], 2);
        }
      }
      if (!alive) break;
    }
  } else if (warp >= 12) {
    // ------------------------------------------------------------------ fold warpgroup
    // After the last P*V of a k-tile: O[q_x,h] accumulates sum_r w_r acc_x[r,h] V2[k_r,h] with
    // w_r = 2^(m_r - M) over the valid rows, merged into the query's running (max, sum, output).
    const int wq = warp & 3;
    const int row = wq * 32 + lane;
    const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
    const float* stats = (const float*)(smem + Cfg::kOffStats);
    float* red = (float*)(smem + Cfg::kOffRed);      // [2][4][D]
    float* fstat = (float*)(smem + Cfg::kOffFstat);  // [2][8]
    uint32_t kt_count = 0, sync_phase = 0;
    bool alive = true;
    auto fold_sync = [&]() -> bool {
      mbar_arrive(&bars.fold_sync);
      const bool ok = mbar_wait(&bars.fold_sync, sync_phase & 1, abort_flag);
      ++sync_phase;
      return __all_sync(0xffffffffu, ok);
    };
    for (long item = blockIdx.x; item < n_items && alive; item += gridDim.x) {
      int bh, qa, qb, kt0, nkt;
      decode(item, bh, qa, qb);
      k_range(qa, qb, kt0, nkt);
      const T16* V2g = (const T16*)p.v2 + (size_t)bh * T * D;
      // running state per tile; thread `row` (< D) owns output column h = row
      float M_run[2] = {-INFINITY, -INFINITY}, L_run[2] = {0.f, 0.f}, O_run[2] = {0.f, 0.f};
      for (int kt = kt0; kt < kt0 + nkt && alive; ++kt, ++kt_count) {
        const int k_r = kt * 128 + row;
        const uint32_t par = kt_count & 1;
        // row statistics of both tiles
        float m_r[2], l_r[2];
        bool valid[2];
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          alive = alive && __all_sync(0xffffffffu, mbar_wait(&bars.stats_ready[x], par, abort_flag));
          if (!alive) break;
          const float* srow = stats + ((par * 2 + x) * 128 + row) * 4;
          m_r[x] = srow[0];
          l_r[x] = srow[1] + srow[2];
          const int qx = x == 0 ? qa : qb;
          valid[x] = p.causal ? (k_r <= qx && qx - k_r <= p.k2w) : (k_r < T);
          float wm = valid[x] ? m_r[x] : -INFINITY;
#pragma unroll
          for (int o = 16; o >= 1; o >>= 1) wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, o));
          if (lane == 0) fstat[x * 8 + wq] = wm;
        }
        if (!alive) break;
        if (!fold_sync()) { alive = false; break; }
        float Mt[2], w[2];
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          // -inf when no row of this tile saw a valid column for this query (possible under narrow windows): the
          // tile then contributes nothing; a single such row has m_r = -inf and gets weight 0
          Mt[x] = fmaxf(fmaxf(fstat[x * 8], fstat[x * 8 + 1]), fmaxf(fstat[x * 8 + 2], fstat[x * 8 + 3]));
          w[x] = (valid[x] && m_r[x] > -INFINITY) ? exp2f(m_r[x] - Mt[x]) : 0.f;
          float lw = w[x] * l_r[x];
#pragma unroll
          for (int o = 16; o >= 1; o >>= 1) lw += __shfl_xor_sync(0xffffffffu, lw, o);
          if (lane == 0) fstat[x * 8 + 4 + wq] = lw;
        }
        // accumulators: the last P*V of both tiles must have landed
        alive = __all_sync(0xffffffffu, mbar_wait(&bars.o_done, par, abort_flag));
        if (!alive) break;
        tc_fence_after();
        const bool in_range = k_r < T;
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
          // this row's V2 values for the chunk (shared by both tiles)
          float v2f[32];
#pragma unroll
          for (int i4 = 0; i4 < 4; ++i4) {
            const uint4 vv = in_range ? __ldg(reinterpret_cast<const uint4*>(V2g + (size_t)k_r * D + ch * 32 + i4 * 8))
                                      : make_uint4(0, 0, 0, 0);
            const uint32_t wv[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = unpack2<T16>(wv[e]);
              v2f[i4 * 8 + 2 * e] = f.x;
              v2f[i4 * 8 + 2 * e + 1] = f.y;
            }
          }
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            uint32_t o[32];
            tmem_ld32(tmem + lane_base + Cfg::kTmemO + x * D + ch * 32, o);
            tmem_wait_ld();
            if (ch == D / 32 - 1) {
              // last chunk of this tile's accumulator is in registers: it may be overwritten
              tc_fence_before();
              mbar_arrive(&bars.o_free[x]);
            }
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(o[i]) * (w[x] * v2f[i]);
            const float colsum = warp_transpose_sum(v, lane);
            red[(x * 4 + wq) * D + ch * 32 + lane] = colsum;
          }
        }
        if (!fold_sync()) { alive = false; break; }
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (!(Mt[x] > -INFINITY)) continue;   // nothing valid in this tile for this query
          const float Lt = fstat[x * 8 + 4] + fstat[x * 8 + 5] + fstat[x * 8 + 6] + fstat[x * 8 + 7];
          const float Mn = fmaxf(M_run[x], Mt[x]);
          const float ca = exp2f(M_run[x] - Mn), cb = exp2f(Mt[x] - Mn);
          if (row < D) {
            const float Ot = red[(x * 4) * D + row] + red[(x * 4 + 1) * D + row] + red[(x * 4 + 2) * D + row] +
                             red[(x * 4 + 3) * D + row];
            O_run[x] = O_run[x] * ca + Ot * cb;
          }
          L_run[x] = L_run[x] * ca + Lt * cb;
          M_run[x] = Mn;
        }
        if (!fold_sync()) { alive = false; break; }  // red / fstat are rewritten by the next k-tile
      }
      if (!alive) break;
      // ---- store the two output rows and their log-sum-exp
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        const int qx = x == 0 ? qa : qb;
        if (row < D) ((T16*)p.out)[((size_t)bh * T + qx) * D + row] = from_f<T16>(O_run[x] / L_run[x]);
        if (row == 0) p.lse[(size_t)bh * T + qx] = (M_run[x] + log2f(L_run[x])) * kLn2;
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
  if (tid == 0 && bars.abort_flag && p.status) atomicOr(p.status, 2);
}

// Per-head statistics behind the score bounds, over the rows r of the three [BN*T, D] tensors:
//   out[bh] = max_j |K1[bh, j, :]|^2,  out[BN + bh] = max_q |Q[bh, q, :]|^2,  out[2 BN + bh] = max element^2 of K2[bh]
// (fp32, compared as integers: non-negative floats order like their bit patterns).  A warp takes kStatRows
// consecutive rows and issues its three atomics once per head it met, not once per row.  `out` must be zero on entry.
constexpr int kStatRows = 8;
template <typename T16>
__global__ void head_stats_kernel(const T16* __restrict__ k1, const T16* __restrict__ q, const T16* __restrict__ k2,
                                  float* __restrict__ out, size_t rows, int T, int D, int BN) {
  const size_t w = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const size_t r0 = w * kStatRows;
  if (r0 >= rows) return;
  const size_t r1 = r0 + kStatRows < rows ? r0 + kStatRows : rows;
  float m1 = 0.f, mq = 0.f, m2 = 0.f;   // maxima over the rows of the current head
  size_t bh = r0 / T;
  auto flush = [&]() {
    if (lane == 0) {
      atomicMax(reinterpret_cast<int*>(out + bh), __float_as_int(m1));
      atomicMax(reinterpret_cast<int*>(out + BN + bh), __float_as_int(mq));
      atomicMax(reinterpret_cast<int*>(out + 2 * (size_t)BN + bh), __float_as_int(m2));
    }
  };
  for (size_t r = r0; r < r1; ++r) {
    if (r / T != bh) {
      flush();
      bh = r / T;
      m1 = mq = m2 = 0.f;
    }
    const uint32_t* s1 = reinterpret_cast<const uint32_t*>(k1 + r * D);
    const uint32_t* sq = reinterpret_cast<const uint32_t*>(q + r * D);
    const uint32_t* s2 = reinterpret_cast<const uint32_t*>(k2 + r * D);
    float n1 = 0.f, nq = 0.f, e2 = 0.f;
    for (int i = lane; i < D / 2; i += 32) {
      const float2 a = unpack2<T16>(s1[i]), b = unpack2<T16>(sq[i]), c = unpack2<T16>(s2[i]);
      n1 = fmaf(a.x, a.x, fmaf(a.y, a.y, n1));
      nq = fmaf(b.x, b.x, fmaf(b.y, b.y, nq));
      e2 = fmaxf(e2, fmaxf(c.x * c.x, c.y * c.y));
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
      n1 += __shfl_xor_sync(0xffffffffu, n1, o);
      nq += __shfl_xor_sync(0xffffffffu, nq, o);
      e2 = fmaxf(e2, __shfl_xor_sync(0xffffffffu, e2, o));
    }
    m1 = fmaxf(m1, n1);
    mq = fmaxf(mq, nq);
    m2 = fmaxf(m2, e2);
  }
  flush();
}

// What both forward kernels need before they start: SiLU(V1) in the inputs' type at the head of the workspace and,
// when the workspace has the optional tail, the per-head statistics of head_stats_kernel (for the score bounds; the
// returned pointer is to the first of its three arrays of B*N values, the K1 row norms).
template <typename T16>
int prepare_fwd(const TdpArgs& a, T16** sv1_out, float** k1n_out) {
  const int BN = a.B * a.N;
  const size_t n = (size_t)BN * a.T * a.D;
  T16* sv1 = (T16*)a.workspace;
  silu_kernel<T16><<<(unsigned)((n / 8 + 255) / 256 + 1), 256, 0, a.stream>>>((const T16*)a.v1, sv1, n);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  float* k1n = nullptr;
  const size_t tail = align_up(n * 2, 256);
  if (a.workspace_bytes >= tail + 3 * (size_t)BN * sizeof(float)) {
    k1n = reinterpret_cast<float*>((char*)a.workspace + tail);
    TRITT_CUDA_OK(cudaMemsetAsync(k1n, 0, 3 * (size_t)BN * sizeof(float), a.stream));
    const size_t rows = (size_t)BN * a.T;
    const size_t warps = (rows + kStatRows - 1) / kStatRows;
    head_stats_kernel<T16><<<(unsigned)((warps + 7) / 8), 256, 0, a.stream>>>((const T16*)a.k1, (const T16*)a.q,
                                                                             (const T16*)a.k2, k1n, rows, a.T, a.D, BN);
    count_launch();
    TRITT_CUDA_OK(cudaGetLastError());
  }
  *sv1_out = sv1;
  *k1n_out = k1n;
  return 0;
}

template <int D, typename T16>
int launch_fwd(const TdpArgs& a) {
  using Cfg = FwdCfg<D>;
  const int BN = a.B * a.N;
  T16* sv1 = nullptr;
  float* k1n = nullptr;
  int rc = prepare_fwd<T16>(a, &sv1, &k1n);
  if (rc) return rc;
  if (sm100_tdp_fwd_band_applies(a.T, a.mask)) return sm100_tdp_fwd_band(a, sv1, k1n);
  CUtensorMap tmK1, tmK2, tmSV1;
  if ((rc = make_tmap_3d(&tmK1, a.k1, 2, D, a.T, BN, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmSV1, sv1, 2, D, a.T, BN, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmK2, a.k2, 2, D, a.T, BN, 64, 128))) return rc;
  FwdParams p{};
  p.out = a.out_o;
  p.lse = a.out_lse;
  p.q = a.q;
  p.v2 = a.v2;
  p.T = a.T;
  p.BN = BN;
  p.q_mod = a.q_mod;
  p.q_rem = a.q_rem;
  p.nq = a.q_rem < a.T ? (a.T - a.q_rem + a.q_mod - 1) / a.q_mod : 0;
  p.n_pairs = (p.nq + 1) / 2;
  p.causal = a.mask.causal;
  p.k1w = a.mask.k1w;
  p.k2w = a.mask.k2w;
  p.kkl = a.mask.kkl;
  p.kkr = a.mask.kkr;
  p.scale2 = a.alpha * kLog2e;
  p.k1_norm2_max = k1n;
  p.q_norm2_max = k1n ? k1n + BN : nullptr;
  p.k2_elem2_max = k1n ? k1n + 2 * BN : nullptr;
  // P = exp2(S - bound) lies in [2^-2 bound, 1]: normal numbers of the 16-bit type (bf16 2^-126, fp16 2^-14)
  p.bound_limit = std::is_same<T16, __nv_bfloat16>::value ? 40.f : 6.f;
  p.status = a.status_word;
  if (p.nq == 0) return 0;
  auto kern = tdp_fwd_kernel<D, T16>;
  TRITT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
  const long items = (long)p.n_pairs * BN;
  const int grid = (int)(items < num_sms() ? items : num_sms());
  kern<<<grid, kThreads, Cfg::kSmem, a.stream>>>(tmK1, tmK2, tmSV1, p);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace


bool sm100_tdp_supported(int op, int T, int D, int dtype, const TdpMask& m) {
  if (op != TRITT_OP_TDP_FWD && op != TRITT_OP_TDP_BWD) return false;
  if (dtype != TRITT_BF16 && dtype != TRITT_F16) return false;
  if (D != 64 && D != 128) return false;
  (void)m;  // every window of the causal mask is handled
  return T >= 1;
}

// Extra bytes behind the forward's SiLU(V1) copy that enable the score bound (the forward runs without them too).
size_t sm100_tdp_fwd_optional_workspace(int B, int N, int T, int D, int dtype) {
  if (dtype != TRITT_BF16 && dtype != TRITT_F16) return 0;
  const size_t n = (size_t)B * N * T * D;
  return align_up(n * 2, 256) - n * 2 + align_up(3 * (size_t)B * N * sizeof(float), 256);
}

size_t sm100_tdp_workspace(int op, int B, int N, int T, int D, int dtype) {
  if (dtype != TRITT_BF16 && dtype != TRITT_F16) return 0;
  if (op == TRITT_OP_TDP_FWD) return (size_t)B * N * T * D * 2;
  if (op == TRITT_OP_TDP_BWD) return sm100_tdp_bwd_workspace(B, N, T, D);
  return 0;
}

int sm100_tdp_fwd(const TdpArgs& a) {
  // general kernel: the two queries of a pair must fall in the same 128-row block (the band kernel has no such rule)
  if (!sm100_tdp_fwd_band_applies(a.T, a.mask) && (a.q_mod < 1 || a.q_mod > 64 || (a.q_mod & (a.q_mod - 1)))) {
    set_error("tensor-core path needs a power-of-two query shard count <= 64 (got %d)", a.q_mod);
    return -30;
  }
  if (a.dtype == TRITT_BF16) return a.D == 128 ? launch_fwd<128, __nv_bfloat16>(a) : launch_fwd<64, __nv_bfloat16>(a);
  return a.D == 128 ? launch_fwd<128, __half>(a) : launch_fwd<64, __half>(a);
}

}  // namespace tritt
