// Triple-dot-product trittention forward for NARROW (j, k) BANDS on Blackwell tensor cores.
//
// With a causal mask whose band  k - kk_left <= j <= k + kk_right  is narrow (kk_left + kk_right <= 96), a K2 row k
// attends at most 97 K1 columns, and a query attends only k2_window + 1 rows.  The general forward kernel gives a
// whole 128-row tile to one query and walks 128-column slabs, most of which such a mask leaves empty.  Here a tile
// holds FOUR queries x 32 consecutive K2 rows instead,
//     row r = 32 g + i   <->   (query q_g, K2 row k_i = kb0 + i),        A[r,h] = alpha*log2(e) * Q[q_g,h] * K2[k_i,h],
// and the columns every row of the tile can attend, j in [max(kb0 - kk_left, q_0 - k1_window), min(q_last, kb0 + 31 +
// kk_right)], fit in ONE 128-column slab that starts at an arbitrary K1 row (TMA tiles need no row alignment).  A tile
// is therefore a single pass: S = A K1slab^T (tcgen05, accumulator in tensor memory), one soft-max per row, acc = P
// SiLU(V1)slab, and a fold that merges the 32 rows of each query (one warp per query) into that query's running
// (max, sum, output) across its k-blocks.  The reference lists this joint (j, k) band tiling as future work
// (b200/README.md:61-67) and benchmarks the case (b200/bench_b200.py:113: windows 128/128/32/32 at T = 2048).
//
// CTA layout (persistent, 512 threads), two tiles in flight (tile t uses slot t & 1 of every per-tile resource):
//   warp 0       TMA producer: the 32-row K2 and V2 blocks of a tile (four tiles ahead at head dimension 64), then its K1
//                and SiLU(V1) slabs into a ring of eight stages (four at head dimension 128)
//   warp 1       tcgen05.mma issuer: S(t), then P V of tile t - 1, so that a tile's soft-max overlaps its neighbour's products
//   warps 4-7    soft-max warpgroup of slot 0, warps 8-11 of slot 1 (one row per thread; they also form A)
//   warps 12-15  fold warpgroup: warp g owns query q_g (the V2 factor comes from the block in shared memory)
// The kernel is bound by the instruction issue of the soft-max and fold warps (a tile is 16 K exponentials with
// per-element column masks for ~12 M flop), not by the tensor pipe or by memory.
#include "tritt_common.cuh"
#include "tritt_sm100.cuh"
#include "tritt_sm100_tdp.cuh"

#include <type_traits>

namespace tritt {
namespace {
using namespace sm100;

constexpr int kBandThreads = 512;
constexpr int kGQ = 4;    // queries per tile
constexpr int kRK = 32;   // K2 rows per tile

template <int D> struct BandCfg {
  static constexpr int kTileA = 128 * D * 2;          // one 128-row operand / K1 / SiLU(V1) tile
  // K1 / SiLU(V1) slabs in flight: a tile is a short chain of dependent steps (fetch, operand, scores, soft-max,
  // values), so the fetches have to run several tiles ahead; head dimension 128 leaves room for four stages only
  static constexpr int kStages = D == 64 ? 8 : 4;
  static constexpr int kRawSlots = D == 64 ? 4 : 2;   // (K2, V2) blocks in flight
  static constexpr int kBlockBytes = kRK * D * 2;     // one 32-row block as loaded
  static constexpr int kRawBytes = 2 * kBlockBytes;   // the K2 block, then the V2 block of the same rows
  static constexpr int kOffA = 0;                     // A of slot 0, slot 1
  static constexpr int kOffRing = 2 * kTileA;
  static constexpr int kOffRaw = kOffRing + kStages * kTileA;   // (each slot a multiple of 4 KiB: 1024-aligned)
  static constexpr int kOffStats = kOffRaw + kRawSlots * kRawBytes;  // [2 slots][128][2] fp32: row (reference, sum)
  static constexpr int kOffBars = kOffStats + 2 * 128 * 2 * 4;
  static constexpr int kSmem = kOffBars + 384;
  static constexpr int kTmemAcc = 256;                // S_0 | S_1 | acc_0 | acc_1
};

struct BandParams {
  void* out;
  float* lse;
  const void* q;
  int T, BN, nq, q_mod, q_rem, n_groups;
  int k1w, k2w, kkl, kkr;
  float scale2;               // alpha * log2(e)
  const float* k1_norm2_max;  // [BN] largest squared K1 row norm per head, or null
  float bound_limit;
  int* status;
};

struct BandBarriers {
  uint64_t ring_full[8], ring_empty[8];
  uint64_t k2_full[4], raw_free[4];  // per (K2, V2) block slot (tile t uses slot t % kRawSlots)
  uint64_t a_ready[2], s_ready[2], p_ready[2], o_done[2], o_free[2], stats_ready[2];
  uint32_t tmem_base;
  int abort_flag;
};

// One tile of the walk: queries q_0 .. q_last of a group, the K2 block starting at kb0, the K1 slab starting at jlo.
struct BandTile {
  int bh, q0, count, kb0, jlo;
  bool first, last;  // first / last k-block of its query group
};

template <int D, typename T16>
__global__ void __launch_bounds__(kBandThreads, 1)
tdp_fwd_band_kernel(const __grid_constant__ CUtensorMap tmK1, const __grid_constant__ CUtensorMap tmK2b,
                    const __grid_constant__ CUtensorMap tmV2b, const __grid_constant__ CUtensorMap tmSV1, BandParams p) {
  using Cfg = BandCfg<D>;
  constexpr int NS = Cfg::kStages;
  constexpr int KH = D / 64;
  extern __shared__ __align__(1024) uint8_t smem[];
  static_assert(sizeof(BandBarriers) <= 384, "barrier block too large");
  BandBarriers& bars = *reinterpret_cast<BandBarriers*>(smem + Cfg::kOffBars);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (smem_u32(smem) & 1023u) {
    if (tid == 0 && p.status) atomicOr(p.status, 8);
    return;
  }
  if (tid == 0) {
    bars.abort_flag = 0;
    for (int i = 0; i < NS; ++i) {
      mbar_init(&bars.ring_full[i], 1);
      mbar_init(&bars.ring_empty[i], 1);
    }
    for (int r = 0; r < Cfg::kRawSlots; ++r) {
      mbar_init(&bars.k2_full[r], 1);
      mbar_init(&bars.raw_free[r], 256);  // the soft-max warpgroup (K2 block) and the fold warpgroup (V2 block)
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(&bars.a_ready[x], 128);
      mbar_init(&bars.s_ready[x], 1);
      mbar_init(&bars.p_ready[x], 128);
      mbar_init(&bars.o_done[x], 1);
      mbar_init(&bars.o_free[x], 128);
      mbar_init(&bars.stats_ready[x], 128);
    }
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
  const long n_items = (long)p.n_groups * p.BN;

  // Every role walks the same sequence of tiles: items blockIdx.x, blockIdx.x + gridDim.x, ...; inside an item
  // the k-blocks from the lowest attended K2 row upwards.
  struct Walk {
    long item;
    int b, nb, klo, q_first, q_last;
  };
  auto open_item = [&](Walk& w, BandTile& t) {
    t.bh = (int)(w.item % p.BN);
    const int grp = (int)(w.item / p.BN);
    const int idx0 = kGQ * grp;
    t.count = min(kGQ, p.nq - idx0);
    t.q0 = p.q_rem + idx0 * p.q_mod;
    w.q_first = t.q0;
    w.q_last = t.q0 + (t.count - 1) * p.q_mod;
    // K2 rows below max(q - k2w, q - k1w - kkr) see no column of any query of the group
    w.klo = max(0, max(w.q_first - p.k2w, w.q_first - p.k1w - p.kkr));
    w.nb = (w.q_last - w.klo) / kRK + 1;
    w.b = 0;
  };
  auto fill_tile = [&](const Walk& w, BandTile& t) {
    t.kb0 = w.klo + kRK * w.b;
    t.jlo = max(0, max(t.kb0 - p.kkl, w.q_first - p.k1w));
    t.first = w.b == 0;
    t.last = w.b == w.nb - 1;
  };
  // for (tile in walk) body(tile, t_index); body returns false to stop
  auto for_each_tile = [&](auto&& body) {
    Walk w;
    BandTile t;
    uint32_t ti = 0;
    for (w.item = blockIdx.x; w.item < n_items; w.item += gridDim.x) {
      open_item(w, t);
      for (; w.b < w.nb; ++w.b, ++ti) {
        fill_tile(w, t);
        if (!body(t, ti)) return;
      }
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmK1);
      tma_prefetch_desc(&tmK2b);
      tma_prefetch_desc(&tmV2b);
      tma_prefetch_desc(&tmSV1);
      uint32_t pos = 0;
      bool alive = true;
      auto load_stage = [&](const CUtensorMap* tm, int row0, int bh) -> bool {
        const int st = pos % NS;
        if (!mbar_wait(&bars.ring_empty[st], ((pos / NS) & 1) ^ 1, abort_flag)) return false;
        mbar_arrive_expect_tx(&bars.ring_full[st], Cfg::kTileA);
        for (int hh = 0; hh < KH; ++hh)
          tma_load_3d(smem + Cfg::kOffRing + st * Cfg::kTileA + hh * 16384, tm, &bars.ring_full[st], hh * 64, row0, bh);
        ++pos;
        return true;
      };
      for_each_tile([&](const BandTile& t, uint32_t ti) {
        const int rs = ti % Cfg::kRawSlots;
        const uint32_t ru = ti / Cfg::kRawSlots;
        // the block this slot held four tiles ago has been turned into its operand
        if (!mbar_wait(&bars.raw_free[rs], (ru & 1) ^ 1, abort_flag)) return alive = false;
        mbar_arrive_expect_tx(&bars.k2_full[rs], Cfg::kRawBytes);
        for (int hh = 0; hh < KH; ++hh) {
          uint8_t* dst = smem + Cfg::kOffRaw + rs * Cfg::kRawBytes + hh * (kRK * 128);
          tma_load_3d(dst, &tmK2b, &bars.k2_full[rs], hh * 64, t.kb0, t.bh);
          tma_load_3d(dst + Cfg::kBlockBytes, &tmV2b, &bars.k2_full[rs], hh * 64, t.kb0, t.bh);
        }
        if (!load_stage(&tmK1, t.jlo, t.bh)) return alive = false;
        if (!load_stage(&tmSV1, t.jlo, t.bh)) return alive = false;
        return true;
      });
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
    // (the whole warp walks the schedule converged and one elected lane issues: the descriptor arithmetic stays on
    //  the uniform datapath)
    {
      const bool leader = elect_one();
      auto wait_all = [&](uint64_t* bar, uint32_t parity) {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
      };
      auto commit = [&](uint64_t* bar) {
        if (leader) mma_commit(bar);
      };
      constexpr int kFmt = std::is_same<T16, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_s = make_idesc_f16(128, 128, kFmt, false, false);
      constexpr uint32_t idesc_pv = make_idesc_f16(128, D, kFmt, false, true);
      constexpr uint32_t kHi = desc_hi(1024);
      constexpr uint32_t kTile16 = Cfg::kTileA >> 4;
      const uint32_t aLo[2] = {desc_lo(smem_u32(smem + Cfg::kOffA), 16), desc_lo(smem_u32(smem + Cfg::kOffA + Cfg::kTileA), 16)};
      const uint32_t ringK = desc_lo(smem_u32(smem + Cfg::kOffRing), 16);      // K-major view of a stage
      const uint32_t ringMN = desc_lo(smem_u32(smem + Cfg::kOffRing), 16384);  // row-major (MN-major) view
      bool alive = true;
      uint32_t n_tiles = 0;
      // acc_x = P_x * SiLU(V1)slab for tile tt (P_x overlays the first 64 columns of S_x)
      auto issue_pv = [&](uint32_t tt) -> bool {
        const int x = tt & 1;
        const uint32_t u = tt >> 1, pos = 2 * tt + 1;
        if (!wait_all(&bars.p_ready[x], u & 1)) return false;
        // the fold warpgroup must have drained this slot's accumulator of two tiles ago
        if (!wait_all(&bars.o_free[x], (u & 1) ^ 1)) return false;
        if (!wait_all(&bars.ring_full[pos % NS], (pos / NS) & 1)) return false;
        tc_fence_after();
        const uint32_t bLo = ringMN + (pos % NS) * kTile16;
        // (always the full chain of 8: columns of P beyond the attended range are zero, and a loop with a run-time
        //  bound costs the issuing thread more than the skipped instructions save)
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (leader) mma_ts_lo(tmem + Cfg::kTmemAcc + x * D, tmem + x * 128 + k * 8, bLo + k * (2048 >> 4), kHi, idesc_pv, k > 0);
        commit(&bars.o_done[x]);
        commit(&bars.ring_empty[pos % NS]);
        return true;
      };
      for_each_tile([&](const BandTile& t, uint32_t ti) {
        const int x = ti & 1;
        const uint32_t u = ti >> 1, pos = 2 * ti;
        if (!wait_all(&bars.a_ready[x], u & 1)) return alive = false;
        if (!wait_all(&bars.ring_full[pos % NS], (pos / NS) & 1)) return alive = false;
        tc_fence_after();
        const uint32_t bLo = ringK + (pos % NS) * kTile16;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t kk = (k >> 2) * (16384 >> 4) + (k & 3) * 2;
          if (leader) mma_ss_lo(tmem + x * 128, aLo[x] + kk, bLo + kk, kHi, idesc_s, k > 0);
        }
        commit(&bars.s_ready[x]);
        commit(&bars.ring_empty[pos % NS]);
        if (ti > 0 && !issue_pv(ti - 1)) return alive = false;
        n_tiles = ti + 1;
        return true;
      });
      if (alive && n_tiles > 0) issue_pv(n_tiles - 1);
    }
  } else if (warp >= 4 && warp < 12) {
    // ------------------------------------------------------------------ soft-max warpgroups
    const int x = (warp - 4) >> 2;  // slot served by this warpgroup
    const int g = warp & 3;         // query of the group owned by this warp (= TMEM lane quadrant)
    const int row = g * 32 + lane;
    const uint32_t lane_base = (uint32_t)(g * 32) << 16;
    const uint32_t tS = tmem + lane_base + x * 128;
    float* stats = (float*)(smem + Cfg::kOffStats) + x * 256;
    uint8_t* Ax = smem + Cfg::kOffA + x * Cfg::kTileA;
    bool alive = true;
    for_each_tile([&](const BandTile& t, uint32_t ti) {
      if ((int)(ti & 1) != x) return true;
      const uint32_t u = ti >> 1;
      const int q_g = t.q0 + g * p.q_mod, k_i = t.kb0 + lane;
      const bool q_ok = g < t.count;
      const T16* Qrow = (const T16*)p.q + ((size_t)t.bh * T + (q_ok ? q_g : t.q0)) * D;
      // ---- operand formation: A[r, :] = s * Q[q_g, :] (.) K2[k_i, :]   (this thread's whole row)
      const int rs = ti % Cfg::kRawSlots;
      const uint8_t* raw = smem + Cfg::kOffRaw + rs * Cfg::kRawBytes;
      alive = __all_sync(0xffffffffu, mbar_wait(&bars.k2_full[rs], (ti / Cfg::kRawSlots) & 1, abort_flag));
      if (!alive) return false;
      // (the operand buffer is free: this warpgroup has waited for the slot's previous score product, below)
      float nrm = 0.f;
#pragma unroll
      for (int cc = 0; cc < D / 8; ++cc) {
        const int hh = cc >> 3, c = cc & 7;
        const uint4 kv = *reinterpret_cast<const uint4*>(raw + hh * (kRK * 128) + swz128(lane, c));
        const uint4 qv = __ldg(reinterpret_cast<const uint4*>(Qrow + cc * 8));
        const uint32_t wk[4] = {kv.x, kv.y, kv.z, kv.w}, wq[4] = {qv.x, qv.y, qv.z, qv.w};
        uint32_t oa[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 fk = unpack2<T16>(wk[e]), fq = unpack2<T16>(wq[e]);
          const float a0 = fk.x * p.scale2 * fq.x, a1 = fk.y * p.scale2 * fq.y;
          nrm = fmaf(a0, a0, fmaf(a1, a1, nrm));
          oa[e] = pack2<T16>(a0, a1);
        }
        *reinterpret_cast<uint4*>(Ax + hh * 16384 + swz128(row, c)) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
      }
      fence_async_smem();
      mbar_arrive(&bars.a_ready[x]);
      mbar_arrive(&bars.raw_free[rs]);  // the K2 block is consumed
      // columns this row attends: [c_lo, c_hi] (empty for a row outside its query's K2 range)
      const bool in_k = q_ok && k_i <= q_g && q_g - k_i <= p.k2w;
      const int c_lo = max(q_g - p.k1w, k_i - p.kkl);
      const int c_hi = in_k ? min(q_g, k_i + p.kkr) : c_lo - 1;
      const int lo = c_lo - t.jlo, hi = c_hi - t.jlo;
      const float k1_max = p.k1_norm2_max ? sqrtf(__ldg(p.k1_norm2_max + t.bh)) : INFINITY;

      alive = __all_sync(0xffffffffu, mbar_wait(&bars.s_ready[x], u & 1, abort_flag));
      if (!alive) return false;
      tc_fence_after();
      // Score bound of the row, |A_row| max_j |K1_j| (log2 units): where it is small for the whole warp it serves as
      // the soft-max reference (P stays a normal number of the 16-bit type) and the row-maximum pass is skipped.
      const float bound = sqrtf(nrm) * k1_max;
      const bool fast = __all_sync(0xffffffffu, bound <= p.bound_limit);
      const bool full = __all_sync(0xffffffffu, lo <= 0 && hi >= 127);
      // 32-column chunks no row of the warp attends are not read at all (the band leaves a quarter of the slab empty)
      int wlo = lo, whi = hi;
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) {
        wlo = min(wlo, __shfl_xor_sync(0xffffffffu, wlo, o));
        whi = max(whi, __shfl_xor_sync(0xffffffffu, whi, o));
      }
      float m_used = bound;
      if (!fast) {
        float mx = -INFINITY;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          if (ch * 32 + 31 < wlo || ch * 32 > whi) continue;
          uint32_t sr[32];
          tmem_ld32(tS + ch * 32, sr);
          tmem_wait_ld();
          const int l2 = lo - ch * 32, h2 = hi - ch * 32;
#pragma unroll
          for (int c = 0; c < 32; ++c)
            if (c >= l2 && c <= h2) mx = fmaxf(mx, __uint_as_float(sr[c]));
        }
        m_used = mx;  // -inf for a row that attends nothing: every P below is then selected to 0
      }
      float psum = 0.f;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t pk[16];
        if (ch * 32 + 31 < wlo || ch * 32 > whi) {
#pragma unroll
          for (int c = 0; c < 16; ++c) pk[c] = 0u;
        } else {
          uint32_t sr[32];
          tmem_ld32(tS + ch * 32, sr);
          tmem_wait_ld();
          if (full) {
            float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
              const float p0 = exp2f(__uint_as_float(sr[c]) - m_used);
              const float p1 = exp2f(__uint_as_float(sr[c + 1]) - m_used);
              ps0 += p0;
              ps1 += p1;
              pk[c >> 1] = pack2<T16>(p0, p1);
            }
            psum += ps0 + ps1;
          } else {
            const int l2 = lo - ch * 32, h2 = hi - ch * 32;
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
              const float p0 = (c >= l2 && c <= h2) ? exp2f(__uint_as_float(sr[c]) - m_used) : 0.f;
              const float p1 = (c + 1 >= l2 && c + 1 <= h2) ? exp2f(__uint_as_float(sr[c + 1]) - m_used) : 0.f;
              psum += p0 + p1;
              pk[c >> 1] = pack2<T16>(p0, p1);
            }
          }
        }
        // P chunk ch -> columns [16 ch, 16 ch + 16) of S_x, which the chunks before have already read
        tmem_st16(tS + ch * 16, pk);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&bars.p_ready[x]);
      // row statistics for the fold; the slot's previous statistics must have been read (same hand-off as the
      // accumulator's: the fold arrives on o_free after it has taken both)
      alive = __all_sync(0xffffffffu, mbar_wait(&bars.o_free[x], (u & 1) ^ 1, abort_flag));
      if (!alive) return false;
      stats[row * 2] = m_used;
      stats[row * 2 + 1] = psum;
      mbar_arrive(&bars.stats_ready[x]);
      return true;
    });
  } else if (warp >= 12) {
    // ------------------------------------------------------------------ fold warpgroup: warp g owns query q_g
    const int g = warp & 3;
    const int row = g * 32 + lane;
    const uint32_t lane_base = (uint32_t)(g * 32) << 16;
    bool alive = true;
    float M_run = -INFINITY, L_run = 0.f, O_run[D / 32];
    for_each_tile([&](const BandTile& t, uint32_t ti) {
      const int x = ti & 1;
      const uint32_t u = ti >> 1;
      if (t.first) {
        M_run = -INFINITY;
        L_run = 0.f;
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) O_run[ch] = 0.f;
      }
      const int q_g = t.q0 + g * p.q_mod, k_i = t.kb0 + lane;
      const bool q_ok = g < t.count;
      const bool valid = q_ok && k_i <= q_g && q_g - k_i <= p.k2w;
      alive = __all_sync(0xffffffffu, mbar_wait(&bars.stats_ready[x], u & 1, abort_flag));
      if (!alive) return false;
      const float* st = (const float*)(smem + Cfg::kOffStats) + x * 256 + row * 2;
      const float m_r = st[0], l_r = st[1];
      // rows without attended mass do not take part (and do not set the reference)
      const bool live = valid && l_r > 0.f;
      float Mt = live ? m_r : -INFINITY;
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) Mt = fmaxf(Mt, __shfl_xor_sync(0xffffffffu, Mt, o));
      const float w = live ? exp2f(m_r - Mt) : 0.f;
      float Lt = w * l_r;
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) Lt += __shfl_xor_sync(0xffffffffu, Lt, o);
      alive = __all_sync(0xffffffffu, mbar_wait(&bars.o_done[x], u & 1, abort_flag));
      if (!alive) return false;
      tc_fence_after();
      // the V2 rows of the block came in with its K2 rows (the fetch completed before the operand was formed)
      const int rs = ti % Cfg::kRawSlots;
      const uint8_t* v2blk = smem + Cfg::kOffRaw + rs * Cfg::kRawBytes + Cfg::kBlockBytes;
      float Ot[D / 32];
#pragma unroll
      for (int ch = 0; ch < D / 32; ++ch) {
        uint32_t o[32];
        tmem_ld32(tmem + lane_base + Cfg::kTmemAcc + x * D + ch * 32, o);
        float v[32];
#pragma unroll
        for (int i4 = 0; i4 < 4; ++i4) {
          const int cc = ch * 4 + i4;  // 16-byte chunk of the row
          const uint4 vv = *reinterpret_cast<const uint4*>(v2blk + (cc >> 3) * (kRK * 128) + swz128(lane, cc & 7));
          const uint32_t wv[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = unpack2<T16>(wv[e]);
            v[i4 * 8 + 2 * e] = f.x * w;
            v[i4 * 8 + 2 * e + 1] = f.y * w;
          }
        }
        tmem_wait_ld();
        if (ch == D / 32 - 1) {
          // the accumulator and the statistics of this slot are in registers: both may be overwritten, and so may
          // the block slot (its V2 rows have been read)
          tc_fence_before();
          mbar_arrive(&bars.o_free[x]);
          mbar_arrive(&bars.raw_free[rs]);
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= __uint_as_float(o[i]);
        Ot[ch] = warp_transpose_sum(v, lane);  // lane i: column ch*32 + i summed over the warp's 32 rows
      }
      if (Mt > -INFINITY) {
        const float Mn = fmaxf(M_run, Mt);
        const float ca = exp2f(M_run - Mn), cb = exp2f(Mt - Mn);
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) O_run[ch] = O_run[ch] * ca + Ot[ch] * cb;
        L_run = L_run * ca + Lt * cb;
        M_run = Mn;
      }
      if (t.last && q_ok) {
        T16* orow = (T16*)p.out + ((size_t)t.bh * T + q_g) * D;
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) orow[ch * 32 + lane] = from_f<T16>(O_run[ch] / L_run);
        if (lane == 0) p.lse[(size_t)t.bh * T + q_g] = (M_run + log2f(L_run)) * kLn2;
      }
      return true;
    });
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
  if (tid == 0 && bars.abort_flag && p.status) atomicOr(p.status, 2);
}

template <int D, typename T16>
int launch_band(const TdpArgs& a, const void* sv1, const float* k1n) {
  using Cfg = BandCfg<D>;
  const int BN = a.B * a.N;
  CUtensorMap tmK1, tmK2b, tmV2b, tmSV1;
  int rc;
  if ((rc = make_tmap_3d(&tmK1, a.k1, 2, D, a.T, BN, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmSV1, sv1, 2, D, a.T, BN, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmK2b, a.k2, 2, D, a.T, BN, 64, kRK))) return rc;
  if ((rc = make_tmap_3d(&tmV2b, a.v2, 2, D, a.T, BN, 64, kRK))) return rc;
  BandParams p{};
  p.out = a.out_o;
  p.lse = a.out_lse;
  p.q = a.q;
  p.T = a.T;
  p.BN = BN;
  p.q_mod = a.q_mod;
  p.q_rem = a.q_rem;
  p.nq = a.q_rem < a.T ? (a.T - a.q_rem + a.q_mod - 1) / a.q_mod : 0;
  p.n_groups = (p.nq + kGQ - 1) / kGQ;
  p.k1w = a.mask.k1w;
  p.k2w = a.mask.k2w;
  p.kkl = a.mask.kkl;
  p.kkr = a.mask.kkr;
  p.scale2 = a.alpha * kLog2e;
  p.k1_norm2_max = k1n;
  p.bound_limit = std::is_same<T16, __nv_bfloat16>::value ? 40.f : 6.f;
  p.status = a.status_word;
  if (p.nq == 0) return 0;
  auto kern = tdp_fwd_band_kernel<D, T16>;
  TRITT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
  const long items = (long)p.n_groups * BN;
  const int grid = (int)(items < num_sms() ? items : num_sms());
  kern<<<grid, kBandThreads, Cfg::kSmem, a.stream>>>(tmK1, tmK2b, tmV2b, tmSV1, p);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace

// The band kernel serves causal masks whose (j, k) band fits its one-slab tiles (32 K2 rows + the band <= 128 columns);
// short sequences stay on the general kernel, whose single 128-row tile already covers them.
bool sm100_tdp_fwd_band_applies(int T, const TdpMask& m) {
  return m.causal && T > 128 && m.kkl + m.kkr <= 128 - kRK;
}

// `sv1`: SiLU(V1) in the inputs' type; `k1n`: per-head largest squared K1 row norm, or null (both prepared by the caller).
int sm100_tdp_fwd_band(const TdpArgs& a, const void* sv1, const float* k1n) {
  if (a.dtype == TRITT_BF16)
    return a.D == 128 ? launch_band<128, __nv_bfloat16>(a, sv1, k1n) : launch_band<64, __nv_bfloat16>(a, sv1, k1n);
  return a.D == 128 ? launch_band<128, __half>(a, sv1, k1n) : launch_band<64, __half>(a, sv1, k1n);
}

}  // namespace tritt
