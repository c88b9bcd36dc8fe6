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
// One CTA (persistent, 384 threads) processes a pair of queries (qa, qb) of the same
// 64-row block as two concurrent row tiles that share every K1 / SiLU(V1) tile:
//   warp 0      TMA producer: K2/V2 tile per k-tile, then a ring of 64-row K1 and SiLU(V1) tiles
//   warp 1      issues tcgen05.mma: S = A*K1^T (operands in shared memory) into a
//               double-buffered 128x64 fp32 TMEM slab per tile, and acc += P*SiLU(V1) with P
//               read from TMEM and the value tile used row-major (MN-major descriptor)
//   warps 4-7   soft-max warpgroup of tile a (one row per thread), warps 8-11 of tile b:
//               exp2 with lazy rescaling, P written back to TMEM as 16-bit, per-k-tile
//               fold into the query's running (max, sum, output) and the final store.
// Causal structure: for a fixed query the mask is "j <= q" on columns and "k <= q" on rows, so
// whole j-tiles above q are never visited, only the last j-tile is masked (by a column bound that
// is uniform over the rows), and rows with k > q get weight zero in the fold.
#include "tritt_common.cuh"
#include "tritt_sm100.cuh"
#include "tritt_sm100_tdp.cuh"

#include <type_traits>

namespace tritt {
namespace {
using namespace sm100;

constexpr int kThreads = 384;
constexpr int kBJ = 64;           // key columns per MMA slab
constexpr float kRescaleGap = 8.f;  // rescale the accumulator only when the row max grew by more than 2^8

template <int D> struct FwdCfg {
  static constexpr int kTileA = 128 * D * 2;    // bytes of one 128-row operand tile
  static constexpr int kStage = kBJ * D * 2;    // bytes of one 64-row K1 / SiLU(V1) tile
  static constexpr int kStages = D == 128 ? 6 : 8;
  static constexpr int kOffAa = 0;
  static constexpr int kOffAb = kTileA;
  static constexpr int kOffV2 = 2 * kTileA;
  static constexpr int kOffRing = 3 * kTileA;
  static constexpr int kOffRed = kOffRing + kStages * kStage;  // [2][4][D] fp32 cross-warp sums
  static constexpr int kOffStat = kOffRed + 2 * 4 * D * 4;    // [2][8] fp32 cross-warp max / sum
  static constexpr int kSmem = kOffStat + 2 * 8 * 4 + 1024;   // + alignment slack
  static constexpr int kTmemO = 256;                          // accumulators start after the 4 score slabs
};

struct FwdParams {
  void* out;
  float* lse;
  const void* q;
  int T, BN, nq, q_mod, q_rem, causal, n_pairs;
  float scale2;  // alpha * log2(e)
  int* status;
};

struct Barriers {
  uint64_t ring_full[8], ring_empty[8];
  uint64_t k2_full, a_ready, a_free;
  uint64_t s_ready[2][2], p_ready[2][2], pv_done[2], wg_sync[2];
  uint32_t tmem_base;
  int abort_flag;
};

template <int D, typename T16>
__global__ void __launch_bounds__(kThreads, 1)
tdp_fwd_kernel(const __grid_constant__ CUtensorMap tmK1, const __grid_constant__ CUtensorMap tmK2,
               const __grid_constant__ CUtensorMap tmSV1, const __grid_constant__ CUtensorMap tmV2, FwdParams p) {
  using Cfg = FwdCfg<D>;
  constexpr int NS = Cfg::kStages;
  constexpr int KH = D / 64;  // 64-column halves per row
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ Barriers bars;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

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
      for (int b = 0; b < 2; ++b) {
        mbar_init(&bars.s_ready[x][b], 1);
        mbar_init(&bars.p_ready[x][b], 128);
      }
      mbar_init(&bars.pv_done[x], 1);
      mbar_init(&bars.wg_sync[x], 128);
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
  const long n_items = (long)p.n_pairs * p.BN;

  // Work item -> (head, query pair).  Items are ordered by decreasing cost (late queries first).
  auto decode = [&](long item, int& bh, int& qa, int& qb) {
    const int pr = p.n_pairs - 1 - (int)(item / p.BN);
    bh = (int)(item % p.BN);
    const int ia = 2 * pr, ib = min(2 * pr + 1, p.nq - 1);
    qa = p.q_rem + ia * p.q_mod;
    qb = p.q_rem + ib * p.q_mod;
  };
  auto tile_counts = [&](int qa, int qb, int& nkt, int& njt) {
    const int qmax = max(qa, qb);
    nkt = p.causal ? qmax / 128 + 1 : (T + 127) / 128;
    njt = p.causal ? qmax / kBJ + 1 : (T + kBJ - 1) / kBJ;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmK1);
      tma_prefetch_desc(&tmK2);
      tma_prefetch_desc(&tmSV1);
      tma_prefetch_desc(&tmV2);
      uint32_t kt_count = 0, pos = 0;
      bool alive = true;
      auto load_stage = [&](const CUtensorMap* tm, int row0, int bh) -> bool {
        const int st = pos % NS;
        if (!mbar_wait(&bars.ring_empty[st], ((pos / NS) & 1) ^ 1, abort_flag)) return false;
        mbar_arrive_expect_tx(&bars.ring_full[st], Cfg::kStage);
        for (int hh = 0; hh < KH; ++hh)
          tma_load_3d(smem + Cfg::kOffRing + st * Cfg::kStage + hh * (kBJ * 128), tm, &bars.ring_full[st], hh * 64,
                      row0, bh);
        ++pos;
        return true;
      };
      for (long item = blockIdx.x; item < n_items && alive; item += gridDim.x) {
        int bh, qa, qb, nkt, njt;
        decode(item, bh, qa, qb);
        tile_counts(qa, qb, nkt, njt);
        for (int kt = 0; kt < nkt && alive; ++kt, ++kt_count) {
          // the first K1 tiles do not depend on the previous k-tile being folded: fetch them first
          alive = load_stage(&tmK1, 0, bh);
          if (alive && njt > 1) alive = load_stage(&tmK1, kBJ, bh);
          if (!alive || !mbar_wait(&bars.a_free, (kt_count & 1) ^ 1, abort_flag)) { alive = false; break; }
          mbar_arrive_expect_tx(&bars.k2_full, 2 * Cfg::kTileA);
          for (int hh = 0; hh < KH; ++hh) {
            tma_load_3d(smem + Cfg::kOffAa + hh * 16384, &tmK2, &bars.k2_full, hh * 64, kt * 128, bh);
            tma_load_3d(smem + Cfg::kOffV2 + hh * 16384, &tmV2, &bars.k2_full, hh * 64, kt * 128, bh);
          }
          for (int jt = 0; jt < njt && alive; ++jt) {
            alive = load_stage(&tmSV1, jt * kBJ, bh);
            if (alive && jt + 2 < njt) alive = load_stage(&tmK1, (jt + 2) * kBJ, bh);
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
    if (lane == 0) {
      constexpr int kFmt = std::is_same<T16, __nv_bfloat16>::value ? 1 : 0;
      constexpr uint32_t idesc_s = make_idesc_f16(128, kBJ, kFmt, false, false);
      constexpr uint32_t idesc_pv = make_idesc_f16(128, D, kFmt, false, true);
      // descriptor low words; per instruction only a constant (in 16-byte units) is added
      constexpr uint32_t kHi = desc_hi(1024);
      constexpr uint32_t kStage16 = Cfg::kStage >> 4;
      const uint32_t aLo[2] = {desc_lo(smem_u32(smem + Cfg::kOffAa), 16), desc_lo(smem_u32(smem + Cfg::kOffAb), 16)};
      const uint32_t ringK = desc_lo(smem_u32(smem + Cfg::kOffRing), 16);          // K-major view of a stage
      const uint32_t ringMN = desc_lo(smem_u32(smem + Cfg::kOffRing), kBJ * 128);  // row-major (MN-major) view
      uint32_t kt_count = 0, base = 0, n = 0;  // n: score slabs issued per tile so far
      bool alive = true;
      // S_x(slab) = A_x * K1tile^T
      auto issue_s = [&](int x, uint32_t slab_n, uint32_t pos) {
        const uint32_t bLo = ringK + (pos % NS) * kStage16;
        const uint32_t d = tmem + (x * 2 + (slab_n & 1)) * kBJ;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ka = (k >> 2) * (16384 >> 4) + (k & 3) * 2, kb = (k >> 2) * ((kBJ * 128) >> 4) + (k & 3) * 2;
          mma_ss_lo(d, aLo[x] + ka, bLo + kb, kHi, idesc_s, k > 0);
        }
        mma_commit(&bars.s_ready[x][slab_n & 1]);
      };
      // acc_x (+)= P_x(slab) * SiLU(V1)tile
      auto issue_pv = [&](int x, uint32_t slab_n, uint32_t pos, bool accumulate) {
        const uint32_t bLo = ringMN + (pos % NS) * kStage16;
        const uint32_t a = tmem + (x * 2 + (slab_n & 1)) * kBJ;
        const uint32_t d = tmem + Cfg::kTmemO + x * D;
        const uint32_t acc = accumulate ? 1u : 0u;
#pragma unroll
        for (int k = 0; k < kBJ / 16; ++k) mma_ts_lo(d, a + k * 8, bLo + k * (2048 >> 4), kHi, idesc_pv, k > 0 ? 1u : acc);
        mma_commit(&bars.pv_done[x]);
      };
      auto wait_full = [&](uint32_t pos) { return mbar_wait(&bars.ring_full[pos % NS], (pos / NS) & 1, abort_flag); };
      auto release = [&](uint32_t pos) { mma_commit(&bars.ring_empty[pos % NS]); };

      for (long item = blockIdx.x; item < n_items && alive; item += gridDim.x) {
        int bh, qa, qb, nkt, njt;
        decode(item, bh, qa, qb);
        tile_counts(qa, qb, nkt, njt);
        for (int kt = 0; kt < nkt && alive; ++kt, ++kt_count) {
          if (!mbar_wait(&bars.a_ready, kt_count & 1, abort_flag)) { alive = false; break; }
          tc_fence_after();
          uint32_t pos = base;
          const uint32_t n0 = n;
          // first two score slabs of both tiles
          if (!wait_full(pos)) { alive = false; break; }
          issue_s(0, n0, pos);
          issue_s(1, n0, pos);
          release(pos);
          ++pos;
          if (njt > 1) {
            if (!wait_full(pos)) { alive = false; break; }
            issue_s(0, n0 + 1, pos);
            issue_s(1, n0 + 1, pos);
            release(pos);
            ++pos;
          }
          for (int jt = 0; jt < njt && alive; ++jt) {
            const uint32_t pv = pos++;
            const bool more = jt + 2 < njt;
            const uint32_t pk = more ? pos++ : 0;
            const uint32_t sn = n0 + jt;
            for (int x = 0; x < 2 && alive; ++x) {
              if (!mbar_wait(&bars.p_ready[x][sn & 1], (sn >> 1) & 1, abort_flag)) { alive = false; break; }
              tc_fence_after();
              if (x == 0) {
                if (!wait_full(pv)) { alive = false; break; }
              }
              issue_pv(x, sn, pv, jt > 0);
              if (x == 1) release(pv);
              if (more) {
                if (x == 0) {
                  if (!wait_full(pk)) { alive = false; break; }
                }
                issue_s(x, sn + 2, pk);
                if (x == 1) release(pk);
              }
            }
          }
          n = n0 + njt;
          base = pos;
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ soft-max warpgroups
    const int x = (warp - 4) >> 2;          // tile: 0 = query a, 1 = query b
    const int wq = warp & 3;                // TMEM lane quadrant of this warp
    const int row = wq * 32 + lane;         // row of the tile owned by this thread
    const int st = tid - 128;               // 0..255 over both warpgroups
    const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
    float* red = (float*)(smem + Cfg::kOffRed) + x * 4 * D;
    float* stat = (float*)(smem + Cfg::kOffStat) + x * 8;
    uint32_t kt_count = 0, n = 0, wg_phase = 0;
    bool alive = true;
    // warpgroup-wide rendezvous with a bounded wait
    auto wg_sync = [&]() -> bool {
      mbar_arrive(&bars.wg_sync[x]);
      const bool ok = mbar_wait(&bars.wg_sync[x], wg_phase & 1, abort_flag);
      ++wg_phase;
      return __all_sync(0xffffffffu, ok);
    };

    for (long item = blockIdx.x; item < n_items && alive; item += gridDim.x) {
      int bh, qa, qb, nkt, njt;
      decode(item, bh, qa, qb);
      tile_counts(qa, qb, nkt, njt);
      const int qx = x == 0 ? qa : qb;
      const T16* Qg = (const T16*)p.q + (size_t)bh * T * D;
      // running state of the query's output; thread `row` of the warpgroup owns column h = row
      float M_run = -INFINITY, L_run = 0.f, O_run = 0.f;

      for (int kt = 0; kt < nkt && alive; ++kt, ++kt_count) {
        // ---- operand formation: A_a = s*Q[qa] (.) K2tile (in place), A_b = s*Q[qb] (.) K2tile
        alive = __all_sync(0xffffffffu, mbar_wait(&bars.k2_full, kt_count & 1, abort_flag));
        if (!alive) break;
        {
          const int r = st & 127;
          constexpr int CPT = D / 16;  // 16-byte chunks per thread
          const int c0 = (st >> 7) * CPT;
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
              oa[e] = pack2<T16>(k0 * fa.x, k1v * fa.y);
              ob[e] = pack2<T16>(k0 * fb.x, k1v * fb.y);
            }
            *reinterpret_cast<uint4*>(smem + Cfg::kOffAa + off) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
            *reinterpret_cast<uint4*>(smem + Cfg::kOffAb + off) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
          }
        }
        fence_async_smem();   // generic-proxy stores above -> visible to the tensor core's reads
        tc_fence_before();    // this thread's TMEM loads of the previous fold precede the next MMAs
        mbar_arrive(&bars.a_ready);

        // ---- walk over the j-tiles
        float m_used = -INFINITY, l_sum = 0.f;
        for (int jt = 0; jt < njt; ++jt, ++n) {
          const uint32_t buf = n & 1;
          alive = __all_sync(0xffffffffu, mbar_wait(&bars.s_ready[x][buf], (n >> 1) & 1, abort_flag));
          if (!alive) break;
          tc_fence_after();
          const uint32_t tS = tmem + lane_base + (x * 2 + buf) * kBJ;
          uint32_t sr[64];
          tmem_ld64(tS, sr);
          tmem_wait_ld();
          // column bound: j <= q (causal) / j < T
          const int cmax = (p.causal ? qx : T - 1) - jt * kBJ;
          if (cmax < kBJ - 1) {
#pragma unroll
            for (int c = 0; c < kBJ; ++c)
              if (c > cmax) sr[c] = 0xff800000u;  // -inf
          }
          float mx = __uint_as_float(sr[0]);
#pragma unroll
          for (int c = 1; c < kBJ; ++c) mx = fmaxf(mx, __uint_as_float(sr[c]));
          if (jt == 0) {
            m_used = mx;  // nothing accumulated yet in this k-tile
          } else {
            const bool grow = mx > m_used + kRescaleGap;
            if (__any_sync(0xffffffffu, grow)) {
              // some row of this warp moved its max up noticeably: rescale accumulator rows (factor 1
              // for the rows that did not move).  The previous P*V must have landed first.
              const float corr = grow ? exp2f(m_used - mx) : 1.f;
              if (grow) {
                m_used = mx;
                l_sum *= corr;
              }
              alive = __all_sync(0xffffffffu, mbar_wait(&bars.pv_done[x], (n - 1) & 1, abort_flag));
              if (!alive) break;
              tc_fence_after();
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
          float psum = 0.f;
          uint32_t pk[32];
#pragma unroll
          for (int c = 0; c < kBJ; c += 2) {
            const float p0 = exp2f(__uint_as_float(sr[c]) - m_used), p1 = exp2f(__uint_as_float(sr[c + 1]) - m_used);
            psum += p0 + p1;
            pk[c >> 1] = pack2<T16>(p0, p1);
          }
          l_sum += psum;
          if (jt > 0) {
            // Observe every completion of pv_done in order (a parity wait must never fall two
            // phases behind); by now the previous P*V has normally long finished.
            alive = __all_sync(0xffffffffu, mbar_wait(&bars.pv_done[x], (n - 1) & 1, abort_flag));
            if (!alive) break;
          }
          tmem_st32(tS, pk);
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(&bars.p_ready[x][buf]);
        }
        if (!alive) break;

        // ---- fold this k-tile into the query's running output
        alive = __all_sync(0xffffffffu, mbar_wait(&bars.pv_done[x], (n - 1) & 1, abort_flag));
        if (!alive) break;
        tc_fence_after();
        const int k_r = kt * 128 + row;
        const bool valid = p.causal ? (k_r <= qx) : (k_r < T);
        float wm = valid ? m_used : -INFINITY;
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, o));
        if (lane == 0) stat[wq] = wm;
        if (!wg_sync()) { alive = false; break; }
        const float Mt = fmaxf(fmaxf(stat[0], stat[1]), fmaxf(stat[2], stat[3]));  // finite: row k0 <= q is valid
        const float w = valid ? exp2f(m_used - Mt) : 0.f;
        float lw = w * l_sum;
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) lw += __shfl_xor_sync(0xffffffffu, lw, o);
        if (lane == 0) stat[4 + wq] = lw;
        {
          const uint32_t tO = tmem + lane_base + Cfg::kTmemO + x * D;
#pragma unroll
          for (int ch = 0; ch < D / 32; ++ch) {
            uint32_t o[32];
            tmem_ld32(tO + ch * 32, o);
            tmem_wait_ld();
            float v[32];
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4) {
              const uint32_t off = (ch >> 1) * 16384 + swz128(row, (ch & 1) * 4 + i4);
              const uint4 vv = *reinterpret_cast<const uint4*>(smem + Cfg::kOffV2 + off);
              const uint32_t wv[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 f = unpack2<T16>(wv[e]);
                v[i4 * 8 + 2 * e] = __uint_as_float(o[i4 * 8 + 2 * e]) * (w * f.x);
                v[i4 * 8 + 2 * e + 1] = __uint_as_float(o[i4 * 8 + 2 * e + 1]) * (w * f.y);
              }
            }
            const float colsum = warp_transpose_sum(v, lane);
            red[wq * D + ch * 32 + lane] = colsum;
          }
        }
        if (!wg_sync()) { alive = false; break; }
        {
          const float Lt = stat[4] + stat[5] + stat[6] + stat[7];
          const float Mn = fmaxf(M_run, Mt);
          const float ca = exp2f(M_run - Mn), cb = exp2f(Mt - Mn);
          if (row < D) {
            const float Ot = red[row] + red[D + row] + red[2 * D + row] + red[3 * D + row];
            O_run = O_run * ca + Ot * cb;
          }
          L_run = L_run * ca + Lt * cb;
          M_run = Mn;
        }
        if (!wg_sync()) { alive = false; break; }  // red / stat may be rewritten by the next k-tile
        fence_async_smem();  // V2 tile reads above precede the next TMA write of that buffer
        tc_fence_before();
        mbar_arrive(&bars.a_free);
      }
      if (!alive) break;
      // ---- store the query's output row and log-sum-exp
      if (row < D) ((T16*)p.out)[((size_t)bh * T + qx) * D + row] = from_f<T16>(O_run / L_run);
      if (row == 0) p.lse[(size_t)bh * T + qx] = (M_run + log2f(L_run)) * kLn2;
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
  if (tid == 0 && bars.abort_flag && p.status) atomicOr(p.status, 2);
}

template <int D, typename T16>
int launch_fwd(const TdpArgs& a) {
  using Cfg = FwdCfg<D>;
  const int BN = a.B * a.N;
  const size_t n = (size_t)BN * a.T * a.D;
  T16* sv1 = (T16*)a.workspace;
  silu_kernel<T16><<<(unsigned)((n / 8 + 255) / 256 + 1), 256, 0, a.stream>>>((const T16*)a.v1, sv1, n);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  CUtensorMap tmK1, tmK2, tmSV1, tmV2;
  int rc;
  if ((rc = make_tmap_3d(&tmK1, a.k1, 2, D, a.T, BN, 64, kBJ))) return rc;
  if ((rc = make_tmap_3d(&tmSV1, sv1, 2, D, a.T, BN, 64, kBJ))) return rc;
  if ((rc = make_tmap_3d(&tmK2, a.k2, 2, D, a.T, BN, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmV2, a.v2, 2, D, a.T, BN, 64, 128))) return rc;
  FwdParams p{};
  p.out = a.out_o;
  p.lse = a.out_lse;
  p.q = a.q;
  p.T = a.T;
  p.BN = BN;
  p.q_mod = a.q_mod;
  p.q_rem = a.q_rem;
  p.nq = a.q_rem < a.T ? (a.T - a.q_rem + a.q_mod - 1) / a.q_mod : 0;
  p.n_pairs = (p.nq + 1) / 2;
  p.causal = a.mask.causal;
  p.scale2 = a.alpha * kLog2e;
  p.status = a.status_word;
  if (p.nq == 0) return 0;
  auto kern = tdp_fwd_kernel<D, T16>;
  TRITT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
  const long items = (long)p.n_pairs * BN;
  const int grid = (int)(items < num_sms() ? items : num_sms());
  kern<<<grid, kThreads, Cfg::kSmem, a.stream>>>(tmK1, tmK2, tmSV1, tmV2, p);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace

bool sm100_tdp_supported(int op, int T, int D, int dtype, const TdpMask& m) {
  if (op != TRITT_OP_TDP_FWD && op != TRITT_OP_TDP_BWD) return false;
  if (dtype != TRITT_BF16 && dtype != TRITT_F16) return false;
  if (D != 64 && D != 128) return false;
  if (!m.full_windows()) return false;
  return T >= 1;
}

size_t sm100_tdp_workspace(int op, int B, int N, int T, int D, int dtype) {
  if (dtype != TRITT_BF16 && dtype != TRITT_F16) return 0;
  if (op == TRITT_OP_TDP_FWD) return (size_t)B * N * T * D * 2;
  if (op == TRITT_OP_TDP_BWD) return sm100_tdp_bwd_workspace(B, N, T, D);
  return 0;
}

int sm100_tdp_fwd(const TdpArgs& a) {
  // the two queries of a pair must fall in the same 64-row block
  if (a.q_mod < 1 || a.q_mod > 32 || (a.q_mod & (a.q_mod - 1))) {
    set_error("tensor-core path needs a power-of-two query shard count <= 32 (got %d)", a.q_mod);
    return -30;
  }
  if (a.dtype == TRITT_BF16) return a.D == 128 ? launch_fwd<128, __nv_bfloat16>(a) : launch_fwd<64, __nv_bfloat16>(a);
  return a.D == 128 ? launch_fwd<128, __half>(a) : launch_fwd<64, __half>(a);
}

}  // namespace tritt
