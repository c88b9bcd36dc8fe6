// Two-way soft-max attention backward on Blackwell tensor cores: the gradients of the two attentions that make up
// dot-product-sum trittention (see tritt_sm100_attn_fwd.cu for the decomposition).  With P[r,c] =
// exp(alpha X[r].K[c] + bias[c] - lse[r]), dP[r,c] = dOut[r].V[c] and dS = P (dP - drow[r]):
//   row-owner kernel  (COL = false): a CTA owns 128 rows r and walks the column tiles:
//        d_rows[r] = alpha sum_c dS[r,c] K[c]
//   column-owner kernel (COL = true): a CTA owns 128 columns c and walks the row tiles, working on the transposed
//   products S^T = K X^T and dP^T = V dOut^T so that its threads again own one accumulator row each:
//        d_vc[c] = sum_r P[r,c] dOut[r],   d_kc[c] = alpha sum_r dS[r,c] X[r],   gsum[c] = sum_r dS[r,c]
// Neither kernel needs atomics or a transposed operand; the price is that S and dP are formed twice.  (The
// reference splits its backward the same way, a query-owner kernel and a key-owner kernel:
// dot_product_sum/kernels/bwd_dq_kernel.py:28-350, bwd_dk1_dv1_kernel.py:29-416.)
//
// Roles per CTA (256 threads): warp 0 TMA producer (the owner's two operand tiles once, then a two-stage ring of
// the other side's two tiles), warp 1 issues tcgen05.mma (S and dP into TMEM; then the accumulations with P / dS
// read from TMEM, 16-bit, over the columns of S / dP, and the ring tile used row-major), warps 4-7 one owner row
// per thread (P and dS from S, dP and the row / column vectors; epilogue).
#include "tritt_common.cuh"
#include "tritt_sm100.cuh"
#include "tritt_sm100_tdp.cuh"

#include <type_traits>

namespace tritt {
namespace {
using namespace sm100;

constexpr int kAttnBwdThreads = 256;

template <int D> struct AttnBwdCfg {
  static constexpr int kTile = 128 * D * 2;
  static constexpr int kStages = 2;
  static constexpr int kOffOwn = 0;                  // owner tiles: [0] keys side (X or K), [1] values side (dOut or V)
  static constexpr int kOffRing = 2 * kTile;         // stage s: tiles [0], [1] of the other side
  static constexpr int kOffVec = kOffRing + kStages * 2 * kTile;  // [4 warps][2 parities][2 vectors][128] fp32
  static constexpr int kOffBars = kOffVec + 4 * 2 * 2 * 128 * 4;
  static constexpr int kSmem = kOffBars + 128;
  static constexpr int kTmemS = 0, kTmemDP = 128, kTmemAcc0 = 256, kTmemAcc1 = 256 + D;
};

struct AttnBwdParams {
  const float *bias, *lse, *drow;  // per column (or null); per row; per row
  const void *out_rows, *dout_rows;  // row-owner: drow = dout . out computed here (then drow is not read) ...
  float* drow_out;                   // ... and stored for the column-owner launch
  const void* silu_src;            // column-owner epilogue variants (see AttnBwdTcArgs)
  void* d_vc_t;
  const float* mid_y;
  const void* mid_v2;
  void *mid_dv2, *mid_dy_t;
  float* mid_dt;
  void* d_rows_t;                  // row-owner: 16-bit [BN, T, D]
  const float* d_rows_add;         // row-owner: fp32 term added before rounding, or null
  float* d_kc_f32;                 // column-owner: one of the two
  void* d_kc_t;
  float* d_vc_f32;                 // column-owner
  float* gsum;                     // column-owner, or null
  int T, causal, win;
  float scale2, alpha;             // alpha log2(e); alpha
  int* status;
};

struct AttnBwdBarriers {
  uint64_t ring_full[2], ring_empty[2];
  uint64_t own_full, sd_ready, pd_ready, acc_done;
  uint32_t tmem_base;
  int abort_flag;
};

template <int D, typename T16, bool COL>
__global__ void __launch_bounds__(kAttnBwdThreads, 1)
attn_bwd_sm100_kernel(const __grid_constant__ CUtensorMap tmOwn0, const __grid_constant__ CUtensorMap tmOwn1,
                      const __grid_constant__ CUtensorMap tmOth0, const __grid_constant__ CUtensorMap tmOth1,
                      AttnBwdParams p) {
  using Cfg = AttnBwdCfg<D>;
  constexpr int NS = Cfg::kStages;
  constexpr int KH = D / 64;
  extern __shared__ __align__(1024) uint8_t smem[];
  static_assert(sizeof(AttnBwdBarriers) <= 128, "barrier block too large");
  AttnBwdBarriers& bars = *reinterpret_cast<AttnBwdBarriers*>(smem + Cfg::kOffBars);
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
    mbar_init(&bars.own_full, 1);
    mbar_init(&bars.sd_ready, 1);
    mbar_init(&bars.pd_ready, 128);
    mbar_init(&bars.acc_done, 1);
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
  const int n_tiles = (T + 127) / 128;
  const int bh = blockIdx.y;
  // the owner tiles with the most work start first: the last rows / the first columns under the causal mask
  const int ot = COL ? (int)blockIdx.x : n_tiles - 1 - (int)blockIdx.x;
  const int o0 = ot * 128;
  const bool banded = p.causal && p.win < T;
  // tiles of the other side that hold an attended entry of this tile
  int t0 = 0, t1 = n_tiles - 1;
  if (p.causal) {
    if (COL) {
      t0 = ot;
      t1 = banded ? min(o0 + 127 + p.win, T - 1) / 128 : n_tiles - 1;
    } else {
      t0 = banded ? max(0, o0 - p.win) / 128 : 0;
      t1 = min(o0 + 127, T - 1) / 128;
    }
  }
  const int n_t = t1 - t0 + 1;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmOwn0);
      tma_prefetch_desc(&tmOwn1);
      tma_prefetch_desc(&tmOth0);
      tma_prefetch_desc(&tmOth1);
      mbar_arrive_expect_tx(&bars.own_full, 2 * Cfg::kTile);
      for (int hh = 0; hh < KH; ++hh) {
        tma_load_3d(smem + Cfg::kOffOwn + hh * 16384, &tmOwn0, &bars.own_full, hh * 64, o0, bh);
        tma_load_3d(smem + Cfg::kOffOwn + Cfg::kTile + hh * 16384, &tmOwn1, &bars.own_full, hh * 64, o0, bh);
      }
      int issued = 0;
      bool alive = true;
      for (int i = 0; i < n_t && alive; ++i) {
        const int st = i % NS;
        if (!mbar_wait(&bars.ring_empty[st], ((i / NS) & 1) ^ 1, abort_flag)) { alive = false; break; }
        mbar_arrive_expect_tx(&bars.ring_full[st], 2 * Cfg::kTile);
        uint8_t* dst = smem + Cfg::kOffRing + st * 2 * Cfg::kTile;
        for (int hh = 0; hh < KH; ++hh) {
          tma_load_3d(dst + hh * 16384, &tmOth0, &bars.ring_full[st], hh * 64, (t0 + i) * 128, bh);
          tma_load_3d(dst + Cfg::kTile + hh * 16384, &tmOth1, &bars.ring_full[st], hh * 64, (t0 + i) * 128, bh);
        }
        ++issued;
      }
      if (!alive) {
        // give copies still in flight a bounded chance to land before the CTA retires
        const long long ta = clock64();
        while (!mbar_try_wait(&bars.own_full, 0) && clock64() - ta < kWaitTicks / 8) {
        }
        for (int i = issued > NS ? issued - NS : 0; i < issued; ++i) {
          const long long tb = clock64();
          while (!mbar_try_wait(&bars.ring_full[i % NS], (i / NS) & 1) && clock64() - tb < kWaitTicks / 8) {
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
      constexpr uint32_t idesc_acc = make_idesc_f16(128, D, kFmt, false, true);
      constexpr uint32_t kHi = desc_hi(1024);
      const uint32_t own0 = desc_lo(smem_u32(smem + Cfg::kOffOwn), 16);
      const uint32_t own1 = desc_lo(smem_u32(smem + Cfg::kOffOwn + Cfg::kTile), 16);
      // S (or S^T) = own0 * oth0^T,  dP (or dP^T) = own1 * oth1^T
      auto issue_sd = [&](int st) {
        const uint32_t b0 = desc_lo(smem_u32(smem + Cfg::kOffRing + st * 2 * Cfg::kTile), 16);
        const uint32_t b1 = desc_lo(smem_u32(smem + Cfg::kOffRing + st * 2 * Cfg::kTile + Cfg::kTile), 16);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t kk = (k >> 2) * (16384 >> 4) + (k & 3) * 2;
          if (leader) mma_ss_lo(tmem + Cfg::kTmemS, own0 + kk, b0 + kk, kHi, idesc_s, k > 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t kk = (k >> 2) * (16384 >> 4) + (k & 3) * 2;
          if (leader) mma_ss_lo(tmem + Cfg::kTmemDP, own1 + kk, b1 + kk, kHi, idesc_s, k > 0);
        }
        commit(&bars.sd_ready);
      };
      // accumulations with the 16-bit P / dS read from TMEM and the ring tiles used row-major
      auto issue_acc = [&](int st, uint32_t acc) {
        const uint32_t m0 = desc_lo(smem_u32(smem + Cfg::kOffRing + st * 2 * Cfg::kTile), 16384);
        const uint32_t m1 = desc_lo(smem_u32(smem + Cfg::kOffRing + st * 2 * Cfg::kTile + Cfg::kTile), 16384);
        if (COL) {
          // d_vc += P^T * dOut,  d_kc += dS^T * X
#pragma unroll
          for (int k = 0; k < 8; ++k)
            if (leader)
              mma_ts_lo(tmem + Cfg::kTmemAcc0, tmem + Cfg::kTmemS + k * 8, m1 + k * (2048 >> 4), kHi, idesc_acc,
                        k > 0 ? 1u : acc);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            if (leader)
              mma_ts_lo(tmem + Cfg::kTmemAcc1, tmem + Cfg::kTmemDP + k * 8, m0 + k * (2048 >> 4), kHi, idesc_acc,
                        k > 0 ? 1u : acc);
        } else {
          // d_rows += dS * K
#pragma unroll
          for (int k = 0; k < 8; ++k)
            if (leader)
              mma_ts_lo(tmem + Cfg::kTmemAcc0, tmem + Cfg::kTmemDP + k * 8, m0 + k * (2048 >> 4), kHi, idesc_acc,
                        k > 0 ? 1u : acc);
        }
      };
      bool alive = wait_all(&bars.own_full, 0) && wait_all(&bars.ring_full[0], 0);
      if (alive) {
        tc_fence_after();
        issue_sd(0);
      }
      for (int i = 0; i < n_t && alive; ++i) {
        const int st = i % NS;
        if (!wait_all(&bars.pd_ready, i & 1)) { alive = false; break; }
        tc_fence_after();
        issue_acc(st, i > 0);
        commit(&bars.ring_empty[st]);
        if (i + 1 < n_t) {
          if (!wait_all(&bars.ring_full[(i + 1) % NS], ((i + 1) / NS) & 1)) { alive = false; break; }
          tc_fence_after();
          issue_sd((i + 1) % NS);  // (overwrites P / dS of tile i: the pipe runs it after the products above)
        } else {
          commit(&bars.acc_done);
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ P, dS and the epilogue: one owner row per thread
    const int wq = warp & 3;
    const int row = wq * 32 + lane;
    const int own = o0 + row;
    const bool own_ok = own < T;
    const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
    const uint32_t tS = tmem + lane_base + Cfg::kTmemS;
    const uint32_t tD = tmem + lane_base + Cfg::kTmemDP;
    float* svec = reinterpret_cast<float*>(smem + Cfg::kOffVec) + wq * 2 * 2 * 128;
    // the owner's scalars
    float own_a = 0.f, own_b = 0.f;
    if (own_ok) {
      if (COL) {
        own_a = p.bias ? __ldg(p.bias + (size_t)bh * T + own) * kLog2e : 0.f;
      } else {
        own_a = __ldg(p.lse + (size_t)bh * T + own) * kLog2e;
        if (p.out_rows) {
          // drow = sum_h dOut[own, h] Out[own, h]  (the reference's preprocess kernel, bwd_preprocess.py:5-49)
          const uint4* a4 = reinterpret_cast<const uint4*>((const T16*)p.dout_rows + ((size_t)bh * T + own) * D);
          const uint4* b4 = reinterpret_cast<const uint4*>((const T16*)p.out_rows + ((size_t)bh * T + own) * D);
          float acc = 0.f;
#pragma unroll
          for (int i = 0; i < D / 8; ++i) {
            const uint4 av = __ldg(a4 + i), bv = __ldg(b4 + i);
            const uint32_t aw[4] = {av.x, av.y, av.z, av.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 fa = unpack2<T16>(aw[e]), fb = unpack2<T16>(bw[e]);
              acc = fmaf(fa.x, fb.x, fmaf(fa.y, fb.y, acc));
            }
          }
          own_b = acc;
          p.drow_out[(size_t)bh * T + own] = acc;
        } else {
          own_b = __ldg(p.drow + (size_t)bh * T + own);
        }
      }
    }
    // attended indices of the other side for this owner: [j_lo, j_hi]
    int j_lo = 0, j_hi = T - 1;
    if (p.causal) {
      if (COL) {
        j_lo = own;
        j_hi = banded ? min(own + p.win, T - 1) : T - 1;
      } else {
        j_lo = banded ? max(0, own - p.win) : 0;
        j_hi = min(own, T - 1);
      }
    }
    if (!own_ok) { j_lo = 1; j_hi = 0; }
    float gs = 0.f;
    bool alive = true;
    for (int i = 0; i < n_t; ++i) {
      const int j0 = (t0 + i) * 128;
      // per-index vectors of the other side (log2 units where they enter the exponent), staged per warp
      float* va = svec + (i & 1) * 2 * 128;
      float* vb = va + 128;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + lane * 4 + e;
        const bool ok = j < T;
        if (COL) {
          va[lane * 4 + e] = ok ? __ldg(p.lse + (size_t)bh * T + j) * kLog2e : 0.f;
          vb[lane * 4 + e] = ok ? __ldg(p.drow + (size_t)bh * T + j) : 0.f;
        } else {
          va[lane * 4 + e] = (ok && p.bias) ? __ldg(p.bias + (size_t)bh * T + j) * kLog2e : 0.f;
        }
      }
      __syncwarp();
      alive = __all_sync(0xffffffffu, mbar_wait(&bars.sd_ready, i & 1, abort_flag));
      if (!alive) break;
      tc_fence_after();
      const int lo = j_lo - j0, hi = j_hi - j0;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t sr[32], dr[32];
        tmem_ld32(tS + ch * 32, sr);
        tmem_ld32(tD + ch * 32, dr);
        tmem_wait_ld();
        uint32_t pk[16], dk[16];
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float pv[2], dv[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int j = ch * 32 + c + u;
            const bool valid = j >= lo && j <= hi;
            float e2, dr0;
            if (COL) {
              e2 = fmaf(__uint_as_float(sr[c + u]), p.scale2, own_a) - va[j];
              dr0 = vb[j];
            } else {
              e2 = fmaf(__uint_as_float(sr[c + u]), p.scale2, va[j]) - own_a;
              dr0 = own_b;
            }
            pv[u] = valid ? exp2f(e2) : 0.f;
            dv[u] = pv[u] * (__uint_as_float(dr[c + u]) - dr0);
          }
          if (COL) {
            gs += dv[0] + dv[1];
            pk[c >> 1] = pack2<T16>(pv[0], pv[1]);
          }
          dk[c >> 1] = pack2<T16>(dv[0], dv[1]);
        }
        if (COL) tmem_st16(tS + ch * 16, pk);
        tmem_st16(tD + ch * 16, dk);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&bars.pd_ready);
    }
    if (alive) alive = __all_sync(0xffffffffu, mbar_wait(&bars.acc_done, 0, abort_flag));
    if (alive) {
      tc_fence_after();
      const size_t off = ((size_t)bh * T + own) * D;
      float mid_dot = 0.f;  // column owner with the `mid` epilogue: sum_h dY Y of this column
#pragma unroll
      for (int ch = 0; ch < D / 32; ++ch) {
        uint32_t a0[32];
        tmem_ld32(tmem + lane_base + Cfg::kTmemAcc0 + ch * 32, a0);
        tmem_wait_ld();
        if (COL) {
          uint32_t a1[32];
          tmem_ld32(tmem + lane_base + Cfg::kTmemAcc1 + ch * 32, a1);
          tmem_wait_ld();
          if (!own_ok) continue;
          if (p.d_vc_f32) {
#pragma unroll
            for (int e = 0; e < 32; e += 4)
              *reinterpret_cast<float4*>(p.d_vc_f32 + off + ch * 32 + e) =
                  make_float4(__uint_as_float(a0[e]), __uint_as_float(a0[e + 1]), __uint_as_float(a0[e + 2]),
                              __uint_as_float(a0[e + 3]));
          } else if (p.silu_src) {
            // d(value) of a SiLU-gated value tensor: times SiLU'(raw value), in the operands' type
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              const uint4 rv = __ldg(reinterpret_cast<const uint4*>((const T16*)p.silu_src + off + ch * 32 + e));
              const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
              uint32_t o4[4];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const float2 f = unpack2<T16>(rw[k]);
                o4[k] = pack2<T16>(__uint_as_float(a0[e + 2 * k]) * silu_grad_f(f.x),
                                   __uint_as_float(a0[e + 2 * k + 1]) * silu_grad_f(f.y));
              }
              *reinterpret_cast<uint4*>((T16*)p.d_vc_t + off + ch * 32 + e) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
            }
          } else {
            // value tensor W = Y * V2 of the outer attention: dV2 = dW * Y, dY = dW * V2, and the row term of the
            // inner attention's backward, sum_h dY Y (minus the column sums of dS, below)
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              const uint4 vv = __ldg(reinterpret_cast<const uint4*>((const T16*)p.mid_v2 + off + ch * 32 + e));
              const float4 y0 = __ldg(reinterpret_cast<const float4*>(p.mid_y + off + ch * 32 + e));
              const float4 y1 = __ldg(reinterpret_cast<const float4*>(p.mid_y + off + ch * 32 + e + 4));
              const float yy[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
              const uint32_t vw[4] = {vv.x, vv.y, vv.z, vv.w};
              uint32_t o_dv2[4], o_dy[4];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const float2 f = unpack2<T16>(vw[k]);
                const float w0 = __uint_as_float(a0[e + 2 * k]), w1 = __uint_as_float(a0[e + 2 * k + 1]);
                const float dy0 = w0 * f.x, dy1 = w1 * f.y;
                mid_dot = fmaf(dy0, yy[2 * k], fmaf(dy1, yy[2 * k + 1], mid_dot));
                o_dv2[k] = pack2<T16>(w0 * yy[2 * k], w1 * yy[2 * k + 1]);
                o_dy[k] = pack2<T16>(dy0, dy1);
              }
              *reinterpret_cast<uint4*>((T16*)p.mid_dv2 + off + ch * 32 + e) = make_uint4(o_dv2[0], o_dv2[1], o_dv2[2], o_dv2[3]);
              *reinterpret_cast<uint4*>((T16*)p.mid_dy_t + off + ch * 32 + e) = make_uint4(o_dy[0], o_dy[1], o_dy[2], o_dy[3]);
            }
          }
          float v[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(a1[e]) * p.alpha;
          if (p.d_kc_f32) {
#pragma unroll
            for (int e = 0; e < 32; e += 4)
              *reinterpret_cast<float4*>(p.d_kc_f32 + off + ch * 32 + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
          } else {
#pragma unroll
            for (int e = 0; e < 32; e += 8)
              *reinterpret_cast<uint4*>((T16*)p.d_kc_t + off + ch * 32 + e) =
                  make_uint4(pack2<T16>(v[e], v[e + 1]), pack2<T16>(v[e + 2], v[e + 3]),
                             pack2<T16>(v[e + 4], v[e + 5]), pack2<T16>(v[e + 6], v[e + 7]));
          }
        } else {
          if (!own_ok) continue;
          float v[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(a0[e]) * p.alpha;
          if (p.d_rows_add) {
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
              const float4 ad = *reinterpret_cast<const float4*>(p.d_rows_add + off + ch * 32 + e);
              v[e] += ad.x;
              v[e + 1] += ad.y;
              v[e + 2] += ad.z;
              v[e + 3] += ad.w;
            }
          }
#pragma unroll
          for (int e = 0; e < 32; e += 8)
            *reinterpret_cast<uint4*>((T16*)p.d_rows_t + off + ch * 32 + e) =
                make_uint4(pack2<T16>(v[e], v[e + 1]), pack2<T16>(v[e + 2], v[e + 3]), pack2<T16>(v[e + 4], v[e + 5]),
                           pack2<T16>(v[e + 6], v[e + 7]));
        }
      }
      if (COL && own_ok && p.gsum) p.gsum[(size_t)bh * T + own] = gs;
      if (COL && own_ok && p.mid_dt) p.mid_dt[(size_t)bh * T + own] = mid_dot - gs;
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
  if (tid == 0 && bars.abort_flag && p.status) atomicOr(p.status, 32);
}

template <int D, typename T16, bool COL>
int launch_attn_bwd(const AttnBwdTcArgs& a) {
  using Cfg = AttnBwdCfg<D>;
  CUtensorMap tmX, tmK, tmV, tmDO;
  int rc;
  if ((rc = make_tmap_3d(&tmX, a.xq, 2, D, a.T, a.BN, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmK, a.kc, 2, D, a.T, a.BN, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmV, a.vc, 2, D, a.T, a.BN, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmDO, a.dout, 2, D, a.T, a.BN, 64, 128))) return rc;
  AttnBwdParams p{};
  p.bias = a.bias; p.lse = a.lse; p.drow = a.drow;
  p.out_rows = a.out_rows; p.dout_rows = a.dout; p.drow_out = a.drow_out;
  p.silu_src = a.silu_src; p.d_vc_t = a.d_vc_t;
  p.mid_y = a.mid_y; p.mid_v2 = a.mid_v2; p.mid_dv2 = a.mid_dv2; p.mid_dy_t = a.mid_dy_t; p.mid_dt = a.mid_dt;
  p.d_rows_t = a.d_rows_t; p.d_rows_add = a.d_rows_add;
  p.d_kc_f32 = a.d_kc_f32; p.d_kc_t = a.d_kc_t; p.d_vc_f32 = a.d_vc_f32; p.gsum = a.gsum;
  p.T = a.T; p.causal = a.causal; p.win = a.win < 0 ? 0 : (a.win > a.T ? a.T : a.win);
  p.scale2 = a.alpha * kLog2e; p.alpha = a.alpha;
  p.status = a.status;
  auto kern = attn_bwd_sm100_kernel<D, T16, COL>;
  TRITT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
  const dim3 grid((a.T + 127) / 128, a.BN);
  // owner side: rows (X, dOut) or columns (K, V); the other side streams through the ring
  if (COL)
    kern<<<grid, kAttnBwdThreads, Cfg::kSmem, a.stream>>>(tmK, tmV, tmX, tmDO, p);
  else
    kern<<<grid, kAttnBwdThreads, Cfg::kSmem, a.stream>>>(tmX, tmDO, tmK, tmV, p);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}

template <bool COL>
int dispatch_attn_bwd(const AttnBwdTcArgs& a) {
  if (a.dtype == TRITT_BF16)
    return a.D == 128 ? launch_attn_bwd<128, __nv_bfloat16, COL>(a) : launch_attn_bwd<64, __nv_bfloat16, COL>(a);
  return a.D == 128 ? launch_attn_bwd<128, __half, COL>(a) : launch_attn_bwd<64, __half, COL>(a);
}

}  // namespace

int sm100_attn_bwd_rows(const AttnBwdTcArgs& a) { return dispatch_attn_bwd<false>(a); }
int sm100_attn_bwd_cols(const AttnBwdTcArgs& a) { return dispatch_attn_bwd<true>(a); }

}  // namespace tritt
