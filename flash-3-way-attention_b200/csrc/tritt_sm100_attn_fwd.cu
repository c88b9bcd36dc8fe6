// Two-way soft-max attention forward on Blackwell tensor cores (tcgen05 + TMEM + TMA): the building block of
// dot-product-sum trittention, whose score alpha (Q[q].K2[t] + K1[s].K2[t]) separates into two chained attentions
//   inner (rows t = K2, columns s = K1, values SiLU(V1), band s <= t <= s + k_diff):  Y[t], LSEin[t]
//   outer (rows q = Q, columns t = K2, values Y*V2, per-column bias LSEin, t <= q):   O[q], m[q]
// (the reference's kernels run the same two-level log-sum-exp, dot_product_sum/kernels/fwd_kernel.py:102-169,
// 196-220, but recompute the inner leg for every query block).
//
// One CTA owns 128 rows of one head and walks the 128-column tiles its rows attend to:
//   warp 0      TMA producer: the row operand once, then a two-stage ring of (key tile, value tile)
//   warp 1      issues tcgen05.mma:  S = X * Kc^T  (128x128 fp32 in TMEM)  and  acc += P * Vc  with P read from
//               TMEM (16-bit, over the columns of S already consumed) and the value tile used row-major
//   warps 4-7   one row per thread: scale, bias and mask, row maximum, exp2 with lazy rescaling of the accumulator,
//               P written back to TMEM; at the end the row is normalised and stored (fp32 and / or 16-bit, and
//               optionally the 16-bit product with a second tensor, which is the outer leg's value operand)
// The chain S -> soft-max -> P*V of a CTA is serial; two CTAs share an SM when the head dimension is 64.
#include "tritt_common.cuh"
#include "tritt_sm100.cuh"
#include "tritt_sm100_tdp.cuh"

#include <type_traits>

namespace tritt {
namespace {
using namespace sm100;

constexpr int kAttnThreads = 256;
constexpr float kAttnRescaleGap = 8.f;  // rescale the accumulator only when the row max grew by more than 2^8

template <int D> struct AttnCfg {
  static constexpr int kTile = 128 * D * 2;   // bytes of one 128-row operand tile
  static constexpr int kStages = 2;
  static constexpr int kOffX = 0;
  static constexpr int kOffRing = kTile;      // stage s: key tile at kOffRing + 2 s kTile, value tile right behind
  static constexpr int kOffBias = kOffRing + kStages * 2 * kTile;  // [4 warps][2 parities][128] fp32, log2 units
  static constexpr int kOffBars = kOffBias + 4 * 2 * 128 * 4;
  static constexpr int kSmem = kOffBars + 128;
  static constexpr int kTmemO = 128;          // S | acc
  static constexpr int kTmemCols = 256;
};

struct AttnFwdParams {
  const float* bias;   // [BN, T] per column, natural-log units, or null
  float* out_f32;      // [BN, T, D] or null
  void* out_t;         // 16-bit [BN, T, D] or null
  const void* mul;     // 16-bit [BN, T, D]: out_mul = out * mul (both null or both set)
  void* out_mul;
  float* out_lse;      // [BN, T] natural log
  int T, causal, win;  // valid(r, c): not causal, or c <= r and r - c <= win
  float scale2;        // alpha * log2(e)
  int* status;
};

struct AttnBarriers {
  uint64_t ring_full[2], ring_empty[2];
  uint64_t x_full, s_ready, p_ready, o_done;
  uint32_t tmem_base;
  int abort_flag;
};

template <int D, typename T16>
__global__ void __launch_bounds__(kAttnThreads, D == 64 ? 2 : 1)
attn_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, AttnFwdParams p) {
  using Cfg = AttnCfg<D>;
  constexpr int NS = Cfg::kStages;
  constexpr int KH = D / 64;
  extern __shared__ __align__(1024) uint8_t smem[];
  static_assert(sizeof(AttnBarriers) <= 128, "barrier block too large");
  AttnBarriers& bars = *reinterpret_cast<AttnBarriers*>(smem + Cfg::kOffBars);
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
    mbar_init(&bars.x_full, 1);
    mbar_init(&bars.s_ready, 1);
    mbar_init(&bars.p_ready, 128);
    mbar_init(&bars.o_done, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&bars.tmem_base, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars.tmem_base;
  volatile int* abort_flag = &bars.abort_flag;

  const int T = p.T;
  const int n_row_tiles = (T + 127) / 128;
  const int rt = n_row_tiles - 1 - (int)blockIdx.x;  // the row tiles with the most columns start first
  const int bh = blockIdx.y;
  const int r0 = rt * 128;
  // column tiles attended by any row of this tile
  int ct0 = 0, ct1 = n_row_tiles - 1;
  if (p.causal) {
    const int last_row = min(r0 + 127, T - 1);
    const int lo_c = max(0, p.win >= T ? 0 : r0 - p.win);
    ct0 = lo_c / 128;
    ct1 = last_row / 128;
  }
  const int n_ct = ct1 - ct0 + 1;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmX);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_arrive_expect_tx(&bars.x_full, Cfg::kTile);
      for (int hh = 0; hh < KH; ++hh)
        tma_load_3d(smem + Cfg::kOffX + hh * 16384, &tmX, &bars.x_full, hh * 64, r0, bh);
      int issued = 0;
      bool alive = true;
      for (int i = 0; i < n_ct && alive; ++i) {
        const int st = i % NS;
        if (!mbar_wait(&bars.ring_empty[st], ((i / NS) & 1) ^ 1, abort_flag)) { alive = false; break; }
        mbar_arrive_expect_tx(&bars.ring_full[st], 2 * Cfg::kTile);
        uint8_t* kdst = smem + Cfg::kOffRing + st * 2 * Cfg::kTile;
        for (int hh = 0; hh < KH; ++hh) {
          tma_load_3d(kdst + hh * 16384, &tmK, &bars.ring_full[st], hh * 64, (ct0 + i) * 128, bh);
          tma_load_3d(kdst + Cfg::kTile + hh * 16384, &tmV, &bars.ring_full[st], hh * 64, (ct0 + i) * 128, bh);
        }
        ++issued;
      }
      if (!alive) {
        // give copies still in flight a bounded chance to land before the CTA retires
        const long long t0 = clock64();
        while (!mbar_try_wait(&bars.x_full, 0) && clock64() - t0 < kWaitTicks / 8) {
        }
        for (int i = issued > NS ? issued - NS : 0; i < issued; ++i) {
          const long long t1 = clock64();
          while (!mbar_try_wait(&bars.ring_full[i % NS], (i / NS) & 1) && clock64() - t1 < kWaitTicks / 8) {
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
      const uint32_t xLo = desc_lo(smem_u32(smem + Cfg::kOffX), 16);
      auto issue_s = [&](int st) {
        const uint32_t bLo = desc_lo(smem_u32(smem + Cfg::kOffRing + st * 2 * Cfg::kTile), 16);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t kk = (k >> 2) * (16384 >> 4) + (k & 3) * 2;
          if (leader) mma_ss_lo(tmem, xLo + kk, bLo + kk, kHi, idesc_s, k > 0);
        }
        commit(&bars.s_ready);
      };
      auto issue_pv = [&](int st, uint32_t acc) {
        // value tile used row-major: 64-column blocks 16 KiB apart, 16 rows (one instruction) 2 KiB apart
        const uint32_t bLo = desc_lo(smem_u32(smem + Cfg::kOffRing + st * 2 * Cfg::kTile + Cfg::kTile), 16384);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (leader) mma_ts_lo(tmem + Cfg::kTmemO, tmem + k * 8, bLo + k * (2048 >> 4), kHi, idesc_pv, k > 0 ? 1u : acc);
      };
      bool alive = wait_all(&bars.x_full, 0) && wait_all(&bars.ring_full[0], 0);
      if (alive) {
        tc_fence_after();
        issue_s(0);
      }
      for (int i = 0; i < n_ct && alive; ++i) {
        const int st = i % NS;
        if (!wait_all(&bars.p_ready, i & 1)) { alive = false; break; }
        tc_fence_after();
        issue_pv(st, i > 0);
        commit(&bars.ring_empty[st]);
        if (i + 1 < n_ct) {
          if (!wait_all(&bars.ring_full[(i + 1) % NS], ((i + 1) / NS) & 1)) { alive = false; break; }
          tc_fence_after();
          issue_s((i + 1) % NS);   // (overwrites P(i): the pipe runs it after P(i)*V(i), issued just above)
        } else {
          commit(&bars.o_done);
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ soft-max and epilogue, one row per thread
    const int wq = warp & 3;
    const int row = wq * 32 + lane;
    const int r = r0 + row;
    const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
    const uint32_t tS = tmem + lane_base;
    const uint32_t tO = tmem + lane_base + Cfg::kTmemO;
    float* sbias = reinterpret_cast<float*>(smem + Cfg::kOffBias);
    // this row's attended columns [c_lo, c_hi]
    const int c_hi = p.causal ? min(r, T - 1) : T - 1;
    const int c_lo = (p.causal && p.win < T) ? max(0, r - p.win) : 0;
    float m_used = -INFINITY, l_sum = 0.f;
    bool alive = true;
    for (int i = 0; i < n_ct; ++i) {
      const int c0 = (ct0 + i) * 128;
      // this tile's column biases (log2 units), staged per warp so that no hand-off between warps is needed
      float* sb = sbias + (wq * 2 + (i & 1)) * 128;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int c = c0 + lane * 4 + e;
        sb[lane * 4 + e] = (p.bias && c < T) ? __ldg(p.bias + (size_t)bh * T + c) * kLog2e : 0.f;
      }
      __syncwarp();
      alive = __all_sync(0xffffffffu, mbar_wait(&bars.s_ready, i & 1, abort_flag));
      if (!alive) break;
      tc_fence_after();
      const int lo = c_lo - c0, hi = c_hi - c0;
      const bool full = __all_sync(0xffffffffu, lo <= 0 && hi >= 127);
      // pass 1: row maximum of scale * S + bias over the attended columns
      float mx = -INFINITY;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t sr[64];
        tmem_ld64(tS + hf * 64, sr);
        tmem_wait_ld();
        if (full) {
          float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
          for (int c = 0; c < 64; c += 4) {
            const float4 b = *reinterpret_cast<const float4*>(sb + hf * 64 + c);
            m0 = fmaxf(m0, fmaf(__uint_as_float(sr[c]), p.scale2, b.x));
            m1 = fmaxf(m1, fmaf(__uint_as_float(sr[c + 1]), p.scale2, b.y));
            m2 = fmaxf(m2, fmaf(__uint_as_float(sr[c + 2]), p.scale2, b.z));
            m3 = fmaxf(m3, fmaf(__uint_as_float(sr[c + 3]), p.scale2, b.w));
          }
          mx = fmaxf(mx, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
        } else {
          const int l2 = lo - hf * 64, h2 = hi - hf * 64;
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (c >= l2 && c <= h2) mx = fmaxf(mx, fmaf(__uint_as_float(sr[c]), p.scale2, sb[hf * 64 + c]));
        }
      }
      if (i == 0) {
        m_used = mx;  // nothing accumulated yet
      } else {
        const bool grow = mx > m_used + kAttnRescaleGap;
        if (__any_sync(0xffffffffu, grow)) {
          // (s_ready of this tile was committed after the previous P*V, so that product has landed)
          const float corr = grow ? exp2f(m_used - mx) : 1.f;
          if (grow) {
            m_used = mx;
            l_sum *= corr;
          }
#pragma unroll
          for (int ch = 0; ch < D / 32; ++ch) {
            uint32_t o[32];
            tmem_ld32(tO + ch * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * corr);
            tmem_st32(tO + ch * 32, o);
          }
        }
      }
      // pass 2: P = exp2(scale * S + bias - m), packed to 16 bits over the columns already consumed
      float psum = 0.f;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t sr[64];
        tmem_ld64(tS + hf * 64, sr);
        tmem_wait_ld();
        uint32_t pk[32];
        if (full) {
          float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
          for (int c = 0; c < 64; c += 2) {
            const float2 b = *reinterpret_cast<const float2*>(sb + hf * 64 + c);
            const float p0 = exp2f(fmaf(__uint_as_float(sr[c]), p.scale2, b.x) - m_used);
            const float p1 = exp2f(fmaf(__uint_as_float(sr[c + 1]), p.scale2, b.y) - m_used);
            ps0 += p0;
            ps1 += p1;
            pk[c >> 1] = pack2<T16>(p0, p1);
          }
          psum += ps0 + ps1;
        } else {
          // (a row with no attended column so far has m_used = -inf and selects 0 everywhere)
          const int l2 = lo - hf * 64, h2 = hi - hf * 64;
#pragma unroll
          for (int c = 0; c < 64; c += 2) {
            const float p0 = (c >= l2 && c <= h2)
                                 ? exp2f(fmaf(__uint_as_float(sr[c]), p.scale2, sb[hf * 64 + c]) - m_used) : 0.f;
            const float p1 = (c + 1 >= l2 && c + 1 <= h2)
                                 ? exp2f(fmaf(__uint_as_float(sr[c + 1]), p.scale2, sb[hf * 64 + c + 1]) - m_used) : 0.f;
            psum += p0 + p1;
            pk[c >> 1] = pack2<T16>(p0, p1);
          }
        }
        tmem_st32(tS + hf * 32, pk);
      }
      l_sum += psum;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&bars.p_ready);
    }
    if (alive) alive = __all_sync(0xffffffffu, mbar_wait(&bars.o_done, 0, abort_flag));
    if (alive) {
      tc_fence_after();
      const float inv = 1.f / l_sum;
      const bool in_range = r < T;
      const size_t off = ((size_t)bh * T + r) * D;
#pragma unroll
      for (int ch = 0; ch < D / 32; ++ch) {
        uint32_t o[32];
        tmem_ld32(tO + ch * 32, o);
        tmem_wait_ld();
        if (!in_range) continue;
        float v[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(o[e]) * inv;
        if (p.out_f32) {
#pragma unroll
          for (int e = 0; e < 32; e += 4)
            *reinterpret_cast<float4*>(p.out_f32 + off + ch * 32 + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
        }
        if (p.out_t) {
#pragma unroll
          for (int e = 0; e < 32; e += 8)
            *reinterpret_cast<uint4*>((T16*)p.out_t + off + ch * 32 + e) =
                make_uint4(pack2<T16>(v[e], v[e + 1]), pack2<T16>(v[e + 2], v[e + 3]), pack2<T16>(v[e + 4], v[e + 5]),
                           pack2<T16>(v[e + 6], v[e + 7]));
        }
        if (p.out_mul) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            const uint4 mv = __ldg(reinterpret_cast<const uint4*>((const T16*)p.mul + off + ch * 32 + e));
            const float2 a0 = unpack2<T16>(mv.x), a1 = unpack2<T16>(mv.y), a2 = unpack2<T16>(mv.z),
                         a3 = unpack2<T16>(mv.w);
            *reinterpret_cast<uint4*>((T16*)p.out_mul + off + ch * 32 + e) =
                make_uint4(pack2<T16>(v[e] * a0.x, v[e + 1] * a0.y), pack2<T16>(v[e + 2] * a1.x, v[e + 3] * a1.y),
                           pack2<T16>(v[e + 4] * a2.x, v[e + 5] * a2.y), pack2<T16>(v[e + 6] * a3.x, v[e + 7] * a3.y));
          }
        }
      }
      if (in_range && p.out_lse) p.out_lse[(size_t)bh * T + r] = (m_used + log2f(l_sum)) * kLn2;
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, Cfg::kTmemCols);
  if (tid == 0 && bars.abort_flag && p.status) atomicOr(p.status, 16);
}

template <int D, typename T16>
int launch_attn_fwd(const AttnTcArgs& a) {
  using Cfg = AttnCfg<D>;
  CUtensorMap tmX, tmK, tmV;
  int rc;
  if ((rc = make_tmap_3d(&tmX, a.xq, 2, D, a.T, a.BN, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmK, a.kc, 2, D, a.T, a.BN, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmV, a.vc, 2, D, a.T, a.BN, 64, 128))) return rc;
  AttnFwdParams p{};
  p.bias = a.bias;
  p.out_f32 = a.out_f32;
  p.out_t = a.out_t;
  p.mul = a.mul;
  p.out_mul = a.out_mul;
  p.out_lse = a.out_lse;
  p.T = a.T;
  p.causal = a.causal;
  p.win = a.win < 0 ? 0 : a.win;
  p.scale2 = a.alpha * kLog2e;
  p.status = a.status;
  auto kern = attn_fwd_sm100_kernel<D, T16>;
  TRITT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem));
  const dim3 grid((a.T + 127) / 128, a.BN);
  kern<<<grid, kAttnThreads, Cfg::kSmem, a.stream>>>(tmX, tmK, tmV, p);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace

bool sm100_attn_fwd_supported(int T, int D, int dtype) {
  return T >= 1 && (D == 64 || D == 128) && (dtype == TRITT_F16 || dtype == TRITT_BF16);
}

int sm100_attn_fwd(const AttnTcArgs& a) {
  if (a.dtype == TRITT_BF16)
    return a.D == 128 ? launch_attn_fwd<128, __nv_bfloat16>(a) : launch_attn_fwd<64, __nv_bfloat16>(a);
  return a.D == 128 ? launch_attn_fwd<128, __half>(a) : launch_attn_fwd<64, __half>(a);
}

int sm100_silu_16(const void* in, void* out, size_t n, int dtype, cudaStream_t stream) {
  const unsigned blocks = (unsigned)((n / 8 + 255) / 256 + 1);
  if (dtype == TRITT_BF16)
    silu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, n);
  else
    silu_kernel<__half><<<blocks, 256, 0, stream>>>((const __half*)in, (__half*)out, n);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace tritt
