// Register-resident variant of the general CUDA-core triple-dot-product kernel for head dimensions 16 to 128.
// LPR consecutive lanes (four; eight for head dimension 128) own one pair row (q, x); each lane keeps its share of the
// row's vectors (a = alpha*Q[q]*X[x], a' = dO[q]*Y[x], the G and U sums) in registers, dot products are finished
// with two or three shuffles inside the group, and the tiles of the column axis are staged in shared memory and read with
// broadcast 16-byte loads.  Same arithmetic, modes, masks and outputs as tdp_simt_kernel (which keeps the vectors
// in shared memory and serves the other head dimensions); about an order of magnitude fewer instructions per
// attended triple.  Included by tritt_simt_tdp.cu after SimtTdpParams and the MODE_* constants.
#pragma once

constexpr int kQuadCols = 32;   // column-axis rows staged per step

// sum over the LPR lanes that own one row
template <int LPR> __device__ __forceinline__ float tdp_row_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  if (LPR == 8) v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}
// sum over the row groups of a warp that hold the same share of the head dimension
template <int LPR> __device__ __forceinline__ float tdp_rows_sum(float v) {
  if (LPR == 4) v += __shfl_xor_sync(0xffffffffu, v, 4);
  v += __shfl_xor_sync(0xffffffffu, v, 8);
  v += __shfl_xor_sync(0xffffffffu, v, 16);
  return v;
}

template <typename T, int MODE, int DQ, int LPR>
__global__ void __launch_bounds__(128) tdp_simt_quad_kernel(SimtTdpParams p) {
  constexpr int D = DQ * LPR;
  constexpr int kQuadRows = 128 / LPR;   // pair rows per pass of a CTA (128 threads)
  __shared__ __align__(16) float tK[kQuadCols * D];
  __shared__ __align__(16) float tV[kQuadCols * D];
  __shared__ float qs[D], qr[D], dor[D], outacc[D];
  __shared__ float red[128];
  const int tid = threadIdx.x, lane = tid & 31, qd = tid & (LPR - 1), T_ = p.T;
  const int bh = blockIdx.y;
  const int qi = p.nq - 1 - (int)blockIdx.x;  // long rows first
  const int q = p.q_rem + qi * p.q_mod;
  const size_t base = (size_t)bh * T_ * D;
  const T* Q = (const T*)p.q + base;
  const T* Xp = (const T*)(p.role == 0 ? p.k2 : p.k1) + base;
  const T* Yp = (const T*)(p.role == 0 ? p.v2 : p.v1) + base;
  const T* Kc = (const T*)(p.role == 0 ? p.k1 : p.k2) + base;
  const T* Vc = (const T*)(p.role == 0 ? p.v1 : p.v2) + base;
  const bool silu_y = p.role == 1, silu_vc = p.role == 0;

  float dq_part = 0.f;
  for (int h = tid; h < D; h += 128) {
    const float qv = to_f(Q[(size_t)q * D + h]);
    qr[h] = qv;
    qs[h] = qv * p.alpha * kLog2e;
    outacc[h] = 0.f;
    if (MODE == MODE_BWD) {
      const float dv = to_f(((const T*)p.d_o + base)[(size_t)q * D + h]);
      dor[h] = dv;
      dq_part += dv * to_f(((const T*)p.o + base)[(size_t)q * D + h]);
    }
  }
  float lse2 = 0.f, Dq = 0.f;
  if (MODE != MODE_LSE) lse2 = p.lse[(size_t)bh * T_ + q] * kLog2e;
  if (MODE == MODE_BWD) {
    // Dq = sum_h dO[q,h] * O[q,h]  (reference flash_trittention.py:167)
    red[tid] = dq_part;
    __syncthreads();
    for (int s = 64; s > 0; s >>= 1) {
      if (tid < s) red[tid] += red[tid + s];
      __syncthreads();
    }
    Dq = red[0];
  }
  __syncthreads();

  const TdpMask mk = p.mask;
  const bool single = mk.single_pair(q);         // one attended pair: the score gradient is exactly zero
  const int xw = p.role == 0 ? mk.k2w : mk.k1w;  // window of the row axis against q
  const int cw = p.role == 0 ? mk.k1w : mk.k2w;
  // band of the column axis around a row index x: c in [x - below, x + above]
  const int below = p.role == 0 ? mk.kkl : mk.kkr;
  const int above = p.role == 0 ? mk.kkr : mk.kkl;
  int xlo = 0, xhi = T_ - 1, clo_q = 0, chi_q = T_ - 1;
  if (mk.causal) {
    xlo = max(0, q - xw);
    xhi = q;
    clo_q = max(0, q - cw);
    chi_q = q;
  }

  float m_run = -INFINITY, l_run = 0.f;  // MODE_LSE, base-2 units (the same in the four lanes of a quad)

  for (int xb = xlo; xb <= xhi; xb += kQuadRows) {
    const int x = xb + tid / LPR;
    const bool active = x <= xhi;
    float a[DQ], ay[DQ], g[DQ], u[DQ];   // ay, g: MODE_BWD only; u: the P*V sum of MODE_FWD / MODE_BWD
#pragma unroll
    for (int i = 0; i < DQ; ++i) {
      const int h = qd * DQ + i;
      a[i] = active ? qs[h] * to_f(Xp[(size_t)x * D + h]) : 0.f;
      ay[i] = 0.f;
      g[i] = 0.f;
      u[i] = 0.f;
      if (MODE == MODE_BWD && active) {
        float y = to_f(Yp[(size_t)x * D + h]);
        if (silu_y) y = silu_f(y);
        ay[i] = dor[h] * y;
      }
    }
    int clo = clo_q, chi = chi_q;
    if (mk.causal) {
      // widest column band any row of this batch can see
      const long lo = (long)xb - below, hi = (long)min(xb + kQuadRows - 1, xhi) + above;
      clo = (int)max((long)clo, lo);
      chi = (int)min((long)chi, hi);
    }
    // the next tile is fetched into registers while the current one is being used
    constexpr int kPer = kQuadCols * D / 128;   // tile elements per thread
    float rk[kPer], rv[kPer];
    auto fetch = [&](int c0) {
#pragma unroll
      for (int e = 0; e < kPer; ++e) {
        const int i = tid + e * 128;
        const int c = c0 + i / D, h = i % D;
        float kv = 0.f, vv = 0.f;
        if (c < T_) {
          kv = to_f(Kc[(size_t)c * D + h]);
          if (MODE != MODE_LSE) vv = to_f(Vc[(size_t)c * D + h]);
        }
        rk[e] = kv;
        rv[e] = vv;
      }
    };
    const int c_first = clo - (clo % kQuadCols);
    if (c_first <= chi) fetch(c_first);
    for (int c0 = c_first; c0 <= chi; c0 += kQuadCols) {
      __syncthreads();
#pragma unroll
      for (int e = 0; e < kPer; ++e) {
        const int i = tid + e * 128;
        tK[i] = rk[e];
        tV[i] = (MODE != MODE_LSE && silu_vc) ? silu_f(rv[e]) : rv[e];
      }
      __syncthreads();
      if (c0 + kQuadCols <= chi) fetch(c0 + kQuadCols);
      if (MODE == MODE_LSE) {
        // scores of the whole tile first, then one update of the running (max, sum): the exponentials of a tile
        // do not wait for one another
        float sc[kQuadCols];
        float tmax = -INFINITY;
#pragma unroll
        for (int cc = 0; cc < kQuadCols; ++cc) {
          const int c = c0 + cc;
          const int j = p.role == 0 ? c : x, k = p.role == 0 ? x : c;
          const bool ok = active && c >= clo && c <= chi && mk.valid(q, j, k);
          const float4* k4 = reinterpret_cast<const float4*>(tK + cc * D + qd * DQ);
          float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;   // four independent chains
#pragma unroll
          for (int i = 0; i < DQ / 4; ++i) {
            const float4 kv = k4[i];
            s0 = fmaf(a[4 * i], kv.x, s0);
            s1 = fmaf(a[4 * i + 1], kv.y, s1);
            s2 = fmaf(a[4 * i + 2], kv.z, s2);
            s3 = fmaf(a[4 * i + 3], kv.w, s3);
          }
          const float s = tdp_row_sum<LPR>((s0 + s1) + (s2 + s3));
          sc[cc] = ok ? s : -INFINITY;
          tmax = fmaxf(tmax, sc[cc]);
        }
        if (tmax > -INFINITY) {
          if (tmax > m_run) {
            l_run *= exp2f(m_run - tmax);   // (0 when nothing was seen before)
            m_run = tmax;
          }
          float add = 0.f;
#pragma unroll
          for (int cc = 0; cc < kQuadCols; ++cc) add += exp2f(sc[cc] - m_run);
          l_run += add;
        }
        continue;
      }
      // Columns go in groups of eight: a group no row of the warp attends is skipped; inside a group masked
      // columns run with weight 0, so that the loads and shuffles of its columns can overlap.
      for (int cg = 0; cg < kQuadCols; cg += 8) {
        bool any_ok = false;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int c = c0 + cg + e;
          any_ok = any_ok || (active && c >= clo && c <= chi && mk.valid(q, p.role == 0 ? c : x, p.role == 0 ? x : c));
        }
        if (!__any_sync(0xffffffffu, any_ok)) continue;
#pragma unroll
      for (int cc = cg; cc < cg + 8; ++cc) {
        const int c = c0 + cc;
        const int j = p.role == 0 ? c : x, k = p.role == 0 ? x : c;
        const bool ok = active && c >= clo && c <= chi && mk.valid(q, j, k);
        const float4* k4 = reinterpret_cast<const float4*>(tK + cc * D + qd * DQ);
        const float4* v4 = reinterpret_cast<const float4*>(tV + cc * D + qd * DQ);
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
        for (int i = 0; i < DQ / 4; ++i) {
          const float4 kv = k4[i];
          s0 = fmaf(a[4 * i], kv.x, s0);
          s1 = fmaf(a[4 * i + 1], kv.y, s1);
          s2 = fmaf(a[4 * i + 2], kv.z, s2);
          s3 = fmaf(a[4 * i + 3], kv.w, s3);
        }
        const float s = tdp_row_sum<LPR>((s0 + s1) + (s2 + s3));
        {
          const float pr = ok ? exp2f(s - lse2) : 0.f;
          float ds = 0.f;
          if (MODE == MODE_BWD) {
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
            for (int i = 0; i < DQ / 4; ++i) {
              const float4 vv = v4[i];
              d0 = fmaf(ay[4 * i], vv.x, d0);
              d1 = fmaf(ay[4 * i + 1], vv.y, d1);
              d2 = fmaf(ay[4 * i + 2], vv.z, d2);
              d3 = fmaf(ay[4 * i + 3], vv.w, d3);
            }
            const float dp = tdp_row_sum<LPR>((d0 + d1) + (d2 + d3));
            ds = single ? 0.f : pr * (dp - Dq);
          }
#pragma unroll
          for (int i = 0; i < DQ / 4; ++i) {
            const float4 vv = v4[i];
            u[4 * i] = fmaf(pr, vv.x, u[4 * i]);
            u[4 * i + 1] = fmaf(pr, vv.y, u[4 * i + 1]);
            u[4 * i + 2] = fmaf(pr, vv.z, u[4 * i + 2]);
            u[4 * i + 3] = fmaf(pr, vv.w, u[4 * i + 3]);
            if (MODE == MODE_BWD) {
              const float4 kv = k4[i];
              g[4 * i] = fmaf(ds, kv.x, g[4 * i]);
              g[4 * i + 1] = fmaf(ds, kv.y, g[4 * i + 1]);
              g[4 * i + 2] = fmaf(ds, kv.z, g[4 * i + 2]);
              g[4 * i + 3] = fmaf(ds, kv.w, g[4 * i + 3]);
            }
          }
        }
      }
      }
    }
    // per-row epilogue (rows that are not active hold zeros)
    if (MODE == MODE_FWD) {
#pragma unroll
      for (int i = 0; i < DQ; ++i) {
        const int h = qd * DQ + i;
        float v = active ? u[i] * to_f(Yp[(size_t)x * D + h]) : 0.f;
        v = tdp_rows_sum<LPR>(v);
        if (lane < LPR) atomicAdd(&outacc[h], v);
      }
    } else if (MODE == MODE_BWD) {
      float* dX = p.dX + base + (size_t)x * D;
      float* dY = p.dY + base + (size_t)x * D;
#pragma unroll
      for (int i = 0; i < DQ; ++i) {
        const int h = qd * DQ + i;
        const float gg = p.alpha * g[i];
        if (active) {
          atomicAdd(&dX[h], gg * qr[h]);
          atomicAdd(&dY[h], u[i] * dor[h]);
        }
        if (p.role == 0) {
          float v = active ? gg * to_f(Xp[(size_t)x * D + h]) : 0.f;
          v = tdp_rows_sum<LPR>(v);
          if (lane < LPR) atomicAdd(&outacc[h], v);
        }
      }
    }
  }

  if (MODE == MODE_LSE) {
    red[tid] = m_run;
    __syncthreads();
    for (int s = 64; s > 0; s >>= 1) {
      if (tid < s) red[tid] = fmaxf(red[tid], red[tid + s]);
      __syncthreads();
    }
    const float M = red[0];
    __syncthreads();
    // every row is held by LPR lanes: count it once
    red[tid] = (qd != 0 || m_run == -INFINITY) ? 0.f : l_run * exp2f(m_run - M);
    __syncthreads();
    for (int s = 64; s > 0; s >>= 1) {
      if (tid < s) red[tid] += red[tid + s];
      __syncthreads();
    }
    if (tid == 0) p.out_lse[(size_t)bh * T_ + q] = (M + log2f(red[0])) * kLn2;
  } else {
    __syncthreads();
    if (MODE == MODE_FWD) {
      for (int h = tid; h < D; h += 128) ((T*)p.out_o + base)[(size_t)q * D + h] = from_f<T>(outacc[h]);
    } else if (p.role == 0) {
      for (int h = tid; h < D; h += 128) ((T*)p.dq + base)[(size_t)q * D + h] = from_f<T>(outacc[h]);
    }
  }
}
