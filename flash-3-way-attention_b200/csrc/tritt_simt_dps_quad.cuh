// Register-resident variants of the three generic attention kernels of the dot-product-sum path, for
// head dimensions up to 128.  Four consecutive lanes (a "quad") own one row (forward, row-owner
// backward) or one column (column-owner backward); each lane keeps a quarter of the head dimension of
// every per-owner vector in registers, dot products are finished with two shuffles inside the quad, and
// the tiles of the other axis are staged in shared memory and read with broadcast 16-byte loads.
// Included by tritt_simt_dps.cuh after AttnParams / load_src / attn_valid are defined.
#pragma once

constexpr int kQuadOwners = 32;   // owners per CTA (128 threads)
constexpr int kQuadTile = 32;     // rows / columns of the other axis staged per step

__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

// ---------------------------------------------------------------- forward: quad per row
template <typename T, int DQ>
__global__ void __launch_bounds__(128) attn_fwd_quad(AttnParams p) {
  constexpr int D = DQ * 4;
  __shared__ __align__(16) float tK[kQuadTile * D];
  __shared__ __align__(16) float tV[kQuadTile * D];
  __shared__ float tB[kQuadTile];
  const int tid = threadIdx.x, T_ = p.T, qd = tid & 3;
  const size_t base = (size_t)blockIdx.y * T_ * D, vbase = (size_t)blockIdx.y * T_;
  const int r0 = blockIdx.x * kQuadOwners, r = r0 + (tid >> 2);
  const bool active = r < T_;
  float x[DQ], acc[DQ];
#pragma unroll
  for (int i = 0; i < DQ; ++i) {
    x[i] = active ? load_src<T>(p.xq, base + (size_t)r * D + qd * DQ + i) * p.alpha * kLog2e : 0.f;
    acc[i] = 0.f;
  }
  const int rlast = min(r0 + kQuadOwners, T_) - 1;
  int clo = 0, chi = T_ - 1;
  if (p.causal) {
    clo = max(0, r0 - p.win);
    chi = rlast;
  }
  float m = -INFINITY, l = 0.f;
  for (int c0 = clo - (clo % kQuadTile); c0 <= chi; c0 += kQuadTile) {
    __syncthreads();
    for (int i = tid; i < kQuadTile * D; i += 128) {
      const int c = c0 + i / D;
      tK[i] = c < T_ ? load_src<T>(p.kc, base + (size_t)c * D + (i % D)) : 0.f;
      tV[i] = c < T_ ? load_src<T>(p.vc, base + (size_t)c * D + (i % D)) : 0.f;
    }
    if (tid < kQuadTile) tB[tid] = (p.bias && c0 + tid < T_) ? p.bias[vbase + c0 + tid] * kLog2e : 0.f;
    __syncthreads();
    for (int cc = 0; cc < kQuadTile; ++cc) {
      const int c = c0 + cc;
      const bool ok = active && c < T_ && attn_valid(p, r, c);
      if (!__any_sync(0xffffffffu, ok)) continue;
      const float4* k4 = reinterpret_cast<const float4*>(tK + cc * D + qd * DQ);
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < DQ / 4; ++i) {
        const float4 kv = k4[i];
        s = fmaf(x[4 * i], kv.x, s);
        s = fmaf(x[4 * i + 1], kv.y, s);
        s = fmaf(x[4 * i + 2], kv.z, s);
        s = fmaf(x[4 * i + 3], kv.w, s);
      }
      s = quad_sum(s) + tB[cc];
      if (!ok) continue;
      float pr;
      if (s > m) {
        const float corr = exp2f(m - s);
        l = l * corr + 1.f;
#pragma unroll
        for (int i = 0; i < DQ; ++i) acc[i] *= corr;
        m = s;
        pr = 1.f;
      } else {
        pr = exp2f(s - m);
        l += pr;
      }
      const float4* v4 = reinterpret_cast<const float4*>(tV + cc * D + qd * DQ);
#pragma unroll
      for (int i = 0; i < DQ / 4; ++i) {
        const float4 vv = v4[i];
        acc[4 * i] = fmaf(pr, vv.x, acc[4 * i]);
        acc[4 * i + 1] = fmaf(pr, vv.y, acc[4 * i + 1]);
        acc[4 * i + 2] = fmaf(pr, vv.z, acc[4 * i + 2]);
        acc[4 * i + 3] = fmaf(pr, vv.w, acc[4 * i + 3]);
      }
    }
  }
  if (active) {
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < DQ; ++i) {
      const size_t idx = base + (size_t)r * D + qd * DQ + i;
      const float o = acc[i] * inv;
      if (p.out_f32) p.out_f32[idx] = o;
      if (p.out_t) ((T*)p.out_t)[idx] = from_f<T>(o);
    }
    if (qd == 0) p.out_lse[vbase + r] = (m + log2f(l)) * kLn2;
  }
}

// ---------------------------------------------------------------- backward: quad per row
template <typename T, int DQ>
__global__ void __launch_bounds__(128) attn_bwd_row_quad(AttnParams p) {
  constexpr int D = DQ * 4;
  __shared__ __align__(16) float tK[kQuadTile * D];
  __shared__ __align__(16) float tV[kQuadTile * D];
  __shared__ float tB[kQuadTile];
  const int tid = threadIdx.x, T_ = p.T, qd = tid & 3;
  const size_t base = (size_t)blockIdx.y * T_ * D, vbase = (size_t)blockIdx.y * T_;
  const int r0 = blockIdx.x * kQuadOwners, r = r0 + (tid >> 2);
  const bool active = r < T_;
  float x[DQ], dout[DQ], acc[DQ];
#pragma unroll
  for (int i = 0; i < DQ; ++i) {
    const size_t idx = base + (size_t)r * D + qd * DQ + i;
    x[i] = active ? load_src<T>(p.xq, idx) * p.alpha * kLog2e : 0.f;
    dout[i] = active ? load_src<T>(p.dout, idx) : 0.f;
    acc[i] = 0.f;
  }
  const float lse2 = active ? p.lse[vbase + r] * kLog2e : 0.f;
  const float dr = active ? p.drow[vbase + r] : 0.f;
  const int rlast = min(r0 + kQuadOwners, T_) - 1;
  int clo = 0, chi = T_ - 1;
  if (p.causal) {
    clo = max(0, r0 - p.win);
    chi = rlast;
  }
  for (int c0 = clo - (clo % kQuadTile); c0 <= chi; c0 += kQuadTile) {
    __syncthreads();
    for (int i = tid; i < kQuadTile * D; i += 128) {
      const int c = c0 + i / D;
      tK[i] = c < T_ ? load_src<T>(p.kc, base + (size_t)c * D + (i % D)) : 0.f;
      tV[i] = c < T_ ? load_src<T>(p.vc, base + (size_t)c * D + (i % D)) : 0.f;
    }
    if (tid < kQuadTile) tB[tid] = (p.bias && c0 + tid < T_) ? p.bias[vbase + c0 + tid] * kLog2e : 0.f;
    __syncthreads();
    for (int cc = 0; cc < kQuadTile; ++cc) {
      const int c = c0 + cc;
      const bool ok = active && c < T_ && attn_valid(p, r, c);
      if (!__any_sync(0xffffffffu, ok)) continue;
      const float4* k4 = reinterpret_cast<const float4*>(tK + cc * D + qd * DQ);
      const float4* v4 = reinterpret_cast<const float4*>(tV + cc * D + qd * DQ);
      float s = 0.f, dp = 0.f;
#pragma unroll
      for (int i = 0; i < DQ / 4; ++i) {
        const float4 kv = k4[i], vv = v4[i];
        s = fmaf(x[4 * i], kv.x, s);
        s = fmaf(x[4 * i + 1], kv.y, s);
        s = fmaf(x[4 * i + 2], kv.z, s);
        s = fmaf(x[4 * i + 3], kv.w, s);
        dp = fmaf(dout[4 * i], vv.x, dp);
        dp = fmaf(dout[4 * i + 1], vv.y, dp);
        dp = fmaf(dout[4 * i + 2], vv.z, dp);
        dp = fmaf(dout[4 * i + 3], vv.w, dp);
      }
      s = quad_sum(s) + tB[cc];
      dp = quad_sum(dp);
      if (!ok) continue;
      const float ds = exp2f(s - lse2) * (dp - dr);
#pragma unroll
      for (int i = 0; i < DQ / 4; ++i) {
        const float4 kv = k4[i];
        acc[4 * i] = fmaf(ds, kv.x, acc[4 * i]);
        acc[4 * i + 1] = fmaf(ds, kv.y, acc[4 * i + 1]);
        acc[4 * i + 2] = fmaf(ds, kv.z, acc[4 * i + 2]);
        acc[4 * i + 3] = fmaf(ds, kv.w, acc[4 * i + 3]);
      }
    }
  }
  if (active) {
#pragma unroll
    for (int i = 0; i < DQ; ++i) {
      const size_t idx = base + (size_t)r * D + qd * DQ + i;
      const float g = p.alpha * acc[i];
      if (p.d_rows_f32) p.d_rows_f32[idx] = p.d_rows_accumulate ? p.d_rows_f32[idx] + g : g;
      if (p.d_rows_t) ((T*)p.d_rows_t)[idx] = from_f<T>(p.d_rows_accumulate ? p.d_rows_f32[idx] : g);
    }
  }
}

// ---------------------------------------------------------------- backward: quad per column
template <typename T, int DQ>
__global__ void __launch_bounds__(128) attn_bwd_col_quad(AttnParams p) {
  constexpr int D = DQ * 4;
  __shared__ __align__(16) float tX[kQuadTile * D];   // rows: xq (raw)
  __shared__ __align__(16) float tD[kQuadTile * D];   // rows: dout
  __shared__ float tL[kQuadTile], tR[kQuadTile];
  const int tid = threadIdx.x, T_ = p.T, qd = tid & 3;
  const size_t base = (size_t)blockIdx.y * T_ * D, vbase = (size_t)blockIdx.y * T_;
  const int c0 = blockIdx.x * kQuadOwners, c = c0 + (tid >> 2);
  const bool active = c < T_;
  float kc[DQ], vc[DQ], dk[DQ], dv[DQ];
#pragma unroll
  for (int i = 0; i < DQ; ++i) {
    const size_t idx = base + (size_t)c * D + qd * DQ + i;
    kc[i] = active ? load_src<T>(p.kc, idx) * p.alpha * kLog2e : 0.f;
    vc[i] = active ? load_src<T>(p.vc, idx) : 0.f;
    dk[i] = 0.f;
    dv[i] = 0.f;
  }
  const float bias2 = (active && p.bias) ? p.bias[vbase + c] * kLog2e : 0.f;
  float g = 0.f;
  const int clast = min(c0 + kQuadOwners, T_) - 1;
  int rlo = 0, rhi = T_ - 1;
  if (p.causal) {
    rlo = c0;
    rhi = (int)min((long)T_ - 1, (long)clast + p.win);
  }
  for (int r0 = rlo - (rlo % kQuadTile); r0 <= rhi; r0 += kQuadTile) {
    __syncthreads();
    for (int i = tid; i < kQuadTile * D; i += 128) {
      const int r = r0 + i / D;
      tX[i] = r < T_ ? load_src<T>(p.xq, base + (size_t)r * D + (i % D)) : 0.f;
      tD[i] = r < T_ ? load_src<T>(p.dout, base + (size_t)r * D + (i % D)) : 0.f;
    }
    if (tid < kQuadTile) {
      tL[tid] = r0 + tid < T_ ? p.lse[vbase + r0 + tid] * kLog2e : 0.f;
      tR[tid] = r0 + tid < T_ ? p.drow[vbase + r0 + tid] : 0.f;
    }
    __syncthreads();
    for (int rr = 0; rr < kQuadTile; ++rr) {
      const int r = r0 + rr;
      const bool ok = active && r < T_ && attn_valid(p, r, c);
      if (!__any_sync(0xffffffffu, ok)) continue;
      const float4* x4 = reinterpret_cast<const float4*>(tX + rr * D + qd * DQ);
      const float4* d4 = reinterpret_cast<const float4*>(tD + rr * D + qd * DQ);
      float s = 0.f, dp = 0.f;
#pragma unroll
      for (int i = 0; i < DQ / 4; ++i) {
        const float4 xv = x4[i], dd = d4[i];
        s = fmaf(kc[4 * i], xv.x, s);
        s = fmaf(kc[4 * i + 1], xv.y, s);
        s = fmaf(kc[4 * i + 2], xv.z, s);
        s = fmaf(kc[4 * i + 3], xv.w, s);
        dp = fmaf(vc[4 * i], dd.x, dp);
        dp = fmaf(vc[4 * i + 1], dd.y, dp);
        dp = fmaf(vc[4 * i + 2], dd.z, dp);
        dp = fmaf(vc[4 * i + 3], dd.w, dp);
      }
      s = quad_sum(s) + bias2;
      dp = quad_sum(dp);
      if (!ok) continue;
      const float pr = exp2f(s - tL[rr]);
      const float ds = pr * (dp - tR[rr]);
      g += ds;
#pragma unroll
      for (int i = 0; i < DQ / 4; ++i) {
        const float4 xv = x4[i], dd = d4[i];
        dk[4 * i] = fmaf(ds, xv.x, dk[4 * i]);
        dk[4 * i + 1] = fmaf(ds, xv.y, dk[4 * i + 1]);
        dk[4 * i + 2] = fmaf(ds, xv.z, dk[4 * i + 2]);
        dk[4 * i + 3] = fmaf(ds, xv.w, dk[4 * i + 3]);
        dv[4 * i] = fmaf(pr, dd.x, dv[4 * i]);
        dv[4 * i + 1] = fmaf(pr, dd.y, dv[4 * i + 1]);
        dv[4 * i + 2] = fmaf(pr, dd.z, dv[4 * i + 2]);
        dv[4 * i + 3] = fmaf(pr, dd.w, dv[4 * i + 3]);
      }
    }
  }
  if (active) {
#pragma unroll
    for (int i = 0; i < DQ; ++i) {
      const size_t idx = base + (size_t)c * D + qd * DQ + i;
      const float dkv = p.alpha * dk[i];
      if (p.d_kc_f32) p.d_kc_f32[idx] = dkv;
      if (p.d_kc_t) ((T*)p.d_kc_t)[idx] = from_f<T>(dkv);
      p.d_vc_f32[idx] = dv[i];
    }
    if (p.gsum && qd == 0) p.gsum[vbase + c] = g;
  }
}
