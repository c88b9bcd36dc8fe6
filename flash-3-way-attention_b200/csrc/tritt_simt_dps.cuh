// CUDA-core (fp32) soft-max attention kernels of the dot-product-sum path: generic forward, row-owner and
// column-owner backward, the small element-wise passes between them, and their launchers.  Included by
// tritt_dps.cu (the one translation unit that sequences them).
//
// The score S[q,s,t] = alpha (Q[q].K2[t] + K1[s].K2[t]) is separable, so the whole
// operator is two chained soft-max attentions of cost O(T^2 D):
//   inner (per K2 row t):  E[s,t] = alpha K1[s].K2[t]    over s <= t, t - s <= k_diff
//                          LSEin[t] = log sum_s exp E,    Y[t] = softmax_s(E) SiLU(V1)
//   outer (per query q):   F[q,t] = alpha Q[q].K2[t] + LSEin[t]   over t <= q
//                          O[q] = softmax_t(F) (Y*V2),    m[q] = log sum_t exp F
// The reference kernels use the same two-level log-sum-exp but recompute the inner leg
// for every query block (dot_product_sum/kernels/fwd_kernel.py:102-108,196-204); here it
// is computed once.  Backward differentiates the two attentions in turn; each uses a
// row-owner kernel (gradient of the "query" side) and a column-owner kernel (gradients
// of the "key"/"value" side), so no atomics are needed.
#pragma once
#include "tritt_common.cuh"

namespace tritt {
namespace {

constexpr int kTile = 16;

// A [rows, D] operand that is read element-wise through one of a few recipes.
enum { SRC_RAW = 0, SRC_F32 = 1, SRC_SILU = 2, SRC_F32_TIMES_RAW = 3 };
struct Src {
  const void* p;
  const void* p2;
  int kind;
};
template <typename T>
__device__ __forceinline__ float load_src(const Src& s, size_t i) {
  switch (s.kind) {
    case SRC_RAW: return to_f(((const T*)s.p)[i]);
    case SRC_F32: return ((const float*)s.p)[i];
    case SRC_SILU: return silu_f(to_f(((const T*)s.p)[i]));
    default: return ((const float*)s.p)[i] * to_f(((const T*)s.p2)[i]);
  }
}

struct AttnParams {
  Src xq, kc, vc, dout;     // rows: xq/dout, columns: kc/vc
  const float* bias;        // per column, natural-log units, may be null
  const float* lse;         // per row (backward), natural log
  const float* drow;        // per row (backward): sum_h dout*out (minus extra terms)
  float* out_f32;           // forward: fp32 output rows (may be null)
  void* out_t;              // forward: dtype output rows (may be null)
  float* out_lse;           // forward
  // backward outputs
  float* d_rows_f32; void* d_rows_t; int d_rows_accumulate;  // row-owner: alpha * sum_c dS Kc
  float* d_kc_f32; void* d_kc_t;                            // col-owner: alpha * sum_r dS Xq
  float* d_vc_f32;                                          // col-owner: sum_r P dout
  float* gsum;                                              // col-owner: sum_r dS
  int T, D, causal, win;
  float alpha;
};

// valid(r, c): not causal, or c <= r and r - c <= win
__device__ __forceinline__ bool attn_valid(const AttnParams& p, int r, int c) {
  return !p.causal || (c <= r && r - c <= p.win);
}

// ---------------------------------------------------------------- forward, thread per row
template <typename T>
__global__ void attn_fwd_kernel(AttnParams p) {
  extern __shared__ float smem[];
  const int NT = blockDim.x, tid = threadIdx.x, D = p.D, T_ = p.T;
  const size_t base = (size_t)blockIdx.y * T_ * D, vbase = (size_t)blockIdx.y * T_;
  float* vec = smem;                      // [2][D][NT]: x, acc
  float* tK = vec + (size_t)2 * D * NT;   // [kTile][D]
  float* tV = tK + kTile * D;
  float* tB = tV + kTile * D;             // [kTile]
#define VEC(v, h) vec[((size_t)(v)*D + (h)) * NT + tid]
  const int r0 = blockIdx.x * NT, r = r0 + tid;
  const bool active = r < T_;
  if (active)
    for (int h = 0; h < D; ++h) {
      VEC(0, h) = load_src<T>(p.xq, base + (size_t)r * D + h) * p.alpha * kLog2e;
      VEC(1, h) = 0.f;
    }
  const int rlast = min(r0 + NT, T_) - 1;
  int clo = 0, chi = T_ - 1;
  if (p.causal) {
    clo = max(0, r0 - p.win);
    chi = rlast;
  }
  float m = -INFINITY, l = 0.f;
  for (int c0 = clo - (clo % kTile); c0 <= chi; c0 += kTile) {
    __syncthreads();
    for (int i = tid; i < kTile * D; i += NT) {
      int c = c0 + i / D;
      tK[i] = c < T_ ? load_src<T>(p.kc, base + (size_t)c * D + (i % D)) : 0.f;
      tV[i] = c < T_ ? load_src<T>(p.vc, base + (size_t)c * D + (i % D)) : 0.f;
    }
    if (tid < kTile) tB[tid] = (p.bias && c0 + tid < T_) ? p.bias[vbase + c0 + tid] * kLog2e : 0.f;
    __syncthreads();
    if (!active) continue;
    for (int cc = 0; cc < kTile; ++cc) {
      const int c = c0 + cc;
      if (c >= T_ || !attn_valid(p, r, c)) continue;
      float s = tB[cc];
      for (int h = 0; h < D; ++h) s = fmaf(VEC(0, h), tK[cc * D + h], s);
      float pr;
      if (s > m) {
        const float corr = exp2f(m - s);
        l = l * corr + 1.f;
        for (int h = 0; h < D; ++h) VEC(1, h) *= corr;
        m = s;
        pr = 1.f;
      } else {
        pr = exp2f(s - m);
        l += pr;
      }
      for (int h = 0; h < D; ++h) VEC(1, h) = fmaf(pr, tV[cc * D + h], VEC(1, h));
    }
  }
  if (active) {
    const float inv = 1.f / l;
    for (int h = 0; h < D; ++h) {
      const float o = VEC(1, h) * inv;
      if (p.out_f32) p.out_f32[base + (size_t)r * D + h] = o;
      if (p.out_t) ((T*)p.out_t)[base + (size_t)r * D + h] = from_f<T>(o);
    }
    p.out_lse[vbase + r] = (m + log2f(l)) * kLn2;
  }
#undef VEC
}

// ---------------------------------------------------------------- backward, thread per row
template <typename T>
__global__ void attn_bwd_row_kernel(AttnParams p) {
  extern __shared__ float smem[];
  const int NT = blockDim.x, tid = threadIdx.x, D = p.D, T_ = p.T;
  const size_t base = (size_t)blockIdx.y * T_ * D, vbase = (size_t)blockIdx.y * T_;
  float* vec = smem;                      // [3][D][NT]: x, dout, acc
  float* tK = vec + (size_t)3 * D * NT;
  float* tV = tK + kTile * D;
  float* tB = tV + kTile * D;
#define VEC(v, h) vec[((size_t)(v)*D + (h)) * NT + tid]
  const int r0 = blockIdx.x * NT, r = r0 + tid;
  const bool active = r < T_;
  float lse2 = 0.f, dr = 0.f;
  if (active) {
    for (int h = 0; h < D; ++h) {
      VEC(0, h) = load_src<T>(p.xq, base + (size_t)r * D + h) * p.alpha * kLog2e;
      VEC(1, h) = load_src<T>(p.dout, base + (size_t)r * D + h);
      VEC(2, h) = 0.f;
    }
    lse2 = p.lse[vbase + r] * kLog2e;
    dr = p.drow[vbase + r];
  }
  const int rlast = min(r0 + NT, T_) - 1;
  int clo = 0, chi = T_ - 1;
  if (p.causal) {
    clo = max(0, r0 - p.win);
    chi = rlast;
  }
  for (int c0 = clo - (clo % kTile); c0 <= chi; c0 += kTile) {
    __syncthreads();
    for (int i = tid; i < kTile * D; i += NT) {
      int c = c0 + i / D;
      tK[i] = c < T_ ? load_src<T>(p.kc, base + (size_t)c * D + (i % D)) : 0.f;
      tV[i] = c < T_ ? load_src<T>(p.vc, base + (size_t)c * D + (i % D)) : 0.f;
    }
    if (tid < kTile) tB[tid] = (p.bias && c0 + tid < T_) ? p.bias[vbase + c0 + tid] * kLog2e : 0.f;
    __syncthreads();
    if (!active) continue;
    for (int cc = 0; cc < kTile; ++cc) {
      const int c = c0 + cc;
      if (c >= T_ || !attn_valid(p, r, c)) continue;
      float s = tB[cc], dp = 0.f;
      for (int h = 0; h < D; ++h) {
        s = fmaf(VEC(0, h), tK[cc * D + h], s);
        dp = fmaf(VEC(1, h), tV[cc * D + h], dp);
      }
      const float ds = exp2f(s - lse2) * (dp - dr);
      for (int h = 0; h < D; ++h) VEC(2, h) = fmaf(ds, tK[cc * D + h], VEC(2, h));
    }
  }
  if (active)
    for (int h = 0; h < D; ++h) {
      const size_t i = base + (size_t)r * D + h;
      const float g = p.alpha * VEC(2, h);
      if (p.d_rows_f32) p.d_rows_f32[i] = p.d_rows_accumulate ? p.d_rows_f32[i] + g : g;
      if (p.d_rows_t) ((T*)p.d_rows_t)[i] = from_f<T>(p.d_rows_accumulate ? p.d_rows_f32[i] : g);
    }
#undef VEC
}

// ---------------------------------------------------------------- backward, thread per column
template <typename T>
__global__ void attn_bwd_col_kernel(AttnParams p) {
  extern __shared__ float smem[];
  const int NT = blockDim.x, tid = threadIdx.x, D = p.D, T_ = p.T;
  const size_t base = (size_t)blockIdx.y * T_ * D, vbase = (size_t)blockIdx.y * T_;
  float* vec = smem;                      // [4][D][NT]: kc, vc, dKc acc, dVc acc
  float* tX = vec + (size_t)4 * D * NT;   // [kTile][D] rows: xq (scaled)
  float* tXr = tX + kTile * D;            // rows: xq raw
  float* tD = tXr + kTile * D;            // rows: dout
  float* tL = tD + kTile * D;             // [kTile] lse2
  float* tR = tL + kTile;                 // [kTile] drow
#define VEC(v, h) vec[((size_t)(v)*D + (h)) * NT + tid]
  const int c0 = blockIdx.x * NT, c = c0 + tid;
  const bool active = c < T_;
  float bias2 = 0.f, g = 0.f;
  if (active) {
    for (int h = 0; h < D; ++h) {
      VEC(0, h) = load_src<T>(p.kc, base + (size_t)c * D + h);
      VEC(1, h) = load_src<T>(p.vc, base + (size_t)c * D + h);
      VEC(2, h) = 0.f;
      VEC(3, h) = 0.f;
    }
    if (p.bias) bias2 = p.bias[vbase + c] * kLog2e;
  }
  const int clast = min(c0 + NT, T_) - 1;
  int rlo = 0, rhi = T_ - 1;
  if (p.causal) {
    rlo = c0;
    rhi = (int)min((long)T_ - 1, (long)clast + p.win);
  }
  for (int r0 = rlo - (rlo % kTile); r0 <= rhi; r0 += kTile) {
    __syncthreads();
    for (int i = tid; i < kTile * D; i += NT) {
      int r = r0 + i / D;
      float x = r < T_ ? load_src<T>(p.xq, base + (size_t)r * D + (i % D)) : 0.f;
      tXr[i] = x;
      tX[i] = x * p.alpha * kLog2e;
      tD[i] = r < T_ ? load_src<T>(p.dout, base + (size_t)r * D + (i % D)) : 0.f;
    }
    if (tid < kTile) {
      tL[tid] = r0 + tid < T_ ? p.lse[vbase + r0 + tid] * kLog2e : 0.f;
      tR[tid] = r0 + tid < T_ ? p.drow[vbase + r0 + tid] : 0.f;
    }
    __syncthreads();
    if (!active) continue;
    for (int rr = 0; rr < kTile; ++rr) {
      const int r = r0 + rr;
      if (r >= T_ || !attn_valid(p, r, c)) continue;
      float s = bias2, dp = 0.f;
      for (int h = 0; h < D; ++h) {
        s = fmaf(VEC(0, h), tX[rr * D + h], s);
        dp = fmaf(VEC(1, h), tD[rr * D + h], dp);
      }
      const float pr = exp2f(s - tL[rr]);
      const float ds = pr * (dp - tR[rr]);
      g += ds;
      for (int h = 0; h < D; ++h) {
        VEC(2, h) = fmaf(ds, tXr[rr * D + h], VEC(2, h));
        VEC(3, h) = fmaf(pr, tD[rr * D + h], VEC(3, h));
      }
    }
  }
  if (active) {
    for (int h = 0; h < D; ++h) {
      const size_t i = base + (size_t)c * D + h;
      const float dk = p.alpha * VEC(2, h);
      if (p.d_kc_f32) p.d_kc_f32[i] = dk;
      if (p.d_kc_t) ((T*)p.d_kc_t)[i] = from_f<T>(dk);
      p.d_vc_f32[i] = VEC(3, h);
    }
    if (p.gsum) p.gsum[vbase + c] = g;
  }
#undef VEC
}

// Dq[r] = sum_h dO*O  (reference dot_product_sum/kernels/bwd_preprocess.py:5-49)
// out[r] = sum_h a[r,h] b[r,h]; a warp per row, so that consecutive lanes read consecutive elements
template <typename T>
__global__ void rowdot_kernel(const T* a, const T* b, float* out, size_t rows, int D) {
  const size_t r = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  float s = 0.f;
  for (int h = lane; h < D; h += 32) s += to_f(a[r * D + h]) * to_f(b[r * D + h]);
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) out[r] = s;
}

// Between the two backward attentions: dW (gradient of Y*V2) splits into dV2 = dW*Y and
// dY = dW*V2; the inner attention's row term is Dt = sum_h dY*Y - g.
template <typename T>
__global__ void dps_mid_kernel(const float* dW, const float* Y, const T* v2, const float* g, T* dv2, float* dY,
                               float* Dt, size_t rows, int D, T* dY_t = nullptr) {
  // a warp per row, so that consecutive lanes touch consecutive elements
  const size_t r = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  float acc = 0.f;
  for (int h = lane; h < D; h += 32) {
    const size_t i = r * D + h;
    const float dw = dW[i], y = Y[i];
    dv2[i] = from_f<T>(dw * y);
    const float dy = dw * to_f(v2[i]);
    dY[i] = dy;
    if (dY_t) dY_t[i] = from_f<T>(dy);  // operand of the tensor-core inner backward
    acc += dy * y;
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) Dt[r] = acc - g[r];
}

template <typename T>
__global__ void dps_dv1_kernel(const float* dsv1, const T* v1, T* dv1, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dv1[i] = from_f<T>(dsv1[i] * silu_grad_f(to_f(v1[i])));
}

int pick_threads(int nvec, int D) {
  int nt = 128;
  while (nt > 32 && (size_t)nvec * D * nt * 4 > (128u << 10)) nt >>= 1;
  return nt;
}

#include "tritt_simt_dps_quad.cuh"

enum { ATTN_FWD = 0, ATTN_BWD_ROW = 1, ATTN_BWD_COL = 2 };

// Register-resident kernels for head dimensions 16..128 (a quad of lanes per owner).
template <typename T, int DQ>
int launch_quad(int kind, const AttnParams& p, int BN, cudaStream_t stream) {
  const dim3 grid((p.T + kQuadOwners - 1) / kQuadOwners, BN);
  switch (kind) {
    case ATTN_FWD: attn_fwd_quad<T, DQ><<<grid, 128, 0, stream>>>(p); break;
    case ATTN_BWD_ROW: attn_bwd_row_quad<T, DQ><<<grid, 128, 0, stream>>>(p); break;
    default: attn_bwd_col_quad<T, DQ><<<grid, 128, 0, stream>>>(p); break;
  }
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}

template <typename K>
int launch_attn(K kern, const AttnParams& p, int nvec, int ntiles, int BN, cudaStream_t stream) {
  const int nt = pick_threads(nvec, p.D);
  const size_t sm = ((size_t)nvec * p.D * nt + (size_t)ntiles * kTile * p.D + 4 * kTile) * sizeof(float);
  if (sm > (200u << 10)) {
    set_error("head dimension %d is too large for the CUDA-core path", p.D);
    return -1;
  }
  TRITT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
  kern<<<dim3((p.T + nt - 1) / nt, BN), nt, sm, stream>>>(p);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}

// Picks the register-resident kernels when the head dimension allows, else the shared-memory ones.
template <typename T>
int run_attn(int kind, const AttnParams& p, int BN, cudaStream_t stream) {
  switch (p.D) {
    case 16: return launch_quad<T, 4>(kind, p, BN, stream);
    case 32: return launch_quad<T, 8>(kind, p, BN, stream);
    case 64: return launch_quad<T, 16>(kind, p, BN, stream);
    case 128: return launch_quad<T, 32>(kind, p, BN, stream);
    default: break;
  }
  if (kind == ATTN_FWD) return launch_attn(attn_fwd_kernel<T>, p, 2, 2, BN, stream);
  if (kind == ATTN_BWD_ROW) return launch_attn(attn_bwd_row_kernel<T>, p, 3, 2, BN, stream);
  return launch_attn(attn_bwd_col_kernel<T>, p, 4, 3, BN, stream);
}

}  // namespace
}  // namespace tritt
