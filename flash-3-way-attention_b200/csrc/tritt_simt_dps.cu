// CUDA-core (fp32) kernels for dot-product-sum trittention.
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

// workspace layout (floats): Y [n] | LSEin [r] | then, backward only:
//   Dq [r] | dW [n] | g [r] | dY [n] | Dt [r] | dK2a [n] | dsV1 [n]
struct DpsWs {
  float *Y, *lse_in, *Dq, *dW, *g, *dY, *Dt, *dK2a, *dsV1;
  void *sv1_16, *w_16, *dy_16;  // tensor-core path only: SiLU(V1), Y*V2 and dY in the inputs' 16-bit type
};
size_t dps_float_bytes(int op, size_t n, size_t r) {
  return align_up((op == TRITT_OP_DPS_FWD ? n + r : 5 * n + 4 * r) * sizeof(float), 256);
}
// The tensor-core forward serves 16-bit inputs with head dimension 64 or 128 and a non-negative k_diff.
bool dps_fwd_on_tensor_cores(const DpsArgs& a) {
  return !(a.flags & TRITT_FLAG_FORCE_SIMT) && a.k_diff >= 0 && sm100_attn_fwd_supported(a.T, a.D, a.dtype);
}
DpsWs carve(void* ws, size_t n, size_t r, int op) {
  float* f = (float*)ws;
  DpsWs w;
  w.Y = f; f += n;
  w.lse_in = f; f += r;
  w.Dq = f; f += r;
  w.dW = f; f += n;
  w.g = f; f += r;
  w.dY = f; f += n;
  w.Dt = f; f += r;
  w.dK2a = f; f += n;
  w.dsV1 = f;
  w.sv1_16 = (char*)ws + dps_float_bytes(op, n, r);
  w.w_16 = (char*)w.sv1_16 + align_up(n * 2, 256);
  w.dy_16 = (char*)w.w_16 + align_up(n * 2, 256);  // (backward only)
  return w;
}

// Both legs of the forward on the tensor cores: Y (fp32), LSEin and the outer leg's value operand Y*V2; then,
// unless `inner_only`, O and m.
int dps_fwd_tensor_cores(const DpsArgs& a, const DpsWs& w, bool inner_only) {
  const size_t n = (size_t)a.B * a.N * a.T * a.D;
  int rc = sm100_silu_16(a.v1, w.sv1_16, n, a.dtype, a.stream);
  if (rc) return rc;
  AttnTcArgs t{};
  t.xq = a.k2; t.kc = a.k1; t.vc = w.sv1_16;
  t.out_f32 = w.Y; t.out_lse = w.lse_in;
  t.mul = a.v2; t.out_mul = w.w_16;
  t.BN = a.B * a.N; t.T = a.T; t.D = a.D; t.dtype = a.dtype; t.causal = a.causal; t.win = a.k_diff;
  t.alpha = a.alpha; t.status = a.status_word; t.stream = a.stream;
  if ((rc = sm100_attn_fwd(t)) || inner_only) return rc;
  AttnTcArgs u{};
  u.xq = a.q; u.kc = a.k2; u.vc = w.w_16;
  u.bias = w.lse_in;
  u.out_t = a.out_o; u.out_lse = a.out_m;
  u.BN = a.B * a.N; u.T = a.T; u.D = a.D; u.dtype = a.dtype; u.causal = a.causal; u.win = a.T;
  u.alpha = a.alpha; u.status = a.status_word; u.stream = a.stream;
  return sm100_attn_fwd(u);
}

template <typename T>
int dps_inner_fwd(const DpsArgs& a, const DpsWs& w) {
  AttnParams p{};
  p.xq = Src{a.k2, nullptr, SRC_RAW};
  p.kc = Src{a.k1, nullptr, SRC_RAW};
  p.vc = Src{a.v1, nullptr, SRC_SILU};
  p.out_f32 = w.Y;
  p.out_lse = w.lse_in;
  p.T = a.T; p.D = a.D; p.causal = a.causal; p.win = a.k_diff; p.alpha = a.alpha;
  return run_attn<T>(ATTN_FWD, p, a.B * a.N, a.stream);
}

template <typename T>
int dps_fwd_t(const DpsArgs& a) {
  const size_t n = (size_t)a.B * a.N * a.T * a.D, r = (size_t)a.B * a.N * a.T;
  DpsWs w = carve(a.workspace, n, r, TRITT_OP_DPS_FWD);
  if (dps_fwd_on_tensor_cores(a)) return dps_fwd_tensor_cores(a, w, false);
  int rc = dps_inner_fwd<T>(a, w);
  if (rc) return rc;
  AttnParams p{};
  p.xq = Src{a.q, nullptr, SRC_RAW};
  p.kc = Src{a.k2, nullptr, SRC_RAW};
  p.vc = Src{w.Y, a.v2, SRC_F32_TIMES_RAW};
  p.bias = w.lse_in;
  p.out_t = a.out_o;
  p.out_lse = a.out_m;
  p.T = a.T; p.D = a.D; p.causal = a.causal; p.win = a.T; p.alpha = a.alpha;
  return run_attn<T>(ATTN_FWD, p, a.B * a.N, a.stream);
}

// Backward with every attention product on the tensor cores (same eligibility as the forward).
template <typename T>
int dps_bwd_tensor_cores(const DpsArgs& a, const DpsWs& w) {
  const size_t n = (size_t)a.B * a.N * a.T * a.D, r = (size_t)a.B * a.N * a.T;
  int rc = dps_fwd_tensor_cores(a, w, true);  // Y, LSEin, Y*V2 again: cheaper than saving them
  if (rc) return rc;
  rowdot_kernel<T><<<(unsigned)((r + 3) / 4), 128, 0, a.stream>>>((const T*)a.d_o, (const T*)a.o, w.Dq, r, a.D);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  // ---- outer attention: rows q (Q), columns t (K2, W = Y*V2, bias LSEin)
  AttnBwdTcArgs o{};
  o.xq = a.q; o.kc = a.k2; o.vc = w.w_16; o.dout = a.d_o;
  o.bias = w.lse_in; o.lse = a.m_in; o.drow = w.Dq;
  o.BN = a.B * a.N; o.T = a.T; o.D = a.D; o.dtype = a.dtype; o.causal = a.causal; o.win = a.T;
  o.alpha = a.alpha; o.status = a.status_word; o.stream = a.stream;
  AttnBwdTcArgs orow = o;
  orow.d_rows_t = a.dq;
  if ((rc = sm100_attn_bwd_rows(orow))) return rc;
  AttnBwdTcArgs ocol = o;
  ocol.d_kc_f32 = w.dK2a; ocol.d_vc_f32 = w.dW; ocol.gsum = w.g;
  if ((rc = sm100_attn_bwd_cols(ocol))) return rc;
  dps_mid_kernel<T><<<(unsigned)((r + 3) / 4), 128, 0, a.stream>>>(w.dW, w.Y, (const T*)a.v2, w.g, (T*)a.dv2, w.dY,
                                                                        w.Dt, r, a.D, (T*)w.dy_16);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  // ---- inner attention: rows t (K2), columns s (K1, SiLU(V1)); upstream gradient dY
  AttnBwdTcArgs i{};
  i.xq = a.k2; i.kc = a.k1; i.vc = w.sv1_16; i.dout = w.dy_16;
  i.lse = w.lse_in; i.drow = w.Dt;
  i.BN = a.B * a.N; i.T = a.T; i.D = a.D; i.dtype = a.dtype; i.causal = a.causal; i.win = a.k_diff;
  i.alpha = a.alpha; i.status = a.status_word; i.stream = a.stream;
  AttnBwdTcArgs irow = i;
  irow.d_rows_t = a.dk2;      // dK2 = (as outer key) + (as inner query)
  irow.d_rows_add = w.dK2a;
  if ((rc = sm100_attn_bwd_rows(irow))) return rc;
  AttnBwdTcArgs icol = i;
  icol.d_kc_t = a.dk1; icol.d_vc_f32 = w.dsV1;
  if ((rc = sm100_attn_bwd_cols(icol))) return rc;
  dps_dv1_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, a.stream>>>(w.dsV1, (const T*)a.v1, (T*)a.dv1, n);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}

template <typename T>
int dps_bwd_t(const DpsArgs& a) {
  const size_t n = (size_t)a.B * a.N * a.T * a.D, r = (size_t)a.B * a.N * a.T;
  DpsWs w = carve(a.workspace, n, r, TRITT_OP_DPS_BWD);
  if (dps_fwd_on_tensor_cores(a)) return dps_bwd_tensor_cores<T>(a, w);
  const int BN = a.B * a.N;
  // inner leg again (Y, LSEin): cheaper than saving it between forward and backward
  int rc = dps_inner_fwd<T>(a, w);
  if (rc) return rc;
  rowdot_kernel<T><<<(unsigned)((r + 3) / 4), 128, 0, a.stream>>>((const T*)a.d_o, (const T*)a.o, w.Dq, r, a.D);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  // ---- outer attention: rows q (Q), columns t (K2, W = Y*V2, bias LSEin)
  AttnParams p{};
  p.xq = Src{a.q, nullptr, SRC_RAW};
  p.kc = Src{a.k2, nullptr, SRC_RAW};
  p.vc = Src{w.Y, a.v2, SRC_F32_TIMES_RAW};
  p.dout = Src{a.d_o, nullptr, SRC_RAW};
  p.bias = w.lse_in;
  p.lse = a.m_in;
  p.drow = w.Dq;
  p.T = a.T; p.D = a.D; p.causal = a.causal; p.win = a.T; p.alpha = a.alpha;
  AttnParams pr = p;
  pr.d_rows_t = a.dq;
  rc = run_attn<T>(ATTN_BWD_ROW, pr, BN, a.stream);
  if (rc) return rc;
  AttnParams pc = p;
  pc.d_kc_f32 = w.dK2a;
  pc.d_vc_f32 = w.dW;
  pc.gsum = w.g;
  rc = run_attn<T>(ATTN_BWD_COL, pc, BN, a.stream);
  if (rc) return rc;
  dps_mid_kernel<T><<<(unsigned)((r + 3) / 4), 128, 0, a.stream>>>(w.dW, w.Y, (const T*)a.v2, w.g, (T*)a.dv2, w.dY,
                                                                        w.Dt, r, a.D);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  // ---- inner attention: rows t (K2), columns s (K1, SiLU(V1)); upstream gradient dY
  AttnParams q{};
  q.xq = Src{a.k2, nullptr, SRC_RAW};
  q.kc = Src{a.k1, nullptr, SRC_RAW};
  q.vc = Src{a.v1, nullptr, SRC_SILU};
  q.dout = Src{w.dY, nullptr, SRC_F32};
  q.lse = w.lse_in;
  q.drow = w.Dt;
  q.T = a.T; q.D = a.D; q.causal = a.causal; q.win = a.k_diff; q.alpha = a.alpha;
  AttnParams qr = q;
  qr.d_rows_f32 = w.dK2a;  // dK2 = (as outer key) + (as inner query)
  qr.d_rows_t = a.dk2;
  qr.d_rows_accumulate = 1;
  rc = run_attn<T>(ATTN_BWD_ROW, qr, BN, a.stream);
  if (rc) return rc;
  AttnParams qc = q;
  qc.d_kc_t = a.dk1;
  qc.d_vc_f32 = w.dsV1;
  rc = run_attn<T>(ATTN_BWD_COL, qc, BN, a.stream);
  if (rc) return rc;
  dps_dv1_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, a.stream>>>(w.dsV1, (const T*)a.v1, (T*)a.dv1, n);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace

size_t simt_dps_workspace(int op, int B, int N, int T, int D, int dtype) {
  const size_t n = (size_t)B * N * T * D, r = (size_t)B * N * T;
  // SiLU(V1), Y*V2 and (backward) dY in the inputs' type
  const size_t scratch16 = dtype == TRITT_F32 ? 0 : (op == TRITT_OP_DPS_FWD ? 2 : 3) * align_up(n * 2, 256);
  return dps_float_bytes(op, n, r) + scratch16;
}

int simt_dps_fwd(const DpsArgs& a) {
  switch (a.dtype) {
    case TRITT_F32: return dps_fwd_t<float>(a);
    case TRITT_F16: return dps_fwd_t<__half>(a);
    case TRITT_BF16: return dps_fwd_t<__nv_bfloat16>(a);
  }
  set_error("unknown dtype %d", a.dtype);
  return -1;
}

int simt_dps_bwd(const DpsArgs& a) {
  switch (a.dtype) {
    case TRITT_F32: return dps_bwd_t<float>(a);
    case TRITT_F16: return dps_bwd_t<__half>(a);
    case TRITT_BF16: return dps_bwd_t<__nv_bfloat16>(a);
  }
  set_error("unknown dtype %d", a.dtype);
  return -1;
}

}  // namespace tritt
