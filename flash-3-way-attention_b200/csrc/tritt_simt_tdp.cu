// Plain CUDA-core (fp32) kernels for triple-dot-product trittention.
//
// This is the general path: any dtype, any power-of-two head dimension, every window
// combination.  It computes in fp32 and is what fp32 inputs and narrow-window calls run
// on; the tensor-core path takes over for the shapes it supports.
//
// (Head dimensions 16 to 128 run the register-resident variant in tritt_simt_tdp_quad.cuh: four or eight lanes
// per pair row; the kernel below keeps the per-row vectors in shared memory and serves the other dimensions.)
// One thread owns one "pair row" (q, x): x indexes K2/V2 (role 0) or K1/V1 (role 1) and
// the thread walks the other key axis c, so that a row behaves like an ordinary
// attention query with the pre-scaled vector a[h] = alpha*Q[q,h]*X[x,h]:
//   s = a . Kc[c],  p = exp(s - lse[q]),  dp = (dO[q]*Y[x]) . Vc[c],  ds = p (dp - Dq)
//   G[h] += ds Kc[c,h],  U[h] += p Vc[c,h]
// Role 0 gives dQ, dK2, dV2; role 1 (the same kernel with the two key axes swapped - the
// score and the gated value are symmetric under that swap) gives dK1 and dSiLU(V1).
// The reference computes the same quantities with one Triton kernel per gradient
// (triple_dot_product/kernels/bwd_dq.py, bwd_dk1.py, bwd_dk2.py, bwd_dv1.py, bwd_dv2.py).
#include "tritt_common.cuh"

namespace tritt {
namespace {

constexpr int kTileC = 16;  // key rows staged in shared memory per step

enum { MODE_LSE = 0, MODE_FWD = 1, MODE_BWD = 2 };

struct SimtTdpParams {
  const void *q, *k1, *k2, *v1, *v2, *o, *d_o;
  const float* lse;  // MODE_FWD / MODE_BWD: natural-log lse per row
  float* out_lse;    // MODE_LSE
  void* out_o;       // MODE_FWD
  void* dq;          // MODE_BWD role 0
  float *dX, *dY;    // MODE_BWD: fp32 accumulators for the row-side tensors
  int T, D, nq;
  float alpha;
  TdpMask mask;
  int q_mod, q_rem, role;
};

template <int MODE> __host__ __device__ constexpr int num_vecs() { return MODE == MODE_LSE ? 1 : (MODE == MODE_FWD ? 2 : 4); }

template <typename T, int MODE>
__global__ void tdp_simt_kernel(SimtTdpParams p) {
  extern __shared__ float smem[];
  const int NT = blockDim.x, tid = threadIdx.x, D = p.D, T_ = p.T;
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

  // shared memory carve-up
  constexpr int NV = num_vecs<MODE>();
  float* vec = smem;                      // [NV][D][NT]
  float* tK = vec + (size_t)NV * D * NT;  // [kTileC][D]
  float* tV = tK + kTileC * D;            // [kTileC][D]
  float* qs = tV + kTileC * D;            // [D] alpha*log2e*Q[q]
  float* qr = qs + D;                     // [D] Q[q]
  float* dor = qr + D;                    // [D] dO[q]
  float* outacc = dor + D;                // [D]
  float* red = outacc + D;                // [2*NT]
#define VEC(v, h) vec[((size_t)(v)*D + (h)) * NT + tid]

  for (int h = tid; h < D; h += NT) {
    float qv = to_f(Q[(size_t)q * D + h]);
    qr[h] = qv;
    qs[h] = qv * p.alpha * kLog2e;
    outacc[h] = 0.f;
    if (MODE == MODE_BWD) dor[h] = to_f(((const T*)p.d_o + base)[(size_t)q * D + h]);
  }
  float lse2 = 0.f, Dq = 0.f;
  if (MODE != MODE_LSE) lse2 = p.lse[(size_t)bh * T_ + q] * kLog2e;
  if (MODE == MODE_BWD) {
    // Dq = sum_h dO[q,h] * O[q,h]  (reference flash_trittention.py:167)
    float part = 0.f;
    for (int h = tid; h < D; h += NT)
      part += to_f(((const T*)p.d_o + base)[(size_t)q * D + h]) * to_f(((const T*)p.o + base)[(size_t)q * D + h]);
    red[tid] = part;
    __syncthreads();
    for (int s = NT / 2; s > 0; s >>= 1) {
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

  float m_run = -INFINITY, l_run = 0.f;  // MODE_LSE, base-2 units

  for (int xb = xlo; xb <= xhi; xb += NT) {
    const int x = xb + tid;
    const bool active = x <= xhi;
    if (active) {
      for (int h = 0; h < D; ++h) {
        VEC(0, h) = qs[h] * to_f(Xp[(size_t)x * D + h]);
        if (MODE == MODE_FWD) VEC(1, h) = 0.f;
        if (MODE == MODE_BWD) {
          float y = to_f(Yp[(size_t)x * D + h]);
          if (silu_y) y = silu_f(y);
          VEC(1, h) = dor[h] * y;
          VEC(2, h) = 0.f;
          VEC(3, h) = 0.f;
        }
      }
    }
    int clo = clo_q, chi = chi_q;
    if (mk.causal) {
      // widest column band any row of this batch can see
      long lo = (long)xb - below, hi = (long)min(xb + NT - 1, xhi) + above;
      clo = (int)max((long)clo, lo);
      chi = (int)min((long)chi, hi);
    }
    for (int c0 = clo - (clo % kTileC); c0 <= chi; c0 += kTileC) {
      __syncthreads();
      for (int i = tid; i < kTileC * D; i += NT) {
        int c = c0 + i / D, h = i % D;
        float kv = 0.f, vv = 0.f;
        if (c < T_) {
          kv = to_f(Kc[(size_t)c * D + h]);
          if (MODE != MODE_LSE) {
            vv = to_f(Vc[(size_t)c * D + h]);
            if (silu_vc) vv = silu_f(vv);
          }
        }
        tK[i] = kv;
        tV[i] = vv;
      }
      __syncthreads();
      if (!active) continue;
      for (int cc = 0; cc < kTileC; ++cc) {
        const int c = c0 + cc;
        if (c < clo || c > chi) continue;
        const int j = p.role == 0 ? c : x, k = p.role == 0 ? x : c;
        if (!mk.valid(q, j, k)) continue;
        float s = 0.f;
        for (int h = 0; h < D; ++h) s = fmaf(VEC(0, h), tK[cc * D + h], s);
        if (MODE == MODE_LSE) {
          if (s > m_run) {
            l_run = l_run * exp2f(m_run - s) + 1.f;
            m_run = s;
          } else {
            l_run += exp2f(s - m_run);
          }
        } else {
          const float pr = exp2f(s - lse2);
          if (MODE == MODE_FWD) {
            for (int h = 0; h < D; ++h) VEC(1, h) = fmaf(pr, tV[cc * D + h], VEC(1, h));
          } else {
            float dp = 0.f;
            for (int h = 0; h < D; ++h) dp = fmaf(VEC(1, h), tV[cc * D + h], dp);
            const float ds = single ? 0.f : pr * (dp - Dq);
            for (int h = 0; h < D; ++h) {
              VEC(2, h) = fmaf(ds, tK[cc * D + h], VEC(2, h));
              VEC(3, h) = fmaf(pr, tV[cc * D + h], VEC(3, h));
            }
          }
        }
      }
    }
    // per-row epilogue
    if (active) {
      if (MODE == MODE_FWD) {
        for (int h = 0; h < D; ++h) atomicAdd(&outacc[h], VEC(1, h) * to_f(Yp[(size_t)x * D + h]));
      } else if (MODE == MODE_BWD) {
        float* dX = p.dX + base + (size_t)x * D;
        float* dY = p.dY + base + (size_t)x * D;
        for (int h = 0; h < D; ++h) {
          const float g = p.alpha * VEC(2, h);
          atomicAdd(&dX[h], g * qr[h]);
          atomicAdd(&dY[h], VEC(3, h) * dor[h]);
          if (p.role == 0) atomicAdd(&outacc[h], g * to_f(Xp[(size_t)x * D + h]));
        }
      }
    }
  }

  if (MODE == MODE_LSE) {
    red[tid] = m_run;
    __syncthreads();
    for (int s = NT / 2; s > 0; s >>= 1) {
      if (tid < s) red[tid] = fmaxf(red[tid], red[tid + s]);
      __syncthreads();
    }
    const float M = red[0];
    __syncthreads();
    red[tid] = (m_run == -INFINITY) ? 0.f : l_run * exp2f(m_run - M);
    __syncthreads();
    for (int s = NT / 2; s > 0; s >>= 1) {
      if (tid < s) red[tid] += red[tid + s];
      __syncthreads();
    }
    if (tid == 0) p.out_lse[(size_t)bh * T_ + q] = (M + log2f(red[0])) * kLn2;
  } else {
    __syncthreads();
    if (MODE == MODE_FWD) {
      for (int h = tid; h < D; h += NT) ((T*)p.out_o + base)[(size_t)q * D + h] = from_f<T>(outacc[h]);
    } else if (p.role == 0) {
      for (int h = tid; h < D; h += NT) ((T*)p.dq + base)[(size_t)q * D + h] = from_f<T>(outacc[h]);
    }
  }
#undef VEC
}

#include "tritt_simt_tdp_quad.cuh"

template <typename T>
__global__ void tdp_finalize_kernel(const T* v1, T* dk1, T* dk2, T* dv1, T* dv2, const float* part, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  dk1[i] = from_f<T>(part[i]);
  dk2[i] = from_f<T>(part[n + i]);
  dv1[i] = from_f<T>(part[2 * n + i] * silu_grad_f(to_f(v1[i])));
  dv2[i] = from_f<T>(part[3 * n + i]);
}

int pick_threads(int nvec, int D) {
  // per-thread vectors live in shared memory: nvec * D * NT * 4 bytes, keep below ~128 KiB
  int nt = 128;
  while (nt > 32 && (size_t)nvec * D * nt * 4 > (128u << 10)) nt >>= 1;
  return nt;
}

size_t smem_bytes(int nvec, int D, int nt) {
  return ((size_t)nvec * D * nt + 2 * kTileC * D + 4 * D + 2 * nt) * sizeof(float);
}

template <typename T, int MODE, int DQ, int LPR>
int launch_quad(const SimtTdpParams& p, int BN, cudaStream_t stream) {
  if (p.nq <= 0) return 0;
  tdp_simt_quad_kernel<T, MODE, DQ, LPR><<<dim3(p.nq, BN), 128, 0, stream>>>(p);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}

template <typename T, int MODE>
int launch(const SimtTdpParams& p, int BN, cudaStream_t stream) {
  // head dimensions 16 to 128: the register-resident kernels (four lanes per row, eight at 128)
  if (p.D == 128) return launch_quad<T, MODE, 16, 8>(p, BN, stream);
  if (p.D == 64) return launch_quad<T, MODE, 16, 4>(p, BN, stream);
  if (p.D == 32) return launch_quad<T, MODE, 8, 4>(p, BN, stream);
  if (p.D == 16) return launch_quad<T, MODE, 4, 4>(p, BN, stream);
  constexpr int NV = num_vecs<MODE>();
  const int nt = pick_threads(NV, p.D);
  const size_t sm = smem_bytes(NV, p.D, nt);
  if (sm > (200u << 10)) {
    set_error("head dimension %d is too large for the CUDA-core path", p.D);
    return -1;
  }
  auto kern = tdp_simt_kernel<T, MODE>;
  TRITT_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
  if (p.nq <= 0) return 0;
  kern<<<dim3(p.nq, BN), nt, sm, stream>>>(p);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}

template <int MODE>
int launch_dtype(const SimtTdpParams& p, int BN, int dtype, cudaStream_t stream) {
  switch (dtype) {
    case TRITT_F32: return launch<float, MODE>(p, BN, stream);
    case TRITT_F16: return launch<__half, MODE>(p, BN, stream);
    case TRITT_BF16: return launch<__nv_bfloat16, MODE>(p, BN, stream);
  }
  set_error("unknown dtype %d", dtype);
  return -1;
}

SimtTdpParams base_params(const TdpArgs& a) {
  SimtTdpParams p{};
  p.q = a.q; p.k1 = a.k1; p.k2 = a.k2; p.v1 = a.v1; p.v2 = a.v2; p.o = a.o; p.d_o = a.d_o;
  p.T = a.T; p.D = a.D;
  p.alpha = a.alpha;
  p.mask = a.mask;
  p.q_mod = a.q_mod; p.q_rem = a.q_rem;
  p.nq = a.q_rem < a.T ? (a.T - a.q_rem + a.q_mod - 1) / a.q_mod : 0;
  return p;
}

}  // namespace

size_t simt_tdp_workspace(int op, int B, int N, int T, int D, int /*dtype*/) {
  if (op == TRITT_OP_TDP_BWD) return 4 * (size_t)B * N * T * D * sizeof(float);
  return 0;
}

int simt_tdp_fwd(const TdpArgs& a) {
  SimtTdpParams p = base_params(a);
  p.role = 0;
  p.out_lse = a.out_lse;
  int rc = launch_dtype<MODE_LSE>(p, a.B * a.N, a.dtype, a.stream);
  if (rc) return rc;
  p.lse = a.out_lse;
  p.out_o = a.out_o;
  return launch_dtype<MODE_FWD>(p, a.B * a.N, a.dtype, a.stream);
}

int simt_tdp_bwd_finalize(const void* v1, void* dk1, void* dk2, void* dv1, void* dv2, size_t n, int dtype,
                          const float* part, cudaStream_t stream) {
  const int nt = 256;
  const unsigned nb = (unsigned)((n + nt - 1) / nt);
  if (n == 0) return 0;
  switch (dtype) {
    case TRITT_F32:
      tdp_finalize_kernel<float><<<nb, nt, 0, stream>>>((const float*)v1, (float*)dk1, (float*)dk2, (float*)dv1, (float*)dv2, part, n);
      count_launch();
      break;
    case TRITT_F16:
      tdp_finalize_kernel<__half><<<nb, nt, 0, stream>>>((const __half*)v1, (__half*)dk1, (__half*)dk2, (__half*)dv1, (__half*)dv2, part, n);
      count_launch();
      break;
    case TRITT_BF16:
      tdp_finalize_kernel<__nv_bfloat16><<<nb, nt, 0, stream>>>((const __nv_bfloat16*)v1, (__nv_bfloat16*)dk1, (__nv_bfloat16*)dk2, (__nv_bfloat16*)dv1, (__nv_bfloat16*)dv2, part, n);
      count_launch();
      break;
    default:
      set_error("unknown dtype %d", dtype);
      return -1;
  }
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}

int simt_tdp_bwd(const TdpArgs& a) {
  const size_t n = (size_t)a.B * a.N * a.T * a.D;
  float* part = (float*)a.workspace;
  TRITT_CUDA_OK(cudaMemsetAsync(part, 0, 4 * n * sizeof(float), a.stream));
  SimtTdpParams p = base_params(a);
  p.lse = a.lse_in;
  p.dq = a.dq;
  // role 0: rows (q, k): dQ, dK2, dV2
  p.role = 0;
  p.dX = part + n;      // dK2
  p.dY = part + 3 * n;  // dV2
  int rc = launch_dtype<MODE_BWD>(p, a.B * a.N, a.dtype, a.stream);
  if (rc) return rc;
  // role 1: rows (q, j): dK1, dSiLU(V1)
  p.role = 1;
  p.dX = part;          // dK1
  p.dY = part + 2 * n;  // dSiLU(V1)
  rc = launch_dtype<MODE_BWD>(p, a.B * a.N, a.dtype, a.stream);
  if (rc) return rc;
  if (a.flags & TRITT_FLAG_BWD_PARTIAL) return 0;
  return simt_tdp_bwd_finalize(a.v1, a.dk1, a.dk2, a.dv1, a.dv2, n, a.dtype, part, a.stream);
}

}  // namespace tritt
