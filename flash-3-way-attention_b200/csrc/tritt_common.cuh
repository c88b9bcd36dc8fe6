// Shared helpers for the trittention kernels: dtype conversion, error reporting,
// the attention-mask predicates, and launch-argument bundles.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/tritt.h"

namespace tritt {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---------------------------------------------------------------- error reporting
void set_error(const char* fmt, ...);
void count_launch();  // bumps the process-wide count of kernels this library has enqueued
const char* get_error();
unsigned long long launches();

#define TRITT_CUDA_OK(expr)                                                              \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess) {                                                             \
      ::tritt::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return (int)_e;                                                                    \
    }                                                                                    \
  } while (0)

// ---------------------------------------------------------------- dtype helpers
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float silu_grad_f(float x) {
  float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

inline size_t dtype_size(int dtype) { return dtype == TRITT_F32 ? 4 : 2; }

// ---------------------------------------------------------------- masks
// Triple-dot-product mask (reference triple_dot_product/kernels/utils.py:75-90 and
// trittention_pytorch.py:68-75): (q, j, k) is attended iff
//   j <= q <= j + k1w,  k <= q <= k + k2w,  k - kkl <= j <= k + kkr     (causal)
// and always when not causal.  Windows are normalised on the host so that
// "unlimited" (anything >= T) equals T; negative windows are refused at the entry points.
struct TdpMask {
  int causal, T, k1w, k2w, kkl, kkr;
  __host__ __device__ bool valid(int q, int j, int k) const {
    if (!causal) return true;
    return j <= q && q - j <= k1w && k <= q && q - k <= k2w && k - j <= kkl && j - k <= kkr;
  }
  // Query q attends the single pair (q, q) (or, not causal, T == 1).  Its soft-max is then the constant 1 and the
  // gradient of its scores is exactly zero; the backward kernels use that instead of forming P (dP - Dq), whose two
  // terms agree only up to the 16-bit rounding of the stored output when P = 1.
  // (Another pair exists iff one of (q-1, q), (q, q-1), (q-1, q-1) is attended.)
  __host__ __device__ bool single_pair(int q) const {
    if (!causal) return T == 1;
    if (q == 0) return true;
    return !((k1w >= 1 && kkl >= 1) || (k2w >= 1 && kkr >= 1) || (k1w >= 1 && k2w >= 1));
  }
  // full windows: the mask is the plain "j <= q and k <= q" wedge
  __host__ __device__ bool full_windows() const {
    return !causal || (k1w >= T - 1 && k2w >= T - 1 && kkl >= T - 1 && kkr >= T - 1);
  }
};

inline TdpMask make_tdp_mask(int causal, int T, int k1w, int k2w, int kkl, int kkr) {
  auto norm = [T](int w) { return w > T ? T : (w < 0 ? 0 : w); };
  return TdpMask{causal ? 1 : 0, T, norm(k1w), norm(k2w), norm(kkl), norm(kkr)};
}

// ---------------------------------------------------------------- argument bundle
struct TdpArgs {
  const void *q, *k1, *k2, *v1, *v2, *o, *d_o;
  const float* lse_in;  // backward: saved log-sum-exp
  void *out_o;          // forward output
  float* out_lse;
  void *dq, *dk1, *dk2, *dv1, *dv2;
  int B, N, T, D, dtype;
  float alpha;
  TdpMask mask;
  int q_mod, q_rem;
  void* workspace;
  size_t workspace_bytes;
  int* status_word;
  int flags;
  cudaStream_t stream;
};

struct DpsArgs {
  const void *q, *k1, *k2, *v1, *v2, *o, *d_o;
  const float* m_in;
  void* out_o;
  float* out_m;
  void *dq, *dk1, *dk2, *dv1, *dv2;
  int B, N, T, D, dtype;
  float alpha;
  int causal, k_diff;
  void* workspace;
  size_t workspace_bytes;
  const void* fwd_state;  // backward: the forward call's workspace, still holding Y, LSEin, SiLU(V1), Y*V2 (or null)
  int* status_word;
  int flags;
  cudaStream_t stream;
};

// kernel families (defined in their own translation units)
int simt_tdp_fwd(const TdpArgs& a);
int simt_tdp_bwd(const TdpArgs& a);
int simt_tdp_bwd_finalize(const void* v1, void* dk1, void* dk2, void* dv1, void* dv2, size_t n_elems, int dtype,
                          const float* partials, cudaStream_t stream);
size_t simt_tdp_workspace(int op, int B, int N, int T, int D, int dtype);

int dps_fwd(const DpsArgs& a);
int dps_bwd(const DpsArgs& a);
size_t dps_workspace(int op, int B, int N, int T, int D, int dtype);

bool sm100_tdp_supported(int op, int T, int D, int dtype, const TdpMask& m);
int sm100_tdp_fwd(const TdpArgs& a);
int sm100_tdp_bwd(const TdpArgs& a);
size_t sm100_tdp_workspace(int op, int B, int N, int T, int D, int dtype);
size_t sm100_tdp_bwd_workspace(int B, int N, int T, int D);
size_t sm100_tdp_fwd_optional_workspace(int B, int N, int T, int D, int dtype);
// forward kernel for causal masks with a narrow (j, k) band (tiles of four queries x 32 K2 rows)
bool sm100_tdp_fwd_band_applies(int T, const TdpMask& m);
int sm100_tdp_fwd_band(const TdpArgs& a, const void* sv1, const float* k1n);

// fp32 inputs, and bf16 inputs with TRITT_FLAG_WIDE_OPERANDS, on the tensor cores through fp16 operand copies
bool tdp_wide_applies(int op, int T, int D, int dtype, const TdpMask& m, int flags);
size_t tdp_wide_workspace(int op, int B, int N, int T, int D);
int tdp_wide_fwd(const TdpArgs& a);
int tdp_wide_bwd(const TdpArgs& a);

// Two-way soft-max attention forward on the tensor cores (16-bit operands [BN, T, D], head dimension 64 or 128):
// out[r] = softmax_c(alpha x[r].k[c] + bias[c]) v[c] over the columns with (not causal, or c <= r <= c + win).
struct AttnTcArgs {
  const void *xq, *kc, *vc;  // row operand, column keys, column values
  const float* bias;         // [BN, T] per column, natural-log units, or null
  float* out_f32;            // [BN, T, D] fp32 result, or null
  void* out_t;               // the same in the operands' type, or null
  const void* mul;           // with out_mul: out_mul = out * mul element-wise, in the operands' type
  void* out_mul;
  float* out_lse;            // [BN, T] natural-log log-sum-exp of the rows
  int BN, T, D, dtype, causal, win;
  float alpha;
  int* status;
  cudaStream_t stream;
};
bool sm100_attn_fwd_supported(int T, int D, int dtype);
int sm100_attn_fwd(const AttnTcArgs& a);
int sm100_silu_16(const void* in, void* out, size_t n, int dtype, cudaStream_t stream);  // out = SiLU(in), 16-bit

// Backward of the same attention, as a row-owner and a column-owner kernel.  With P = exp(alpha x.k + bias - lse),
// dP = dout.v and dS = P (dP - drow):  rows: d_rows_t = alpha sum_c dS k (+ d_rows_add);  columns: d_vc_f32 =
// sum_r P dout, d_kc = alpha sum_r dS x (fp32 or the operands' type), gsum = sum_r dS.
struct AttnBwdTcArgs {
  const void *xq, *kc, *vc, *dout;  // 16-bit [BN, T, D]
  const float *bias, *lse, *drow;   // [BN, T]: per column (or null), per row, per row
  // row owner: with `out_rows` (the attention's 16-bit output) drow[r] = dout[r] . out_rows[r] is computed by the
  // kernel, used, and stored to `drow_out` for the column-owner launch that follows
  const void* out_rows;
  float* drow_out;
  void* d_rows_t;
  const float* d_rows_add;          // [BN, T, D] or null
  float* d_kc_f32;
  void* d_kc_t;
  float* d_vc_f32;                  // column owner: sum_r P dout, fp32, or null when one of the two forms below is asked
  // column owner, instead of d_vc_f32: d_vc_t = d_vc * SiLU'(silu_src)  (16-bit; silu_src = the raw value tensor)
  const void* silu_src;
  void* d_vc_t;
  // column owner, instead of d_vc_f32 (with dW = d_vc): mid_dv2 = dW * mid_y, mid_dy_t = dW * mid_v2 (both 16-bit),
  // mid_dt[c] = sum_h (dW mid_v2 mid_y)[c, h] - gsum[c]
  const float* mid_y;
  const void* mid_v2;
  void *mid_dv2, *mid_dy_t;
  float* mid_dt;
  float* gsum;                      // [BN, T] or null
  int BN, T, D, dtype, causal, win;
  float alpha;
  int* status;
  cudaStream_t stream;
};
int sm100_attn_bwd_rows(const AttnBwdTcArgs& a);
int sm100_attn_bwd_cols(const AttnBwdTcArgs& a);

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace tritt
