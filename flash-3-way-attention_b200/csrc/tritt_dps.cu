// Dot-product-sum trittention: workspace layout and the sequence of launches of forward and backward, on
// either kernel family (tcgen05 soft-max attention kernels for 16-bit inputs with head dimension 64 / 128,
// CUDA-core kernels otherwise).
//
// The score S[q,s,t] = alpha (Q[q].K2[t] + K1[s].K2[t]) is separable, so the whole operator is two chained
// soft-max attentions of cost O(T^2 D):
//   inner (per K2 row t):  E[s,t] = alpha K1[s].K2[t]    over s <= t, t - s <= k_diff
//                          LSEin[t] = log sum_s exp E,    Y[t] = softmax_s(E) SiLU(V1)
//   outer (per query q):   F[q,t] = alpha Q[q].K2[t] + LSEin[t]   over t <= q
//                          O[q] = softmax_t(F) (Y*V2),    m[q] = log sum_t exp F
// (the reference recomputes the inner leg for every query block, dot_product_sum/kernels/fwd_kernel.py:102-108,
// 196-204).  The backward differentiates the two attentions in turn, each with a row-owner and a column-owner kernel.
#include "tritt_simt_dps.cuh"

namespace tritt {
namespace {

// workspace layout: the forward's state  Y [n] fp32 | LSEin [r] fp32 | SiLU(V1) [n] | Y*V2 [n]  (the last two in the
// inputs' 16-bit type, absent for fp32 inputs), then, backward only, fp32
//   Dq [r] | dW [n] | g [r] | dY [n] | Dt [r] | dK2a [n] | dsV1 [n]   and   dY [n] in the 16-bit type.
// A backward that is handed the forward's workspace (`fwd_state`) reads the state there instead of recomputing it.
// Every segment starts on a 256-byte boundary (lengths are rounded up): the tensor-core kernels store the [n]
// buffers with 16-byte vector stores, and r = B*N*T may be odd.
struct DpsWs {
  float *Y, *lse_in, *Dq, *dW, *g, *dY, *Dt, *dK2a, *dsV1;
  void *sv1_16, *w_16, *dy_16;  // tensor-core path only: SiLU(V1), Y*V2 and dY in the inputs' 16-bit type
};
size_t dps_state_bytes(size_t n, size_t r, int dtype) {
  return (align_up(n, 64) + align_up(r, 64)) * sizeof(float) + (dtype == TRITT_F32 ? 0 : 2 * align_up(n * 2, 256));
}
// The tensor-core forward serves 16-bit inputs with head dimension 64 or 128 and a non-negative k_diff.
bool dps_fwd_on_tensor_cores(const DpsArgs& a) {
  return !(a.flags & TRITT_FLAG_FORCE_SIMT) && a.k_diff >= 0 && sm100_attn_fwd_supported(a.T, a.D, a.dtype);
}
DpsWs carve(void* ws, const void* fwd_state, size_t n, size_t r, int dtype) {
  const size_t np = align_up(n, 64), rp = align_up(r, 64), h = align_up(n * 2, 256);
  DpsWs w;
  // the state: in the forward's own workspace when the caller kept it, else at the head of this one
  char* st = fwd_state ? (char*)const_cast<void*>(fwd_state) : (char*)ws;
  w.Y = (float*)st;
  w.lse_in = w.Y + np;
  w.sv1_16 = st + (np + rp) * sizeof(float);
  w.w_16 = (char*)w.sv1_16 + h;
  float* f = (float*)((char*)ws + dps_state_bytes(n, r, dtype));
  w.Dq = f; f += rp;
  w.dW = f; f += np;
  w.g = f; f += rp;
  w.dY = f; f += np;
  w.Dt = f; f += rp;
  w.dK2a = f; f += np;
  w.dsV1 = f; f += np;
  w.dy_16 = f;  // (16-bit inputs only)
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
  DpsWs w = carve(a.workspace, nullptr, n, r, a.dtype);
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
  int rc = 0;
  // Y, LSEin, SiLU(V1), Y*V2: taken from the forward's workspace when the caller kept it, else computed again
  if (!a.fwd_state && (rc = dps_fwd_tensor_cores(a, w, true))) return rc;
  // ---- outer attention: rows q (Q), columns t (K2, W = Y*V2, bias LSEin).  The row owner also forms
  // Dq = sum_h dO O per query and leaves it for the column owner; the column owner's epilogue turns dW into
  // dV2 = dW * Y, dY = dW * V2 and the inner attention's row term Dt = sum_h dY Y - sum_q dS.
  AttnBwdTcArgs o{};
  o.xq = a.q; o.kc = a.k2; o.vc = w.w_16; o.dout = a.d_o;
  o.bias = w.lse_in; o.lse = a.m_in; o.drow = w.Dq;
  o.BN = a.B * a.N; o.T = a.T; o.D = a.D; o.dtype = a.dtype; o.causal = a.causal; o.win = a.T;
  o.alpha = a.alpha; o.status = a.status_word; o.stream = a.stream;
  AttnBwdTcArgs orow = o;
  orow.d_rows_t = a.dq;
  orow.out_rows = a.o; orow.drow_out = w.Dq;
  if ((rc = sm100_attn_bwd_rows(orow))) return rc;
  AttnBwdTcArgs ocol = o;
  ocol.d_kc_f32 = w.dK2a;
  ocol.mid_y = w.Y; ocol.mid_v2 = a.v2; ocol.mid_dv2 = a.dv2; ocol.mid_dy_t = w.dy_16; ocol.mid_dt = w.Dt;
  if ((rc = sm100_attn_bwd_cols(ocol))) return rc;
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
  icol.d_kc_t = a.dk1;
  icol.silu_src = a.v1; icol.d_vc_t = a.dv1;  // dV1 = dSiLU(V1) * SiLU'(V1) in the epilogue
  return sm100_attn_bwd_cols(icol);
}

template <typename T>
int dps_bwd_t(const DpsArgs& a) {
  const size_t n = (size_t)a.B * a.N * a.T * a.D, r = (size_t)a.B * a.N * a.T;
  DpsWs w = carve(a.workspace, a.fwd_state, n, r, a.dtype);
  if (dps_fwd_on_tensor_cores(a)) return dps_bwd_tensor_cores<T>(a, w);
  const int BN = a.B * a.N;
  // inner leg again (Y, LSEin) unless the caller kept the forward's workspace
  int rc = a.fwd_state ? 0 : dps_inner_fwd<T>(a, w);
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

size_t dps_workspace(int op, int B, int N, int T, int D, int dtype) {
  const size_t n = (size_t)B * N * T * D, r = (size_t)B * N * T;
  const size_t np = align_up(n, 64), rp = align_up(r, 64);
  const size_t state = dps_state_bytes(n, r, dtype);
  if (op == TRITT_OP_DPS_FWD) return state;
  return state + (4 * np + 3 * rp) * sizeof(float) + (dtype == TRITT_F32 ? 0 : align_up(n * 2, 256));
}

int dps_fwd(const DpsArgs& a) {
  switch (a.dtype) {
    case TRITT_F32: return dps_fwd_t<float>(a);
    case TRITT_F16: return dps_fwd_t<__half>(a);
    case TRITT_BF16: return dps_fwd_t<__nv_bfloat16>(a);
  }
  set_error("unknown dtype %d", a.dtype);
  return -1;
}

int dps_bwd(const DpsArgs& a) {
  switch (a.dtype) {
    case TRITT_F32: return dps_bwd_t<float>(a);
    case TRITT_F16: return dps_bwd_t<__half>(a);
    case TRITT_BF16: return dps_bwd_t<__nv_bfloat16>(a);
  }
  set_error("unknown dtype %d", a.dtype);
  return -1;
}

}  // namespace tritt
