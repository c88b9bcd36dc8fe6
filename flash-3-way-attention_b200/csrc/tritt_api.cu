// extern "C" entry points of libtritt_sm100.so: argument checks and dispatch between
// the tensor-core (tcgen05) kernels and the general CUDA-core kernels.
#include "tritt_common.cuh"

#include <atomic>
#include <cstring>

namespace tritt {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
const char* get_error() { return g_err; }

static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
unsigned long long launches() { return g_launches.load(std::memory_order_relaxed); }

namespace {

bool pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

int check_common(const void* const* ptrs, int nptr, int B, int N, int T, int D, int dtype) {
  if (B <= 0 || N <= 0 || T <= 0 || D <= 0) {
    set_error("B, N, T, D must be positive (got %d, %d, %d, %d)", B, N, T, D);
    return -1;
  }
  if (!pow2(D)) {
    set_error("head_dim must be a power of 2, got %d", D);
    return -2;
  }
  if (dtype != TRITT_F32 && dtype != TRITT_F16 && dtype != TRITT_BF16) {
    set_error("unknown dtype code %d", dtype);
    return -3;
  }
  for (int i = 0; i < nptr; ++i) {
    if (!ptrs[i]) {
      set_error("null tensor pointer (argument %d)", i);
      return -4;
    }
    if ((uintptr_t)ptrs[i] & 15) {
      set_error("tensor pointer %d is not 16-byte aligned", i);
      return -5;
    }
  }
  return 0;
}

int check_ws(size_t need, void* ws, size_t have) {
  if (need == 0) return 0;
  if (!ws || have < need) {
    set_error("workspace too small: need %zu bytes, got %zu", need, ws ? have : (size_t)0);
    return -6;
  }
  if ((uintptr_t)ws & 255) {
    set_error("workspace must be 256-byte aligned");
    return -7;
  }
  return 0;
}

// Windows are distances: the reference applies negative values literally (a negative k1 / k2 window or k_diff leaves
// query rows without any attended pair, whose soft-max is undefined), so they are refused here instead.
int check_windows(int causal, int a, int b, int c, int d) {
  if (causal && (a < 0 || b < 0 || c < 0 || d < 0)) {
    set_error("window arguments must be >= 0 (got %d, %d, %d, %d); pass T or more for an unlimited window", a, b, c, d);
    return -10;
  }
  return 0;
}

// B*N is a grid dimension of the CUDA-core kernels.
int check_heads(int B, int N) {
  if ((long long)B * N > 65535) {
    set_error("B*N = %lld exceeds the 65535 (batch*head) slices one call can take; split the batch", (long long)B * N);
    return -11;
  }
  return 0;
}

int check_shard(int q_mod, int q_rem) {
  if (q_mod < 1 || q_rem < 0 || q_rem >= q_mod) {
    set_error("invalid query shard (q_mod=%d, q_rem=%d)", q_mod, q_rem);
    return -8;
  }
  return 0;
}

bool use_sm100(int op, int T, int D, int dtype, const TdpMask& m, int flags) {
  if (flags & TRITT_FLAG_FORCE_SIMT) return false;
  return sm100_tdp_supported(op, T, D, dtype, m);
}

}  // namespace
}  // namespace tritt

using namespace tritt;

extern "C" {

int tritt_version(void) { return 100; }

unsigned long long tritt_kernel_launches(void) { return tritt::launches(); }

const char* tritt_last_error(void) { return get_error(); }

int tritt_tdp_path(int op, int T, int D, int dtype, int causal, int k1_window, int k2_window, int kk_left,
                   int kk_right, int flags) {
  TdpMask m = make_tdp_mask(causal, T, k1_window, k2_window, kk_left, kk_right);
  if (tdp_wide_applies(op, T, D, dtype, m, flags)) return TRITT_PATH_TCGEN05;
  return use_sm100(op, T, D, dtype, m, flags) ? TRITT_PATH_TCGEN05 : TRITT_PATH_SIMT;
}

int tritt_dps_path(int T, int D, int dtype, int k_diff, int flags) {
  const bool tc = !(flags & TRITT_FLAG_FORCE_SIMT) && k_diff >= 0 && sm100_attn_fwd_supported(T, D, dtype);
  return tc ? TRITT_PATH_TCGEN05 : TRITT_PATH_SIMT;
}

size_t tritt_workspace_bytes(int op, int B, int N, int T, int D, int dtype) {
  return tritt_workspace_bytes_flags(op, B, N, T, D, dtype, 0);
}

size_t tritt_workspace_bytes_flags(int op, int B, int N, int T, int D, int dtype, int flags) {
  if (B <= 0 || N <= 0 || T <= 0 || D <= 0) return 0;
  size_t a = 0, b = 0;
  switch (op) {
    case TRITT_OP_TDP_FWD:
    case TRITT_OP_TDP_BWD: {
      a = simt_tdp_workspace(op, B, N, T, D, dtype);
      b = sm100_tdp_workspace(op, B, N, T, D, dtype);
      if (op == TRITT_OP_TDP_FWD && b) b += sm100_tdp_fwd_optional_workspace(B, N, T, D, dtype);
      const TdpMask any = make_tdp_mask(1, T, T, T, T, T);
      if (tdp_wide_applies(op, T, D, dtype, any, flags)) {
        const size_t w = tdp_wide_workspace(op, B, N, T, D);
        b = w > b ? w : b;
      }
      break;
    }
    case TRITT_OP_DPS_FWD:
    case TRITT_OP_DPS_BWD:
      a = dps_workspace(op, B, N, T, D, dtype);
      break;
    default:
      return 0;
  }
  return align_up(a > b ? a : b, 256);
}

size_t tritt_tdp_bwd_partials_offset(int, int, int, int, int) { return 0; }

// Bytes of scratch the forward cannot run without on the kernel family it will take (the optional tail of the
// tensor-core forward is not counted).  Shared with the allocation-free entry point.
size_t tritt_tdp_fwd_min_workspace(int B, int N, int T, int D, int dtype, int causal, int k1_window, int k2_window,
                                   int kk_left, int kk_right, int flags) {
  const TdpMask m = make_tdp_mask(causal, T, k1_window, k2_window, kk_left, kk_right);
  if (tdp_wide_applies(TRITT_OP_TDP_FWD, T, D, dtype, m, flags))
    return tdp_wide_workspace(TRITT_OP_TDP_FWD, B, N, T, D) - sm100_tdp_fwd_optional_workspace(B, N, T, D, TRITT_F16);
  if (use_sm100(TRITT_OP_TDP_FWD, T, D, dtype, m, flags)) return sm100_tdp_workspace(TRITT_OP_TDP_FWD, B, N, T, D, dtype);
  return simt_tdp_workspace(TRITT_OP_TDP_FWD, B, N, T, D, dtype);
}

int tritt_tdp_fwd(const void* q, const void* k1, const void* k2, const void* v1, const void* v2, void* o,
                  float* lse, int B, int N, int T, int D, int dtype, float alpha, int causal, int k1_window,
                  int k2_window, int kk_left, int kk_right, int q_mod, int q_rem, void* workspace,
                  size_t workspace_bytes, int* status_word, int flags, tritt_stream_t stream) {
  const void* ptrs[] = {q, k1, k2, v1, v2, o, lse};
  int rc = check_common(ptrs, 7, B, N, T, D, dtype);
  if (rc) return rc;
  if ((rc = check_shard(q_mod, q_rem))) return rc;
  if ((rc = check_heads(B, N))) return rc;
  if ((rc = check_windows(causal, k1_window, k2_window, kk_left, kk_right))) return rc;
  TdpArgs a{};
  a.q = q; a.k1 = k1; a.k2 = k2; a.v1 = v1; a.v2 = v2;
  a.out_o = o; a.out_lse = lse;
  a.B = B; a.N = N; a.T = T; a.D = D; a.dtype = dtype; a.alpha = alpha;
  a.mask = make_tdp_mask(causal, T, k1_window, k2_window, kk_left, kk_right);
  a.q_mod = q_mod; a.q_rem = q_rem;
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  a.status_word = status_word; a.flags = flags; a.stream = (cudaStream_t)stream;
  const bool wide = tdp_wide_applies(TRITT_OP_TDP_FWD, T, D, dtype, a.mask, flags);
  const bool fast = use_sm100(TRITT_OP_TDP_FWD, T, D, dtype, a.mask, flags);
  const size_t need = tritt_tdp_fwd_min_workspace(B, N, T, D, dtype, causal, k1_window, k2_window, kk_left, kk_right, flags);
  if ((rc = check_ws(need, workspace, workspace_bytes))) return rc;
  if (wide) return tdp_wide_fwd(a);
  return fast ? sm100_tdp_fwd(a) : simt_tdp_fwd(a);
}

int tritt_tdp_bwd(const void* q, const void* k1, const void* k2, const void* v1, const void* v2, const void* o,
                  const void* d_o, const float* lse, void* dq, void* dk1, void* dk2, void* dv1, void* dv2, int B,
                  int N, int T, int D, int dtype, float alpha, int causal, int k1_window, int k2_window,
                  int kk_left, int kk_right, int q_mod, int q_rem, void* workspace, size_t workspace_bytes,
                  int* status_word, int flags, tritt_stream_t stream) {
  const bool partial = flags & TRITT_FLAG_BWD_PARTIAL;
  const void* ptrs[] = {q, k1, k2, v1, v2, o, d_o, lse, dq, partial ? q : dk1, partial ? q : dk2,
                        partial ? q : dv1, partial ? q : dv2};
  int rc = check_common(ptrs, 13, B, N, T, D, dtype);
  if (rc) return rc;
  if ((rc = check_shard(q_mod, q_rem))) return rc;
  if ((rc = check_heads(B, N))) return rc;
  if ((rc = check_windows(causal, k1_window, k2_window, kk_left, kk_right))) return rc;
  if (!partial && q_mod != 1) {
    set_error("a query-sharded backward yields partial key-side sums: pass TRITT_FLAG_BWD_PARTIAL");
    return -9;
  }
  TdpArgs a{};
  a.q = q; a.k1 = k1; a.k2 = k2; a.v1 = v1; a.v2 = v2; a.o = o; a.d_o = d_o; a.lse_in = lse;
  a.dq = dq; a.dk1 = dk1; a.dk2 = dk2; a.dv1 = dv1; a.dv2 = dv2;
  a.B = B; a.N = N; a.T = T; a.D = D; a.dtype = dtype; a.alpha = alpha;
  a.mask = make_tdp_mask(causal, T, k1_window, k2_window, kk_left, kk_right);
  a.q_mod = q_mod; a.q_rem = q_rem;
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  a.status_word = status_word; a.flags = flags; a.stream = (cudaStream_t)stream;
  const bool wide = tdp_wide_applies(TRITT_OP_TDP_BWD, T, D, dtype, a.mask, flags);
  const bool fast = use_sm100(TRITT_OP_TDP_BWD, T, D, dtype, a.mask, flags);
  const size_t need = wide   ? tdp_wide_workspace(TRITT_OP_TDP_BWD, B, N, T, D)
                      : fast ? sm100_tdp_workspace(TRITT_OP_TDP_BWD, B, N, T, D, dtype)
                             : simt_tdp_workspace(TRITT_OP_TDP_BWD, B, N, T, D, dtype);
  if ((rc = check_ws(need, workspace, workspace_bytes))) return rc;
  if (wide) return tdp_wide_bwd(a);
  return fast ? sm100_tdp_bwd(a) : simt_tdp_bwd(a);
}

int tritt_tdp_bwd_finalize(const void* v1, void* dk1, void* dk2, void* dv1, void* dv2, int B, int N, int T, int D,
                           int dtype, void* workspace, size_t workspace_bytes, tritt_stream_t stream) {
  const void* ptrs[] = {v1, dk1, dk2, dv1, dv2};
  int rc = check_common(ptrs, 5, B, N, T, D, dtype);
  if (rc) return rc;
  const size_t n = (size_t)B * N * T * D;
  if ((rc = check_ws(4 * n * sizeof(float), workspace, workspace_bytes))) return rc;
  return simt_tdp_bwd_finalize(v1, dk1, dk2, dv1, dv2, n, dtype, (const float*)workspace, (cudaStream_t)stream);
}

static int norm_kdiff(int k_diff, int T) { return k_diff > T ? T : k_diff; }

int tritt_dps_fwd(const void* q, const void* k1, const void* k2, const void* v1, const void* v2, void* o, float* m,
                  int B, int N, int T, int D, int dtype, float alpha, int causal, int k_diff, void* workspace,
                  size_t workspace_bytes, int* status_word, int flags, tritt_stream_t stream) {
  const void* ptrs[] = {q, k1, k2, v1, v2, o, m};
  int rc = check_common(ptrs, 7, B, N, T, D, dtype);
  if (rc) return rc;
  if ((rc = check_heads(B, N))) return rc;
  if ((rc = check_windows(causal, k_diff, 0, 0, 0))) return rc;
  if ((rc = check_ws(dps_workspace(TRITT_OP_DPS_FWD, B, N, T, D, dtype), workspace, workspace_bytes))) return rc;
  DpsArgs a{};
  a.q = q; a.k1 = k1; a.k2 = k2; a.v1 = v1; a.v2 = v2; a.out_o = o; a.out_m = m;
  a.B = B; a.N = N; a.T = T; a.D = D; a.dtype = dtype; a.alpha = alpha;
  a.causal = causal ? 1 : 0; a.k_diff = norm_kdiff(k_diff, T);
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  a.status_word = status_word; a.flags = flags; a.stream = (cudaStream_t)stream;
  return dps_fwd(a);
}

static int dps_bwd_entry(const void* q, const void* k1, const void* k2, const void* v1, const void* v2, const void* o,
                         const void* d_o, const float* m, void* dq, void* dk1, void* dk2, void* dv1, void* dv2, int B,
                         int N, int T, int D, int dtype, float alpha, int causal, int k_diff, void* workspace,
                         size_t workspace_bytes, int* status_word, int flags, const void* fwd_workspace,
                         size_t fwd_workspace_bytes, tritt_stream_t stream) {
  const void* ptrs[] = {q, k1, k2, v1, v2, o, d_o, m, dq, dk1, dk2, dv1, dv2};
  int rc = check_common(ptrs, 13, B, N, T, D, dtype);
  if (rc) return rc;
  if ((rc = check_heads(B, N))) return rc;
  if ((rc = check_windows(causal, k_diff, 0, 0, 0))) return rc;
  if ((rc = check_ws(dps_workspace(TRITT_OP_DPS_BWD, B, N, T, D, dtype), workspace, workspace_bytes))) return rc;
  if (fwd_workspace) {
    if ((uintptr_t)fwd_workspace & 255) {
      set_error("the forward workspace must be 256-byte aligned");
      return -7;
    }
    if (fwd_workspace_bytes < dps_workspace(TRITT_OP_DPS_FWD, B, N, T, D, dtype)) {
      set_error("the forward workspace is smaller than tritt_workspace_bytes(TRITT_OP_DPS_FWD, ...)");
      return -6;
    }
  }
  DpsArgs a{};
  a.q = q; a.k1 = k1; a.k2 = k2; a.v1 = v1; a.v2 = v2; a.o = o; a.d_o = d_o; a.m_in = m;
  a.dq = dq; a.dk1 = dk1; a.dk2 = dk2; a.dv1 = dv1; a.dv2 = dv2;
  a.B = B; a.N = N; a.T = T; a.D = D; a.dtype = dtype; a.alpha = alpha;
  a.causal = causal ? 1 : 0; a.k_diff = norm_kdiff(k_diff, T);
  a.workspace = workspace; a.workspace_bytes = workspace_bytes; a.fwd_state = fwd_workspace;
  a.status_word = status_word; a.flags = flags; a.stream = (cudaStream_t)stream;
  return dps_bwd(a);
}

int tritt_dps_bwd(const void* q, const void* k1, const void* k2, const void* v1, const void* v2, const void* o,
                  const void* d_o, const float* m, void* dq, void* dk1, void* dk2, void* dv1, void* dv2, int B,
                  int N, int T, int D, int dtype, float alpha, int causal, int k_diff, void* workspace,
                  size_t workspace_bytes, int* status_word, int flags, tritt_stream_t stream) {
  return dps_bwd_entry(q, k1, k2, v1, v2, o, d_o, m, dq, dk1, dk2, dv1, dv2, B, N, T, D, dtype, alpha, causal, k_diff,
                       workspace, workspace_bytes, status_word, flags, nullptr, 0, stream);
}

int tritt_dps_bwd_saved(const void* q, const void* k1, const void* k2, const void* v1, const void* v2, const void* o,
                        const void* d_o, const float* m, void* dq, void* dk1, void* dk2, void* dv1, void* dv2, int B,
                        int N, int T, int D, int dtype, float alpha, int causal, int k_diff, void* workspace,
                        size_t workspace_bytes, const void* fwd_workspace, size_t fwd_workspace_bytes,
                        int* status_word, int flags, tritt_stream_t stream) {
  if (!fwd_workspace) {
    set_error("tritt_dps_bwd_saved needs the forward call's workspace");
    return -4;
  }
  return dps_bwd_entry(q, k1, k2, v1, v2, o, d_o, m, dq, dk1, dk2, dv1, dv2, B, N, T, D, dtype, alpha, causal, k_diff,
                       workspace, workspace_bytes, status_word, flags, fwd_workspace, fwd_workspace_bytes, stream);
}

}  // extern "C"
