/*
 * tritt.h - C ABI of libtritt_sm100.so: three-way ("trittention") attention for
 * NVIDIA B200 (sm_100a).
 *
 * The library replaces the device side of the reference package flash_trittention
 * (Triton kernels launched from Python); each entry point below names the reference
 * launch site it stands in for.  Host glue (argument validation, torch.autograd
 * plumbing) lives above this ABI and mirrors the reference's Python modules.
 *
 * Conventions
 *   - every tensor is row-major [B, N, T, D], innermost stride 1, base pointer 16-byte
 *     aligned, all of one dtype (TRITT_F32 / TRITT_F16 / TRITT_BF16); lse / m vectors
 *     are fp32 [B, N, T] holding the natural-log log-sum-exp of the scaled logits;
 *   - pointers are DEVICE pointers; the caller owns every buffer including `workspace`
 *     and keeps them alive until the work enqueued on `stream` has run;
 *   - calls only enqueue work on `stream` (no synchronisation, no device allocation);
 *   - return value 0 = success, negative = invalid argument, positive = cudaError_t of
 *     a failed runtime call.  tritt_last_error() gives a thread-local message;
 *   - `status_word` (an int the GPU can address: device memory or page-locked host memory; may be NULL)
 *     is OR-ed with a non-zero code by a kernel whose bounded barrier wait ran out (1 tensor-core
 *     self-test, 2 / 4 triple-dot-product forward / backward, 8 misaligned shared memory, 16 / 32
 *     soft-max attention forward / backward of the dot-product-sum path, 128 wait-expiry self-test) or,
 *     bit 64, by the fp16 operand conversion of an fp32 / wide-operand call that met an element beyond 65504;
 *     the caller zeroes and reads it.  A non-zero word means the results of that call are invalid;
 *   - window arguments (k1_window, k2_window, kk_left, kk_right, k_diff) are distances >= 0; a value
 *     >= T means "unlimited".  Negative values are refused with an argument error when `causal` is set
 *     (the reference applies them literally, which leaves query rows with nothing to attend to);
 *   - B*N may not exceed 65535.
 */
#ifndef TRITT_H_
#define TRITT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* tritt_stream_t; /* a cudaStream_t / CUstream */

enum { TRITT_F32 = 0, TRITT_F16 = 1, TRITT_BF16 = 2 };

/* operations, for tritt_workspace_bytes() */
enum { TRITT_OP_TDP_FWD = 0, TRITT_OP_TDP_BWD = 1, TRITT_OP_DPS_FWD = 2, TRITT_OP_DPS_BWD = 3 };

/* flags */
enum {
  TRITT_FLAG_FORCE_SIMT = 1,  /* use the plain fp32 CUDA-core kernels even where the tensor-core path applies */
  TRITT_FLAG_BWD_PARTIAL = 2, /* tritt_tdp_bwd: leave the fp32 key-side partial sums in the workspace and do not
                                 write dk1/dk2/dv1/dv2 (the caller reduces them across ranks, then calls
                                 tritt_tdp_bwd_finalize) */
  TRITT_FLAG_WIDE_OPERANDS = 4, /* triple-dot-product, bf16 inputs: form the operands with 11 significant bits (fp16
                                 copies) instead of bf16's 8, what the reference's `convert_to_float32` asks of its TF32
                                 dot products.  fp32 inputs always take that path on the tensor cores (head dimension
                                 64 / 128); fp16 inputs already have it.  Needs the larger workspace that
                                 tritt_workspace_bytes_flags() reports; an input element beyond fp16's range (65504)
                                 sets status bit 64. */
  TRITT_FLAG_BWD_CTA_PAIRS = 8  /* tritt_tdp_bwd, 16-bit inputs, head dimension 128, no windows, an even number of
                                 queries: run the backward kernel as clusters of two CTAs that share every key / value
                                 tile (tcgen05 cta_group::2, 256-row products).  Same results up to the order of the
                                 fp32 reduce-adds; measured 2 % slower than one CTA per item on a B200, so it is not
                                 the default.  Ignored where it does not apply. */
};

/* kernel families, as reported by tritt_tdp_path() */
enum { TRITT_PATH_SIMT = 0, TRITT_PATH_TCGEN05 = 1 };

int tritt_version(void);
/* Number of kernels this library has enqueued in the calling process so far (bookkeeping for benchmarks). */
unsigned long long tritt_kernel_launches(void);
const char* tritt_last_error(void);

/* Bytes of caller-provided scratch to pass to the given operation (0 if none).  For TRITT_OP_TDP_FWD on 16-bit inputs
   the figure includes a small tail (three floats per (batch, head), behind the SiLU(V1) copy of B*N*T*D elements) that
   lets the forward bound its scores and skip the row-maximum pass; a workspace without the tail is accepted and runs
   the two-pass soft-max. */
size_t tritt_workspace_bytes(int op, int B, int N, int T, int D, int dtype);
/* The same for a call that will pass `flags` (TRITT_FLAG_WIDE_OPERANDS enlarges the triple-dot-product workspace of bf16
   inputs by the fp16 operand copies; tritt_workspace_bytes() equals flags = 0). */
size_t tritt_workspace_bytes_flags(int op, int B, int N, int T, int D, int dtype, int flags);

/* Bytes of scratch tritt_tdp_fwd cannot run without for these arguments (the optional score-bound tail excluded). */
size_t tritt_tdp_fwd_min_workspace(int B, int N, int T, int D, int dtype, int causal, int k1_window, int k2_window,
                                   int kk_left, int kk_right, int flags);

/* Which kernel family a TDP call with these arguments runs on. */
int tritt_tdp_path(int op, int T, int D, int dtype, int causal, int k1_window, int k2_window, int kk_left,
                   int kk_right, int flags);
/* Which kernel family the two soft-max attentions of a DPS forward, and their row-owner / column-owner backward
   kernels, run on. */
int tritt_dps_path(int T, int D, int dtype, int k_diff, int flags);

/*
 * Triple-dot-product forward.  Replaces the launch of `_tritt_fwd` and the host-side
 * SiLU / `M + log(L)` passes around it in the reference
 * (src/flash_trittention/triple_dot_product/flash_trittention.py:61-62,92-128).
 *   S[q,j,k] = alpha * sum_h q[q,h] k1[j,h] k2[k,h];  softmax over the attended (j,k);
 *   o[q,h]   = sum_jk P[q,j,k] SiLU(v1[j,h]) v2[k,h];  lse[q] = log sum_jk exp(S).
 * (q_mod, q_rem): only query rows q with q % q_mod == q_rem are computed and written
 * (query-row sharding across devices); pass (1, 0) for all rows.
 */
int tritt_tdp_fwd(const void* q, const void* k1, const void* k2, const void* v1, const void* v2, void* o,
                  float* lse, int B, int N, int T, int D, int dtype, float alpha, int causal, int k1_window,
                  int k2_window, int kk_left, int kk_right, int q_mod, int q_rem, void* workspace,
                  size_t workspace_bytes, int* status_word, int flags, tritt_stream_t stream);

/*
 * Triple-dot-product backward.  Replaces the five launches `_tritt_bwd_dq/_dk1/_dk2/_dv1/_dv2`
 * and the host-side SiLU, D = sum(dO*O), zero-init and SiLU' passes of the reference
 * (src/flash_trittention/triple_dot_product/flash_trittention.py:158-173,191-391).
 * v1 is the RAW (pre-SiLU) tensor; dv1 is the gradient w.r.t. it.  With (q_mod, q_rem) != (1, 0)
 * only the selected rows of dq are written and the key-side gradients are partial sums.
 */
int tritt_tdp_bwd(const void* q, const void* k1, const void* k2, const void* v1, const void* v2, const void* o,
                  const void* d_o, const float* lse, void* dq, void* dk1, void* dk2, void* dv1, void* dv2, int B,
                  int N, int T, int D, int dtype, float alpha, int causal, int k1_window, int k2_window,
                  int kk_left, int kk_right, int q_mod, int q_rem, void* workspace, size_t workspace_bytes,
                  int* status_word, int flags, tritt_stream_t stream);

/*
 * Second half of a TRITT_FLAG_BWD_PARTIAL backward: converts the fp32 partial sums
 * (workspace layout: dK1 | dK2 | dSiLU(V1) | dV2, each [B,N,T,D] fp32, starting at
 * tritt_tdp_bwd_partials_offset() bytes) to the output dtype and applies SiLU'(v1) to dv1
 * (reference flash_trittention.py:390-391).  No counterpart launch in the reference: the
 * reference has no multi-device path.
 */
int tritt_tdp_bwd_finalize(const void* v1, void* dk1, void* dk2, void* dv1, void* dv2, int B, int N, int T, int D,
                           int dtype, void* workspace, size_t workspace_bytes, tritt_stream_t stream);
size_t tritt_tdp_bwd_partials_offset(int B, int N, int T, int D, int dtype);

/*
 * Dot-product-sum forward.  Replaces the launch of the reference's `_tritt_fwd`
 * (src/flash_trittention/dot_product_sum/trittention_triton.py:90-120).
 *   S[q,s,t] = alpha * (q[q].k2[t] + k1[s].k2[t]);  causal: s <= t <= q and t - s <= k_diff;
 *   o[q,h]   = sum_st P[q,s,t] SiLU(v1[s,h]) v2[t,h];  m[q] = log sum_st exp(S).
 */
int tritt_dps_fwd(const void* q, const void* k1, const void* k2, const void* v1, const void* v2, void* o, float* m,
                  int B, int N, int T, int D, int dtype, float alpha, int causal, int k_diff, void* workspace,
                  size_t workspace_bytes, int* status_word, int flags, tritt_stream_t stream);

/*
 * Dot-product-sum backward.  Replaces `_tritt_bwd_preprocess`, `_tritt_bwd_dq`, `_tritt_bwd_dk_dv`
 * and the host-side SiLU / SiLU' / dk2 merge passes of the reference
 * (src/flash_trittention/dot_product_sum/trittention_triton.py:160,183-356).
 */
int tritt_dps_bwd(const void* q, const void* k1, const void* k2, const void* v1, const void* v2, const void* o,
                  const void* d_o, const float* m, void* dq, void* dk1, void* dk2, void* dv1, void* dv2, int B,
                  int N, int T, int D, int dtype, float alpha, int causal, int k_diff, void* workspace,
                  size_t workspace_bytes, int* status_word, int flags, tritt_stream_t stream);

/*
 * The same backward for a caller that kept the forward call's workspace untouched (same inputs, same arguments):
 * the inner attention's results the forward left there (Y, its log-sum-exp, SiLU(V1), Y*V2) are read instead of being
 * computed again, which removes two launches.  `workspace` is still this call's own scratch of
 * tritt_workspace_bytes(TRITT_OP_DPS_BWD, ...) bytes.  The reference keeps no such state between its forward and
 * backward (it recomputes per query block, dot_product_sum/kernels/bwd_dq_kernel.py:28-350).
 */
int tritt_dps_bwd_saved(const void* q, const void* k1, const void* k2, const void* v1, const void* v2, const void* o,
                        const void* d_o, const float* m, void* dq, void* dk1, void* dk2, void* dv1, void* dv2, int B,
                        int N, int T, int D, int dtype, float alpha, int causal, int k_diff, void* workspace,
                        size_t workspace_bytes, const void* fwd_workspace, size_t fwd_workspace_bytes,
                        int* status_word, int flags, tritt_stream_t stream);

/*
 * Triple-dot-product forward for callers that may not allocate device memory (a plugin inside
 * another program's enqueue hook, a process whose device memory all belongs to a pool this call
 * site cannot use, a section that must avoid the allocator's device-wide synchronisation).
 * Same computation and checks as tritt_tdp_fwd for all query rows, but the scratch is an 8 MiB array
 * built into the library image (tritt_noalloc_scratch_bytes()), held by every GPU whose context has
 * loaded that image until the process exits (with CUDA's lazy module loading the driver may load it,
 * and reserve its memory, only at the first call).  Limits: 16-bit inputs on the tensor-core path
 * (head dimension 64 or 128) with B*N*T*D > 4 194 304 elements are rejected (the CUDA-core path - fp32
 * inputs, other head dimensions, TRITT_FLAG_FORCE_SIMT - needs no scratch); calls that overlap in time
 * on one GPU share the array and race; the first call on a device resolves the array's address and
 * should precede any stream capture on that device; the cached address does not survive
 * cudaDeviceReset.  It calls no allocation routine of the CUDA runtime or of any library.  This entry
 * point has no counterpart in the reference.
 */
int tritt_tdp_fwd_noalloc(const void* q, const void* k1, const void* k2, const void* v1, const void* v2, void* o,
                          float* lse, int B, int N, int T, int D, int dtype, float alpha, int causal,
                          int k1_window, int k2_window, int kk_left, int kk_right, int* status_word, int flags,
                          tritt_stream_t stream);
size_t tritt_noalloc_scratch_bytes(void);

/*
 * Self-test of the tensor-core building blocks (TMA tile loads, shared-memory operand
 * descriptors, a 16-bit operand held in tensor memory): one CTA computes
 *   C = A * Bm^T   and   C2 = round16(C) * V      (all matrices 128 x 128, row-major)
 * so that a host test can compare against a plain matmul.  No counterpart in the
 * reference (its kernels are Triton; the compiler picks the matrix instructions).
 */
int tritt_selftest_umma(const void* A, const void* Bm, const void* V, float* C, float* C2, int dtype,
                        int* status_word, tritt_stream_t stream);

/*
 * Self-test of the bounded barrier wait that every tensor-core kernel uses: a one-CTA kernel in which one
 * thread is to arrive on an mbarrier and a warp waits for it, giving up after `limit_ticks` clock ticks
 * (1 .. 2e9).  With skip_arrival != 0 the arrival is left out on purpose: the wait runs out, the kernel ORs
 * 128 into `status_word`, frees its tensor memory and returns; nothing faults and the context stays usable.
 * No counterpart in the reference (Triton kernels have no hand-written waits).
 */
int tritt_selftest_wait_expiry(int skip_arrival, long long limit_ticks, int* status_word, tritt_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TRITT_H_ */
