// Triple-dot-product trittention for fp32 inputs (and for bf16 inputs when the caller asks for wider operands, the
// reference's `convert_to_float32`) on the tensor cores.
//
// The reference's kernels take fp32 operands into TF32 dot products (its Blackwell forward forms the Q*K2 pre-product
// in fp32 and runs the score product in TF32 on purpose, b200/fwd_b200.py:173-176,253): 11 significant bits per
// operand, fp32 accumulation.  fp16 carries the same 11 significant bits and runs at twice TF32's rate on tcgen05
// with half the shared memory per tile, so this path converts the operands to fp16 copies in the workspace and runs
// the fp16 tensor-core kernels on them; soft-max state, accumulators, the log-sum-exp and the key-side gradient sums
// stay fp32.  What fp16 lacks is TF32's exponent range, which is handled where it matters:
//   * the upstream gradient dO (arbitrarily small in training) is scaled by a power of two taken from its largest
//     magnitude (found on the device, no host synchronisation) and the five gradients, all linear in dO, are
//     scaled back;
//   * an input element beyond fp16's largest finite value (65504) cannot be represented: the conversion records
//     status bit 64 (the results of that call are invalid); magnitudes below 6e-8 flush to zero, an absolute
//     error far below the rounding of the O(1) elements they are summed with.
// TRITT_FLAG_FORCE_SIMT keeps the exact-fp32 CUDA-core kernels for such data.
#include "tritt_common.cuh"

namespace tritt {
namespace {

struct CvtBatch {
  const void* src[8];
  __half* dst[8];
  int scaled;  // index of the tensor that is multiplied by the power-of-two scale, or -1
};

__device__ __forceinline__ float pow2_scale(const unsigned* absmax_bits) {
  // largest magnitude m * 2^e with m in [0.5, 1)  ->  2^-e, so that the scaled tensor peaks in (0.5, 1]
  const float mx = __uint_as_float(*absmax_bits);
  if (!(mx > 0.f) || !isfinite(mx)) return 1.f;
  int e;
  frexpf(mx, &e);
  return ldexpf(1.f, -e);
}

template <typename TI>
__global__ void absmax_kernel(const TI* __restrict__ x, size_t n, unsigned* out_bits) {
  float m = 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(to_f(x[i])));
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax(out_bits, __float_as_uint(m));  // non-negative floats order like their bits
}

template <typename TI>
__global__ void to_half_kernel(CvtBatch b, size_t n, const unsigned* absmax_bits, int* status) {
  const int t = blockIdx.y;
  const TI* src = (const TI*)b.src[t];
  __half* dst = b.dst[t];
  const float sc = (t == b.scaled) ? pow2_scale(absmax_bits) : 1.f;
  bool bad = false;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float v = to_f(src[i]) * sc;
    bad |= !(fabsf(v) <= 65504.f);  // also catches NaN
    dst[i] = __float2half_rn(v);
  }
  if (bad && status) atomicOr(status, 64);
}

template <typename TO>
__global__ void from_half_kernel(const __half* __restrict__ src, TO* __restrict__ dst, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = from_f<TO>(__half2float(src[i]));
}

// dq (fp16, from the kernel) and the fp32 key-side sums dK1 | dK2 | dSiLU(V1) | dV2 -> the five gradients in the
// inputs' type, with the dO scale divided out and SiLU'(V1) applied (reference flash_trittention.py:390-391).
template <typename TO>
__global__ void wide_bwd_finalize_kernel(const __half* __restrict__ dq16, const float* __restrict__ part,
                                         const TO* __restrict__ v1, TO* dq, TO* dk1, TO* dk2, TO* dv1, TO* dv2, size_t n,
                                         const unsigned* absmax_bits) {
  const float inv = 1.f / pow2_scale(absmax_bits);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    dq[i] = from_f<TO>(__half2float(dq16[i]) * inv);
    dk1[i] = from_f<TO>(part[i] * inv);
    dk2[i] = from_f<TO>(part[n + i] * inv);
    dv1[i] = from_f<TO>(part[2 * n + i] * inv * silu_grad_f(to_f(v1[i])));
    dv2[i] = from_f<TO>(part[3 * n + i] * inv);
  }
}

unsigned blocks_for(size_t n) { return (unsigned)((n + 256 * 4 - 1) / (256 * 4) < 2048 ? (n + 256 * 4 - 1) / (256 * 4) : 2048); }

template <typename TI>
int convert_in(const CvtBatch& b, int count, size_t n, const unsigned* absmax_bits, int* status, cudaStream_t s) {
  to_half_kernel<TI><<<dim3(blocks_for(n), count), 256, 0, s>>>(b, n, absmax_bits, status);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}

size_t half_seg(size_t n) { return align_up(n * 2, 256); }

}  // namespace

bool tdp_wide_applies(int op, int T, int D, int dtype, const TdpMask& m, int flags) {
  if (flags & TRITT_FLAG_FORCE_SIMT) return false;
  const bool asked = dtype == TRITT_F32 || (dtype == TRITT_BF16 && (flags & TRITT_FLAG_WIDE_OPERANDS));
  return asked && sm100_tdp_supported(op, T, D, TRITT_F16, m);
}

size_t tdp_wide_workspace(int op, int B, int N, int T, int D) {
  const size_t n = (size_t)B * N * T * D;
  if (op == TRITT_OP_TDP_FWD)
    return 6 * half_seg(n) + align_up(sm100_tdp_workspace(op, B, N, T, D, TRITT_F16) +
                                      sm100_tdp_fwd_optional_workspace(B, N, T, D, TRITT_F16), 256);
  return 8 * half_seg(n) + 256 + align_up(sm100_tdp_workspace(op, B, N, T, D, TRITT_F16), 256);
}

int tdp_wide_fwd(const TdpArgs& a) {
  const size_t n = (size_t)a.B * a.N * a.T * a.D, h = half_seg(n);
  char* ws = (char*)a.workspace;
  CvtBatch b{};
  const void* src[5] = {a.q, a.k1, a.k2, a.v1, a.v2};
  for (int i = 0; i < 5; ++i) {
    b.src[i] = src[i];
    b.dst[i] = (__half*)(ws + i * h);
  }
  b.scaled = -1;
  int rc = a.dtype == TRITT_F32 ? convert_in<float>(b, 5, n, nullptr, a.status_word, a.stream)
                                : convert_in<__nv_bfloat16>(b, 5, n, nullptr, a.status_word, a.stream);
  if (rc) return rc;
  __half* o16 = (__half*)(ws + 5 * h);
  TdpArgs in = a;
  in.q = b.dst[0]; in.k1 = b.dst[1]; in.k2 = b.dst[2]; in.v1 = b.dst[3]; in.v2 = b.dst[4];
  in.out_o = o16;
  in.dtype = TRITT_F16;
  in.workspace = ws + 6 * h;
  in.workspace_bytes = a.workspace_bytes - 6 * h;
  if ((rc = sm100_tdp_fwd(in))) return rc;
  if (a.dtype == TRITT_F32)
    from_half_kernel<float><<<blocks_for(n), 256, 0, a.stream>>>(o16, (float*)a.out_o, n);
  else
    from_half_kernel<__nv_bfloat16><<<blocks_for(n), 256, 0, a.stream>>>(o16, (__nv_bfloat16*)a.out_o, n);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}

int tdp_wide_bwd(const TdpArgs& a) {
  if (a.flags & TRITT_FLAG_BWD_PARTIAL) {
    set_error("query-sharded partial sums are not offered for fp32 / wide-operand calls");
    return -12;
  }
  const size_t n = (size_t)a.B * a.N * a.T * a.D, h = half_seg(n);
  char* ws = (char*)a.workspace;
  unsigned* absmax = (unsigned*)(ws + 8 * h);
  TRITT_CUDA_OK(cudaMemsetAsync(absmax, 0, 4, a.stream));
  if (a.dtype == TRITT_F32)
    absmax_kernel<float><<<blocks_for(n), 256, 0, a.stream>>>((const float*)a.d_o, n, absmax);
  else
    absmax_kernel<__nv_bfloat16><<<blocks_for(n), 256, 0, a.stream>>>((const __nv_bfloat16*)a.d_o, n, absmax);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  CvtBatch b{};
  const void* src[7] = {a.q, a.k1, a.k2, a.v1, a.v2, a.o, a.d_o};
  for (int i = 0; i < 7; ++i) {
    b.src[i] = src[i];
    b.dst[i] = (__half*)(ws + i * h);
  }
  b.scaled = 6;
  int rc = a.dtype == TRITT_F32 ? convert_in<float>(b, 7, n, absmax, a.status_word, a.stream)
                                : convert_in<__nv_bfloat16>(b, 7, n, absmax, a.status_word, a.stream);
  if (rc) return rc;
  __half* dq16 = (__half*)(ws + 7 * h);
  TdpArgs in = a;
  in.q = b.dst[0]; in.k1 = b.dst[1]; in.k2 = b.dst[2]; in.v1 = b.dst[3]; in.v2 = b.dst[4];
  in.o = b.dst[5]; in.d_o = b.dst[6];
  in.dq = dq16;
  in.dk1 = in.dk2 = in.dv1 = in.dv2 = nullptr;
  in.dtype = TRITT_F16;
  in.flags = a.flags | TRITT_FLAG_BWD_PARTIAL;  // leave the fp32 key-side sums in the inner workspace
  in.workspace = ws + 8 * h + 256;
  in.workspace_bytes = a.workspace_bytes - (8 * h + 256);
  if ((rc = sm100_tdp_bwd(in))) return rc;
  const float* part = (const float*)in.workspace;
  if (a.dtype == TRITT_F32)
    wide_bwd_finalize_kernel<float><<<blocks_for(n), 256, 0, a.stream>>>(
        dq16, part, (const float*)a.v1, (float*)a.dq, (float*)a.dk1, (float*)a.dk2, (float*)a.dv1, (float*)a.dv2, n, absmax);
  else
    wide_bwd_finalize_kernel<__nv_bfloat16><<<blocks_for(n), 256, 0, a.stream>>>(
        dq16, part, (const __nv_bfloat16*)a.v1, (__nv_bfloat16*)a.dq, (__nv_bfloat16*)a.dk1, (__nv_bfloat16*)a.dk2,
        (__nv_bfloat16*)a.dv1, (__nv_bfloat16*)a.dv2, n, absmax);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace tritt
