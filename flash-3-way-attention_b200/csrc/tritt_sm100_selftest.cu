// Self-test of the sm_100a PTX layer: one CTA runs the two matrix products every
// attention step is made of and writes both results out, so that a host-side test can
// check operand layouts (TMA 128-byte swizzle, K-major and MN-major shared-memory
// descriptors, bf16 operand in tensor memory, TMEM load/store lane mapping) against a
// plain matmul.
//   C  [128,128] = A [128,128] * Bm[128,128]^T          (both operands in shared memory)
//   C2 [128,128] = round_16bit(C) [128,128] * V [128,128]  (left operand in tensor memory,
//                                                        right operand stored row-major)
#include "tritt_common.cuh"
#include "tritt_sm100.cuh"

namespace tritt {

namespace {
using namespace sm100;

template <bool BF16>
__global__ void __launch_bounds__(128, 1)
umma_selftest_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmV, float* C, float* C2, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;               // 2 x [128 rows][64] 16-bit, 16 KiB each
  uint8_t* sB = smem + 32768;
  uint8_t* sV = smem + 65536;
  __shared__ uint64_t bar_load, bar_mma1, bar_mma2;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&bar_load, 1);
    mbar_init(&bar_mma1, 1);
    mbar_init(&bar_mma2, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = tmem_base_s;
  const uint32_t tC = tbase, tP = tbase + 128, tC2 = tbase + 256;

  if (tid == 0) {
    mbar_arrive_expect_tx(&bar_load, 3 * 32768);
    for (int half = 0; half < 2; ++half) {
      tma_load_3d(sA + half * 16384, &tmA, &bar_load, half * 64, 0, 0);
      tma_load_3d(sB + half * 16384, &tmB, &bar_load, half * 64, 0, 0);
      tma_load_3d(sV + half * 16384, &tmV, &bar_load, half * 64, 0, 0);
    }
  }
  bool ok = mbar_wait(&bar_load, 0, &abort_flag);
  if (ok && tid == 0) {
    tc_fence_after();
    constexpr uint32_t idesc = make_idesc_f16(128, 128, BF16 ? 1 : 0, false, false);
    for (int k = 0; k < 8; ++k) {
      const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
      mma_ss(tC, make_smem_desc(smem_u32(sA) + off, 16, 1024), make_smem_desc(smem_u32(sB) + off, 16, 1024), idesc,
             k > 0);
    }
    mma_commit(&bar_mma1);
  }
  ok = ok && mbar_wait(&bar_mma1, 0, &abort_flag);
  if (ok) {
    tc_fence_after();
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const int row = tid;
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(tC + lane_base + c * 32, r);
      tmem_wait_ld();
      uint32_t pk[16];
      for (int i = 0; i < 32; ++i) C[row * 128 + c * 32 + i] = __uint_as_float(r[i]);
      for (int i = 0; i < 16; ++i) {
        const float lo = __uint_as_float(r[2 * i]), hi = __uint_as_float(r[2 * i + 1]);
        if (BF16) {
          __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
          pk[i] = *(uint32_t*)&v;
        } else {
          __half2 v = __floats2half2_rn(lo, hi);
          pk[i] = *(uint32_t*)&v;
        }
      }
      tmem_st16(tP + lane_base + c * 16, pk);
    }
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  if (ok && tid == 0) {
    tc_fence_after();
    constexpr uint32_t idesc = make_idesc_f16(128, 128, BF16 ? 1 : 0, false, true);
    for (int k = 0; k < 8; ++k)
      mma_ts(tC2, tP + k * 8, make_smem_desc(smem_u32(sV) + k * 2048, 16384, 1024), idesc, k > 0);
    mma_commit(&bar_mma2);
  }
  ok = ok && mbar_wait(&bar_mma2, 0, &abort_flag);
  if (ok) {
    tc_fence_after();
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(tC2 + lane_base + c * 32, r);
      tmem_wait_ld();
      for (int i = 0; i < 32; ++i) C2[tid * 128 + c * 32 + i] = __uint_as_float(r[i]);
    }
  }
  if (!ok && tid == 0 && status) atomicOr(status, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 512);
}

// Exercises the time-out path every tensor-core kernel shares: one thread is meant to arrive on an mbarrier, a
// warp waits for it with the bounded wait.  With `skip_arrival` the arrival never happens, the wait gives up after
// `limit_ticks` clock ticks, the CTA records status bit 128, releases its tensor memory and returns normally.
__global__ void __launch_bounds__(64, 1) wait_expiry_kernel(int skip_arrival, long long limit_ticks, int* status) {
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 32);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  bool ok = true;
  if (warp == 0) {
    if (tid == 0 && !skip_arrival) mbar_arrive(&bar);
  } else {
    ok = __all_sync(0xffffffffu, mbar_wait_limit(&bar, 0, &abort_flag, limit_ticks));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base_s, 32);
  if (tid == 32 && !ok && status) atomicOr(status, 128);
}

}  // namespace
}  // namespace tritt

extern "C" int tritt_selftest_wait_expiry(int skip_arrival, long long limit_ticks, int* status_word,
                                          tritt_stream_t stream) {
  using namespace tritt;
  if (limit_ticks < 1 || limit_ticks > sm100::kWaitTicks) {
    set_error("limit_ticks must lie in [1, %lld]", sm100::kWaitTicks);
    return -1;
  }
  wait_expiry_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(skip_arrival, limit_ticks, status_word);
  count_launch();
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int tritt_selftest_umma(const void* A, const void* Bm, const void* V, float* C, float* C2, int dtype,
                                   int* status_word, tritt_stream_t stream) {
  using namespace tritt;
  if (dtype != TRITT_BF16 && dtype != TRITT_F16) {
    set_error("selftest runs on 16-bit inputs only");
    return -1;
  }
  CUtensorMap tmA, tmB, tmV;
  int rc;
  if ((rc = make_tmap_3d(&tmA, A, 2, 128, 128, 1, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmB, Bm, 2, 128, 128, 1, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tmV, V, 2, 128, 128, 1, 64, 128))) return rc;
  const int smem = 3 * 32768 + 1024;
  if (dtype == TRITT_BF16) {
    TRITT_CUDA_OK(cudaFuncSetAttribute(umma_selftest_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    umma_selftest_kernel<true><<<1, 128, smem, (cudaStream_t)stream>>>(tmA, tmB, tmV, C, C2, status_word);
    count_launch();
  } else {
    TRITT_CUDA_OK(cudaFuncSetAttribute(umma_selftest_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    umma_selftest_kernel<false><<<1, 128, smem, (cudaStream_t)stream>>>(tmA, tmB, tmV, C, C2, status_word);
    count_launch();
  }
  TRITT_CUDA_OK(cudaGetLastError());
  return 0;
}
