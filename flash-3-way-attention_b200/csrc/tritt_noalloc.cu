// tritt_tdp_fwd_noalloc: the triple-dot-product forward for callers that cannot hand the library a
// scratch buffer because they are not allowed to allocate device memory at all.
//
// Who that is: a plugin running inside another program's enqueue hook (the host program owns every
// device allocation and forbids cudaMalloc there), a process that gave all device memory to a pool it
// cannot reach from this call site, or a latency-critical section that must not take the allocator's
// implicit device-wide synchronisation.  Such callers still own the inputs and outputs; what they
// lack is the kernel's scratch (the SiLU(V1) copy that tritt_tdp_fwd keeps in `workspace`).
//
// The scratch therefore lives in a fixed array in this library's device image.  Consequences a user
// must know:
//   * every GPU whose context has loaded this library's device image holds kNoAllocScratchBytes (8 MiB)
//     from then until the process exits.  With CUDA's default lazy module loading the driver may load
//     the image only at the first call that needs it, and that load reserves device memory inside the
//     driver: "allocates nothing" means that this entry point calls no allocation routine of the CUDA
//     runtime or of any library, not that the driver never touches device memory on its behalf;
//   * problems whose scratch does not fit are rejected with an error: 16-bit inputs on the
//     tensor-core path (head dimension 64 or 128) with B*N*T*D > 4 194 304 elements.  Calls that run on
//     the CUDA-core path (fp32 inputs, other head dimensions, TRITT_FLAG_FORCE_SIMT) need no scratch and
//     are not limited;
//   * all calls on one GPU share the one array.  Nothing in it has to start at zero (each call
//     rewrites the part it reads), but two calls that overlap in time on the same GPU - different
//     streams or different host threads - race on it and produce garbage.  Serialise them;
//   * the first call on each device looks up the array's device address; make that first call
//     before starting any stream capture on that device.  The address is cached per device ordinal
//     and does not survive cudaDeviceReset or the destruction of the device's primary context: a
//     process that does either must not call this entry point afterwards.
#include "tritt_common.cuh"

#include <mutex>

namespace {

constexpr size_t kNoAllocScratchBytes = 8u << 20;
constexpr int kMaxDevices = 64;

// Host code must never pass this name to a kernel: here it is only a handle for
// cudaGetSymbolAddress.  The device address is resolved once per device below.
static __device__ __align__(256) unsigned char g_tdp_fwd_scratch[kNoAllocScratchBytes];

std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch array on the current device (resolved on first use).
int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    tritt::set_error("cudaGetDevice failed: %s", cudaGetErrorString(e));
    return (int)e;
  }
  if (dev < 0 || dev >= kMaxDevices) {
    tritt::set_error("device ordinal %d is outside the supported range", dev);
    return -40;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_tdp_fwd_scratch);
    if (e != cudaSuccess || !p) {
      tritt::set_error("cudaGetSymbolAddress(scratch) failed on device %d: %s", dev, cudaGetErrorString(e));
      return e != cudaSuccess ? (int)e : -41;
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

extern "C" size_t tritt_noalloc_scratch_bytes(void) { return kNoAllocScratchBytes; }

extern "C" int tritt_tdp_fwd_noalloc(const void* q, const void* k1, const void* k2, const void* v1, const void* v2,
                                     void* o, float* lse, int B, int N, int T, int D, int dtype, float alpha,
                                     int causal, int k1_window, int k2_window, int kk_left, int kk_right,
                                     int* status_word, int flags, tritt_stream_t stream) {
  // The bytes the kernel family this call will run on cannot do without (the same choice tritt_tdp_fwd makes; the
  // optional tail that tritt_workspace_bytes adds is used when the scratch has room for it).
  const size_t need =
      tritt_tdp_fwd_min_workspace(B, N, T, D, dtype, causal, k1_window, k2_window, kk_left, kk_right, flags);
  if (need > kNoAllocScratchBytes) {
    tritt::set_error(
        "tritt_tdp_fwd_noalloc: this problem needs %zu bytes of scratch, above the built-in maximum of %zu bytes "
        "(16-bit inputs on the tensor-core path are limited to B*N*T*D <= %zu elements, fp32 inputs there to a "
        "seventh of that); use tritt_tdp_fwd with a caller-provided workspace",
        need, kNoAllocScratchBytes, kNoAllocScratchBytes / 2);
    return -42;
  }
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  // Same kernels, same argument checks as the allocating-caller entry point; only the scratch differs.
  return tritt_tdp_fwd(q, k1, k2, v1, v2, o, lse, B, N, T, D, dtype, alpha, causal, k1_window, k2_window, kk_left,
                       kk_right, /*q_mod=*/1, /*q_rem=*/0, scratch, kNoAllocScratchBytes, status_word, flags, stream);
}
