// Host-side construction of the TMA tensor maps the tensor-core kernels take as launch parameters
// (cuTensorMapEncodeTiled, looked up through the runtime so that the library has no link-time dependency on
// libcuda): 3-D tiled maps over [B*N, rows, cols] tensors, 128-byte swizzle for 16-bit operand tiles, and fp32
// maps for the destinations of TMA reduce-adds.
#include "tritt_common.cuh"
#include "tritt_sm100.cuh"

namespace tritt {

namespace {
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !p) return nullptr;
    fn = (EncodeFn)p;
  }
  return fn;
}
int encode_3d(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, CUtensorMapSwizzle swz, const void* base,
              uint64_t cols, uint64_t rows, uint64_t bn, uint32_t box_cols, uint32_t box_rows) {
  EncodeFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return -20;
  }
  cuuint64_t dims[3] = {cols, rows, bn};
  cuuint64_t strides[2] = {cols * elem_bytes, rows * cols * elem_bytes};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (cols=%llu rows=%llu bn=%llu)", (int)r,
              (unsigned long long)cols, (unsigned long long)rows, (unsigned long long)bn);
    return -22;
  }
  return 0;
}
}  // namespace

int make_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t cols, uint64_t rows, uint64_t bn,
                 uint32_t box_cols, uint32_t box_rows) {
  if (elem_bytes != 2) {
    set_error("make_tmap_3d is for 16-bit elements");
    return -21;
  }
  return encode_3d(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, CU_TENSOR_MAP_SWIZZLE_128B, base, cols, rows, bn, box_cols,
                   box_rows);
}

int make_tmap_3d_f32(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t bn,
                     uint32_t box_cols, uint32_t box_rows) {
  // box rows are box_cols * 4 bytes wide: 64 bytes -> 64-byte swizzle, 128 bytes -> 128-byte swizzle
  const CUtensorMapSwizzle swz = box_cols * 4 == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                 : box_cols * 4 == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                      : CU_TENSOR_MAP_SWIZZLE_NONE;
  return encode_3d(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, swz, base, cols, rows, bn, box_cols, box_rows);
}

}  // namespace tritt
