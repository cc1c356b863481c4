// Host-side tensor-map encoding. cuTensorMapEncodeTiled is looked up through the runtime's
// driver-entry-point query, so the library does not link against libcuda.

#include <cudaTypedefs.h>

#include <mutex>

#include "bsr_gemm.cuh"

namespace sb {
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult result = cudaDriverEntryPointSymbolNotFound;
    const cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &result);
    if (err == cudaSuccess && result == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

}  // namespace

int encode_bf16_2d_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                       const char* what) {
  const EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return fail(SB_ERR_CUDA, "%s: the CUDA driver does not export cuTensorMapEncodeTiled", what);
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};  // bytes between rows
  const cuuint32_t box[2] = {64, box_rows};  // 64 bf16 = 128 bytes = one swizzle row
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                             elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    return fail(SB_ERR_TENSOR_MAP, "%s: cuTensorMapEncodeTiled failed with CUresult %d (rows %llu, cols %llu)", what,
                static_cast<int>(rc), (unsigned long long)rows, (unsigned long long)cols);
  return SB_OK;
}

}  // namespace sb
