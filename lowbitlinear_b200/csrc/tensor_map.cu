#include "tensor_map.h"

namespace lbl {
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_entry() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &query) !=
            cudaSuccess ||
        query != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

}  // namespace

bool encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                       const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                       CUtensorMapSwizzle swizzle) {
  EncodeTiledFn encode = encode_tiled_entry();
  if (encode == nullptr || rank < 1 || rank > 3) return false;
  cuuint64_t g_dims[3];
  cuuint64_t g_strides[2];
  cuuint32_t g_box[3];
  cuuint32_t elem_strides[3] = {1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    g_dims[i] = dims[i];
    g_box[i] = box[i];
  }
  for (int i = 0; i + 1 < rank; ++i) g_strides[i] = strides_bytes[i];
  const CUresult rc =
      encode(map, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), g_dims, g_strides,
             g_box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS;
}

}  // namespace lbl
