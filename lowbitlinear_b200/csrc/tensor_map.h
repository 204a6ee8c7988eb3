// Host-side creation of TMA tensor maps and the device-side tiled loads that consume them.
// The driver entry point is looked up through the runtime, so the library does not link libcuda.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lbl {

// Encodes a tiled tensor map of rank 1..3 (no interleave, zero fill outside the tensor,
// L2 promotion to 256 bytes).  `dims`/`box` have `rank` entries, `strides_bytes` has rank - 1.
// Returns false when the driver rejects the description or the entry point is missing.
bool encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                       const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                       CUtensorMapSwizzle swizzle);

#ifdef __CUDACC__
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
      "l"(map), "r"(c0), "r"(c1), "r"(static_cast<uint32_t>(__cvta_generic_to_shared(bar)))
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(static_cast<uint32_t>(__cvta_generic_to_shared(bar)))
      : "memory");
}

// Three-dimensional tiled load with an L2 eviction policy (see l2_evict_first_policy): weights are read once
// per call, so they should be the first lines the L2 gives up, not the activations and results
// that the neighbouring kernels are about to touch.
__device__ __forceinline__ void tma_load_3d_hint(void* smem_dst, const CUtensorMap* map, int c0,
                                                 int c1, int c2, uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(static_cast<uint32_t>(__cvta_generic_to_shared(bar))),
      "l"(policy)
      : "memory");
}

__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
#endif

}  // namespace lbl
