// Tensor maps for tiled TMA copies (cp.async.bulk.tensor), built on the host.
// The driver's encoder is looked up through the runtime, so that nothing links against the driver.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "mma.cuh"

namespace zb {

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiled tensor_map_encoder() {
  static EncodeTiled encoder = [] {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult found;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &found) != cudaSuccess ||
        found != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      return static_cast<EncodeTiled>(nullptr);
    }
    return reinterpret_cast<EncodeTiled>(entry);
  }();
  return encoder;
}

// One tiled copy of a two-dimensional box at (x, y) into shared memory; x * element size must be a
// multiple of 16 bytes.  Completion is counted in bytes on `bar`.
__device__ __forceinline__ void tiled_copy_2d_g2s(void* smem_dst, const CUtensorMap* map, int x, int y,
                                                  unsigned long long* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
               ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

}  // namespace zb
