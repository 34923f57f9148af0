// Host-side construction of TMA tensor maps (CUtensorMap) without linking libcuda: the driver
// entry point is fetched through the runtime at first use.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// Up to 5 dimensions, innermost first.  strides_bytes[i] is the byte stride of dimension i+1
// (dimension 0 is dense).  Returns 0 or a negative B200_E* code (message stored).
int make_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle,
              CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_256B);

}  // namespace b200
