// Host-side helpers shared by the C-ABI entry points: error codes, the TMA descriptor
// encoder (driver entry point resolved at run time, so the library links without
// libcuda), the per-device status word and cached device properties.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/triton_b200.h"

namespace tb200 {

// Device address of the status word of the current device (nullptr on failure).
int* status_ptr();
// Number of SMs of the current device (cached per device), 0 on failure.
int sm_count();

// Encodes a tiled tensor map of rank 2..5. dims/box are innermost-first; strides_bytes has
// rank-1 entries (stride of dims 1..rank-1). Returns TB200_OK or TB200_ERR_TMAP.
int encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle,
                CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_256B);

inline int cuda_err(cudaError_t e) { return e == cudaSuccess ? TB200_OK : TB200_ERR_CUDA; }

}  // namespace tb200
