// Host-side helpers shared by the kernels' launchers: status codes, the device status word,
// and tensor-map construction through the driver entry point (no link-time libcuda dependency).
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/mx8.h"

namespace mx8 {

// One word per device, written by a kernel whose bounded wait gave up; read by mx8_device_status.
int* device_status_ptr();        // device address of the word on the current device (nullptr on failure)

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();  // nullptr if the driver entry point is unavailable

// dims/strides innermost first; strides in bytes for dims 1..rank-1
int make_tmap(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz,
              CUtensorMapL2promotion l2 = CU_TENSOR_MAP_L2_PROMOTION_L2_256B);

int sm_count();                   // multiprocessors of the current device (cached)
int check_device_sm100();         // MX8_OK or MX8_ERR_UNSUPPORTED

void note_cuda_error(const char* what, const char* detail);  // remembered per thread for mx8_last_cuda_error

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace mx8
