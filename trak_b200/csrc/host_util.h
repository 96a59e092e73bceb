// Host-side helpers shared by the C-ABI translation units: error bookkeeping,
// device checks and TMA tensor-map encoding through the driver entry point
// (the library does not link against libcuda).
#pragma once
#include <cstdint>
#include <cstdio>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/trak_b200.h"

namespace tb {

void set_cuda_error(const char* what, const char* file, int line);

#define TB_CUDA(call)                                                        \
    do {                                                                     \
        cudaError_t e__ = (call);                                            \
        if (e__ != cudaSuccess) {                                            \
            ::tb::set_cuda_error(cudaGetErrorString(e__), __FILE__, __LINE__); \
            return TB_ERR_CUDA;                                              \
        }                                                                    \
    } while (0)

// TB_OK if `device` exists and is compute capability 10.x; sets it current.
int select_device(int device, int* sm_count);

// TB_OK, or the code tb_project returns for these arguments before it looks at workspace or device.
int validate_project_args(const void* grads, int dtype, int64_t B, int64_t F, int64_t ld, const float* out,
                          int64_t ld_out, uint32_t N, uint32_t num_feature_tiles, int proj_type);

// Device address of the status word of `device` (valid after select_device).
uint32_t* status_ptr(int device);

// Encodes a tiled tensor map (rank 2 or 3, zero fill; the box's inner extent must equal the
// swizzle width).
// dims / box are innermost first; strides_bytes has rank-1 entries.
int encode_tmap(CUtensorMap* map, CUtensorMapDataType dt, uint32_t rank, const void* base,
                const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B);

// Events armed by tb_profile_events for this thread (null when not armed); taking clears them.
void take_profile_events(cudaEvent_t* before, cudaEvent_t* after);

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace tb
