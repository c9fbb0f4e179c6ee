// Host-side helpers shared by the translation units of the library (not part of the C ABI).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nvfp4_b200.h"

namespace nvfp4 {

// Number of SMs of a device (cached).
int sm_count(int dev);
// Device-visible status word of a device (mapped pinned host memory, allocated on first use).
// A kernel whose bounded wait expires stores a DeviceStatus code there; nullptr if allocation failed.
int* status_word(int dev);
// Budget, in nanoseconds, after which a device-side wait gives up (NVFP4_WAIT_BUDGET_MS, default 2000 ms).
unsigned long long wait_budget_ns();

// cuTensorMapEncodeTiled through the runtime's driver entry point (the library does not link libcuda).
// dims / box in elements (innermost first), strides in bytes for dimensions 1..rank-1.
int encode_tiled(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                 const uint64_t* strides, const uint32_t* box, CUtensorMapSwizzle swizzle);

// Tensor-core streaming GEMV (gemv_tc_sm100.cu); arguments as nvfp4_gemv, already validated.
int launch_gemv_tc(const void* a, const void* x, const void* sfa_sw, const void* sfx_sw, void* c, int M, int K, int L,
                   int x_rows, float alpha, int dev, cudaStream_t stream);

}  // namespace nvfp4
