// Entry points whose kernels are not built yet: they refuse loudly instead of computing anything.
#include "nvfp4_internal.h"

extern "C" int nvfp4_grouped_gemm(const nvfp4_group_t*, int, float, void*) { return NVFP4_ERR_UNSUPPORTED; }
