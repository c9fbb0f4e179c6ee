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

// Encoding a tensor map costs about a microsecond of host time, which matters for calls whose kernel runs for ten,
// so the maps a thread has made are kept, two-way set-associative on a hash of everything that goes into them.  256
// sets: a caller that rotates through dozens of problems (the harness times 50 inputs in turn) still finds its maps.
struct TmapKey {
    uint64_t base;
    int32_t a, b, c, d;   // the dimensions and box sizes the map depends on
};
template <int SETS = 256>
struct TmapCache {
    struct Entry { TmapKey k; CUtensorMap m; bool valid; };
    Entry e[SETS][2];          // two ways per set; `old[s]` is the way to replace next
    unsigned char old[SETS];
    static unsigned slot(const TmapKey& k) {
        uint64_t h = (k.base >> 4) * 0x9E3779B97F4A7C15ull;
        h ^= ((uint64_t)(uint32_t)k.a << 32 | (uint32_t)k.b) * 0xC2B2AE3D27D4EB4Full;
        h ^= ((uint64_t)(uint32_t)k.c << 32 | (uint32_t)k.d) * 0x165667B19E3779F9ull;
        return (unsigned)(h >> 40) % SETS;
    }
    static bool same(const TmapKey& x, const TmapKey& y) {
        return x.base == y.base && x.a == y.a && x.b == y.b && x.c == y.c && x.d == y.d;
    }
    bool find(const TmapKey& k, CUtensorMap* out) {
        const unsigned s = slot(k);
        for (int w = 0; w < 2; w++) {
            const Entry& en = e[s][w];
            if (en.valid && same(en.k, k)) {
                *out = en.m;
                old[s] = (unsigned char)(1 - w);
                return true;
            }
        }
        return false;
    }
    void put(const TmapKey& k, const CUtensorMap& m) {
        const unsigned s = slot(k);
        Entry& en = e[s][old[s] & 1];
        en.k = k; en.m = m; en.valid = true;
        old[s] = (unsigned char)(1 - (old[s] & 1));
    }
};

// Tensor-core streaming GEMV (gemv_tc_sm100.cu); arguments as nvfp4_gemv, already validated.
int launch_gemv_tc(const void* a, const void* x, const void* sfa_sw, const void* sfx_sw, void* c, int M, int K, int L,
                   int x_rows, float alpha, int dev, cudaStream_t stream);

}  // namespace nvfp4
