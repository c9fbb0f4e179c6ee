// fp32 -> NVFP4 quantiser: the step in front of the GEMM path (the reference has none: its generators draw bit
// patterns directly, eval/nvfp4_gemm/reference.py:35-38).  One launch turns a row-major fp32 operand
// [L][rows][K] into the kernels' input format: packed e2m1 [L][rows][K/2] and e4m3 block scales written
// straight into the swizzled 128x4-tile layout (eval/common/scale_helpers.py:41-68), rows padded to 128.
//
// Per 16-element block, bit for bit what formats.quantize_nvfp4 does with torch ops:
//   scale = RNE_e4m3(min(amax * fl(1/6), 448));  q = RNE_e2m1(x * fl(1/scale)) (saturating at 6, zero if
//   scale == 0); a negative value that rounds to zero keeps its sign bit.
// HBM-bound: 4 bytes read and 0.5625 bytes written per element.
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "nvfp4_internal.h"

namespace nvfp4 {

// Two floats -> one byte of two e2m1 codes (first value in the low nibble), round to nearest even, saturating.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
    uint16_t r;
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

// A warp takes 32 consecutive blocks (512 floats = 2 KB) of the flattened [L*rows][K] operand per step: load i of a
// lane is float4 number i*32 + lane of that span, so every load instruction is one contiguous 512-byte access.
// Four neighbouring lanes hold the four quarters of one block: the block maximum comes from two shuffles, each lane
// quantises its 4 values to 2 bytes and stores them (64 contiguous bytes per warp and store instruction); the lane
// holding the first quarter also writes the scale byte.
__global__ void __launch_bounds__(256)
quantize_f32_kernel(const float* __restrict__ x, uint8_t* __restrict__ packed, uint8_t* __restrict__ sf_sw, int rows,
                    int K, int L, long long total_blocks) {
    const int kbs = K / 16;
    const int R = (rows + 127) / 128, Kb4 = (kbs + 3) / 4;
    const int lane = threadIdx.x & 31;
    const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    const long long spans = (total_blocks + 31) / 32;
    const bool rows_of_8 = (kbs & 7) == 0;   // then the 8 blocks of one load step lie in one row
    for (long long sp = warp0; sp < spans; sp += nwarps) {
        const float4* src = reinterpret_cast<const float4*>(x) + sp * 128;
        float4 v[4];
        bool live[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const long long blk = sp * 32 + i * 8 + (lane >> 2);
            live[i] = blk < total_blocks;
            v[i] = live[i] ? __ldg(src + i * 32 + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        // row and k-block of the span's first block: one warp-uniform division per span
        const unsigned b0 = (unsigned)(sp * 32);
        unsigned lr_s = b0 / (unsigned)kbs, kb_s = b0 - lr_s * (unsigned)kbs;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float amax = fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w)));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            const float want = fminf(__fmul_rn(amax, (float)(1.0 / 6.0)), 448.0f);
            const __nv_fp8_storage_t sbits = __nv_cvt_float_to_fp8(want, __NV_SATFINITE, __NV_E4M3);
            const __half_raw hr = __nv_cvt_fp8_to_halfraw(sbits, __NV_E4M3);
            const float s = __half2float(*reinterpret_cast<const __half*>(&hr));
            uint32_t w = 0;
            if (s > 0.f) {
                const float rs = __frcp_rn(s);
                w = cvt_e2m1x2(__fmul_rn(v[i].x, rs), __fmul_rn(v[i].y, rs)) |
                    (cvt_e2m1x2(__fmul_rn(v[i].z, rs), __fmul_rn(v[i].w, rs)) << 8);
            }
            // position of this lane's block
            unsigned lr, kb;
            if (rows_of_8) {
                lr = lr_s; kb = kb_s + (unsigned)(lane >> 2);         // kb_s is a multiple of 8, so no wrap inside
                kb_s += 8;
                if (kb_s >= (unsigned)kbs) { kb_s -= (unsigned)kbs; lr_s++; }
            } else {
                const unsigned blk = b0 + (unsigned)(i * 8 + (lane >> 2));
                lr = blk / (unsigned)kbs; kb = blk - lr * (unsigned)kbs;
            }
            if (live[i]) {
                // packed bytes of the whole operand: 8 per block, this lane holds quarter lane % 4
                *reinterpret_cast<uint16_t*>(packed + ((size_t)b0 + i * 8 + (lane >> 2)) * 8 + (lane & 3) * 2) = (uint16_t)w;
                if ((lane & 3) == 0) {
                    const unsigned l = lr / (unsigned)rows, r = lr - l * (unsigned)rows;
                    const size_t off = ((size_t)l * R + r / 128) * (size_t)Kb4 * 512 + (size_t)(kb / 4) * 512 +
                                       (r % 32) * 16 + ((r % 128) / 32) * 4 + (kb % 4);
                    sf_sw[off] = (uint8_t)sbits;
                }
            }
        }
    }
}

}  // namespace nvfp4

using namespace nvfp4;

extern "C" int nvfp4_quantize_f32(const void* x, void* packed, void* sf_sw, int rows, int K, int L, void* stream) {
    if (!x || !packed || !sf_sw) return NVFP4_ERR_NULL;
    if (rows <= 0 || K <= 0 || L <= 0) return NVFP4_ERR_SHAPE;
    if (K % 16 != 0) return NVFP4_ERR_K_MULTIPLE;
    if (((uintptr_t)x & 15) || ((uintptr_t)packed & 7)) return NVFP4_ERR_ALIGN;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    cudaStream_t st = (cudaStream_t)stream;
    // padding rows / k-blocks of the scale buffer must read as zero
    const size_t sf_bytes = (size_t)L * ((rows + 127) / 128) * ((K / 16 + 3) / 4) * 512;
    if (rows % 128 != 0 || (K / 16) % 4 != 0) {
        e = cudaMemsetAsync(sf_sw, 0, sf_bytes, st);
        if (e != cudaSuccess) return (int)e;
    }
    const long long total = (long long)L * rows * (K / 16);
    if (total >= (1ll << 31)) return NVFP4_ERR_UNSUPPORTED;   // block indices are 32-bit inside the kernel
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)sm_count(dev) * 16;
    if (blocks > cap) blocks = cap;
    quantize_f32_kernel<<<(unsigned)blocks, 256, 0, st>>>((const float*)x, (uint8_t*)packed, (uint8_t*)sf_sw, rows, K, L,
                                                          total);
    e = cudaGetLastError();
    return e == cudaSuccess ? NVFP4_OK : (int)e;
}
