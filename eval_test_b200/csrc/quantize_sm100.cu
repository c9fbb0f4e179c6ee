// fp32 -> NVFP4 quantiser: the step in front of the GEMM path (the reference has none: its generators draw bit
// patterns directly, eval/nvfp4_gemm/reference.py:35-38).  One launch turns a row-major fp32 operand
// [L][rows][K] into the kernels' input format: packed e2m1 [L][rows][K/2] and e4m3 block scales written
// straight into the swizzled 128x4-tile layout (eval/common/scale_helpers.py:41-68), rows padded to 128.
//
// Per 16-element block, bit for bit what formats.quantize_nvfp4 does with torch ops:
//   scale = RNE_e4m3(min(amax * fl(1/6), 448));  q = RNE_e2m1(x / scale) (saturating at 6, zero if scale == 0);
//   a zero result carries no sign.
// HBM-bound: 4 bytes read and 0.5625 bytes written per element.  A thread owns one block (64 bytes in, 8 bytes
// + 1 scale byte out); the four 16-byte loads of a thread cover whole sectors between them.
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
    uint32_t b = r;
    // -0 -> +0 (a code whose magnitude bits are zero carries no sign)
    if ((b & 0x07u) == 0u) b &= ~0x08u;
    if ((b & 0x70u) == 0u) b &= ~0x80u;
    return b;
}

__global__ void __launch_bounds__(256)
quantize_f32_kernel(const float* __restrict__ x, uint8_t* __restrict__ packed, uint8_t* __restrict__ sf_sw, int rows,
                    int K, int L, long long total_blocks) {
    const int kbs = K / 16;
    const int R = (rows + 127) / 128, Kb4 = (kbs + 3) / 4;
    for (long long blk = (long long)blockIdx.x * blockDim.x + threadIdx.x; blk < total_blocks;
         blk += (long long)gridDim.x * blockDim.x) {
        const int kb = (int)(blk % kbs);
        const long long lr = blk / kbs;          // l * rows + r
        const int r = (int)(lr % rows), l = (int)(lr / rows);
        const float4* src = reinterpret_cast<const float4*>(x + (size_t)lr * K + (size_t)kb * 16);
        float v[16];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float4 t = __ldg(src + i);
            v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(v[i]));
        const float want = fminf(__fmul_rn(amax, (float)(1.0 / 6.0)), 448.0f);
        const __nv_fp8_storage_t sbits = __nv_cvt_float_to_fp8(want, __NV_SATFINITE, __NV_E4M3);
        const __half_raw hr = __nv_cvt_fp8_to_halfraw(sbits, __NV_E4M3);
        const float s = __half2float(*reinterpret_cast<const __half*>(&hr));
        uint32_t w0 = 0, w1 = 0;
        if (s > 0.f) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                w0 |= cvt_e2m1x2(__fdiv_rn(v[2 * i], s), __fdiv_rn(v[2 * i + 1], s)) << (8 * i);
                w1 |= cvt_e2m1x2(__fdiv_rn(v[8 + 2 * i], s), __fdiv_rn(v[8 + 2 * i + 1], s)) << (8 * i);
            }
        }
        *reinterpret_cast<uint2*>(packed + (size_t)lr * (K / 2) + (size_t)kb * 8) = make_uint2(w0, w1);
        const size_t off = ((size_t)l * R + r / 128) * (size_t)Kb4 * 512 + (size_t)(kb / 4) * 512 + (r % 32) * 16 +
                           ((r % 128) / 32) * 4 + (kb % 4);
        sf_sw[off] = (uint8_t)sbits;
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
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)sm_count(dev) * 16;
    if (blocks > cap) blocks = cap;
    quantize_f32_kernel<<<(unsigned)blocks, 256, 0, st>>>((const float*)x, (uint8_t*)packed, (uint8_t*)sf_sw, rows, K, L,
                                                          total);
    e = cudaGetLastError();
    return e == cudaSuccess ? NVFP4_OK : (int)e;
}
