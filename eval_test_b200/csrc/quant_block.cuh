// One 16-element block of fp32 values -> its e4m3 scale byte and 16 e2m1 codes (8 bytes), the rule of the
// quantiser in front of the path (and of formats.quantize_nvfp4 in the Python package, bit for bit):
//   scale = RNE_e4m3(min(amax * fl(1/6), 448));  q = RNE_e2m1(x * fl(1/scale)) (saturating at 6, zero if
//   scale == 0); a negative value that rounds to zero keeps its sign bit.
#pragma once
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace nvfp4 {

// Two floats -> one byte of two e2m1 codes (first value in the low nibble), round to nearest even, saturating.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
    uint16_t r;
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

// x[0..15] -> packed codes (w0: elements 0..7, w1: 8..15; element 2i in the low nibble of byte i); returns the scale byte.
__device__ __forceinline__ uint32_t quantize_block16(const float* x, uint32_t& w0, uint32_t& w1) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(x[i]));
    const float want = fminf(__fmul_rn(amax, (float)(1.0 / 6.0)), 448.0f);
    const __nv_fp8_storage_t sbits = __nv_cvt_float_to_fp8(want, __NV_SATFINITE, __NV_E4M3);
    const __half_raw hr = __nv_cvt_fp8_to_halfraw(sbits, __NV_E4M3);
    const float s = __half2float(*reinterpret_cast<const __half*>(&hr));
    w0 = 0; w1 = 0;
    if (s > 0.f) {
        const float rs = __frcp_rn(s);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            w0 |= cvt_e2m1x2(__fmul_rn(x[2 * i], rs), __fmul_rn(x[2 * i + 1], rs)) << (8 * i);
            w1 |= cvt_e2m1x2(__fmul_rn(x[8 + 2 * i], rs), __fmul_rn(x[8 + 2 * i + 1], rs)) << (8 * i);
        }
    }
    return (uint32_t)sbits;
}

}  // namespace nvfp4
