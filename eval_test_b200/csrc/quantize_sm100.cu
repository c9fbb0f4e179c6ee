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
#include "quant_block.cuh"

namespace nvfp4 {

// A warp takes 32 consecutive blocks (512 floats = 2 KB) of the flattened [L*rows][K] operand per step and every
// lane one whole block: four 16-byte loads (the four instructions of a warp together read the 2 KB once; L1 serves
// the second half of each sector), block maximum, scale, 16 products, 8 conversions - all in the lane, no shuffles -
// then one 8-byte store of the packed block (256 contiguous bytes per warp).  Four neighbouring lanes hold the four
// k-blocks of one row that share a 4-byte group of a swizzle atom: their scale bytes are gathered into one 32-bit
// store when K % 64 == 0.  The loads of the warp's next span are issued before the current one is processed.
// KIND: 0 fp32, 1 fp16, 2 bf16 input (16-bit inputs: two 16-byte loads per lane; values are widened to fp32, which is
// exact, and quantised by the same rule).
template <int KIND>
__global__ void __launch_bounds__(256)
quantize_kernel(const void* __restrict__ x, uint8_t* __restrict__ packed, uint8_t* __restrict__ sf_sw, int rows,
                    int K, int L, long long total_blocks) {
    const unsigned kbs = (unsigned)(K / 16);
    const int R = (rows + 127) / 128, Kb4 = (int)(kbs + 3) / 4;
    const int lane = threadIdx.x & 31;
    const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    const long long spans = (total_blocks + 31) / 32;
    const bool words = (kbs & 3) == 0;       // then lanes 4a..4a+3 hold one aligned word of one atom
    const bool uniform_row = (kbs & 31) == 0;   // then a span lies in one row
    constexpr int NV = KIND == 0 ? 4 : 2;    // 16-byte loads per block
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);

    auto load_span = [&](long long sp, uint4 (&v)[NV]) {
        const long long blk = sp * 32 + lane;
        const uint4* src = reinterpret_cast<const uint4*>(x) + blk * NV;
        const bool live = blk < total_blocks;
#pragma unroll
        for (int i = 0; i < NV; i++) v[i] = live ? __ldg(src + i) : zero4;
    };

    uint4 v[NV], nxt[NV];
    if (warp0 < spans) load_span(warp0, v);
    for (long long sp = warp0; sp < spans; sp += nwarps) {
        const bool more = sp + nwarps < spans;
        if (more) load_span(sp + nwarps, nxt);
        const unsigned blk = (unsigned)(sp * 32) + (unsigned)lane;      // total_blocks < 2^31 (checked by the caller)
        const bool live = (long long)blk < total_blocks;
        float xs[16];
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const uint32_t wv[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (KIND == 0) {
                    xs[4 * i + j] = __uint_as_float(wv[j]);
                } else if (KIND == 1) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&wv[j]));
                    xs[8 * i + 2 * j] = f.x; xs[8 * i + 2 * j + 1] = f.y;
                } else {   // bf16 is the upper half of an fp32
                    xs[8 * i + 2 * j] = __uint_as_float(wv[j] << 16);
                    xs[8 * i + 2 * j + 1] = __uint_as_float(wv[j] & 0xffff0000u);
                }
            }
        }
        uint32_t w0, w1;
        const uint32_t sbits = quantize_block16(xs, w0, w1);
        if (live) *reinterpret_cast<uint2*>(packed + (size_t)blk * 8) = make_uint2(w0, w1);
        // where this block's scale byte goes
        unsigned lr, kb;
        if (uniform_row) {
            const unsigned b0 = (unsigned)(sp * 32);
            lr = b0 / kbs; kb = b0 - lr * kbs + (unsigned)lane;
        } else {
            lr = blk / kbs; kb = blk - lr * kbs;
        }
        const unsigned l = lr / (unsigned)rows, r = lr - l * (unsigned)rows;
        const size_t off = ((size_t)l * R + r / 128) * (size_t)Kb4 * 512 + (size_t)(kb / 4) * 512 + (r % 32) * 16 +
                           ((r % 128) / 32) * 4 + (kb % 4);
        if (words) {
            // (the operand ends on a multiple of 4 blocks here, so the 4 lanes of a group are live together)
            uint32_t word = sbits;
            word |= __shfl_down_sync(0xffffffffu, sbits, 1) << 8;
            word |= __shfl_down_sync(0xffffffffu, sbits, 2) << 16;
            word |= __shfl_down_sync(0xffffffffu, sbits, 3) << 24;
            if (live && (lane & 3) == 0) *reinterpret_cast<uint32_t*>(sf_sw + off) = word;
        } else if (live) {
            sf_sw[off] = (uint8_t)sbits;
        }
        if (more) {
#pragma unroll
            for (int i = 0; i < NV; i++) v[i] = nxt[i];
        }
    }
}

}  // namespace nvfp4

using namespace nvfp4;

template <int KIND>
static int quantize_any(const void* x, void* packed, void* sf_sw, int rows, int K, int L, void* stream) {
    if (!x || !packed || !sf_sw) return NVFP4_ERR_NULL;
    if (rows <= 0 || K <= 0 || L <= 0) return NVFP4_ERR_SHAPE;
    if (K % 16 != 0) return NVFP4_ERR_K_MULTIPLE;
    if (((uintptr_t)x & 15) || ((uintptr_t)packed & 7) || ((uintptr_t)sf_sw & 3)) return NVFP4_ERR_ALIGN;
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
    // a grid-stride loop over spans: as many blocks as are resident at once (no partial last wave)
    static int per_sm[64] = {};
    if (dev < 64 && !per_sm[dev]) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, quantize_kernel<KIND>, 256, 0) != cudaSuccess || n < 1) n = 4;
        per_sm[dev] = n;
    }
    long long blocks = (total + 255) / 256;   // 8 warps x 32 blocks per thread block and step
    const long long cap = (long long)sm_count(dev) * (dev < 64 ? per_sm[dev] : 4);
    if (blocks > cap) blocks = cap;
    quantize_kernel<KIND><<<(unsigned)blocks, 256, 0, st>>>(x, (uint8_t*)packed, (uint8_t*)sf_sw, rows, K, L, total);
    e = cudaGetLastError();
    return e == cudaSuccess ? NVFP4_OK : (int)e;
}

extern "C" int nvfp4_quantize_f32(const void* x, void* packed, void* sf_sw, int rows, int K, int L, void* stream) {
    return quantize_any<0>(x, packed, sf_sw, rows, K, L, stream);
}
extern "C" int nvfp4_quantize_f16(const void* x, void* packed, void* sf_sw, int rows, int K, int L, void* stream) {
    return quantize_any<1>(x, packed, sf_sw, rows, K, L, stream);
}
extern "C" int nvfp4_quantize_bf16(const void* x, void* packed, void* sf_sw, int rows, int K, int L, void* stream) {
    return quantize_any<2>(x, packed, sf_sw, rows, K, L, stream);
}
