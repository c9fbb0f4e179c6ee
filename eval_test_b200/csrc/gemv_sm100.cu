// NVFP4 block-scaled GEMV for sm_100a: an HBM-streaming kernel, no tensor cores.
//
//   c[m, 0, l] = fp16( alpha * sum_kb sfa[m,kb,l] * sfx[kb,l] * sum_{j<16} a[m,16kb+j,l] * x[16kb+j,l] )
//
// Replaces the reference's GEMV entry, which runs a 128-column padded tensor-core GEMM through
// torch._scaled_mm and keeps column 0 (eval/nvfp4_gemv/submission.py:28-54).
//
// Work unit = 32 rows of one 128-row block of one batch: rows {128*rb + 32*g + 8*j + i : g<4, i<8}.
// That row set is chosen because its scale factors form one contiguous 128-byte slice of every
// 512-byte atom of the swizzled scale layout, so scales stream with full sector use.
// A persistent CTA walks its units; a producer feeds a shared-memory ring, consumer warps decode and
// accumulate.  The ring is filled by two tiled TMA loads per stage when M is a multiple of 128 - a
// 5-D view of A (k, row-in-8, j, g, row-block) brings the unit's 32 row segments in one instruction,
// a 4-D view of the scales brings its 128-byte slices of consecutive atoms (128-byte swizzle, which
// also spreads the consumers' reads over the banks); measured on B200, per-row 1-D bulk copies cost
// about 32 ns each per SM whatever their size and cap the kernel far below HBM speed, so they are
// kept only for ragged M.  Consumers:
//   * e2m1 -> int8 (2*value) with one byte-permute per 4 elements: the permute's selector nibble
//     is the e2m1 nibble itself, its 3 low bits index an 8-entry table held in two registers, and
//     its top bit (the sign) makes the permute return 0, so "positives" and (after flipping the
//     sign bits) "negatives" come out as two unsigned byte vectors;
//     the two tables are biased so that the permute's by-products cancel: positives look up v+1 (v = 2*|a|,
//     0 stays 0) and negatives -v; a positive element makes the negative lookup return -1 (replicated MSB of
//     a negative table byte), a negative element makes the positive lookup return 0, so the two byte vectors
//     always add up to the signed value and both can be fed to dp4a against the same vector;
//   * 4-way int8 dot products (exact) against the vector, which sits in shared memory as int8;
//   * one fp32 FMA per 16-element block with sfa*sfx; lanes split K, rows are reduced by shuffles.
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "nvfp4_internal.h"
#include "ptx_sm100.cuh"

namespace nvfp4 {

struct GemvParams {
    const uint8_t* a;     // [L][M][K/2]
    const uint8_t* x;     // [L][x_rows][K/2], row 0 is the vector
    const uint8_t* sfa;   // swizzled, rows padded to 128
    const uint8_t* sfx;   // swizzled, x_rows rows
    __half* c;            // [L][M]
    int M, K, L, x_rows;
    float alpha;
    int* status;
    unsigned long long budget_ns;
};

constexpr int SF_SLOT = 144;  // ragged-M path: 128-byte scale slice + 16 bytes of padding (spreads banks)

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

constexpr uint32_t LUT_LO = 0x03020100u;  // 2*|e2m1| for codes 0..3
constexpr uint32_t LUT_HI = 0x0C080604u;  // 2*|e2m1| for codes 4..7
constexpr uint32_t POS_LO = 0x04030200u;  // v + 1 (0 for v = 0): looked up by non-negative elements
constexpr uint32_t POS_HI = 0x0D090705u;
constexpr uint32_t NEG_LO = 0xFDFEFF00u;  // -v: looked up by negative elements (sign bit flipped first)
constexpr uint32_t NEG_HI = 0xF4F8FAFCu;

// Exact dot product of 8 e2m1 elements (one 32-bit word of A) with 8 int8 values (x0, x1 = 2*x).
__device__ __forceinline__ int dot8(uint32_t w, uint32_t x0, uint32_t x1, int d) {
    const uint32_t wn = w ^ 0x88888888u;
    d = __dp4a((int)prmt(POS_LO, POS_HI, w), (int)x0, d);
    d = __dp4a((int)prmt(POS_LO, POS_HI, w >> 16), (int)x1, d);
    d = __dp4a((int)prmt(NEG_LO, NEG_HI, wn), (int)x0, d);
    d = __dp4a((int)prmt(NEG_LO, NEG_HI, wn >> 16), (int)x1, d);
    return d;
}

__device__ __forceinline__ float2 e4m3x2_to_float2(uint16_t v) {
    __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)v, __NV_E4M3);
    return __half22float2(*reinterpret_cast<__half2*>(&h));
}

template <int KC, bool TILED>
struct GemvStage {
    static constexpr int A_BYTES = 32 * (KC / 2);
    static constexpr int SF_BYTES = (KC / 64) * (TILED ? 128 : SF_SLOT);
    static constexpr int BYTES = (A_BYTES + SF_BYTES + 1023) / 1024 * 1024;  // scales first, then A
    static constexpr int A_OFF = (SF_BYTES + 127) / 128 * 128;
};

// TILED: tiled TMA loads (needs M % 128 == 0); otherwise per-row bulk copies.
// MODE 1 skips the arithmetic (measures the copy pipeline alone; tuning aid).
template <int CW, int KC, int STAGES, int MINB, int MODE, bool TILED>
__global__ void __launch_bounds__((CW + 1) * 32, MINB)
gemv_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_sf,
            const GemvParams p) {
    using St = GemvStage<KC, TILED>;
    constexpr int RPW = 32 / CW;                 // rows per consumer warp
    constexpr int STAGE = St::BYTES;
    static_assert(32 % CW == 0 && KC % 1024 == 0, "bad tile");

    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 2];

    const int K = p.K, M = p.M;
    const int kbs = K / 16;
    uint8_t* xs = smem;                                   // K int8: 2*x
    float* sxs = reinterpret_cast<float*>(smem + K);      // K/16 floats: 0.25 * sfx
    // ring: 1024-byte aligned (the swizzled scale slices need it)
    uint8_t* ring = smem + (((smem_u32(smem) + K + kbs * 4 + 1023u) & ~1023u) - smem_u32(smem));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, CW);
        }
        mbar_init(smem_u32(&bars[2 * STAGES]), CW);      // consumers done with the old vector
        mbar_init(smem_u32(&bars[2 * STAGES + 1]), CW);  // new vector written
        fence_mbar_init();
    }
    __syncthreads();

    const int RB = (M + 127) / 128;
    const int Kb4 = (kbs + 3) / 4;
    const int units_per_l = RB * 4;
    const int total_units = p.L * units_per_l;
    const int nchunks = (K + KC - 1) / KC;

    if (warp == CW) {
        // ---------------------------------------------------------------- producer warp
        uint32_t it = 0;
        const int g = lane >> 3, i = lane & 7;
        bool alive = true;
        for (int u = blockIdx.x; alive && u < total_units; u += gridDim.x) {
            const int l = u / units_per_l, rem = u % units_per_l;
            const int rb = rem >> 2, j = rem & 3;
            const int row = rb * 128 + g * 32 + j * 8 + i;
            int nvalid = 0;  // rows of this unit that exist
#pragma unroll
            for (int gg = 0; gg < 4; gg++) {
                int lo = rb * 128 + gg * 32 + j * 8;
                nvalid += max(0, min(8, M - lo));
            }
            const uint8_t* arow = p.a + ((size_t)l * M + row) * (size_t)(K / 2);
            const uint8_t* sfsrc = p.sfa + ((size_t)l * RB + rb) * (size_t)Kb4 * 512 + j * 128;
            for (int c = 0; c < nchunks; c++, it++) {
                const int slot = it % STAGES;
                const uint32_t par = ((it / STAGES) & 1) ^ 1;
                if (!mbar_wait(empty0 + 8 * slot, par, p.budget_ns)) {
                    if (lane == 0) report_status(p.status, DEV_TIMEOUT_PRODUCER);
                    alive = false;
                    break;
                }
                const int k0 = c * KC;
                const uint32_t full = full0 + 8 * slot;
                const uint32_t sbase = smem_u32(ring + (size_t)slot * STAGE);
                if (TILED) {
                    // out-of-range k (last chunk) is zero-filled and still counted, so the byte count is fixed
                    if (lane == 0) {
                        mbar_arrive_expect_tx(full, (uint32_t)(St::A_BYTES + St::SF_BYTES));
                        tma_load_4d(sbase, &tmap_sf, 0, j, k0 / 64, l * RB + rb, full);
                        tma_load_5d(sbase + St::A_OFF, &tmap_a, k0 / 16, 0, j, 0, l * RB + rb, full);
                    }
                } else {
                    const int kc = min(KC, K - k0);
                    const int nq = (kc + 63) / 64;
                    if (lane == 0) mbar_arrive_expect_tx(full, (uint32_t)(nvalid * (kc / 2) + nq * 128));
                    __syncwarp();
                    if (row < M) bulk_g2s(sbase + St::A_OFF + lane * (KC / 2), arow + k0 / 2, (uint32_t)(kc / 2), full);
                    for (int q = lane; q < nq; q += 32)
                        bulk_g2s(sbase + q * SF_SLOT, sfsrc + (size_t)(k0 / 64 + q) * 512, 128u, full);
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- consumer warps
        uint32_t it = 0;
        int cur_l = -1;
        bool alive = true;
        uint32_t xpar = 0;
        const uint32_t xbar0 = smem_u32(&bars[2 * STAGES]), xbar1 = xbar0 + 8;
        for (int u = blockIdx.x; alive && u < total_units; u += gridDim.x) {
            const int l = u / units_per_l, rem = u % units_per_l;
            const int rb = rem >> 2, j = rem & 3;
            if (l != cur_l) {
                // (re)load the vector of batch l: int8 2*x and 0.25*sfx, shared by every row
                __syncwarp();
                if (lane == 0) mbar_arrive(xbar0);
                if (!mbar_wait(xbar0, xpar, p.budget_ns)) {
                    if (lane == 0) report_status(p.status, DEV_TIMEOUT_CONSUMER);
                    break;
                }
                const uint8_t* xg = p.x + (size_t)l * p.x_rows * (size_t)(K / 2);
                const int xR = (p.x_rows + 127) / 128;
                const uint8_t* sg = p.sfx + (size_t)l * xR * (size_t)Kb4 * 512;
                for (int w4 = threadIdx.x; w4 < K / 8; w4 += CW * 32) {
                    const uint32_t w = reinterpret_cast<const uint32_t*>(xg)[w4];
                    const uint32_t wn = w ^ 0x88888888u;
                    const uint32_t p0 = prmt(LUT_LO, LUT_HI, w), p1 = prmt(LUT_LO, LUT_HI, w >> 16);
                    const uint32_t q0 = prmt(LUT_LO, LUT_HI, wn), q1 = prmt(LUT_LO, LUT_HI, wn >> 16);
                    reinterpret_cast<uint2*>(xs)[w4] = make_uint2(__vsub4(p0, q0), __vsub4(p1, q1));
                }
                for (int kb = threadIdx.x; kb < kbs; kb += CW * 32) {
                    const uint8_t b = sg[(size_t)(kb >> 2) * 512 + (kb & 3)];
                    __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
                    sxs[kb] = 0.25f * __half2float(*reinterpret_cast<__half*>(&h));
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(xbar1);
                if (!mbar_wait(xbar1, xpar, p.budget_ns)) {
                    if (lane == 0) report_status(p.status, DEV_TIMEOUT_CONSUMER);
                    break;
                }
                xpar ^= 1;
                cur_l = l;
            }
            float acc[RPW];
#pragma unroll
            for (int rr = 0; rr < RPW; rr++) acc[rr] = 0.f;
            // per-row offsets inside a stage, for segment `lane` of a 1024-element sub-chunk:
            // A: row ur, 16 bytes per segment; scales: slice q = lane/2 (+16 per sub-chunk), 16-byte chunk i
            // (XOR q%8 in the swizzled tiled layout; 16*sub keeps q%8), word g, byte pair lane%2
            int aoff[RPW], soff[RPW];
#pragma unroll
            for (int rr = 0; rr < RPW; rr++) {
                const int ur = warp * RPW + rr, q = lane >> 1;
                aoff[rr] = St::A_OFF + ur * (KC / 2) + lane * 16;
                soff[rr] = (TILED ? q * 128 + ((((ur & 7) ^ (q & 7)) << 4) | ((ur >> 3) << 2))
                                  : q * SF_SLOT + (((ur & 7) << 4) | ((ur >> 3) << 2))) + (lane & 1) * 2;
            }

            for (int c = 0; c < nchunks; c++, it++) {
                const int slot = it % STAGES;
                const uint32_t par = (it / STAGES) & 1;
                if (!mbar_wait(full0 + 8 * slot, par, p.budget_ns)) {
                    if (lane == 0) report_status(p.status, DEV_TIMEOUT_CONSUMER);
                    alive = false;
                    break;
                }
                const int k0 = c * KC;
                const int kc = min(KC, K - k0);
                const uint8_t* Ss = ring + (size_t)slot * STAGE;
#pragma unroll
                for (int sub = 0; sub < KC / 1024; sub++) {
                    const int kseg = sub * 1024 + lane * 32;  // this lane's 32-element segment of the chunk
                    if (MODE == 0 && kseg < kc) {
                        const int kg = k0 + kseg;
                        const uint4 xa = *reinterpret_cast<const uint4*>(xs + kg);
                        const uint4 xb = *reinterpret_cast<const uint4*>(xs + kg + 16);
                        const float2 sx = *reinterpret_cast<const float2*>(sxs + (kg >> 4));
#pragma unroll
                        for (int rr = 0; rr < RPW; rr++) {
                            const uint4 av = *reinterpret_cast<const uint4*>(Ss + aoff[rr] + sub * 512);
                            const uint16_t sfw = *reinterpret_cast<const uint16_t*>(
                                Ss + soff[rr] + sub * 16 * (TILED ? 128 : SF_SLOT));
                            const float2 sa = e4m3x2_to_float2(sfw);
                            int d0 = dot8(av.x, xa.x, xa.y, 0);
                            d0 = dot8(av.y, xa.z, xa.w, d0);
                            int d1 = dot8(av.z, xb.x, xb.y, 0);
                            d1 = dot8(av.w, xb.z, xb.w, d1);
                            acc[rr] = fmaf((float)d0, sa.x * sx.x, acc[rr]);
                            acc[rr] = fmaf((float)d1, sa.y * sx.y, acc[rr]);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * slot);
            }
            if (!alive) break;
#pragma unroll
            for (int rr = 0; rr < RPW; rr++) {
                float v = acc[rr];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                const int ur = warp * RPW + rr;
                const int row = rb * 128 + (ur >> 3) * 32 + j * 8 + (ur & 7);
                if (lane == 0 && row < M) p.c[(size_t)l * M + row] = __float2half_rn(p.alpha * v);
            }
        }
    }
    __syncthreads();
}

template <int CW, int KC, int STAGES, int MINB = 1, int MODE = 0>
static int launch_gemv(const GemvParams& p, cudaStream_t stream) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 64) return NVFP4_ERR_UNSUPPORTED;
    const bool tiled = (p.M % 128 == 0);
    const int stage = tiled ? GemvStage<KC, true>::BYTES : GemvStage<KC, false>::BYTES;
    const size_t smem = (size_t)p.K + (size_t)(p.K / 16) * 4 + 1024 + (size_t)STAGES * stage;
    if (smem > 227 * 1024 - 256) return NVFP4_ERR_UNSUPPORTED;
    const int RB = (p.M + 127) / 128;
    const int Kb4 = (p.K / 16 + 3) / 4;
    const int units = p.L * RB * 4;
    const int slots = sm_count(dev) * MINB;
    const int grid = units < slots ? units : slots;
    CUtensorMap ta, tsf;
    memset(&ta, 0, sizeof(ta));
    memset(&tsf, 0, sizeof(tsf));
    if (tiled) {
        // A as 8-byte elements: (k, row within 8, j, g, batch*row-block); one box = the unit's 32 rows x KC/2 bytes
        const uint64_t rowb = (uint64_t)(p.K / 2);
        const uint64_t ad[5] = {(uint64_t)(p.K / 16), 8, 4, 4, (uint64_t)p.L * RB};
        const uint64_t as[4] = {rowb, 8 * rowb, 32 * rowb, 128 * rowb};
        const uint32_t ab[5] = {(uint32_t)(KC / 16), 8, 1, 4, 1};
        int rc = encode_tiled(&ta, CU_TENSOR_MAP_DATA_TYPE_INT64, 5, p.a, ad, as, ab, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
        // scales as bytes: (byte within a 128-byte slice, j, 64-element group, batch*row-block)
        const uint64_t sd[4] = {128, 4, (uint64_t)Kb4, (uint64_t)p.L * RB};
        const uint64_t ss[3] = {128, 512, (uint64_t)Kb4 * 512};
        const uint32_t sb[4] = {128, 1, (uint32_t)(KC / 64), 1};
        rc = encode_tiled(&tsf, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, p.sfa, sd, ss, sb, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }
    static size_t configured[64][2] = {};
    if (tiled) {
        auto kern = gemv_kernel<CW, KC, STAGES, MINB, MODE, true>;
        if (configured[dev][1] < smem) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            configured[dev][1] = smem;
        }
        kern<<<grid, (CW + 1) * 32, smem, stream>>>(ta, tsf, p);
    } else {
        auto kern = gemv_kernel<CW, KC, STAGES, MINB, MODE, false>;
        if (configured[dev][0] < smem) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            configured[dev][0] = smem;
        }
        kern<<<grid, (CW + 1) * 32, smem, stream>>>(ta, tsf, p);
    }
    e = cudaGetLastError();
    return e == cudaSuccess ? NVFP4_OK : (int)e;
}

}  // namespace nvfp4

using namespace nvfp4;

extern "C" int nvfp4_gemv(const void* a, const void* x, const void* sfa_sw, const void* sfx_sw, void* c, int M, int K,
                          int L, int x_rows, float alpha, void* stream) {
    if (!a || !x || !sfa_sw || !sfx_sw || !c) return NVFP4_ERR_NULL;
    if (M <= 0 || K <= 0 || L <= 0 || x_rows <= 0) return NVFP4_ERR_SHAPE;
    if (K % 64 != 0) return NVFP4_ERR_K_MULTIPLE;
    if (((uintptr_t)a | (uintptr_t)x | (uintptr_t)sfa_sw | (uintptr_t)sfx_sw) & 15) return NVFP4_ERR_ALIGN;
    if ((uintptr_t)c & 1) return NVFP4_ERR_ALIGN;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    // Two kernels.  The tensor-core stream (gemv_tc_sm100.cu) works in tiles of 128 rows and wins once there are
    // enough of them; the kernel of this file (decode on the CUDA cores) works in units of 32 rows, spreads a small
    // problem over four times as many SMs and starts faster (measured on B200: 16 tiles, 8 us against 12 us;
    // 56 tiles, 27 us against 25 us; 512 tiles, 112 us against 96 us).  NVFP4_GEMV_PATH=alu / =tensor forces one
    // (read on every call, so that one process can compare the two).
    const char* path = getenv("NVFP4_GEMV_PATH");
    const long tiles = (long)L * ((M + 127) / 128);
    const bool tensor = path && path[0] == 't' ? true : path && path[0] == 'a' ? false : tiles > 32;
    if (tensor || K > 65536)
        return launch_gemv_tc(a, x, sfa_sw, sfx_sw, c, M, K, L, x_rows, alpha, dev, (cudaStream_t)stream);
    GemvParams p;
    p.a = (const uint8_t*)a; p.x = (const uint8_t*)x; p.sfa = (const uint8_t*)sfa_sw; p.sfx = (const uint8_t*)sfx_sw;
    p.c = (__half*)c; p.M = M; p.K = K; p.L = L; p.x_rows = x_rows; p.alpha = alpha;
    p.status = status_word(dev);
    p.budget_ns = wait_budget_ns();
    cudaStream_t s = (cudaStream_t)stream;
    static const int variant = [] { const char* e = getenv("NVFP4_GEMV_VARIANT"); return e ? atoi(e) : 0; }();
    if (K > 32768) return launch_gemv<8, 1024, 3>(p, s);
    if (K > 16384) return launch_gemv<8, 2048, 4>(p, s);
    switch (variant) {  // tuning knob; 0 is the shipped configuration
        case 1: return launch_gemv<8, 1024, 4, 2>(p, s);
        case 2: return launch_gemv<8, 2048, 5, 1>(p, s);
        case 3: return launch_gemv<16, 2048, 5, 1>(p, s);
        case 6: return launch_gemv<8, 2048, 2, 2, 1>(p, s);   // no arithmetic: the copy pipeline alone
        default: return launch_gemv<8, 2048, 2, 2>(p, s);
    }

}
