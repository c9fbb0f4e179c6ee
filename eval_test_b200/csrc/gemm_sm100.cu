// NVFP4 block-scaled GEMM and dual GEMM (SiLU gating) for sm_100a on the 5th-generation tensor cores.
//
//   GEMM : C[l] = fp16( alpha * (A*sfa)[l] @ (B*sfb)[l]^T )
//   DUAL : C[l] = fp16( silu(alpha * A@B1^T) * (alpha * A@B2^T) )
//
// Replaces the reference's CuTe-DSL kernels (eval/nvfp4_gemm/submission.py:45-664 and
// eval/nvfp4_dual_gemm/submission.py:45-844: one CTA per 128x128 tile, one shared-memory stage, a
// single warp doing loads and MMAs in turn).  Here:
//   * persistent CTAs (one per SM) walk output tiles of 128 x BN in an L2-friendly order;
//   * warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..5 = epilogue;
//   * a ring of shared-memory stages, each holding 256 K-elements of A (128 rows), of B (BN rows) and
//     their scale-factor atoms; operand tiles arrive by tiled TMA with the 128-byte swizzle, the
//     scale atoms (contiguous in the swizzled global layout) by 1-D bulk copies - no multicast;
//   * tcgen05.cp moves each 512-byte scale atom into tensor memory, tcgen05.mma
//     kind::mxf4nvf4.block_scale.block16 accumulates 128 x BN x 64 per issue into tensor memory,
//     tcgen05.commit releases the stage / publishes the accumulator through mbarriers;
//   * the epilogue reads the accumulator with tcgen05.ld, applies alpha (and silu(x)*y for the dual
//     GEMM, whose two products share one 256-column accumulator: B1 rows then B2 rows form one B
//     tile), rounds once to fp16 and stores rows with 16-byte stores.
// Every mbarrier wait is bounded; on expiry the role records a status code and leaves its loop, the
// CTA still frees its tensor memory and exits.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <mutex>

#include "nvfp4_internal.h"
#include "ptx_sm100.cuh"

namespace nvfp4 {

constexpr int BM = 128;        // rows of A per tile = TMEM lanes
constexpr int BK = 256;        // K elements per stage = 128 bytes per row = one swizzle atom
constexpr int GEMM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;

struct GemmParams {
    const uint8_t* sfa;   // swizzled scales of A  [L][ceil(M/128)][K/64][512]
    const uint8_t* sfb;   // swizzled scales of B (B1 for the dual GEMM)
    const uint8_t* sfb2;  // swizzled scales of B2 (dual GEMM only)
    __half* c;            // [L][M][N]
    int M, N, K, L;
    float alpha;
    int* status;
    unsigned long long budget_ns;
};

// Tile order: bands of 16 row-tiles; inside a band the row-tile index runs fastest, so the CTAs that
// run together share a few A row-tiles and B column-tiles in L2.
struct TileCoord { int l, mt, nt; };
__device__ __forceinline__ TileCoord tile_coord(int t, int tiles_m, int tiles_n) {
    constexpr int BAND = 16;
    const int per_l = tiles_m * tiles_n;
    TileCoord tc;
    tc.l = t / per_l;
    int r = t - tc.l * per_l;
    const int band = r / (BAND * tiles_n);
    r -= band * BAND * tiles_n;
    const int rows_in_band = min(BAND, tiles_m - band * BAND);
    tc.nt = r / rows_in_band;
    tc.mt = band * BAND + (r - tc.nt * rows_in_band);
    return tc;
}

__device__ __forceinline__ float silu_mul(float x, float y) { return x / (1.0f + __expf(-x)) * y; }

// BN: output columns per tile (GEMM: 128 or 256; DUAL: 128, the MMA is 256 wide over [B1;B2]).
template <int BN, bool DUAL, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ CUtensorMap tmap_b2, const GemmParams p) {
    constexpr int MMA_N = DUAL ? 2 * BN : BN;          // rows of the B tile in shared memory
    constexpr int NB_BLOCKS = MMA_N / 128;             // 128-row scale blocks of B per stage
    constexpr uint32_t A_BYTES = BM * 128;
    constexpr uint32_t B_BYTES = MMA_N * 128;
    constexpr uint32_t SFA_BYTES = 4 * 512;            // 4 k-steps of 64 elements
    constexpr uint32_t SFB_BYTES = NB_BLOCKS * 4 * 512;
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
    constexpr uint32_t SF_COLS = 16 + 4 * (MMA_N / 32);  // TMEM columns of one stage's scales
    static_assert(MMA_N == 128 || MMA_N == 256, "MMA N");
    static_assert(MMA_N + 2 * SF_COLS <= TMEM_COLS, "tensor memory");

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 2];
    __shared__ uint32_t tmem_base_slot;

    // operand tiles need 1024-byte alignment for the 128-byte swizzle
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t acc_full = smem_u32(&bars[2 * STAGES]), acc_empty = acc_full + 8;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 4);  // one arrival per epilogue warp
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
        if (DUAL) prefetch_tmap(&tmap_b2);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    const int tiles_m = (p.M + BM - 1) / BM;
    const int tiles_n = (p.N + BN - 1) / BN;
    const int total_tiles = tiles_m * tiles_n * p.L;
    const int kiters = p.K / BK;
    const int RA = tiles_m;                  // 128-row scale blocks of A per batch
    const int RB = (p.N + 127) / 128;        // 128-row scale blocks of B per batch
    const size_t sf_row_block = (size_t)(p.K / 64) * 512;   // bytes of one 128-row scale block

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (one lane)
        if (elect_one()) {
            uint32_t it = 0;
            bool alive = true;
            for (int t = blockIdx.x; alive && t < total_tiles; t += gridDim.x) {
                const TileCoord tc = tile_coord(t, tiles_m, tiles_n);
                const int m0 = tc.mt * BM, n0 = tc.nt * BN;
                const uint8_t* sfa_t = p.sfa + ((size_t)tc.l * RA + tc.mt) * sf_row_block;
                // scale blocks of B rows [n0, n0 + BN): index of the first 128-row block
                const size_t sfb_blk0 = (size_t)tc.l * RB + n0 / 128;
                int nb_valid = NB_BLOCKS;  // 128-row blocks of the B tile that exist (N tail)
                if (!DUAL) nb_valid = min(NB_BLOCKS, RB - n0 / 128);
                for (int kit = 0; kit < kiters; kit++, it++) {
                    const int slot = it % STAGES;
                    if (!mbar_wait(empty0 + 8 * slot, ((it / STAGES) & 1) ^ 1, p.budget_ns)) {
                        report_status(p.status, DEV_TIMEOUT_PRODUCER);
                        alive = false;
                        break;
                    }
                    const uint32_t full = full0 + 8 * slot;
                    const uint32_t sA = smem0 + slot * STAGE_BYTES;
                    const uint32_t sB = sA + A_BYTES;
                    const uint32_t sSFA = sB + B_BYTES;
                    const uint32_t sSFB = sSFA + SFA_BYTES;
                    const int k0 = kit * BK;
                    const uint32_t tx = A_BYTES + B_BYTES + SFA_BYTES + (uint32_t)nb_valid * 2048u;
                    mbar_arrive_expect_tx(full, tx);
                    tma_load_3d(sA, &tmap_a, k0, m0, tc.l, full);
                    if (DUAL) {
                        tma_load_3d(sB, &tmap_b, k0, n0, tc.l, full);
                        tma_load_3d(sB + BN * 128, &tmap_b2, k0, n0, tc.l, full);
                    } else {
                        tma_load_3d(sB, &tmap_b, k0, n0, tc.l, full);
                    }
                    const size_t koff = (size_t)(k0 / 64) * 512;
                    bulk_g2s(sSFA, sfa_t + koff, 2048u, full);
                    if (DUAL) {
                        bulk_g2s(sSFB, p.sfb + sfb_blk0 * sf_row_block + koff, 2048u, full);
                        bulk_g2s(sSFB + 2048u, p.sfb2 + sfb_blk0 * sf_row_block + koff, 2048u, full);
                    } else {
                        for (int j = 0; j < nb_valid; j++)
                            bulk_g2s(sSFB + j * 2048u, p.sfb + (sfb_blk0 + j) * sf_row_block + koff, 2048u, full);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (one lane)
        if (elect_one()) {
            constexpr uint32_t idesc = make_idesc_nvfp4(BM, MMA_N);
            uint32_t it = 0, tile_it = 0;
            bool alive = true;
            for (int t = blockIdx.x; alive && t < total_tiles; t += gridDim.x, tile_it++) {
                // the epilogue must have drained the accumulator of the previous tile
                if (!mbar_wait(acc_empty, (tile_it & 1) ^ 1, p.budget_ns)) {
                    report_status(p.status, DEV_TIMEOUT_MMA_ACC);
                    break;
                }
                tc_fence_after_sync();
                for (int kit = 0; kit < kiters; kit++, it++) {
                    const int slot = it % STAGES;
                    if (!mbar_wait(full0 + 8 * slot, (it / STAGES) & 1, p.budget_ns)) {
                        report_status(p.status, DEV_TIMEOUT_CONSUMER);
                        alive = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t sA = smem0 + slot * STAGE_BYTES;
                    const uint32_t sB = sA + A_BYTES;
                    const uint32_t sSFA = sB + B_BYTES;
                    const uint32_t sSFB = sSFA + SFA_BYTES;
                    // scales of this stage: two alternating TMEM regions after the accumulator columns
                    const uint32_t t_sfa = tmem_base + MMA_N + (it & 1) * SF_COLS;
                    const uint32_t t_sfb = t_sfa + 16;
#pragma unroll
                    for (int ks = 0; ks < 4; ks++) {
                        tc_cp_sf_atom(t_sfa + 4 * ks, make_desc_sf(sSFA + 512 * ks));
#pragma unroll
                        for (int j = 0; j < NB_BLOCKS; j++)
                            tc_cp_sf_atom(t_sfb + ks * (MMA_N / 32) + 4 * j, make_desc_sf(sSFB + j * 2048 + 512 * ks));
                    }
#pragma unroll
                    for (int ks = 0; ks < 4; ks++) {
                        tc_mma_nvfp4(tmem_base, make_desc_k_sw128(sA + 32 * ks), make_desc_k_sw128(sB + 32 * ks), idesc,
                                     t_sfa + 4 * ks, t_sfb + ks * (MMA_N / 32), (kit | ks) != 0 ? 1u : 0u);
                    }
                    tc_commit(empty0 + 8 * slot);  // frees the stage once these MMAs have read it
                }
                if (alive) tc_commit(acc_full);     // accumulator complete
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps 2..5
        const int q = warp & 3;                      // TMEM lane quadrant this warp may access
        const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
        uint32_t tile_it = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, tile_it++) {
            const TileCoord tc = tile_coord(t, tiles_m, tiles_n);
            const int row = tc.mt * BM + q * 32 + lane;
            const int n0 = tc.nt * BN;
            if (!mbar_wait(acc_full, tile_it & 1, p.budget_ns)) {
                if (lane == 0) report_status(p.status, DEV_TIMEOUT_EPILOGUE);
                break;
            }
            tc_fence_after_sync();
            __half* crow = p.c + ((size_t)tc.l * p.M + (size_t)(row < p.M ? row : 0)) * p.N + n0;
#pragma unroll 1
            for (int cc = 0; cc < BN / 32; cc++) {
                uint32_t v[32];
                __align__(16) __half2 h[16];
                tc_ld_32x32(t_lane + cc * 32, v);
                if (DUAL) {
                    uint32_t w[32];
                    tc_ld_32x32(t_lane + BN + cc * 32, w);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const float x0 = p.alpha * __uint_as_float(v[2 * i]), x1 = p.alpha * __uint_as_float(v[2 * i + 1]);
                        const float y0 = p.alpha * __uint_as_float(w[2 * i]), y1 = p.alpha * __uint_as_float(w[2 * i + 1]);
                        h[i] = __floats2half2_rn(silu_mul(x0, y0), silu_mul(x1, y1));
                    }
                } else {
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; i++)
                        h[i] = __floats2half2_rn(p.alpha * __uint_as_float(v[2 * i]), p.alpha * __uint_as_float(v[2 * i + 1]));
                }
                if (row < p.M && n0 + cc * 32 < p.N) {
                    uint4* dst = reinterpret_cast<uint4*>(crow + cc * 32);
                    const uint4* src = reinterpret_cast<const uint4*>(h);
#pragma unroll
                    for (int i = 0; i < 4; i++) dst[i] = src[i];
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------ host side
// Tensor map over a packed-e2m1 operand [L][rows][K/2]: dimensions (K elements, rows, L), box
// (256 elements = 128 bytes, box_rows, 1), 128-byte swizzle, out-of-range rows read as zero.
int make_operand_tmap(CUtensorMap* map, const void* base, int rows, int K, int L, int box_rows) {
    const uint64_t dims[3] = {(uint64_t)K, (uint64_t)rows, (uint64_t)L};
    const uint64_t strides[2] = {(uint64_t)(K / 2), (uint64_t)rows * (uint64_t)(K / 2)};
    const uint32_t box[3] = {256u, (uint32_t)box_rows, 1u};
    return encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN8B, 3, base, dims, strides, box,
                        CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int BN, bool DUAL, int STAGES>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const GemmParams& p,
                       cudaStream_t stream) {
    constexpr int MMA_N = DUAL ? 2 * BN : BN;
    constexpr size_t STAGE = 128 * 128 + MMA_N * 128 + 2048 + (MMA_N / 128) * 2048;
    constexpr size_t SMEM = STAGES * STAGE + 1024;  // + slack for the 1024-byte alignment
    static_assert(SMEM <= 227 * 1024 - 256, "shared memory");
    auto kern = gemm_kernel<BN, DUAL, STAGES>;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 64) return NVFP4_ERR_UNSUPPORTED;
    if (!configured[dev]) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }
    const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * p.L;
    const int grid = tiles < sm_count(dev) ? tiles : sm_count(dev);
    kern<<<grid, GEMM_THREADS, SMEM, stream>>>(ta, tb, tb2, p);
    e = cudaGetLastError();
    return e == cudaSuccess ? NVFP4_OK : (int)e;
}

static int check_common(const void* const* ptrs, int nptr, int M, int N, int K, int L) {
    for (int i = 0; i < nptr; i++) {
        if (!ptrs[i]) return NVFP4_ERR_NULL;
        if ((uintptr_t)ptrs[i] & 15) return NVFP4_ERR_ALIGN;
    }
    if (M <= 0 || N <= 0 || K <= 0 || L <= 0) return NVFP4_ERR_SHAPE;
    if (K % BK != 0) return NVFP4_ERR_K_MULTIPLE;
    if (N % 128 != 0) return NVFP4_ERR_N_MULTIPLE;
    return NVFP4_OK;
}

}  // namespace nvfp4

using namespace nvfp4;

extern "C" int nvfp4_gemm(const void* a, const void* b, const void* sfa_sw, const void* sfb_sw, void* c, int M, int N,
                          int K, int L, float alpha, void* stream) {
    const void* ptrs[5] = {a, b, sfa_sw, sfb_sw, c};
    int rc = check_common(ptrs, 5, M, N, K, L);
    if (rc) return rc;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    // 256-wide tiles when N allows and they still fill the machine, else 128-wide
    const long tiles256 = (long)((M + 127) / 128) * (N / 256) * L;
    const bool wide = (N % 256 == 0) && tiles256 >= sm_count(dev);
    CUtensorMap ta, tb;
    rc = make_operand_tmap(&ta, a, M, K, L, 128);
    if (rc) return rc;
    rc = make_operand_tmap(&tb, b, N, K, L, wide ? 256 : 128);
    if (rc) return rc;
    GemmParams p;
    p.sfa = (const uint8_t*)sfa_sw; p.sfb = (const uint8_t*)sfb_sw; p.sfb2 = nullptr; p.c = (__half*)c;
    p.M = M; p.N = N; p.K = K; p.L = L; p.alpha = alpha;
    p.status = status_word(dev);
    p.budget_ns = wait_budget_ns();
    if (wide) return launch_gemm<256, false, 4>(ta, tb, tb, p, (cudaStream_t)stream);
    return launch_gemm<128, false, 6>(ta, tb, tb, p, (cudaStream_t)stream);
}

extern "C" int nvfp4_dual_gemm(const void* a, const void* b1, const void* b2, const void* sfa_sw, const void* sfb1_sw,
                               const void* sfb2_sw, void* c, int M, int N, int K, int L, float alpha, void* stream) {
    const void* ptrs[7] = {a, b1, b2, sfa_sw, sfb1_sw, sfb2_sw, c};
    int rc = check_common(ptrs, 7, M, N, K, L);
    if (rc) return rc;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    CUtensorMap ta, tb1, tb2;
    rc = make_operand_tmap(&ta, a, M, K, L, 128);
    if (rc) return rc;
    rc = make_operand_tmap(&tb1, b1, N, K, L, 128);
    if (rc) return rc;
    rc = make_operand_tmap(&tb2, b2, N, K, L, 128);
    if (rc) return rc;
    GemmParams p;
    p.sfa = (const uint8_t*)sfa_sw; p.sfb = (const uint8_t*)sfb1_sw; p.sfb2 = (const uint8_t*)sfb2_sw;
    p.c = (__half*)c; p.M = M; p.N = N; p.K = K; p.L = L; p.alpha = alpha;
    p.status = status_word(dev);
    p.budget_ns = wait_budget_ns();
    return launch_gemm<128, true, 4>(ta, tb1, tb2, p, (cudaStream_t)stream);
}
