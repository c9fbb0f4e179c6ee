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

#include <string.h>

#include <mutex>
#include <vector>

#include "gemm_common.cuh"
#include "nvfp4_internal.h"
#include "ptx_sm100.cuh"

namespace nvfp4 {

// BN: output columns per tile (GEMM: 128 or 256; DUAL: 128, the MMA is 256 wide over [B1;B2]).
// QOUT: the epilogue writes NVFP4 (packed codes + swizzled block scales) instead of fp16.
// GATHER: the fp16 output goes to the full C buffer of every rank of an N-sharded run (fused all-gather).
template <int BN, bool DUAL, bool GROUPED, int STAGES, bool QOUT = false, bool GATHER = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ CUtensorMap tmap_b2,
            const __grid_constant__ typename GatherMapsOf<GATHER>::type gmaps, const GemmParams p) {
    constexpr int MMA_N = DUAL ? 2 * BN : BN;          // rows of the B tile in shared memory
    constexpr int NB_BLOCKS = MMA_N / 128;             // 128-row scale blocks of B per stage
    constexpr uint32_t A_BYTES = BM * 128;
    constexpr uint32_t B_BYTES = MMA_N * 128;
    constexpr uint32_t SFA_BYTES = 4 * 512;            // 4 k-steps of 64 elements
    constexpr uint32_t SFB_BYTES = NB_BLOCKS * 4 * 512;
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
    constexpr uint32_t SF_COLS = 16 + 4 * (MMA_N / 32);  // TMEM columns of one stage's scales
    // Tensor memory: two accumulators and two alternating scale regions.  Two 256-column accumulators do
    // not fit beside the scales, so the second one starts early and overlaps the tail of the first by
    // OVERLAP columns; the epilogue drains the shared columns first and releases them on their own barrier.
    constexpr uint32_t SF_BASE = TMEM_COLS - 2 * SF_COLS;
    constexpr uint32_t ACC1_OFF = (2 * MMA_N <= SF_BASE) ? MMA_N : SF_BASE - MMA_N;
    constexpr uint32_t OVERLAP = MMA_N - ACC1_OFF;
    constexpr int OV_CHUNKS = OVERLAP / 32;             // 32-column chunks the two buffers share
    static_assert(MMA_N == 128 || MMA_N == 256, "MMA N");
    static_assert(OVERLAP % 32 == 0 && ACC1_OFF % 32 == 0, "accumulator overlap");

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 5];
    __shared__ uint32_t tmem_base_slot;
#ifdef NVFP4_PROFILE
    __shared__ long long prof_issue[STAGES];   // clock at which the producer issued a stage's loads
#endif

    // operand tiles need 1024-byte alignment for the 128-byte swizzle
    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t acc_full0 = smem_u32(&bars[2 * STAGES]);   // [2] accumulator complete
    const uint32_t acc_empty0 = acc_full0 + 16;               // [2] accumulator drained
    const uint32_t ovl_free = acc_full0 + 32;                 // shared columns drained (once per tile)

    if (threadIdx.x == 0) {
        if (!GROUPED) {
            prefetch_tmap(&tmap_a);
            prefetch_tmap(&tmap_b);
            if (DUAL) prefetch_tmap(&tmap_b2);
        }
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, 4);  // one arrival per epilogue warp
        }
        mbar_init(ovl_free, 4);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), TMEM_COLS);
        tmem_relinquish();
    }
    // The producer warp initialised the barriers itself and needs no tensor memory: it publishes the barriers and
    // starts loading at once (0.6 us earlier, which counts for calls that take ten); the other warps wait for the
    // barriers and for the tensor-memory address.
    uint32_t tmem_base = 0;
    if (warp == 0) {
        __syncwarp();
        named_bar_arrive(1, GEMM_THREADS);
    } else {
        tc_fence_before_sync();
        named_bar_sync(1, GEMM_THREADS);
        tc_fence_after_sync();
        tmem_base = tmem_base_slot;
    }

    const int total_tiles = p.total_tiles;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (one lane)
        if (elect_one()) {
            uint32_t it = 0;
            bool alive = true;
#ifdef NVFP4_PROFILE
            long long prof_empty = 0;
#endif
            for (int t = blockIdx.x; alive && t < total_tiles; t += gridDim.x) {
                const TileInfo ti = locate<BN, DUAL, GROUPED>(t, p, &tmap_a, &tmap_b, &tmap_b2);
                for (int kit = 0; kit < ti.kiters; kit++, it++) {
                    const int slot = it % STAGES;
                    bool free_;
                    {
                        PROF_T0();
                        free_ = mbar_wait(empty0 + 8 * slot, ((it / STAGES) & 1) ^ 1, p.budget_ns);
                        PROF_ADD(prof_empty);
                    }
                    if (!free_) {
                        report_status(p.status, DEV_TIMEOUT_PRODUCER);
                        alive = false;
                        break;
                    }
#ifdef NVFP4_PROFILE
                    prof_issue[slot] = clock64();
#endif
                    const uint32_t full = full0 + 8 * slot;
                    const uint32_t sA = smem0 + slot * STAGE_BYTES;
                    const uint32_t sB = sA + A_BYTES;
                    const uint32_t sSFA = sB + B_BYTES;
                    const uint32_t sSFB = sSFA + SFA_BYTES;
                    const int k0 = kit * BK;
                    const uint32_t tx = A_BYTES + B_BYTES + SFA_BYTES + (uint32_t)ti.nb_valid * 2048u;
                    mbar_arrive_expect_tx(full, tx);
                    tma_load_3d(sA, ti.ta, k0, ti.m0, ti.l, full);
                    tma_load_3d(sB, ti.tb, k0, ti.n0, ti.l, full);
                    if (DUAL) tma_load_3d(sB + BN * 128, ti.tb2, k0, ti.n0, ti.l, full);
                    const size_t koff = (size_t)(k0 / 64) * 512;
                    bulk_g2s(sSFA, ti.sfa_t + koff, 2048u, full);
                    if (DUAL) {
                        bulk_g2s(sSFB, ti.sfb_t + koff, 2048u, full);
                        bulk_g2s(sSFB + 2048u, ti.sfb2_t + koff, 2048u, full);
                    } else {
                        for (int j = 0; j < ti.nb_valid; j++)
                            bulk_g2s(sSFB + j * 2048u, ti.sfb_t + j * ti.sf_row_block + koff, 2048u, full);
                    }
                }
            }
#ifdef NVFP4_PROFILE
            if (p.prof) p.prof[8 * blockIdx.x + 4] = prof_empty;
#endif
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (one lane)
        if (elect_one()) {
            constexpr uint32_t idesc = make_idesc_nvfp4(BM, MMA_N);
            uint32_t it = 0, tile_it = 0;
            bool alive = true;
#ifdef NVFP4_PROFILE
            long long prof_acc = 0, prof_full = 0, prof_lat = 0, prof_late = 0;
            const long long prof_begin = clock64();
#endif
            for (int t = blockIdx.x; alive && t < total_tiles; t += gridDim.x, tile_it++) {
                // this buffer's previous tile (two tiles back) must be drained, and the previous tile's
                // epilogue must have released the columns the two buffers share
                const uint32_t buf = tile_it & 1;
                bool ok;
                {
                    PROF_T0();
                    ok = mbar_wait(acc_empty0 + 8 * buf, ((tile_it >> 1) & 1) ^ 1, p.budget_ns);
                    if (ok && OVERLAP > 0 && tile_it > 0) ok = mbar_wait(ovl_free, (tile_it - 1) & 1, p.budget_ns);
                    PROF_ADD(prof_acc);
                }
                if (!ok) {
                    report_status(p.status, DEV_TIMEOUT_MMA_ACC);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t t_acc = tmem_base + buf * ACC1_OFF;
                const int kiters = locate<BN, DUAL, GROUPED>(t, p, &tmap_a, &tmap_b, &tmap_b2).kiters;
                for (int kit = 0; kit < kiters; kit++, it++) {
                    const int slot = it % STAGES;
                    bool got;
                    {
                        PROF_T0();
#ifdef NVFP4_PROFILE
                        if (!mbar_try_wait(full0 + 8 * slot, (it / STAGES) & 1)) prof_late++;
#endif
                        got = mbar_wait(full0 + 8 * slot, (it / STAGES) & 1, p.budget_ns);
                        PROF_ADD(prof_full);
                    }
                    if (!got) {
                        report_status(p.status, DEV_TIMEOUT_CONSUMER);
                        alive = false;
                        break;
                    }
#ifdef NVFP4_PROFILE
                    prof_lat += clock64() - prof_issue[slot];   // upper bound of the load latency when the stage was waited for
#endif
                    tc_fence_after_sync();
                    const uint32_t sA = smem0 + slot * STAGE_BYTES;
                    const uint32_t sB = sA + A_BYTES;
                    const uint32_t sSFA = sB + B_BYTES;
                    const uint32_t sSFB = sSFA + SFA_BYTES;
                    // scales of this stage: two alternating TMEM regions after the accumulator columns
                    const uint32_t t_sfa = tmem_base + SF_BASE + (it & 1) * SF_COLS;
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
                        tc_mma_nvfp4(t_acc, make_desc_k_sw128(sA + 32 * ks), make_desc_k_sw128(sB + 32 * ks), idesc,
                                     t_sfa + 4 * ks, t_sfb + ks * (MMA_N / 32), (kit | ks) != 0 ? 1u : 0u);
                    }
                    tc_commit(empty0 + 8 * slot);  // frees the stage once these MMAs have read it
                }
                if (alive) tc_commit(acc_full0 + 8 * buf);  // accumulator complete
            }
#ifdef NVFP4_PROFILE
            if (p.prof) {
                p.prof[8 * blockIdx.x + 0] = prof_acc;
                p.prof[8 * blockIdx.x + 1] = prof_full;
                p.prof[8 * blockIdx.x + 2] = clock64() - prof_begin;
                p.prof[8 * blockIdx.x + 3] = prof_lat;
                p.prof[8 * blockIdx.x + 5] = prof_late;
                p.prof[8 * blockIdx.x + 6] = it;
            }
#endif
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps 2..5
        const int q = warp & 3;                      // TMEM lane quadrant this warp may access
        uint32_t tile_it = 0;
        GatherCtx gc;
        if constexpr (GATHER) {
            gc.maps = gmaps.m;
            gc.n = p.gather.n;
            gc.stage_smem = smem0 + STAGES * STAGE_BYTES + (uint32_t)(warp - 2) * (GATHER_BOXES * 4096u);
#ifdef NVFP4_PROFILE
            gc.mask = p.gather.mask;
#endif
            gc.stage = reinterpret_cast<uint4*>(smem_raw + (gc.stage_smem - smem_u32(smem_raw)));
            gc.uses = 0;
        }
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, tile_it++) {
            const TileInfo ti = locate<BN, DUAL, GROUPED>(t, p, &tmap_a, &tmap_b, &tmap_b2);
            const int row = ti.m0 + q * 32 + lane;
            const int n0 = ti.n0;
            const uint32_t buf = tile_it & 1;
            if (!mbar_wait(acc_full0 + 8 * buf, (tile_it >> 1) & 1, p.budget_ns)) {
                if (lane == 0) report_status(p.status, DEV_TIMEOUT_EPILOGUE);
                break;
            }
            tc_fence_after_sync();
            const uint32_t t_lane = tmem_base + buf * ACC1_OFF + ((uint32_t)(q * 32) << 16);
            const int srow = row < ti.M ? row : 0;
            const int wrow0 = ti.m0 + q * 32;          // first row of this warp
            __half* crow = GATHER ? nullptr : ti.c + (size_t)srow * ti.N + n0;
            if constexpr (GATHER) {
                gc.x = p.gather.col0 + n0;
                gc.y = wrow0;
                gc.z = ti.l;
                gc.rows_exist = wrow0 < ti.M;
            }
            QuantOut qo;
            if (QOUT) {
                const size_t grow = (size_t)ti.l * ti.M + srow;                       // row of the [L*M][N] output
                qo.codes = p.cq + grow * (size_t)(ti.N / 2) + n0 / 2;
                const size_t rb = (size_t)ti.l * ((ti.M + 127) / 128) + srow / 128;   // 128-row block of the scales
                qo.scales = p.sfc + (rb * (size_t)(ti.N / 64) + n0 / 64) * 512 + (srow % 32) * 16 + ((srow % 128) / 32) * 4;
            }
            // buffer 0 shares its last OVERLAP columns, buffer 1 its first
            if (buf == 0)
                epilogue_tile<BN, DUAL, int(ACC1_OFF) / 32, OV_CHUNKS, false, QOUT, GATHER>(
                    t_lane, crow, row < ti.M, n0, ti.N, p.alpha, ovl_free, lane, &qo, &gc);
            else
                epilogue_tile<BN, DUAL, 0, OV_CHUNKS, false, QOUT, GATHER>(t_lane, crow, row < ti.M, n0, ti.N, p.alpha,
                                                                          ovl_free, lane, &qo, &gc);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
        }
        // the boxes stay in this CTA's shared memory until the last bulk store has read them, and the kernel's
        // results are complete only when the stores are
        if constexpr (GATHER) {
            if (lane < gc.n) tma_store_wait_all<0>();
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
// (256 elements = 128 bytes, box_rows, 1), 128-byte swizzle, out-of-range rows read as zero.  Kept per thread
// (TmapCache), keyed by everything that goes into it.
int make_operand_tmap(CUtensorMap* map, const void* base, int rows, int K, int L, int box_rows) {
    thread_local TmapCache<> cache = {};
    // K and the box share a field: K is a multiple of 64 and the box at most 256 rows
    const TmapKey key{(uint64_t)(uintptr_t)base, rows, K, L, box_rows};
    if (cache.find(key, map)) return NVFP4_OK;
    // (describing the same bytes as a UINT8 tensor with 128-byte rows instead of 256 four-bit elements was measured
    // at the same speed: the packed nibbles travel unchanged either way)
    const uint64_t dims[3] = {(uint64_t)K, (uint64_t)rows, (uint64_t)L};
    const uint64_t strides[2] = {(uint64_t)(K / 2), (uint64_t)rows * (uint64_t)(K / 2)};
    const uint32_t box[3] = {256u, (uint32_t)box_rows, 1u};
    int rc = encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN8B, 3, base, dims, strides, box,
                          CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    cache.put(key, *map);
    return NVFP4_OK;
}

int make_scale_tmap(CUtensorMap* map, const void* base, long atoms) {
    struct Entry { const void* base; long atoms; CUtensorMap m; bool valid; };
    constexpr int WAYS = 8;
    thread_local Entry cache[WAYS] = {};
    thread_local int victim = 0;
    for (int i = 0; i < WAYS; i++)
        if (cache[i].valid && cache[i].base == base && cache[i].atoms == atoms) {
            *map = cache[i].m;
            return NVFP4_OK;
        }
    const uint64_t dims[2] = {64u, (uint64_t)atoms};
    const uint64_t strides[1] = {512u};
    const uint32_t box[2] = {64u, 4u};
    int rc = encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    cache[victim] = Entry{base, atoms, *map, true};
    victim = (victim + 1) % WAYS;
    return NVFP4_OK;
}

template <int BN, bool DUAL, bool GROUPED, int STAGES, bool QOUT = false, bool GATHER = false>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const GemmParams& p,
                       cudaStream_t stream, const typename GatherMapsOf<GATHER>::type& gm = {}) {
    constexpr int MMA_N = DUAL ? 2 * BN : BN;
    constexpr size_t STAGE = 128 * 128 + MMA_N * 128 + 2048 + (MMA_N / 128) * 2048;
    // + slack for the 1024-byte alignment (+ the 4 KB boxes of the epilogue warps for the gathering stores)
    constexpr size_t SMEM = STAGES * STAGE + 1024 + (GATHER ? 4 * GATHER_BOXES * 4096 : 0);
    static_assert(SMEM <= 227 * 1024 - 256, "shared memory");
    auto kern = gemm_kernel<BN, DUAL, GROUPED, STAGES, QOUT, GATHER>;
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
    if (p.total_tiles <= 0) return NVFP4_OK;
    const int grid = p.total_tiles < sm_count(dev) ? p.total_tiles : sm_count(dev);
    kern<<<grid, GEMM_THREADS, SMEM, stream>>>(ta, tb, tb2, gm, p);
    e = cudaGetLastError();
    return e == cudaSuccess ? NVFP4_OK : (int)e;
}

static int check_common(const void* const* ptrs, int nptr, int M, int N, int K, int L) {
    for (int i = 0; i < nptr; i++) {
        if (!ptrs[i]) return NVFP4_ERR_NULL;
        if ((uintptr_t)ptrs[i] & 15) return NVFP4_ERR_ALIGN;
    }
    if ((uintptr_t)ptrs[nptr - 1] & 31) return NVFP4_ERR_ALIGN;  // the output is written with 256-bit stores
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
    // CTA-pair kernel (256 x 256 tiles on two SMs): a third fewer bytes per SM and K step; 192-196 us against 224 us
    // at 8192^3.  Used wherever pair_kernel_suits() says so; NVFP4_GEMM_PAIR=0 turns it off, =1 forces it wherever
    // the shape allows it at all.
    static const int pair_mode = [] { const char* e_ = getenv("NVFP4_GEMM_PAIR"); return e_ ? atoi(e_) : 2; }();
    const bool use_pair = pair_mode != 0 && N % 256 == 0 && M >= 256 &&
                          (pair_mode == 1 || pair_kernel_suits(M, N, K, L, false, dev));
    // few tiles and a long K loop: split K across a cluster (NVFP4_GEMM_SPLITK=0 turns it off)
    // (NVFP4_GEMM_SPLITK = 2, 4 or 8 forces that cluster size where the shape allows it: tuning aid)
    static const int splitk_mode = [] { const char* e_ = getenv("NVFP4_GEMM_SPLITK"); return e_ ? atoi(e_) : -1; }();
    int split = (splitk_mode != 0 && !use_pair) ? splitk_factor(M, N, K, L, dev) : 0;
    if (splitk_mode >= 2 && !use_pair && (long)((M + 127) / 128) * (N / 128) * L * splitk_mode <= 2 * sm_count(dev) &&
        K / BK >= splitk_mode)
        split = splitk_mode;
    CUtensorMap ta, tb;
    rc = make_operand_tmap(&ta, a, M, K, L, 128);
    if (rc) return rc;
    rc = make_operand_tmap(&tb, b, N, K, L, (wide && !use_pair && !split) ? 256 : 128);
    if (rc) return rc;
    GemmParams p;
    p.sfa = (const uint8_t*)sfa_sw; p.sfb = (const uint8_t*)sfb_sw; p.sfb2 = nullptr; p.c = (__half*)c;
    p.M = M; p.N = N; p.K = K; p.L = L; p.alpha = alpha;
    p.status = status_word(dev);
    p.budget_ns = wait_budget_ns();
    p.table = nullptr; p.G = 0;
    p.total_tiles = ((M + BM - 1) / BM) * (N / (wide ? 256 : 128)) * L;
#ifdef NVFP4_PROFILE
    { const char* e_ = getenv("NVFP4_PROF_PTR"); p.prof = e_ ? (unsigned long long*)strtoull(e_, nullptr, 0) : nullptr; }
#endif
    if (split) return launch_gemm_splitk(split, ta, tb, p, (cudaStream_t)stream);
    if (use_pair) return launch_gemm_pair(false, ta, tb, tb, p, (cudaStream_t)stream);
    if (wide) return launch_gemm<256, false, false, 4>(ta, tb, tb, p, (cudaStream_t)stream);
    return launch_gemm<128, false, false, 6>(ta, tb, tb, p, (cudaStream_t)stream);
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
    p.table = nullptr; p.G = 0;
    p.total_tiles = ((M + BM - 1) / BM) * (N / 128) * L;
    static const int pair_mode = [] { const char* e_ = getenv("NVFP4_GEMM_PAIR"); return e_ ? atoi(e_) : 2; }();
    if (pair_mode != 0 && M >= 256 && (pair_mode == 1 || pair_kernel_suits(M, N, K, L, true, dev)))
        return launch_gemm_pair(true, ta, tb1, tb2, p, (cudaStream_t)stream);
    // few tiles and a long K loop: split K across a cluster of 2 or 4, as for the GEMM (a CTA streams its operands
    // at what its shared memory holds in flight divided by the load latency, so the SMs that would idle are worth
    // more than the reduction costs); NVFP4_GEMM_SPLITK = 0 turns it off, 2 or 4 forces that size where it fits
    static const int splitk_mode = [] { const char* e_ = getenv("NVFP4_GEMM_SPLITK"); return e_ ? atoi(e_) : -1; }();
    int split = splitk_mode != 0 ? splitk_factor(M, N, K, L, dev) : 0;
    if ((splitk_mode == 2 || splitk_mode == 4) && (long)p.total_tiles * splitk_mode <= 2 * sm_count(dev) &&
        K / BK >= splitk_mode)
        split = splitk_mode;
    if (split) return launch_dual_gemm_splitk(split, ta, tb1, tb2, p, (cudaStream_t)stream);
    return launch_gemm<128, true, false, 4>(ta, tb1, tb2, p, (cudaStream_t)stream);
}

extern "C" int nvfp4_dual_gemm_nvfp4(const void* a, const void* b1, const void* b2, const void* sfa_sw,
                                     const void* sfb1_sw, const void* sfb2_sw, void* c_packed, void* sfc_sw, int M, int N,
                                     int K, int L, float alpha, void* stream) {
    const void* ptrs[8] = {a, b1, b2, sfa_sw, sfb1_sw, sfb2_sw, sfc_sw, c_packed};
    int rc = check_common(ptrs, 8, M, N, K, L);
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
    p.c = nullptr; p.cq = (uint8_t*)c_packed; p.sfc = (uint8_t*)sfc_sw;
    p.M = M; p.N = N; p.K = K; p.L = L; p.alpha = alpha;
    p.status = status_word(dev);
    p.budget_ns = wait_budget_ns();
    p.table = nullptr; p.G = 0;
    p.total_tiles = ((M + BM - 1) / BM) * (N / 128) * L;
    return launch_gemm<128, true, false, 4, true>(ta, tb1, tb2, p, (cudaStream_t)stream);
}

// Tensor map over one rank's full C, [L][M][ldc] fp16: box 64 columns x 32 rows (one epilogue warp's rows, 128
// bytes of each), 128-byte swizzle; rows past M are clipped by the store.  Kept per thread like the operand maps.
static int make_output_tmap(CUtensorMap* map, const void* base, int M, int ldc, int L) {
    struct Entry { const void* base; int M, ldc, L; CUtensorMap m; bool valid; };
    constexpr int WAYS = 16;
    thread_local Entry cache[WAYS] = {};
    thread_local int victim = 0;
    for (int i = 0; i < WAYS; i++) {
        const Entry& e = cache[i];
        if (e.valid && e.base == base && e.M == M && e.ldc == ldc && e.L == L) {
            *map = e.m;
            return NVFP4_OK;
        }
    }
    const uint64_t dims[3] = {(uint64_t)ldc, (uint64_t)M, (uint64_t)L};
    const uint64_t strides[2] = {(uint64_t)ldc * 2u, (uint64_t)M * (uint64_t)ldc * 2u};
    const uint32_t box[3] = {64u, 32u, 1u};
    int rc = encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    cache[victim] = Entry{base, M, ldc, L, *map, true};
    victim = (victim + 1) % WAYS;
    return NVFP4_OK;
}

// Fills the gather description and the ranks' output maps of a launch from the ranks' buffer addresses.
static int fill_gather(GatherOut& g, GatherMaps& gm, void* const* c_all, int world, int rank, int M, int N_local, int L) {
    if (!c_all) return NVFP4_ERR_NULL;
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return NVFP4_ERR_SHAPE;
    g.n = world; g.ldc = N_local * world; g.col0 = rank * N_local;
#ifdef NVFP4_PROFILE
    {   // timing experiments: "own" = only this rank's copy, "peers" = every copy but this rank's, else a bit mask
        const char* e_ = getenv("NVFP4_GATHER_MASK");
        if (e_ && !strcmp(e_, "own")) g.mask = 1u << rank;
        else if (e_ && !strcmp(e_, "peers")) g.mask = ~(1u << rank);
        else if (e_) g.mask = (unsigned)strtoul(e_, nullptr, 0);
    }
#endif
    for (int r = 0; r < 8; r++) {
        void* c = c_all[r < world ? r : 0];   // unused entries repeat a valid map
        if (!c) return NVFP4_ERR_NULL;
        if ((uintptr_t)c & 31) return NVFP4_ERR_ALIGN;
        int rc = make_output_tmap(&gm.m[r], c, M, g.ldc, L);
        if (rc) return rc;
    }
    return NVFP4_OK;
}

extern "C" int nvfp4_gemm_allgather(const void* a, const void* b, const void* sfa_sw, const void* sfb_sw,
                                    void* const* c_all, int world, int rank, int M, int N_local, int K, int L,
                                    float alpha, void* stream) {
    const void* ptrs[5] = {a, b, sfa_sw, sfb_sw, c_all ? c_all[0] : nullptr};
    int rc = check_common(ptrs, 5, M, N_local, K, L);
    if (rc) return rc;
    // one rank: nothing to gather, and the plain epilogue is the faster one for local memory (measured at 8192^3:
    // 223 us against 300 us through the staged stores)
    if (world == 1 && rank == 0 && c_all) return nvfp4_gemm(a, b, sfa_sw, sfb_sw, c_all[0], M, N_local, K, L, alpha, stream);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    GemmParams p;
    GatherMaps gm;
    rc = fill_gather(p.gather, gm, c_all, world, rank, M, N_local, L);
    if (rc) return rc;
    const long tiles256 = (long)((M + 127) / 128) * (N_local / 256) * L;
    const bool wide = (N_local % 256 == 0) && tiles256 >= sm_count(dev);
    CUtensorMap ta, tb;
    rc = make_operand_tmap(&ta, a, M, K, L, 128);
    if (rc) return rc;
    rc = make_operand_tmap(&tb, b, N_local, K, L, wide ? 256 : 128);
    if (rc) return rc;
    p.sfa = (const uint8_t*)sfa_sw; p.sfb = (const uint8_t*)sfb_sw; p.sfb2 = nullptr; p.c = nullptr;
    p.M = M; p.N = N_local; p.K = K; p.L = L; p.alpha = alpha;
    p.status = status_word(dev);
    p.budget_ns = wait_budget_ns();
    p.table = nullptr; p.G = 0;
    p.total_tiles = ((M + BM - 1) / BM) * (N_local / (wide ? 256 : 128)) * L;
#ifdef NVFP4_PROFILE
    { const char* e_ = getenv("NVFP4_PROF_PTR"); p.prof = e_ ? (unsigned long long*)strtoull(e_, nullptr, 0) : nullptr; }
#endif
    // one stage less than the plain kernels: the room goes to the epilogue warps' store boxes
    if (wide) return launch_gemm<256, false, false, 3, false, true>(ta, tb, tb, p, (cudaStream_t)stream, gm);
    return launch_gemm<128, false, false, (GATHER_BOXES <= 2 ? 5 : 4), false, true>(ta, tb, tb, p, (cudaStream_t)stream, gm);
}

extern "C" int nvfp4_dual_gemm_allgather(const void* a, const void* b1, const void* b2, const void* sfa_sw,
                                         const void* sfb1_sw, const void* sfb2_sw, void* const* c_all, int world,
                                         int rank, int M, int N_local, int K, int L, float alpha, void* stream) {
    const void* ptrs[7] = {a, b1, b2, sfa_sw, sfb1_sw, sfb2_sw, c_all ? c_all[0] : nullptr};
    int rc = check_common(ptrs, 7, M, N_local, K, L);
    if (rc) return rc;
    if (world == 1 && rank == 0 && c_all)
        return nvfp4_dual_gemm(a, b1, b2, sfa_sw, sfb1_sw, sfb2_sw, c_all[0], M, N_local, K, L, alpha, stream);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    GemmParams p;
    GatherMaps gm;
    rc = fill_gather(p.gather, gm, c_all, world, rank, M, N_local, L);
    if (rc) return rc;
    CUtensorMap ta, tb1, tb2;
    rc = make_operand_tmap(&ta, a, M, K, L, 128);
    if (rc) return rc;
    rc = make_operand_tmap(&tb1, b1, N_local, K, L, 128);
    if (rc) return rc;
    rc = make_operand_tmap(&tb2, b2, N_local, K, L, 128);
    if (rc) return rc;
    p.sfa = (const uint8_t*)sfa_sw; p.sfb = (const uint8_t*)sfb1_sw; p.sfb2 = (const uint8_t*)sfb2_sw; p.c = nullptr;
    p.M = M; p.N = N_local; p.K = K; p.L = L; p.alpha = alpha;
    p.status = status_word(dev);
    p.budget_ns = wait_budget_ns();
    p.table = nullptr; p.G = 0;
    p.total_tiles = ((M + BM - 1) / BM) * (N_local / 128) * L;
    return launch_gemm<128, true, false, 3, false, true>(ta, tb1, tb2, p, (cudaStream_t)stream, gm);
}

// ------------------------------------------------------------------------------------------ grouped GEMM
namespace nvfp4 {
namespace {

// The problem table of a launch lives in device memory that the library owns: per device a small ring of
// (pinned host staging buffer, device buffer, events) slots.  A slot is rewritten only after every launch that
// read it has finished (`done`), so concurrent streams and back-to-back calls never share a table that is being
// changed.  When the ring wraps onto a slot whose last launch is still running, the host waits for it
// (cudaEventSynchronize): 32 different descriptor arrays may be in flight per device before a call blocks.
// A repeated call reuses its slot's table; if it comes on another stream than the one that uploaded the table,
// its launch is ordered after the upload (`uploaded`), and `done` is re-recorded so that it still covers the
// launches of the earlier streams.
constexpr int TABLE_SLOTS = 32;   // (the harness times 15 grouped problems in turn: each keeps its table)
struct TableSlot {
    unsigned char* host = nullptr;   // GroupEntry[] or PairGroupEntry[]
    unsigned char* dev = nullptr;
    size_t capacity = 0;             // bytes
    cudaEvent_t done = nullptr;      // after the latest launch that reads this table (and, transitively, all earlier ones)
    cudaEvent_t uploaded = nullptr;  // after the host-to-device copy of the table
    cudaStream_t last_stream = nullptr;  // stream of the latest upload or launch
    bool used = false;
    // the call this slot's device table was built for: an identical call (same pointers and sizes, the usual
    // case when a layer runs again) reuses the table without re-encoding or uploading anything
    std::vector<nvfp4_group_t> key;
    int live = 0, tiles = 0, bn = 0;   // bn: tile width of the single-CTA kernel (128 / 256), or 2 = CTA pairs
};
struct TableRing {
    TableSlot slots[TABLE_SLOTS];
    int next = 0;
};
std::mutex g_table_mu;
TableRing g_rings[64];

int acquire_slot(int dev, size_t bytes, TableSlot** out) {
    TableRing& ring = g_rings[dev];
    TableSlot& s = ring.slots[ring.next];
    ring.next = (ring.next + 1) % TABLE_SLOTS;
    s.key.clear();
    cudaError_t e;
    if (s.used) {
        e = cudaEventSynchronize(s.done);
        if (e != cudaSuccess) return (int)e;
    }
    if (!s.done) {
        e = cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming);
        if (e != cudaSuccess) return (int)e;
    }
    if (!s.uploaded) {
        e = cudaEventCreateWithFlags(&s.uploaded, cudaEventDisableTiming);
        if (e != cudaSuccess) return (int)e;
    }
    s.used = false;
    if (s.capacity < bytes) {
        size_t cap = 32 * 1024;
        while (cap < bytes) cap *= 2;
        if (s.host) cudaFreeHost(s.host);
        if (s.dev) cudaFree(s.dev);
        s.host = nullptr; s.dev = nullptr; s.capacity = 0;
        e = cudaHostAlloc((void**)&s.host, cap, cudaHostAllocDefault);
        if (e != cudaSuccess) return (int)e;
        e = cudaMalloc((void**)&s.dev, cap);
        if (e != cudaSuccess) return (int)e;
        s.capacity = cap;
    }
    *out = &s;
    return NVFP4_OK;
}

}  // namespace
}  // namespace nvfp4

// Launch on a slot's finished table.  kind: 128 / 256 = tile width of the single-CTA kernel, 2 = CTA pairs.
static int launch_grouped(const TableSlot& slot, GemmParams& p, cudaStream_t st) {
    p.G = slot.live; p.total_tiles = slot.tiles;
    if (slot.bn == 2) {
        p.table = nullptr; p.pair_table = slot.dev;
        return launch_gemm_pair_grouped(p, st);
    }
    p.table = reinterpret_cast<const GroupEntry*>(slot.dev); p.pair_table = nullptr;
    const CUtensorMap& dm = reinterpret_cast<const GroupEntry*>(slot.host)[0].ta;
    return slot.bn == 256 ? launch_gemm<256, false, true, 4>(dm, dm, dm, p, st)
                          : launch_gemm<128, false, true, 6>(dm, dm, dm, p, st);
}

extern "C" int nvfp4_grouped_gemm(const nvfp4_group_t* groups, int G, float alpha, void* stream) {
    if (!groups) return NVFP4_ERR_NULL;
    if (G <= 0) return NVFP4_ERR_SHAPE;
    if (G > 65536) return NVFP4_ERR_TOO_MANY_GROUPS;
    bool wide = true;
    int live = 0;
    long tiles256 = 0;
    for (int g = 0; g < G; g++) {
        const nvfp4_group_t& q = groups[g];
        if (q.M < 0 || q.N <= 0 || q.K <= 0) return NVFP4_ERR_SHAPE;
        if (q.K % BK != 0) return NVFP4_ERR_K_MULTIPLE;
        if (q.N % 128 != 0) return NVFP4_ERR_N_MULTIPLE;
        if (q.M == 0) continue;  // empty group: nothing to read or write
        const void* ptrs[5] = {q.a, q.b, q.sfa_sw, q.sfb_sw, q.c};
        for (const void* ptr : ptrs) {
            if (!ptr) return NVFP4_ERR_NULL;
            if ((uintptr_t)ptr & 15) return NVFP4_ERR_ALIGN;
        }
        if ((uintptr_t)q.c & 31) return NVFP4_ERR_ALIGN;
        if (q.N % 256 != 0) wide = false;
        tiles256 += (long)((q.M + BM - 1) / BM) * (q.N / 256);
        live++;
    }
    if (live == 0) return NVFP4_OK;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 64) return NVFP4_ERR_UNSUPPORTED;
    // 256-wide tiles only when they still fill the machine, as for the plain GEMM (two groups of 3072 or 4096 columns:
    // 60 - 64 wide tiles for 148 SMs; 128-wide ones took 9.7 against 13.0 us and 7.4 against 9.4 us)
    if (tiles256 < sm_count(dev)) wide = false;
    // CTA pairs (256 x 256 tiles, gemm_pair_kernel<false, true>) are opt-in here (NVFP4_GEMM_PAIR=1): on the expert
    // layer of 64 groups with M_g around 128 they measured 234.7 us against 214.2 us for the single-CTA kernel.  The
    // layer streams its weights from HBM; a pair advances only when BOTH CTAs' halves of a stage have arrived, and
    // every group with M_g <= 128 leaves the second CTA's tensor work wasted.
    static const int pair_mode = [] { const char* e_ = getenv("NVFP4_GEMM_PAIR"); return e_ ? atoi(e_) : 2; }();
    const bool use_pair = wide && pair_mode == 1 && max_pairs_grouped(dev) > 0;
    const int bn = use_pair ? 2 : (wide ? 256 : 128);

    std::lock_guard<std::mutex> lk(g_table_mu);
    cudaStream_t st = (cudaStream_t)stream;
    GemmParams p;
    p.sfa = p.sfb = p.sfb2 = nullptr; p.c = nullptr;
    p.M = p.N = p.K = 0; p.L = 1; p.alpha = alpha;
    p.status = status_word(dev);
    p.budget_ns = wait_budget_ns();
#ifdef NVFP4_PROFILE
    { const char* e_ = getenv("NVFP4_PROF_PTR"); p.prof = e_ ? (unsigned long long*)strtoull(e_, nullptr, 0) : nullptr; }
#endif
    TableSlot* slot = nullptr;
    for (TableSlot& cand : g_rings[dev].slots) {
        if (cand.used && cand.key.size() == (size_t)G &&
            memcmp(cand.key.data(), groups, sizeof(nvfp4_group_t) * G) == 0) {
            slot = &cand;
            break;
        }
    }
    if (slot) {
        const bool other_stream = st != slot->last_stream;
        if (other_stream) {
            // the table may still be on its way to the device on the stream that built it
            e = cudaStreamWaitEvent(st, slot->uploaded, 0);
            if (e != cudaSuccess) return (int)e;
        }
        int rc2 = launch_grouped(*slot, p, st);
        if (other_stream) {
            // `done` is about to move to this stream: first make this stream's record wait for the launches the
            // old record stood for, so that the slot is not rewritten while any of them still reads the table
            e = cudaStreamWaitEvent(st, slot->done, 0);
            if (e != cudaSuccess) return (int)e;
            slot->last_stream = st;
        }
        e = cudaEventRecord(slot->done, st);
        if (rc2) return rc2;
        return e == cudaSuccess ? NVFP4_OK : (int)e;
    }
    const size_t entry_bytes = use_pair ? sizeof(PairGroupEntry) : sizeof(GroupEntry);
    int rc = acquire_slot(dev, entry_bytes * live, &slot);
    if (rc) return rc;
    int tiles = 0, n = 0;
    for (int g = 0; g < G; g++) {
        const nvfp4_group_t& q = groups[g];
        if (q.M == 0) continue;
        if (use_pair) {
            PairGroupEntry& en = reinterpret_cast<PairGroupEntry*>(slot->host)[n++];
            rc = make_operand_tmap(&en.ta, q.a, q.M, q.K, 1, 128);
            if (rc) return rc;
            rc = make_operand_tmap(&en.tb, q.b, q.N, q.K, 1, 128);
            if (rc) return rc;
            rc = make_scale_tmap(&en.tsa, q.sfa_sw, (long)((q.M + 127) / 128) * (q.K / 64));
            if (rc) return rc;
            rc = make_scale_tmap(&en.tsb, q.sfb_sw, (long)(q.N / 128) * (q.K / 64));
            if (rc) return rc;
            en.c = (__half*)q.c;
            en.M = q.M; en.N = q.N; en.K = q.K;
            en.tiles_m = (q.M + 255) / 256; en.tiles_n = q.N / 256;
            en.tile_start = tiles;
            tiles += en.tiles_m * en.tiles_n;
            continue;
        }
        GroupEntry& en = reinterpret_cast<GroupEntry*>(slot->host)[n++];
        rc = make_operand_tmap(&en.ta, q.a, q.M, q.K, 1, 128);
        if (rc) return rc;
        rc = make_operand_tmap(&en.tb, q.b, q.N, q.K, 1, bn);
        if (rc) return rc;
        en.sfa = (const uint8_t*)q.sfa_sw; en.sfb = (const uint8_t*)q.sfb_sw; en.c = (__half*)q.c;
        en.M = q.M; en.N = q.N; en.K = q.K;
        en.tiles_m = (q.M + BM - 1) / BM; en.tiles_n = q.N / bn;
        en.tile_start = tiles;
        tiles += en.tiles_m * en.tiles_n;
    }
    e = cudaMemcpyAsync(slot->dev, slot->host, entry_bytes * live, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return (int)e;
    e = cudaEventRecord(slot->uploaded, st);
    if (e != cudaSuccess) return (int)e;
    slot->last_stream = st;
    slot->key.assign(groups, groups + G);
    slot->live = live; slot->tiles = tiles; slot->bn = bn;
    rc = launch_grouped(*slot, p, st);
    slot->used = true;
    e = cudaEventRecord(slot->done, st);
    if (rc) return rc;
    return e == cudaSuccess ? NVFP4_OK : (int)e;
}

// Frees what the library allocated on first use: the grouped-GEMM problem tables of every device (pinned staging,
// device tables, events) and the status words.  The caller must have synchronised the streams it used.
namespace nvfp4 {
void free_status_words();
void free_stream_k_scratch();
}
extern "C" int nvfp4_shutdown(void) {
    std::lock_guard<std::mutex> lk(g_table_mu);
    int cur = 0;
    if (cudaGetDevice(&cur) != cudaSuccess) return NVFP4_ERR_INTERNAL;
    for (int dev = 0; dev < 64; dev++) {
        bool any = false;
        for (const TableSlot& sl : g_rings[dev].slots) any = any || sl.host || sl.dev || sl.done || sl.uploaded;
        if (!any) continue;
        cudaSetDevice(dev);
        for (TableSlot& sl : g_rings[dev].slots) {
            if (sl.host) cudaFreeHost(sl.host);
            if (sl.dev) cudaFree(sl.dev);
            if (sl.done) cudaEventDestroy(sl.done);
            if (sl.uploaded) cudaEventDestroy(sl.uploaded);
            sl = TableSlot();
        }
        g_rings[dev].next = 0;
    }
    cudaSetDevice(cur);
    free_stream_k_scratch();
    free_status_words();
    return NVFP4_OK;
}

// ------------------------------------------------------------------------------------------ grouped GEMM, no allocation
// Some callers cannot let this library allocate: a serving process whose own allocator has already claimed
// all of HBM (a cudaMalloc from a library would fail, or would have to be carved out of the budget up front),
// or a real-time loop that must not meet the implicit device-wide synchronisation of cudaMalloc / cudaFree.
// nvfp4_grouped_gemm() keeps its problem tables in memory it allocates on first use; the variant below keeps
// ONE table in a fixed array that is part of the library image, so every GPU that loads the library holds
// these bytes until the process exits, whether or not the entry point is ever called.
namespace nvfp4 {
namespace {

constexpr int STATIC_MAX_GROUPS = 256;  // non-empty groups per call (256 * 320 B = 80 KB of device memory)
static __device__ __align__(256) unsigned char g_static_table[STATIC_MAX_GROUPS * sizeof(GroupEntry)];

// In host code the array's name is only a handle for the runtime, not a device address: the address the
// kernel needs comes from cudaGetSymbolAddress, asked once per device with that device current.
GroupEntry* g_static_table_addr[64] = {};
std::mutex g_static_mu;
GroupEntry g_static_host[STATIC_MAX_GROUPS];  // host image of the table (plain pageable memory)

}  // namespace

// Status word of a device if an earlier call has already created it, else nullptr (defined in common.cu).
int* status_word_if_allocated(int dev);

}  // namespace nvfp4

extern "C" int nvfp4_grouped_gemm_noalloc(const nvfp4_group_t* groups, int G, float alpha, void* stream) {
    if (!groups) return NVFP4_ERR_NULL;
    if (G <= 0) return NVFP4_ERR_SHAPE;
    bool wide = true;
    int live = 0;
    for (int g = 0; g < G; g++) {
        const nvfp4_group_t& q = groups[g];
        if (q.M < 0 || q.N <= 0 || q.K <= 0) return NVFP4_ERR_SHAPE;
        if (q.K % BK != 0) return NVFP4_ERR_K_MULTIPLE;
        if (q.N % 128 != 0) return NVFP4_ERR_N_MULTIPLE;
        if (q.M == 0) continue;
        const void* ptrs[5] = {q.a, q.b, q.sfa_sw, q.sfb_sw, q.c};
        for (const void* ptr : ptrs) {
            if (!ptr) return NVFP4_ERR_NULL;
            if ((uintptr_t)ptr & 15) return NVFP4_ERR_ALIGN;
        }
        if ((uintptr_t)q.c & 31) return NVFP4_ERR_ALIGN;
        if (q.N % 256 != 0) wide = false;
        live++;
    }
    if (live > STATIC_MAX_GROUPS) return NVFP4_ERR_TOO_MANY_GROUPS;  // the fixed table holds 256 non-empty groups
    if (live == 0) return NVFP4_OK;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 64) return NVFP4_ERR_UNSUPPORTED;
    const int bn = wide ? 256 : 128;

    // Under stream capture the copy below would become a graph node that re-reads the shared host image at every
    // replay, whatever a later call has left there: refuse instead of recording a graph that cannot be trusted.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    e = cudaStreamIsCapturing((cudaStream_t)stream, &cap);
    if (e != cudaSuccess) return (int)e;
    if (cap != cudaStreamCaptureStatusNone) return NVFP4_ERR_UNSUPPORTED;

    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_table_addr[dev]) {
        // first call on this device: resolve the array's device address (do this before any stream capture)
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_table);
        if (e != cudaSuccess) return (int)e;
        g_static_table_addr[dev] = (GroupEntry*)ptr;
    }
    GroupEntry* table = g_static_table_addr[dev];
    int tiles = 0, n = 0;
    for (int g = 0; g < G; g++) {
        const nvfp4_group_t& q = groups[g];
        if (q.M == 0) continue;
        GroupEntry& en = g_static_host[n++];
        int rc = make_operand_tmap(&en.ta, q.a, q.M, q.K, 1, 128);
        if (rc) return rc;
        rc = make_operand_tmap(&en.tb, q.b, q.N, q.K, 1, bn);
        if (rc) return rc;
        en.sfa = (const uint8_t*)q.sfa_sw; en.sfb = (const uint8_t*)q.sfb_sw; en.c = (__half*)q.c;
        en.M = q.M; en.N = q.N; en.K = q.K;
        en.tiles_m = (q.M + BM - 1) / BM; en.tiles_n = q.N / bn;
        en.tile_start = tiles;
        tiles += en.tiles_m * en.tiles_n;
    }
    cudaStream_t st = (cudaStream_t)stream;
    // From pageable memory this copy is staged by the runtime before it returns, so the host image may be
    // rewritten by the next call at once.  Only entries [0, live) are ever read: nothing needs clearing.
    e = cudaMemcpyAsync(table, g_static_host, sizeof(GroupEntry) * live, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return (int)e;
    GemmParams p;
    p.sfa = p.sfb = p.sfb2 = nullptr; p.c = nullptr;
    p.M = p.N = p.K = 0; p.L = 1; p.alpha = alpha;
    p.status = status_word_if_allocated(dev);
    p.budget_ns = wait_budget_ns();
    p.table = table; p.G = live; p.total_tiles = tiles;
    const CUtensorMap& dm = g_static_host[0].ta;
    return wide ? launch_gemm<256, false, true, 4>(dm, dm, dm, p, st)
                : launch_gemm<128, false, true, 6>(dm, dm, dm, p, st);
}
