// NVFP4 GEMM / dual GEMM on CTA PAIRS (cluster of 2, tcgen05 cta_group::2) for sm_100a.
//
// Why: with one CTA per 128 x 256 tile every SM pulls 54 KB per 256-element K step from L2 (A 16 KB, B 32 KB,
// scales 6 KB) and the MMA issuer waits for data a third of the time (measured: 685 cycles per K step against
// 512 cycles of MMA work, i.e. about 79 B/clk per SM).  A pair of CTAs computes a 256 x 256 tile with ONE
// 256 x 256 x 64 MMA per issue: each CTA keeps its own 128 rows of A and only HALF of the B tile (128 rows) in
// shared memory, the tensor cores read the other half from the peer's shared memory.  38 KB per K step and CTA.
//
// Roles are those of the single-CTA kernel (warp 0 producer, warp 1 MMA, warps 2..5 epilogue) with these changes:
//   * both CTAs run a producer for their own tiles with plain TMA loads (no multicast: each CTA fetches what it
//     keeps; the scales of B are needed by both CTAs and are fetched by both).  Every load of either CTA counts its
//     bytes on the LEADER's "full" barrier of the stage (cp.async.bulk.tensor ... .cta_group::2 lets the barrier
//     live in the other CTA of the pair), so one barrier says "both halves have landed" and no thread relays
//     anything.  (A relay by a remote mbarrier.arrive.release.cluster per stage was measured at about 850 cycles
//     per K step, serialised in the relaying thread: the pair ran at 1 350 cycles per K step instead of 512.)
//     The scale atoms therefore come through 2-D tensor maps over the scale buffers (rows of 512 bytes) instead
//     of 1-D bulk copies, which cannot signal a barrier in another CTA;
//   * only the leader CTA (cluster rank 0) issues tcgen05.cp / tcgen05.mma (.cta_group::2);
//   * tcgen05.commit signals the barrier at the same shared-memory offset in both CTAs, which frees the stage for
//     both producers / publishes the accumulator to both epilogues;
//   * both CTAs' epilogue warps drain their own 128 accumulator rows and arrive on the LEADER's "drained" barriers.
// The dual GEMM fits naturally: the leader keeps the B1 tile, the peer the B2 tile, the pair produces 256 x 128
// outputs of silu(A.B1) * (A.B2).
// Every mbarrier wait is bounded; the two hardware cluster barriers (after set-up, before exit) are reached by
// every thread on every path.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_common.cuh"
#include "nvfp4_internal.h"
#include "ptx_sm100.cuh"

namespace nvfp4 {

constexpr int PAIR_STAGES = 5;
constexpr uint32_t PAIR_A_BYTES = 128 * 128;
constexpr uint32_t PAIR_B_BYTES = 128 * 128;       // this CTA's half of the 256-row B tile
constexpr uint32_t PAIR_SFA_BYTES = 4 * 512;
constexpr uint32_t PAIR_SFB_BYTES = 2 * 4 * 512;   // scales of all 256 B rows
constexpr uint32_t PAIR_STAGE_BYTES = PAIR_A_BYTES + PAIR_B_BYTES + PAIR_SFA_BYTES + PAIR_SFB_BYTES;
constexpr size_t PAIR_SMEM = PAIR_STAGES * PAIR_STAGE_BYTES + 1024;

// Pair tile t -> batch, 256-row tile, column tile; same banded order as the single-CTA kernel.
// GEMM: column tile = 256 output columns.  DUAL: 128 output columns.
template <bool DUAL>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_b2, const __grid_constant__ CUtensorMap tmap_sfa,
                 const __grid_constant__ CUtensorMap tmap_sfb, const __grid_constant__ CUtensorMap tmap_sfb2,
                 const GemmParams p) {
    constexpr int BN = DUAL ? 128 : 256;                 // output columns of the pair tile
    constexpr uint32_t SF_COLS = 16 + 32;                // TMEM columns of one stage's scales (A 16, B 32)
    constexpr uint32_t SF_BASE = TMEM_COLS - 2 * SF_COLS;
    constexpr uint32_t ACC1_OFF = SF_BASE - 256;         // second accumulator overlaps the first by 96 columns
    constexpr uint32_t OVERLAP = 256 - ACC1_OFF;
    constexpr int OV_CHUNKS = OVERLAP / 32;
    constexpr int STAGES = PAIR_STAGES;

    extern __shared__ uint8_t smem_raw[];
    // same layout in both CTAs (remote arrivals and pair-wide commits address barriers by offset)
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 5];
    __shared__ uint32_t tmem_base_slot;

    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();             // 0 = leader
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t acc_full0 = smem_u32(&bars[2 * STAGES]);           // [2], signalled in both CTAs
    const uint32_t acc_empty0 = acc_full0 + 16;                       // [2], leader's copy used, 8 arrivals
    const uint32_t ovl_free = acc_full0 + 32;                         // leader's copy used, 8 arrivals

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);      // the leader's copy is the one used: one arrival + both CTAs' bytes
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, 8);   // four epilogue warps of each CTA
        }
        mbar_init(ovl_free, 8);
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
        prefetch_tmap(&tmap_sfa);
        prefetch_tmap(&tmap_sfb);
        if (DUAL) {
            prefetch_tmap(&tmap_b2);
            prefetch_tmap(&tmap_sfb2);
        }
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(&tmem_base_slot), TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();   // the peer's barriers exist before anything is sent to them
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    const int tiles_m = (p.M + 255) / 256, tiles_n = p.N / BN;
    const int total_tiles = tiles_m * tiles_n * p.L;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int kiters = p.K / BK;
    const int RA = (p.M + 127) / 128, RB = p.N / 128;
    const int atoms_per_block = p.K / 64;                // scale atoms (512 bytes) of one 128-row block

    if (warp == 0) {
        // ------------------------------------------------------------------ producer (both CTAs, own tiles)
        if (elect_one()) {
            uint32_t it = 0;
            bool alive = true;
            const uint32_t leader_full0 = mapa_shared(full0, 0);
            for (int t = pair; alive && t < total_tiles; t += npairs) {
                const TileCoord tc = tile_coord(t, tiles_m, tiles_n);
                const int m0 = tc.mt * 256 + (int)rank * 128;     // this CTA's A rows
                const int n0 = tc.nt * BN;
                const bool a_rows_exist = m0 < p.M;
                const bool peer_rows_exist = tc.mt * 256 + 128 < p.M;
                const int atom_a = (tc.l * RA + (m0 >> 7)) * atoms_per_block;
                const int atom_b = (tc.l * RB + n0 / 128) * atoms_per_block;
                for (int kit = 0; kit < kiters; kit++, it++) {
                    const int slot = it % STAGES;
                    if (!mbar_wait_cluster(empty0 + 8 * slot, ((it / STAGES) & 1) ^ 1, p.budget_ns)) {
                        report_status(p.status, DEV_TIMEOUT_PRODUCER);
                        alive = false;
                        break;
                    }
                    const uint32_t full = leader_full0 + 8 * slot;
                    const uint32_t sA = smem0 + slot * PAIR_STAGE_BYTES;
                    const uint32_t sB = sA + PAIR_A_BYTES;
                    const uint32_t sSFA = sB + PAIR_B_BYTES;
                    const uint32_t sSFB = sSFA + PAIR_SFA_BYTES;
                    const int k0 = kit * BK;
                    const int ka = k0 / 64;
                    // the leader announces the bytes of BOTH CTAs.  Rows of A beyond M (second CTA of the last row
                    // tile) read as zeros; their scale block does not exist and is not fetched
                    if (rank == 0)
                        mbar_arrive_expect_tx(full0 + 8 * slot, 2u * (PAIR_A_BYTES + PAIR_B_BYTES + PAIR_SFB_BYTES) +
                                                                    PAIR_SFA_BYTES + (peer_rows_exist ? PAIR_SFA_BYTES : 0u));
                    tma_load_3d_pair(sA, &tmap_a, k0, m0, tc.l, full);
                    if (a_rows_exist) tma_load_2d_pair(sSFA, &tmap_sfa, 0, atom_a + ka, full);
                    if (DUAL) {
                        // leader keeps the B1 tile, peer the B2 tile; both need both scale blocks
                        tma_load_3d_pair(sB, rank == 0 ? &tmap_b : &tmap_b2, k0, n0, tc.l, full);
                        tma_load_2d_pair(sSFB, &tmap_sfb, 0, atom_b + ka, full);
                        tma_load_2d_pair(sSFB + 2048u, &tmap_sfb2, 0, atom_b + ka, full);
                    } else {
                        tma_load_3d_pair(sB, &tmap_b, k0, n0 + (int)rank * 128, tc.l, full);
                        tma_load_2d_pair(sSFB, &tmap_sfb, 0, atom_b + ka, full);
                        tma_load_2d_pair(sSFB + 2048u, &tmap_sfb, 0, atom_b + atoms_per_block + ka, full);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            if (rank == 0) {
                // -------------------------------------------------------------- leader: MMA issuer for the pair
                constexpr uint32_t idesc = make_idesc_nvfp4(256, 256);
                uint32_t it = 0, tile_it = 0;
                bool alive = true;
#ifdef NVFP4_PROFILE
                long long prof_acc = 0, prof_full = 0;
                const long long prof_begin = clock64();
#endif
                for (int t = pair; alive && t < total_tiles; t += npairs, tile_it++) {
                    const uint32_t buf = tile_it & 1;
                    bool ok;
                    {
                        PROF_T0();
                        ok = mbar_wait_cluster(acc_empty0 + 8 * buf, ((tile_it >> 1) & 1) ^ 1, p.budget_ns);
                        if (ok && tile_it > 0) ok = mbar_wait_cluster(ovl_free, (tile_it - 1) & 1, p.budget_ns);
                        PROF_ADD(prof_acc);
                    }
                    if (!ok) {
                        report_status(p.status, DEV_TIMEOUT_MMA_ACC);
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t t_acc = tmem_base + buf * ACC1_OFF;
                    for (int kit = 0; kit < kiters; kit++, it++) {
                        const int slot = it % STAGES;
                        const uint32_t par = (it / STAGES) & 1;
                        bool got;
                        {
                            PROF_T0();
                            got = mbar_wait_cluster(full0 + 8 * slot, par, p.budget_ns);   // both CTAs' bytes
                            PROF_ADD(prof_full);
                        }
                        if (!got) {
                            report_status(p.status, DEV_TIMEOUT_CONSUMER);
                            alive = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t sA = smem0 + slot * PAIR_STAGE_BYTES;
                        const uint32_t sB = sA + PAIR_A_BYTES;
                        const uint32_t sSFA = sB + PAIR_B_BYTES;
                        const uint32_t sSFB = sSFA + PAIR_SFA_BYTES;
                        const uint32_t t_sfa = tmem_base + SF_BASE + (it & 1) * SF_COLS;
                        const uint32_t t_sfb = t_sfa + 16;
#pragma unroll
                        for (int ks = 0; ks < 4; ks++) {
                            tc_cp_sf_atom_pair(t_sfa + 4 * ks, make_desc_sf(sSFA + 512 * ks));
                            tc_cp_sf_atom_pair(t_sfb + 8 * ks, make_desc_sf(sSFB + 512 * ks));
                            tc_cp_sf_atom_pair(t_sfb + 8 * ks + 4, make_desc_sf(sSFB + 2048 + 512 * ks));
                        }
#pragma unroll
                        for (int ks = 0; ks < 4; ks++)
                            tc_mma_nvfp4_pair(t_acc, make_desc_k_sw128(sA + 32 * ks), make_desc_k_sw128(sB + 32 * ks),
                                              idesc, t_sfa + 4 * ks, t_sfb + 8 * ks, (kit | ks) != 0 ? 1u : 0u);
                        tc_commit_pair(empty0 + 8 * slot, 3);     // frees the stage in both CTAs
                    }
                    if (alive) tc_commit_pair(acc_full0 + 8 * buf, 3);  // accumulators complete in both CTAs
                }
#ifdef NVFP4_PROFILE
                if (p.prof) {
                    p.prof[8 * blockIdx.x + 0] = prof_acc;
                    p.prof[8 * blockIdx.x + 1] = prof_full;
                    p.prof[8 * blockIdx.x + 2] = clock64() - prof_begin;
                    p.prof[8 * blockIdx.x + 6] = it;
                }
#endif
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps 2..5 (both CTAs)
        const int q = warp & 3;
        const uint32_t l_acc_empty0 = mapa_shared(acc_empty0, 0), l_ovl_free = mapa_shared(ovl_free, 0);
        uint32_t tile_it = 0;
        for (int t = pair; t < total_tiles; t += npairs, tile_it++) {
            const TileCoord tc = tile_coord(t, tiles_m, tiles_n);
            const int row = tc.mt * 256 + (int)rank * 128 + q * 32 + lane;
            const int n0 = tc.nt * BN;
            const uint32_t buf = tile_it & 1;
            if (!mbar_wait(acc_full0 + 8 * buf, (tile_it >> 1) & 1, p.budget_ns)) {
                if (lane == 0) report_status(p.status, DEV_TIMEOUT_EPILOGUE);
                break;
            }
            tc_fence_after_sync();
            const uint32_t t_lane = tmem_base + buf * ACC1_OFF + ((uint32_t)(q * 32) << 16);
            __half* crow = p.c + ((size_t)tc.l * p.M + (size_t)(row < p.M ? row : 0)) * p.N + n0;
            // the shared columns are released through the leader's barrier by a cluster-scope arrive
            if (buf == 0)
                epilogue_tile<BN, DUAL, int(ACC1_OFF) / 32, OV_CHUNKS, true>(t_lane, crow, row < p.M, n0, p.N, p.alpha,
                                                                            l_ovl_free, lane);
            else
                epilogue_tile<BN, DUAL, 0, OV_CHUNKS, true>(t_lane, crow, row < p.M, n0, p.N, p.alpha, l_ovl_free, lane);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster_relaxed(l_acc_empty0 + 8 * buf);   // accumulator read out (see ovl_free)
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();   // neither CTA frees tensor memory or exits while the other may still touch it
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------ host side
namespace {

template <bool DUAL>
int configure(int dev) {
    static bool done[64] = {};
    if (done[dev]) return NVFP4_OK;
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)PAIR_SMEM);
    if (e != cudaSuccess) return (int)e;
    done[dev] = true;
    return NVFP4_OK;
}

template <bool DUAL>
int max_pairs(int dev) {
    static int cached[64] = {};
    if (cached[dev]) return cached[dev];
    // the occupancy query fails for more dynamic shared memory than the kernel has been allowed so far
    if (configure<DUAL>(dev) != NVFP4_OK) return -1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * sm_count(dev));
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = PAIR_SMEM;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<DUAL>, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = 0;
    }
    cached[dev] = n > 0 ? n : -1;
    return cached[dev];
}

template <bool DUAL>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const GemmParams& p,
           cudaStream_t stream) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 64) return NVFP4_ERR_UNSUPPORTED;
    int rc = configure<DUAL>(dev);
    if (rc) return rc;
    const int pairs_max = max_pairs<DUAL>(dev);
    if (pairs_max <= 0) return NVFP4_ERR_UNSUPPORTED;
    const int tiles = ((p.M + 255) / 256) * (p.N / (DUAL ? 128 : 256)) * p.L;
    if (tiles <= 0) return NVFP4_OK;
    const int pairs = tiles < pairs_max ? tiles : pairs_max;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = PAIR_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const long ka = p.K / 64;
    CUtensorMap tsa, tsb, tsb2;
    rc = make_scale_tmap(&tsa, p.sfa, (long)p.L * ((p.M + 127) / 128) * ka);
    if (rc) return rc;
    rc = make_scale_tmap(&tsb, p.sfb, (long)p.L * (p.N / 128) * ka);
    if (rc) return rc;
    tsb2 = tsb;
    if (DUAL) {
        rc = make_scale_tmap(&tsb2, p.sfb2, (long)p.L * (p.N / 128) * ka);
        if (rc) return rc;
    }
    e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<DUAL>, ta, tb, tb2, tsa, tsb, tsb2, p);
    return e == cudaSuccess ? NVFP4_OK : (int)e;
}

}  // namespace

bool pair_kernel_suits(int M, int N, int K, int L, bool dual, int dev) {
    if (M < 256 || N % (dual ? 128 : 256) != 0 || dev >= 64) return false;
    const int pairs = dual ? max_pairs<true>(dev) : max_pairs<false>(dev);
    if (pairs <= 0) return false;
    const long tiles = (long)((M + 255) / 256) * (N / (dual ? 128 : 256)) * L;
    // rows of the last 256-row tile that do not exist are wasted work for one CTA of the pair
    const bool ragged_waste = (M % 256 != 0) && (M < 2048);
    return tiles >= pairs && !ragged_waste;
}

int launch_gemm_pair(bool dual, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const GemmParams& p,
                     cudaStream_t stream) {
    return dual ? launch<true>(ta, tb, tb2, p, stream) : launch<false>(ta, tb, tb2, p, stream);
}

}  // namespace nvfp4
