// NVFP4 block-scaled GEMV for sm_100a as a pure HBM stream: TMA -> shared memory -> tcgen05.mma, no decode
// on the CUDA cores.
//
//   c[m, 0, l] = fp16( alpha * sum_kb sfa[m,kb,l] * sfx[kb,l] * sum_{j<16} a[m,16kb+j,l] * x[16kb+j,l] )
//
// Replaces the reference's GEMV entry, which pads the vector to 128 columns and runs a whole tensor-core GEMM
// through torch._scaled_mm (eval/nvfp4_gemv/submission.py:28-54).
//
// The decode-on-CUDA-cores kernel (gemv_sm100.cu) is bound by instruction issue: about 1.2 instructions per
// element to turn e2m1 nibbles into int8 and feed dp4a.  The block-scaled tensor-core instruction takes the
// packed nibbles and the e4m3 scales as they lie in memory, so here the SM only moves bytes:
//   * a 128-row block of A is the M side of a 128 x 16 x 64 MMA (kind::mxf4nvf4.block_scale.block16); the
//     vector is row 0 of the 16-row N side (rows 1..15 hold whatever shared memory held - every bit pattern
//     is a finite e2m1 value - and their result columns are never read);
//   * a stage is 512 K-elements: the A tile (32 KB: one 5-D TMA box with the 128-byte swizzle when M % 8 == 0 and
//     K % 256 == 0, else one 128-row box per 256 elements; rows past M and K past the end read as zero), 128 bytes
//     of the vector per 256 elements, and the scale atoms of A and of the vector (512 bytes per 64 K-elements
//     each, contiguous in the swizzled global layout); a ring of 5 stages (220 KB) keeps about 145 KB of HBM
//     reads in flight per SM;
//   * the MMA thread copies the atoms into tensor memory (tcgen05.cp) and issues the MMAs; tcgen05.commit frees
//     the stage; four epilogue warps read column 0 of the accumulator (tcgen05.ld), scale and store fp16.
// Work distribution: a tile is 128 rows over all of K.  The grid has one thread-block cluster per tile; the
// clusters that get SMs keep them and take over the tiles of clusters that have not started, one at a time, with
// cluster launch control (clusterlaunchcontrol.try_cancel): SMs that stream faster run more tiles, nothing is
// kept in global memory between launches.  The S CTAs of a cluster (S = 1 or 2) share a tile by splitting K
// and add their partial sums through distributed shared memory.  To keep the result independent of S, K is always
// cut into the same V segments (V = 8 when K has at least 8 stages), every segment is accumulated in its own
// tensor-memory columns, and the V partial sums are added in segment order whichever CTA produced them: a row's
// bits depend on K only, not on M, L or the cluster size.  No global scratch, no atomics.
// Every mbarrier wait is bounded; on expiry the role records a status code and leaves its loop; every thread
// reaches the closing barriers and the CTA frees its tensor memory.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "gemm_common.cuh"
#include "nvfp4_internal.h"
#include "ptx_sm100.cuh"

namespace nvfp4 {

struct GemvTcParams {
    const uint8_t* sfa;   // swizzled scales of A [L][ceil(M/128)][K/64][512]
    const uint8_t* sfx;   // swizzled scales of the vector tensor [L][ceil(x_rows/128)][K/64][512]
    __half* c;            // [L][M]
    int M, K, L;
    int row_blocks;       // ceil(M/128)
    int x_row_blocks;     // ceil(x_rows/128)
    int tiles;            // L * row_blocks
    int a_boxes;          // 1: one 4-D box per stage (rows of 8 x chunk x row groups); GT_KCH: one 3-D box per chunk
    int V;                // K segments (power of two, 1..8, at most K/256 rounded up)
    float alpha;
    int* status;
    unsigned long long budget_ns;
#ifdef NVFP4_PROFILE
    unsigned long long* prof = nullptr;  // per CTA: producer wait / MMA wait-for-data / MMA issue / MMA total cycles
#endif
};

constexpr int GT_N = 16;                       // MMA N: the vector and 15 rows that are never looked at
constexpr int GT_KCH = 2;                      // 256-element K chunks per stage
constexpr int GT_STAGES = 5;
constexpr int GT_THREADS = 192;
constexpr int GT_VMAX = 8;
constexpr int GT_Q = 16;                       // slots of the tile queue
constexpr uint32_t GT_A_BYTES = GT_KCH * 128 * 128;   // 128 rows x 256 e2m1 per chunk
constexpr uint32_t GT_X_BYTES = GT_KCH * GT_N * 128;
constexpr uint32_t GT_SF_BYTES = GT_KCH * 4 * 512;    // 4 atoms per chunk
constexpr int GT_BK = GT_KCH * BK;                    // K elements per stage
constexpr uint32_t GT_STAGE_BYTES = GT_A_BYTES + GT_X_BYTES + 2 * GT_SF_BYTES;
constexpr size_t GT_SMEM = (size_t)GT_STAGES * GT_STAGE_BYTES + 1024;
static_assert(GT_STAGE_BYTES % 1024 == 0, "stage alignment");
static_assert(GT_SMEM + 4096 + 512 <= 227 * 1024, "shared memory");

// First stage of K segment v when `stages` stages are cut into V segments.
__host__ __device__ __forceinline__ int seg_start(int v, int stages, int V) {
    const int base = stages / V, rem = stages % V;
    return v * base + (v < rem ? v : rem);
}

__device__ __forceinline__ float ld_cluster_f32(uint32_t cluster_addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
    return v;
}

template <int S>
__global__ void __launch_bounds__(GT_THREADS, 1)
gemv_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_x,
               const GemvTcParams p) {
    constexpr int STAGES = GT_STAGES;
    constexpr int Q = GT_Q;
    constexpr uint32_t TCOLS = 512;
    constexpr uint32_t ACC_STRIDE = GT_VMAX * GT_N;    // columns of one accumulator buffer (one 16-column group per segment)
    constexpr uint32_t SF_BASE = 2 * ACC_STRIDE;       // two alternating scale regions follow
    constexpr uint32_t SF_COLS = 16 * GT_KCH;          // columns of one stage's scale atoms of one operand
    static_assert(SF_BASE + 4 * SF_COLS <= TCOLS, "tensor memory");
    constexpr int JMAX = GT_VMAX / S;                  // segments one CTA can hold
    constexpr int RED_J = S > 1 ? JMAX : 1;            // (no exchange when the cluster is one CTA)
    static_assert(S == 1 || S == 2, "cluster size");

#ifdef NVFP4_PROFILE
    const unsigned long long prof_t_entry = globaltimer_ns();
#endif
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(16) uint8_t clc_resp[2][16];  // answers of the cluster-launch-control requests (rank 0)
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 6 + 2 * Q + 2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int tileq[Q];                           // tile indices in the order this cluster runs them; -1 ends
    __shared__ __align__(16) float red[2][RED_J][128]; // partial sums by tile parity, segment, row

    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = S > 1 ? cluster_ctarank() : 0u;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t acc_full0 = smem_u32(&bars[2 * STAGES]);
    const uint32_t acc_empty0 = acc_full0 + 16;
    const uint32_t red_ready0 = acc_full0 + 32;        // [2] by tile parity: 4 epilogue warps of each of the S CTAs
    const uint32_t q_full0 = acc_full0 + 48;           // [Q] slot written (one arrival, by the scheduler)
    const uint32_t q_empty0 = q_full0 + 8 * Q;         // [Q] rank 0 only: slot read by every consumer of the cluster
    const uint32_t clc_bar0 = q_empty0 + 8 * Q;        // [2] rank 0 only: answer landed

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, 4);
            mbar_init(red_ready0 + 8 * b, 4 * S);
            mbar_init(clc_bar0 + 8 * b, 1);
        }
        for (int s = 0; s < Q; s++) {
            mbar_init(q_full0 + 8 * s, 1);
            mbar_init(q_empty0 + 8 * s, 6 * S - 1);   // producer thread, MMA thread, 4 epilogue warps per CTA, less the scheduler
        }
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_x);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), TCOLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();              // every CTA's barriers exist before a peer arrives on them
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    // K range of this CTA: segments [rank*VS, (rank+1)*VS) of the V the whole K loop is cut into
    const int stages_all = (p.K + GT_BK - 1) / GT_BK;
    const int atoms_all = p.K / 64;
    const int V = p.V, VS = V / S;
    const int kfirst = seg_start((int)rank * VS, stages_all, V);
    const int kend = seg_start((int)rank * VS + VS, stages_all, V);
    const size_t sf_row_block = (size_t)atoms_all * 512;

    // Tile queue.  A consumer reads entry n (-1: no more tiles, -2: the wait ran out) ...
    auto pop = [&](uint32_t n) -> int {
        const uint32_t slot = n % Q;
        if (!mbar_wait_cluster(q_full0 + 8 * slot, (n / Q) & 1, p.budget_ns)) return -2;
        return reinterpret_cast<volatile int*>(tileq)[slot];
    };
    // ... and then tells the scheduler (rank 0) that it is done with the slot.
    auto release = [&](uint32_t n) { mbar_arrive_cluster(mapa_shared(q_empty0 + 8 * (n % Q), 0u)); };

    if (warp == 0) {
        // ------------------------------------------------------------------ producer (one lane); on rank 0 also the scheduler
        if (elect_one()) {
            uint32_t it = 0;
#ifdef NVFP4_PROFILE
            long long prof_wait = 0;
            const long long prof_begin = clock64();
#endif
            auto load_tile = [&](int t) -> bool {
                const int l = t / p.row_blocks, m0 = (t - l * p.row_blocks) * BM;
                const uint8_t* sfa_t = p.sfa + (size_t)t * sf_row_block;
                const uint8_t* sfx_t = p.sfx + (size_t)l * p.x_row_blocks * sf_row_block;
                for (int ks = kfirst; ks < kend; ks++, it++) {
                    const int slot = it % STAGES;
                    bool got;
                    {
                        PROF_T0();
                        got = mbar_wait(empty0 + 8 * slot, ((it / STAGES) & 1) ^ 1, p.budget_ns);
                        PROF_ADD(prof_wait);
                    }
                    if (!got) {
                        report_status(p.status, DEV_TIMEOUT_PRODUCER);
                        return false;
                    }
                    const uint32_t full = full0 + 8 * slot;
                    const uint32_t sA = smem0 + slot * GT_STAGE_BYTES, sX = sA + GT_A_BYTES;
                    const uint32_t sSFA = sX + GT_X_BYTES, sSFX = sSFA + GT_SF_BYTES;
                    const int nat = min(4 * GT_KCH, atoms_all - ks * 4 * GT_KCH);   // 64-element groups of this stage inside K
                    // (chunks past the end of K read as zero and still count their bytes)
                    mbar_arrive_expect_tx(full, GT_A_BYTES + GT_KCH * 128u + (uint32_t)nat * 1024u);
                    if (p.a_boxes == 1) {
                        tma_load_5d(sA, &tmap_a, 0, 0, ks * GT_KCH, m0 / 8, l, full);
                    } else {
#pragma unroll
                        for (int c = 0; c < GT_KCH; c++)
                            tma_load_3d(sA + c * 16384u, &tmap_a, (ks * GT_KCH + c) * BK, m0, l, full);
                    }
#pragma unroll
                    for (int c = 0; c < GT_KCH; c++)
                        tma_load_3d(sX + c * (GT_N * 128u), &tmap_x, (ks * GT_KCH + c) * BK, 0, l, full);
                    bulk_g2s(sSFA, sfa_t + (size_t)ks * GT_SF_BYTES, (uint32_t)nat * 512u, full);
                    bulk_g2s(sSFX, sfx_t + (size_t)ks * GT_SF_BYTES, (uint32_t)nat * 512u, full);
                }
                return true;
            };
            if (rank == 0) {
                // Scheduler: this cluster's own tile first; while a tile's loads are issued the hardware is asked
                // to cancel one more cluster of the grid that has not started, whose tile this cluster then runs.
                auto publish = [&](uint32_t n, int t) {
#pragma unroll
                    for (int c = 0; c < S; c++) {
                        st_cluster_u32(mapa_shared(smem_u32(&tileq[n % Q]), (uint32_t)c), (uint32_t)t);
                        mbar_arrive_cluster(mapa_shared(q_full0 + 8 * (n % Q), (uint32_t)c));
                    }
                };
                int tile = (int)(blockIdx.x / S);
                uint32_t n = 0;
                publish(0, tile);
                while (true) {
                    const uint32_t cb = clc_bar0 + 8 * (n & 1), cr = smem_u32(&clc_resp[n & 1][0]);
                    mbar_arrive_expect_tx(cb, 16u);
                    clc_try_cancel(cr, cb);
                    const bool loaded = load_tile(tile);
                    // (the answer is awaited even when the loads gave up: nothing may land in a CTA that has left)
                    if (!mbar_wait(cb, (n >> 1) & 1, p.budget_ns)) {
                        report_status(p.status, DEV_TIMEOUT_PRODUCER);
                        break;
                    }
                    uint32_t first = 0;
                    int next = -1;
                    if (clc_query(cr, &first)) {
                        next = (int)(first / S);
                        if (next >= p.tiles) next = -1;   // cannot happen: the grid has exactly tiles * S CTAs
                    }
                    fence_proxy_async_smem();             // the answer is read before a later request may overwrite it
                    if (!loaded) break;
                    n++;
                    if (n >= (uint32_t)Q && !mbar_wait_cluster(q_empty0 + 8 * (n % Q), ((n / Q) - 1) & 1, p.budget_ns)) {
                        report_status(p.status, DEV_TIMEOUT_PRODUCER);
                        break;
                    }
                    publish(n, next);
                    if (next < 0) break;                  // after a failed request no further request is allowed
                    tile = next;
                }
            } else {
                for (uint32_t n = 0;; n++) {
                    const int t = pop(n);
                    if (t == -2) report_status(p.status, DEV_TIMEOUT_PRODUCER);
                    if (t < 0) break;
                    release(n);
                    if (!load_tile(t)) break;
                }
            }
#ifdef NVFP4_PROFILE
            if (p.prof) {
                p.prof[10 * blockIdx.x + 0] = prof_wait;
                p.prof[10 * blockIdx.x + 1] = clock64() - prof_begin;
            }
#endif
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (one lane)
        if (elect_one()) {
            constexpr uint32_t idesc = make_idesc_nvfp4(BM, GT_N);
            // A tile in shared memory: one 4-D box leaves the chunks of an 8-row group side by side (groups
            // GT_KCH KB apart), one box per chunk leaves whole 16 KB chunk tiles (groups 1 KB apart)
            const uint32_t a_chunk = p.a_boxes == 1 ? 1024u : 16384u;
            const uint32_t a_sbo = p.a_boxes == 1 ? GT_KCH * 1024u : 1024u;
            uint32_t it = 0;
            bool alive = true;
#ifdef NVFP4_PROFILE
            long long prof_full = 0, prof_issue = 0;
            const long long prof_begin = clock64();
#endif
            for (uint32_t tile_it = 0; alive; tile_it++) {
                const int t = pop(tile_it);
                if (t == -2) report_status(p.status, DEV_TIMEOUT_CONSUMER);
                if (t < 0) break;
                release(tile_it);
                const uint32_t buf = tile_it & 1;
                if (!mbar_wait(acc_empty0 + 8 * buf, ((tile_it >> 1) & 1) ^ 1, p.budget_ns)) {
                    report_status(p.status, DEV_TIMEOUT_MMA_ACC);
                    break;
                }
                tc_fence_after_sync();
                for (int j = 0; alive && j < VS; j++) {
                    const uint32_t t_acc = tmem_base + buf * ACC_STRIDE + (uint32_t)j * GT_N;
                    const int s0 = seg_start((int)rank * VS + j, stages_all, V);
                    const int s1 = seg_start((int)rank * VS + j + 1, stages_all, V);
                    for (int ks = s0; ks < s1; ks++, it++) {
                        const int slot = it % STAGES;
                        bool got;
                        {
                            PROF_T0();
                            got = mbar_wait(full0 + 8 * slot, (it / STAGES) & 1, p.budget_ns);
                            PROF_ADD(prof_full);
                        }
                        PROF_T0();
                        if (!got) {
                            report_status(p.status, DEV_TIMEOUT_CONSUMER);
                            alive = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t sA = smem0 + slot * GT_STAGE_BYTES, sX = sA + GT_A_BYTES;
                        const uint32_t sSFA = sX + GT_X_BYTES, sSFX = sSFA + GT_SF_BYTES;
                        const uint32_t t_sfa = tmem_base + SF_BASE + (it & 1) * (2 * SF_COLS), t_sfx = t_sfa + SF_COLS;
                        const int nat = min(4 * GT_KCH, atoms_all - ks * 4 * GT_KCH);
#pragma unroll
                        for (int a = 0; a < 4 * GT_KCH; a++) {
                            if (a < nat) {
                                tc_cp_sf_atom(t_sfa + 4 * a, make_desc_sf(sSFA + 512 * a));
                                tc_cp_sf_atom(t_sfx + 4 * a, make_desc_sf(sSFX + 512 * a));
                            }
                        }
#pragma unroll
                        for (int a = 0; a < 4 * GT_KCH; a++) {
                            if (a < nat) {
                                const int c = a >> 2, k4 = a & 3;   // chunk of the stage, 64-element step inside the chunk
                                tc_mma_nvfp4(t_acc, make_desc_k_sw128_sbo(sA + c * a_chunk + 32 * k4, a_sbo),
                                             make_desc_k_sw128(sX + c * (GT_N * 128u) + 32 * k4), idesc, t_sfa + 4 * a,
                                             t_sfx + 4 * a, (ks != s0 || a != 0) ? 1u : 0u);
                            }
                        }
                        tc_commit(empty0 + 8 * slot);
                        PROF_ADD(prof_issue);
                    }
                }
                if (alive) tc_commit(acc_full0 + 8 * buf);
            }
#ifdef NVFP4_PROFILE
            if (p.prof) {
                p.prof[10 * blockIdx.x + 2] = prof_full;
                p.prof[10 * blockIdx.x + 3] = prof_issue;
                p.prof[10 * blockIdx.x + 4] = clock64() - prof_begin;
                p.prof[10 * blockIdx.x + 9] = it;   // stages this CTA ran
            }
#endif
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps 2..5
        const int q = warp & 3;                       // TMEM lane quadrant this warp may access
        const int row_in_tile = q * 32 + lane;
        for (uint32_t tile_it = 0;; tile_it++) {
            const int t = pop(tile_it);
            if (t == -2 && lane == 0) report_status(p.status, DEV_TIMEOUT_EPILOGUE);
            if (t < 0) break;
            __syncwarp();                             // every lane has read the slot before it is handed back
            if (lane == 0) release(tile_it);
            const int l = t / p.row_blocks, m0 = (t - l * p.row_blocks) * BM;
            const uint32_t buf = tile_it & 1;
            const uint32_t par = (tile_it >> 1) & 1;
            bool ok = mbar_wait(acc_full0 + 8 * buf, par, p.budget_ns);
            if (!ok && lane == 0) report_status(p.status, DEV_TIMEOUT_EPILOGUE);
            float part[JMAX];
#pragma unroll
            for (int j = 0; j < JMAX; j++) part[j] = 0.f;
            if (ok) {
                tc_fence_after_sync();
                const uint32_t t_lane = tmem_base + buf * ACC_STRIDE + ((uint32_t)(q * 32) << 16);
#pragma unroll
                for (int j = 0; j < JMAX; j++)
                    if (j < VS) part[j] = __uint_as_float(tc_ld_32x1(t_lane + (uint32_t)j * GT_N));
                tc_wait_ld();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
            }
            const int row = m0 + row_in_tile;
            if (S == 1) {
                if (!ok) break;
                float sum = part[0];
#pragma unroll
                for (int j = 1; j < JMAX; j++)
                    if (j < VS) sum += part[j];
                if (row < p.M) p.c[(size_t)l * p.M + row] = __float2half_rn(p.alpha * sum);
            } else {
#pragma unroll
                for (int j = 0; j < RED_J; j++)
                    if (j < VS) red[buf][j][row_in_tile] = part[j];
                // tell every CTA of the cluster (this one included) that this warp's rows are written; a warp whose
                // accumulator never completed still arrives, so that no peer waits for it in vain
                __syncwarp();
                // (one lane per CTA: a thread's release-arrives on remote barriers queue up behind one another)
                if (lane < S) mbar_arrive_cluster(mapa_shared(red_ready0 + 8 * buf, (uint32_t)lane));
                if (!ok) break;
                if (!mbar_wait_cluster(red_ready0 + 8 * buf, par, p.budget_ns)) {
                    if (lane == 0) report_status(p.status, DEV_TIMEOUT_EPILOGUE);
                    break;
                }
                // CTA r finishes rows [r*128/S, (r+1)*128/S): segments in order, whichever CTA holds them
                if (row_in_tile / (128 / S) == (int)rank) {
                    float sum = 0.f;
                    bool first = true;
#pragma unroll
                    for (int c = 0; c < S; c++) {
                        for (int j = 0; j < VS; j++) {
                            const float v = ld_cluster_f32(mapa_shared(smem_u32(&red[buf][j][row_in_tile]), (uint32_t)c));
                            sum = first ? v : sum + v;
                            first = false;
                        }
                    }
                    if (row < p.M) p.c[(size_t)l * p.M + row] = __float2half_rn(p.alpha * sum);
                }
            }
        }
    }

#ifdef NVFP4_PROFILE
    if (p.prof && threadIdx.x == GT_THREADS - 1) {   // an epilogue thread: the last role to finish
        p.prof[10 * blockIdx.x + 5] = prof_t_entry;
        p.prof[10 * blockIdx.x + 7] = globaltimer_ns();
    }
#endif
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();              // no CTA exits while a peer may still read its partial sums or write its queue
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TCOLS);
    }
}

// ------------------------------------------------------------------------------------------ host side
namespace {

template <int S>
int launch_tc(const CUtensorMap& ta, const CUtensorMap& tx, const GemvTcParams& p, int dev, cudaStream_t stream) {
    static bool configured[64] = {};
    auto kern = gemv_tc_kernel<S>;
    cudaError_t e;
    if (!configured[dev]) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GT_SMEM);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }
    // one cluster per tile: the clusters that get an SM keep it and take over the tiles of those still waiting
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.tiles * S);
    cfg.blockDim = dim3(GT_THREADS);
    cfg.dynamicSmemBytes = GT_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = S; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kern, ta, tx, p);
    return e == cudaSuccess ? NVFP4_OK : (int)e;
}

}  // namespace

// Tensor map of A for the one-box-per-stage layout (cached like the operand maps: encoding costs about a microsecond).
static int make_gemv_a_tmap(CUtensorMap* map, const void* base, int M, int K, int L) {
    thread_local TmapCache<> cache = {};
    const TmapKey key{(uint64_t)(uintptr_t)base, M, K, L, 0};
    if (cache.find(key, map)) return NVFP4_OK;
    const uint64_t rowb = (uint64_t)(K / 2);
    const uint64_t dims[5] = {256, 8, (uint64_t)(K / BK), (uint64_t)(M / 8), (uint64_t)L};
    const uint64_t strides[4] = {rowb, 128, 8 * rowb, (uint64_t)M * rowb};
    const uint32_t box[5] = {256, 8, (uint32_t)GT_KCH, 16, 1};
    int rc = encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN8B, 5, base, dims, strides, box,
                          CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    cache.put(key, *map);
    return NVFP4_OK;
}

// Cluster size for a shape.  Measured on B200 (clusters of 4 and 8 CTAs fit only 132 and 120 of the 148 SMs and were
// slower on every shape tried, so they are not built): pairs win when the tiles do not divide well over the SMs
// (M = K = 16384, L = 4: 512 tiles, 96 us against 104 us) or are fewer than the SMs; single CTAs win by a few
// percent otherwise (one reduction step less per tile).  Score = share of SM time spent streaming, counting half
// of the idle tail of the last round (tiles are handed out one at a time), pairs marked down by 3 %.
// NVFP4_GEMV_SPLIT = 1 or 2 forces a size (read on every call: tests compare the two in one process).
static int pick_cluster(int tiles, int V, int dev) {
    const char* e_ = getenv("NVFP4_GEMV_SPLIT");
    const int forced = e_ ? atoi(e_) : 0;
    if ((forced == 1 || forced == 2) && forced <= V) return forced;
    if (V < 2) return 1;
    const int sms = sm_count(dev);
    double eff[2];
    for (int i = 0; i < 2; i++) {
        const int s = i + 1;
        const int cap = sms / s;
        const int clusters = tiles < cap ? tiles : cap;
        const double rounds = (double)tiles / clusters;
        const double tail = 0.5 * ((double)((tiles + clusters - 1) / clusters) - rounds);
        eff[i] = (double)clusters * s / sms * rounds / (rounds + tail);
    }
    return eff[1] * 0.97 > eff[0] ? 2 : 1;
}

int launch_gemv_tc(const void* a, const void* x, const void* sfa_sw, const void* sfx_sw, void* c, int M, int K, int L,
                   int x_rows, float alpha, int dev, cudaStream_t stream) {
    if (dev >= 64) return NVFP4_ERR_UNSUPPORTED;
    GemvTcParams p;
    CUtensorMap ta, tx;
    int rc;
    // A: when M is a multiple of 8 and K of 256, one box per stage over the view (256 elements, row within a group
    // of 8, chunk, group, batch): the chunks of a row are then asked of memory right after one another.  Otherwise
    // (or with NVFP4_GEMV_ABOX=3d, read on every call: tuning aid) one 128-row box per chunk.
    const char* abox = getenv("NVFP4_GEMV_ABOX");
    if (M % 8 == 0 && K % BK == 0 && !(abox && abox[0] == '3')) {
        rc = make_gemv_a_tmap(&ta, a, M, K, L);
        p.a_boxes = 1;
    } else {
        rc = make_operand_tmap(&ta, a, M, K, L, 128);
        p.a_boxes = GT_KCH;
    }
    if (rc) return rc;
    rc = make_operand_tmap(&tx, x, x_rows, K, L, 1);
    if (rc) return rc;
    p.sfa = (const uint8_t*)sfa_sw; p.sfx = (const uint8_t*)sfx_sw; p.c = (__half*)c;
    p.M = M; p.K = K; p.L = L;
    p.row_blocks = (M + BM - 1) / BM;
    p.x_row_blocks = (x_rows + 127) / 128;
    p.tiles = L * p.row_blocks;
    const int stages = (K + GT_BK - 1) / GT_BK;
    int V = 1;
    while (V * 2 <= GT_VMAX && V * 2 <= stages) V *= 2;
    p.V = V;
    p.alpha = alpha;
    p.status = status_word(dev);
    p.budget_ns = wait_budget_ns();
#ifdef NVFP4_PROFILE
    { const char* e_ = getenv("NVFP4_PROF_PTR"); p.prof = e_ ? (unsigned long long*)strtoull(e_, nullptr, 0) : nullptr; }
#endif
    if (pick_cluster(p.tiles, V, dev) == 2) return launch_tc<2>(ta, tx, p, dev, stream);
    return launch_tc<1>(ta, tx, p, dev, stream);
}

}  // namespace nvfp4
