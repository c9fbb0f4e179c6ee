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
//     vector is row 0 of the 16-row N side (rows 1..15 are zero and their result columns are never read);
//   * per stage (256 K-elements) the producer thread issues four copies: the A tile (tiled TMA, 128-byte
//     swizzle, rows past M read as zero), 128 bytes of the vector, and the scale atoms of A and of the vector
//     (512 bytes per 64 K-elements each, contiguous in the swizzled global layout);
//   * a ring of 10 stages (220 KB) keeps about 180 KB of HBM reads in flight per SM;
//   * the MMA thread copies the atoms into tensor memory (tcgen05.cp) and issues the MMAs; tcgen05.commit frees
//     the stage; four epilogue warps read column 0 of the accumulator (tcgen05.ld), scale and store fp16.
// Load balance: a tile is 128 rows over all of K, and 512 tiles do not divide over 148 SMs, so the S CTAs of a
// thread-block cluster (S = 1, 2, 4, 8) share a tile by splitting K and add their partial sums through distributed
// shared memory.  To keep the result independent of S, K is always cut into the same V segments (V = 8 when K
// has at least 8 stages), every segment is accumulated in its own tensor-memory columns, and the V partial sums
// are added in segment order whichever CTA produced them: a row's bits depend on K only, not on M, L or the
// cluster size.  No global scratch, no atomics.
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
    int V;                // K segments (power of two, 1..8, at most K/256 rounded up)
    float alpha;
    int* status;
    unsigned long long budget_ns;
#ifdef NVFP4_PROFILE
    unsigned long long* prof = nullptr;  // per CTA: producer wait / MMA wait-for-data / MMA issue / MMA total cycles
#endif
};

constexpr int GT_N = 16;                       // MMA N: the vector and 15 zero rows
constexpr int GT_STAGES = 10;
constexpr int GT_THREADS = 192;
constexpr int GT_VMAX = 8;
constexpr uint32_t GT_A_BYTES = 128 * 128;     // 128 rows x 256 e2m1
constexpr uint32_t GT_X_BYTES = GT_N * 128;
constexpr uint32_t GT_SF_BYTES = 4 * 512;      // 4 atoms
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
    constexpr uint32_t TCOLS = 512;
    constexpr uint32_t ACC_STRIDE = GT_VMAX * GT_N;    // columns of one accumulator buffer (one 16-column group per segment)
    constexpr uint32_t SF_BASE = 2 * ACC_STRIDE;       // two alternating scale regions of 32 columns follow
    static_assert(S == 1 || S == 2 || S == 4 || S == 8, "cluster size");

#ifdef NVFP4_PROFILE
    const unsigned long long prof_t_entry = globaltimer_ns();
#endif
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 6];
    __shared__ uint32_t tmem_base_slot;
    constexpr int JMAX = GT_VMAX / S;                  // segments one CTA can hold
    constexpr int RED_J = S > 1 ? JMAX : 1;            // (no exchange when the cluster is one CTA)
    __shared__ __align__(16) float red[2][RED_J][128]; // partial sums by tile parity, segment, row

    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = S > 1 ? cluster_ctarank() : 0u;
    const int cluster_id = blockIdx.x / S, nclusters = gridDim.x / S;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t acc_full0 = smem_u32(&bars[2 * STAGES]);
    const uint32_t acc_empty0 = acc_full0 + 16;
    const uint32_t red_ready0 = acc_full0 + 32;           // [2] by tile parity: 4 epilogue warps of each of the S CTAs

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, 4);
            mbar_init(red_ready0 + 8 * b, 4 * S);
        }
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_x);
    }
    {
        // rows 1..15 of every stage's vector tile stay zero for the whole kernel (the copies only write row 0)
        uint8_t* base = smem_raw + (smem0 - smem_u32(smem_raw));
        for (int i = threadIdx.x; i < STAGES * (int)(GT_X_BYTES / 16); i += GT_THREADS) {
            const int s = i / (int)(GT_X_BYTES / 16), o = i % (int)(GT_X_BYTES / 16);
            *reinterpret_cast<uint4*>(base + (size_t)s * GT_STAGE_BYTES + GT_A_BYTES + o * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async_smem();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), TCOLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    if (S > 1) cluster_sync_all();   // every CTA's barriers exist before a peer arrives on them
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
#ifdef NVFP4_PROFILE
    const unsigned long long prof_t_setup = globaltimer_ns();
#endif

    // K range of this CTA: segments [rank*VS, (rank+1)*VS) of the V the whole K loop is cut into
    const int stages_all = (p.K + BK - 1) / BK;
    const int atoms_all = p.K / 64;
    const int V = p.V, VS = V / S;
    const int kfirst = seg_start((int)rank * VS, stages_all, V);
    const int kend = seg_start((int)rank * VS + VS, stages_all, V);
    const size_t sf_row_block = (size_t)atoms_all * 512;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer (one lane)
        if (elect_one()) {
            uint32_t it = 0;
            bool alive = true;
#ifdef NVFP4_PROFILE
            long long prof_wait = 0;
            const long long prof_begin = clock64();
#endif
            for (int t = cluster_id; alive && t < p.tiles; t += nclusters) {
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
                        alive = false;
                        break;
                    }
                    const uint32_t full = full0 + 8 * slot;
                    const uint32_t sA = smem0 + slot * GT_STAGE_BYTES, sX = sA + GT_A_BYTES;
                    const uint32_t sSFA = sX + GT_X_BYTES, sSFX = sSFA + GT_SF_BYTES;
                    const int nat = min(4, atoms_all - ks * 4);       // 64-element groups of this stage inside K
                    mbar_arrive_expect_tx(full, GT_A_BYTES + 128u + (uint32_t)nat * 1024u);
                    tma_load_3d(sA, &tmap_a, ks * BK, m0, l, full);   // K past the end reads as zero
                    tma_load_3d(sX, &tmap_x, ks * BK, 0, l, full);
                    bulk_g2s(sSFA, sfa_t + (size_t)ks * 2048, (uint32_t)nat * 512u, full);
                    bulk_g2s(sSFX, sfx_t + (size_t)ks * 2048, (uint32_t)nat * 512u, full);
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
            uint32_t it = 0, tile_it = 0;
            bool alive = true;
#ifdef NVFP4_PROFILE
            long long prof_full = 0, prof_issue = 0;
            const long long prof_begin = clock64();
#endif
            for (int t = cluster_id; alive && t < p.tiles; t += nclusters, tile_it++) {
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
                        const uint32_t t_sfa = tmem_base + SF_BASE + (it & 1) * 32, t_sfx = t_sfa + 16;
                        const int nat = min(4, atoms_all - ks * 4);
#pragma unroll
                        for (int a = 0; a < 4; a++) {
                            if (a < nat) {
                                tc_cp_sf_atom(t_sfa + 4 * a, make_desc_sf(sSFA + 512 * a));
                                tc_cp_sf_atom(t_sfx + 4 * a, make_desc_sf(sSFX + 512 * a));
                            }
                        }
#pragma unroll
                        for (int a = 0; a < 4; a++) {
                            if (a < nat)
                                tc_mma_nvfp4(t_acc, make_desc_k_sw128(sA + 32 * a), make_desc_k_sw128(sX + 32 * a), idesc,
                                             t_sfa + 4 * a, t_sfx + 4 * a, (ks != s0 || a != 0) ? 1u : 0u);
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
            }
#endif
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps 2..5
        const int q = warp & 3;                       // TMEM lane quadrant this warp may access
        const int row_in_tile = q * 32 + lane;
        uint32_t tile_it = 0;
        for (int t = cluster_id; t < p.tiles; t += nclusters, tile_it++) {
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
                if (lane == 0) {
#pragma unroll
                    for (int c = 0; c < S; c++) mbar_arrive_cluster(mapa_shared(red_ready0 + 8 * buf, (uint32_t)c));
                }
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
    const unsigned long long prof_t_roles = globaltimer_ns();
#endif
    tc_fence_before_sync();
    __syncthreads();
    if (S > 1) cluster_sync_all();   // no CTA exits while a peer may still read its partial sums
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TCOLS);
    }
#ifdef NVFP4_PROFILE
    if (p.prof && threadIdx.x == GT_THREADS - 1) {   // an epilogue thread: the last role to finish
        p.prof[10 * blockIdx.x + 5] = prof_t_entry;
        p.prof[10 * blockIdx.x + 6] = prof_t_setup;
        p.prof[10 * blockIdx.x + 7] = prof_t_roles;
        p.prof[10 * blockIdx.x + 8] = globaltimer_ns();
    }
#endif
}

// ------------------------------------------------------------------------------------------ host side
namespace {

template <int S>
int launch_tc(const CUtensorMap& ta, const CUtensorMap& tx, const GemvTcParams& p, int dev, cudaStream_t stream) {
    static bool configured[64] = {};
    static int max_clusters[64] = {};
    auto kern = gemv_tc_kernel<S>;
    cudaError_t e;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(GT_THREADS);
    cfg.dynamicSmemBytes = GT_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = S; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (!configured[dev]) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GT_SMEM);
        if (e != cudaSuccess) return (int)e;
        // clusters of S CTAs (one CTA per SM) the device can hold at once
        int n = sm_count(dev) / S;
        if (S > 1) {
            cfg.gridDim = dim3((unsigned)(sm_count(dev) / S * S));
            int active = 0;
            e = cudaOccupancyMaxActiveClusters(&active, kern, &cfg);
            if (e != cudaSuccess) return (int)e;
            if (active > 0 && active < n) n = active;
        }
        max_clusters[dev] = n > 0 ? n : 1;
        configured[dev] = true;
    }
    const int clusters = p.tiles < max_clusters[dev] ? p.tiles : max_clusters[dev];
    cfg.gridDim = dim3((unsigned)(clusters * S));
    e = cudaLaunchKernelEx(&cfg, kern, ta, tx, p);
    return e == cudaSuccess ? NVFP4_OK : (int)e;
}

}  // namespace

// Cluster size for a shape: the one that keeps the most SMs streaming over the whole call
// (tiles / (rounds * clusters) * share of SMs in whole clusters); ties go to the smaller cluster.
// NVFP4_GEMV_SPLIT = 1, 2, 4 or 8 forces a size where the shape allows it (tuning aid).
static int pick_cluster(int tiles, int V, int dev) {
    const char* e_ = getenv("NVFP4_GEMV_SPLIT");   // read on every call: tests compare cluster sizes in one process
    const int forced = e_ ? atoi(e_) : 0;
    if ((forced == 1 || forced == 2 || forced == 4 || forced == 8) && forced <= V) return forced;
    const int sms = sm_count(dev);
    int best = 1;
    double best_eff = 0.0;
    for (int s = 1; s <= V && s <= 8; s *= 2) {
        const int clusters = sms / s;
        if (clusters <= 0) break;
        const int rounds = (tiles + clusters - 1) / clusters;
        const int used = tiles < clusters ? tiles : clusters;
        const double eff = (double)tiles / ((double)rounds * used) * ((double)used * s / sms);
        if (eff > best_eff + 1e-9) { best_eff = eff; best = s; }
    }
    return best;
}

int launch_gemv_tc(const void* a, const void* x, const void* sfa_sw, const void* sfx_sw, void* c, int M, int K, int L,
                   int x_rows, float alpha, int dev, cudaStream_t stream) {
    if (dev >= 64) return NVFP4_ERR_UNSUPPORTED;
    CUtensorMap ta, tx;
    int rc = make_operand_tmap(&ta, a, M, K, L, 128);
    if (rc) return rc;
    rc = make_operand_tmap(&tx, x, x_rows, K, L, 1);
    if (rc) return rc;
    GemvTcParams p;
    p.sfa = (const uint8_t*)sfa_sw; p.sfx = (const uint8_t*)sfx_sw; p.c = (__half*)c;
    p.M = M; p.K = K; p.L = L;
    p.row_blocks = (M + BM - 1) / BM;
    p.x_row_blocks = (x_rows + 127) / 128;
    p.tiles = L * p.row_blocks;
    const int stages = (K + BK - 1) / BK;
    int V = 1;
    while (V * 2 <= GT_VMAX && V * 2 <= stages) V *= 2;
    p.V = V;
    p.alpha = alpha;
    p.status = status_word(dev);
    p.budget_ns = wait_budget_ns();
#ifdef NVFP4_PROFILE
    { const char* e_ = getenv("NVFP4_PROF_PTR"); p.prof = e_ ? (unsigned long long*)strtoull(e_, nullptr, 0) : nullptr; }
#endif
    switch (pick_cluster(p.tiles, V, dev)) {
        case 1: return launch_tc<1>(ta, tx, p, dev, stream);
        case 2: return launch_tc<2>(ta, tx, p, dev, stream);
        case 4: return launch_tc<4>(ta, tx, p, dev, stream);
        case 8: return launch_tc<8>(ta, tx, p, dev, stream);
        default: return NVFP4_ERR_INTERNAL;
    }
}

}  // namespace nvfp4
