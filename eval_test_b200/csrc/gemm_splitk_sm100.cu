// NVFP4 GEMM for shapes with few output tiles and a long K loop (the skinny-M shapes of the reference's own
// benchmark list, eval/nvfp4_gemm/benchmarks.txt:1-3): split K across a thread-block CLUSTER.
//
// With M = 128 and N = 7168 there are 56 tiles of 128 x 128 for 148 SMs, each CTA walks 64 K steps one after the
// other and a single CTA cannot pull more than about 100-180 GB/s through its stages: a long K loop on a
// third of the machine.  Here the
// S CTAs of a cluster (S = 2, 4 or 8) share ONE output tile: CTA r accumulates K steps [r*k/S, (r+1)*k/S) in its
// own tensor memory, then the partial sums are reduced through distributed shared memory:
//   * CTA r owns the column slice [r*128/S, (r+1)*128/S) of the tile: it keeps its own partial sums of that slice
//     in registers and writes the other slices of its fp32 partial tile to its own shared memory (over the stage
//     ring, which is idle by then),
//   * each warp tells the S-1 other CTAs (cluster-scope mbarrier) that its rows are written,
//   * CTA r reads its slice of every peer's partial tile with ld.shared::cluster, adds the partials in a fixed order
//     (its own, then ranks r+1, r+2, ... modulo S: deterministic), applies alpha, rounds to fp16 and stores.
// The TMA producer starts loading before the rest of the CTA has finished its set-up: it needs only the barriers it
// initialised itself.
// No global scratch, no atomics.  One tile per cluster (the shapes this serves have fewer tiles than SMs).
// Every mbarrier wait is bounded; the closing hardware cluster barrier is reached by every thread on every path.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_common.cuh"
#include "nvfp4_internal.h"
#include "ptx_sm100.cuh"

namespace nvfp4 {

constexpr int SK_BN = 128;   // output columns per tile; the dual GEMM's MMA is 256 wide over [B1; B2]
// GEMM: six stages of 36 KB (with a cold L2 - how the harness times a call - M=128 N=7168 K=16384 takes 21.3 us
// against 23.8 us with four stages); dual GEMM: four stages of 54 KB
__host__ __device__ constexpr int sk_stages(bool dual) { return dual ? 4 : 6; }
constexpr uint32_t SK_A_BYTES = 128 * 128, SK_B_BYTES = 128 * 128, SK_SF_BYTES = 2048;
__host__ __device__ constexpr uint32_t sk_stage_bytes(bool dual) { return SK_A_BYTES + (dual ? 2 : 1) * (SK_B_BYTES + SK_SF_BYTES) + SK_SF_BYTES; }
__host__ __device__ constexpr uint32_t sk_red_bytes(bool dual) { return 128 * SK_BN * 4 * (dual ? 2 : 1); }   // fp32 partial tile
// the partial tile reuses the stage ring: once "accumulator complete" has fired, every load has landed and every
// MMA has read its stage
static_assert(sk_stages(false) * sk_stage_bytes(false) >= sk_red_bytes(false) &&
              sk_stages(true) * sk_stage_bytes(true) >= sk_red_bytes(true), "the partial tile lives in the stage ring");
__host__ __device__ constexpr size_t sk_smem(bool dual) { return sk_stages(dual) * sk_stage_bytes(dual) + 1024; }

__device__ __forceinline__ float4 ld_cluster_f4(uint32_t cluster_addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(cluster_addr)
                 : "memory");
    return v;
}

template <int S, bool DUAL>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_splitk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const __grid_constant__ CUtensorMap tmap_b2, const GemmParams p) {
    constexpr int STAGES = sk_stages(DUAL);
    constexpr uint32_t SK_STAGE_BYTES = sk_stage_bytes(DUAL);
    constexpr int MMA_N = DUAL ? 2 * SK_BN : SK_BN;    // accumulator columns: x = A.B1 in 0..127, y = A.B2 in 128..255
    constexpr uint32_t SF_COLS = 16 + 4 * (MMA_N / 32);   // TMEM columns of one stage's scales
    constexpr uint32_t SF_BASE = MMA_N;
    constexpr uint32_t TCOLS = DUAL ? 512 : 256;       // accumulator + two alternating scale regions, a power of two
    static_assert(SF_BASE + 2 * SF_COLS <= TCOLS, "tensor memory");
    constexpr int SLICE = SK_BN / S;                   // output columns this CTA reduces
    static_assert(S == 2 || S == 4 || S == 8, "cluster size");
    static_assert(!DUAL || SLICE >= 32, "dual GEMM: whole 32-column chunks per CTA");

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * STAGES + 2];
    __shared__ uint32_t tmem_base_slot;

    const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t red0 = smem0;                               // same offset in every CTA of the cluster
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    const uint32_t acc_full = smem_u32(&bars[2 * STAGES]);
    const uint32_t red_ready = acc_full + 8;                   // 4 epilogue warps of each of the S CTAs

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
        if (DUAL) prefetch_tmap(&tmap_b2);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(red_ready, 4 * (S - 1));
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), TCOLS);
        tmem_relinquish();
    }
    // Peers arrive on this CTA's red_ready barrier only after their cluster_wait_acquire() below, i.e. after every
    // thread here has arrived, thread 0 (which initialised the barrier) among them.  The producer warp arrives
    // after it has issued its loads (a release-arrive takes about half a microsecond, and nobody needs it before
    // this CTA's partial sums exist).
    if (warp != 0) cluster_arrive_release();
    uint32_t tmem_base = 0;
    if (warp == 0) {
        __syncwarp();                        // the loading lane sees the barriers lane 0 initialised
        named_bar_arrive(1, GEMM_THREADS);   // ... and so will the other warps; this one does not wait for them
    } else {
        tc_fence_before_sync();
        named_bar_sync(1, GEMM_THREADS);
        tc_fence_after_sync();
        tmem_base = tmem_base_slot;
    }

    // tile of this cluster, K range of this CTA
    const int tiles_m = (p.M + BM - 1) / BM, tiles_n = p.N / SK_BN;
    const int t = blockIdx.x / S;
    const int l = t / (tiles_m * tiles_n);
    const int r_ = t - l * tiles_m * tiles_n;
    const int nt = r_ / tiles_m, mt = r_ - nt * tiles_m;       // row tiles of one column tile run together
    const int m0 = mt * BM, n0 = nt * SK_BN;
    const int kiters_all = p.K / BK;
    const int kbase = kiters_all / S, krem = kiters_all % S;
    const int kcount = kbase + ((int)rank < krem ? 1 : 0);
    const int kfirst = (int)rank * kbase + min((int)rank, krem);
    const size_t sf_row_block = (size_t)(p.K / 64) * 512;
    const uint8_t* sfa_t = p.sfa + ((size_t)l * tiles_m + mt) * sf_row_block;
    const uint8_t* sfb_t = p.sfb + ((size_t)l * tiles_n + nt) * sf_row_block;
    const uint8_t* sfb2_t = DUAL ? p.sfb2 + ((size_t)l * tiles_n + nt) * sf_row_block : nullptr;

    if (warp == 0) {
        if (elect_one()) {
            for (int it = 0; it < kcount; it++) {
                const int slot = it % STAGES;
                if (!mbar_wait(empty0 + 8 * slot, ((it / STAGES) & 1) ^ 1, p.budget_ns)) {
                    report_status(p.status, DEV_TIMEOUT_PRODUCER);
                    break;
                }
                const uint32_t full = full0 + 8 * slot;
                const uint32_t sA = smem0 + slot * SK_STAGE_BYTES, sB = sA + SK_A_BYTES;
                const uint32_t sSFA = sB + (DUAL ? 2 : 1) * SK_B_BYTES, sSFB = sSFA + SK_SF_BYTES;
                const int k0 = (kfirst + it) * BK;
                mbar_arrive_expect_tx(full, SK_STAGE_BYTES);
                tma_load_3d(sA, &tmap_a, k0, m0, l, full);
                tma_load_3d(sB, &tmap_b, k0, n0, l, full);
                if (DUAL) tma_load_3d(sB + SK_B_BYTES, &tmap_b2, k0, n0, l, full);
                const size_t koff = (size_t)(k0 / 64) * 512;
                bulk_g2s(sSFA, sfa_t + koff, 2048u, full);
                bulk_g2s(sSFB, sfb_t + koff, 2048u, full);
                if (DUAL) bulk_g2s(sSFB + 2048u, sfb2_t + koff, 2048u, full);
            }
        }
        __syncwarp();
        cluster_arrive_release();
        cluster_wait_acquire();
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc = make_idesc_nvfp4(BM, MMA_N);
            bool alive = true;
            for (int it = 0; it < kcount; it++) {
                const int slot = it % STAGES;
                if (!mbar_wait(full0 + 8 * slot, (it / STAGES) & 1, p.budget_ns)) {
                    report_status(p.status, DEV_TIMEOUT_CONSUMER);
                    alive = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t sA = smem0 + slot * SK_STAGE_BYTES, sB = sA + SK_A_BYTES;
                const uint32_t sSFA = sB + (DUAL ? 2 : 1) * SK_B_BYTES, sSFB = sSFA + SK_SF_BYTES;
                const uint32_t t_sfa = tmem_base + SF_BASE + (it & 1) * SF_COLS, t_sfb = t_sfa + 16;
#pragma unroll
                for (int ks = 0; ks < 4; ks++) {
                    tc_cp_sf_atom(t_sfa + 4 * ks, make_desc_sf(sSFA + 512 * ks));
#pragma unroll
                    for (int j = 0; j < MMA_N / 128; j++)
                        tc_cp_sf_atom(t_sfb + ks * (MMA_N / 32) + 4 * j, make_desc_sf(sSFB + j * 2048 + 512 * ks));
                }
#pragma unroll
                for (int ks = 0; ks < 4; ks++)
                    tc_mma_nvfp4(tmem_base, make_desc_k_sw128(sA + 32 * ks), make_desc_k_sw128(sB + 32 * ks), idesc,
                                 t_sfa + 4 * ks, t_sfb + ks * (MMA_N / 32), (it | ks) != 0 ? 1u : 0u);
                tc_commit(empty0 + 8 * slot);
            }
            if (alive) tc_commit(acc_full);
        }
        cluster_wait_acquire();
    } else {
        // ------------------------------------------------------------------ epilogue warps: partial -> smem -> reduce
        const int q = warp & 3;
        const int row_in_tile = q * 32 + lane;
        constexpr int OWN_CHUNKS = SLICE >= 32 ? SLICE / 32 : 1;        // 32-column chunks that hold this CTA's slice
        constexpr int PER_CHUNK = SLICE >= 32 ? 1 : 32 / SLICE;         // slices per chunk
        const int own_chunk0 = (int)rank * OWN_CHUNKS / PER_CHUNK;
        bool ok = mbar_wait(acc_full, 0, p.budget_ns);
        if (!ok && lane == 0) report_status(p.status, DEV_TIMEOUT_EPILOGUE);
        const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
        if (ok) {
            tc_fence_after_sync();
            // partial tile layout: 16-byte chunk c4 of row r at (c4 * 128 + r) * 16 -> consecutive lanes,
            // consecutive addresses, for the writes here and for the peers' reads below
            uint8_t* red_local = smem_raw + (red0 - smem_u32(smem_raw));
#pragma unroll
            for (int cc = 0; cc < MMA_N / 32; cc++) {
                // a chunk that holds nothing but this CTA's own slice (of x or of y) stays in tensor memory
                if (SLICE >= 32 && (cc & 3) >= own_chunk0 && (cc & 3) < own_chunk0 + OWN_CHUNKS) continue;
                uint32_t v[32];
                tc_ld_32x32(t_lane + cc * 32, v);
                tc_wait_ld();
#pragma unroll
                for (int j = 0; j < 8; j++)
                    *reinterpret_cast<uint4*>(red_local + ((size_t)((cc * 8 + j) * 128 + row_in_tile)) * 16) =
                        make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            }
        }
        // tell the other CTAs of the cluster that this warp's rows are written, one lane per peer (a release-arrive
        // on a remote barrier takes hundreds of cycles, and one thread's arrives queue up behind one another); a
        // warp whose accumulator never completed still arrives, so that no peer waits for it in vain
        cluster_wait_acquire();     // the peers' barriers exist
        __syncwarp();
        if (lane < S && lane != (int)rank) mbar_arrive_cluster(mapa_shared(red_ready, (uint32_t)lane));
        constexpr int HALVES = DUAL ? 2 : 1;        // dual GEMM: the slice of x, then the same slice of y
        float acc[HALVES * SLICE];
        if (ok) {
            // this CTA's own slice, while the peers' signals are on their way
            if constexpr (SLICE >= 32) {
#pragma unroll
                for (int h = 0; h < HALVES; h++)
#pragma unroll
                    for (int i = 0; i < OWN_CHUNKS; i++) {
                        uint32_t v[32];
                        tc_ld_32x32(t_lane + (h * 4 + own_chunk0 + i) * 32, v);
                        tc_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; j++) acc[h * SLICE + 32 * i + j] = __uint_as_float(v[j]);
                    }
            } else {
                uint32_t v[32];
                tc_ld_32x32(t_lane + own_chunk0 * 32, v);
                tc_wait_ld();
                const int part = (int)rank % PER_CHUNK;
#pragma unroll
                for (int j = 0; j < SLICE; j++) {
                    float x = __uint_as_float(v[j]);
#pragma unroll
                    for (int h = 1; h < PER_CHUNK; h++)
                        if (part == h) x = __uint_as_float(v[h * SLICE + j]);
                    acc[j] = x;
                }
            }
            ok = mbar_wait_cluster(red_ready, 0, p.budget_ns);
            if (!ok && lane == 0) report_status(p.status, DEV_TIMEOUT_EPILOGUE);
        }
        if (ok) {
            const int row = m0 + row_in_tile;
#pragma unroll
            for (int i = 1; i < S; i++) {
                const uint32_t peer = mapa_shared(red0, (rank + (uint32_t)i) % (uint32_t)S);
#pragma unroll
                for (int h = 0; h < HALVES; h++)
#pragma unroll
                    for (int j = 0; j < SLICE / 4; j++) {
                        const int c4 = h * (SK_BN / 4) + (int)rank * (SLICE / 4) + j;
                        const float4 v = ld_cluster_f4(peer + (uint32_t)((c4 * 128 + row_in_tile) * 16));
                        float* a4 = acc + h * SLICE + 4 * j;
                        a4[0] += v.x; a4[1] += v.y; a4[2] += v.z; a4[3] += v.w;
                    }
            }
            if (row < p.M) {
                __half* dst = p.c + ((size_t)l * p.M + row) * p.N + n0 + (int)rank * SLICE;
                uint32_t o[SLICE / 2];
#pragma unroll
                for (int i = 0; i < SLICE / 2; i++) {
                    float r0 = p.alpha * acc[2 * i], r1 = p.alpha * acc[2 * i + 1];
                    if (DUAL) {
                        r0 = silu_mul(r0, p.alpha * acc[(HALVES - 1) * SLICE + 2 * i]);
                        r1 = silu_mul(r1, p.alpha * acc[(HALVES - 1) * SLICE + 2 * i + 1]);
                    }
                    __half2 h = __floats2half2_rn(r0, r1);
                    o[i] = *reinterpret_cast<uint32_t*>(&h);
                }
#pragma unroll
                for (int i = 0; i < SLICE / 16; i++) {
                    const uint32_t w8[8] = {o[8 * i], o[8 * i + 1], o[8 * i + 2], o[8 * i + 3],
                                            o[8 * i + 4], o[8 * i + 5], o[8 * i + 6], o[8 * i + 7]};
                    st_global_256(dst + 16 * i, w8);
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();     // no CTA exits (or frees its shared memory) while a peer may still read its partial tile
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TCOLS);
    }
}

// ------------------------------------------------------------------------------------------ host side
namespace {

template <int S, bool DUAL>
int launch_splitk(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const GemmParams& p, int tiles,
                  cudaStream_t stream) {
    static bool done[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 64) return NVFP4_ERR_UNSUPPORTED;
    if (!done[dev]) {
        e = cudaFuncSetAttribute(gemm_splitk_kernel<S, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)sk_smem(DUAL));
        if (e != cudaSuccess) return (int)e;
        done[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles * S);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = sk_smem(DUAL);
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = S; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, gemm_splitk_kernel<S, DUAL>, ta, tb, tb2, p);
    return e == cudaSuccess ? NVFP4_OK : (int)e;
}

}  // namespace

// Cluster size to split K with, or 0 when the shape is better served by the persistent kernel.
// Measured on B200, device time of one call with a cold L2 (a 512 MiB fill before every call, which is how the
// harness times): M=128 N=7168 K=16384 (56 tiles, 64 K steps) 25.3 us unsplit, 20.3 us with S=2, 30 us with S=4
// (224 CTAs: two rounds); M=128 N=4096 K=7168 (32 tiles, 28 K steps) 11.8 us unsplit, 10.6 us with S=2, 10.1 us
// with S=4; M=128 N=7168 K=2048 (8 K steps) 7.0 us unsplit, 8.0 us with S=2.  The reduction through distributed
// shared memory costs about 2 us, a K step about 0.2 us.  Hence: all CTAs resident at once, at most half the SMs busy
// without splitting, and at least 7 K steps per CTA.
int splitk_factor(int M, int N, int K, int L, int dev) {
    const long tiles = (long)((M + BM - 1) / BM) * (N / SK_BN) * L;
    const int kiters = K / BK;
    const int sms = sm_count(dev);
    if (tiles <= 0 || tiles * 2 > sms) return 0;
    for (int s = 4; s >= 2; s /= 2)
        if (tiles * s <= sms && kiters / s >= 7) return s;
    return 0;
}

int launch_gemm_splitk(int S, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream) {
    const int tiles = ((p.M + BM - 1) / BM) * (p.N / SK_BN) * p.L;
    switch (S) {
        case 2: return launch_splitk<2, false>(ta, tb, tb, p, tiles, stream);
        case 4: return launch_splitk<4, false>(ta, tb, tb, p, tiles, stream);
        case 8: return launch_splitk<8, false>(ta, tb, tb, p, tiles, stream);
        default: return NVFP4_ERR_INTERNAL;
    }
}

// The dual GEMM on the same kernel (S = 2 or 4): both products are reduced across the cluster before silu(x) * y.
int launch_dual_gemm_splitk(int S, const CUtensorMap& ta, const CUtensorMap& tb1, const CUtensorMap& tb2, const GemmParams& p,
                            cudaStream_t stream) {
    const int tiles = ((p.M + BM - 1) / BM) * (p.N / SK_BN) * p.L;
    switch (S) {
        case 2: return launch_splitk<2, true>(ta, tb1, tb2, p, tiles, stream);
        case 4: return launch_splitk<4, true>(ta, tb1, tb2, p, tiles, stream);
        default: return NVFP4_ERR_INTERNAL;
    }
}

}  // namespace nvfp4
