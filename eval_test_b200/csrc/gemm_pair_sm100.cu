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
// GROUPED: the pair tiles of all groups form one launch-wide list (PairGroupEntry table in device memory, binary
// search tile -> group, row tile fastest inside a group); every group has its own four tensor maps.  Opt-in
// (NVFP4_GEMM_PAIR=1): on an expert layer with M_g around 128, which is bound by streaming the weights from HBM, it
// measured 9 % slower than the single-CTA kernel (a pair advances only when both CTAs' halves of a stage have
// arrived, and the second CTA of a group with M_g <= 128 computes on rows that do not exist); it pays for groups
// with several hundred rows each.
// Every mbarrier wait is bounded; the two hardware cluster barriers (after set-up, before exit) are reached by
// every thread on every path.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdlib.h>

#include <mutex>

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

// Everything a role of one CTA needs to know about one pair tile.
struct PairTile {
    const CUtensorMap *ta, *tb, *tb2, *tsa, *tsb, *tsb2;
    __half* c;            // output of this problem / batch, [M][N]
    int M, N, kiters, l;
    int m0;               // first row of THIS CTA's 128 rows
    int n0;               // first output column of the pair tile
    int atom_a, atom_b;   // scale atoms (512 bytes) of this CTA's A rows / of the tile's first 128 B rows at k = 0
    int apb;              // atoms of one 128-row scale block = K / 64
    bool a_rows_exist, peer_rows_exist;
};

// Pair tile t -> problem, batch, 256-row tile, column tile.  Plain / dual GEMM: the banded order of the single-CTA
// kernel.  GROUPED: binary search of the group whose tile range holds t.
// GEMM: column tile = 256 output columns.  DUAL: 128 output columns.
template <bool DUAL, bool GROUPED>
__device__ __forceinline__ PairTile locate_pair(int t, const GemmParams& p, uint32_t rank, const CUtensorMap* ta,
                                                const CUtensorMap* tb, const CUtensorMap* tb2, const CUtensorMap* tsa,
                                                const CUtensorMap* tsb, const CUtensorMap* tsb2) {
    constexpr int BN = DUAL ? 128 : 256;
    PairTile ti;
    int mt;
    if (GROUPED) {
        const PairGroupEntry* tab = reinterpret_cast<const PairGroupEntry*>(p.pair_table);
        int lo = 0, hi = p.G - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (__ldg(&tab[mid].tile_start) <= t) lo = mid; else hi = mid - 1;
        }
        const PairGroupEntry* e = tab + lo;
        const int r = t - __ldg(&e->tile_start);
        const int tiles_m = __ldg(&e->tiles_m);
        const int nt = r / tiles_m;
        mt = r - nt * tiles_m;
        ti.ta = &e->ta; ti.tb = &e->tb; ti.tb2 = &e->tb; ti.tsa = &e->tsa; ti.tsb = &e->tsb; ti.tsb2 = &e->tsb;
        ti.M = __ldg(&e->M); ti.N = __ldg(&e->N);
        const int K = __ldg(&e->K);
        ti.kiters = K / BK; ti.apb = K / 64; ti.l = 0;
        ti.n0 = nt * BN;
        ti.c = e->c;
        ti.m0 = mt * 256 + (int)rank * 128;
        ti.atom_a = (ti.m0 >> 7) * ti.apb;
        ti.atom_b = (ti.n0 / 128) * ti.apb;
    } else {
        const int tiles_m = (p.M + 255) / 256, tiles_n = p.N / BN;
        const TileCoord tc = tile_coord(t, tiles_m, tiles_n);
        const int RA = (p.M + 127) / 128, RB = p.N / 128;
        mt = tc.mt;
        ti.ta = ta; ti.tb = tb; ti.tb2 = tb2; ti.tsa = tsa; ti.tsb = tsb; ti.tsb2 = tsb2;
        ti.M = p.M; ti.N = p.N; ti.kiters = p.K / BK; ti.apb = p.K / 64; ti.l = tc.l;
        ti.n0 = tc.nt * BN;
        ti.c = p.c + (size_t)tc.l * p.M * p.N;
        ti.m0 = mt * 256 + (int)rank * 128;
        ti.atom_a = (tc.l * RA + (ti.m0 >> 7)) * ti.apb;
        ti.atom_b = (tc.l * RB + ti.n0 / 128) * ti.apb;
    }
    ti.a_rows_exist = ti.m0 < ti.M;
    ti.peer_rows_exist = mt * 256 + 128 < ti.M;
    return ti;
}

// What one pair does, in order.  Plain schedule: the tiles pair, pair + npairs, ... whole.  Stream-K: a contiguous
// share [u0, u1) of the launch-wide list of K steps (tile-major).  The share's partial piece at its END (a tile whose
// last K steps belong to the next pair) is computed FIRST and left as a partial accumulator; the piece at its BEGINNING
// (a tile started by the previous pairs) comes SECOND and finishes that tile - the partials it needs were the first
// thing their pairs produced, and its slower epilogue (it reads them back) overlaps the MMAs of the whole tiles, which
// follow.  (With the finishing piece last, its epilogue was an un-overlapped tail of about 12 us.)
struct PairWork {
    int tile, k0, k1;
    int kind;           // 0 whole tile, 1 partial out (does not hold the tile's last K step), 2 finish (k0 > 0)
};
template <bool STREAMK>
struct PairSched {
    int n;                                   // work items of this pair
    int pair, npairs, kiters;
    int ft, lt, fk, lk;                      // stream-K: first / last tile of the share, first K step, end K step
    bool c, f;                               // stream-K: the last tile is a partial-out piece / the first one a finish piece
    long long U;
    __device__ __forceinline__ long long share_begin(int q) const { return U * q / npairs; }
    __device__ __forceinline__ PairSched(int pair_, int npairs_, int total_tiles, int kiters_)
        : pair(pair_), npairs(npairs_), kiters(kiters_) {
        if (!STREAMK) {
            n = pair < total_tiles ? (total_tiles - pair + npairs - 1) / npairs : 0;
            ft = lt = fk = lk = 0; c = f = false; U = 0;
            return;
        }
        U = (long long)total_tiles * kiters;
        const long long u0 = share_begin(pair), u1 = share_begin(pair + 1);
        if (u1 <= u0) { n = 0; ft = lt = fk = lk = 0; c = f = false; return; }
        ft = (int)(u0 / kiters); fk = (int)(u0 - (long long)ft * kiters);
        lt = (int)((u1 - 1) / kiters); lk = (int)(u1 - (long long)lt * kiters);
        n = lt - ft + 1;
        c = lk < kiters;
        f = ft != lt && fk > 0;
    }
    __device__ __forceinline__ PairWork item(int i) const {
        PairWork w;
        if (!STREAMK) {
            w.tile = pair + i * npairs; w.k0 = 0; w.k1 = kiters; w.kind = 0;
            return w;
        }
        int j;
        if (c && i == 0) j = lt;
        else {
            const int idx = i - (c ? 1 : 0);                           // index among the other tiles ft..(c ? lt-1 : lt)
            j = ft + idx;                                              // the finishing piece, if any, is tile ft: first of them
        }
        w.tile = j;
        w.k0 = j == ft ? fk : 0;
        w.k1 = j == lt ? lk : kiters;
        w.kind = w.k1 < kiters ? 1 : (w.k0 > 0 ? 2 : 0);
        return w;
    }
};

template <bool DUAL, bool GROUPED = false, bool STREAMK = false>
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
        if (!GROUPED) {
            prefetch_tmap(&tmap_a);
            prefetch_tmap(&tmap_b);
            prefetch_tmap(&tmap_sfa);
            prefetch_tmap(&tmap_sfb);
            if (DUAL) {
                prefetch_tmap(&tmap_b2);
                prefetch_tmap(&tmap_sfb2);
            }
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

    const int total_tiles = p.total_tiles;               // pair tiles of the launch
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
#define LOCATE_PAIR(t) locate_pair<DUAL, GROUPED>(t, p, rank, &tmap_a, &tmap_b, &tmap_b2, &tmap_sfa, &tmap_sfb, &tmap_sfb2)
    static_assert(!(STREAMK && GROUPED), "stream-K shares assume the same number of K steps in every tile");
    const PairSched<STREAMK> sched(pair, npairs, total_tiles, p.K / BK);

    if (warp == 0) {
        // ------------------------------------------------------------------ producer (both CTAs, own tiles)
        if (elect_one()) {
            uint32_t it = 0;
            bool alive = true;
            const uint32_t leader_full0 = mapa_shared(full0, 0);
            for (int wi = 0; alive && wi < sched.n; wi++) {
                const PairWork wk = sched.item(wi);
                const PairTile ti = LOCATE_PAIR(wk.tile);
                const int k_begin = STREAMK ? wk.k0 : 0, k_end = STREAMK ? wk.k1 : ti.kiters;
                for (int kit = k_begin; kit < k_end; kit++, it++) {
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
                                                                    PAIR_SFA_BYTES + (ti.peer_rows_exist ? PAIR_SFA_BYTES : 0u));
                    tma_load_3d_pair(sA, ti.ta, k0, ti.m0, ti.l, full);
                    if (ti.a_rows_exist) tma_load_2d_pair(sSFA, ti.tsa, 0, ti.atom_a + ka, full);
                    if (DUAL) {
                        // leader keeps the B1 tile, peer the B2 tile; both need both scale blocks
                        tma_load_3d_pair(sB, rank == 0 ? ti.tb : ti.tb2, k0, ti.n0, ti.l, full);
                        tma_load_2d_pair(sSFB, ti.tsb, 0, ti.atom_b + ka, full);
                        tma_load_2d_pair(sSFB + 2048u, ti.tsb2, 0, ti.atom_b + ka, full);
                    } else {
                        tma_load_3d_pair(sB, ti.tb, k0, ti.n0 + (int)rank * 128, ti.l, full);
                        tma_load_2d_pair(sSFB, ti.tsb, 0, ti.atom_b + ka, full);
                        tma_load_2d_pair(sSFB + 2048u, ti.tsb, 0, ti.atom_b + ti.apb + ka, full);
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
                for (int wi = 0; alive && wi < sched.n; wi++, tile_it++) {
                    const PairWork wk = sched.item(wi);
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
                    const int k_begin = STREAMK ? wk.k0 : 0, k_end = STREAMK ? wk.k1 : LOCATE_PAIR(wk.tile).kiters;
                    for (int kit = k_begin; kit < k_end; kit++, it++) {
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
                                              idesc, t_sfa + 4 * ks, t_sfb + 8 * ks, ((kit - k_begin) | ks) != 0 ? 1u : 0u);
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
        for (int wi = 0; wi < sched.n; wi++, tile_it++) {
            const PairWork wk = sched.item(wi);
            const PairTile ti = LOCATE_PAIR(wk.tile);
            const int row = ti.m0 + q * 32 + lane;
            const int n0 = ti.n0;
            const uint32_t buf = tile_it & 1;
            if (!mbar_wait(acc_full0 + 8 * buf, (tile_it >> 1) & 1, p.budget_ns)) {
                if (lane == 0) report_status(p.status, DEV_TIMEOUT_EPILOGUE);
                break;
            }
            tc_fence_after_sync();
            const uint32_t t_lane = tmem_base + buf * ACC1_OFF + ((uint32_t)(q * 32) << 16);
            __half* crow = ti.c + (size_t)(row < ti.M ? row : 0) * ti.N + n0;
            if (STREAMK && wk.kind != 0) {
                // this thread's row in a pair's scratch slot: [pair][CTA of the pair][128 rows][256 fp32]
                const size_t my_row = ((size_t)rank * 128 + q * 32 + lane) * 256;
                SkEpi sk;
                bool ready = true;
                if (wk.kind == 1) {
                    sk.out = p.sk_scratch + (size_t)pair * (2 * 128 * 256) + my_row;
                } else {
                    // the pairs before this one whose shares hold the tile's earlier K steps, lowest first
                    int q0 = pair - 1;
                    while (q0 > 0 && sched.share_begin(q0) > (long long)wk.tile * sched.kiters) q0--;
                    sk.n_in = pair - q0;
                    for (int j = 0; j < sk.n_in && j < 8; j++) {
                        sk.in[j] = p.sk_scratch + (size_t)(q0 + j) * (2 * 128 * 256) + my_row;
                        // the same warp of the same CTA of that pair wrote these rows
                        if (lane == 0) {
                            const unsigned int* flag = p.sk_flags + (size_t)(q0 + j) * 8 + rank * 4 + q;
                            const uint64_t t0 = globaltimer_ns();
                            while (ld_acquire_gpu_u32(flag) != p.sk_epoch) {
                                if (globaltimer_ns() - t0 > p.budget_ns) {
                                    report_status(p.status, DEV_TIMEOUT_EPILOGUE);
                                    ready = false;
                                    break;
                                }
                            }
                        }
                    }
                    ready = __all_sync(0xffffffffu, ready);
                    if (sk.n_in > 8) ready = false;      // never: the host does not split a tile over more than 8 shares
                }
                if (wk.kind == 1) {
                    if (buf == 0)
                        epilogue_tile<256, false, int(ACC1_OFF) / 32, OV_CHUNKS, true, false, false, 1>(
                            t_lane, crow, true, 0, 256, p.alpha, l_ovl_free, lane, nullptr, nullptr, &sk);
                    else
                        epilogue_tile<256, false, 0, OV_CHUNKS, true, false, false, 1>(t_lane, crow, true, 0, 256, p.alpha,
                                                                                      l_ovl_free, lane, nullptr, nullptr, &sk);
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) st_release_gpu_u32(p.sk_flags + (size_t)pair * 8 + rank * 4 + q, p.sk_epoch);
                } else if (buf == 0) {
                    epilogue_tile<BN, DUAL, int(ACC1_OFF) / 32, OV_CHUNKS, true, false, false, 2>(
                        t_lane, crow, ready && row < ti.M, n0, ti.N, p.alpha, l_ovl_free, lane, nullptr, nullptr, &sk);
                } else {
                    epilogue_tile<BN, DUAL, 0, OV_CHUNKS, true, false, false, 2>(
                        t_lane, crow, ready && row < ti.M, n0, ti.N, p.alpha, l_ovl_free, lane, nullptr, nullptr, &sk);
                }
            } else
            // the shared columns are released through the leader's barrier by a cluster-scope arrive
            if (buf == 0)
                epilogue_tile<BN, DUAL, int(ACC1_OFF) / 32, OV_CHUNKS, true>(t_lane, crow, row < ti.M, n0, ti.N, p.alpha,
                                                                            l_ovl_free, lane);
            else
                epilogue_tile<BN, DUAL, 0, OV_CHUNKS, true>(t_lane, crow, row < ti.M, n0, ti.N, p.alpha, l_ovl_free, lane);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster_relaxed(l_acc_empty0 + 8 * buf);   // accumulator read out (see ovl_free)
        }
    }

#undef LOCATE_PAIR
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

template <bool DUAL, bool GROUPED, bool STREAMK>
int configure(int dev) {
    static bool done[64] = {};
    if (done[dev]) return NVFP4_OK;
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<DUAL, GROUPED, STREAMK>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PAIR_SMEM);
    if (e != cudaSuccess) return (int)e;
    done[dev] = true;
    return NVFP4_OK;
}

template <bool DUAL, bool GROUPED, bool STREAMK>
int max_pairs(int dev) {
    static int cached[64] = {};
    if (cached[dev]) return cached[dev];
    // the occupancy query fails for more dynamic shared memory than the kernel has been allowed so far
    if (configure<DUAL, GROUPED, STREAMK>(dev) != NVFP4_OK) return -1;
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
    if (cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<DUAL, GROUPED, STREAMK>, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = 0;
    }
    cached[dev] = n > 0 ? n : -1;
    return cached[dev];
}

// Stream-K scratch of a device: one partial accumulator per pair (2 CTAs x 128 rows x 256 fp32) and eight flag words
// per pair, allocated on first use.  Launches that use it are ordered one after the other: on one stream by the
// stream, across streams by an event.
struct StreamKState {
    float* scratch = nullptr;
    unsigned int* flags = nullptr;
    int pairs = 0;
    unsigned int epoch = 0;
    cudaEvent_t done = nullptr;
    cudaStream_t last_stream = nullptr;
    bool used = false;
};
std::mutex g_sk_mu;
StreamKState g_sk[64];

// tiles: pair tiles of the launch; the maps are the plain / dual GEMM's (ignored by the grouped kernel).
template <bool DUAL, bool GROUPED, bool STREAMK>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const CUtensorMap& tsa,
           const CUtensorMap& tsb, const CUtensorMap& tsb2, const GemmParams& p, int tiles, cudaStream_t stream) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 64) return NVFP4_ERR_UNSUPPORTED;
    int rc = configure<DUAL, GROUPED, STREAMK>(dev);
    if (rc) return rc;
    const int pairs_max = max_pairs<DUAL, GROUPED, STREAMK>(dev);
    if (pairs_max <= 0) return NVFP4_ERR_UNSUPPORTED;
    if (tiles <= 0) return NVFP4_OK;
    const int pairs = (STREAMK || tiles >= pairs_max) ? pairs_max : tiles;
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
    GemmParams q = p;
    q.total_tiles = tiles;
    if (!STREAMK) {
        e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<DUAL, GROUPED, STREAMK>, ta, tb, tb2, tsa, tsb, tsb2, q);
        return e == cudaSuccess ? NVFP4_OK : (int)e;
    }
    std::lock_guard<std::mutex> lk(g_sk_mu);
    StreamKState& sk = g_sk[dev];
    if (sk.pairs < pairs) {
        if (sk.used && (e = cudaEventSynchronize(sk.done)) != cudaSuccess) return (int)e;
        if (sk.scratch) cudaFree(sk.scratch);
        if (sk.flags) cudaFree(sk.flags);
        sk.scratch = nullptr; sk.flags = nullptr; sk.pairs = 0;
        e = cudaMalloc((void**)&sk.scratch, (size_t)pairs * 2 * 128 * 256 * sizeof(float));
        if (e != cudaSuccess) return (int)e;
        e = cudaMalloc((void**)&sk.flags, (size_t)pairs * 8 * sizeof(unsigned int));
        if (e != cudaSuccess) return (int)e;
        e = cudaMemset(sk.flags, 0, (size_t)pairs * 8 * sizeof(unsigned int));
        if (e != cudaSuccess) return (int)e;
        sk.pairs = pairs;
        sk.epoch = 0;
    }
    if (!sk.done && (e = cudaEventCreateWithFlags(&sk.done, cudaEventDisableTiming)) != cudaSuccess) return (int)e;
    if (sk.used && sk.last_stream != stream && (e = cudaStreamWaitEvent(stream, sk.done, 0)) != cudaSuccess) return (int)e;
    q.sk_scratch = sk.scratch; q.sk_flags = sk.flags; q.sk_epoch = ++sk.epoch;
    e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<DUAL, GROUPED, STREAMK>, ta, tb, tb2, tsa, tsb, tsb2, q);
    if (e != cudaSuccess) return (int)e;
    sk.used = true; sk.last_stream = stream;
    e = cudaEventRecord(sk.done, stream);
    return e == cudaSuccess ? NVFP4_OK : (int)e;
}

// Stream-K is OPT-IN (NVFP4_GEMM_STREAMK=1 takes it wherever the tiles do not fill the last round of pairs and every
// share still spans at least half a tile's K loop; =2 only where the last round is less than 92 % full).  It is
// correct and balanced, and it measured SLOWER than the plain schedule on the shapes it was written for: the 8-way
// column shard of 8192^3 (128 tiles on 74 pairs) 39.5 us against 28.6 us, the 4-way shard 62.9 against 52.6 us.  Two
// reasons, both measured: (1) the board is power-limited on these operands, so the pairs that idle in a partly filled
// last round hand their power to the busy ones (SM clock 1.25 GHz with the plain schedule, 1.09 GHz with every pair
// busy to the end) - a perfectly balanced schedule finishes no earlier; (2) the pieces are short, so the two
// accumulator buffers no longer hide the epilogues of the partial pieces (MMA issuer waiting for an accumulator: 7 400
// cycles per pair against 900).
bool use_stream_k(int tiles, int pairs, int kiters) {
    static const int mode = [] { const char* e_ = getenv("NVFP4_GEMM_STREAMK"); return e_ ? atoi(e_) : 0; }();
    if (mode == 0 || tiles <= 0 || pairs <= 0 || kiters < 4) return false;
    const long long units = (long long)tiles * kiters;
    if (units / pairs < (kiters + 1) / 2) return false;          // a tile would be cut into more than a few pieces
    if (mode == 1) return tiles % pairs != 0;
    const int rounds = (tiles + pairs - 1) / pairs;
    return tiles % pairs != 0 && (double)tiles / ((double)pairs * rounds) < 0.92;
}

template <bool DUAL>
int launch_plain(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const GemmParams& p,
                 cudaStream_t stream) {
    const int tiles = ((p.M + 255) / 256) * (p.N / (DUAL ? 128 : 256)) * p.L;
    const long ka = p.K / 64;
    CUtensorMap tsa, tsb, tsb2;
    int rc = make_scale_tmap(&tsa, p.sfa, (long)p.L * ((p.M + 127) / 128) * ka);
    if (rc) return rc;
    rc = make_scale_tmap(&tsb, p.sfb, (long)p.L * (p.N / 128) * ka);
    if (rc) return rc;
    tsb2 = tsb;
    if (DUAL) {
        rc = make_scale_tmap(&tsb2, p.sfb2, (long)p.L * (p.N / 128) * ka);
        if (rc) return rc;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev >= 64) return NVFP4_ERR_UNSUPPORTED;
    if (use_stream_k(tiles, max_pairs<DUAL, false, true>(dev), p.K / BK))
        return launch<DUAL, false, true>(ta, tb, tb2, tsa, tsb, tsb2, p, tiles, stream);
    return launch<DUAL, false, false>(ta, tb, tb2, tsa, tsb, tsb2, p, tiles, stream);
}

}  // namespace

bool pair_kernel_suits(int M, int N, int K, int L, bool dual, int dev) {
    if (M < 256 || N % (dual ? 128 : 256) != 0 || dev >= 64) return false;
    const int pairs = dual ? max_pairs<true, false, false>(dev) : max_pairs<false, false, false>(dev);
    if (pairs <= 0) return false;
    const long tiles = (long)((M + 255) / 256) * (N / (dual ? 128 : 256)) * L;
    // rows of the last 256-row tile that do not exist are wasted work for one CTA of the pair
    const bool ragged_waste = (M % 256 != 0) && (M < 2048);
    return tiles >= pairs && !ragged_waste;
}

int launch_gemm_pair(bool dual, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const GemmParams& p,
                     cudaStream_t stream) {
    return dual ? launch_plain<true>(ta, tb, tb2, p, stream) : launch_plain<false>(ta, tb, tb2, p, stream);
}

int max_pairs_grouped(int dev) { return dev < 64 ? max_pairs<false, true, false>(dev) : -1; }

int launch_gemm_pair_grouped(const GemmParams& p, cudaStream_t stream) {
    // the kernel takes its maps from the table; the six map parameters only have to be valid objects
    static const CUtensorMap dummy = {};
    return launch<false, true, false>(dummy, dummy, dummy, dummy, dummy, dummy, p, p.total_tiles, stream);
}

// Called by nvfp4_shutdown(): the stream-K scratch of every device (the caller has synchronised its streams).
void free_stream_k_scratch() {
    std::lock_guard<std::mutex> lk(g_sk_mu);
    int cur = 0;
    if (cudaGetDevice(&cur) != cudaSuccess) return;
    for (int dev = 0; dev < 64; dev++) {
        StreamKState& sk = g_sk[dev];
        if (!sk.scratch && !sk.flags && !sk.done) continue;
        cudaSetDevice(dev);
        if (sk.scratch) cudaFree(sk.scratch);
        if (sk.flags) cudaFree(sk.flags);
        if (sk.done) cudaEventDestroy(sk.done);
        sk = StreamKState();
    }
    cudaSetDevice(cur);
}

}  // namespace nvfp4
