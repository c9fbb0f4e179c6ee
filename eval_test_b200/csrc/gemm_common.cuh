// Declarations shared by the tcgen05 GEMM kernels (one CTA per tile, and CTA pairs): launch parameters, the
// grouped-GEMM problem table entry, tile location and the epilogue.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "nvfp4_internal.h"
#include "ptx_sm100.cuh"
#include "quant_block.cuh"

namespace nvfp4 {

constexpr int BM = 128;        // rows of A per tile = TMEM lanes
constexpr int BK = 256;        // K elements per stage = 128 bytes per row = one swizzle atom
constexpr int GEMM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;

// One problem of a grouped GEMM as the kernel sees it (an array of these lives in device memory).
struct alignas(64) GroupEntry {
    CUtensorMap ta, tb;   // operand maps of this group (A: box 128 rows, B: box BN rows)
    const uint8_t* sfa;
    const uint8_t* sfb;
    __half* c;            // [M][N]
    int M, N, K;
    int tile_start;       // index of this group's first tile in the launch-wide tile order
    int tiles_m, tiles_n;
};

// One problem of a grouped GEMM as the CTA-pair kernel sees it: its tiles are 256 x 256, the B map has 128-row
// boxes (each CTA of a pair keeps half a B tile) and the scales come through tensor maps too.
struct alignas(64) PairGroupEntry {
    CUtensorMap ta, tb, tsa, tsb;
    __half* c;            // [M][N]
    int M, N, K;
    int tile_start;       // index of this group's first pair tile in the launch-wide tile order
    int tiles_m, tiles_n; // ceil(M / 256), N / 256
};

// Fused all-gather of an N-sharded GEMM: every output tile is stored into the full C buffer of every rank (peer
// memory mapped into this process) by asynchronous bulk tensor stores out of shared memory, one per rank, so that
// the warps that drain the accumulators do not wait for NVLink (8192^3 on 2 GPUs: 154 us per step against 175 us with
// plain stores issued by those warps).  What is left is in the memory system: while a tile's stores are on their way
// the operand loads of the same SM arrive later (the MMA issuer waits twice as long for its stages); four separate
// sending warps with plain stores behaved the same, and so did pacing them.
#ifndef NVFP4_GATHER_BOXES
#define NVFP4_GATHER_BOXES 2
#endif
constexpr int GATHER_BOXES = NVFP4_GATHER_BOXES;   // 4 KB boxes per epilogue warp, filled in turn

struct GatherOut {
    int n = 0;                  // ranks (0: not a gathering launch)
#ifdef NVFP4_PROFILE
    unsigned mask = 0xffu;      // ranks whose copy is actually stored (timing experiments)
#endif
    int ldc = 0;                // row pitch of the full C in elements (N of all ranks together)
    int col0 = 0;               // first column of this rank's slice
};

// One tensor map per rank over its full C, [L][M][ldc] fp16, box 64 columns x 32 rows, 128-byte swizzle: a kernel
// parameter of the gathering instantiations only.
struct GatherMaps { CUtensorMap m[8]; };
struct NoGatherMaps { int unused; };
template <bool GATHER> struct GatherMapsOf { using type = NoGatherMaps; };
template <> struct GatherMapsOf<true> { using type = GatherMaps; };

// What one epilogue warp needs for a gathering store: the maps, GATHER_BOXES x 4 KB of shared memory of its own (1024-byte
// aligned; a box of 32 rows x 128 bytes each, filled in turn) and where its rows are in the full C.
struct GatherCtx {
    const CUtensorMap* maps;
    int n;                 // ranks
    uint4* stage;          // the warp's 8 KB ...
    uint32_t stage_smem;   // ... and their shared-memory address
    uint32_t uses;         // boxes filled so far by this warp (modulo GATHER_BOXES picks the box)
    int x, y, z;           // the tile's first column in the full C, the warp's first row, the batch
    bool rows_exist;       // the warp's first row is inside M (the store clips the rest)
#ifdef NVFP4_PROFILE
    unsigned mask;
    __device__ bool enabled(int r) const { return (mask >> r) & 1u; }
#else
    __device__ bool enabled(int) const { return true; }
#endif
    int cc;                // chunk of the tile being stored
};

struct GemmParams {
    const uint8_t* sfa;   // swizzled scales of A  [L][ceil(M/128)][K/64][512]
    const uint8_t* sfb;   // swizzled scales of B (B1 for the dual GEMM)
    const uint8_t* sfb2;  // swizzled scales of B2 (dual GEMM only)
    __half* c;            // [L][M][N]
    uint8_t* cq = nullptr;   // NVFP4 output instead of fp16: packed e2m1 [L][M][N/2] ...
    uint8_t* sfc = nullptr;  // ... and its block scales, swizzled [L][ceil(M/128)][N/64][512]
    GatherOut gather;
    int M, N, K, L;
    float alpha;
    int* status;
    unsigned long long budget_ns;
    const GroupEntry* table;  // grouped GEMM only: G entries, empty groups left out
    const void* pair_table = nullptr;  // grouped GEMM on CTA pairs: G PairGroupEntry
    float* sk_scratch = nullptr;       // stream-K: one partial accumulator (2 CTAs x 128 rows x 256 fp32) per pair
    unsigned int* sk_flags = nullptr;  // stream-K: [pair][8 epilogue warps of the pair] = epoch once the partial is written
    unsigned int sk_epoch = 0;
    int G;
    int total_tiles;
#ifdef NVFP4_PROFILE
    unsigned long long* prof = nullptr;  // per CTA: cycles the MMA issuer spent waiting for accumulators / for data / in total
#endif
};

#ifdef NVFP4_PROFILE
#define PROF_T0() const long long prof_t0_ = clock64()
#define PROF_ADD(var) var += clock64() - prof_t0_
#else
#define PROF_T0()
#define PROF_ADD(var)
#endif

// Everything a role needs to know about one output tile.
struct TileInfo {
    const CUtensorMap *ta, *tb, *tb2;
    const uint8_t *sfa_t;     // scale block row of this tile's A rows (k = 0)
    const uint8_t *sfb_t;     // scale block row of this tile's first 128 B rows (k = 0)
    const uint8_t *sfb2_t;
    __half* c;                // output of this problem / batch
    size_t sf_row_block;      // bytes of one 128-row scale block = K/64 * 512
    int M, N, kiters, l, m0, n0, nb_valid;
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

// silu(x) * y with the fast exponential and the approximate (2 ulp) division: an IEEE division here made the dual
// GEMM's epilogue three times longer than its main loop; the result is rounded to fp16 anyway.
__device__ __forceinline__ float silu_mul(float x, float y) { return __fdividef(x, 1.0f + __expf(-x)) * y; }

// Tile t of a plain / dual GEMM (all batches share the maps; the batch is the third TMA coordinate) or of a
// grouped GEMM (binary search of the group whose tile range holds t; column tile fastest inside a group).
template <int BN, bool DUAL, bool GROUPED>
__device__ __forceinline__ TileInfo locate(int t, const GemmParams& p, const CUtensorMap* ta, const CUtensorMap* tb,
                                           const CUtensorMap* tb2) {
    constexpr int NB_BLOCKS = (DUAL ? 2 * BN : BN) / 128;
    TileInfo ti;
    if (GROUPED) {
        int lo = 0, hi = p.G - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (__ldg(&p.table[mid].tile_start) <= t) lo = mid; else hi = mid - 1;
        }
        const GroupEntry* e = p.table + lo;
        // Column tile fastest inside a group: first every column tile of the first 128 rows, then of the next 128, ...
        // The row tiles of one column tile still run within one round of CTAs of each other, so the weights come from
        // HBM once.  (With the row tile fastest and an even number of tiles in every group, CTAs with an even index
        // got every first-row tile - the ones that stream the weights from HBM, about twice as long - and the odd ones
        // the cheap remainder tiles: half the machine idled at the end of an expert layer.)
        const int r = t - __ldg(&e->tile_start);
        const int tiles_n = __ldg(&e->tiles_n);
        const int mt = r / tiles_n, nt = r - mt * tiles_n;
        ti.ta = &e->ta; ti.tb = &e->tb; ti.tb2 = &e->tb;
        ti.M = __ldg(&e->M); ti.N = __ldg(&e->N);
        const int K = __ldg(&e->K);
        ti.kiters = K / BK;
        ti.sf_row_block = (size_t)(K / 64) * 512;
        ti.l = 0; ti.m0 = mt * BM; ti.n0 = nt * BN;
        ti.sfa_t = e->sfa + (size_t)mt * ti.sf_row_block;
        ti.sfb_t = e->sfb + (size_t)(ti.n0 / 128) * ti.sf_row_block;
        ti.sfb2_t = nullptr;
        ti.c = e->c;
        ti.nb_valid = min(NB_BLOCKS, ti.N / 128 - ti.n0 / 128);
    } else {
        const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
        const TileCoord tc = tile_coord(t, tiles_m, tiles_n);
        const int RB = p.N / 128;
        ti.ta = ta; ti.tb = tb; ti.tb2 = tb2;
        ti.M = p.M; ti.N = p.N; ti.kiters = p.K / BK;
        ti.sf_row_block = (size_t)(p.K / 64) * 512;
        ti.l = tc.l; ti.m0 = tc.mt * BM; ti.n0 = tc.nt * BN;
        ti.sfa_t = p.sfa + ((size_t)tc.l * tiles_m + tc.mt) * ti.sf_row_block;
        const size_t blk = (size_t)tc.l * RB + ti.n0 / 128;
        ti.sfb_t = p.sfb + blk * ti.sf_row_block;
        ti.sfb2_t = DUAL ? p.sfb2 + blk * ti.sf_row_block : nullptr;
        ti.c = p.c + (size_t)tc.l * p.M * p.N;
        ti.nb_valid = DUAL ? NB_BLOCKS : min(NB_BLOCKS, RB - ti.n0 / 128);
    }
    return ti;
}

// fp32 accumulator chunk(s) -> 32 fp16 outputs of one row, written as two whole 32-byte sectors
// (16-byte stores left half-written sectors behind and cost 35 us at 8192^3).
// GATHER: dst is unused and pred only says that the columns exist; the warp's rows go through shared memory and
// from there, as boxes of 32 rows x 128 bytes, into every rank's C (see GatherCtx).
template <bool DUAL, bool GATHER = false>
__device__ __forceinline__ void store_chunk(__half* dst, const uint32_t (&v)[32], const uint32_t (&w)[32], float alpha,
                                            bool pred, const GatherCtx* gc = nullptr) {
    uint32_t o[16];
#pragma unroll
    for (int i = 0; i < 16; i++) {
        __half2 h;
        if (DUAL) {
            const float x0 = alpha * __uint_as_float(v[2 * i]), x1 = alpha * __uint_as_float(v[2 * i + 1]);
            const float y0 = alpha * __uint_as_float(w[2 * i]), y1 = alpha * __uint_as_float(w[2 * i + 1]);
            h = __floats2half2_rn(silu_mul(x0, y0), silu_mul(x1, y1));
        } else {
            h = __floats2half2_rn(alpha * __uint_as_float(v[2 * i]), alpha * __uint_as_float(v[2 * i + 1]));
        }
        o[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    if (GATHER) {
        // Two chunks (128 bytes of every row) are collected in one of the warp's two 4 KB boxes, 16-byte pieces
        // XOR-swizzled by the row exactly as the 128-byte swizzle of the tensor maps expects (and so that the
        // row-wise writes use every bank); then one lane per rank issues the bulk tensor store of the box into that
        // rank's C.  The stores run on their own: the warp goes back to the accumulator, and comes back to a box
        // only after the stores that read it two boxes ago have done so.
        GatherCtx& g = *const_cast<GatherCtx*>(gc);
        const int lane = threadIdx.x & 31;
        const int half = g.cc & 1;
        const uint32_t b = g.uses % (uint32_t)GATHER_BOXES;
        uint4* st = g.stage + b * 256;
        if (!half && g.uses >= (uint32_t)GATHER_BOXES) {
            if (lane < g.n) tma_store_wait_read<GATHER_BOXES - 1>();
            __syncwarp();
        }
#pragma unroll
        for (int j = 0; j < 4; j++)
            st[lane * 8 + ((4 * half + j) ^ (lane & 7))] = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
        if (!half) return;
        fence_proxy_async_smem();   // the box was written by ordinary stores, the bulk store reads it as the async proxy
        __syncwarp();
        if (lane < g.n) {
            if (pred && g.rows_exist && g.enabled(lane))
                tma_store_3d(&g.maps[lane], g.stage_smem + b * 4096u, g.x + (g.cc >> 1) * 64, g.y, g.z);
            tma_store_commit();      // (also when nothing was stored: the count of groups is what picks the box)
        }
        g.uses++;
        return;
    }
    if (pred) {
        const uint32_t lo[8] = {o[0], o[1], o[2], o[3], o[4], o[5], o[6], o[7]};
        const uint32_t hi[8] = {o[8], o[9], o[10], o[11], o[12], o[13], o[14], o[15]};
        // written once, never read by this kernel: evict-first keeps the operands in L2 instead
        const uint64_t pol = policy_evict_first();
        st_global_256_hint(dst, lo, pol);
        st_global_256_hint(dst + 16, hi, pol);
    }
}

// NVFP4 output: where one thread (one row) puts the packed codes and scale bytes of the tile, and the first
// chunk of a pair of 32-column chunks, held until the second one completes a 32-byte sector and a 4-byte scale group.
struct QuantOut {
    uint8_t* codes;    // the row's packed bytes at the tile's first column
    uint8_t* scales;   // the row's 4-byte group in the scale atom of the tile's first 64 columns
    uint32_t held[5];
};

// 32 results of one row -> fp16 (the rounding of the fp16 output) -> two blocks of NVFP4, exactly what
// nvfp4_quantize_f32 makes of the fp16 output.  Chunk cc of the tile; odd chunks store their pair.
template <bool DUAL>
__device__ __forceinline__ void store_chunk_q(QuantOut& q, int cc, const uint32_t (&v)[32], const uint32_t (&w)[32],
                                              float alpha, bool pred) {
    float f[32];
#pragma unroll
    for (int i = 0; i < 32; i++) {
        const float x = alpha * __uint_as_float(v[i]);
        const float r = DUAL ? silu_mul(x, alpha * __uint_as_float(w[i])) : x;
        f[i] = __half2float(__float2half_rn(r));
    }
    uint32_t a0, a1, b0, b1;
    const uint32_t s0 = quantize_block16(f, a0, a1);
    const uint32_t s1 = quantize_block16(f + 16, b0, b1);
    if ((cc & 1) == 0) {
        q.held[0] = a0; q.held[1] = a1; q.held[2] = b0; q.held[3] = b1;
        q.held[4] = s0 | (s1 << 8);
    } else if (pred) {
        const uint32_t o[8] = {q.held[0], q.held[1], q.held[2], q.held[3], a0, a1, b0, b1};
        st_global_256(q.codes + (cc - 1) * 16, o);
        *reinterpret_cast<uint32_t*>(q.scales + (cc >> 1) * 512) = q.held[4] | (s0 << 16) | (s1 << 24);
    }
}

// Stream-K: when the tiles of a launch do not fill the last round of the machine, the K steps of all tiles form one
// list and every CTA (pair) takes a contiguous share of it, so a tile may be computed by two or more of them.  A
// share that ends inside a tile leaves its fp32 partial accumulator in a scratch slot of its own (mode 1); the
// share that holds the tile's last K step adds the partials in ascending K order to its own accumulator and writes
// the output (mode 2).  A thread owns one accumulator row: `out` / `in[j]` point at that row's 256 floats.
struct SkEpi {
    float* out = nullptr;
    const float* in[8] = {};
    int n_in = 0;
};

// 32 accumulator values of this thread's row -> scratch (whole 32-byte sectors).
__device__ __forceinline__ void sk_store_chunk(float* dst, const uint32_t (&v)[32]) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint32_t w8[8] = {v[8 * j], v[8 * j + 1], v[8 * j + 2], v[8 * j + 3],
                                v[8 * j + 4], v[8 * j + 5], v[8 * j + 6], v[8 * j + 7]};
        st_global_256(dst + 8 * j, w8);
    }
}

// s = (in[0] + in[1]) + ... for 32 columns of this thread's row: the partial sums in the order of their K ranges
// (issued before the accumulator chunk is waited for, so that the two latencies overlap).
__device__ __forceinline__ void sk_load_chunk(float (&s)[32], const SkEpi& sk, int col) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float4 t = __ldcg(reinterpret_cast<const float4*>(sk.in[0] + col) + i);
        s[4 * i] = t.x; s[4 * i + 1] = t.y; s[4 * i + 2] = t.z; s[4 * i + 3] = t.w;
    }
    for (int j = 1; j < sk.n_in; j++) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float4 t = __ldcg(reinterpret_cast<const float4*>(sk.in[j] + col) + i);
            s[4 * i] += t.x; s[4 * i + 1] += t.y; s[4 * i + 2] += t.z; s[4 * i + 3] += t.w;
        }
    }
}
// out = s + own: the finishing share's own K range comes last.
__device__ __forceinline__ void sk_add_chunk(uint32_t (&out)[32], const uint32_t (&own)[32], const float (&s)[32]) {
#pragma unroll
    for (int i = 0; i < 32; i++) out[i] = __float_as_uint(s[i] + __uint_as_float(own[i]));
}

// Epilogue of one tile for one warp (its 32 accumulator rows).  C0 is the first 32-column chunk, relative to
// the accumulator base, that this buffer shares with the other one (OVC chunks; OVC = 0: nothing shared).
// The shared chunks are pulled into registers first and released at once, so the next tile's MMAs wait only
// for those loads, not for the conversion and stores.
// CLUSTER: ovl_free is a shared::cluster address (the barrier may live in the peer CTA).
// QOUT: NVFP4 output through q instead of fp16 through crow.
// GATHER: fp16 output to every rank's buffer (crow unused, see store_chunk and GatherCtx).
// SK: 0 = whole tile; 1 = stream-K partial out (all BN columns as fp32 to sk->out; use BN = 256, DUAL = false);
//     2 = stream-K finish (sk->in partials added before the normal epilogue).
template <int BN, bool DUAL, int C0, int OVC, bool CLUSTER = false, bool QOUT = false, bool GATHER = false, int SK = 0>
__device__ __forceinline__ void epilogue_tile(uint32_t t_lane, __half* crow, bool row_ok, int n0, int N, float alpha,
                                              uint32_t ovl_free, int lane, QuantOut* q = nullptr,
                                              const GatherCtx* gc = nullptr, const SkEpi* sk = nullptr) {
    constexpr int NCH = BN / 32;
    uint32_t ov[OVC > 0 ? OVC : 1][32];
    if (OVC > 0) {
#pragma unroll
        for (int j = 0; j < OVC; j++) tc_ld_32x32(t_lane + (C0 + j) * 32, ov[j]);
        tc_wait_ld();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
            // "these columns have been read" (tcgen05.wait::ld above): no memory of this thread is published, so the
            // signal to the other CTA needs no release (which cost about 1 400 cycles per tile in the pair kernel)
            if (CLUSTER) mbar_arrive_cluster_relaxed(ovl_free);
            else mbar_arrive(ovl_free);
        }
    }
#pragma unroll
    for (int cc = 0; cc < NCH; cc++) {
        constexpr int YOFF = BN / 32;  // dual GEMM: column chunk of the second product
        uint32_t v[32], w[32];
        const bool v_pre = OVC > 0 && cc >= C0 && cc < C0 + OVC;
        const bool w_pre = DUAL && OVC > 0 && cc + YOFF >= C0 && cc + YOFF < C0 + OVC;
        float sx[SK == 2 ? 32 : 1], sy[(SK == 2 && DUAL) ? 32 : 1];
        if (SK == 2) {
            sk_load_chunk(reinterpret_cast<float(&)[32]>(sx), *sk, cc * 32);
            if (DUAL) sk_load_chunk(reinterpret_cast<float(&)[32]>(sy), *sk, (cc + YOFF) * 32);
        }
        if (!v_pre) tc_ld_32x32(t_lane + cc * 32, v);
        if (DUAL && !w_pre) tc_ld_32x32(t_lane + (cc + YOFF) * 32, w);
        if (!v_pre || (DUAL && !w_pre)) tc_wait_ld();
        const bool pred = (GATHER || row_ok) && n0 + cc * 32 < N;
        // (index clamps only keep the never-taken branch in range for the compiler)
        if (SK == 1) {
            sk_store_chunk(sk->out + cc * 32, v_pre ? ov[(cc - C0) < 0 || (cc - C0) >= OVC ? 0 : cc - C0] : v);
            continue;
        }
        if (SK == 2) {
            uint32_t vs[32], ws[32];
            sk_add_chunk(vs, v_pre ? ov[(cc - C0) < 0 || (cc - C0) >= OVC ? 0 : cc - C0] : v,
                         reinterpret_cast<const float(&)[32]>(sx));
            if (DUAL)
                sk_add_chunk(ws, w_pre ? ov[(cc + YOFF - C0) < 0 || (cc + YOFF - C0) >= OVC ? 0 : cc + YOFF - C0] : w,
                             reinterpret_cast<const float(&)[32]>(sy));
            store_chunk<DUAL, false>(crow + cc * 32, vs, ws, alpha, pred);
            continue;
        }
        if (QOUT)
            store_chunk_q<DUAL>(*q, cc, v_pre ? ov[(cc - C0) < 0 || (cc - C0) >= OVC ? 0 : cc - C0] : v,
                                w_pre ? ov[(cc + YOFF - C0) < 0 || (cc + YOFF - C0) >= OVC ? 0 : cc + YOFF - C0] : w, alpha,
                                pred);
        else {
            if (GATHER) const_cast<GatherCtx*>(gc)->cc = cc;
            store_chunk<DUAL, GATHER>(crow + cc * 32, v_pre ? ov[(cc - C0) < 0 || (cc - C0) >= OVC ? 0 : cc - C0] : v,
                          w_pre ? ov[(cc + YOFF - C0) < 0 || (cc + YOFF - C0) >= OVC ? 0 : cc + YOFF - C0] : w, alpha,
                          pred, gc);
        }
    }
}

// Tensor map over a packed-e2m1 operand [L][rows][K/2] (defined in gemm_sm100.cu).
int make_operand_tmap(CUtensorMap* map, const void* base, int rows, int K, int L, int box_rows);
// Tensor map over a swizzled scale buffer seen as rows of one 512-byte atom each: dimensions (64 x 8 bytes, atoms),
// box (64, 4) = the four atoms of one 256-element K step of one 128-row block, which are consecutive in memory.
int make_scale_tmap(CUtensorMap* map, const void* base, long atoms);


// CTA-pair kernels (gemm_pair_sm100.cu).  pair_tiles_wanted(): true when the shape suits them (M >= 256, enough
// 256-row tiles to fill the machine).  launch_gemm_pair(): maps with 128-row boxes.
bool pair_kernel_suits(int M, int N, int K, int L, bool dual, int dev);
int launch_gemm_pair(bool dual, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const GemmParams& p,
                     cudaStream_t stream);
// Grouped GEMM on CTA pairs: p.pair_table (device), p.G entries, p.total_tiles pair tiles.  max_pairs_grouped():
// pairs that can be resident on the device (<= 0: the kernel cannot run there).
int launch_gemm_pair_grouped(const GemmParams& p, cudaStream_t stream);
int max_pairs_grouped(int dev);

// Cluster split-K kernel for few-tile, long-K shapes (gemm_splitk_sm100.cu).  splitk_factor() returns the cluster
// size (2, 4, 8) or 0 when the persistent kernel should be used; maps with 128-row boxes.
int splitk_factor(int M, int N, int K, int L, int dev);
int launch_gemm_splitk(int S, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream);
// The dual GEMM on the same kernel, S = 2 or 4 (both products are reduced across the cluster before silu(x) * y).
int launch_dual_gemm_splitk(int S, const CUtensorMap& ta, const CUtensorMap& tb1, const CUtensorMap& tb2, const GemmParams& p,
                            cudaStream_t stream);

}  // namespace nvfp4
