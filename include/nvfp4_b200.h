/*
 * C ABI of libnvfp4_b200: NVFP4 (e2m1 data, one ue4m3 scale per 16 K-elements) kernels for
 * NVIDIA B200 (sm_100a).  Plain pointers and sizes; every pointer is DEVICE memory owned by the
 * caller; every call is asynchronous on the given CUDA stream (a cudaStream_t passed as void*).
 *
 * Each entry point is the native counterpart of one `custom_kernel(data)` of the reference
 * harness (file:line below are paths inside jIab-b/eval_test).  Shared conventions, all taken
 * from the reference's input generators:
 *   - operands: uint8, two e2m1 per byte (element 2i in bits 3..0), K-major rows, batch
 *     outermost in memory: a is [L][M][K/2], b is [L][N][K/2]
 *     (eval/nvfp4_gemm/reference.py:35-38);
 *   - scales: e4m3fn bytes in the swizzled layout of the reference's `*_permuted` tensors
 *     (eval/common/scale_helpers.py:41-68): 512-byte atoms of 128 rows x 4 k-blocks, ordered
 *     [L][ceil(rows/128)][ceil(K/64)], byte (r%32)*16 + ((r%128)/32)*4 + kb%4 inside an atom;
 *     rows are padded to a multiple of 128;
 *   - output: fp16, [L][M][N] (eval/nvfp4_gemm/reference.py:40), fully overwritten;
 *   - inputs are never written; nothing is allocated per call.
 *
 * Return value: 0 on success; < 0 an argument was rejected (NVFP4_ERR_*); > 0 a cudaError_t.
 * A device-side wait that runs out of its budget (a pipeline fault) does not hang: the kernel
 * returns and leaves a code >= 101 in the per-device status word read by nvfp4_device_status().
 */
#ifndef NVFP4_B200_H
#define NVFP4_B200_H

#ifdef __cplusplus
extern "C" {
#endif

#define NVFP4_ABI_VERSION 1

enum {
    NVFP4_OK = 0,
    NVFP4_ERR_NULL = -1,
    NVFP4_ERR_SHAPE = -2,
    NVFP4_ERR_K_MULTIPLE = -3,
    NVFP4_ERR_N_MULTIPLE = -4,
    NVFP4_ERR_ALIGN = -5,
    NVFP4_ERR_UNSUPPORTED = -6,
    NVFP4_ERR_TENSORMAP = -7,
    NVFP4_ERR_INTERNAL = -8,
    NVFP4_ERR_TOO_MANY_GROUPS = -9
};

/* Batched GEMV  c[l][m] = fp16(alpha * sum_k (a*sfa)[l][m][k] * (x*sfx)[l][k]).
 * Replaces custom_kernel of eval/nvfp4_gemv/submission.py:28-54 (tuple of
 * eval/nvfp4_gemv/reference.py:31-49): x is the reference's `b` operand, [L][x_rows][K/2] with the
 * vector in row 0 (x_rows = 128 there), sfx_sw its swizzled scales; c is [L][M].
 * K % 64 == 0 (any K: few 128-row tiles with K <= 65536 take the decode kernel, everything else the tensor-core
 * streaming kernel, which has no K limit); a, x, scales 16-byte aligned. */
int nvfp4_gemv(const void* a, const void* x, const void* sfa_sw, const void* sfx_sw, void* c,
               int M, int K, int L, int x_rows, float alpha, void* stream);

/* GEMM  c[l] = fp16(alpha * (a*sfa)[l] @ (b*sfb)[l]^T).
 * Replaces custom_kernel of eval/nvfp4_gemm/submission.py:708-761 (tuple of
 * eval/nvfp4_gemm/reference.py:31-46).  N % 128 == 0, K % 256 == 0; M arbitrary (> 0). */
int nvfp4_gemm(const void* a, const void* b, const void* sfa_sw, const void* sfb_sw, void* c,
               int M, int N, int K, int L, float alpha, void* stream);

/* Dual GEMM with SiLU gating  c[l] = fp16( silu(alpha * A@B1^T) * (alpha * A@B2^T) ).
 * Replaces custom_kernel of eval/nvfp4_dual_gemm/submission.py:894-957 (tuple of
 * eval/nvfp4_dual_gemm/reference.py:48-73).  N % 128 == 0, K % 256 == 0. */
int nvfp4_dual_gemm(const void* a, const void* b1, const void* b2, const void* sfa_sw,
                    const void* sfb1_sw, const void* sfb2_sw, void* c,
                    int M, int N, int K, int L, float alpha, void* stream);

/* The same dual GEMM with the result emitted as NVFP4, ready to be the A operand of the next GEMM (the
 * down-projection of an MLP): c_packed [L][M][N/2] e2m1 codes and sfc_sw, their block-16 e4m3 scales in the
 * swizzled layout [L][ceil(M/128)][N/64][512] (rows padded to 128; padding rows are not written).
 * Bit for bit nvfp4_quantize_f32 applied to the fp16 output of nvfp4_dual_gemm.
 * No counterpart in the reference, whose dual GEMM ends in fp16 (eval/nvfp4_dual_gemm/reference.py:11-45).
 * c_packed 32-byte aligned, the rest 16-byte aligned; N % 128 == 0, K % 256 == 0. */
int nvfp4_dual_gemm_nvfp4(const void* a, const void* b1, const void* b2, const void* sfa_sw,
                          const void* sfb1_sw, const void* sfb2_sw, void* c_packed, void* sfc_sw,
                          int M, int N, int K, int L, float alpha, void* stream);

/* N-sharded GEMM / dual GEMM with the all-gather of the output fused into the epilogue: this rank computes the
 * columns [rank*N_local, (rank+1)*N_local) of C and stores every piece of them into the full C buffer
 * [L][M][N_local*world] of EVERY rank: c_all[r] is rank r's buffer as mapped into this process (peer memory:
 * symmetric memory or an IPC mapping; c_all[rank] is the local one), 32-byte aligned; world <= 8.  Asynchronous bulk
 * tensor stores (TMA stores, no multicast) out of shared memory over NVLink, no collective call.  The caller provides two orderings across ranks: "all ranks have finished" (a
 * barrier on the stream) before C is read, and "all ranks' readers have finished" (a second barrier, or a second
 * buffer used in alternation) before the next call into the same buffers - a rank that has passed the first
 * barrier would otherwise overwrite a copy that a peer is still reading.
 * No counterpart in the reference (a single-GPU harness); replaces gemm + ncclAllGather of the column shards. */
int nvfp4_gemm_allgather(const void* a, const void* b, const void* sfa_sw, const void* sfb_sw,
                         void* const* c_all, int world, int rank, int M, int N_local, int K, int L,
                         float alpha, void* stream);
int nvfp4_dual_gemm_allgather(const void* a, const void* b1, const void* b2, const void* sfa_sw,
                              const void* sfb1_sw, const void* sfb2_sw, void* const* c_all, int world,
                              int rank, int M, int N_local, int K, int L, float alpha, void* stream);

/* One problem of a grouped GEMM (L = 1): c[M][N] = fp16(alpha * (a*sfa) @ (b*sfb)^T). */
typedef struct nvfp4_group {
    const void* a;       /* [M][K/2] */
    const void* b;       /* [N][K/2] */
    const void* sfa_sw;  /* swizzled, rows padded to 128 */
    const void* sfb_sw;
    void* c;             /* [M][N] fp16 */
    int M, N, K;         /* M >= 0 (empty groups are skipped), N % 128 == 0, K % 256 == 0 */
    int reserved;
} nvfp4_group_t;

/* Grouped GEMM over a HOST array of G problem descriptors (device pointers inside).
 * Replaces custom_kernel + grouped_gemm_launch of
 * eval/nvfp4_grouped_gemm/submission.py:1045-1155,1196-1237 (tuple of
 * eval/nvfp4_grouped_gemm/reference.py:137-201). */
int nvfp4_grouped_gemm(const nvfp4_group_t* groups, int G, float alpha, void* stream);

/* The same grouped GEMM for callers that must not let the library allocate memory (a process whose own
 * allocator already owns all of HBM; a loop that cannot afford the device-wide synchronisation of
 * cudaMalloc / cudaFree).  Same arguments and results as nvfp4_grouped_gemm.  No counterpart in the reference.
 *  - The problem table lives in ONE fixed device array inside the library image (80 KB, held by every GPU that
 *    loads the library until the process exits): at most 256 non-empty groups per call, more are refused with
 *    NVFP4_ERR_TOO_MANY_GROUPS.
 *  - It calls no cudaMalloc / cudaFree / cudaHostAlloc and creates no events.  The first call on a device
 *    resolves the array's device address; make that call before any stream capture.  A call on a stream that is
 *    being captured is refused with NVFP4_ERR_UNSUPPORTED (the table upload reads a host image that later calls
 *    rewrite, so a recorded copy of it could not be replayed faithfully).
 *  - Every call rewrites the same array (the previous call's entries stay behind, only the first `live`
 *    entries are read): calls that overlap on the GPU - different streams - race; keep them on one stream or
 *    order them yourself.
 *  - A device-side wait that expires is recorded only if an earlier call of another entry point has already
 *    created the device's status word; the kernel still returns instead of hanging. */
int nvfp4_grouped_gemm_noalloc(const nvfp4_group_t* groups, int G, float alpha, void* stream);

/* fp32 -> NVFP4 quantiser (the step in front of the path; the reference has no counterpart, its generators draw
 * bit patterns, eval/nvfp4_gemm/reference.py:35-38): x is [L][rows][K] fp32 row-major; writes packed e2m1
 * [L][rows][K/2] and the e4m3 block scales (amax/6, RNE) directly in the swizzled layout (rows padded to 128,
 * padding zeroed).  K % 16 == 0; x 16-byte, packed 8-byte, sf_sw 4-byte aligned. */
int nvfp4_quantize_f32(const void* x, void* packed, void* sf_sw, int rows, int K, int L, void* stream);
/* The same for fp16 and bf16 activations (widened to fp32 exactly, then the same rule). */
int nvfp4_quantize_f16(const void* x, void* packed, void* sf_sw, int rows, int K, int L, void* stream);
int nvfp4_quantize_bf16(const void* x, void* packed, void* sf_sw, int rows, int K, int L, void* stream);

/* Last device-side status code of device `dev` (0 = none); clear != 0 resets it.
 * Call after synchronising the stream.  No counterpart in the reference, whose kernels spin
 * without bound (eval/nvfp4_grouped_gemm/submission.py:91-104). */
int nvfp4_device_status(int dev, int clear);

/* Launches a one-thread kernel that waits on a barrier nothing arrives on, with a budget of
 * budget_ms (1..2000): the wait must expire, leave status 105 and return.  Synchronises the stream.
 * No counterpart in the reference. */
int nvfp4_wait_selftest(int budget_ms, double* elapsed_ms, void* stream);

/* Frees the memory the library allocated on first use (grouped-GEMM problem tables, status words).  Synchronise
 * the streams first; later calls allocate again.  The reference frees per call instead (eight cudaMalloc /
 * cudaFree pairs in grouped_gemm_launch, eval/nvfp4_grouped_gemm/submission.py:1111-1152). */
int nvfp4_shutdown(void);

/* Text for any value returned by the functions above or by nvfp4_device_status(). */
const char* nvfp4_strerror(int code);

int nvfp4_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* NVFP4_B200_H */
