/*
 * CPU oracle for the NVFP4 hot path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of what the reference computes for its four problems
 * (block-scaled FP4 GEMV, GEMM, dual GEMM with SiLU gating, grouped GEMM).
 * Only the parity tests, the smoke check and the CPU-baseline leg of the bench
 * may call it; the shipped library never does.
 *
 * The reference has no CPU implementation of this arithmetic: every
 * ref_kernel hands the packed operands to torch._scaled_mm (cuBLASLt, closed
 * source; the reference pins no version beyond its container image
 * pytorch/pytorch:2.9.1-cuda13.0, modal/app.py:13).  What is restated here is
 * therefore the published NVFP4 definition anchored on the reference's call
 * sites:
 *   - operand meaning and transposition  eval/nvfp4_gemm/reference.py:16-27
 *       C[m,n,l] = sum_k (a[m,k,l]*sfa[m,k/16,l]) * (b[n,k,l]*sfb[n,k/16,l])
 *   - GEMV = column 0 of a GEMM against a 128-row padded vector
 *                                         eval/nvfp4_gemv/reference.py:19-27,35-39
 *   - dual GEMM epilogue silu(r1)*r2 in fp32, one cast to fp16
 *                                         eval/nvfp4_dual_gemm/reference.py:24-44
 *   - grouped GEMM = independent problems, L = 1
 *                                         eval/nvfp4_grouped_gemm/reference.py:48-74
 *   - block size 16                       eval/common/scale_helpers.py:3
 *   - swizzled scale layout               eval/common/scale_helpers.py:10-17,41-68
 *   - tensor strides (K-major rows, batch outermost in memory)
 *                                         eval/nvfp4_gemm/reference.py:35-40
 * Parity status: the reference holds no stored golden vectors for this path
 * ("parity unpinned" in the stored-vector sense).  The pins that exist are
 * committed under tests/golden/: the scale-layout permutation produced by the
 * reference's own to_blocked(), and outputs of torch._scaled_mm recorded on a
 * B200 with the reference's call signature.
 *
 * Arithmetic: inside one 16-element block the products 2a*2b are small
 * integers, so the block dot product is computed exactly in int32; it is
 * scaled by sfa*sfb and accumulated in fp32 in ascending-k order; alpha is
 * applied in fp32; one round-to-nearest-even cast to fp16.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define SF_VEC 16

/* twice the e2m1 magnitude for the 3-bit code e1 e0 m: {0,.5,1,1.5,2,3,4,6}*2 */
static const int8_t E2M1_X2[8] = {0, 1, 2, 3, 4, 6, 8, 12};

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* e2m1 nibble (s e1 e0 m) -> value */
float oracle_e2m1_decode(unsigned code) {
    float v = 0.5f * (float)E2M1_X2[code & 7];
    return (code & 8) ? -v : v;
}

/* e4m3fn byte (s eeee mmm, bias 7, subnormals, no inf, NaN = S.1111.111) */
float oracle_e4m3_decode(unsigned byte) {
    unsigned s = (byte >> 7) & 1, e = (byte >> 3) & 15, m = byte & 7;
    float v;
    if (e == 15 && m == 7) return NAN;
    if (e == 0) v = ldexpf((float)m, -9);
    else        v = ldexpf((float)(8 + m), (int)e - 10);
    return s ? -v : v;
}

/* Byte offset of scale (row r, k-block kb, batch l) in the swizzled layout:
 * 512-byte atoms of 128 rows x 4 k-blocks, atoms ordered [l][r/128][kb/4]. */
size_t oracle_sf_offset(int r, int kb, int l, int rows, int K) {
    size_t R = (size_t)((rows + 127) / 128);
    size_t Kb = (size_t)(((K / SF_VEC) + 3) / 4);
    return (size_t)l * R * Kb * 512 + (size_t)(r / 128) * Kb * 512 + (size_t)(kb / 4) * 512
         + (size_t)(r % 32) * 16 + (size_t)((r % 128) / 32) * 4 + (size_t)(kb % 4);
}

static uint16_t f32_to_f16_bits(float f) {
    _Float16 h = (_Float16)f; /* round to nearest even */
    uint16_t u;
    memcpy(&u, &h, 2);
    return u;
}

/* rows x K nibbles -> rows x K int8 holding 2*value (element 2i = low nibble of byte i) */
static void decode_x2(const uint8_t *p, int8_t *out, size_t rows, size_t K) {
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; r++) {
        const uint8_t *src = p + r * (K / 2);
        int8_t *dst = out + r * K;
        for (size_t i = 0; i < K / 2; i++) {
            unsigned b = src[i];
            int8_t lo = E2M1_X2[b & 7], hi = E2M1_X2[(b >> 4) & 7];
            dst[2 * i] = (b & 8) ? (int8_t)-lo : lo;
            dst[2 * i + 1] = (b & 0x80) ? (int8_t)-hi : hi;
        }
    }
}

/* swizzled scales of one batch -> row-major float [rows][K/16] */
static void decode_sf(const uint8_t *sf_sw, float *out, int rows, int K, int l) {
    int kbs = K / SF_VEC;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++)
        for (int kb = 0; kb < kbs; kb++)
            out[(size_t)r * kbs + kb] = oracle_e4m3_decode(sf_sw[oracle_sf_offset(r, kb, l, rows, K)]);
}

/* acc[m][n] = sum_kb sfa*sfb * (exact int block dot)/4, fp32, ascending kb */
static void block_scaled_mm(const int8_t *A, const float *SA, const int8_t *B, const float *SB,
                            float *acc, int M, int N, int K) {
    int kbs = K / SF_VEC;
#pragma omp parallel for schedule(dynamic, 4)
    for (int m = 0; m < M; m++) {
        const int8_t *ar = A + (size_t)m * K;
        const float *sa = SA + (size_t)m * kbs;
        for (int n = 0; n < N; n++) {
            const int8_t *br = B + (size_t)n * K;
            const float *sb = SB + (size_t)n * kbs;
            float s = 0.f;
            for (int kb = 0; kb < kbs; kb++) {
                int d = 0;
                for (int j = 0; j < SF_VEC; j++) d += (int)ar[kb * SF_VEC + j] * (int)br[kb * SF_VEC + j];
                s += (sa[kb] * sb[kb]) * (0.25f * (float)d);
            }
            acc[(size_t)m * N + n] = s;
        }
    }
}

/* GEMM.  a:[L][M][K/2]  b:[L][N][K/2]  sfa_sw,sfb_sw: swizzled  c:[L][M][N] fp16 bits.
 * sfa_rows / sfb_rows: row counts the swizzled buffers were built for (>= M, N). */
int oracle_gemm(const uint8_t *a, const uint8_t *b, const uint8_t *sfa_sw, const uint8_t *sfb_sw,
                uint16_t *c, int M, int N, int K, int L, float alpha) {
    if (M < 0 || N <= 0 || K <= 0 || K % SF_VEC || L <= 0) return -1;
    if (M == 0) return 0;
    int kbs = K / SF_VEC;
    int8_t *A = malloc((size_t)M * K), *B = malloc((size_t)N * K);
    float *SA = malloc(sizeof(float) * (size_t)M * kbs), *SB = malloc(sizeof(float) * (size_t)N * kbs);
    float *acc = malloc(sizeof(float) * (size_t)M * N);
    if (!A || !B || !SA || !SB || !acc) { free(A); free(B); free(SA); free(SB); free(acc); return -2; }
    for (int l = 0; l < L; l++) {
        decode_x2(a + (size_t)l * M * (K / 2), A, M, K);
        decode_x2(b + (size_t)l * N * (K / 2), B, N, K);
        decode_sf(sfa_sw, SA, M, K, l);
        decode_sf(sfb_sw, SB, N, K, l);
        block_scaled_mm(A, SA, B, SB, acc, M, N, K);
        uint16_t *cl = c + (size_t)l * M * N;
        for (size_t i = 0; i < (size_t)M * N; i++) cl[i] = f32_to_f16_bits(alpha * acc[i]);
    }
    free(A); free(B); free(SA); free(SB); free(acc);
    return 0;
}

/* Dual GEMM: c = fp16( silu(alpha*A.B1) * (alpha*A.B2) ), silu(x) = x / (1 + exp(-x)) in fp32 */
int oracle_dual_gemm(const uint8_t *a, const uint8_t *b1, const uint8_t *b2, const uint8_t *sfa_sw,
                     const uint8_t *sfb1_sw, const uint8_t *sfb2_sw, uint16_t *c,
                     int M, int N, int K, int L, float alpha) {
    if (M <= 0 || N <= 0 || K <= 0 || K % SF_VEC || L <= 0) return -1;
    int kbs = K / SF_VEC;
    int8_t *A = malloc((size_t)M * K), *B = malloc((size_t)N * K);
    float *SA = malloc(sizeof(float) * (size_t)M * kbs), *SB = malloc(sizeof(float) * (size_t)N * kbs);
    float *r1 = malloc(sizeof(float) * (size_t)M * N), *r2 = malloc(sizeof(float) * (size_t)M * N);
    if (!A || !B || !SA || !SB || !r1 || !r2) { free(A); free(B); free(SA); free(SB); free(r1); free(r2); return -2; }
    for (int l = 0; l < L; l++) {
        decode_x2(a + (size_t)l * M * (K / 2), A, M, K);
        decode_sf(sfa_sw, SA, M, K, l);
        decode_x2(b1 + (size_t)l * N * (K / 2), B, N, K);
        decode_sf(sfb1_sw, SB, N, K, l);
        block_scaled_mm(A, SA, B, SB, r1, M, N, K);
        decode_x2(b2 + (size_t)l * N * (K / 2), B, N, K);
        decode_sf(sfb2_sw, SB, N, K, l);
        block_scaled_mm(A, SA, B, SB, r2, M, N, K);
        uint16_t *cl = c + (size_t)l * M * N;
#pragma omp parallel for schedule(static)
        for (size_t i = 0; i < (size_t)M * N; i++) {
            float x = alpha * r1[i], y = alpha * r2[i];
            float silu = x / (1.0f + expf(-x));
            cl[i] = f32_to_f16_bits(silu * y);
        }
    }
    free(A); free(B); free(SA); free(SB); free(r1); free(r2);
    return 0;
}

/* GEMV.  a:[L][M][K/2]  x:[L][x_rows][K/2] (row 0 is the vector)  c:[L][M] fp16 bits.
 * sfx_sw is the swizzled scale buffer of the x_rows-row padded vector operand. */
int oracle_gemv(const uint8_t *a, const uint8_t *x, const uint8_t *sfa_sw, const uint8_t *sfx_sw,
                uint16_t *c, int M, int K, int L, int x_rows, float alpha) {
    if (M <= 0 || K <= 0 || K % SF_VEC || L <= 0 || x_rows <= 0) return -1;
    int kbs = K / SF_VEC;
    int8_t *X = malloc((size_t)K);
    float *SX = malloc(sizeof(float) * (size_t)kbs);
    if (!X || !SX) { free(X); free(SX); return -2; }
    for (int l = 0; l < L; l++) {
        decode_x2(x + (size_t)l * x_rows * (K / 2), X, 1, K);
        for (int kb = 0; kb < kbs; kb++) SX[kb] = oracle_e4m3_decode(sfx_sw[oracle_sf_offset(0, kb, l, x_rows, K)]);
        const uint8_t *al = a + (size_t)l * M * (K / 2);
#pragma omp parallel for schedule(static)
        for (int m = 0; m < M; m++) {
            const uint8_t *row = al + (size_t)m * (K / 2);
            float s = 0.f;
            for (int kb = 0; kb < kbs; kb++) {
                int d = 0;
                for (int j = 0; j < SF_VEC / 2; j++) {
                    unsigned by = row[kb * 8 + j];
                    int lo = E2M1_X2[by & 7], hi = E2M1_X2[(by >> 4) & 7];
                    if (by & 8) lo = -lo;
                    if (by & 0x80) hi = -hi;
                    d += lo * X[kb * 16 + 2 * j] + hi * X[kb * 16 + 2 * j + 1];
                }
                float sa = oracle_e4m3_decode(sfa_sw[oracle_sf_offset(m, kb, l, M, K)]);
                s += (sa * SX[kb]) * (0.25f * (float)d);
            }
            c[(size_t)l * M + m] = f32_to_f16_bits(alpha * s);
        }
    }
    free(X); free(SX);
    return 0;
}

/* Dequantise one operand: p:[L][rows][K/2] packed e2m1, sf_sw swizzled e4m3 scales -> out:[L][rows][K] fp32
 * (value * scale of its 16-element block).  First half of the "dequantise, then fp32 matmul" route, the shape of
 * computation the reference's oracle has on the GPU (eval/nvfp4_gemm/reference.py:16-27); the matmul half is a
 * library fp32 GEMM called from nvfp4_oracle.py. */
int oracle_dequant(const uint8_t *p, const uint8_t *sf_sw, float *out, int rows, int K, int L) {
    if (rows <= 0 || K <= 0 || K % SF_VEC || L <= 0) return -1;
    static const float LUT[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};
    int kbs = K / SF_VEC;
    for (int l = 0; l < L; l++) {
#pragma omp parallel for schedule(static)
        for (int r = 0; r < rows; r++) {
            const uint8_t *src = p + ((size_t)l * rows + r) * (K / 2);
            float *dst = out + ((size_t)l * rows + r) * K;
            for (int kb = 0; kb < kbs; kb++) {
                float s = oracle_e4m3_decode(sf_sw[oracle_sf_offset(r, kb, l, rows, K)]);
                for (int j = 0; j < SF_VEC / 2; j++) {
                    unsigned b = src[kb * 8 + j];
                    dst[kb * 16 + 2 * j] = LUT[b & 15] * s;
                    dst[kb * 16 + 2 * j + 1] = LUT[b >> 4] * s;
                }
            }
        }
    }
    return 0;
}
