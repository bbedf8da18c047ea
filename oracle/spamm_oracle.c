/*
 * spamm_oracle.c -- TEST INFRASTRUCTURE, not product code.
 *
 * A plain-C, CPU restatement of the SpAMM algorithm of buaa-hipo/cuSpAMM for
 * the hot path "tile norm map -> per-C-tile skip list -> gated half-precision
 * block multiply".  It is the checker the CUDA path is compared against in the
 * tests, in the smoke run and in the benchmark's CPU-baseline leg; the
 * shipped library never links or calls it.
 *
 * PARITY STATUS: the reference ships no tests, golden vectors or fixtures and its own host loop is commented out
 * (tool.cu:79-126), so no reference TEST pins this restatement.  It is pinned instead on outputs of the
 * reference itself: oracle/build_ref.sh compiles the reference's unmodified kernels for sm_100a into oracle/_ref/,
 * and tests/test_gpu_reference_crosscheck.py runs them on a B200 on the same inputs (get_C_FP16_B32 fed with this
 * checker's norm maps and threshold agrees with oracle_gated_multiply to 2e-6 relative Frobenius error, including
 * the reference's default 2048^3 run; unroll_get_Fnorm_pri agrees with oracle_norm_map to 2e-6).  Further pins,
 * all CPU-only: known-answer cases from the algorithm's definition, numpy restatements of every stage, the
 * committed fixture tests/golden/spamm_small.npz, and the survivor count of the reference's default configuration
 * (12 850 of 262 144).
 *
 * Reference lines each function follows (paths inside the reference project):
 *   norm map layout and definition  cuSpAMM.cu:28-34, 68-70  (sqrt of the sum of squares of a 32x32 tile,
 *                                   row-major (rows/32) x (cols/32) map)
 *   skip rule                       cuSpAMM.cu:302-312 and tool.cu:500-518 (countValid):
 *                                   float product of the two tile norms, kept when  product >= Norm
 *   compaction order                cuSpAMM.cu:315-326 (ascending k)
 *   gated product                   cuSpAMM.cu:357-375, 391 and the authors' host loop tool.cu:84-118:
 *                                   half inputs, float accumulation, C tile is zero when nothing survives
 *   input rounding                  tool.cu:418 (__float2half, round to nearest even)
 *   generators                      tool.cu:409-422 (c * v^|i-j|), tool.cu:426-436 (c / (|i-j|^v + 1))
 *
 * The one place where the reference's arithmetic is NOT imitated: in half mode
 * the reference squares and partially sums in half precision inside
 * unroll_get_Fnorm_FP16 (cuSpAMM.cu:98-102).  The contract here is float norms
 * of the float data, reduced in the fixed order written in spamm_norm_order
 * below, which the CUDA kernel reproduces bit for bit.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see oracle/Makefile).
 * -ffp-contract=off matters: the only fused operations are the explicit fmaf().
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define TILE 32

/* ------------------------------------------------------------------ half */

/* float -> IEEE binary16 bits, round to nearest even (what __float2half does, tool.cu:418). */
uint16_t oracle_f2h_bits(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) {                      /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | ((ax > 0x7f800000u) ? 0x0200u : 0u));
    }
    if (ax >= 0x477ff000u) {                      /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (ax < 0x33000001u) {                       /* <= 2^-25 -> +-0 (ties to even gives 0 at exactly 2^-25) */
        return (uint16_t)sign;
    }
    int32_t e = (int32_t)(ax >> 23) - 127;        /* unbiased exponent */
    uint32_t m = (ax & 0x7fffffu) | 0x800000u;    /* 24-bit significand */
    int shift;
    uint32_t hexp;
    if (e >= -14) {                               /* normal half */
        shift = 13;
        hexp = (uint32_t)(e + 15);
    } else {                                      /* subnormal half */
        shift = 13 + (-14 - e);
        hexp = 0;
    }
    uint32_t keep = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (keep & 1u))) keep++;
    uint32_t h;
    if (hexp) {
        /* keep has the implicit bit at position 10; a carry out bumps the exponent naturally */
        h = ((hexp - 1u) << 10) + keep;
    } else {
        h = keep;                                 /* carry into 0x400 makes the smallest normal */
    }
    return (uint16_t)(sign | h);
}

float oracle_h2f(uint16_t h)
{
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu;
    uint32_t m = h & 0x3ffu;
    uint32_t x;
    if (e == 0) {
        if (m == 0) {
            x = sign;
        } else {
            int k = 0;
            while (!(m & 0x400u)) { m <<= 1; k++; }
            m &= 0x3ffu;
            x = sign | ((uint32_t)(127 - 15 - k + 1) << 23) | (m << 13);
        }
    } else if (e == 31) {
        x = sign | 0x7f800000u | (m << 13);
    } else {
        x = sign | ((e + 127 - 15) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &x, 4);
    return f;
}

/* out[i] = float(half(in[i])) */
void oracle_round_to_half(const float *in, float *out, int64_t n)
{
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) out[i] = oracle_h2f(oracle_f2h_bits(in[i]));
}

/* ------------------------------------------------------------- norm map */

/*
 * Canonical reduction order of one 32x32 tile (the CUDA kernel uses the same):
 *   eight accumulators g = 0..7, accumulator g owns columns 4g..4g+3;
 *   rows r = 0..31 in order, inside a row the four columns left to right,
 *   each step acc = fmaf(x, x, acc) starting from +0;
 *   then p[g] = acc[g] + acc[g+4] (g<4), q[g] = p[g] + p[g+2] (g<2), s = q[0] + q[1];
 *   norm = sqrtf(s).
 */
static float spamm_norm_order(const float *t, int64_t ld)
{
    float acc[8];
    for (int g = 0; g < 8; g++) acc[g] = 0.0f;
    for (int r = 0; r < TILE; r++) {
        const float *row = t + (int64_t)r * ld;
        for (int g = 0; g < 8; g++) {
            float a = acc[g];
            a = fmaf(row[4 * g + 0], row[4 * g + 0], a);
            a = fmaf(row[4 * g + 1], row[4 * g + 1], a);
            a = fmaf(row[4 * g + 2], row[4 * g + 2], a);
            a = fmaf(row[4 * g + 3], row[4 * g + 3], a);
            acc[g] = a;
        }
    }
    float p0 = acc[0] + acc[4], p1 = acc[1] + acc[5], p2 = acc[2] + acc[6], p3 = acc[3] + acc[7];
    float q0 = p0 + p2, q1 = p1 + p3;
    return sqrtf(q0 + q1);
}

/* map is (rows/32) x (cols/32), row-major: map[tr*(cols/32)+tc]  (cuSpAMM.cu:28-30,69) */
int oracle_norm_map(const float *X, int rows, int cols, int64_t ld, float *map)
{
    if (rows % TILE || cols % TILE || rows < 0 || cols < 0) return 1;
    int tr_n = rows / TILE, tc_n = cols / TILE;
#pragma omp parallel for schedule(static)
    for (int tr = 0; tr < tr_n; tr++)
        for (int tc = 0; tc < tc_n; tc++)
            map[(int64_t)tr * tc_n + tc] = spamm_norm_order(X + (int64_t)tr * TILE * ld + (int64_t)tc * TILE, ld);
    return 0;
}

/* ------------------------------------------------------------ skip lists */

/*
 * counts[i*TN+j] = number of k with  nA[i,k]*nB[k,j] >= tau   (float product, cuSpAMM.cu:305-306).
 * Returns the total S.  Rows [row_begin, row_begin+row_count) of the A map only
 * (the reference's main_row_offset, cuSpAMM.cu:291,530); counts is indexed from row_begin.
 */
int64_t oracle_count_lists(const float *nA, const float *nB, int TK, int TN,
                           int row_begin, int row_count, float tau, int32_t *counts)
{
    int64_t total = 0;
#pragma omp parallel for schedule(static) reduction(+ : total)
    for (int i = 0; i < row_count; i++) {
        const float *a = nA + (int64_t)(row_begin + i) * TK;
        for (int j = 0; j < TN; j++) {
            int c = 0;
            for (int k = 0; k < TK; k++) {
                volatile float prod = a[k] * nB[(int64_t)k * TN + j];
                if (prod >= tau) c++;
            }
            counts[(int64_t)i * TN + j] = c;
            total += c;
        }
    }
    return total;
}

/*
 * CSR form: offsets has row_count*TN+1 entries (exclusive prefix of counts),
 * kidx[offsets[t] .. offsets[t+1]) are the surviving k of tile t in ascending order (cuSpAMM.cu:315-326).
 */
void oracle_fill_lists(const float *nA, const float *nB, int TK, int TN,
                       int row_begin, int row_count, float tau,
                       const int64_t *offsets, int32_t *kidx)
{
#pragma omp parallel for schedule(static)
    for (int i = 0; i < row_count; i++) {
        const float *a = nA + (int64_t)(row_begin + i) * TK;
        for (int j = 0; j < TN; j++) {
            int64_t o = offsets[(int64_t)i * TN + j];
            for (int k = 0; k < TK; k++) {
                volatile float prod = a[k] * nB[(int64_t)k * TN + j];
                if (prod >= tau) kidx[o++] = k;
            }
        }
    }
}

/* --------------------------------------------------------- gated product */

/*
 * C(i,j) = sum over surviving k (ascending) of  half(A(i,k)) * half(B(k,j)) for the row_count tile rows of one
 * row block (Ah, C and the lists are all indexed from the block's first row),
 * float accumulation in the order of the authors' host loop (tool.cu:108-114):
 * for every surviving k, for every element, kk = 0..31 added one at a time.
 * Ah, Bh hold the half-rounded inputs as floats (oracle_round_to_half).
 * C has row_count*32 rows, leading dimension N; tiles with no survivor are zero (cuSpAMM.cu:300,391).
 */
void oracle_gated_multiply(const float *Ah, const float *Bh, int K, int N,
                           int row_count, const int64_t *offsets,
                           const int32_t *kidx, float *C)
{
    int TN = N / TILE;
#pragma omp parallel for schedule(dynamic, 1)
    for (int i = 0; i < row_count; i++) {
        for (int j = 0; j < TN; j++) {
            float acc[TILE][TILE];
            memset(acc, 0, sizeof(acc));
            int64_t t = (int64_t)i * TN + j;
            for (int64_t o = offsets[t]; o < offsets[t + 1]; o++) {
                int k = kidx[o];
                const float *a = Ah + ((int64_t)i * TILE) * K + (int64_t)k * TILE;
                const float *b = Bh + ((int64_t)k * TILE) * N + (int64_t)j * TILE;
                for (int r = 0; r < TILE; r++) {
                    for (int kk = 0; kk < TILE; kk++) {
                        float av = a[(int64_t)r * K + kk];
                        const float *brow = b + (int64_t)kk * N;
                        for (int c = 0; c < TILE; c++) {
                            float prod = av * brow[c];       /* exact in float: both are half values */
                            acc[r][c] = acc[r][c] + prod;
                        }
                    }
                }
            }
            for (int r = 0; r < TILE; r++)
                memcpy(C + ((int64_t)i * TILE + r) * N + (int64_t)j * TILE, acc[r], TILE * sizeof(float));
        }
    }
}

/*
 * The same gated sum on the UNROUNDED float inputs with double accumulation, rounded to float once at the end:
 * what the reference's float build (USINGHALF 0: get_C_Threads1Element_Mul, cuSpAMM.cu:203-266) approximates with
 * float accumulation on CUDA cores.  Checker for the split-precision mode of the library (three half products
 * per tile product), which aims at float-level accuracy on tensor cores.
 */
void oracle_gated_multiply_exact(const float *A, const float *B, int K, int N,
                                 int row_count, const int64_t *offsets,
                                 const int32_t *kidx, float *C)
{
    int TN = N / TILE;
#pragma omp parallel for schedule(dynamic, 1)
    for (int i = 0; i < row_count; i++) {
        for (int j = 0; j < TN; j++) {
            double acc[TILE][TILE];
            memset(acc, 0, sizeof(acc));
            int64_t t = (int64_t)i * TN + j;
            for (int64_t o = offsets[t]; o < offsets[t + 1]; o++) {
                int k = kidx[o];
                const float *a = A + ((int64_t)i * TILE) * K + (int64_t)k * TILE;
                const float *b = B + ((int64_t)k * TILE) * N + (int64_t)j * TILE;
                for (int r = 0; r < TILE; r++) {
                    for (int kk = 0; kk < TILE; kk++) {
                        double av = (double)a[(int64_t)r * K + kk];
                        const float *brow = b + (int64_t)kk * N;
                        for (int c = 0; c < TILE; c++) acc[r][c] += av * (double)brow[c];
                    }
                }
            }
            for (int r = 0; r < TILE; r++)
                for (int c = 0; c < TILE; c++)
                    C[((int64_t)i * TILE + r) * N + (int64_t)j * TILE + c] = (float)acc[r][c];
        }
    }
}

/*
 * Whole path on host matrices: norm maps of the float data, lists, product of the
 * half-rounded data.  nA_out (row_count x TK, this row block only), nB_out (TK x TN)
 * and counts_out (row_count x TN) may be NULL.  Returns S (surviving tile products) or -1.
 */
int64_t oracle_spamm(const float *A, const float *B, float *C, int M, int K, int N,
                     int row_begin, int row_count, float tau,
                     float *nA_out, float *nB_out, int32_t *counts_out)
{
    if (M % TILE || K % TILE || N % TILE) return -1;
    int TK = K / TILE, TN = N / TILE, TM = M / TILE;
    if (row_begin < 0 || row_count < 0 || row_begin + row_count > TM) return -1;
    float *nA = (float *)malloc(sizeof(float) * (size_t)TM * TK);
    float *nB = (float *)malloc(sizeof(float) * (size_t)TK * TN);
    int32_t *counts = (int32_t *)malloc(sizeof(int32_t) * (size_t)(row_count ? row_count : 1) * TN);
    int64_t ntile = (int64_t)row_count * TN;
    int64_t *offsets = (int64_t *)malloc(sizeof(int64_t) * (size_t)(ntile + 1));
    size_t a_rows = (size_t)row_count * TILE;
    float *Ah = (float *)malloc(sizeof(float) * (a_rows ? a_rows : 1) * K);
    float *Bh = (float *)malloc(sizeof(float) * (size_t)K * N);
    int64_t S = -1;
    if (!nA || !nB || !counts || !offsets || !Ah || !Bh) goto done;
    memset(nA, 0, sizeof(float) * (size_t)TM * TK);
    oracle_norm_map(A + (int64_t)row_begin * TILE * K, row_count * TILE, K, K, nA + (int64_t)row_begin * TK);
    oracle_norm_map(B, K, N, N, nB);
    S = oracle_count_lists(nA, nB, TK, TN, row_begin, row_count, tau, counts);
    offsets[0] = 0;
    for (int64_t t = 0; t < ntile; t++) offsets[t + 1] = offsets[t] + counts[t];
    {
        int32_t *kidx = (int32_t *)malloc(sizeof(int32_t) * (size_t)(S ? S : 1));
        if (!kidx) { S = -1; goto done; }
        oracle_fill_lists(nA, nB, TK, TN, row_begin, row_count, tau, offsets, kidx);
        oracle_round_to_half(A + (int64_t)row_begin * TILE * K, Ah, (int64_t)a_rows * K);
        oracle_round_to_half(B, Bh, (int64_t)K * N);
        oracle_gated_multiply(Ah, Bh, K, N, row_count, offsets, kidx, C);
        free(kidx);
    }
    if (nA_out) memcpy(nA_out, nA + (int64_t)row_begin * TK, sizeof(float) * (size_t)row_count * TK);
    if (nB_out) memcpy(nB_out, nB, sizeof(float) * (size_t)TK * TN);
    if (counts_out) memcpy(counts_out, counts, sizeof(int32_t) * (size_t)ntile);
done:
    free(nA); free(nB); free(counts); free(offsets); free(Ah); free(Bh);
    return S;
}

/* ------------------------------------------------------- threshold tuner */

/*
 * tuneValidRate, tool.cu:438-490 (constants main.h:35-38): count the products >= Norm and sum all products
 * (the float product widened to double, tool.cu:457-459); stop when |rate - expected| < tolerance; the first
 * pass sets Norm to the mean product, later passes bisect.  rate is (float)count/total as at tool.cu:468.
 * Returns (float)Norm; *rate_out and *iters_out report the last pass.
 */
float oracle_tune_valid_rate(const float *nA, const float *nB, int TM, int TK, int TN,
                             double expected, int max_iters, double tolerance,
                             double *rate_out, int *iters_out)
{
    double Norm = 0, up = 0, down = 0, validRate = 0;
    double total = (double)TM * TK * TN;
    int Ti;
    for (Ti = 0; Ti < max_iters; Ti++) {
        int64_t count = 0;
        double ave = 0;
        for (int i = 0; i < TM; i++)
            for (int j = 0; j < TN; j++)
                for (int k = 0; k < TK; k++) {
                    volatile float prod = nA[(int64_t)i * TK + k] * nB[(int64_t)k * TN + j];
                    double norm = prod;
                    ave += norm;
                    if (norm >= Norm) count++;
                }
        validRate = total > 0 ? (double)((float)count / (float)total) : 0.0;
        if (fabs(validRate - expected) < tolerance) break;
        if (Ti == 0) {
            Norm = total > 0 ? ave / total : 0.0;
            up = Norm;
            continue;
        }
        if (validRate > expected) {
            if (up == Norm) up *= 2;
            down = Norm;
            Norm = (Norm + up) / 2;
        } else {
            up = Norm;
            Norm = (Norm + down) / 2;
        }
    }
    if (rate_out) *rate_out = validRate;
    if (iters_out) *iters_out = Ti;
    return (float)Norm;
}

/* ------------------------------------------------------------ generators */

/* tool.cu:409-422: a_ij = c * v^|i-j|, evaluated as (float)pow(v, |i-j|) with v a float. */
void oracle_gen_decay_exp(float *A, float c, float v, int m, int n)
{
#pragma omp parallel for schedule(static)
    for (int i = 0; i < m; i++)
        for (int j = 0; j < n; j++)
            A[(int64_t)i * n + j] = c * (float)pow((double)v, (double)abs(i - j));
}

/* tool.cu:426-436: a_ij = c / (|i-j|^v + 1) */
void oracle_gen_decay_alg(float *A, float c, float v, int m, int n)
{
#pragma omp parallel for schedule(static)
    for (int i = 0; i < m; i++)
        for (int j = 0; j < n; j++)
            A[(int64_t)i * n + j] = (float)c / ((float)pow((double)abs(i - j), (double)v) + 1);
}

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
