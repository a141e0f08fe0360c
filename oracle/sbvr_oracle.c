/*
 * CPU restatement of the SBVR decode and fp16-activation linear.  TEST INFRASTRUCTURE ONLY:
 * the checker for the CUDA kernels and the timed CPU baseline; never linked into, called by
 * or shipped with the product library.
 *
 * Arithmetic follows the reference (MaverickJune/sbvr-cpu-arm):
 *   - bit meaning and packing   sbvr/core.py:345-351, :815-818, :842-876
 *   - GPU tensor layout         sbvr/core.py:726-730, :783-800
 *   - decode                    sbvr/core.py:926-949 (fp32 sum over planes in order, one
 *                               round-to-nearest-even to fp16)
 *   - linear                    test_sbvr.py:321 / sbvr_utils/utils_llama.py:147
 *                               (x @ decode().T + bias, fp32 accumulate, fp16 out; bias is
 *                               added before the final conversion as in
 *                               sbvr/kernels/sbvr_kernel.cu:145-189)
 * The reference's own native CPU kernels (sbvr/kernels/sbvr_kernel.cpp, sbvr_kernel_v2.cpp)
 * are ARM-NEON only and take SBVR-encoded activations; they cannot be compiled on x86 and
 * compute a different product, so this file restates the fp16-activation path instead.
 *
 * Parity pinned by tests/golden (outputs of the reference's sbvr/core.py).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static float h2f_table[65536];
static int table_ready = 0;

static float half_bits_to_float(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t out;
    if (exp == 0) {
        if (man == 0) {
            out = sign;
        } else {                                 /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            man &= 0x3FFu;
            out = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        out = sign | 0x7F800000u | (man << 13);
    } else {
        out = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &out, 4);
    return f;
}

/* float -> half, round to nearest even (what torch and __float2half_rn do) */
static uint16_t float_to_half_bits(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) {                   /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? 0x200u : 0));
    }
    if (absx >= 0x477FF000u) {                   /* >= 65520 rounds to inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (absx < 0x38800000u) {                    /* below the smallest normal half */
        if (absx < 0x33000000u) return (uint16_t)sign;   /* < 2^-25 -> 0 */
        int e = (int)(absx >> 23);               /* biased fp32 exponent, 102..112 */
        uint32_t man = (absx & 0x7FFFFFu) | 0x800000u;
        int shift = 126 - e;                     /* 14..24: bits to drop to reach the 2^-24 grid */
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1u))) half_man++;
        return (uint16_t)(sign | half_man);
    }
    uint32_t e = (absx >> 23) - 112u;
    uint32_t man = absx & 0x7FFFFFu;
    uint32_t h = (e << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
    return (uint16_t)(sign | h);
}

static void init_table(void)
{
    if (table_ready) return;
    for (uint32_t i = 0; i < 65536; i++) h2f_table[i] = half_bits_to_float((uint16_t)i);
    table_ready = 1;
}

/* Sets the number of OpenMP threads the checker uses (launchers such as torchrun export OMP_NUM_THREADS=1). */
void sbvr_oracle_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int sbvr_oracle_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* coefficient line of (group g, row n): pointer to S halves */
static inline const uint16_t *coeff_line(const void *idx, int idx_bytes, const uint16_t *coeff,
                                         int g, int n, int N, int S)
{
    if (idx_bytes == 0) return coeff + ((size_t)g * N + n) * S;
    size_t line = (idx_bytes == 1) ? ((const uint8_t *)idx)[(size_t)g * N + n]
                                   : ((const uint16_t *)idx)[(size_t)g * N + n];
    return coeff + line * S;
}

/* all 2^S values a group can take, as fp16 bit patterns; selector = planes MSB first */
static inline void group_points(const uint16_t *line, int S, uint16_t *pts)
{
    int n = 1 << S;
    for (int sel = 0; sel < n; sel++) {
        float acc = 0.0f;
        for (int s = 0; s < S; s++)
            if ((sel >> (S - 1 - s)) & 1) acc += h2f_table[line[s]];
        pts[sel] = float_to_half_bits(acc);
    }
}

/* W[N, K] (row pitch K) from packed tensors.  K is the padded length (multiple of G). */
int sbvr_oracle_decode(const uint32_t *bvr, const void *idx, int idx_bytes, const uint16_t *coeff,
                       uint16_t *W, int N, int K, int S, int G, int threads)
{
    if (S < 1 || S > 11 || G % 32 || K % G) return -1;
    init_table();
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#endif
    int wpg = G / 32;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        uint16_t pts[2048];
        for (int g = 0; g < K / G; g++) {
            group_points(coeff_line(idx, idx_bytes, coeff, g, n, N, S), S, pts);
            for (int w = 0; w < wpg; w++) {
                int kw = g * wpg + w;
                const uint32_t *words = bvr + ((size_t)kw * N + n) * S;
                for (int j = 0; j < 32; j++) {
                    int sel = 0;
                    for (int s = 0; s < S; s++) sel = (sel << 1) | ((words[s] >> j) & 1u);
                    W[(size_t)n * K + kw * 32 + j] = pts[sel];
                }
            }
        }
    }
    return 0;
}

/* y[M, N] = fp16( x[M, K] . W[N, K]^T + bias ), fp32 accumulation, decode fused (no dense W) */
int sbvr_oracle_linear(const uint16_t *x, const uint32_t *bvr, const void *idx, int idx_bytes,
                       const uint16_t *coeff, const uint16_t *bias, uint16_t *y,
                       int M, int N, int K, int S, int G, int threads)
{
    if (S < 1 || S > 11 || G % 32 || K % G || M < 1) return -1;
    init_table();
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#endif
    float *xf = (float *)malloc(sizeof(float) * (size_t)M * K);
    if (!xf) return -2;
    for (size_t i = 0; i < (size_t)M * K; i++) xf[i] = h2f_table[x[i]];
    int wpg = G / 32;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        uint16_t pts[2048];
        float ptsf[2048];
        float wrow[32];
        float *acc = (float *)calloc((size_t)M, sizeof(float));
        for (int g = 0; g < K / G; g++) {
            group_points(coeff_line(idx, idx_bytes, coeff, g, n, N, S), S, pts);
            for (int i = 0; i < (1 << S); i++) ptsf[i] = h2f_table[pts[i]];
            for (int w = 0; w < wpg; w++) {
                int kw = g * wpg + w;
                const uint32_t *words = bvr + ((size_t)kw * N + n) * S;
                for (int j = 0; j < 32; j++) {
                    int sel = 0;
                    for (int s = 0; s < S; s++) sel = (sel << 1) | ((words[s] >> j) & 1u);
                    wrow[j] = ptsf[sel];
                }
                for (int m = 0; m < M; m++) {
                    const float *xr = xf + (size_t)m * K + kw * 32;
                    float a = 0.0f;
                    for (int j = 0; j < 32; j++) a += xr[j] * wrow[j];
                    acc[m] += a;
                }
            }
        }
        for (int m = 0; m < M; m++) {
            float v = acc[m];
            if (bias) v += h2f_table[bias[n]];
            y[(size_t)m * N + n] = float_to_half_bits(v);
        }
        free(acc);
    }
    free(xf);
    return 0;
}
