/*
 * CPU oracle for the codebook decode-and-matmul operator, plain C.
 * TEST INFRASTRUCTURE ONLY: used by tests/, the smoke check and the CPU-baseline
 * legs of bench.py as the checker and the timed CPU baseline; never linked into
 * or called from the CUDA library.
 *
 * Parity: the slow sign convention is pinned (tests compare oracle_decode_table
 * with the table the reference's own decode() produced for all 65 536 code
 * words); the fast convention and the fp16 family are parity unpinned (the
 * reference has no CPU definition of them).
 *
 * Scalar semantics follow test_decode_matmul.py:29-55 (decode) and :58-71
 * (triple-loop matmul); the fast sign map follows
 * decode_matmul_cuda/fast_decode_matmul_cuda.cu:52-53; the tile layout
 * follows test_decode_matmul.py:101-109.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* One code word -> 8 int8 values (4 x weight).  test_decode_matmul.py:29-55. */
void oracle_decode_code(uint16_t code, const int64_t *cb64, int convention, int8_t out[8])
{
    uint32_t idx = code & 0xFFu;               /* :30 */
    uint32_t s7 = (code >> 8) & 0x7Fu;         /* :31 */
    uint32_t parity = (uint32_t)__builtin_popcount(s7) & 1u;
    uint32_t s8 = convention == 0 ? (s7 | (parity << 7))    /* :32 */
                                  : ((s7 << 1) | parity);   /* fast_decode_matmul_cuda.cu:52-53 */
    int shift = (code >> 15) & 1;              /* :33 */
    uint64_t entry = (uint64_t)cb64[idx];      /* :35 */
    for (int i = 0; i < 8; ++i) {
        int8_t v = (int8_t)(entry & 0xFFu);    /* :38 */
        if (s8 & 1u) v = (int8_t)(-v);         /* :41-42 */
        v = (int8_t)(shift ? v - 1 : v + 1);   /* :44-47 */
        out[i] = v;
        entry >>= 8;                           /* :50 */
        s8 >>= 1;                              /* :51 */
    }
}

void oracle_decode_table(const int64_t *cb64, int convention, int8_t *table /* [65536*8] */)
{
    for (uint32_t c = 0; c < 65536u; ++c)
        oracle_decode_code((uint16_t)c, cb64, convention, table + 8 * (size_t)c);
}

/* logical codes [N, K/8] -> int8 [N, K] */
void oracle_decode_weights(const int16_t *codes, const int64_t *cb64, int convention,
                           int64_t N, int64_t K, int8_t *w)
{
    int8_t *table = (int8_t *)malloc(65536 * 8);
    oracle_decode_table(cb64, convention, table);
    int64_t total = N * (K / 8);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < total; ++i)
        memcpy(w + 8 * i, table + 8 * (size_t)(uint16_t)codes[i], 8);
    free(table);
}

/* out[M,N] (int32) = x[M,K] (int8) . decode(codes)[N,K]^T.  test_decode_matmul.py:58-71 */
void oracle_matmul_i8(const int8_t *x, const int16_t *codes, const int64_t *cb64, int convention,
                      int64_t M, int64_t N, int64_t K, int32_t *out)
{
    int8_t *table = (int8_t *)malloc(65536 * 8);
    oracle_decode_table(cb64, convention, table);
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t m = 0; m < M; ++m) {
            int32_t acc = 0;
            const int8_t *xr = x + m * K;
            for (int64_t j = 0; j < K / 8; ++j) {
                const int8_t *w = table + 8 * (size_t)(uint16_t)codes[n * (K / 8) + j];
                for (int i = 0; i < 8; ++i) acc += (int32_t)xr[8 * j + i] * (int32_t)w[i];
            }
            out[m * N + n] = acc;
        }
    }
    free(table);
}

/*
 * out[M,N] (float) = scale * x[M,K] . (decode(codes)/4)[N,K]^T, x given as float
 * (the caller widens fp16 exactly).  Accumulates in double, rounds once: this is the
 * checker.  The timed "decode + fp32 matmul" CPU baseline is oracle_matmul_f32 below.
 */
void oracle_matmul_f64acc(const float *x, const int16_t *codes, const int64_t *cb64, int convention,
                          double scale, int64_t M, int64_t N, int64_t K, float *out)
{
    int8_t *table = (int8_t *)malloc(65536 * 8);
    oracle_decode_table(cb64, convention, table);
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        for (int64_t m = 0; m < M; ++m) {
            double acc = 0.0;
            const float *xr = x + m * K;
            for (int64_t j = 0; j < K / 8; ++j) {
                const int8_t *w = table + 8 * (size_t)(uint16_t)codes[n * (K / 8) + j];
                for (int i = 0; i < 8; ++i) acc += (double)xr[8 * j + i] * (double)w[i];
            }
            out[m * N + n] = (float)(scale * 0.25 * acc);
        }
    }
    free(table);
}

/* Same product with float accumulation: the decode-then-fp32-matmul CPU baseline. */
void oracle_matmul_f32(const float *x, const int16_t *codes, const int64_t *cb64, int convention,
                       float scale, int64_t M, int64_t N, int64_t K, float *out)
{
    int8_t *table = (int8_t *)malloc(65536 * 8);
    oracle_decode_table(cb64, convention, table);
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        float wrow[8];
        for (int64_t m = 0; m < M; ++m) {
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            const float *xr = x + m * K;
            for (int64_t j = 0; j < K / 8; ++j) {
                const int8_t *w = table + 8 * (size_t)(uint16_t)codes[n * (K / 8) + j];
                for (int i = 0; i < 8; ++i) wrow[i] = 0.25f * (float)w[i];
                for (int i = 0; i < 8; ++i) acc[i] += xr[8 * j + i] * wrow[i];
            }
            float s = 0.f;
            for (int i = 0; i < 8; ++i) s += acc[i];
            out[m * N + n] = scale * s;
        }
    }
    free(table);
}

/* logical [N, K/8] -> tile layout [N/16][K/32][g:8][t:4][h:2].  test_decode_matmul.py:101-109 */
void oracle_tile_pack(const int16_t *logical, int64_t N, int64_t K, int16_t *tiled)
{
    int64_t K8 = K / 8, KT = K / 32;
    for (int64_t n = 0; n < N; ++n) {
        int64_t nt = n / 16, h = (n % 16) / 8, g = n % 8;
        for (int64_t j = 0; j < K8; ++j) {
            int64_t kt = j / 4, t = j % 4;
            tiled[((nt * KT + kt) * 8 + g) * 8 + 2 * t + h] = logical[n * K8 + j];
        }
    }
}

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
