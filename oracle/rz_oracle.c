/*
 * Plain-C restatement of the RzLinear ROBE-Z hot path (CPU, scalar loops).
 *
 * TEST INFRASTRUCTURE ONLY: built into oracle/librz_oracle.so by oracle/Makefile and
 * loaded by the tests as a second, independent statement of the hash and of the
 * materialised-weight arithmetic.  The shipped library never links or loads it.
 *
 * Follows (paths relative to the reference repository):
 *   hash, single level ....... python/rz_linear/impl/RzLinearIdx.py:70-71, rz_linear_kernel.cu:34-35
 *   hash, two level .......... python/rz_linear/impl/RzLinearForward.py:316,349
 *   slice layout ............. python/rz_linear/impl/RzLinearIdx.py:62-77
 *   forward .................. python/tests/test_rz_linear.py:68-71
 *   input gradient ........... python/tests/test_rz_linear.py:131-134
 *   hashed-weight gradient ... python/tests/test_rz_linear.py:77-90
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static int64_t tile_offset(int64_t pk, int64_t pn, int64_t H, int64_t L, const int64_t *R, int mode)
{
    if (mode == 0)
        return ((pk * R[3] + pn * R[2] + R[1]) % R[0]) % (H - L);
    int64_t a = (pk * R[3] + pn * R[2] + R[1]) % R[0];
    int64_t b = (pk * R[7] + pn * R[5] + R[4]) % R[0];
    return (a * R[0] + b) % (H - L);
}

/* out[(K+BK-1)/BK][(N+BN-1)/BN] */
int rzo_tile_offsets(int64_t K, int64_t N, int64_t H, int64_t BK, int64_t BN,
                     const int64_t *R, int mode, int64_t *out)
{
    int64_t L = BK * BN;
    if (H <= L) return -1;
    int64_t nk = (K + BK - 1) / BK, nn = (N + BN - 1) / BN;
    for (int64_t pk = 0; pk < nk; ++pk)
        for (int64_t pn = 0; pn < nn; ++pn)
            out[pk * nn + pn] = tile_offset(pk, pn, H, L, R, mode);
    return 0;
}

static int64_t elem_index(int64_t k, int64_t n, int64_t H, int64_t BK, int64_t BN,
                          const int64_t *R, int mode)
{
    return tile_offset(k / BK, n / BN, H, BK * BN, R, mode) + (k % BK) * BN + (n % BN);
}

/* W[K][N] = hashed[index(k, n)] */
int rzo_materialize(const float *hashed, int64_t K, int64_t N, int64_t H, int64_t BK, int64_t BN,
                    const int64_t *R, int mode, float *W)
{
    if (H <= BK * BN) return -1;
    for (int64_t k = 0; k < K; ++k)
        for (int64_t n = 0; n < N; ++n)
            W[k * N + n] = hashed[elem_index(k, n, H, BK, BN, R, mode)];
    return 0;
}

/* Y[M][N] = alpha * X[M][K] @ W ; double accumulation */
int rzo_forward(const float *X, const float *hashed, int64_t M, int64_t K, int64_t N, int64_t H,
                int64_t BK, int64_t BN, const int64_t *R, int mode, double alpha, double *Y)
{
    float *W = (float *)malloc(sizeof(float) * (size_t)K * (size_t)N);
    if (!W) return -2;
    if (rzo_materialize(hashed, K, N, H, BK, BN, R, mode, W)) { free(W); return -1; }
    for (int64_t m = 0; m < M; ++m) {
        double *y = Y + m * N;
        memset(y, 0, sizeof(double) * (size_t)N);
        for (int64_t k = 0; k < K; ++k) {
            double x = X[m * K + k];
            const float *w = W + k * N;
            for (int64_t n = 0; n < N; ++n) y[n] += x * (double)w[n];
        }
        for (int64_t n = 0; n < N; ++n) y[n] *= alpha;
    }
    free(W);
    return 0;
}

/* dX[M][K] = alpha * dY[M][N] @ W^T */
int rzo_backward_input(const float *dY, const float *hashed, int64_t M, int64_t K, int64_t N, int64_t H,
                       int64_t BK, int64_t BN, const int64_t *R, int mode, double alpha, double *dX)
{
    float *W = (float *)malloc(sizeof(float) * (size_t)K * (size_t)N);
    if (!W) return -2;
    if (rzo_materialize(hashed, K, N, H, BK, BN, R, mode, W)) { free(W); return -1; }
    for (int64_t m = 0; m < M; ++m)
        for (int64_t k = 0; k < K; ++k) {
            double s = 0.0;
            const float *w = W + k * N, *g = dY + m * N;
            for (int64_t n = 0; n < N; ++n) s += (double)g[n] * (double)w[n];
            dX[m * K + k] = alpha * s;
        }
    free(W);
    return 0;
}

/* dH[index(k, n)] += alpha * sum_m X[m][k] * dY[m][n] ; dH zeroed here */
int rzo_backward_weight(const float *X, const float *dY, int64_t M, int64_t K, int64_t N, int64_t H,
                        int64_t BK, int64_t BN, const int64_t *R, int mode, double alpha, double *dH)
{
    if (H <= BK * BN) return -1;
    memset(dH, 0, sizeof(double) * (size_t)H);
    double *row = (double *)malloc(sizeof(double) * (size_t)N);
    if (!row) return -2;
    for (int64_t k = 0; k < K; ++k) {
        memset(row, 0, sizeof(double) * (size_t)N);
        for (int64_t m = 0; m < M; ++m) {
            double x = X[m * K + k];
            const float *g = dY + m * N;
            for (int64_t n = 0; n < N; ++n) row[n] += x * (double)g[n];
        }
        for (int64_t n = 0; n < N; ++n)
            dH[elem_index(k, n, H, BK, BN, R, mode)] += alpha * row[n];
    }
    free(row);
    return 0;
}
