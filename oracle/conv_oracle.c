/*
 * TEST INFRASTRUCTURE — CPU restatement of the fused convolution and its VJP.
 *
 * Only the tests, the smoke check and the CPU-baseline / reference arm of the
 * benchmark may load this file's library; the product path never does.
 *
 * Algorithm followed (paths relative to the e3j project root):
 *   forward   lib/e3j_ops/tests/test_convolution.cpp:64-106  (cpu_convolution):
 *             out[r,i,u] = sum_{e in CSR(r)} sum_n val_n x[snd(e),j_n,u] y[e,k_n] s[e,l_n,u]
 *             which is the gather -> CG product -> scalar mixing -> scatter-add of
 *             src/e3j/core/convolution.py:172-191.
 *   backward  lib/e3j_ops/tests/test_convolution_bwd.cpp:112-182 (cpu_convolution_bwd):
 *             ds[e,l,u] += val x_j y_k dm_i ; dx[snd,j,u] += val (s_l dm_i) y_k ;
 *             dy[e,k]  += sum_u val (s_l dm_i) x_j
 *   padding   edges whose sender lies outside [0, N) are skipped in both passes
 *             (lib/e3j_ops/cuda/convolution/fwd.cuh:367-368); their dy/ds and every
 *             edge outside the CSR segments are exact zeros
 *             (lib/e3j_ops/cuda/convolution/bwd.cuh:308-319).
 *
 * Accumulation is in double when `wide` is non-zero (truth for tolerance
 * checks), else in float in the loop order above (same-precision comparison).
 * OpenMP parallelises over receivers (forward, ds, dy) and over senders (dx).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    float val;
    int32_t i, j, k, l;
} oracle_coef;

#define IN_RANGE(a, n) ((a) >= 0 && (a) < (n))

int oracle_conv_fwd(const oracle_coef *coef, int nnz, const float *x, const float *y,
                    const float *s, const int32_t *sender, const int32_t *receiver_ptr,
                    float *out, int N, int64_t E, int X, int Y, int Z, int S, int C, int wide)
{
    (void)E;
#pragma omp parallel
    {
        double *acc = (double *)malloc(sizeof(double) * (size_t)Z * C);
        float *accf = (float *)malloc(sizeof(float) * (size_t)Z * C);
#pragma omp for schedule(dynamic, 16)
        for (int r = 0; r < N; r++) {
            memset(acc, 0, sizeof(double) * (size_t)Z * C);
            memset(accf, 0, sizeof(float) * (size_t)Z * C);
            for (int64_t e = receiver_ptr[r]; e < receiver_ptr[r + 1]; e++) {
                int32_t a = sender[e];
                if (!IN_RANGE(a, N)) continue;
                const float *xa = x + (size_t)a * X * C;
                const float *ye = y + (size_t)e * Y;
                const float *se = s + (size_t)e * S * C;
                for (int n = 0; n < nnz; n++) {
                    const oracle_coef c = coef[n];
                    const float *xj = xa + (size_t)c.j * C;
                    const float *sl = se + (size_t)c.l * C;
                    if (wide) {
                        double w = (double)c.val * (double)ye[c.k];
                        double *o = acc + (size_t)c.i * C;
                        for (int u = 0; u < C; u++) o[u] += w * (double)xj[u] * (double)sl[u];
                    } else {
                        float yk = ye[c.k];
                        float *o = accf + (size_t)c.i * C;
                        for (int u = 0; u < C; u++) o[u] += c.val * xj[u] * yk * sl[u];
                    }
                }
            }
            float *o = out + (size_t)r * Z * C;
            if (wide) for (size_t t = 0; t < (size_t)Z * C; t++) o[t] = (float)acc[t];
            else memcpy(o, accf, sizeof(float) * (size_t)Z * C);
        }
        free(acc);
        free(accf);
    }
    return 0;
}

/* dx is accumulated per sender over the sender-sorted view (sender_ptr_t, perm_t:
 * position -> original edge) so that threads own disjoint rows.  recv_of_edge[e]
 * is the receiver of original edge e, or an out-of-range value for padding. */
int oracle_conv_bwd(const oracle_coef *coef, int nnz, const float *x, const float *y,
                    const float *s, const float *dm, const int32_t *sender,
                    const int32_t *receiver_ptr, const int32_t *sender_ptr_t,
                    const int32_t *perm_t, float *dx, float *dy, float *ds, int N, int64_t E,
                    int X, int Y, int Z, int S, int C, int wide)
{
    int32_t *recv_of_edge = (int32_t *)malloc(sizeof(int32_t) * (size_t)(E > 0 ? E : 1));
    for (int64_t e = 0; e < E; e++) recv_of_edge[e] = -1;
    for (int r = 0; r < N; r++)
        for (int64_t e = receiver_ptr[r]; e < receiver_ptr[r + 1]; e++) recv_of_edge[e] = r;

    memset(dy, 0, sizeof(float) * (size_t)E * Y);
    memset(ds, 0, sizeof(float) * (size_t)E * S * C);

#pragma omp parallel
    {
        double *dsacc = (double *)malloc(sizeof(double) * (size_t)S * C);
        double *dyacc = (double *)malloc(sizeof(double) * (size_t)Y);
#pragma omp for schedule(dynamic, 16)
        for (int r = 0; r < N; r++) {
            const float *g = dm + (size_t)r * Z * C;
            for (int64_t e = receiver_ptr[r]; e < receiver_ptr[r + 1]; e++) {
                int32_t a = sender[e];
                if (!IN_RANGE(a, N)) continue;
                const float *xa = x + (size_t)a * X * C;
                const float *ye = y + (size_t)e * Y;
                const float *se = s + (size_t)e * S * C;
                memset(dsacc, 0, sizeof(double) * (size_t)S * C);
                memset(dyacc, 0, sizeof(double) * (size_t)Y);
                for (int n = 0; n < nnz; n++) {
                    const oracle_coef c = coef[n];
                    const float *xj = xa + (size_t)c.j * C;
                    const float *sl = se + (size_t)c.l * C;
                    const float *gi = g + (size_t)c.i * C;
                    double *dsl = dsacc + (size_t)c.l * C;
                    if (wide) {
                        double vy = (double)c.val * (double)ye[c.k];
                        double t = 0.0;
                        for (int u = 0; u < C; u++) {
                            dsl[u] += vy * (double)xj[u] * (double)gi[u];
                            t += (double)c.val * ((double)sl[u] * (double)gi[u]) * (double)xj[u];
                        }
                        dyacc[c.k] += t;
                    } else {
                        float yk = ye[c.k];
                        float t = 0.f;
                        for (int u = 0; u < C; u++) {
                            dsl[u] = (double)((float)dsl[u] + c.val * xj[u] * yk * gi[u]);
                            t += c.val * (sl[u] * gi[u]) * xj[u];
                        }
                        dyacc[c.k] = (double)((float)dyacc[c.k] + t);
                    }
                }
                float *dse = ds + (size_t)e * S * C;
                for (size_t t = 0; t < (size_t)S * C; t++) dse[t] = (float)dsacc[t];
                for (int k = 0; k < Y; k++) dy[(size_t)e * Y + k] = (float)dyacc[k];
            }
        }
        free(dsacc);
        free(dyacc);

        double *dxacc = (double *)malloc(sizeof(double) * (size_t)X * C);
#pragma omp for schedule(dynamic, 16)
        for (int a = 0; a < N; a++) {
            memset(dxacc, 0, sizeof(double) * (size_t)X * C);
            for (int64_t p = sender_ptr_t[a]; p < sender_ptr_t[a + 1]; p++) {
                int64_t e = perm_t[p];
                int32_t r = recv_of_edge[e];
                if (!IN_RANGE(r, N)) continue;
                const float *g = dm + (size_t)r * Z * C;
                const float *ye = y + (size_t)e * Y;
                const float *se = s + (size_t)e * S * C;
                for (int n = 0; n < nnz; n++) {
                    const oracle_coef c = coef[n];
                    const float *sl = se + (size_t)c.l * C;
                    const float *gi = g + (size_t)c.i * C;
                    double *o = dxacc + (size_t)c.j * C;
                    if (wide) {
                        double vy = (double)c.val * (double)ye[c.k];
                        for (int u = 0; u < C; u++) o[u] += vy * ((double)sl[u] * (double)gi[u]);
                    } else {
                        float yk = ye[c.k];
                        for (int u = 0; u < C; u++)
                            o[u] = (double)((float)o[u] + c.val * (sl[u] * gi[u]) * yk);
                    }
                }
            }
            float *o = dx + (size_t)a * X * C;
            for (size_t t = 0; t < (size_t)X * C; t++) o[t] = (float)dxacc[t];
        }
        free(dxacc);
    }
    free(recv_of_edge);
    return 0;
}
