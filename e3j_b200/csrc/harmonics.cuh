// Real harmonics of edge vectors and their vector-Jacobian product.
//
// y[e, row] = sum_m coef_m a^i b^j c^k over the monomials of that row, with (a, b, c) the
// edge vector, optionally projected on the sphere with the reference's safe norm
// sqrt(|r|^2 + 1e-7) (src/e3j/utils/safe.py:24-46).  The monomial table is built on the
// host from the reference's ladder construction (src/e3j/utils/spherical_harmonics.py,
// src/e3j/core/harmonics.py:45-101) and arrives as data, so any degree / normalisation
// runs through the same kernel.  One thread per edge; the table is staged in shared memory.
#pragma once

#include "common.cuh"

namespace e3jb {
namespace harmonics {

constexpr int kMaxDim = 64;     // output components per edge (lmax <= 7)
constexpr int kMaxDegree = 8;   // highest monomial degree
constexpr float kSafeEps = 1e-7f;

struct Table {
    const float *coef;   // [M]
    const int32_t *desc;  // [M] packed: i | j << 4 | k << 8 | row << 12
    int32_t M, dim, normalize;
};

__device__ __forceinline__ void powers(float v, float (&p)[kMaxDegree + 1]) {
    p[0] = 1.f;
#pragma unroll
    for (int d = 1; d <= kMaxDegree; d++) p[d] = p[d - 1] * v;
}

__global__ void __launch_bounds__(128) fwd_kernel(Table t, const float *__restrict__ r, float *__restrict__ y, int64_t E) {
    extern __shared__ __align__(16) unsigned char smem[];
    float *scoef = reinterpret_cast<float *>(smem);
    int32_t *sdesc = reinterpret_cast<int32_t *>(scoef + t.M);
    for (int m = threadIdx.x; m < t.M; m += blockDim.x) {
        scoef[m] = t.coef[m];
        sdesc[m] = t.desc[m];
    }
    __syncthreads();
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < E; e += (int64_t)gridDim.x * blockDim.x) {
        float a = r[3 * e], b = r[3 * e + 1], c = r[3 * e + 2];
        if (t.normalize) {
            const float inv = 1.f / sqrtf(a * a + b * b + c * c + kSafeEps);
            a *= inv; b *= inv; c *= inv;
        }
        float pa[kMaxDegree + 1], pb[kMaxDegree + 1], pc[kMaxDegree + 1];
        powers(a, pa); powers(b, pb); powers(c, pc);
        float *ye = y + e * t.dim;
        // rows are contiguous in the table: accumulate a row, store it when the row changes
        int cur = -1;
        float acc = 0.f;
        for (int m = 0; m < t.M; m++) {
            const int d = sdesc[m];
            const int row = d >> 12;
            if (row != cur) {
                if (cur >= 0) ye[cur] = acc;
                cur = row;
                acc = 0.f;
            }
            acc = fmaf(scoef[m] * pa[d & 15], pb[(d >> 4) & 15] * pc[(d >> 8) & 15], acc);
        }
        if (cur >= 0) ye[cur] = acc;
    }
}

// dr[e, :] = J(e)^T dy[e, :]
__global__ void __launch_bounds__(128) bwd_kernel(Table t, const float *__restrict__ r, const float *__restrict__ dy,
                                                  float *__restrict__ dr, int64_t E) {
    extern __shared__ __align__(16) unsigned char smem[];
    float *scoef = reinterpret_cast<float *>(smem);
    int32_t *sdesc = reinterpret_cast<int32_t *>(scoef + t.M);
    for (int m = threadIdx.x; m < t.M; m += blockDim.x) {
        scoef[m] = t.coef[m];
        sdesc[m] = t.desc[m];
    }
    __syncthreads();
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < E; e += (int64_t)gridDim.x * blockDim.x) {
        const float ra = r[3 * e], rb = r[3 * e + 1], rc = r[3 * e + 2];
        float a = ra, b = rb, c = rc, inv = 1.f;
        if (t.normalize) {
            inv = 1.f / sqrtf(ra * ra + rb * rb + rc * rc + kSafeEps);
            a *= inv; b *= inv; c *= inv;
        }
        float pa[kMaxDegree + 1], pb[kMaxDegree + 1], pc[kMaxDegree + 1];
        powers(a, pa); powers(b, pb); powers(c, pc);
        const float *g = dy + e * t.dim;
        float da = 0.f, db = 0.f, dc = 0.f;
        for (int m = 0; m < t.M; m++) {
            const int d = sdesc[m];
            const int i = d & 15, j = (d >> 4) & 15, k = (d >> 8) & 15;
            const float w = scoef[m] * g[d >> 12];
            if (i) da = fmaf(w * (float)i, pa[i - 1] * pb[j] * pc[k], da);
            if (j) db = fmaf(w * (float)j, pa[i] * pb[j - 1] * pc[k], db);
            if (k) dc = fmaf(w * (float)k, pa[i] * pb[j] * pc[k - 1], dc);
        }
        if (t.normalize) {
            // u = r / n  =>  dr = du / n - r (r . du) / n^3
            const float dot = ra * da + rb * db + rc * dc;
            const float inv3 = inv * inv * inv;
            da = da * inv - ra * dot * inv3;
            db = db * inv - rb * dot * inv3;
            dc = dc * inv - rc * dot * inv3;
        }
        dr[3 * e] = da; dr[3 * e + 1] = db; dr[3 * e + 2] = dc;
    }
}

}  // namespace harmonics
}  // namespace e3jb
