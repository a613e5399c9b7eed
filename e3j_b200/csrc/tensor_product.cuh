// Standalone sparse tensor product on rows (no graph), TRAILING_CHANNELS layout:
//
//     out[n, i, c] = sum_t val_t * x[n, j_t, u] * y[n, k_t, v]
//
// with the channel rule of the mode (the reference's MixingMode, src/e3j/utils/options.py:154-168):
//     OUTER (0): c = u * CY + v for every u < CX, v < CY   (CY = 1: y without channels)
//     MAP   (2): c = u = v                                  (CX == CY)
// and its cotangents dx, dy for a cotangent dz of out.  Functional counterpart of the
// reference's "tensor_product" / "tensor_product_bwd" targets (lib/e3j_ops/ffi/e3j_ops.h:124-373)
// for that layout; table-driven and deterministic (every sum in a fixed order, no atomics).
// The fused convolution does not call these kernels.
#pragma once

#include "common.cuh"

namespace e3jb {
namespace tp {

constexpr int kThreads = 128;
constexpr int kMaxY = 64;  // y rows the channel-less dy reduction keeps per warp
enum Mode { OUTER = 0, INNER = 1, MAP = 2 };

struct Table {  // rows {val, (i, j, k, unused)} sorted by the column the kernel groups by
    const float *val;
    const int4 *idx;
    int32_t nnz;
};

struct Shape {
    int32_t X, Y, Z, CX, CY, CZ, mode;
};

__device__ __forceinline__ void channels_of(const Shape &sh, int c, int &u, int &v) {
    if (sh.mode == MAP) {
        u = v = c;
    } else {
        u = c / sh.CY;
        v = c - u * sh.CY;
    }
}

// Forward: one block per row of the batch (grid-stride), threads over output channels.
// `by_i` is sorted by output row, so each output element is one running sum.
__global__ void __launch_bounds__(kThreads) fwd_kernel(Table by_i, const float *__restrict__ x,
                                                       const float *__restrict__ y, float *__restrict__ out,
                                                       int64_t rows, Shape sh) {
    for (int64_t n = blockIdx.x; n < rows; n += gridDim.x) {
        const float *xn = x + n * sh.X * sh.CX, *yn = y + n * sh.Y * sh.CY;
        float *on = out + n * sh.Z * sh.CZ;
        for (int c = threadIdx.x; c < sh.CZ; c += blockDim.x) {
            int u, v;
            channels_of(sh, c, u, v);
            int t = 0;
            for (int i = 0; i < sh.Z; i++) {  // rows without table entries are written as zeros
                float acc = 0.f;
                for (; t < by_i.nnz && by_i.idx[t].x == i; t++) {
                    const int4 id = by_i.idx[t];
                    acc = fmaf(by_i.val[t] * yn[id.z * sh.CY + v], xn[id.y * sh.CX + u], acc);
                }
                on[(int64_t)i * sh.CZ + c] = acc;
            }
        }
    }
}

// dx[n, j, u] = sum_{t: j_t = j} val_t * sum_v y[n, k_t, v] * dz[n, i_t, c(u, v)];  `by_j` sorted by j.
__global__ void __launch_bounds__(kThreads) bwd_dx_kernel(Table by_j, const float *__restrict__ y,
                                                          const float *__restrict__ dz, float *__restrict__ dx,
                                                          int64_t rows, Shape sh) {
    for (int64_t n = blockIdx.x; n < rows; n += gridDim.x) {
        const float *yn = y + n * sh.Y * sh.CY, *gn = dz + n * sh.Z * sh.CZ;
        float *dn = dx + n * sh.X * sh.CX;
        for (int u = threadIdx.x; u < sh.CX; u += blockDim.x) {
            int t = 0;
            for (int j = 0; j < sh.X; j++) {
                float acc = 0.f;
                for (; t < by_j.nnz && by_j.idx[t].y == j; t++) {
                    const int4 id = by_j.idx[t];
                    float inner = 0.f;
                    if (sh.mode == MAP) {
                        inner = yn[id.z * sh.CY + u] * gn[(int64_t)id.x * sh.CZ + u];
                    } else {
                        for (int v = 0; v < sh.CY; v++)
                            inner = fmaf(yn[id.z * sh.CY + v], gn[(int64_t)id.x * sh.CZ + u * sh.CY + v], inner);
                    }
                    acc = fmaf(by_j.val[t], inner, acc);
                }
                dn[j * sh.CX + u] = acc;
            }
        }
    }
}

// dy[n, k, v] = sum_{t: k_t = k} val_t * sum_u x[n, j_t, u] * dz[n, i_t, c(u, v)];  `by_k` sorted by k.
// MAP: one thread per channel.  OUTER with CY == 1 (y without channels): the threads split the
// sum over u and combine it with a fixed tree (butterfly inside a warp, then the warps in order).
// OUTER with CY > 1: one thread per v, serial sum over u.
__global__ void __launch_bounds__(kThreads) bwd_dy_kernel(Table by_k, const float *__restrict__ x,
                                                          const float *__restrict__ dz, float *__restrict__ dy,
                                                          int64_t rows, Shape sh) {
    __shared__ float part[(kThreads / 32) * kMaxY];
    for (int64_t n = blockIdx.x; n < rows; n += gridDim.x) {
        const float *xn = x + n * sh.X * sh.CX, *gn = dz + n * sh.Z * sh.CZ;
        float *dn = dy + n * sh.Y * sh.CY;
        if (sh.mode == MAP) {
            for (int v = threadIdx.x; v < sh.CY; v += blockDim.x) {
                int t = 0;
                for (int k = 0; k < sh.Y; k++) {
                    float acc = 0.f;
                    for (; t < by_k.nnz && by_k.idx[t].z == k; t++) {
                        const int4 id = by_k.idx[t];
                        acc = fmaf(by_k.val[t] * xn[id.y * sh.CX + v], gn[(int64_t)id.x * sh.CZ + v], acc);
                    }
                    dn[k * sh.CY + v] = acc;
                }
            }
        } else if (sh.CY == 1) {
            // y without channels: dy[n, k] sums over all CX channels; threads split u, fixed reduction
            // tree (butterfly inside a warp, then the warps' partial sums in order), Y <= kMaxY
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
            int t = 0;
            for (int k = 0; k < sh.Y; k++) {
                int t1 = t;
                while (t1 < by_k.nnz && by_k.idx[t1].z == k) t1++;
                float acc = 0.f;
                for (int u = threadIdx.x; u < sh.CX; u += blockDim.x)
                    for (int q = t; q < t1; q++) {
                        const int4 id = by_k.idx[q];
                        acc = fmaf(by_k.val[q] * xn[id.y * sh.CX + u], gn[(int64_t)id.x * sh.CZ + u], acc);
                    }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (lane == 0) part[warp * kMaxY + k] = acc;
                t = t1;
            }
            __syncthreads();
            for (int k = threadIdx.x; k < sh.Y; k += blockDim.x) {
                float total = 0.f;
                for (int w = 0; w < nwarp; w++) total += part[w * kMaxY + k];
                dn[k] = total;
            }
            __syncthreads();
        } else {
            for (int v = threadIdx.x; v < sh.CY; v += blockDim.x) {
                int t = 0;
                for (int k = 0; k < sh.Y; k++) {
                    float acc = 0.f;
                    for (; t < by_k.nnz && by_k.idx[t].z == k; t++) {
                        const int4 id = by_k.idx[t];
                        float inner = 0.f;
                        for (int u = 0; u < sh.CX; u++)
                            inner = fmaf(xn[id.y * sh.CX + u], gn[(int64_t)id.x * sh.CZ + u * sh.CY + v], inner);
                        acc = fmaf(by_k.val[t], inner, acc);
                    }
                    dn[k * sh.CY + v] = acc;
                }
            }
        }
    }
}

}  // namespace tp
}  // namespace e3jb
