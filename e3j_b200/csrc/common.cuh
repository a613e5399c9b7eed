// Shared host/device helpers of the e3j_b200 library.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/e3j_b200.h"

namespace e3jb {

// Canonical device form of one Coef4D row (lib/e3j_ops/cuda/convolution.cuh:31-37):
// value plus (i = output row, j = x row, k = y component, l = scalar index).
struct TableRow {
    float val;
    int32_t i, j, k, l;
};

struct Dims {
    int32_t X, Y, Z, S, C;
};

// Device-resident tables of a plan.
struct DeviceTable {
    const float *val = nullptr;  // [nnz]
    const int4 *idx = nullptr;   // [nnz] (i, j, k, l)
    int32_t nnz = 0;
};

// ---- error plumbing ------------------------------------------------------
// Mirrors e3j::Error's categories and message prefixes (lib/e3j_ops/ffi/error.h:25-104).
int set_error(int code, const std::string &msg);

#define E3JB_CUDA_TRY(expr)                                                          \
    do {                                                                             \
        cudaError_t _e = (expr);                                                     \
        if (_e != cudaSuccess)                                                       \
            return ::e3jb::set_error(E3J_B200_CUDA_RUNTIME,                          \
                                     std::string(#expr) + ": " + cudaGetErrorString(_e)); \
    } while (0)

// Launch check, and a full synchronisation when debug > 0
// (lib/e3j_ops/cuda/convolution/launch_fwd.cuh:255-263).
int check_launch(const char *what, int debug, cudaStream_t stream);

__host__ __device__ inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- device helpers ------------------------------------------------------
__device__ __forceinline__ bool in_range(int32_t a, int32_t n) {
    return static_cast<uint32_t>(a) < static_cast<uint32_t>(n);
}

// Streaming loads/stores: data touched once (s, ds, dy, dx messages) should not
// displace the node rows (x, dm) that are re-read through L2.
__device__ __forceinline__ float4 ld_stream4(const float *p) {
    float4 v;
    asm volatile("ld.global.L1::no_allocate.L2::evict_first.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream4(float *p, float4 v) {
    asm volatile("st.global.L1::no_allocate.L2::evict_first.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p),
                 "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}

}  // namespace e3jb
