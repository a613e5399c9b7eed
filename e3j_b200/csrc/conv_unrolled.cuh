// Unrolled (sparsity-pattern-specialised) convolution kernels: interface.
#pragma once

#include <vector>

#include "common.cuh"

namespace e3jb {
namespace unrolled {

struct DevicePlan {
    void *tables = nullptr;
};

inline int resolve(const std::vector<TableRow> &, const Dims &, DevicePlan &, int &variant) {
    variant = E3J_B200_VARIANT_GENERIC;
    return E3J_B200_OK;
}
inline void release(DevicePlan &) {}
inline int launch_fwd(int, const DevicePlan &, int, const float *, const float *, const float *,
                      const int32_t *, const int32_t *, float *, int32_t, int64_t, int, cudaStream_t) {
    return set_error(E3J_B200_INTERNAL, "no unrolled variant built");
}
inline int launch_bwd_edges(int, const DevicePlan &, int, const float *, const float *, const float *,
                            const float *, const int32_t *, const int32_t *, float *, float *, float *,
                            int32_t, int64_t, int, cudaStream_t) {
    return set_error(E3J_B200_INTERNAL, "no unrolled variant built");
}

}  // namespace unrolled
}  // namespace e3jb
