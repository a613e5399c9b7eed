// TEST / BENCH INFRASTRUCTURE — C entry points around the reference's own CUDA
// convolution kernels, compiled from the reference tree where it lies (never copied).
//
// Built by oracle/build_ref.py into oracle/_ref/libe3j_ref_conv.so together with
// lib/e3j_ops/cuda/convolution.cu and convolution_bwd.cu of the reference.  Used as a
// numerical cross-check of the B200 kernels and as "the kernel to beat" in profiles;
// never loaded by the product path.
#include <cstdint>
#include <cstring>
#include <string>

#include "cuda/convolution.cuh"
#include "cuda/convolution_bwd.cuh"

namespace {
thread_local std::string g_msg;
using Coef = e3j::convolution::Coef4D<std::uint8_t, float>;

e3j::convolution::Params make_params(int N, int nnz, int X, int Y, int Z, int S, int C, int E) {
    e3j::convolution::Params p;
    std::memset(&p, 0, sizeof(p));
    p.num_nodes = N; p.num_coef = nnz; p.num_x = X; p.num_y = Y; p.num_out = Z;
    p.num_scalars = S; p.channels_x = C; p.num_edges = E;
    return p;
}
int finish(const e3j::Error &err) {
    if (err.success()) return 0;
    g_msg = err.message();
    return 1;
}
}  // namespace

extern "C" {

const char *ref_last_error() { return g_msg.c_str(); }

// registers per thread of kernel<uint8, float, N> (forward) / kernel_bwd (backward)
int ref_registers(int backward, int N) {
    return backward ? e3j::convolution::get_registers_bwd<std::uint8_t, float>(N)
                    : e3j::convolution::get_registers<std::uint8_t, float>(N);
}

// coef: device, nnz rows of Coef4D<uint8, float>, already permuted for `coef_ranges`
int ref_conv_fwd(const void *coef, const float *x, const float *y, const float *s, int32_t *sender,
                 int32_t *receiver_ptr, float *out, int N, int nnz, int X, int Y, int Z, int S, int C, int E,
                 int block_y, const int *coef_ranges, cudaStream_t stream) {
    e3j::convolution::AdjacencyCSR adj = {sender, receiver_ptr};
    return finish(e3j::convolution::launch<std::uint8_t, float>(static_cast<const Coef *>(coef), x, y, s, adj, out,
                                                                make_params(N, nnz, X, Y, Z, S, C, E), stream, 0,
                                                                block_y, coef_ranges));
}

// coef3: device, the (dx, dy, ds) transposed tables stacked, 3 * nnz rows
int ref_conv_bwd(const void *coef3, const float *x, const float *y, const float *s, const float *dm,
                 int32_t *recv_t, int32_t *sender_ptr_t, const int32_t *edge_perm, float *dx, float *dy, float *ds,
                 int N, int nnz, int X, int Y, int Z, int S, int C, int E, int block_y, const int *coef_ranges,
                 cudaStream_t stream) {
    e3j::convolution::AdjacencyCSR adj = {recv_t, sender_ptr_t};
    return finish(e3j::convolution::launch_bwd<std::uint8_t, float>(
        static_cast<const Coef *>(coef3), x, y, s, dm, adj, edge_perm, dx, dy, ds,
        make_params(N, nnz, X, Y, Z, S, C, E), stream, 0, block_y, coef_ranges));
}

}  // extern "C"
