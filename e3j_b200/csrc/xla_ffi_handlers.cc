// XLA FFI handlers "convolution" and "convolution_bwd" on top of the e3j_b200 C ABI.
//
// Operand lists, attribute names and dtypes are exactly those of the reference's handlers
// (lib/e3j_ops/ffi/e3j_ops.h:379-472 and :478-594), so e3j's Python side
// (src/e3j/ops/convolution.py:229-242, :433-452) can call these unmodified after
// `jax.ffi.register_ffi_target(name, capsule, platform="CUDA")` (src/e3j/ops/__init__.py:23-24).
// Built only where the XLA FFI headers are available (they are third-party files and are
// included, never retyped); see e3j_b200/_lib.py:build_xla_handlers.
//
// What the handlers add on top of the C ABI:
//   * the plan.  The coefficient table arrives as a device buffer; it is copied to the host
//     (a few KB, one stream synchronisation) and the plan is looked up in a cache keyed by
//     device and table bytes.  With E3J_B200_XLA_TRUST_COEF_POINTER=1 the copy is skipped
//     when the same device address and size were seen before.
//   * the backward's receiver-sorted graph view, rebuilt on the device from the sender-sorted
//     view the reference passes (e3j_b200_csr_untranspose + e3j_b200_csr_ptr), and the
//     forward table recovered from the first of the three transposed tables.
//   * scratch from the call frame's ScratchAllocator.
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/e3j_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

ffi::Error Status(int rc) {
    if (rc == E3J_B200_OK) return ffi::Error::Success();
    const ffi::ErrorCode code = rc == E3J_B200_INVALID_ARGUMENT ? ffi::ErrorCode::kInvalidArgument
                                : rc == E3J_B200_UNIMPLEMENTED  ? ffi::ErrorCode::kUnimplemented
                                                                : ffi::ErrorCode::kInternal;
    return ffi::Error(code, e3j_b200_last_error());
}

ffi::Error CudaStatus(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return ffi::Error::Success();
    return ffi::Error(ffi::ErrorCode::kInternal,
                      std::string("E3J_ERROR[CudaRuntime]: ") + what + ": " + cudaGetErrorString(e));
}

struct PlanKey {
    int device;
    std::vector<int32_t> dims;
    std::string bytes;
    bool operator<(const PlanKey &o) const {
        if (device != o.device) return device < o.device;
        if (dims != o.dims) return dims < o.dims;
        return bytes < o.bytes;
    }
};

std::mutex g_mu;
std::map<PlanKey, e3j_b200_plan *> g_plans;
std::map<std::pair<const void *, size_t>, e3j_b200_plan *> g_by_pointer;

// Plan for the packed table `host` (nnz rows of 8 or 32 bytes) on the current device.
e3j_b200_plan *GetPlan(const std::string &host, int nnz, int idx_bytes, int X, int Y, int Z, int S, int C) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    PlanKey key{dev, {nnz, idx_bytes, X, Y, Z, S, C}, host};
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_plans.find(key);
    if (it != g_plans.end()) return it->second;
    e3j_b200_plan *plan = nullptr;
    if (e3j_b200_plan_create(host.data(), nnz, idx_bytes, X, Y, Z, S, C, 0, &plan) != E3J_B200_OK) return nullptr;
    g_plans.emplace(std::move(key), plan);
    return plan;
}

bool TrustPointer() {
    static const bool v = [] {
        const char *e = std::getenv("E3J_B200_XLA_TRUST_COEF_POINTER");
        return e && e[0] == '1';
    }();
    return v;
}

// Copies `bytes` of device memory to the host, ordered after the work already on `stream`.
ffi::Error FetchTable(const void *dev_ptr, size_t bytes, cudaStream_t stream, std::string &out) {
    out.resize(bytes);
    if (bytes == 0) return ffi::Error::Success();
    if (auto e = CudaStatus(cudaMemcpyAsync(&out[0], dev_ptr, bytes, cudaMemcpyDeviceToHost, stream), "cudaMemcpyAsync");
        e.failure())
        return e;
    return CudaStatus(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
}

struct TableShape {
    int nnz, idx_bytes;
    size_t row_bytes;
};

bool Describe(const ffi::AnyBuffer &coef, int tables, TableShape &t) {
    if (coef.element_type() == ffi::U8) t.idx_bytes = 1;
    else if (coef.element_type() == ffi::S32) t.idx_bytes = 4;
    else return false;
    t.row_bytes = t.idx_bytes == 1 ? 8 : 32;  // Coef4D<Idx, float>, lib/e3j_ops/cuda/convolution.cuh:39-44
    const size_t total = coef.element_count() * (size_t)t.idx_bytes;
    if (total % (t.row_bytes * tables)) return false;
    t.nnz = (int)(total / (t.row_bytes * tables));
    return true;
}

ffi::Error ConvolutionImpl(cudaStream_t stream, ffi::AnyBuffer coef, ffi::AnyBuffer x, ffi::AnyBuffer y,
                           ffi::AnyBuffer s, ffi::BufferR1<ffi::S32> sender, ffi::BufferR1<ffi::S32> receiver_ptr,
                           ffi::BufferR1<ffi::S32> /*coef_ranges*/, ffi::Result<ffi::AnyBuffer> out,
                           int32_t num_nodes, int32_t debug) {
    if (x.element_type() != ffi::F32 || y.element_type() != ffi::F32 || s.element_type() != ffi::F32)
        return ffi::Error(ffi::ErrorCode::kUnimplemented,
                          "E3J_ERROR[Unimplemented]: the B200 kernels compute in float32");
    const auto dx = x.dimensions();
    const auto dy = y.dimensions();
    if (dx.size() < 2 || dy.size() != 2 || s.dimensions().size() < 2 || out->dimensions().size() < 2)
        return ffi::Error(ffi::ErrorCode::kInvalidArgument, "E3J_ERROR[InvalidArgument]: unexpected operand ranks");
    const int X = (int)dx[1], C = dx.size() > 2 ? (int)dx.back() : 1, Y = (int)dy[1];
    const int Z = (int)out->dimensions()[1], S = (int)s.dimensions()[1];
    TableShape t;
    if (!Describe(coef, 1, t))
        return ffi::Error(ffi::ErrorCode::kInvalidArgument, "E3J_ERROR[InvalidArgument]: unsupported (IDX, VAL) dtype pair");
    e3j_b200_plan *plan = nullptr;
    const auto pkey = std::make_pair((const void *)coef.untyped_data(), (size_t)t.nnz * t.row_bytes);
    if (TrustPointer()) {
        std::lock_guard<std::mutex> lock(g_mu);
        auto it = g_by_pointer.find(pkey);
        if (it != g_by_pointer.end()) plan = it->second;
    }
    if (!plan) {
        std::string host;
        if (auto e = FetchTable(coef.untyped_data(), pkey.second, stream, host); e.failure()) return e;
        plan = GetPlan(host, t.nnz, t.idx_bytes, X, Y, Z, S, C);
        if (!plan) return Status(E3J_B200_INVALID_ARGUMENT);
        std::lock_guard<std::mutex> lock(g_mu);
        g_by_pointer[pkey] = plan;
    }
    return Status(e3j_b200_conv_fwd(plan, x.typed_data<float>(), y.typed_data<float>(), s.typed_data<float>(),
                                    sender.typed_data(), receiver_ptr.typed_data(), out->typed_data<float>(),
                                    num_nodes, dy[0], debug, stream));
}

ffi::Error ConvolutionBwdImpl(cudaStream_t stream, ffi::ScratchAllocator scratch, ffi::AnyBuffer coef,
                              ffi::AnyBuffer x, ffi::AnyBuffer y, ffi::AnyBuffer s, ffi::AnyBuffer dm,
                              ffi::BufferR1<ffi::S32> recv_t, ffi::BufferR1<ffi::S32> sender_ptr_t,
                              ffi::BufferR1<ffi::S32> edge_perm, ffi::BufferR1<ffi::S32> /*coef_ranges*/,
                              ffi::Result<ffi::AnyBuffer> dxo, ffi::Result<ffi::AnyBuffer> dyo,
                              ffi::Result<ffi::AnyBuffer> dso, int32_t num_nodes, int32_t debug) {
    if (x.element_type() != ffi::F32 || dm.element_type() != ffi::F32)
        return ffi::Error(ffi::ErrorCode::kUnimplemented,
                          "E3J_ERROR[Unimplemented]: the B200 kernels compute in float32");
    const auto dx = x.dimensions();
    const auto dy = y.dimensions();
    const int X = (int)dx[1], C = dx.size() > 2 ? (int)dx.back() : 1, Y = (int)dy[1];
    const int Z = (int)dm.dimensions()[1], S = (int)s.dimensions()[1];
    const int64_t E = dy[0];
    const int32_t N = num_nodes;
    TableShape t;
    if (!Describe(coef, 3, t))
        return ffi::Error(ffi::ErrorCode::kInvalidArgument, "E3J_ERROR[InvalidArgument]: unsupported (IDX, VAL) dtype pair");
    // forward table from the dx-ordered one: rows {val, i = x row, j = out row, k, l} -> swap i and j
    std::string host;
    if (auto e = FetchTable(coef.untyped_data(), (size_t)t.nnz * t.row_bytes, stream, host); e.failure()) return e;
    for (int n = 0; n < t.nnz; n++) {
        char *row = &host[n * t.row_bytes];
        if (t.idx_bytes == 1) {
            std::swap(row[4], row[5]);
        } else {
            int32_t q[2];
            std::memcpy(q, row + 4, 8);
            std::swap(q[0], q[1]);
            std::memcpy(row + 4, q, 8);
        }
    }
    e3j_b200_plan *plan = GetPlan(host, t.nnz, t.idx_bytes, X, Y, Z, S, C);
    if (!plan) return Status(E3J_B200_INVALID_ARGUMENT);

    auto round = [](size_t b) { return (b + 255) / 256 * 256; };
    const size_t idx_bytes = round((size_t)E * 4), ptr_bytes = round(((size_t)N + 2) * 4);
    const size_t ws_bytes = e3j_b200_conv_bwd_workspace_bytes(plan, N, E);
    if (edge_perm.element_count() == 0 && E != 0) {
        // SENDER graph ordering (src/e3j/ops/convolution.py:413-425): the edges are stored sorted by
        // sender, `recv_t` holds their receivers and `sender_ptr_t` is the CSR of the stored order.
        // The per-edge pass walks receivers, so build the receiver-sorted view of the stored edges.
        const size_t tws_bytes = round(e3j_b200_csr_transpose_workspace_bytes(N, E));
        auto mem = scratch.Allocate(3 * idx_bytes + ptr_bytes + tws_bytes + ws_bytes, 256);
        if (!mem.has_value())
            return ffi::Error(ffi::ErrorCode::kResourceExhausted, "E3J_ERROR[Internal]: scratch allocation failed");
        char *base = static_cast<char *>(*mem);
        int32_t *sender = reinterpret_cast<int32_t *>(base);
        int32_t *receiver = reinterpret_cast<int32_t *>(base + idx_bytes);
        int32_t *perm_r = reinterpret_cast<int32_t *>(base + 2 * idx_bytes);
        int32_t *receiver_ptr = reinterpret_cast<int32_t *>(base + 3 * idx_bytes);
        void *tws = base + 3 * idx_bytes + ptr_bytes;
        void *workspace = base + 3 * idx_bytes + ptr_bytes + tws_bytes;
        int rc = e3j_b200_csr_untranspose(sender_ptr_t.typed_data(), nullptr, recv_t.typed_data(), N, E, sender,
                                          receiver, stream);
        if (rc) return Status(rc);
        rc = e3j_b200_csr_transpose(receiver, E, N, receiver_ptr, perm_r, tws, tws_bytes, stream);
        if (rc) return Status(rc);
        return Status(e3j_b200_conv_bwd_by_sender(plan, x.typed_data<float>(), y.typed_data<float>(),
                                                  s.typed_data<float>(), dm.typed_data<float>(), sender,
                                                  sender_ptr_t.typed_data(), receiver_ptr, perm_r,
                                                  dxo->typed_data<float>(), dyo->typed_data<float>(),
                                                  dso->typed_data<float>(), workspace, ws_bytes, N, N, E, debug,
                                                  stream));
    }
    auto mem = scratch.Allocate(2 * idx_bytes + ptr_bytes + ws_bytes, 256);
    if (!mem.has_value())
        return ffi::Error(ffi::ErrorCode::kResourceExhausted, "E3J_ERROR[Internal]: scratch allocation failed");
    char *base = static_cast<char *>(*mem);
    int32_t *sender = reinterpret_cast<int32_t *>(base);
    int32_t *receiver = reinterpret_cast<int32_t *>(base + idx_bytes);
    int32_t *receiver_ptr = reinterpret_cast<int32_t *>(base + 2 * idx_bytes);
    void *workspace = base + 2 * idx_bytes + ptr_bytes;

    int rc = e3j_b200_csr_untranspose(sender_ptr_t.typed_data(), edge_perm.typed_data(), recv_t.typed_data(), N, E,
                                      sender, receiver, stream);
    if (rc) return Status(rc);
    rc = e3j_b200_csr_ptr(receiver, E, N, receiver_ptr, stream);
    if (rc) return Status(rc);
    return Status(e3j_b200_conv_bwd(plan, x.typed_data<float>(), y.typed_data<float>(), s.typed_data<float>(),
                                    dm.typed_data<float>(), sender, receiver_ptr, sender_ptr_t.typed_data(),
                                    edge_perm.typed_data(), dxo->typed_data<float>(), dyo->typed_data<float>(),
                                    dso->typed_data<float>(), workspace, ws_bytes, N, E, debug, stream));
}

}  // namespace

XLA_FFI_DEFINE_HANDLER(e3j_b200_xla_convolution_impl, ConvolutionImpl,
                       ffi::Ffi::Bind()
                           .Ctx<ffi::PlatformStream<cudaStream_t>>()
                           .Arg<ffi::AnyBuffer>()            // coef
                           .Arg<ffi::AnyBuffer>()            // x
                           .Arg<ffi::AnyBuffer>()            // y
                           .Arg<ffi::AnyBuffer>()            // s
                           .Arg<ffi::BufferR1<ffi::S32>>()   // sender
                           .Arg<ffi::BufferR1<ffi::S32>>()   // receiver_ptr
                           .Arg<ffi::BufferR1<ffi::S32>>()   // coef_ranges (ignored)
                           .Ret<ffi::AnyBuffer>()            // out
                           .Attr<int32_t>("num_nodes")
                           .Attr<int32_t>("debug"));

XLA_FFI_DEFINE_HANDLER(e3j_b200_xla_convolution_bwd_impl, ConvolutionBwdImpl,
                       ffi::Ffi::Bind()
                           .Ctx<ffi::PlatformStream<cudaStream_t>>()
                           .Ctx<ffi::ScratchAllocator>()
                           .Arg<ffi::AnyBuffer>()            // coef (3 transposed tables)
                           .Arg<ffi::AnyBuffer>()            // x
                           .Arg<ffi::AnyBuffer>()            // y
                           .Arg<ffi::AnyBuffer>()            // s
                           .Arg<ffi::AnyBuffer>()            // dm
                           .Arg<ffi::BufferR1<ffi::S32>>()   // receivers in sender order
                           .Arg<ffi::BufferR1<ffi::S32>>()   // sender CSR offsets
                           .Arg<ffi::BufferR1<ffi::S32>>()   // edge_perm
                           .Arg<ffi::BufferR1<ffi::S32>>()   // coef_ranges (ignored)
                           .Ret<ffi::AnyBuffer>()            // dx
                           .Ret<ffi::AnyBuffer>()            // dy
                           .Ret<ffi::AnyBuffer>()            // ds
                           .Attr<int32_t>("num_nodes")
                           .Attr<int32_t>("debug"));

// C symbols of type XLA_FFI_Error* (*)(XLA_FFI_CallFrame*): what a PyCapsule handed to
// jax.ffi.register_ffi_target wraps (lib/e3j_ops/ffi/kernel_helpers.h:39-45).
extern "C" XLA_FFI_Error *e3j_b200_xla_convolution(XLA_FFI_CallFrame *frame) {
    return e3j_b200_xla_convolution_impl(frame);
}
extern "C" XLA_FFI_Error *e3j_b200_xla_convolution_bwd(XLA_FFI_CallFrame *frame) {
    return e3j_b200_xla_convolution_bwd_impl(frame);
}
