"""A hand-built XLA FFI call frame (ctypes), standing in for the XLA runtime in tests.

Mirrors the C structs of the XLA FFI API version 0.2 (xla/ffi/api/c_api.h: XLA_FFI_Api,
XLA_FFI_CallFrame, XLA_FFI_Buffer, XLA_FFI_Scalar, ...) and provides the few API callbacks a
stream-ordered handler uses: error creation, stream lookup, scratch allocation.
"""

import ctypes as C

import torch

DTYPES = {torch.float32: 11, torch.int32: 4, torch.uint8: 6, torch.float64: 12, torch.float16: 10}
S32 = 4


class ByteSpan(C.Structure):
    _fields_ = [("ptr", C.c_char_p), ("len", C.c_size_t)]


class Buffer(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("dtype", C.c_int),
                ("data", C.c_void_p), ("rank", C.c_int64), ("dims", C.POINTER(C.c_int64))]  # fmt: skip


class Scalar(C.Structure):
    _fields_ = [("dtype", C.c_int), ("value", C.c_void_p)]


class Args(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("size", C.c_int64),
                ("types", C.POINTER(C.c_int)), ("args", C.POINTER(C.c_void_p))]  # fmt: skip


class Attrs(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("size", C.c_int64),
                ("types", C.POINTER(C.c_int)), ("names", C.POINTER(C.POINTER(ByteSpan))),
                ("attrs", C.POINTER(C.c_void_p))]  # fmt: skip


class ApiVersion(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("major", C.c_int), ("minor", C.c_int)]


FN = C.CFUNCTYPE(C.c_void_p, C.c_void_p)  # XLA_FFI_Error* fn(Args*)
API_FUNCTIONS = ["Error_Create", "Error_GetMessage", "Error_Destroy", "Handler_Register", "Stream_Get",
                 "Type_Register", "ExecutionContext_Get", "State_Set", "State_Get", "DeviceMemory_Allocate",
                 "DeviceMemory_Free", "ThreadPool_Schedule", "ThreadPool_NumThreads", "Future_Create",
                 "Future_SetAvailable", "Future_SetError", "RunId_Get", "DeviceOrdinal_Get"]  # fmt: skip


class Api(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("api_version", ApiVersion),
                ("internal_api", C.c_void_p)] + [(n, FN) for n in API_FUNCTIONS]  # fmt: skip


class CallFrame(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("api", C.POINTER(Api)),
                ("ctx", C.c_void_p), ("stage", C.c_int), ("args", Args), ("rets", Args), ("attrs", Attrs),
                ("future", C.c_void_p)]  # fmt: skip


class ErrorCreateArgs(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("message", C.c_char_p), ("errc", C.c_int)]


class StreamGetArgs(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("ctx", C.c_void_p), ("stream", C.c_void_p)]


class AllocArgs(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("ctx", C.c_void_p),
                ("size", C.c_size_t), ("alignment", C.c_size_t), ("data", C.c_void_p)]  # fmt: skip


class FreeArgs(C.Structure):
    _fields_ = [("struct_size", C.c_size_t), ("extension_start", C.c_void_p), ("ctx", C.c_void_p),
                ("size", C.c_size_t), ("data", C.c_void_p)]  # fmt: skip


class FakeRuntime:
    """Owns the API table and whatever a call allocates; collects errors as (code, message)."""

    def __init__(self, device):
        self.device = device
        self.errors = []
        self.scratch = {}
        self.allocated_bytes = 0
        self._keep = []

        def error_create(p):
            a = C.cast(p, C.POINTER(ErrorCreateArgs)).contents
            self.errors.append((a.errc, a.message.decode()))
            return len(self.errors)  # any non-null token

        def stream_get(p):
            a = C.cast(p, C.POINTER(StreamGetArgs)).contents
            a.stream = torch.cuda.current_stream(self.device).cuda_stream
            return None

        def allocate(p):
            a = C.cast(p, C.POINTER(AllocArgs)).contents
            t = torch.empty(max(int(a.size), 1) + 256, dtype=torch.uint8, device=self.device)
            addr = (t.data_ptr() + 255) // 256 * 256
            self.scratch[addr] = t
            self.allocated_bytes += int(a.size)
            a.data = addr
            return None

        def free(p):
            a = C.cast(p, C.POINTER(FreeArgs)).contents
            self.scratch.pop(a.data, None)
            return None

        def unsupported(p):
            self.errors.append((-1, "unexpected API call"))
            return len(self.errors)

        table = {"Error_Create": error_create, "Stream_Get": stream_get, "DeviceMemory_Allocate": allocate,
                 "DeviceMemory_Free": free}  # fmt: skip
        self.api = Api()
        self.api.struct_size = C.sizeof(Api)
        self.api.api_version = ApiVersion(C.sizeof(ApiVersion), None, 0, 2)
        for name in API_FUNCTIONS:
            fn = FN(table.get(name, unsupported))
            self._keep.append(fn)
            setattr(self.api, name, fn)

    def call(self, handler, args, rets, attrs):
        """`args` / `rets`: lists of torch tensors; `attrs`: dict name -> int32.  Returns the list of errors."""
        keep = []

        def buffers(tensors):
            n = len(tensors)
            types = (C.c_int * n)(*([1] * n))
            ptrs = (C.c_void_p * n)()
            for i, t in enumerate(tensors):
                dims = (C.c_int64 * max(t.ndim, 1))(*t.shape)
                b = Buffer(C.sizeof(Buffer), None, DTYPES[t.dtype], t.data_ptr() if t.numel() else None, t.ndim, dims)
                keep.extend([dims, b])
                ptrs[i] = C.addressof(b)
            keep.extend([types, ptrs])
            return Args(C.sizeof(Args), None, n, types, ptrs)

        names = sorted(attrs)
        n = len(names)
        atypes = (C.c_int * n)(*([3] * n))  # XLA_FFI_AttrType_SCALAR
        anames = (C.POINTER(ByteSpan) * n)()
        avals = (C.c_void_p * n)()
        for i, name in enumerate(names):
            raw = name.encode()
            span = ByteSpan(raw, len(raw))
            val = C.c_int32(attrs[name])
            sc = Scalar(S32, C.addressof(val))
            keep.extend([raw, span, val, sc])
            anames[i] = C.pointer(span)
            avals[i] = C.addressof(sc)
        frame = CallFrame()
        frame.struct_size = CallFrame.future.offset  # XLA_FFI_CallFrame_STRUCT_SIZE ends with `attrs`
        frame.api = C.pointer(self.api)
        frame.ctx = None
        frame.stage = 3  # XLA_FFI_ExecutionStage_EXECUTE
        frame.args = buffers(args)
        frame.rets = buffers(rets)
        frame.attrs = Attrs(C.sizeof(Attrs), None, n, atypes, anames, avals)
        self.errors = []
        handler.restype = C.c_void_p
        handler.argtypes = [C.c_void_p]
        handler(C.byref(frame))
        return list(self.errors)
