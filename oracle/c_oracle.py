"""TEST INFRASTRUCTURE: ctypes front end of ``conv_oracle.c``."""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libconv_oracle.so")
_lib = None

COEF_DTYPE = np.dtype([("val", "f4"), ("i", "i4"), ("j", "i4"), ("k", "i4"), ("l", "i4")])


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "conv_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", _LIB_PATH], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.oracle_conv_fwd.restype = ctypes.c_int
        _lib.oracle_conv_bwd.restype = ctypes.c_int
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def pack_coef(val, idx4) -> np.ndarray:
    idx4 = np.asarray(idx4)
    out = np.zeros(len(val), COEF_DTYPE)
    out["val"] = val
    for n, name in enumerate("ijkl"):
        out[name] = idx4[:, n]
    return out


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def conv_fwd(val, idx4, x, y, s, sender, receiver_ptr, num_out, *, wide=True) -> np.ndarray:
    coef = pack_coef(val, idx4)
    x, y, s = _c(x, np.float32), _c(y, np.float32), _c(s, np.float32)
    sender, receiver_ptr = _c(sender, np.int32), _c(receiver_ptr, np.int32)
    n, nx, ch = x.shape
    out = np.empty((n, num_out, ch), np.float32)
    lib().oracle_conv_fwd(
        _p(coef), ctypes.c_int(len(coef)), _p(x), _p(y), _p(s), _p(sender), _p(receiver_ptr), _p(out),
        ctypes.c_int(n), ctypes.c_int64(y.shape[0]), ctypes.c_int(nx), ctypes.c_int(y.shape[1]),
        ctypes.c_int(num_out), ctypes.c_int(s.shape[1]), ctypes.c_int(ch), ctypes.c_int(int(wide)),
    )  # fmt: skip
    return out


def conv_bwd(val, idx4, x, y, s, dm, sender, receiver_ptr, sender_ptr_t, perm_t, *, wide=True):
    coef = pack_coef(val, idx4)
    x, y, s, dm = (_c(a, np.float32) for a in (x, y, s, dm))
    sender, receiver_ptr = _c(sender, np.int32), _c(receiver_ptr, np.int32)
    sender_ptr_t, perm_t = _c(sender_ptr_t, np.int32), _c(perm_t, np.int32)
    n, nx, ch = x.shape
    dx, dy, ds = np.empty_like(x), np.empty_like(y), np.empty_like(s)
    lib().oracle_conv_bwd(
        _p(coef), ctypes.c_int(len(coef)), _p(x), _p(y), _p(s), _p(dm), _p(sender), _p(receiver_ptr),
        _p(sender_ptr_t), _p(perm_t), _p(dx), _p(dy), _p(ds), ctypes.c_int(n), ctypes.c_int64(y.shape[0]),
        ctypes.c_int(nx), ctypes.c_int(y.shape[1]), ctypes.c_int(dm.shape[1]), ctypes.c_int(s.shape[1]),
        ctypes.c_int(ch), ctypes.c_int(int(wide)),
    )  # fmt: skip
    return dx, dy, ds


def transpose_csr(sender, num_nodes):
    """Stable sender-sorted view: (sender_ptr_t, perm_t) with perm_t[p] = original edge.
    Edges with an out-of-range sender fall outside every segment."""
    sender = np.asarray(sender, np.int64)
    ok = (sender >= 0) & (sender < num_nodes)
    key = np.where(ok, sender, num_nodes)
    perm = np.argsort(key, kind="stable").astype(np.int32)
    ptr = np.zeros(num_nodes + 1, np.int64)
    np.add.at(ptr, sender[ok] + 1, 1)
    return np.cumsum(ptr).astype(np.int32), perm
