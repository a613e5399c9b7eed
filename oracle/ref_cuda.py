"""TEST / BENCH INFRASTRUCTURE: drives the reference's own CUDA kernels (oracle/_ref).

Restates the host-side preparation the reference's Python does before its FFI calls
(src/e3j/ops/convolution.py:166-208 and :366-404; src/e3j/ops/coef_ranges.py:54-198):
thread shape `launch_threads_x`, shared-memory estimate, the choice of `blockDim.y`
that minimises critical path / resident blocks, the longest-first assignment of whole
output rows to warps, and the three transposed tables of the backward pass.  Graph
transposition (argsort by sender) follows src/e3j/data/graph.py:59-72.
"""

from __future__ import annotations

import ctypes
import os

import numpy as np
import torch

from e3j_b200.coef import Coef4D

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libe3j_ref_conv.so")
_lib = None
MAX_BLOCK_Y = 16


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.ref_last_error.restype = ctypes.c_char_p
    return _lib


def launch_threads_x(channels):
    if channels // 4 >= 32 and channels % 4 == 0:
        n = 4
    elif channels // 2 >= 32 and channels % 2 == 0:
        n = 2
    else:
        n = 1
    return max(32, (channels // n // 32) * 32), n


def estimate_smem_bytes(load_elems, coef_elems, coef_bytes, val_bytes=4, extra_bytes=0):
    align = lambda v: -(-v // 16) * 16  # noqa: E731
    return sum(align(e * val_bytes) for e in load_elems) + extra_bytes + align(coef_elems * coef_bytes)


def _pass_rows(out_idx, num_coef):
    begins = [0] + [c for c in range(1, num_coef) if out_idx[c] != out_idx[c - 1]]
    ends = begins[1:] + [num_coef]
    return [(b, e - b) for b, e in zip(begins, ends)]


def _assign_rows(passes, num_coef, num_warps):
    rows = [_pass_rows(o, num_coef) for o in passes]
    loads = np.zeros((len(rows), num_warps), dtype=np.int64)
    assign = [[[] for _ in range(num_warps)] for _ in rows]
    items = [(w, p, r) for p in range(len(rows)) for r, (_b, w) in enumerate(rows[p])]
    items.sort(key=lambda it: (-it[0], it[1], it[2]))
    for weight, p, r in items:
        w = int(np.argmin(loads.sum(axis=0)))
        assign[p][w].append(r)
        loads[p, w] += weight
    perms, endpoints = [], np.empty((len(rows), num_warps), dtype=np.int32)
    for p, pass_rows in enumerate(rows):
        perm, cursor = [], 0
        for w in range(num_warps):
            for r in sorted(assign[p][w]):
                begin, weight = pass_rows[r]
                perm.extend(range(begin, begin + weight))
                cursor += weight
            endpoints[p, w] = cursor
        perms.append(np.asarray(perm, dtype=np.int64))
    return perms, endpoints, loads


def choose_block_y(passes, num_coef, channels, props, *, max_block_size, smem_bytes, registers):
    threads_x, _ = launch_threads_x(channels)
    cap = max(1, min(MAX_BLOCK_Y, max_block_size // threads_x))
    max_blocks_smem = max(1, props["smem_max"] // smem_bytes)

    def cost(y):
        crit = int(_assign_rows(passes, num_coef, y)[2].sum(axis=0).max())
        by_regs = max(1, props["regs_per_sm"] // (threads_x * y * registers))
        resident = max(1, min(props["max_blocks_per_sm"], max_blocks_smem, by_regs,
                              props["max_threads_per_sm"] // (threads_x * y)))  # fmt: skip
        return crit / resident

    def fits(y):
        warps = -(-threads_x * y // 32)
        return warps * (-(-32 * registers // 256) * 256) <= props["regs_per_sm"]

    return min((y for y in range(1, cap + 1) if y == 1 or fits(y)), key=cost)


class RefConvolution:
    """Forward / backward of the reference kernels for one table (uint8 indices, float32)."""

    def __init__(self, coef: Coef4D, dims, props: dict, device):
        self.X, self.Y, self.Z, self.S, self.C = dims
        self.dev = device
        c = Coef4D(coef.val, coef.idx, idx_dtype="uint8")
        nnz = len(c.val)
        self.nnz = nnz
        threads_x, n = launch_threads_x(self.C)
        unroll = min(threads_x * n, self.C)
        row_bytes = c.dtype.itemsize
        # forward
        smem = estimate_smem_bytes([unroll * self.X, self.Y, unroll * self.Z, unroll * self.S], nnz, row_bytes)
        regs = lib().ref_registers(0, n)
        out_idx = [c.idx[:, 0]]
        self.by_f = choose_block_y(out_idx, nnz, self.C, props, max_block_size=512, smem_bytes=smem, registers=regs)
        (perm,), ranges, _ = _assign_rows(out_idx, nnz, self.by_f)
        self.coef_f = torch.as_tensor(c.pack()[perm]).to(device)
        self.ranges_f = torch.as_tensor(ranges.reshape(-1).astype(np.int32)).to(device)
        # backward
        tabs = [c.transpose((1, 0, 2, 3)), c.transpose((2, 0, 1, 3)), c.transpose((3, 0, 2, 1))]
        passes = [t.idx[:, 0] for t in tabs]
        warps_x = max(1, threads_x // 32)
        smem_b = estimate_smem_bytes([unroll * self.Z, unroll * self.X, self.Y, unroll * self.S], 3 * nnz, row_bytes,
                                     extra_bytes=warps_x * self.Y * 4)  # fmt: skip
        regs_b = lib().ref_registers(1, n)
        self.by_b = choose_block_y(passes, nnz, self.C, props, max_block_size=1024, smem_bytes=smem_b, registers=regs_b)
        perms, ranges_b, _ = _assign_rows(passes, nnz, self.by_b)
        packed = np.stack([t.pack()[p] for t, p in zip(tabs, perms)])
        self.coef_b = torch.as_tensor(packed).to(device)
        self.ranges_b = torch.as_tensor(ranges_b.reshape(-1).astype(np.int32)).to(device)

    @staticmethod
    def _p(t):
        return ctypes.c_void_p(t.data_ptr())

    def _check(self, rc):
        if rc:
            raise RuntimeError("reference kernel: " + lib().ref_last_error().decode())

    def forward(self, x, y, s, sender, receiver_ptr):
        n, e = x.shape[0], y.shape[0]
        out = torch.empty((n, self.Z, self.C), device=self.dev)
        p = self._p
        self._check(lib().ref_conv_fwd(p(self.coef_f), p(x), p(y), p(s), p(sender), p(receiver_ptr), p(out), n,
                                       self.nnz, self.X, self.Y, self.Z, self.S, self.C, e, self.by_f, p(self.ranges_f),
                                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))  # fmt: skip
        return out

    def transpose_graph(self, sender, receiver, n):
        """What GraphCSR.transpose() yields: perm, receivers in sender order, sender CSR."""
        perm = torch.argsort(sender.to(torch.int64), stable=True).to(torch.int32)
        recv_t = receiver[perm.long()].contiguous()
        counts = torch.bincount(sender.to(torch.int64), minlength=n)
        ptr_t = torch.zeros(n + 1, dtype=torch.int64, device=sender.device)
        ptr_t[1:] = torch.cumsum(counts, 0)
        return perm, recv_t, ptr_t.to(torch.int32)

    def backward(self, x, y, s, dm, perm, recv_t, ptr_t):
        n, e = x.shape[0], y.shape[0]
        dx, dy, ds = torch.empty_like(x), torch.empty_like(y), torch.empty_like(s)
        p = self._p
        self._check(lib().ref_conv_bwd(p(self.coef_b), p(x), p(y), p(s), p(dm), p(recv_t), p(ptr_t), p(perm), p(dx),
                                       p(dy), p(ds), n, self.nnz, self.X, self.Y, self.Z, self.S, self.C, e, self.by_b,
                                       p(self.ranges_b), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))  # fmt: skip
        return dx, dy, ds
