"""Convolution over edge windows with the per-edge scalars produced on the fly.

At a million nodes the mixing scalars ``s`` (E, S, C) and their cotangent do not fit
in device memory (12 KB per edge each for the l <= 3 hidden layer), so the graph is
run as consecutive receiver ranges ("windows") whose edges fit a fixed budget: the
scalars of a window are produced right before the kernels read them, and in the
backward pass they are produced again, the window's ``ds`` is handed back to the
producer (which folds it into its parameter gradients) and both buffers are reused
for the next window.  The reference has no such mode: its operator takes ``s`` whole
(src/e3j/core/convolution.py:342-420).

`WindowedConvOps` has the call signature of `e3j_b200.halo.CudaConvOps`, with a
producer object in the place of the ``s`` tensor, so the partitioned operator
(`e3j_b200.halo.HaloConvolution`) runs windows without change.
"""

from __future__ import annotations

import ctypes
import math

import numpy as np
import torch

from . import _lib, ops
from .radial import SILU_2MOM


def plan_windows(receiver_ptr: np.ndarray, r_lo: int, r_hi: int, max_edges: int) -> list[tuple[int, int, int, int]]:
    """Greedy split of the receivers [r_lo, r_hi) into ranges of at most `max_edges`
    edges.  Returns (r0, r1, e0, e1) per window; a receiver with more edges than the
    budget is an error (its segment cannot be split)."""
    ptr = np.asarray(receiver_ptr, dtype=np.int64)
    out = []
    r0 = r_lo
    while r0 < r_hi:
        e0 = int(ptr[r0])
        # largest r1 <= r_hi with ptr[r1] - e0 <= max_edges
        r1 = int(np.searchsorted(ptr[r0 : r_hi + 1], e0 + max_edges, side="right")) - 1 + r0
        if r1 <= r0:
            raise ValueError(f"receiver {r0} has {int(ptr[r0 + 1]) - e0} edges, more than the window budget {max_edges}")
        out.append((r0, r1, e0, int(ptr[r1])))
        r0 = r1
    return out


def split_tf32(t: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """t = hi + lo exactly, with hi holding the top 10 mantissa bits (exact in TF32)."""
    hi = (t.view(torch.int32) & -8192).view(torch.float32)
    return hi, t - hi


class RadialProducer:
    """``s = radial MLP(enveloped Bessel basis)`` evaluated per window, and its parameter
    gradients accumulated window by window.

    rbf: (E, B) basis values of every local edge; w1 (B, H), w2 (H, S * C).

    `precision`: "fp32" evaluates the wide last layer as one fp32 matrix product;
    "tf32x3" evaluates it on the tensor cores as h_hi W_hi + h_hi W_lo + h_lo W_hi, the
    three products being one TF32 product over a three times longer inner dimension
    ([h_hi, h_hi, h_lo] [W_hi; W_lo; W_hi]) with fp32 accumulation; the dropped lo x lo
    term and the rounding of the lo parts are of relative size 2^-20.  The backward
    products are fp32 in both modes.
    """

    def __init__(self, rbf: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, precision: str = "fp32"):
        if precision not in ("fp32", "tf32x3"):
            raise ValueError(f"unknown precision {precision!r}")
        self.rbf, self.w1, self.w2, self.precision = rbf, w1, w2, precision
        self.a1 = 1.0 / math.sqrt(w1.shape[0])
        self.a2 = 1.0 / math.sqrt(w2.shape[0])
        self.w2s = (w2 * self.a2).contiguous()
        if precision == "tf32x3":
            hi, lo = split_tf32(self.w2s)
            self.w2s3 = torch.cat([hi, lo, hi], dim=0).contiguous()
        self.dw1 = torch.zeros_like(w1)
        self.dw2 = torch.zeros_like(w2)

    def zero_grad(self) -> None:
        self.dw1.zero_()
        self.dw2.zero_()

    def _hidden(self, e0: int, e1: int):
        pre = (self.rbf[e0:e1] @ self.w1) * self.a1
        return pre, SILU_2MOM * torch.nn.functional.silu(pre)

    def forward(self, e0: int, e1: int, s_w: torch.Tensor) -> None:
        """Fills `s_w` (e1 - e0, S, C)."""
        _, h = self._hidden(e0, e1)
        if self.precision == "fp32":
            torch.matmul(h, self.w2s, out=s_w.view(e1 - e0, -1))
            return
        hi, lo = split_tf32(h)
        h3 = torch.cat([hi, hi, lo], dim=1)
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True
        try:
            torch.matmul(h3, self.w2s3, out=s_w.view(e1 - e0, -1))
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev

    def backward(self, e0: int, e1: int, ds_w: torch.Tensor) -> None:
        """Adds this window's contribution to dw1, dw2."""
        pre, h = self._hidden(e0, e1)
        d = ds_w.view(e1 - e0, -1)
        self.dw2.addmm_(h.t(), d, alpha=self.a2)
        dh = d @ self.w2s.t()
        sig = torch.sigmoid(pre)
        dpre = dh * (SILU_2MOM * sig * (1 + pre * (1 - sig)))
        self.dw1.addmm_(self.rbf[e0:e1].t(), dpre, alpha=self.a1)


class TensorProducer:
    """Scalars that already exist as one tensor (small graphs, tests): windows are
    copied out of it, and the ds windows are written back into `ds`."""

    def __init__(self, s: torch.Tensor, ds: torch.Tensor | None = None):
        self.s, self.ds = s, ds

    def forward(self, e0, e1, s_w):
        s_w.copy_(self.s[e0:e1])

    def backward(self, e0, e1, ds_w):
        if self.ds is not None:
            self.ds[e0:e1].copy_(ds_w)


class WindowedConvOps:
    """Forward / backward over receiver windows through the C ABI
    (`e3j_b200_conv_fwd_window`, `e3j_b200_conv_bwd_window`)."""

    def __init__(self, plan: ops.ConvPlan, max_edges: int):
        self.plan, self.max_edges = plan, int(max_edges)
        self._ptr_host = {}
        self._s = self._ds = self._ws = None
        self.windows_run = 0

    def _host_ptr(self, receiver_ptr: torch.Tensor) -> np.ndarray:
        key = (receiver_ptr.data_ptr(), receiver_ptr.numel())
        if key not in self._ptr_host:
            self._ptr_host[key] = receiver_ptr.cpu().numpy().astype(np.int64)
        return self._ptr_host[key]

    def _buffers(self, device, need_bwd: bool):
        _, _, _, S, C = self.plan.dims
        if self._s is None:
            self._s = torch.empty((self.max_edges, S, C), device=device, dtype=torch.float32)
        if need_bwd and self._ds is None:
            self._ds = torch.empty((self.max_edges, S, C), device=device, dtype=torch.float32)
            need = int(_lib.lib().e3j_b200_conv_bwd_workspace_bytes(self.plan.handle, 1, self.max_edges))
            self._ws = torch.empty(need, dtype=torch.uint8, device=device)

    def forward(self, x, y, producer, sender, receiver_ptr, out, r0: int, r1: int, n_send: int) -> None:
        if r1 <= r0:
            return
        _, Y, Z, _, C = self.plan.dims
        self._buffers(x.device, False)
        vp = ctypes.c_void_p
        for w0, w1, e0, e1 in plan_windows(self._host_ptr(receiver_ptr), r0, r1, self.max_edges):
            s_w = self._s[: e1 - e0]
            if e1 > e0:
                producer.forward(e0, e1, s_w)
            _lib.check(_lib.lib().e3j_b200_conv_fwd_window(
                self.plan.handle, ops._ptr(x), vp(y.data_ptr() + 4 * e0 * Y), ops._ptr(s_w),
                vp(sender.data_ptr() + 4 * e0), vp(receiver_ptr.data_ptr() + 4 * w0),
                vp(out.data_ptr() + 4 * w0 * Z * C), w1 - w0, n_send, e0, e1 - e0, ops.DEBUG_LEVEL, ops._stream()))  # fmt: skip
            self.windows_run += 1

    def backward(self, x, y, producer, dm, sender, receiver_ptr, sender_ptr_t, perm_t, dx, dy, ds, n_recv, n_send) -> None:
        """`ds` is ignored (each window's ds goes to `producer.backward`)."""
        _, Y, Z, _, C = self.plan.dims
        self._buffers(x.device, True)
        vp = ctypes.c_void_p
        windows = plan_windows(self._host_ptr(receiver_ptr), 0, n_recv, self.max_edges)
        if not windows:
            dx.zero_()
            return
        for k, (w0, w1, e0, e1) in enumerate(windows):
            s_w, ds_w = self._s[: e1 - e0], self._ds[: e1 - e0]
            if e1 > e0:
                producer.forward(e0, e1, s_w)
            _lib.check(_lib.lib().e3j_b200_conv_bwd_window(
                self.plan.handle, ops._ptr(x), vp(y.data_ptr() + 4 * e0 * Y), ops._ptr(s_w),
                vp(dm.data_ptr() + 4 * w0 * Z * C), vp(sender.data_ptr() + 4 * e0),
                vp(receiver_ptr.data_ptr() + 4 * w0), ops._ptr(sender_ptr_t), ops._ptr(perm_t), ops._ptr(dx),
                vp(dy.data_ptr() + 4 * e0 * Y), ops._ptr(ds_w), ops._ptr(self._ws), self._ws.numel(),
                w1 - w0, n_send, e0, e1 - e0, int(k > 0), ops.DEBUG_LEVEL, ops._stream()))  # fmt: skip
            if e1 > e0:
                producer.backward(e0, e1, ds_w)
            self.windows_run += 1
        tail = windows[-1][3]
        if tail < dy.shape[0]:  # edges of no receiver (padding): exact zeros
            dy[tail:].zero_()
