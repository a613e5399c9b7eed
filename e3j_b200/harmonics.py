"""Real solid harmonics in the e3nn (y, z, x) convention, as explicit polynomials.

The reference builds complex harmonic polynomials from the top weight
``(X + iY)**l`` by repeated application of the lowering operator and then
forms real combinations (src/e3j/utils/spherical_harmonics.py:27-147), with the
physical axes ``(X, Y, Z)`` mapped to the input components ``(z, x, y)``
(:29-46).  ``Harmonics`` evaluates them on (optionally normalised) edge
vectors with a per-degree factor (src/e3j/core/harmonics.py:26-101).

This module restates that construction with a tiny dictionary polynomial
algebra and then expands every component into real monomials
``coef * a**i * b**j * c**k`` of the input vector ``r = (a, b, c)``.  The
monomial table is what both the CPU evaluation here and the CUDA kernel
(`e3j_b200_harmonics_fwd/bwd`) consume, so the two sides share one definition.
"""

from __future__ import annotations

import functools
import math

import numpy as np

from .spaces import O3Space, full_space

# ---------------------------------------------------------------------------
# complex harmonics in the generator basis  u = X - iY, v = Z, w = X + iY
# polynomial = {(p, q, r): complex}  meaning  sum coef * u**p v**q w**r
# ---------------------------------------------------------------------------


def _lower(poly: dict) -> dict:
    """Lowering operator J_- by the Leibniz rule with
    J_-(w) = -2 v, J_-(u) = 0, J_-(v) = u
    (src/e3j/utils/spherical_harmonics.py:84-116)."""
    out: dict = {}
    for (p, q, r), c in poly.items():
        if r > 0:
            key = (p, q + 1, r - 1)
            out[key] = out.get(key, 0) + (-2 * r) * c
        if q > 0:
            key = (p + 1, q - 1, r)
            out[key] = out.get(key, 0) + q * c
    return out


def _scale(poly: dict, s) -> dict:
    return {k: s * c for k, c in poly.items()}


def _add(a: dict, b: dict) -> dict:
    out = dict(a)
    for k, c in b.items():
        out[k] = out.get(k, 0) + c
    return out


def _norm_s2(l: int) -> float:  # noqa: E741
    """L2 norm on the unit sphere of (x + iy)**l: sqrt(4 pi (2l)!! / (2l+1)!!)
    (src/e3j/utils/spherical_harmonics.py:133-147)."""
    even = (2**l) * math.factorial(l)  # (2l)!!
    odd = math.factorial(2 * l + 1) / even  # (2l+1)!!
    return math.sqrt(4 * math.pi * even / odd)


@functools.cache
def complex_harmonic(l: int, m: int) -> dict:  # noqa: E741
    """Y_l^m as a generator-basis polynomial, unit L2 norm on the sphere."""
    if m == l:
        return {(0, 0, l): 1.0 / _norm_s2(l)}
    ladder = math.sqrt((l + m + 1) * (l - m))  # c_(l, m+1)
    return _scale(_lower(complex_harmonic(l, m + 1)), 1.0 / ladder)


@functools.cache
def real_harmonic(l: int, m: int) -> dict:  # noqa: E741
    """Real combination with the reference's sign rule
    (src/e3j/utils/spherical_harmonics.py:64-75)."""
    sign = (-1) ** (l + m) if m >= 0 else (-1) ** (l + 1)
    if m == 0:
        return _scale(complex_harmonic(l, 0), sign)
    ylm, yl_m = complex_harmonic(l, m), complex_harmonic(l, -m)
    if m > 0:
        return _scale(_add(ylm, _scale(yl_m, (-1) ** m)), sign * math.sqrt(0.5))
    return _scale(_add(ylm, _scale(yl_m, -((-1) ** m))), sign * (-1j) * math.sqrt(0.5))


# ---------------------------------------------------------------------------
# expansion into real monomials of the input components (a, b, c)
# X = c, Y = a, Z = b   =>   u = c - i a, v = b, w = c + i a
# ---------------------------------------------------------------------------


def _binomial_expand(p: int, r: int) -> dict:
    """(c - i a)**p (c + i a)**r  ->  {(i_a, k_c): complex}."""
    out: dict = {}
    for s in range(p + 1):
        cs = math.comb(p, s) * (-1j) ** s
        for t in range(r + 1):
            ct = math.comb(r, t) * (1j) ** t
            key = (s + t, p + r - s - t)
            out[key] = out.get(key, 0) + cs * ct
    return out


@functools.cache
def real_monomials(l: int, m: int) -> tuple[tuple[float, int, int, int], ...]:  # noqa: E741
    """Y_lm(a, b, c) = sum coef * a**i b**j c**k, as a sorted tuple of
    ``(coef, i, j, k)``; imaginary parts cancel and are checked."""
    acc: dict = {}
    for (p, q, r), c in real_harmonic(l, m).items():
        for (ia, kc), e in _binomial_expand(p, r).items():
            key = (ia, q, kc)
            acc[key] = acc.get(key, 0) + c * e
    out = []
    for (i, j, k), c in sorted(acc.items()):
        if abs(c.imag) > 1e-12:
            raise AssertionError(f"non-real coefficient in Y({l},{m})")
        if abs(c.real) > 1e-14:
            out.append((float(c.real), i, j, k))
    return tuple(out)


def _normalization_factor(l: int, normalization: str) -> float:  # noqa: E741
    """Per-degree factor relative to the unit-integral convention
    (src/e3j/core/harmonics.py:26-42)."""
    if normalization == "integral":
        return 1.0
    if normalization == "component":
        return math.sqrt(4 * math.pi)
    if normalization == "norm":
        return math.sqrt(4 * math.pi / (2 * l + 1))
    raise NotImplementedError(
        f"We don't support {normalization} normalization for now. "
        'We only support "integral", "component" and "norm"'
    )


SAFE_NORM_EPS = 1e-7  # src/e3j/utils/safe.py:24-46


class Harmonics:
    """Evaluate real harmonic polynomials on a 3D point cloud.

    Mirrors ``e3j.core.Harmonics(target, normalize, normalization)``
    (src/e3j/core/harmonics.py:45-101) for real harmonics.  ``target`` is an
    integer ``l_max`` or an irreps string of multiplicity-1 blocks.
    """

    def __init__(self, target, normalize: bool = False, normalization: str = "component"):
        self.target = full_space(target) if isinstance(target, int) else O3Space(target)
        self.normalize = normalize
        self.normalization = normalization
        coef, expo, comp = [], [], []
        row = 0
        for mul, ir in self.target:
            if mul != 1:
                raise ValueError("Harmonics target must have multiplicity-1 blocks")
            f = _normalization_factor(ir.l, normalization)
            for m in range(-ir.l, ir.l + 1):
                for c, i, j, k in real_monomials(ir.l, m):
                    coef.append(f * c)
                    expo.append((i, j, k))
                    comp.append(row)
                row += 1
        self.dim = row
        #: monomial table: value, exponents (i, j, k) of (a, b, c), output row
        self.mono_coef = np.asarray(coef, dtype=np.float64)
        self.mono_exp = np.asarray(expo, dtype=np.int32).reshape(-1, 3)
        self.mono_row = np.asarray(comp, dtype=np.int32)
        self.max_degree = int(self.mono_exp.sum(axis=1).max()) if len(coef) else 0

    # -- numpy evaluation (float64 or float32 following the input) ----------
    def project(self, r: np.ndarray) -> np.ndarray:
        if not self.normalize:
            return r
        norm = np.sqrt(np.sum(r * r, axis=-1) + r.dtype.type(SAFE_NORM_EPS))
        return r / norm[:, None]

    def polynomial(self, u: np.ndarray) -> np.ndarray:
        powers = [np.ones_like(u)]
        for _ in range(self.max_degree):
            powers.append(powers[-1] * u)
        pw = np.stack(powers, axis=0)  # [deg, E, 3]
        e = self.mono_exp
        terms = pw[e[:, 0], :, 0] * pw[e[:, 1], :, 1] * pw[e[:, 2], :, 2]  # [M, E]
        terms = terms * self.mono_coef.astype(u.dtype)[:, None]
        out = np.zeros((self.dim, u.shape[0]), dtype=u.dtype)
        np.add.at(out, self.mono_row, terms)
        return np.ascontiguousarray(out.T)

    def __call__(self, r: np.ndarray) -> np.ndarray:
        r = np.asarray(r)
        return self.polynomial(self.project(r))

    def cuda(self, r):
        """Evaluate on a CUDA tensor (E, 3) -> (E, dim) with the library kernel; differentiable
        with respect to `r` (first order)."""
        import torch

        key = str(r.device)
        cache = self.__dict__.setdefault("_device_tables", {})
        if key not in cache:
            e = self.mono_exp.astype(np.int64)
            desc = (e[:, 0] | (e[:, 1] << 4) | (e[:, 2] << 8) | (self.mono_row.astype(np.int64) << 12)).astype(np.int32)
            cache[key] = (torch.as_tensor(self.mono_coef.astype(np.float32)).to(r.device),
                          torch.as_tensor(desc).to(r.device))  # fmt: skip
        coef, desc = cache[key]
        return _HarmonicsFn.get().apply(r, coef, desc, self.dim, self.normalize)

    def vjp(self, r: np.ndarray, dy: np.ndarray) -> np.ndarray:
        """Cotangent of ``r`` given the cotangent ``dy`` of the output."""
        r = np.asarray(r)
        u = self.project(r)
        powers = [np.ones_like(u)]
        for _ in range(self.max_degree):
            powers.append(powers[-1] * u)
        pw = np.stack(powers, axis=0)
        e = self.mono_exp
        g = dy.T[self.mono_row] * self.mono_coef.astype(u.dtype)[:, None]  # [M, E]
        du = np.zeros_like(u)
        for ax in range(3):
            ee = e.copy()
            k = ee[:, ax].copy()
            ee[:, ax] = np.maximum(k - 1, 0)
            t = pw[ee[:, 0], :, 0] * pw[ee[:, 1], :, 1] * pw[ee[:, 2], :, 2]
            du[:, ax] = np.sum(g * t * k.astype(u.dtype)[:, None], axis=0)
        if not self.normalize:
            return du
        n = np.sqrt(np.sum(r * r, axis=-1) + r.dtype.type(SAFE_NORM_EPS))[:, None]
        # u = r / n  =>  dr = du / n - r (r . du) / n**3
        return du / n - r * np.sum(r * du, axis=-1, keepdims=True) / n**3


class _HarmonicsFn:
    """Lazy holder of the torch autograd function (torch is imported on first use)."""

    fn = None

    @classmethod
    def get(cls):
        if cls.fn is None:
            import ctypes

            import torch

            from . import _lib

            def ptr(t):
                return ctypes.c_void_p(t.data_ptr())

            def stream():
                return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

            class HarmonicsFunction(torch.autograd.Function):
                @staticmethod
                def forward(ctx, r, coef, desc, dim, normalize):
                    if r.device.type != "cuda":
                        raise RuntimeError("Harmonics.cuda runs on CUDA tensors only; use __call__ for numpy arrays")
                    r = r.contiguous().float()
                    y = torch.empty((r.shape[0], dim), device=r.device, dtype=torch.float32)
                    with torch.cuda.device(r.device):
                        _lib.check(_lib.lib().e3j_b200_harmonics_fwd(ptr(coef), ptr(desc), coef.numel(), dim,
                                                                      int(normalize), ptr(r), ptr(y), r.shape[0], stream()))  # fmt: skip
                    ctx.save_for_backward(r, coef, desc)
                    ctx.meta = (dim, normalize)
                    return y

                @staticmethod
                def backward(ctx, dy):
                    r, coef, desc = ctx.saved_tensors
                    dim, normalize = ctx.meta
                    dy = dy.contiguous().float()
                    dr = torch.empty_like(r)
                    with torch.cuda.device(r.device):
                        _lib.check(_lib.lib().e3j_b200_harmonics_bwd(ptr(coef), ptr(desc), coef.numel(), dim,
                                                                      int(normalize), ptr(r), ptr(dy), ptr(dr), r.shape[0], stream()))  # fmt: skip
                    return dr, None, None, None, None

            cls.fn = HarmonicsFunction
        return cls.fn


def wigner_D(l: int, rot: np.ndarray, *, seed: int = 0) -> np.ndarray:  # noqa: E741, N802
    """Representation matrix D with ``Y_l(R r) = D Y_l(r)``, recovered by least
    squares from the harmonics themselves (float64).  Used by the equivariance
    checks; plays the role of ``O3Space.action`` (src/e3j/spaces/o3.py:232-238)."""
    rng = np.random.default_rng(seed)
    pts = rng.normal(size=(8 * (2 * l + 1), 3))
    pts /= np.linalg.norm(pts, axis=-1, keepdims=True)
    h = Harmonics(f"{l}{'e' if l % 2 == 0 else 'o'}", normalization="integral")
    a = h(pts)  # [P, 2l+1]
    b = h(pts @ rot.T)
    sol, *_ = np.linalg.lstsq(a, b, rcond=None)
    return sol.T
