"""Real Clebsch-Gordan tensors in the e3nn convention.

The reference takes these values from the third-party package e3nn-jax
(pinned 0.21.0 in uv.lock:440-441) at src/e3j/core/tensor_product.py:238,
``e3nn.clebsch_gordan(l0, l1, l2)``.  That package is not vendored with the
reference, so its published algorithm is restated here:

  1. SU(2) Clebsch-Gordan coefficients <j1 m1 j2 m2 | j3 m3> by Racah's
     closed formula (Condon-Shortley phases), exact rational arithmetic
     under the square root;
  2. change of basis from complex to real harmonics in the (y, z, x) frame
     with the extra factor (-i)**l that makes the result real;
  3. Frobenius normalisation of each (l1, l2, l3) block to 1.

What is verified locally (tests): realness, unit norm, orthogonality of the
output rows, equivariance against the Wigner matrices of the restated
harmonics, and proportionality to the Gaunt integrals of those harmonics.
The absolute sign of each block relative to e3nn-jax 0.21.0 cannot be checked
without that package: parity unpinned for that sign only.
"""

from __future__ import annotations

import functools
import math
from fractions import Fraction

import numpy as np


def _f(n) -> int:
    return math.factorial(round(n))


def _su2_cg(j1, m1, j2, m2, j3, m3) -> float:
    """<j1 m1 j2 m2 | j3 m3> (Racah 1942)."""
    if m3 != m1 + m2:
        return 0.0
    vmin = int(max(-j1 + j2 + m3, -j1 + m1, 0))
    vmax = int(min(j2 + j3 + m1, j3 - j1 + j2, j3 + m3))
    pref = (2 * j3 + 1) * Fraction(
        _f(j3 + j1 - j2) * _f(j3 - j1 + j2) * _f(j1 + j2 - j3) * _f(j3 + m3) * _f(j3 - m3),
        _f(j1 + j2 + j3 + 1) * _f(j1 - m1) * _f(j1 + m1) * _f(j2 - m2) * _f(j2 + m2),
    )
    total = Fraction(0)
    for v in range(vmin, vmax + 1):
        total += (-1) ** int(v + j2 + m2) * Fraction(
            _f(j2 + j3 + m1 - v) * _f(j1 - m1 + v),
            _f(v) * _f(j3 - j1 + j2 - v) * _f(j3 + m3 - v) * _f(v + j1 - j2 - m3),
        )
    return math.sqrt(pref) * float(total)


@functools.cache
def su2_clebsch_gordan(j1: int, j2: int, j3: int) -> np.ndarray:
    mat = np.zeros((2 * j1 + 1, 2 * j2 + 1, 2 * j3 + 1))
    if abs(j1 - j2) <= j3 <= j1 + j2:
        for m1 in range(-j1, j1 + 1):
            for m2 in range(-j2, j2 + 1):
                if abs(m1 + m2) <= j3:
                    mat[j1 + m1, j2 + m2, j3 + m1 + m2] = _su2_cg(j1, m1, j2, m2, j3, m1 + m2)
    return mat


@functools.cache
def change_basis_real_to_complex(l: int) -> np.ndarray:  # noqa: E741
    """Unitary taking real-harmonic coordinates to complex ones, times (-i)**l."""
    q = np.zeros((2 * l + 1, 2 * l + 1), dtype=np.complex128)
    s = 1 / math.sqrt(2)
    for m in range(-l, 0):
        q[l + m, l + abs(m)] = s
        q[l + m, l - abs(m)] = -1j * s
    q[l, l] = 1
    for m in range(1, l + 1):
        q[l + m, l + abs(m)] = (-1) ** m * s
        q[l + m, l - abs(m)] = 1j * (-1) ** m * s
    return (-1j) ** l * q


@functools.cache
def clebsch_gordan(l1: int, l2: int, l3: int) -> np.ndarray:
    """Real tensor of shape (2 l1 + 1, 2 l2 + 1, 2 l3 + 1), Frobenius norm 1,
    zero unless |l2 - l3| <= l1 <= l2 + l3.  float64."""
    if not abs(l2 - l3) <= l1 <= l2 + l3:
        return np.zeros((2 * l1 + 1, 2 * l2 + 1, 2 * l3 + 1))
    c = su2_clebsch_gordan(l1, l2, l3)
    q1 = change_basis_real_to_complex(l1)
    q2 = change_basis_real_to_complex(l2)
    q3 = change_basis_real_to_complex(l3)
    c = np.einsum("ij,kl,mn,ikn->jlm", q1, q2, np.conj(q3.T), c)
    if np.abs(c.imag).max() > 1e-9:
        raise AssertionError("complex Clebsch-Gordan tensor after change of basis")
    c = np.real(c)
    c[np.abs(c) < 1e-14] = 0.0
    return c / np.linalg.norm(c)
