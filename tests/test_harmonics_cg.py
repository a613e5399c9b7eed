"""Harmonics and Clebsch-Gordan tables: known values and structural invariants
(the reference checks these against e3nn-jax, tests/test_harmonics.py:162-216 and
tests/test_tensor_product.py:146-149; that package is unavailable, so published
closed forms and representation-theoretic identities are used instead)."""

import itertools

import numpy as np
import pytest

from e3j_b200.convolution import Convolution
from e3j_b200.harmonics import Harmonics, wigner_D
from e3j_b200.wigner import clebsch_gordan
from oracle import numpy_oracle


def _rot(rng):
    q, _ = np.linalg.qr(rng.normal(size=(3, 3)))
    if np.linalg.det(q) < 0:
        q[:, 0] *= -1
    return q


def test_low_degree_closed_forms():
    """Component-normalised real harmonics in the (y, z, x) frame: l = 1 is
    sqrt(3) r_hat, l = 2 has the familiar five quadratic forms."""
    rng = np.random.default_rng(0)
    r = rng.normal(size=(64, 3))
    r /= np.linalg.norm(r, axis=1, keepdims=True)
    y = Harmonics(2, normalize=False, normalization="component")(r)
    a, b, c = r.T
    assert np.allclose(y[:, 0], 1.0)
    assert np.allclose(y[:, 1:4], np.sqrt(3) * r)
    want = np.stack(
        [np.sqrt(15) * a * c, np.sqrt(15) * a * b, np.sqrt(5) * (b * b - 0.5 * (a * a + c * c)),
         np.sqrt(15) * b * c, np.sqrt(15) / 2 * (c * c - a * a)], axis=1)  # fmt: skip
    assert np.allclose(y[:, 4:9], want)


@pytest.mark.parametrize("normalization,norm2", [("component", lambda l: 2 * l + 1), ("norm", lambda l: 1.0),
                                                 ("integral", lambda l: (2 * l + 1) / (4 * np.pi))])  # fmt: skip
def test_normalisation(normalization, norm2):
    rng = np.random.default_rng(1)
    r = rng.normal(size=(16, 3))
    y = Harmonics(3, normalize=True, normalization=normalization)(r)
    for l in range(4):  # noqa: E741
        assert np.allclose(np.sum(y[:, l * l : (l + 1) ** 2] ** 2, axis=1), norm2(l), rtol=1e-5)


def test_equivariance_and_parity():
    rng = np.random.default_rng(2)
    r = rng.normal(size=(10, 3))
    rot = _rot(rng)
    h = Harmonics(3, normalize=True)
    y, yr, ym = h(r), h(r @ rot.T), h(-r)
    for l in range(4):  # noqa: E741
        sl = slice(l * l, (l + 1) ** 2)
        assert np.allclose(yr[:, sl], y[:, sl] @ wigner_D(l, rot).T, atol=1e-9)
        assert np.allclose(ym[:, sl], (-1) ** l * y[:, sl], atol=1e-12)


def test_harmonics_vjp_matches_finite_differences():
    rng = np.random.default_rng(3)
    r = rng.normal(size=(5, 3))
    dy = rng.normal(size=(5, 16))
    h = Harmonics(3, normalize=True)
    g = h.vjp(r, dy)
    num = np.zeros_like(r)
    eps = 1e-6
    for e, ax in itertools.product(range(5), range(3)):
        d = np.zeros_like(r)
        d[e, ax] = eps
        num[e, ax] = np.sum((h(r + d) - h(r - d)) * dy) / (2 * eps)
    assert np.allclose(g, num, atol=1e-6)


def test_safe_norm_at_origin_is_finite():
    y = Harmonics(3, normalize=True)(np.zeros((1, 3), np.float32))
    assert np.isfinite(y).all()


@pytest.mark.parametrize("l0,l1,l2", [t for t in itertools.product(range(4), repeat=3) if abs(t[1] - t[2]) <= t[0] <= t[1] + t[2]])
def test_clebsch_gordan_blocks(l0, l1, l2):
    c = clebsch_gordan(l0, l1, l2)
    assert np.isclose(np.linalg.norm(c), 1.0)
    # rows are orthogonal with equal norms: C C^T = I / (2 l0 + 1)
    m = c.reshape(2 * l0 + 1, -1)
    assert np.allclose(m @ m.T, np.eye(2 * l0 + 1) / (2 * l0 + 1), atol=1e-12)
    rot = _rot(np.random.default_rng(4))
    d0, d1, d2 = wigner_D(l0, rot), wigner_D(l1, rot), wigner_D(l2, rot)
    assert np.allclose(np.einsum("ijk,jb,kc->ibc", c, d1, d2), np.einsum("ia,abc->ibc", d0, c), atol=1e-9)


def test_clebsch_gordan_known_values():
    # 1 x 1 -> 0: delta / sqrt(3); 1 x 1 -> 1: Levi-Civita / sqrt(6); anything x 0: identity / sqrt(dim)
    assert np.allclose(clebsch_gordan(0, 1, 1)[0], np.eye(3) / np.sqrt(3))
    eps = np.zeros((3, 3, 3))
    for a, b, c in [(0, 1, 2), (1, 2, 0), (2, 0, 1)]:
        eps[a, b, c], eps[a, c, b] = 1, -1
    assert np.allclose(clebsch_gordan(1, 1, 1), eps / np.sqrt(6))
    assert np.allclose(clebsch_gordan(2, 2, 0)[:, :, 0], np.eye(5) / np.sqrt(5))


def test_products_of_harmonics_are_harmonics_with_positive_sign():
    """For l0 + l1 + l2 even, C . (Y_l1 (x) Y_l2) is a positive multiple of Y_l0
    (Gaunt integrals of the restated harmonics): fixes each block up to that sign."""
    rng = np.random.default_rng(5)
    r = rng.normal(size=(32, 3))
    r /= np.linalg.norm(r, axis=1, keepdims=True)
    y = Harmonics(3, normalization="integral")(r)
    sl = lambda l: slice(l * l, (l + 1) ** 2)  # noqa: E731, E741
    for l0, l1, l2 in itertools.product(range(4), repeat=3):
        if not abs(l1 - l2) <= l0 <= l1 + l2 or (l0 + l1 + l2) % 2:
            continue
        z = np.einsum("ijk,ej,ek->ei", clebsch_gordan(l0, l1, l2), y[:, sl(l1)], y[:, sl(l2)])
        ratio = np.sum(z * y[:, sl(l0)], axis=1) / np.sum(y[:, sl(l0)] ** 2, axis=1)
        assert np.allclose(z, ratio[:, None] * y[:, sl(l0)], atol=1e-12)
        assert (ratio > 0).all() and np.allclose(ratio, ratio[0])


def test_convolution_is_equivariant():
    """Rotating node features and edge vectors rotates the output
    (tests/test_convolution.py:153-167 of the reference), on the float64 oracle."""
    rng = np.random.default_rng(6)
    conv = Convolution(("0e+1o+2e", "0e+1o+2e+3o"), "0e+1o+2e+3o", graph_ordering="RECEIVER")
    n, e, c = 5, 14, 3
    snd, rcv = rng.integers(0, n, e), np.sort(rng.integers(0, n, e))
    vec = rng.normal(size=(e, 3))
    x = rng.normal(size=(n, 9, c))
    s = rng.normal(size=(e, conv.num_scalars, c))
    rot = _rot(rng)
    h = Harmonics(3, normalize=True)

    def block_diag(ls):
        out = np.zeros((sum(2 * l + 1 for l in ls),) * 2)
        o = 0
        for l in ls:  # noqa: E741
            out[o : o + 2 * l + 1, o : o + 2 * l + 1] = wigner_D(l, rot)
            o += 2 * l + 1
        return out

    dx = block_diag([0, 1, 2])
    dz = block_diag([ir.l for ir in conv._otimes.target_irreps])
    val, idx4 = conv.coef.val, conv.coef.idx
    out = numpy_oracle.conv_fwd(val, idx4, x, h(vec), s, snd, rcv, conv.target.dim)
    out_r = numpy_oracle.conv_fwd(val, idx4, np.einsum("ab,nbc->nac", dx, x), h(vec @ rot.T), s, snd, rcv, conv.target.dim)
    assert np.allclose(out_r, np.einsum("ab,nbc->nac", dz, out), atol=1e-6)
