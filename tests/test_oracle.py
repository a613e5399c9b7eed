"""The oracle against the reference's fixture, the committed vectors and an
independent autograd derivation."""

import os

import numpy as np
import pytest
import torch

from oracle import c_oracle, numpy_oracle
from tests.conftest import assert_close, csr_ptr, random_graph, random_table
from tests.golden import strip_fixture

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "conv_small.npz")


@pytest.mark.parametrize("strips,channels,scale", strip_fixture.CASES)
def test_reference_fixture_exact(strips, channels, scale):
    """Exact equality, as the reference demands of its kernels on this fixture."""
    f = strip_fixture.make(strips, channels, scale)
    for wide in (True, False):
        out = c_oracle.conv_fwd(f["val"], f["idx4"], f["x"], f["y"], f["s"], f["sender"], f["receiver_ptr"], f["num_out"], wide=wide)
        assert (out == f["out"]).all()
        ptr_t, perm_t = c_oracle.transpose_csr(f["sender"], strip_fixture.NUM_NODES)
        dx, dy, ds = c_oracle.conv_bwd(f["val"], f["idx4"], f["x"], f["y"], f["s"], f["dz"], f["sender"],
                                       f["receiver_ptr"], ptr_t, perm_t, wide=wide)  # fmt: skip
        assert (dx == f["dx"]).all() and (dy == f["dy"]).all() and (ds == f["ds"]).all()
    out = numpy_oracle.conv_fwd(f["val"], f["idx4"], f["x"], f["y"], f["s"], f["sender"], f["receiver"], f["num_out"])
    assert (out == f["out"]).all()


def test_committed_vectors():
    g = np.load(GOLDEN)
    n = g["x"].shape[0]
    ptr = csr_ptr(g["receiver"], n)
    out = c_oracle.conv_fwd(g["val"], g["idx4"], g["x"], g["y"], g["s"], g["sender"], ptr, g["out"].shape[1])
    assert_close(out, g["out"], what="out")
    ptr_t, perm_t = c_oracle.transpose_csr(g["sender"], n)
    dx, dy, ds = c_oracle.conv_bwd(g["val"], g["idx4"], g["x"], g["y"], g["s"], g["dm"], g["sender"], ptr, ptr_t, perm_t)
    for got, name in ((dx, "dx"), (dy, "dy"), (ds, "ds")):
        assert_close(got, g[name], what=name)
    out64 = numpy_oracle.conv_fwd(g["val"], g["idx4"], g["x"], g["y"], g["s"], g["sender"], g["receiver"], g["out"].shape[1])
    assert np.array_equal(out64, g["out"])


def _dense_reference(val, idx4, x, y, s, snd, rcv, nz):
    """Independent formulation: dense coefficient tensor + einsum + index_add (torch, float64)."""
    dense = torch.zeros(nz, x.shape[1], y.shape[1], s.shape[1], dtype=torch.float64)
    for v, (i, j, k, l) in zip(val, idx4):  # noqa: E741
        dense[i, j, k, l] += float(v)
    msg = torch.einsum("ijkl,ejc,ek,elc->eic", dense, x[snd], y, s)
    return torch.zeros(x.shape[0], nz, x.shape[2], dtype=torch.float64).index_add_(0, rcv, msg)


@pytest.mark.parametrize("seed,channels", [(0, 1), (1, 4), (2, 32)])
def test_against_autograd_of_a_dense_formulation(seed, channels):
    rng = np.random.default_rng(seed)
    n, e, nx, ny, nz, ns = 7, 30, 5, 4, 9, 3
    val, idx4 = random_table(rng, 40, nx, ny, nz, ns)
    snd, rcv = random_graph(rng, n, e)
    x, y, s, dm = (rng.standard_normal(sh).astype(np.float32) for sh in [(n, nx, channels), (e, ny), (e, ns, channels), (n, nz, channels)])
    tx, ty, ts = (torch.tensor(a, dtype=torch.float64, requires_grad=True) for a in (x, y, s))
    out_t = _dense_reference(val, idx4, tx, ty, ts, torch.tensor(snd, dtype=torch.long), torch.tensor(rcv, dtype=torch.long), nz)
    gx, gy, gs = torch.autograd.grad(out_t, (tx, ty, ts), torch.tensor(dm, dtype=torch.float64))
    ptr = csr_ptr(rcv, n)
    ptr_t, perm_t = c_oracle.transpose_csr(snd, n)
    for wide in (True, False):
        out = c_oracle.conv_fwd(val, idx4, x, y, s, snd, ptr, nz, wide=wide)
        dx, dy, ds = c_oracle.conv_bwd(val, idx4, x, y, s, dm, snd, ptr, ptr_t, perm_t, wide=wide)
        tol = dict(rtol=1e-6, atol=1e-6) if wide else dict(rtol=2e-5, atol=1e-5)
        assert_close(out, out_t.detach().numpy(), what="out", **tol)
        assert_close(dx, gx.numpy(), what="dx", **tol)
        assert_close(dy, gy.numpy(), what="dy", **tol)
        assert_close(ds, gs.numpy(), what="ds", **tol)
    o64 = numpy_oracle.conv_fwd(val, idx4, x, y, s, snd, rcv, nz)
    d64 = numpy_oracle.conv_bwd(val, idx4, x, y, s, dm, snd, rcv)
    assert np.allclose(o64, out_t.detach().numpy(), atol=1e-12)
    for a, b in zip(d64, (gx, gy, gs)):
        assert np.allclose(a, b.numpy(), atol=1e-12)


def test_padding_edges_contribute_nothing():
    rng = np.random.default_rng(3)
    n, e = 6, 20
    val, idx4 = random_table(rng, 25, 3, 4, 6, 2)
    snd, rcv = random_graph(rng, n, e)
    x, y, s, dm = (rng.standard_normal(sh).astype(np.float32) for sh in [(n, 3, 4), (e, 4), (e, 2, 4), (n, 6, 4)])
    # pad: 3 trailing dummy edges plus one in-segment edge with a dummy sender
    big = 2**31 - 1
    snd_p = np.concatenate([snd, [big] * 3]).astype(np.int32)
    rcv_p = np.concatenate([rcv, [big] * 3]).astype(np.int32)
    snd_p[4] = big
    y_p = np.concatenate([y, np.full((3, 4), np.nan, np.float32)])
    s_p = np.concatenate([s, np.full((3, 2, 4), np.nan, np.float32)])
    keep = np.ones(e, bool)
    keep[4] = False
    ptr = csr_ptr(rcv_p, n)
    out = c_oracle.conv_fwd(val, idx4, x, y_p, s_p, snd_p, ptr, 6)
    want = numpy_oracle.conv_fwd(val, idx4, x, y[keep], s[keep], snd[keep], rcv[keep], 6)
    assert_close(out, want)
    ptr_t, perm_t = c_oracle.transpose_csr(snd_p, n)
    dx, dy, ds = c_oracle.conv_bwd(val, idx4, x, y_p, s_p, dm, snd_p, ptr, ptr_t, perm_t)
    wdx, wdy, wds = numpy_oracle.conv_bwd(val, idx4, x, y[keep], s[keep], dm, snd[keep], rcv[keep])
    assert_close(dx, wdx)
    assert_close(dy[:e][keep], wdy)
    assert_close(ds[:e][keep], wds)
    assert (dy[e:] == 0).all() and (ds[e:] == 0).all() and (dy[4] == 0).all() and (ds[4] == 0).all()
