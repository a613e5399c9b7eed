"""Harmonics kernels, and the whole config-1 style step: positions -> harmonics / radial MLP
-> convolution -> loss, with gradients w.r.t. node features, MLP weights and positions,
against a float64 torch-CPU restatement differentiated by autograd."""

import math

import numpy as np
import pytest
import torch

from e3j_b200 import problems
from e3j_b200.convolution import Convolution
from e3j_b200.harmonics import Harmonics
from e3j_b200.radial import SILU_2MOM, bessel_envelope
from tests.conftest import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("normalize", [True, False])
@pytest.mark.parametrize("normalization", ["component", "integral", "norm"])
def test_harmonics_kernels_match_numpy(normalize, normalization):
    rng = np.random.default_rng(0)
    r = rng.normal(size=(1000, 3)).astype(np.float32) * 2.0
    r[0] = 0.0  # safe norm at the origin
    h = Harmonics(3, normalize=normalize, normalization=normalization)
    rt = torch.as_tensor(r).to(DEV).requires_grad_()
    y = h.cuda(rt)
    want = h(r.astype(np.float64))
    assert_close(y.detach().cpu().numpy(), want, what="y", rtol=2e-6 if normalize else 1e-5)
    dy = rng.normal(size=want.shape).astype(np.float32)
    (y * torch.as_tensor(dy).to(DEV)).sum().backward()
    wdr = h.vjp(r.astype(np.float64), dy.astype(np.float64))
    if normalize:  # the origin has a 1/sqrt(eps) Jacobian: compare the regular points
        assert_close(rt.grad.cpu().numpy()[1:], wdr[1:], what="dr", rtol=1e-5)
        assert np.isfinite(rt.grad.cpu().numpy()[0]).all()
    else:
        assert_close(rt.grad.cpu().numpy(), wdr, what="dr", rtol=1e-5)


def test_harmonics_other_degrees():
    rng = np.random.default_rng(1)
    r = rng.normal(size=(257, 3)).astype(np.float32)
    for target in (0, 1, 5, "1o+3o"):
        h = Harmonics(target, normalize=True)
        y = h.cuda(torch.as_tensor(r).to(DEV))
        assert_close(y.cpu().numpy(), h(r.astype(np.float64)), what=str(target), rtol=5e-6)


def _harmonics_torch(h: Harmonics, vec: torch.Tensor) -> torch.Tensor:
    """float64 torch evaluation of the same monomial table (autograd reference)."""
    u = vec / torch.sqrt((vec * vec).sum(-1, keepdim=True) + 1e-7) if h.normalize else vec
    e = torch.as_tensor(h.mono_exp, dtype=torch.long)
    terms = torch.as_tensor(h.mono_coef)[None, :] * u[:, 0:1] ** e[:, 0] * u[:, 1:2] ** e[:, 1] * u[:, 2:3] ** e[:, 2]
    out = torch.zeros(vec.shape[0], h.dim, dtype=torch.float64)
    return out.index_add(1, torch.as_tensor(h.mono_row, dtype=torch.long), terms)


def test_full_step_gradients_features_weights_positions():
    cfg, n_nodes, C = 0, 90, 128
    conv = Convolution((problems.X_IRREPS[cfg], problems.Y_IRREPS), problems.OUT_FILTER, graph_ordering="RECEIVER",
                       avg_num_neighbors=30.0)  # fmt: skip
    g = problems.make_graph(cfg, 0, num_nodes=n_nodes)
    S, Z, cutoff = conv.num_scalars, conv.target.dim, problems.CUTOFF[cfg]
    rng = np.random.default_rng(0)
    x0 = rng.standard_normal((n_nodes, 4, C)).astype(np.float32)
    w1_0 = rng.standard_normal((8, 64)).astype(np.float32)
    w2_0 = rng.standard_normal((64, S * C)).astype(np.float32)
    pos0 = g.positions.astype(np.float32)
    snd, rcv = torch.as_tensor(g.sender, dtype=torch.long), torch.as_tensor(g.receiver, dtype=torch.long)
    h = Harmonics(3, normalize=True, normalization="component")

    def radial(r, w1, w2):
        hid = SILU_2MOM * torch.nn.functional.silu(bessel_envelope(r, cutoff) @ w1 / math.sqrt(8))
        return (hid @ w2 / math.sqrt(64)).view(-1, S, C)

    # ---- CUDA path -------------------------------------------------------------
    x, w1, w2, pos = (torch.as_tensor(a).to(DEV).requires_grad_() for a in (x0, w1_0, w2_0, pos0))
    vec = pos[rcv.to(DEV)] - pos[snd.to(DEV)]
    y = h.cuda(vec)
    s = radial(torch.sqrt((vec * vec).sum(-1)), w1, w2)
    out = conv(x, y, s, torch.as_tensor(g.sender).to(DEV), torch.as_tensor(g.receiver).to(DEV))
    loss = (out * out).sum()
    loss.backward()

    # ---- float64 reference, differentiated by autograd ---------------------------
    xr, w1r, w2r, posr = (torch.tensor(a, dtype=torch.float64, requires_grad=True) for a in (x0, w1_0, w2_0, pos0))
    vr = posr[rcv] - posr[snd]
    yr = _harmonics_torch(h, vr)
    sr = radial(torch.sqrt((vr * vr).sum(-1)), w1r, w2r)
    dense = torch.zeros(Z, 4, 16, S, dtype=torch.float64)
    for v, (i, j, k, l) in zip(conv.coef.val, conv.coef.idx.astype(int)):  # noqa: E741
        dense[i, j, k, l] += float(v)
    msg = torch.einsum("ijkl,ejc,ek,elc->eic", dense, xr[snd], yr, sr)
    outr = torch.zeros(n_nodes, Z, C, dtype=torch.float64).index_add_(0, rcv, msg)
    lossr = (outr * outr).sum()
    lossr.backward()

    assert abs(loss.item() - lossr.item()) <= 1e-5 * abs(lossr.item())
    assert_close(out.detach().cpu().numpy(), outr.detach().numpy(), what="out")
    # gradients are sums of many fp32 terms: tolerance relative to each tensor's scale
    for got, want, name in ((x.grad, xr.grad, "dx"), (w1.grad, w1r.grad, "dw1"), (w2.grad, w2r.grad, "dw2"),
                            (pos.grad, posr.grad, "dpos")):  # fmt: skip
        assert_close(got.cpu().numpy(), want.numpy(), what=name, rtol=3e-5)
