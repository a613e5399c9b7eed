"""SENDER graph ordering (edges stored sorted by sender; src/e3j/core/convolution.py:236-246,
src/e3j/ops/convolution.py:166-176, 413-425) against the oracle run on the receiver-sorted
permutation of the same edges."""

import numpy as np
import pytest
import torch

from e3j_b200 import ops, problems
from e3j_b200.coef import Coef4D
from e3j_b200.convolution import Convolution
from oracle import c_oracle
from tests.conftest import assert_close, csr_ptr, random_graph, random_table

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a, dtype=None):
    return torch.as_tensor(np.ascontiguousarray(a), dtype=dtype).to(DEV)


def by_sender(snd, rcv):
    """Stable order of a receiver-sorted edge list by sender (padding stays at the tail)."""
    return np.lexsort((rcv, snd))


@pytest.mark.parametrize("force_generic", [False, True])
@pytest.mark.parametrize("channels", [128, 32])
def test_backward_by_sender_on_a_random_directed_graph(channels, force_generic):
    """No symmetry assumed: the backward of the true forward, with per-edge arrays in sender order."""
    rng = np.random.default_rng(7)
    n, e, nx, ny, nz, ns = 40, 300, 6, 5, 11, 4
    val, idx4 = random_table(rng, 60, nx, ny, nz, ns)
    pad = 6
    snd, rcv = random_graph(rng, n, e - pad)  # receiver-sorted; padding edges follow at the tail
    snd = np.concatenate([snd, [problems.DUMMY_INDEX] * pad]).astype(np.int32)
    rcv = np.concatenate([rcv, [problems.DUMMY_INDEX] * pad]).astype(np.int32)
    x, y, s, dm = (rng.standard_normal(sh).astype(np.float32) for sh in [(n, nx, channels), (e, ny), (e, ns, channels), (n, nz, channels)])
    ptr = csr_ptr(rcv, n)
    ptr_t, perm_t = c_oracle.transpose_csr(snd, n)
    want_dx, want_dy, want_ds = c_oracle.conv_bwd(val, idx4, x, y, s, dm, snd, ptr, ptr_t, perm_t)

    y[e - pad :], s[e - pad :] = np.nan, np.nan  # never read
    order = by_sender(snd, rcv)
    plan = ops.get_plan(Coef4D(val, idx4, idx_dtype="int32").pack(), (nx, ny, nz, ns, channels), torch.device(DEV), force_generic)
    graph = ops.ConvGraph.build(n, dev(snd[order]), dev(rcv[order]), "SENDER")
    dx, dy, ds = ops.conv_bwd_by_sender_raw(plan, dev(x), dev(y[order]), dev(s[order]), dev(dm), graph)
    assert_close(dx.cpu().numpy(), want_dx, what="dx")
    assert_close(dy.cpu().numpy(), want_dy[order], what="dy")
    assert_close(ds.cpu().numpy(), want_ds[order], what="ds")
    # padding edges: exact zeros, also in memory that held NaN
    pad = (snd[order] < 0) | (snd[order] >= n)
    assert pad.any() and not dy.cpu().numpy()[pad].any() and not ds.cpu().numpy()[pad].any()


@pytest.mark.parametrize("cfg,n,generic", [(0, 400, False), (2, 300, False), (0, 200, True)])
def test_module_with_sender_ordering_matches_receiver_ordering(cfg, n, generic):
    """A radius graph is symmetric and its harmonics flip with the edge direction, so the
    SENDER-ordered operator must give the outputs and gradients of the RECEIVER-ordered one."""
    g = problems.make_graph(cfg, seed=1, num_nodes=n)
    kw = dict(avg_num_neighbors=30.0)
    conv_r = Convolution((problems.X_IRREPS[cfg], problems.Y_IRREPS), problems.OUT_FILTER, graph_ordering="RECEIVER", **kw)
    conv_s = Convolution((problems.X_IRREPS[cfg], problems.Y_IRREPS), problems.OUT_FILTER, graph_ordering="SENDER", **kw)
    conv_r.force_generic = conv_s.force_generic = generic
    inp = problems.make_inputs(g, cfg, conv_r.num_scalars, conv_r.source[0].dim, seed=1)
    order = by_sender(g.sender, g.receiver)

    val, idx4 = conv_r.coef.val, conv_r.coef.idx.astype(np.int32)
    ptr = csr_ptr(g.receiver, g.num_nodes)
    want = c_oracle.conv_fwd(val, idx4, inp.x, inp.y, inp.s, g.sender, ptr, conv_r.target.dim)
    ptr_t, perm_t = c_oracle.transpose_csr(g.sender, g.num_nodes)
    w_dx, w_dy, w_ds = c_oracle.conv_bwd(val, idx4, inp.x, inp.y, inp.s, 2 * want, g.sender, ptr, ptr_t, perm_t)

    x = dev(inp.x).requires_grad_()
    y = dev(inp.y[order]).requires_grad_()
    s = dev(inp.s[order]).requires_grad_()
    out = conv_s(x, y, s, dev(g.sender[order]), dev(g.receiver[order]))
    assert_close(out.detach().cpu().numpy(), want, what="out")
    # cotangent 2 * (oracle output): the same one the oracle's backward was given
    out.backward(dev(2 * want))
    assert_close(x.grad.cpu().numpy(), w_dx, what="dx")
    assert_close(y.grad.cpu().numpy(), w_dy[order], what="dy")
    assert_close(s.grad.cpu().numpy(), w_ds[order], what="ds")

    # prepared graph, and the ordering check on it
    graph = conv_s.prepare_graph(g.num_nodes, dev(g.sender[order]), dev(g.receiver[order]))
    out2 = conv_s(x.detach(), y.detach(), s.detach(), graph)
    assert torch.equal(out2, out.detach())
    with pytest.raises(ValueError):
        conv_r(x.detach(), y.detach(), s.detach(), graph)


def test_ordering_none_is_rejected_and_sender_needs_parity():
    conv = Convolution(("0e+1o", "0e+1o+2e+3o"), "0e+1o+2e+3o", graph_ordering="NONE")
    t = torch.zeros((2, 4, 128), device=DEV)
    with pytest.raises(NotImplementedError):
        conv(t, torch.zeros((1, 16), device=DEV), torch.zeros((1, 10, 128), device=DEV), dev([0]), dev([1]))
    c = Convolution(("0e+1o", "0e+1o+2e+3o"), "0e+1o+2e+3o", graph_ordering="SENDER")
    with pytest.raises(ValueError):
        ops.convolution(c._coef_packed, t, torch.zeros((1, 16), device=DEV), torch.zeros((1, 10, 128), device=DEV),
                        dev([0]), dev([1]), c.params, "SENDER", None)
