"""Edge windows (scalars produced per receiver range) and the per-rank builder of
periodic slabs: planner and partition on CPU; on the GPU the windowed passes against
the one-pass kernels (bitwise) and a two-rank periodic case against the oracle."""

import math

import numpy as np
import pytest
import torch

from e3j_b200 import problems
from e3j_b200.chunked import plan_windows
from e3j_b200.convolution import Convolution
from e3j_b200.harmonics import Harmonics
from e3j_b200.partition import morton_order, partition_slabs, periodic_slab_part
from e3j_b200.radial import SILU_2MOM, RadialMLP, bessel_envelope_np
from oracle import c_oracle
from tests.conftest import assert_close, csr_ptr

DEV = "cuda:0"


def test_plan_windows():
    ptr = np.array([0, 3, 3, 7, 12, 12, 15])
    assert plan_windows(ptr, 0, 6, 5) == [(0, 2, 0, 3), (2, 3, 3, 7), (3, 5, 7, 12), (5, 6, 12, 15)]
    assert plan_windows(ptr, 2, 6, 100) == [(2, 6, 3, 15)]
    assert plan_windows(ptr, 3, 3, 5) == []
    with pytest.raises(ValueError):
        plan_windows(ptr, 0, 6, 4)
    rng = np.random.default_rng(0)
    ptr = np.concatenate([[0], np.cumsum(rng.integers(0, 9, 200))])
    for budget in (8, 13, 50, 10**6):
        w = plan_windows(ptr, 5, 190, budget)
        assert w[0][0] == 5 and w[-1][1] == 190
        assert all(a[1] == b[0] and a[3] == b[2] for a, b in zip(w, w[1:]))
        assert all(e1 - e0 <= budget and e0 == ptr[r0] and e1 == ptr[r1] for r0, r1, e0, e1 in w)
        # greedy: one more receiver would not have fitted
        assert all(r1 == 190 or ptr[r1 + 1] - e0 > budget for r0, r1, e0, e1 in w)


def test_morton_order_is_a_permutation_that_clusters():
    rng = np.random.default_rng(1)
    pos = rng.uniform(0, 40, (5000, 3))
    order = morton_order(pos, 2.5)
    assert sorted(order.tolist()) == list(range(5000))
    step = np.linalg.norm(np.diff(pos[order], axis=0), axis=1).mean()
    assert step < 0.3 * np.linalg.norm(np.diff(pos, axis=0), axis=1).mean()


@pytest.mark.parametrize("n,world,cell", [(3000, 2, None), (3000, 3, 2.5), (6000, 4, 2.5), (2000, 1, 2.5)])
def test_periodic_slab_part_equals_partition_of_the_global_graph(n, world, cell):
    box = (n / 0.1) ** (1 / 3)
    pos = np.random.default_rng(0).uniform(0, box, (n, 3))
    snd, rcv, vec = problems.radius_graph(pos, 5.0, box)
    parts = partition_slabs(pos, snd, rcv, world, 0.0, box, cell=cell)
    for g in range(world):
        q, v = periodic_slab_part(g, world, pos, box, 5.0, cell=cell)
        p = parts[g]
        assert (p.n_int, p.n_own, p.n_loc) == (q.n_int, q.n_own, q.n_loc)
        assert (p.global_ids == q.global_ids).all()
        assert (p.sender == q.sender).all() and (p.receiver == q.receiver).all()
        assert p.recv_slice == q.recv_slice and set(p.send_rows) == set(q.send_rows)
        assert all((p.send_rows[k] == q.send_rows[k]).all() for k in p.send_rows)
        np.testing.assert_allclose(v, vec[p.edge_ids], atol=1e-12)


def test_periodic_slab_part_rejects_slabs_whose_halo_would_wrap():
    box = 17.0
    pos = np.random.default_rng(0).uniform(0, box, (500, 3))
    with pytest.raises(ValueError):
        periodic_slab_part(0, 2, pos, box, 5.0)


def _case(cfg, n, seed=0):
    g = problems.make_graph(cfg, seed=seed, num_nodes=n)
    conv = Convolution((problems.X_IRREPS[cfg], problems.Y_IRREPS), problems.OUT_FILTER, graph_ordering="RECEIVER")
    inp = problems.make_inputs(g, cfg, conv.num_scalars, conv.source[0].dim, seed=seed)
    return g, conv, inp


@pytest.mark.gpu
@pytest.mark.parametrize("cfg,n,generic", [(0, 300, False), (2, 300, False), (0, 200, True)])
def test_windowed_passes_equal_one_pass_bitwise(cfg, n, generic):
    from e3j_b200 import ops
    from e3j_b200.chunked import TensorProducer, WindowedConvOps

    g, conv, inp = _case(cfg, n)
    dev = torch.device(DEV)
    X, Z, S, C = conv.source[0].dim, conv.target.dim, conv.num_scalars, 128
    plan = ops.get_plan(conv._coef_packed, (X, 16, Z, S, C), dev, generic)
    assert plan.variant == (0 if generic else (1 if cfg == 0 else 2))
    to = lambda a, dt=None: torch.as_tensor(np.ascontiguousarray(a), dtype=dt).to(dev)  # noqa: E731
    graph = ops.ConvGraph.build(g.num_nodes, to(g.sender), to(g.receiver))
    x, y, s = to(inp.x), to(inp.y), to(inp.s)
    out1 = ops.conv_fwd_raw(plan, x, y, s, graph)
    dm = 2 * out1
    dx1, dy1, ds1 = ops.conv_bwd_raw(plan, x, y, s, dm, graph)
    ptr_t, perm_t = graph.transposed()
    e = y.shape[0]
    deg = int(np.diff(csr_ptr(g.receiver, g.num_nodes)).max())
    for budget in (max(deg, e // 7), e // 2 + deg, e):
        w = WindowedConvOps(plan, budget)
        out = torch.full_like(out1, float("nan"))
        cut = g.num_nodes // 3  # two calls, as the partitioned operator makes them
        w.forward(x, y, TensorProducer(s), graph.sender, graph.receiver_ptr, out, 0, cut, g.num_nodes)
        w.forward(x, y, TensorProducer(s), graph.sender, graph.receiver_ptr, out, cut, g.num_nodes, g.num_nodes)
        assert torch.equal(out, out1)
        dx, dy, ds = (torch.full_like(t, float("nan")) for t in (dx1, dy1, ds1))
        w.backward(x, y, TensorProducer(s, ds), dm, graph.sender, graph.receiver_ptr, ptr_t, perm_t, dx, dy, None,
                   g.num_nodes, g.num_nodes)  # fmt: skip
        assert torch.equal(dx, dx1) and torch.equal(dy, dy1) and torch.equal(ds, ds1)
        assert w.windows_run >= (3 if budget == e else 5)


@pytest.mark.gpu
def test_two_periodic_slabs_with_windows_and_radial_producer():
    """Ranks emulated on one GPU (exchange replaced by copies): periodic slabs built per rank,
    scalars from the radial MLP per window, weight gradients accumulated over the windows."""
    from e3j_b200 import ops
    from e3j_b200.chunked import RadialProducer, WindowedConvOps
    from e3j_b200.halo import CudaRowOps, HaloConvolution

    cfg, n, world, cutoff = 2, 1300, 2, 5.0
    box = (n / 0.1) ** (1 / 3)
    rng = np.random.default_rng(5)
    pos = rng.uniform(0, box, (n, 3))
    conv = Convolution((problems.X_IRREPS[cfg], problems.Y_IRREPS), problems.OUT_FILTER, graph_ordering="RECEIVER")
    X, Z, S, C = conv.source[0].dim, conv.target.dim, conv.num_scalars, 128
    dims = (X, 16, Z, S, C)
    dev = torch.device(DEV)
    plan = ops.get_plan(conv._coef_packed, dims, dev)
    mlp = RadialMLP.init(8, 64, S * C, seed=1)
    x = rng.standard_normal((n, X, C)).astype(np.float32)
    harm = Harmonics(3, normalize=True, normalization="component")

    # global reference on the CPU
    snd, rcv, vec = problems.radius_graph(pos, cutoff, box)
    y_g = harm(vec).astype(np.float32)
    rbf_g = bessel_envelope_np(np.linalg.norm(vec, axis=1), cutoff, 8).astype(np.float32)
    s_g = mlp.forward_np(rbf_g, np.float32).reshape(-1, S, C)
    val, idx4 = conv.coef.val, conv.coef.idx.astype(np.int32)
    ptr = csr_ptr(rcv, n)
    out_g = c_oracle.conv_fwd(val, idx4, x, y_g, s_g, snd, ptr, Z)
    ptr_t, perm_t = c_oracle.transpose_csr(snd, n)
    dx_g, dy_g, ds_g = c_oracle.conv_bwd(val, idx4, x, y_g, s_g, 2 * out_g, snd, ptr, ptr_t, perm_t)
    pre = rbf_g.astype(np.float64) @ mlp.w1 / math.sqrt(8)
    sig = 1 / (1 + np.exp(-pre))
    h = SILU_2MOM * pre * sig
    d = ds_g.reshape(-1, S * C).astype(np.float64)
    dw2_g = h.T @ d / 8.0
    dpre = (d @ mlp.w2.T.astype(np.float64) / 8.0) * (SILU_2MOM * sig * (1 + pre * (1 - sig)))
    dw1_g = rbf_g.T.astype(np.float64) @ dpre / math.sqrt(8)

    ranks = []
    for r in range(world):
        p, v = periodic_slab_part(r, world, pos, box, cutoff, cell=2.5)
        y = torch.from_numpy(harm(v).astype(np.float32)).to(dev)
        rbf = torch.from_numpy(bessel_envelope_np(np.linalg.norm(v, axis=1), cutoff, 8).astype(np.float32)).to(dev)
        prod = RadialProducer(rbf, torch.from_numpy(mlp.w1).to(dev), torch.from_numpy(mlp.w2).to(dev))
        h_op = HaloConvolution(p, dims, dev, WindowedConvOps(plan, max(200, y.shape[0] // 5)), CudaRowOps)
        x_loc = torch.full((p.n_loc, X, C), float("nan"), device=dev)
        x_loc[: p.n_own] = torch.from_numpy(x[p.global_ids[: p.n_own]]).to(dev)
        ranks.append((p, h_op, x_loc, y, prod))
    for p, h_op, x_loc, _, _ in ranks:  # forward exchange by copies
        for peer in h_op.peers:
            if peer.send_rows is not None:
                buf = torch.empty((peer.send_rows.numel(), X, C), device=dev)
                CudaRowOps.gather(buf, x_loc, peer.send_rows)
                a, b = ranks[peer.rank][0].recv_slice[p.rank]
                ranks[peer.rank][2][a:b] = buf
    dx_locs, dw1, dw2 = [], 0, 0
    for p, h_op, x_loc, y, prod in ranks:
        out = torch.full((p.n_own, Z, C), float("nan"), device=dev)
        c = h_op.conv
        c.forward(x_loc, y, prod, h_op.sender, h_op.receiver_ptr, out, 0, p.n_int, p.n_loc)
        c.forward(x_loc, y, prod, h_op.sender, h_op.receiver_ptr, out, p.n_int, p.n_own, p.n_loc)
        assert_close(out.cpu().numpy(), out_g[p.global_ids[: p.n_own]], what=f"out rank {p.rank}")
        dx_loc, dy = torch.full_like(x_loc, float("nan")), torch.full_like(y, float("nan"))
        c.backward(x_loc, y, prod, out.mul_(2), h_op.sender, h_op.receiver_ptr, h_op.sender_ptr_t, h_op.perm_t,
                   dx_loc, dy, None, p.n_own, p.n_loc)  # fmt: skip
        # local edges in global numbering: (receiver, sender) pairs are unique
        key_g = rcv.astype(np.int64) * n + snd
        key_l = p.global_ids[p.receiver.astype(np.int64)] * n + p.global_ids[p.sender.astype(np.int64)]
        e_ids = np.searchsorted(key_g, key_l)
        assert (key_g[e_ids] == key_l).all()
        assert_close(dy.cpu().numpy(), dy_g[e_ids], what="dy")
        dx_locs.append(dx_loc)
        dw1, dw2 = dw1 + prod.dw1.double().cpu().numpy(), dw2 + prod.dw2.double().cpu().numpy()
    for p, h_op, _, _, _ in ranks:  # reverse exchange by copies
        for peer in h_op.peers:
            if peer.send_rows is not None:
                a, b = ranks[peer.rank][0].recv_slice[p.rank]
                CudaRowOps.add(dx_locs[p.rank], peer.send_rows, dx_locs[peer.rank][a:b].contiguous())
    for p, *_ in ranks:
        assert_close(dx_locs[p.rank][: p.n_own].cpu().numpy(), dx_g[p.global_ids[: p.n_own]], what=f"dx rank {p.rank}")
    for got, want, name in ((dw1, dw1_g, "dw1"), (dw2, dw2_g, "dw2")):
        assert np.abs(got - want).max() <= 2e-4 * np.abs(want).max(), name


@pytest.mark.gpu
def test_split_tf32_product_of_the_radial_producer():
    """The tensor-core evaluation of the wide layer stays within 3e-6 of the layer's scale."""
    from e3j_b200.chunked import RadialProducer, split_tf32

    dev = torch.device(DEV)
    rng = np.random.default_rng(2)
    e, S, C = 20000, 23, 128
    r = rng.uniform(0.8, 4.99, e)
    rbf = bessel_envelope_np(r, 5.0, 8).astype(np.float32)
    mlp = RadialMLP.init(8, 64, S * C, seed=3)
    want = mlp.forward_np(rbf, np.float64)
    t = torch.from_numpy(rng.standard_normal(1000).astype(np.float32)).to(dev)
    hi, lo = split_tf32(t)
    assert torch.equal(hi + lo, t) and bool(((hi.view(torch.int32) & 8191) == 0).all())
    errs = {}
    for prec in ("fp32", "tf32x3"):
        prod = RadialProducer(torch.from_numpy(rbf).to(dev), torch.from_numpy(mlp.w1).to(dev),
                              torch.from_numpy(mlp.w2).to(dev), precision=prec)  # fmt: skip
        s = torch.empty((e, S, C), device=dev)
        prod.forward(0, e, s)
        errs[prec] = float(np.abs(s.cpu().numpy().reshape(e, -1) - want).max() / np.abs(want).max())
    assert errs["fp32"] < 1e-6 and errs["tf32x3"] < 3e-6, errs
    assert not torch.backends.cuda.matmul.allow_tf32
