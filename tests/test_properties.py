"""Size-independent properties, drawn at random (hypothesis): the oracle is trilinear and its
backward is the adjoint of its forward; the table packing round-trips; CSR views, edge windows
and slab partitions keep every edge exactly once."""

import numpy as np
from hypothesis import given, settings
from hypothesis import strategies as st

from e3j_b200.chunked import plan_windows
from e3j_b200.coef import Coef4D
from e3j_b200.graph import DUMMY_INDEX, GraphCSR, receiver_ptr_from_sorted
from e3j_b200.partition import partition_slabs
from e3j_b200.problems import radius_graph
from oracle import c_oracle
from tests.conftest import csr_ptr, random_graph, random_table

import torch

SETTINGS = dict(max_examples=25, deadline=None)


def _case(seed, channels):
    rng = np.random.default_rng(seed)
    n, e = int(rng.integers(1, 9)), int(rng.integers(0, 40))
    nx, ny, nz, ns = (int(v) for v in rng.integers(1, 6, 4))
    val, idx4 = random_table(rng, int(rng.integers(1, 30)), nx, ny, nz, ns)
    snd, rcv = random_graph(rng, n, e)
    shapes = [(n, nx, channels), (e, ny), (e, ns, channels), (n, nz, channels)]
    x, y, s, dm = (rng.standard_normal(sh).astype(np.float32) for sh in shapes)
    return val, idx4, x, y, s, dm, snd, rcv, n, nz


@settings(**SETTINGS)
@given(st.integers(0, 10**6), st.sampled_from([1, 3, 8]))
def test_oracle_backward_is_the_adjoint_of_its_forward(seed, channels):
    val, idx4, x, y, s, dm, snd, rcv, n, nz = _case(seed, channels)
    ptr = csr_ptr(rcv, n)
    ptr_t, perm_t = c_oracle.transpose_csr(snd, n)
    out = c_oracle.conv_fwd(val, idx4, x, y, s, snd, ptr, nz)
    dx, dy, ds = c_oracle.conv_bwd(val, idx4, x, y, s, dm, snd, ptr, ptr_t, perm_t)
    lhs = float((dm.astype(np.float64) * out).sum())
    scale = float(np.abs(dm.astype(np.float64) * out).sum()) + 1e-30
    for a, b in ((x, dx), (y, dy), (s, ds)):  # trilinear: <dm, out> = <x, dx> = <y, dy> = <s, ds>
        assert abs(lhs - float((a.astype(np.float64) * b).sum())) <= 1e-4 * scale + 1e-6


@settings(**SETTINGS)
@given(st.integers(0, 10**6), st.floats(-3, 3), st.sampled_from("xys"))
def test_oracle_is_linear_in_each_operand(seed, alpha, which):
    val, idx4, x, y, s, dm, snd, rcv, n, nz = _case(seed, 4)
    ptr = csr_ptr(rcv, n)
    rng = np.random.default_rng(seed + 1)
    ops = dict(x=x, y=y, s=s)
    other = rng.standard_normal(ops[which].shape).astype(np.float32)
    f = lambda **kw: c_oracle.conv_fwd(val, idx4, kw.get("x", x), kw.get("y", y), kw.get("s", s), snd, ptr, nz).astype(np.float64)  # noqa: E731
    mixed = f(**{which: (ops[which] + np.float32(alpha) * other)})
    want = f() + np.float64(np.float32(alpha)) * f(**{which: other})
    assert np.abs(mixed - want).max() <= 1e-4 * (np.abs(want).max() + 1.0)


@settings(**SETTINGS)
@given(st.integers(0, 10**6), st.sampled_from(["uint8", "int32"]))
def test_coef4d_pack_round_trip(seed, idx_dtype):
    rng = np.random.default_rng(seed)
    val, idx4 = random_table(rng, int(rng.integers(1, 60)), 7, 6, 9, 5)
    c = Coef4D(val, idx4, idx_dtype=idx_dtype)
    packed = c.pack()
    assert packed.shape == (len(val), 8) and packed.itemsize == (1 if idx_dtype == "uint8" else 4)
    back = Coef4D.unpack(packed, np.float32)
    assert np.array_equal(back.val, c.val) and np.array_equal(back.idx, c.idx)
    swapped = c.transpose((1, 0, 2, 3))  # rows stably sorted by the new first column
    assert (np.diff(swapped.idx[:, 0].astype(int)) >= 0).all()
    assert sorted(map(tuple, swapped.idx[:, [1, 0, 2, 3]].tolist())) == sorted(map(tuple, c.idx.tolist()))


@settings(**SETTINGS)
@given(st.integers(0, 10**6), st.integers(1, 30), st.integers(0, 200), st.integers(0, 6))
def test_csr_views_keep_every_edge_once(seed, n, e, pad):
    rng = np.random.default_rng(seed)
    snd, rcv = random_graph(rng, n, e)
    snd = np.concatenate([snd, np.full(pad, DUMMY_INDEX)]).astype(np.int32)
    rcv = np.concatenate([rcv, np.full(pad, DUMMY_INDEX)]).astype(np.int32)
    ptr = receiver_ptr_from_sorted(n, torch.as_tensor(rcv)).numpy()
    assert ptr[0] == 0 and ptr[-1] == e and (np.diff(ptr) >= 0).all()
    assert all((rcv[ptr[r] : ptr[r + 1]] == r).all() for r in range(n))
    perm, gt, inv = GraphCSR(n, torch.as_tensor(snd), torch.as_tensor(rcv)).transpose()
    perm, inv = perm.numpy(), inv.numpy()
    assert sorted(perm.tolist()) == list(range(e + pad)) and (perm[inv] == np.arange(e + pad)).all()
    assert (np.diff(snd[perm].astype(np.int64)) >= 0).all()  # sorted by sender, padding last
    same = snd[perm][1:] == snd[perm][:-1]
    assert (np.diff(perm)[same] > 0).all()  # stable inside a sender segment
    ptr_t = gt.receiver_ptr.numpy()
    assert ptr_t[-1] == e and all((snd[perm][ptr_t[a] : ptr_t[a + 1]] == a).all() for a in range(n))


@settings(**SETTINGS)
@given(st.integers(0, 10**6), st.integers(1, 60), st.integers(1, 80))
def test_edge_windows_tile_the_receivers(seed, n, budget):
    rng = np.random.default_rng(seed)
    deg = rng.integers(0, budget + 1, n)
    ptr = np.concatenate([[0], np.cumsum(deg)])
    lo, hi = sorted(int(v) for v in rng.integers(0, n + 1, 2))
    w = plan_windows(ptr, lo, hi, budget)
    assert (not w and lo == hi) or (w[0][0] == lo and w[-1][1] == hi)
    assert all(a[1] == b[0] for a, b in zip(w, w[1:]))
    assert all(r1 > r0 and e1 - e0 <= budget and e0 == ptr[r0] and e1 == ptr[r1] for r0, r1, e0, e1 in w)


@settings(max_examples=8, deadline=None)
@given(st.integers(0, 10**6), st.integers(1, 4))
def test_slab_partition_owns_every_edge_once_with_consistent_plans(seed, world):
    rng = np.random.default_rng(seed)
    n = int(rng.integers(20, 200))
    pos = rng.uniform(0, 1, (n, 3)) * np.array([12.0 * world, 9.0, 9.0])
    snd, rcv, _ = radius_graph(pos, 4.5, None)
    parts = partition_slabs(pos, snd, rcv, world, 0.0, 12.0 * world + 1e-9)
    seen = np.concatenate([p.edge_ids for p in parts])
    assert sorted(seen.tolist()) == list(range(len(snd)))
    owned = np.concatenate([p.global_ids[: p.n_own] for p in parts])
    assert sorted(owned.tolist()) == list(range(n))
    for p in parts:
        assert (p.global_ids[p.sender] == snd[p.edge_ids]).all() and (p.global_ids[p.receiver] == rcv[p.edge_ids]).all()
        assert (np.diff(p.receiver) >= 0).all() and (p.receiver < p.n_own).all()
        # interior receivers gather owned rows only
        assert (p.sender[p.receiver < p.n_int] < p.n_own).all()
        for q, (a, b) in p.recv_slice.items():  # what arrives from q is what q sends, in the same order
            rows = parts[q].send_rows[p.rank]
            assert (parts[q].global_ids[rows] == p.global_ids[a:b]).all()


@settings(**SETTINGS)
@given(st.integers(0, 10**6), st.sampled_from([("OUTER", 3, 2), ("OUTER", 4, 1), ("MAP", 5, 5)]))
def test_tensor_product_oracle_backward_is_the_adjoint(seed, shape):
    from oracle import numpy_oracle

    mode, cx, cy = shape
    rng = np.random.default_rng(seed)
    nx, ny, nz, rows = (int(v) for v in rng.integers(1, 6, 4))
    nnz = int(rng.integers(1, 20))
    val = rng.standard_normal(nnz).astype(np.float32)
    idx = np.stack([rng.integers(0, nz, nnz), rng.integers(0, nx, nnz), rng.integers(0, ny, nnz)], axis=-1)
    x, y = rng.standard_normal((rows, nx, cx)), rng.standard_normal((rows, ny, cy))
    out = numpy_oracle.tensor_product(val, idx, x, y, nz, mode)
    dz = rng.standard_normal(out.shape)
    dx, dy = numpy_oracle.tensor_product_vjp(val, idx, x, y, dz, mode)
    lhs = (dz * out).sum()
    assert abs(lhs - (dx * x).sum()) <= 1e-9 * (1 + abs(lhs)) and abs(lhs - (dy * y).sum()) <= 1e-9 * (1 + abs(lhs))
