"""The XLA FFI handlers, driven through hand-built call frames with the reference's exact
operand lists (lib/e3j_ops/ffi/e3j_ops.h:457-472, 575-594) — what unmodified e3j Python passes."""

import ctypes
import os

import numpy as np
import pytest
import torch

from e3j_b200 import _lib, ops, problems
from e3j_b200.coef import Coef4D
from e3j_b200.convolution import Convolution
from e3j_b200.graph import GraphCSR
from tests.xla_frame import FakeRuntime

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not os.path.exists(_lib.XLA_LIB_PATH),
                                                  reason="libe3j_b200_xla.so was not built (no XLA FFI headers)")]  # fmt: skip
DEV = torch.device("cuda:0")


@pytest.fixture(scope="module")
def xla():
    _lib.lib()
    return ctypes.CDLL(_lib.XLA_LIB_PATH)


def _case(config, nodes, idx_dtype):
    conv = Convolution((problems.X_IRREPS[config], problems.Y_IRREPS), problems.OUT_FILTER, graph_ordering="RECEIVER",
                       avg_num_neighbors=12.0)  # fmt: skip
    g = problems.make_graph(config, 1, num_nodes=nodes)
    inp = problems.make_inputs(g, config, conv.num_scalars, conv.source[0].dim, 128, 1)
    c = Coef4D(conv.coef.val, conv.coef.idx, idx_dtype=idx_dtype)
    x, y, s = (torch.as_tensor(a).to(DEV) for a in (inp.x, inp.y, inp.s))
    snd, rcv = torch.as_tensor(g.sender).to(DEV), torch.as_tensor(g.receiver).to(DEV)
    return conv, g, c, x, y, s, snd, rcv


@pytest.mark.parametrize("config,nodes,idx_dtype", [(0, 300, "uint8"), (0, 100, "int32"), (2, 200, "uint8")])
def test_handlers_with_reference_operand_lists(xla, config, nodes, idx_dtype):
    conv, g, c, x, y, s, snd, rcv = _case(config, nodes, idx_dtype)
    n, z = g.num_nodes, conv.target.dim
    rt = FakeRuntime(DEV)
    graph = ops.ConvGraph.build(n, snd, rcv)
    plan = ops.get_plan(conv._coef_packed, (x.shape[1], 16, z, conv.num_scalars, 128), DEV)
    want = ops.conv_fwd_raw(plan, x, y, s, graph)

    # forward: coef, x, y, s, sender, receiver_ptr, coef_ranges -> out ; attrs num_nodes, debug
    coef_dev = torch.as_tensor(c.pack()).to(DEV)
    out = torch.full_like(want, float("nan"))
    ranges = torch.tensor([len(c.val)], dtype=torch.int32, device=DEV)
    errs = rt.call(xla.e3j_b200_xla_convolution, [coef_dev, x, y, s, graph.sender, graph.receiver_ptr.contiguous(), ranges],
                   [out], {"num_nodes": n, "debug": 0})  # fmt: skip
    assert errs == []
    torch.cuda.synchronize()
    assert torch.equal(out, want)

    # backward: coef[3], x, y, s, dm, receivers in sender order, sender CSR, edge_perm, coef_ranges -> dx, dy, ds
    dm = torch.randn_like(want)
    wdx, wdy, wds = ops.conv_bwd_raw(plan, x, y, s, dm, graph)
    perm, gt, _ = GraphCSR(n, snd.cpu(), rcv.cpu()).transpose()
    coef3 = np.stack([c.transpose(a).pack() for a in ((1, 0, 2, 3), (2, 0, 1, 3), (3, 0, 2, 1))])
    dx, dy, ds = (torch.full_like(t, float("nan")) for t in (x, y, s))
    errs = rt.call(xla.e3j_b200_xla_convolution_bwd,
                   [torch.as_tensor(coef3).to(DEV), x, y, s, dm, gt.sender.to(DEV), gt.receiver_ptr.to(DEV),
                    perm.to(DEV), torch.zeros(3, dtype=torch.int32, device=DEV)],
                   [dx, dy, ds], {"num_nodes": n, "debug": 1})  # fmt: skip
    assert errs == []
    torch.cuda.synchronize()
    assert torch.equal(dx, wdx) and torch.equal(dy, wdy) and torch.equal(ds, wds)
    assert rt.allocated_bytes > 0 and not rt.scratch  # scratch came from the frame's allocator and was returned


def test_handler_errors_travel_as_xla_errors(xla):
    conv, g, c, x, y, s, snd, rcv = _case(0, 60, "uint8")
    rt = FakeRuntime(DEV)
    graph = ops.ConvGraph.build(g.num_nodes, snd, rcv)
    out = torch.empty((g.num_nodes, conv.target.dim, 128), device=DEV)
    ranges = torch.tensor([1], dtype=torch.int32, device=DEV)
    coef_dev = torch.as_tensor(c.pack()).to(DEV)
    errs = rt.call(xla.e3j_b200_xla_convolution, [coef_dev, x.double(), y, s, graph.sender, graph.receiver_ptr.contiguous(), ranges],
                   [out], {"num_nodes": g.num_nodes, "debug": 0})  # fmt: skip
    assert len(errs) == 1 and "float32" in errs[0][1]


def test_backward_handler_under_sender_ordering(xla):
    """SENDER ordering reaches the backward as an empty edge_perm, the receivers of the stored
    (sender-sorted) edges and the CSR of the stored order (src/e3j/ops/convolution.py:413-425)."""
    conv, g, c, x, y, s, snd, rcv = _case(0, 200, "uint8")
    n, z = g.num_nodes, conv.target.dim
    order = torch.as_tensor(np.lexsort((g.receiver, g.sender))).to(DEV)
    snd_s, rcv_s, y_s, s_s = snd[order].contiguous(), rcv[order].contiguous(), y[order].contiguous(), s[order].contiguous()
    plan = ops.get_plan(conv._coef_packed, (x.shape[1], 16, z, conv.num_scalars, 128), DEV)
    graph = ops.ConvGraph.build(n, snd_s, rcv_s, "SENDER")
    dm = torch.randn((n, z, 128), device=DEV)
    wdx, wdy, wds = ops.conv_bwd_by_sender_raw(plan, x, y_s, s_s, dm, graph)
    rt = FakeRuntime(DEV)
    coef3 = np.stack([c.transpose(a).pack() for a in ((1, 0, 2, 3), (2, 0, 1, 3), (3, 0, 2, 1))])
    dx, dy, ds = (torch.full_like(t, float("nan")) for t in (x, y_s, s_s))
    errs = rt.call(xla.e3j_b200_xla_convolution_bwd,
                   [torch.as_tensor(coef3).to(DEV), x, y_s, s_s, dm, rcv_s, graph.receiver_ptr.contiguous(),
                    torch.zeros(0, dtype=torch.int32, device=DEV), torch.zeros(3, dtype=torch.int32, device=DEV)],
                   [dx, dy, ds], {"num_nodes": n, "debug": 1})  # fmt: skip
    assert errs == []
    torch.cuda.synchronize()
    assert torch.equal(dx, wdx) and torch.equal(dy, wdy) and torch.equal(ds, wds)


def test_stand_in_module_device_properties():
    """Keys of `e3j_ops.get_device_properties()` (lib/e3j_ops/ffi/e3j_ops.cpp:30-42)."""
    from e3j_b200 import e3j_ops_compat

    props = e3j_ops_compat.get_device_properties()
    assert set(props) == {"device", "smem_max", "smem_opt_in", "smem_per_sm", "max_threads_per_sm",
                          "max_blocks_per_sm", "regs_per_sm"}  # fmt: skip
    assert props["smem_opt_in"] >= 200 * 1024 and props["regs_per_sm"] == 65536
