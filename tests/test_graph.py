"""CSR helpers (facts pinned by tests/test_graph.py:79-183 of the reference)."""

import numpy as np
import torch

from e3j_b200.graph import DUMMY_INDEX, GraphCSR
from e3j_b200.ops import ConvGraph, _wrap_global_index


def test_receiver_ptr_counts_in_range_only():
    snd = torch.tensor([1, 2, 0, 3, DUMMY_INDEX], dtype=torch.int32)
    rcv = torch.tensor([0, 0, 2, 3, DUMMY_INDEX], dtype=torch.int32)
    g = GraphCSR(4, snd, rcv)
    assert g.receiver_ptr.tolist() == [0, 2, 2, 3, 4] and g.receiver_ptr.dtype == torch.int32


def test_transpose_is_a_stable_sort_by_sender():
    snd = torch.tensor([1, 2, 0, 3, 0, 1], dtype=torch.int32)
    rcv = torch.tensor([0, 0, 1, 1, 2, 3], dtype=torch.int32)
    perm, gt, inv = GraphCSR(4, snd, rcv).transpose()
    assert perm.tolist() == [2, 4, 0, 5, 1, 3]
    assert gt.receiver_ptr.tolist() == [0, 2, 4, 5, 6]  # offsets by sender
    assert gt.sender.tolist() == [1, 2, 0, 3, 0, 1]  # receivers in sender order
    assert perm[inv.long()].tolist() == list(range(6))
    cg = ConvGraph.build(4, snd, rcv)
    ptr_t, perm_t = cg.transposed()
    assert ptr_t.tolist() == [0, 2, 4, 5, 6] and perm_t.tolist() == perm.tolist()


def test_mask_edges_marks_both_endpoints():
    snd = torch.tensor([0, 1, 2, 3], dtype=torch.int32)
    rcv = torch.tensor([1, 0, 3, 2], dtype=torch.int32)
    mask = torch.tensor([True, True, True, False])
    s, r = GraphCSR.mask_edges(snd, rcv, mask)
    assert s.tolist() == [0, 1, DUMMY_INDEX, DUMMY_INDEX] and r.tolist() == [1, 0, DUMMY_INDEX, DUMMY_INDEX]


def test_wrap_keeps_the_sentinel():
    idx = torch.tensor([0, 5, 9, DUMMY_INDEX], dtype=torch.int64)
    assert _wrap_global_index(idx, 4).tolist() == [0, 1, 1, DUMMY_INDEX]


def test_dummy_senders_fall_outside_sender_segments():
    snd = torch.tensor([1, DUMMY_INDEX, 0], dtype=torch.int32)
    rcv = torch.tensor([0, 0, 1], dtype=torch.int32)
    ptr_t, perm_t = ConvGraph.build(2, snd, rcv).transposed()
    assert ptr_t.tolist() == [0, 1, 2] and perm_t.tolist()[:2] == [2, 0]
    assert np.array_equal(ConvGraph.build(2, snd, rcv).receiver_ptr.numpy(), [0, 2, 3])
