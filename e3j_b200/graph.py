"""CSR adjacency helpers (torch tensors, any device).

Behaviour follows src/e3j/data/graph.py:20-91: ``DUMMY_INDEX = INT32_MAX``
marks padding endpoints, ``receiver_ptr`` is the cumulative in-range receiver
count, ``transpose`` re-sorts the edges by sender with a stable sort and
``mask_edges`` invalidates edges that touch trailing padding nodes.
All derived index buffers are int32.
"""

from __future__ import annotations

import torch

DUMMY_INDEX = 2**31 - 1


def is_dummy_index(index: torch.Tensor) -> torch.Tensor:
    return index == DUMMY_INDEX


def receiver_ptr_from_sorted(num_nodes: int, receiver: torch.Tensor) -> torch.Tensor:
    """``ptr[n] = #{edges with in-range receiver < n}``, int32, length N + 1.
    Out-of-range (padding) receivers are not counted, so they fall outside
    every segment (src/e3j/data/graph.py:53-56; bincount drops them)."""
    r = receiver.to(torch.int64)
    r = r[(r >= 0) & (r < num_nodes)]
    counts = torch.bincount(r, minlength=num_nodes)
    ptr = torch.zeros(num_nodes + 1, dtype=torch.int64, device=receiver.device)
    ptr[1:] = torch.cumsum(counts, 0)
    return ptr.to(torch.int32)


class GraphCSR:
    """Directed-graph adjacency grouped by receiver."""

    def __init__(self, num_nodes: int, sender: torch.Tensor, receiver: torch.Tensor):
        self.num_nodes = int(num_nodes)
        self.sender = sender.to(torch.int32)
        self.receiver = receiver.to(torch.int32)
        self.receiver_ptr = receiver_ptr_from_sorted(self.num_nodes, self.receiver)

    @classmethod
    def sort(cls, num_nodes: int, sender: torch.Tensor, receiver: torch.Tensor):
        """Return (sigma, graph', sigma^-1) sorting edges by receiver (stable)."""
        perm = torch.argsort(receiver.to(torch.int64), stable=True)
        graph = cls(num_nodes, sender[perm], receiver[perm])
        inv = torch.empty_like(perm)
        inv[perm] = torch.arange(perm.numel(), device=perm.device)
        return perm.to(torch.int32), graph, inv.to(torch.int32)

    def transpose(self):
        """Return (sigma, graph_t, sigma^-1) sorting edges by sender instead;
        in ``graph_t`` the roles of sender and receiver are swapped."""
        return GraphCSR.sort(self.num_nodes, self.receiver, self.sender)

    @staticmethod
    def mask_edges(sender: torch.Tensor, receiver: torch.Tensor, node_mask: torch.Tensor):
        """Mark edges touching a (trailing) padding node with ``DUMMY_INDEX``."""
        num_real = int(torch.count_nonzero(node_mask))
        ok = (sender < num_real) & (receiver < num_real)
        dummy = torch.full_like(sender, DUMMY_INDEX)
        return torch.where(ok, sender, dummy), torch.where(ok, receiver, dummy)
