"""Equivariant message-passing convolution module.

Mirror of ``e3j.core.Convolution`` (src/e3j/core/convolution.py:40-420) for
torch tensors and the B200 kernels: same constructor arguments, same
``__call__`` signature, same derived attributes (``source``, ``target``,
``coef``).  The module owns no learnable weights; it computes

    m_b = 1/avg_num_neighbors * sum_a (x_a (x) y_ab) (.) s_ab

with the sum over the senders ``a`` of receiver ``b``.  Only the fused CUDA
evaluation exists here (the reference's ``convolution="FUSED_CUDA"`` path,
:193-258); the plain gather/product/mix/scatter evaluation lives in the test
oracle, not in the package.
"""

from __future__ import annotations

import functools

import numpy as np
import torch

from .coef import Coef4D
from .graph import GraphCSR
from .ops import ConvGraph, CUDAConvolutionParams, coef4d_from_table, convolution
from .spaces import O3Space
from .tensor_product import TensorProduct, mix_indices, sparse_coo

LAYOUTS = ("TRAILING_CHANNELS",)


class Convolution:
    def __init__(
        self,
        source,
        target=None,
        *,
        graph_ordering,
        layout="TRAILING_CHANNELS",
        avg_num_neighbors: float | None = None,
        normalization="SQRT_DIM_OUT",
        config=None,
    ):
        """
        Args:
            source: representations of the node and edge features; the third
                source space (one scalar per output irrep) is inferred.
            target: optional filter of multiplicity-1 irreps on the output.
            graph_ordering: ``RECEIVER`` (edges sorted by receiver) or ``SENDER``
                (edges sorted by sender; as in the reference the forward then
                aggregates over the reversed edges, which is the same sum for a
                symmetric graph whose edge features flip with the edge direction,
                src/e3j/core/convolution.py:236-246).  ``NONE`` raises
                ``NotImplementedError`` at call time.
            layout: channel axis; only ``TRAILING_CHANNELS`` is supported by the
                fused convolution (src/e3j/core/convolution.py:274-277).
            avg_num_neighbors: if given, folded into the coefficient values
                (src/e3j/core/convolution.py:133-140).
            normalization: ``SQRT_DIM_OUT`` (default) or ``NONE``.
            config: accepted for signature compatibility; there is one
                implementation path.
        """
        del config
        layout = str(layout).upper().split(".")[-1]
        if layout not in LAYOUTS:
            raise NotImplementedError("the fused convolution only supports TRAILING_CHANNELS layout.")
        otimes = TensorProduct((source[0], source[1]), target, normalization=normalization)
        if avg_num_neighbors is not None:
            otimes.coef = sparse_coo(
                otimes.values / avg_num_neighbors, otimes.indices, otimes.coef.shape
            )
        self._otimes = otimes
        self._mix_indices = mix_indices(otimes.target)
        self.num_scalars = otimes.target.num_irreps
        self.source = (*otimes.source, self.num_scalars * O3Space("0e"))
        self.target = otimes.target
        self.avg_num_neighbors = avg_num_neighbors
        self.layout = layout
        self.normalization = otimes.normalization
        self.graph_ordering = str(graph_ordering).upper().split(".")[-1]
        #: set to True to bypass the unrolled kernels (table-driven kernels only)
        self.force_generic = False

    @functools.cached_property
    def coef(self) -> Coef4D:
        """Packed-table source: rows (val, i, j, k, l = mix_idx[i]) sorted by (i, j, k)
        (src/e3j/core/convolution.py:159-170)."""
        return coef4d_from_table(self._otimes.values, self._otimes.indices, self._mix_indices)

    @functools.cached_property
    def _coef_packed(self) -> np.ndarray:
        return self.coef.pack()

    @property
    def params(self) -> CUDAConvolutionParams:
        return CUDAConvolutionParams(num_out=self.target.dim, num_scalars=self.num_scalars)

    def prepare_graph(self, num_nodes: int, senders: torch.Tensor, receivers: torch.Tensor) -> ConvGraph:
        """Derive the CSR views once for a graph that is reused across calls; pass
        the result as ``senders`` (``receivers`` is then ignored)."""
        return ConvGraph.build(num_nodes, senders, receivers, self.graph_ordering)

    @functools.cached_property
    def y_parity(self) -> np.ndarray:
        """O3 parity (+1 / -1) of every edge-feature component (src/e3j/core/convolution.py:238-246)."""
        return np.concatenate([np.full(m * ir.dim, float(ir.p), dtype=np.float32) for m, ir in self._otimes.source[1]])

    def __call__(
        self,
        node_features: torch.Tensor,
        edge_features: torch.Tensor,
        edge_scalars: torch.Tensor,
        senders,
        receivers=None,
        node_mask: torch.Tensor | None = None,
    ) -> torch.Tensor:
        """Sum of messages on receiver nodes.

        Args:
            node_features: (num_nodes, num_x, num_channels)
            edge_features: (num_edges, num_y)
            edge_scalars: (num_edges, num_scalars, num_channels)
            senders, receivers: (num_edges,) indices, edges sorted by the endpoint
                named by ``graph_ordering``; ``DUMMY_INDEX`` marks padding edges.
            node_mask: optional boolean (num_nodes,), ``False`` for trailing
                padding nodes; edges touching them are dropped.
        """
        if self.graph_ordering == "NONE":
            raise NotImplementedError("CUDA convolution only supports SENDER and RECEIVER ordering.")
        if node_mask is not None:
            if isinstance(senders, ConvGraph):
                raise ValueError("node_mask cannot be combined with a prepared graph")
            senders, receivers = GraphCSR.mask_edges(senders, receivers, node_mask)
        dtype = torch.promote_types(torch.promote_types(node_features.dtype, edge_features.dtype), edge_scalars.dtype)
        if edge_scalars.ndim == 2:
            edge_scalars = edge_scalars.reshape(edge_scalars.shape[0], self.num_scalars, -1)
        return convolution(
            self._coef_packed,
            node_features.to(dtype),
            edge_features.to(dtype),
            edge_scalars.to(dtype),
            senders,
            receivers,
            self.params,
            self.graph_ordering,
            self.y_parity if self.graph_ordering == "SENDER" else None,
            force_generic=self.force_generic,
        )
