"""Stacked Clebsch-Gordan table of the convolution's tensor product.

Host-side, numpy, built once per module — mirrors what the reference's
``TensorProduct`` contributes to the fused convolution path:

  * target inference with an (l, p) filter:  src/e3j/core/tensor_product.py:139-145
  * stacking of per-path CG blocks, ``k0 = k1*m2 + k2`` multiplicity order and
    the SQRT_DIM_OUT factor sqrt(2 l0 + 1):   src/e3j/core/tensor_product.py:203-274
  * permutation of the output rows so that blocks are grouped by (l, p):
                                               src/e3j/core/tensor_product.py:184-200
  * COO coalescing (lexicographic sort by (i, j, k), duplicates summed, zeros
    dropped), float32 values, uint8 indices when every dim <= 255:
                                               src/e3j/utils/sparse.py:29-126
  * ``mix_indices`` of ScalarMixing:           src/e3j/core/scalar_mixing.py:62-67
"""

from __future__ import annotations

import itertools
from dataclasses import dataclass

import numpy as np

from .spaces import O3Space
from .wigner import clebsch_gordan

NORMALIZATIONS = ("NONE", "SQRT_DIM_OUT")


def narrow_index_dtype(shape) -> np.dtype:
    return np.dtype(np.uint8) if max(shape) <= 255 else np.dtype(np.int32)


@dataclass(frozen=True, eq=False)
class SparseCOO:
    data: np.ndarray  # (nnz,) float32
    indices: np.ndarray  # (nnz, ndim) uint8 | int32
    shape: tuple

    @property
    def nnz(self) -> int:
        return int(self.indices.shape[0])

    def todense(self) -> np.ndarray:
        dense = np.zeros(self.shape, dtype=self.data.dtype)
        np.add.at(dense, tuple(self.indices.astype(np.int64).T), self.data)
        return dense


def sparse_coo(values, indices, shape) -> SparseCOO:
    """Coalesced COO array: sorted by flat row-major key, duplicates summed,
    exact zeros dropped, values cast to float32."""
    shape = tuple(int(n) for n in shape)
    values = np.asarray(values).astype(np.float32)
    indices = np.asarray(indices, dtype=np.int64).reshape(-1, len(shape))
    if indices.shape[0] != values.shape[0]:
        raise ValueError(f"Got {values.shape[0]} values for {indices.shape[0]} indices.")
    if indices.size and ((indices < 0).any() or (indices >= np.asarray(shape)).any()):
        raise ValueError(f"Out of bounds indices for shape {shape}.")
    keys = np.ravel_multi_index(tuple(indices.T), shape) if indices.size else np.zeros(0, np.int64)
    order = np.argsort(keys, kind="stable")
    keys = keys[order]
    first = np.ones(keys.shape[0], dtype=bool)
    if keys.size:
        first[1:] = keys[1:] != keys[:-1]
    summed = np.zeros(int(np.count_nonzero(first)), dtype=values.dtype)
    np.add.at(summed, np.cumsum(first) - 1, values[order])
    indices = indices[order[first]]
    keep = summed != 0
    return SparseCOO(summed[keep], indices[keep].astype(narrow_index_dtype(shape)), shape)


def stack_clebsch_gordan(target: O3Space, in1: O3Space, in2: O3Space, normalization: str) -> SparseCOO:
    """COO (Z, X, Y) table in *path order* (before the output sort)."""
    keep = {(ir.l, ir.p) for _, ir in target}
    values, indices = [], []
    begin_out = 0
    for ((m1, ir1), s1), ((m2, ir2), s2) in itertools.product(
        zip(in1, in1.slices()), zip(in2, in2.slices())
    ):
        k1, k2 = np.mgrid[:m1, :m2].reshape(2, -1)
        p0 = ir1.p * ir2.p
        for l0 in range(abs(ir1.l - ir2.l), ir1.l + ir2.l + 1):
            if (l0, p0) not in keep:
                continue
            dense = clebsch_gordan(l0, ir1.l, ir2.l)
            nz = np.nonzero(dense)
            data = dense[nz]
            if normalization == "SQRT_DIM_OUT":
                data = data * np.sqrt(2 * l0 + 1)
            values.append(np.tile(data, m1 * m2))
            cg_idx = np.stack(nz, axis=-1)
            dims = np.array([2 * l0 + 1, ir1.dim, ir2.dim])
            mul_grid = np.stack((k1 * m2 + k2, k1, k2), axis=-1)
            offsets = np.array([begin_out, s1.start, s2.start]) + mul_grid * dims
            indices.append((cg_idx[None, :] + offsets[:, None]).reshape(-1, 3))
            begin_out += m1 * m2 * (2 * l0 + 1)
    if not values:
        return sparse_coo(np.zeros(0), np.zeros((0, 3)), (target.dim, in1.dim, in2.dim))
    return sparse_coo(np.concatenate(values), np.concatenate(indices, 0), (target.dim, in1.dim, in2.dim))


class TensorProduct:
    """CG table ``coef[z, x, y]`` of ``source[0] (x) source[1]`` restricted to
    the (l, p) pairs of ``target`` (a multiplicity-1 filter), output rows
    grouped by (l, p)."""

    def __init__(self, source, target=None, *, normalization: str = "NONE"):
        if len(source) != 2:
            raise TypeError("TensorProduct expects a binary tuple as source argument.")
        self.source = (O3Space(source[0]), O3Space(source[1]))
        normalization = str(normalization).upper()
        if normalization not in NORMALIZATIONS:
            raise ValueError(f"normalization must be one of {NORMALIZATIONS}")
        self.normalization = normalization
        unsorted = O3Space.otimes(self.source[0], self.source[1], target)
        raw = stack_clebsch_gordan(unsorted, *self.source, normalization)
        # permute output coordinates: blocks sorted by (l, p), stable
        _, order = unsorted.sort()
        sl = unsorted.slices()
        sigma = (
            np.concatenate([np.arange(sl[i].start, sl[i].stop) for i in order])
            if len(order)
            else np.zeros(0, np.int64)
        )
        sigma_inv = np.argsort(sigma)
        idx = raw.indices.astype(np.int64)
        idx = np.concatenate((sigma_inv[idx[:, 0]][:, None], idx[:, 1:]), axis=-1)
        self.coef = sparse_coo(raw.data, idx, raw.shape)
        self.target = unsorted.regroup()
        #: one entry per output irrep copy, in sorted order: (l, p)
        self.target_irreps = [ir for m, ir in self.target for _ in range(m)]

    @property
    def values(self) -> np.ndarray:
        return self.coef.data

    @property
    def indices(self) -> np.ndarray:
        return self.coef.indices

    @property
    def shape(self):
        return self.coef.shape


def mix_indices(space: O3Space) -> np.ndarray:
    """Map output coordinate -> index of its irrep copy (one scalar each)."""
    repeats = []
    for mul, ir in space:
        repeats.extend([ir.dim] * mul)
    return np.repeat(np.arange(len(repeats)), repeats)
