"""Host-side tables: irreps algebra, CG stacking, output sort, Coef4D packing."""

import numpy as np
import pytest

from e3j_b200.coef import Coef, Coef4D
from e3j_b200.convolution import Convolution
from e3j_b200.spaces import O3Space
from e3j_b200.tensor_product import TensorProduct, mix_indices, sparse_coo


def test_parse_and_dims():
    sp = O3Space("2x0e + 1o+3x2e")
    assert [(m, str(ir)) for m, ir in sp] == [(2, "0e"), (1, "1o"), (3, "2e")]
    assert sp.dim == 2 + 3 + 15 and sp.num_irreps == 6
    assert [(s.start, s.stop) for s in sp.slices()] == [(0, 2), (2, 5), (5, 20)]
    with pytest.raises(ValueError):
        O3Space("0x")


def test_sort_puts_natural_parity_first():
    sp = O3Space("1e+1o+0o+0e")
    assert str(sp.sort()[0]) == "1x0e + 1x0o + 1x1o + 1x1e"


def test_selection_rule_with_filter():
    full = O3Space.otimes("1o", "1o")
    assert str(full) == "1x0e + 1x1e + 1x2e"
    assert str(O3Space.otimes("1o", "1o", "0e+2e")) == "1x0e + 1x2e"
    with pytest.raises(ValueError):
        O3Space.otimes("1o", "1o", "2x0e")


# sizes quoted for the benchmark configurations
@pytest.mark.parametrize(
    "x,dims",
    [("0e+1o", (40, 10, 86, 76)), ("0e+1o+2e+3o", (99, 23, 353, 311))],
)
def test_benchmark_table_sizes(x, dims):
    conv = Convolution((x, "0e+1o+2e+3o"), "0e+1o+2e+3o", graph_ordering="RECEIVER")
    idx = conv.coef.idx.astype(int)
    assert (conv.target.dim, conv.num_scalars, len(conv.coef.val), len({(a, b) for a, b, _, _ in idx})) == dims
    assert conv.coef.idx.dtype == np.uint8  # all dims <= 255 -> narrow indices
    # sorted by (i, j, k); l is the irrep copy of the output row
    keys = idx[:, 0] * 10_000 + idx[:, 1] * 100 + idx[:, 2]
    assert (np.diff(keys) > 0).all()
    assert (idx[:, 3] == mix_indices(conv.target)[idx[:, 0]]).all()
    assert str(conv.source[2]) == f"{conv.num_scalars}x0e"


def test_output_rows_grouped_by_degree():
    tp = TensorProduct(("0e+1o", "0e+1o+2e+3o"), "0e+1o+2e+3o")
    assert str(tp.target) == "2x0e + 3x1o + 3x2e + 2x3o"
    assert [ir.l for ir in tp.target_irreps] == [0, 0, 1, 1, 1, 2, 2, 2, 3, 3]


def test_normalisation_rows_orthonormal():
    """SQRT_DIM_OUT makes every output row of every path a unit vector."""
    tp = TensorProduct(("0e+1o+2e", "0e+1o+2e"), None, normalization="SQRT_DIM_OUT")
    dense = tp.coef.todense().reshape(tp.shape[0], -1).astype(np.float64)
    gram = dense @ dense.T
    assert np.allclose(np.diag(gram), 1.0, atol=1e-6)
    none = TensorProduct(("1o", "1o"), None, normalization="NONE").coef.todense()
    # 0e row of 1o x 1o: delta / sqrt(3) * (norm 1 block) -> each entry 1/sqrt(3)
    assert np.allclose(none[0][np.nonzero(none[0])], 1 / np.sqrt(3), atol=1e-6)


def test_avg_num_neighbors_scales_values():
    a = Convolution(("0e+1o", "0e+1o"), None, graph_ordering="RECEIVER")
    b = Convolution(("0e+1o", "0e+1o"), None, graph_ordering="RECEIVER", avg_num_neighbors=4.0)
    assert np.allclose(b.coef.val * 4.0, a.coef.val)
    assert (a.coef.idx == b.coef.idx).all()


def test_multiplicity_order_k0_row_major():
    """Output copies of a path are ordered k0 = k1 * m2 + k2."""
    tp = TensorProduct(("2x0e", "3x0e"), None, normalization="NONE")
    idx = tp.indices.astype(int)
    assert (idx[:, 0] == idx[:, 1] * 3 + idx[:, 2]).all() and len(idx) == 6


def test_sparse_coo_coalesces():
    c = sparse_coo([1.0, 2.0, -2.0, 5.0], [[1, 0, 0], [0, 1, 1], [0, 1, 1], [1, 0, 0]], (2, 2, 2))
    assert c.nnz == 1 and c.data[0] == 6.0 and tuple(c.indices[0]) == (1, 0, 0)
    assert sparse_coo([1.0], [[300, 0, 0]], (301, 1, 1)).indices.dtype == np.int32


# byte sizes of the device structs (lib/e3j_ops/cuda/convolution.cuh:39-44,
# tests/test_ops/test_coef.py:30-46 in the reference)
@pytest.mark.parametrize(
    "cls,idx,val,size",
    [
        (Coef4D, "int32", "float32", 32), (Coef4D, "uint8", "float32", 8), (Coef4D, "int32", "float64", 32),
        (Coef4D, "uint8", "float64", 16), (Coef4D, "int32", "float16", 32), (Coef4D, "uint8", "float16", 8),
        (Coef, "int32", "float32", 16), (Coef, "uint8", "float32", 8), (Coef, "uint8", "float64", 16),
    ],
)  # fmt: skip
def test_struct_sizes(cls, idx, val, size):
    assert cls.struct_dtype(val, idx).itemsize == size


@pytest.mark.parametrize("idx_dtype", ["uint8", "int32"])
def test_pack_roundtrip_and_layout(idx_dtype):
    rng = np.random.default_rng(0)
    val = rng.standard_normal(7).astype(np.float32)
    idx = rng.integers(0, 200, size=(7, 4))
    packed = Coef4D(val, idx, idx_dtype=idx_dtype).pack()
    assert packed.dtype == np.dtype(idx_dtype) and packed.shape == (7, 8)
    raw = packed.view(np.uint8).reshape(7, -1)
    assert (raw[:, :4].copy().view(np.float32)[:, 0] == val).all()  # value first
    width = np.dtype(idx_dtype).itemsize
    assert (raw[:, 4 : 4 + width].copy().view(idx_dtype)[:, 0] == idx[:, 0]).all()  # then i
    back = Coef4D.unpack(packed, "float32")
    assert (back.val == val).all() and (back.idx == idx).all()


def test_transpose_is_stable_by_new_first_column():
    c = Coef4D(np.arange(4, dtype=np.float32), np.array([[0, 1, 0, 0], [0, 0, 1, 0], [1, 1, 2, 1], [1, 0, 0, 1]]))
    t = c.transpose((1, 0, 2, 3))
    assert t.idx[:, 0].tolist() == [0, 0, 1, 1] and t.val.tolist() == [1.0, 3.0, 0.0, 2.0]
