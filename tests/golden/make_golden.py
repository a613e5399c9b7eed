"""Regenerates tests/golden/conv_small.npz.

The reference's Python package cannot be imported where this repository is
built (its JAX dependencies are absent), so these vectors come from the
float64 numpy restatement in oracle/numpy_oracle.py on seeded inputs.  They
pin the restatement and the CUDA path against silent drift; the reference's
own fixture with closed-form answers lives in strip_fixture.py.

    python tests/golden/make_golden.py
"""

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from e3j_b200.convolution import Convolution  # noqa: E402
from e3j_b200.harmonics import Harmonics  # noqa: E402
from oracle import numpy_oracle  # noqa: E402


def main():
    rng = np.random.default_rng(1234)
    n, e, c = 12, 48, 8
    conv = Convolution(("0e+1o", "0e+1o+2e+3o"), "0e+1o+2e+3o", graph_ordering="RECEIVER", avg_num_neighbors=4.0)
    snd = rng.integers(0, n, e).astype(np.int32)
    rcv = np.sort(rng.integers(0, n, e)).astype(np.int32)
    vec = rng.normal(size=(e, 3))
    x = rng.standard_normal((n, 4, c)).astype(np.float32)
    y = Harmonics(3, normalize=True)(vec).astype(np.float32)
    s = rng.standard_normal((e, conv.num_scalars, c)).astype(np.float32)
    dm = rng.standard_normal((n, conv.target.dim, c)).astype(np.float32)
    val, idx4 = conv.coef.val, conv.coef.idx.astype(np.int32)
    out = numpy_oracle.conv_fwd(val, idx4, x, y, s, snd, rcv, conv.target.dim)
    dx, dy, ds = numpy_oracle.conv_bwd(val, idx4, x, y, s, dm, snd, rcv)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "conv_small.npz")
    np.savez_compressed(path, val=val, idx4=idx4, vec=vec, x=x, y=y, s=s, dm=dm, sender=snd, receiver=rcv,
                        out=out, dx=dx, dy=dy, ds=ds)  # fmt: skip
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
