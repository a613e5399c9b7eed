"""The reference's own kernel fixture, restated with its closed-form answers.

Inputs follow lib/e3j_ops/tests/test_convolution.cpp:123-207 and
lib/e3j_ops/tests/test_convolution_bwd.cpp:202-324 of the reference: 4 nodes,
6 receiver-sorted edges (sender = {1,2,0,3,0,1}, receiver_ptr = {0,2,4,5,6}),
`num_strips` independent strips of coefficients (per strip t: rows
(i, j, k) = (2t, 2t, 3t+k') and (2t+1, 2t+1, 3t+k'), k' = 0..2, value 1, scalar
index l = t), x = {1, 2} per strip on every node and channel, y = {3, 4, 5} per
strip on every edge, s = 1 or s[e, t] = (e + 1)(t + 1), cotangent dz = 1.

The reference checks its kernels against CPU loops on these inputs with exact
equality in the forward (test_convolution.cpp:288-290).  All values are small
integers, so the sums are exact in float32 and the answers can be written in
closed form:
    out[r, 2t]   = 12 * sum_{e in seg(r)} s[e, t]        out[r, 2t+1] = 24 * (same sum)
    ds[e, t]     = 1*12 + 2*12 = 36
    dx[a, 2t]    = dx[a, 2t+1] = 12 * sum_{e sent by a} s[e, t]
    dy[e, 3t+k'] = C * (1 + 2) * s[e, t]
"""

import numpy as np

NUM_NODES = 4
SENDER = np.array([1, 2, 0, 3, 0, 1], np.int32)
RECEIVER_PTR = np.array([0, 2, 4, 5, 6], np.int32)
RECEIVER = np.array([0, 0, 1, 1, 2, 3], np.int32)
NUM_EDGES = 6


def make(num_strips: int, channels: int, scale_r: bool):
    t = np.arange(num_strips)
    i = (np.array([0, 0, 0, 1, 1, 1])[None, :] + 2 * t[:, None]).reshape(-1)
    j = i.copy()
    k = (np.array([0, 1, 2, 0, 1, 2])[None, :] + 3 * t[:, None]).reshape(-1)
    l = np.repeat(t, 6)  # noqa: E741
    idx4 = np.stack([i, j, k, l], axis=-1).astype(np.int32)
    val = np.ones(len(i), np.float32)
    x = np.tile(np.tile([1.0, 2.0], num_strips)[None, :, None], (NUM_NODES, 1, channels)).astype(np.float32)
    y = np.tile(np.tile([3.0, 4.0, 5.0], num_strips)[None, :], (NUM_EDGES, 1)).astype(np.float32)
    if scale_r:
        s2 = (np.arange(NUM_EDGES)[:, None] + 1.0) * (t[None, :] + 1.0)
    else:
        s2 = np.ones((NUM_EDGES, num_strips))
    s = np.tile(s2[:, :, None], (1, 1, channels)).astype(np.float32)
    dz = np.ones((NUM_NODES, 2 * num_strips, channels), np.float32)

    out = np.zeros((NUM_NODES, 2 * num_strips, channels), np.float32)
    dx = np.zeros_like(x)
    for e in range(NUM_EDGES):
        out[RECEIVER[e], 0::2] += 12 * s[e]
        out[RECEIVER[e], 1::2] += 24 * s[e]
        dx[SENDER[e], 0::2] += 12 * s[e]
        dx[SENDER[e], 1::2] += 12 * s[e]
    ds = np.full_like(s, 36.0)
    dy = np.repeat(channels * 3.0 * s2, 3, axis=1).astype(np.float32)
    return dict(val=val, idx4=idx4, x=x, y=y, s=s, dz=dz, sender=SENDER, receiver=RECEIVER,
                receiver_ptr=RECEIVER_PTR, num_out=2 * num_strips, out=out, dx=dx, dy=dy, ds=ds)  # fmt: skip


# (num_strips, channels, scale_r): the cases of test_convolution.cpp:316-384 and
# test_convolution_bwd.cpp:507-591 that a float32 / RECEIVER-ordered build covers
CASES = [(1, 32, False), (1, 64, False), (1, 96, False), (1, 128, False), (2, 128, False), (2, 128, True),
         (4, 32, True), (1, 256, False), (8, 128, True), (40, 64, True)]  # fmt: skip
