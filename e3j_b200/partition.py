"""Spatial slab decomposition of a radius graph across the GPUs of one box.

Not part of the reference (its multi-device mode is data parallel over independent
graphs and issues no collective, src/e3j/ops/convolution.py:213-263); this is the
partitioned large-graph mode of the B200 build.

Rank g owns the receivers whose x coordinate lies in slab g.  The convolution
output of a receiver needs the features of its senders only, so a rank needs, besides
its own nodes, the *halo*: nodes of other ranks that send an edge into the slab.
Local numbering on a rank:

    [ interior owned | boundary owned | halo ]
      0 .. n_int       n_int .. n_own   n_own .. n_loc

"interior" receivers have all their senders owned, so their edges can be processed
while the halo rows are still in flight.  Edges are kept receiver-sorted in local
numbering.  The exchange plan lists, per peer, which owned rows go out
(`send_rows[p]`, local ids) and where that peer's rows land in the halo block
(`recv_slice[p]`); the backward pass runs the same plan in reverse and adds the
returned partial dx rows in ascending peer order, which keeps results reproducible.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class SlabPart:
    rank: int
    world: int
    n_int: int  # interior owned receivers (local ids [0, n_int))
    n_own: int  # owned nodes (local ids [0, n_own))
    n_loc: int  # owned + halo nodes
    global_ids: np.ndarray  # (n_loc,) global id of each local node
    sender: np.ndarray  # (E_loc,) local sender ids, int32
    receiver: np.ndarray  # (E_loc,) local receiver ids (sorted, all < n_own), int32
    edge_ids: np.ndarray  # (E_loc,) global edge index of each local edge
    send_rows: dict = field(default_factory=dict)  # peer -> int64 local ids of owned rows to send
    recv_slice: dict = field(default_factory=dict)  # peer -> (start, stop) in local numbering (halo block)

    @property
    def peers(self) -> list[int]:
        return sorted(set(self.send_rows) | set(self.recv_slice))


def slab_of(x: np.ndarray, lo: float, hi: float, world: int) -> np.ndarray:
    """Slab index of each coordinate for `world` equal slabs of [lo, hi)."""
    w = (hi - lo) / world
    return np.clip(np.floor((x - lo) / w).astype(np.int64), 0, world - 1)


def morton_order(positions: np.ndarray, cell: float) -> np.ndarray:
    """Permutation sorting points along the Z-order curve of a grid of `cell`-sized boxes
    (ties broken by index).  Consecutive points are close in space, so consecutive
    receivers gather largely the same sender rows and those stay in L2."""
    q = np.floor((positions - positions.min(axis=0)) / cell).astype(np.uint64)
    assert q.max(initial=0) < (1 << 21)
    code = np.zeros(q.shape[0], np.uint64)
    for bit in range(21):
        for dim in range(3):
            code |= ((q[:, dim] >> np.uint64(bit)) & np.uint64(1)) << np.uint64(3 * bit + dim)
    return np.lexsort((np.arange(q.shape[0]), code))


def _ordered(ids: np.ndarray, positions: np.ndarray, cell: float | None) -> np.ndarray:
    """`ids` ascending, or along the Z-order curve of their positions when `cell` is given."""
    if cell is None or ids.size == 0:
        return ids
    return ids[morton_order(positions[ids], cell)]


def partition_slabs(positions: np.ndarray, sender: np.ndarray, receiver: np.ndarray, world: int,
                    lo: float | None = None, hi: float | None = None, cell: float | None = None) -> list[SlabPart]:  # fmt: skip
    """Split a receiver-sorted global edge list into per-rank local graphs.

    `sender` / `receiver` are global ids of real edges (no padding).  Returns one
    :class:`SlabPart` per rank with mutually consistent exchange plans.  With `cell`
    the interior and the boundary nodes are each numbered along a Z-order curve
    (:func:`morton_order`) instead of by ascending global id.
    """
    n = positions.shape[0]
    lo = float(positions[:, 0].min()) if lo is None else lo
    hi = float(np.nextafter(positions[:, 0].max(), np.inf)) if hi is None else hi
    owner = slab_of(positions[:, 0], lo, hi, world)
    sender = np.asarray(sender, np.int64)
    receiver = np.asarray(receiver, np.int64)
    parts = []
    halo_of = []  # per rank: dict peer -> sorted global ids needed from that peer
    for g in range(world):
        e_mask = owner[receiver] == g
        e_ids = np.nonzero(e_mask)[0]
        snd_g, rcv_g = sender[e_ids], receiver[e_ids]
        owned = np.nonzero(owner == g)[0]
        foreign = owner[snd_g] != g
        # a receiver is "boundary" if any of its senders is foreign
        is_boundary = np.zeros(n, bool)
        is_boundary[rcv_g[foreign]] = True
        interior = _ordered(owned[~is_boundary[owned]], positions, cell)
        boundary = _ordered(owned[is_boundary[owned]], positions, cell)
        halo = np.unique(snd_g[foreign])
        halo = halo[np.lexsort((halo, owner[halo]))]  # grouped by owning peer, ascending id inside
        gids = np.concatenate([interior, boundary, halo])
        local = np.full(n, -1, np.int64)
        local[gids] = np.arange(gids.size)
        ls, lr = local[snd_g], local[rcv_g]
        order = np.argsort(lr, kind="stable")  # stable: keeps the global (receiver-sorted) edge order inside a segment
        part = SlabPart(g, world, interior.size, owned.size, gids.size, gids, ls[order].astype(np.int32),
                        lr[order].astype(np.int32), e_ids[order])  # fmt: skip
        need = {}
        start = owned.size
        for p in np.unique(owner[halo]):
            ids = halo[owner[halo] == p]
            need[int(p)] = ids
            part.recv_slice[int(p)] = (start, start + ids.size)
            start += ids.size
        halo_of.append(need)
        parts.append(part)
    # send lists: what peer p needs from g, in the order p stores it
    for g, part in enumerate(parts):
        local = np.full(n, -1, np.int64)
        local[part.global_ids[: part.n_own]] = np.arange(part.n_own)
        for p in range(world):
            ids = halo_of[p].get(g)
            if ids is not None and p != g:
                rows = local[ids]
                assert (rows >= 0).all()
                part.send_rows[p] = rows
    return parts


def elongated_box_graph(world: int, nodes_per_slab: int, cutoff: float, density: float = 0.1, seed: int = 0):
    """Open (non-periodic) box of `world` cubes of `nodes_per_slab` nodes each laid along x,
    uniform density; directed radius graph sorted by receiver.  With world == 1 this is the
    single-GPU cube workload."""
    from .problems import Graph, radius_graph

    side = (nodes_per_slab / density) ** (1.0 / 3.0)
    rng = np.random.default_rng(seed)
    n = world * nodes_per_slab
    pos = rng.uniform(0.0, 1.0, size=(n, 3)) * np.array([side * world, side, side])
    snd, rcv, vec = radius_graph(pos, cutoff, None)
    g = Graph(n, pos, snd, rcv, vec, None, n, snd.shape[0], {"side": side, "cutoff": cutoff, "world": world, "seed": seed})
    return g, 0.0, side * world


def periodic_slab_part(rank: int, world: int, positions: np.ndarray, box: float, cutoff: float,
                       cell: float | None = None):  # fmt: skip
    """The :class:`SlabPart` of one rank of a fully periodic cubic box, built from the
    positions alone: only the rank's slab and the `cutoff`-wide layers next to its two
    faces are searched, so a million-node graph never exists in one piece.  Same
    numbering, edge order and exchange plan as ``partition_slabs`` gives for the global
    radius graph (`edge_ids` is left empty).  Returns ``(part, vectors)`` with
    ``vectors[e] = pos[receiver] - pos[sender]`` (minimum image) of the local edges.
    """
    from scipy.spatial import cKDTree

    n = positions.shape[0]
    pos = np.mod(positions, box)
    pos[pos >= box] -= box
    owner = slab_of(pos[:, 0], 0.0, box, world)
    width = box / world
    if world > 1 and width + 2 * cutoff >= box:
        raise ValueError("slabs are too thin for the periodic box: a halo would wrap onto its own slab")
    if world == 1:
        cand = np.arange(n)
        tree = cKDTree(pos, boxsize=box)
    else:
        # x relative to the slab's lower face, unwrapped: [-cutoff, width + cutoff)
        xr = np.mod(pos[:, 0] - rank * width, box)
        xr[xr >= box] -= box
        xu = np.where(xr >= box - cutoff, xr - box, xr)
        mine = owner == rank
        cand = np.nonzero(mine | ((xu >= -cutoff) & (xu < width + cutoff)))[0]
        span = width + 4 * cutoff + 2.0  # wider than the candidates' extent + cutoff: no wrap along x
        pts = np.stack([np.clip(xu[cand] + cutoff + 1.0, 0.0, np.nextafter(span, 0.0)), pos[cand, 1], pos[cand, 2]], axis=1)
        tree = cKDTree(pts, boxsize=[span, box, box])
    pairs = tree.query_pairs(cutoff, output_type="ndarray")
    a, b = cand[pairs[:, 0]], cand[pairs[:, 1]]
    snd = np.concatenate([a, b])
    rcv = np.concatenate([b, a])
    keep = owner[rcv] == rank
    snd_g, rcv_g = snd[keep], rcv[keep]
    foreign = owner[snd_g] != rank
    owned = np.nonzero(owner == rank)[0]
    is_boundary = np.zeros(n, bool)
    is_boundary[rcv_g[foreign]] = True
    interior = _ordered(owned[~is_boundary[owned]], positions, cell)
    boundary = _ordered(owned[is_boundary[owned]], positions, cell)
    halo = np.unique(snd_g[foreign])
    halo = halo[np.lexsort((halo, owner[halo]))]
    gids = np.concatenate([interior, boundary, halo])
    local = np.full(n, -1, np.int64)
    local[gids] = np.arange(gids.size)
    order = np.lexsort((snd_g, local[rcv_g]))  # local receiver major, global sender minor
    snd_g, rcv_g = snd_g[order], rcv_g[order]
    part = SlabPart(rank, world, interior.size, owned.size, gids.size, gids, local[snd_g].astype(np.int32),
                    local[rcv_g].astype(np.int32), np.empty(0, np.int64))  # fmt: skip
    start = owned.size
    for p in np.unique(owner[halo]):
        cnt = int((owner[halo] == p).sum())
        part.recv_slice[int(p)] = (start, start + cnt)
        start += cnt
    # what each peer needs from this rank: the owned senders of the edges into that peer's slab,
    # i.e. the owned ends of the cross pairs found above, in ascending global id
    cross = owner[rcv] != rank
    cs, cr = snd[cross], rcv[cross]
    own_end = owner[cs] == rank
    cs, cr = cs[own_end], cr[own_end]
    for p in np.unique(owner[cr]):
        ids = np.unique(cs[owner[cr] == p])
        part.send_rows[int(p)] = local[ids]
    vec = pos[rcv_g] - pos[snd_g]
    vec -= box * np.round(vec / box)
    return part, vec
