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


def partition_slabs(positions: np.ndarray, sender: np.ndarray, receiver: np.ndarray, world: int,
                    lo: float | None = None, hi: float | None = None) -> list[SlabPart]:  # fmt: skip
    """Split a receiver-sorted global edge list into per-rank local graphs.

    `sender` / `receiver` are global ids of real edges (no padding).  Returns one
    :class:`SlabPart` per rank with mutually consistent exchange plans.
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
        interior = owned[~is_boundary[owned]]
        boundary = owned[is_boundary[owned]]
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
