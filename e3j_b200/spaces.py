"""Minimal O(3) representation bookkeeping for the fused convolution path.

Only what the convolution table builder needs is restated here: parsing of
e3nn-style strings, block slices, the Clebsch-Gordan selection rule with an
output filter, and the (l, p) sort used to order output rows.

Reference behaviour followed (paths relative to the e3j project root):
  * irrep ordering, parity rule ``p == (-1)**l`` first: src/e3j/spaces/o3.py:108-114
  * selection rule + filter: src/e3j/spaces/o3.py:189-230
  * slices / sort / regroup: src/e3j/spaces/space.py:120-182
"""

from __future__ import annotations

import itertools
import re
from dataclasses import dataclass
from typing import Iterable, Iterator

import numpy as np

_BLOCK_RE = re.compile(r"^\s*(?:(\d+)\s*x\s*)?(\d+)([eo])\s*$")


@dataclass(frozen=True)
class O3Irrep:
    """Irreducible representation of O(3): degree ``l`` and parity ``p``."""

    l: int  # noqa: E741
    p: int = 1

    @property
    def dim(self) -> int:
        return 2 * self.l + 1

    def sort_key(self) -> tuple[int, int]:
        """Natural parity ``(-1)**l`` sorts before the pseudo-tensor parity."""
        return (self.l, 0 if self.p == (-1) ** self.l else 1)

    def __str__(self) -> str:
        return f"{self.l}{'e' if self.p == 1 else 'o'}"


class O3Space:
    """Direct sum of ``(multiplicity, irrep)`` blocks."""

    def __init__(self, blocks: "str | O3Space | Iterable"):
        if isinstance(blocks, O3Space):
            self.blocks = list(blocks.blocks)
        elif isinstance(blocks, str):
            self.blocks = self._parse(blocks)
        else:
            self.blocks = [self._coerce(b) for b in blocks]

    @staticmethod
    def _parse(text: str) -> list[tuple[int, O3Irrep]]:
        out = []
        for chunk in text.split("+"):
            m = _BLOCK_RE.match(chunk)
            if m is None:
                raise ValueError(f"Could not parse block '{chunk}' as '(<mul>x)<irrep>'")
            mul = int(m.group(1)) if m.group(1) else 1
            out.append((mul, O3Irrep(int(m.group(2)), 1 if m.group(3) == "e" else -1)))
        return out

    @staticmethod
    def _coerce(block) -> tuple[int, O3Irrep]:
        if len(block) == 3:
            mul, l, p = block
            return int(mul), O3Irrep(int(l), int(p))
        mul, ir = block
        if isinstance(ir, str):
            ir = O3Space._parse(ir)[0][1]
        elif not isinstance(ir, O3Irrep):
            ir = O3Irrep(*ir)
        return int(mul), ir

    def __iter__(self) -> Iterator[tuple[int, O3Irrep]]:
        return iter(self.blocks)

    def __len__(self) -> int:
        return len(self.blocks)

    @property
    def dim(self) -> int:
        return sum(m * ir.dim for m, ir in self.blocks)

    @property
    def num_irreps(self) -> int:
        return sum(m for m, _ in self.blocks)

    @property
    def l_max(self) -> int:
        return max(ir.l for _, ir in self.blocks)

    def slices(self) -> list[slice]:
        out, begin = [], 0
        for m, ir in self.blocks:
            out.append(slice(begin, begin + m * ir.dim))
            begin += m * ir.dim
        return out

    def sort(self) -> tuple["O3Space", np.ndarray]:
        """Stable sort of blocks by (l, parity); returns the block permutation."""
        order = sorted(range(len(self.blocks)), key=lambda i: (self.blocks[i][1].sort_key(), i))
        return O3Space([self.blocks[i] for i in order]), np.asarray(order, dtype=np.int64)

    def regroup(self) -> "O3Space":
        """Sort, then merge neighbouring blocks of equal (l, p)."""
        blocks = self.sort()[0].blocks
        if len(blocks) <= 1:
            return O3Space(blocks)
        merged = [list(blocks[0])]
        for m, ir in blocks[1:]:
            if ir == merged[-1][1]:
                merged[-1][0] += m
            else:
                merged.append([m, ir])
        return O3Space([(m, ir) for m, ir in merged])

    @staticmethod
    def otimes(lhs, rhs, target_filter=None) -> "O3Space":
        """Irreducible content of ``lhs x rhs`` by |l1-l2| <= l <= l1+l2, in
        path order (lhs block major, rhs block, then increasing l), keeping
        only the (l, p) pairs present in ``target_filter`` when one is given."""
        lhs, rhs = O3Space(lhs), O3Space(rhs)
        keep = None
        if target_filter is not None:
            flt = O3Space(target_filter)
            if any(m != 1 for m, _ in flt):
                raise ValueError("Filter `out` should have multiplicities 1")
            keep = {(ir.l, ir.p) for _, ir in flt}
        out = []
        for (m1, ir1), (m2, ir2) in itertools.product(lhs, rhs):
            p = ir1.p * ir2.p
            for l in range(abs(ir1.l - ir2.l), ir1.l + ir2.l + 1):  # noqa: E741
                if keep is not None and (l, p) not in keep:
                    continue
                out.append((m1 * m2, O3Irrep(l, p)))
        return O3Space(out)

    def __mul__(self, n: int) -> "O3Space":
        return O3Space([(n * m, ir) for m, ir in self.blocks])

    __rmul__ = __mul__

    def __eq__(self, other) -> bool:
        return isinstance(other, O3Space) and self.blocks == other.blocks

    def __hash__(self) -> int:
        return hash(tuple(self.blocks))

    def __str__(self) -> str:
        return " + ".join(f"{m}x{ir}" for m, ir in self.blocks)

    def __repr__(self) -> str:
        return f"O3Space('{self}')"


def full_space(l_max: int) -> O3Space:
    """``0e + 1o + 2e + ...`` with natural parities up to ``l_max``."""
    return O3Space([(1, O3Irrep(l, (-1) ** l)) for l in range(l_max + 1)])
