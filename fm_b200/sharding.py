"""How the scan is spread over the GPUs of one box.

Rows (the B*D independent recurrences) shard with no communication at all: each rank owns a
contiguous block of rows and runs the one-GPU kernels on it; the result is bit-identical to the
one-GPU result because no arithmetic crosses a row.  The reference has no multi-GPU code; this
is new.  (Splitting along T is in ``fm_b200.time_split``.)
"""
from __future__ import annotations

from typing import List, Tuple


def row_blocks(rows: int, world: int) -> List[Tuple[int, int]]:
    """Contiguous [begin, end) row ranges, one per rank; sizes differ by at most one row."""
    if rows < 0 or world < 1:
        raise ValueError("rows must be >= 0 and world >= 1")
    base, extra = divmod(rows, world)
    out, begin = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append((begin, begin + n))
        begin += n
    return out


def time_blocks(T: int, world: int) -> List[Tuple[int, int]]:
    """Contiguous [begin, end) time ranges in scan order, one per rank."""
    return row_blocks(T, world)


def shard_rows(tensor, rank: int, world: int):
    """This rank's block of rows of a (B, D, T) or (R, T) tensor, as a contiguous (r, T) view."""
    flat = tensor.reshape(-1, tensor.shape[-1])
    b, e = row_blocks(flat.shape[0], world)[rank]
    return flat[b:e]
