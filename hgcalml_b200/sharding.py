"""Event sharding for multi-GPU runs: events are independent in every op of the path, so a ragged
batch is split into contiguous runs of whole events, one run per rank, balanced by hit count.  No
collective is needed on the data path; ranks only meet to combine timings or to gather results."""
from __future__ import annotations

import numpy as np


def shard_events(row_splits, world_size: int):
    """Contiguous event ranges [(first, last_exclusive)] per rank, balanced by hits: rank r gets the
    events whose midpoint in the cumulative hit count falls into the r-th of world_size equal parts."""
    rs = np.asarray(row_splits, dtype=np.int64)
    n_events = len(rs) - 1
    total = int(rs[-1] - rs[0])
    if n_events <= 0:
        return [(0, 0)] * world_size
    mid = (rs[:-1] + rs[1:]) / 2.0 - rs[0]
    owner = np.minimum((mid * world_size / max(total, 1)).astype(np.int64), world_size - 1)
    out = []
    for r in range(world_size):
        mine = np.nonzero(owner == r)[0]
        out.append((int(mine[0]), int(mine[-1]) + 1) if len(mine) else (0, 0))
    return out


def local_row_splits(row_splits, first: int, last: int):
    """Row splits of the shard, rebased so the shard's first hit is 0, and the hit offset to add to
    neighbour indices when results are merged back into the batch's numbering."""
    rs = np.asarray(row_splits, dtype=np.int64)
    return (rs[first:last + 1] - rs[first]).astype(np.int32), int(rs[first])


def merge_indices(local_idx, hit_offset: int):
    """Neighbour indices of a shard in the batch's numbering (-1 padding stays -1)."""
    local_idx = np.asarray(local_idx)
    return np.where(local_idx < 0, local_idx, local_idx + hit_offset)
