"""Replica data parallelism over independent streams: host-side plumbing.

The reference is single-device (no cudaSetDevice, no collective anywhere).  Streams are independent, so a
batch of streams is cut into contiguous slices, one per rank; every rank holds a full weight replica and its own
recurrent states, and no collective sits on the decode path.  torch.distributed is used only to gather sampled
token ids (and, in check mode, logits) for the cross-rank comparison, and to take the max of the ranks' timings.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np


def partition_streams(n_streams: int, world: int, rank: int) -> Tuple[int, int]:
    """[start, stop) of the stream indices rank `rank` decodes: contiguous, sizes differ by at most one."""
    if world < 1 or not 0 <= rank < world or n_streams < 0:
        raise ValueError("bad partition arguments")
    base, extra = divmod(n_streams, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def launch_groups(n_local: int, max_batch: int) -> List[Tuple[int, int]]:
    """Cut a rank's streams into launches of at most max_batch streams (the kernel decodes <= 8 per launch)."""
    return [(s, min(s + max_batch, n_local)) for s in range(0, n_local, max_batch)]


def gather_ids(local_ids: np.ndarray, n_streams: int, world: int, rank: int, dist=None) -> np.ndarray:
    """All ranks' sampled ids in global stream order, shape [steps, n_streams].  local_ids: [steps, n_local]."""
    if world == 1:
        return np.asarray(local_ids)
    import torch
    steps = local_ids.shape[0]
    width = max(partition_streams(n_streams, world, r)[1] - partition_streams(n_streams, world, r)[0]
                for r in range(world))
    pad = np.full((steps, width), -1, np.int64)
    pad[:, :local_ids.shape[1]] = local_ids
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    mine = torch.from_numpy(pad).to(dev)
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    cols = []
    for r, t in enumerate(parts):
        a, b = partition_streams(n_streams, world, r)
        cols.append(t.cpu().numpy()[:, : b - a])
    return np.concatenate(cols, axis=1)


def max_over_ranks(value: float, world: int, dist=None) -> float:
    if world == 1:
        return float(value)
    import torch
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
