"""Sharding of independent point clouds over the GPUs of one node.

Clouds of a batch never interact (every kernel confines its searches to one
cloud, convolutions act row-wise given the map), so each rank runs the whole
network on its own clouds and the only exchange is the final gather of the
per-voxel outputs.  One process per GPU; NCCL when the tensors are on a GPU,
gloo for the CPU tests.
"""
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist


def assign_clouds(sizes: Sequence[int], world_size: int) -> List[List[int]]:
    """Greedy longest-first balancing of clouds over ranks by voxel count.
    Deterministic; returns the cloud indices of every rank in ascending order."""
    order = sorted(range(len(sizes)), key=lambda i: (-int(sizes[i]), i))
    load = [0] * world_size
    shards: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda k: (load[k], k))
        shards[r].append(i)
        load[r] += int(sizes[i])
    return [sorted(s) for s in shards]


def take_clouds(coords: np.ndarray, batch_dims: np.ndarray, features: Optional[np.ndarray],
                clouds: Sequence[int]) -> Tuple[np.ndarray, np.ndarray, Optional[np.ndarray]]:
    """Sub-batch made of the given clouds (kept in the given order)."""
    rows = [np.arange(batch_dims[c], batch_dims[c + 1]) for c in clouds]
    index = np.concatenate(rows) if rows else np.zeros(0, dtype=np.int64)
    bounds = np.zeros(len(clouds) + 1, dtype=np.int64)
    bounds[1:] = np.cumsum([len(r) for r in rows])
    feats = None if features is None else np.ascontiguousarray(features[index])
    return np.ascontiguousarray(coords[index]), bounds, feats


def gather_rows(local: torch.Tensor, dst: int = 0, group=None) -> Optional[List[torch.Tensor]]:
    """Gather a different number of rows from every rank onto ``dst``.

    Row counts travel with one all_gather; the rows travel as one padded
    ``[max_rows, C]`` block per rank (all_gather_into_tensor on NCCL, gather on
    gloo).  Returns the list of per-rank tensors on ``dst`` and None elsewhere.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    count = torch.tensor([local.shape[0]], dtype=torch.int64, device=local.device)
    counts = torch.empty(world, dtype=torch.int64, device=local.device)
    dist.all_gather_into_tensor(counts, count, group=group)
    counts = counts.cpu().tolist()
    width = local.shape[1]
    padded = torch.zeros((max(counts), width), dtype=local.dtype, device=local.device)
    padded[:local.shape[0]] = local
    if local.is_cuda:
        out = torch.empty((world, max(counts), width), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out.view(-1, width), padded, group=group)
        blocks = list(out.unbind(0))
    else:
        blocks = [torch.empty_like(padded) for _ in range(world)] if rank == dst else None
        dist.gather(padded, blocks, dst=dst, group=group)
    if rank != dst:
        return None
    return [b[:n] for b, n in zip(blocks, counts)]


def reassemble(per_rank: Sequence[torch.Tensor], shards: Sequence[Sequence[int]],
               sizes: Sequence[int]) -> torch.Tensor:
    """Undo assign_clouds: rows back in the original cloud order."""
    pieces = {}
    for rows, clouds in zip(per_rank, shards):
        start = 0
        for c in clouds:
            pieces[c] = rows[start:start + int(sizes[c])]
            start += int(sizes[c])
    return torch.cat([pieces[c] for c in range(len(sizes))], dim=0)
