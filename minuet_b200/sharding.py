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


def gather_rows(local: torch.Tensor, dst: int = 0, group=None,
                counts: Optional[Sequence[int]] = None) -> Optional[List[torch.Tensor]]:
    """Gather a different number of rows from every rank onto ``dst``.

    Every other rank sends exactly its rows to ``dst`` (one point-to-point message
    each, posted as one batch); nothing is padded and nothing travels to the ranks
    that do not need it.  ``counts`` are the row counts of all ranks when the caller
    knows them (for example from the shard plan); without them one small all_gather
    and one host read establish them.  Returns the list of per-rank tensors on
    ``dst`` (its own entry is ``local`` itself) and None elsewhere.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    local = local.contiguous()
    if counts is None:
        count = torch.tensor([local.shape[0]], dtype=torch.int64, device=local.device)
        every = torch.empty(world, dtype=torch.int64, device=local.device)
        dist.all_gather_into_tensor(every, count, group=group)
        counts = every.cpu().tolist()
    if int(counts[rank]) != local.shape[0]:
        raise ValueError(f"rank {rank} holds {local.shape[0]} rows, the plan says {counts[rank]}")
    if rank != dst:
        if local.shape[0] > 0:
            for work in dist.batch_isend_irecv([dist.P2POp(dist.isend, local, dst, group)]):
                work.wait()
        return None
    parts = [local if r == dst else
             torch.empty((int(counts[r]),) + tuple(local.shape[1:]), dtype=local.dtype,
                         device=local.device) for r in range(world)]
    ops = [dist.P2POp(dist.irecv, parts[r], r, group) for r in range(world)
           if r != dst and int(counts[r]) > 0]
    if ops:
        for work in dist.batch_isend_irecv(ops):
            work.wait()
    return parts


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
