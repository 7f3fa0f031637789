"""Voxelisation: float points -> sorted unique integer voxels
(the step before the hot path; API of minuet/nn/functional/voxelize.py)."""
__all__ = ['voxelize']

from typing import Optional

import torch

from minuet_b200.nn.functional.hash import unique_coordinates
from minuet_b200.nn.functional.indexing import build_sorted_index


def voxelize(coordinates: torch.Tensor, voxel_size, batch_dims: Optional[torch.Tensor] = None,
             return_inverse: bool = False):
    """Floor ``coordinates / voxel_size`` to int32 voxels, sort them (cloud-major,
    then lexicographically) and drop duplicates.

    Returns ``(voxels [U, D], batch_dims [B + 1] or None)`` and, with
    ``return_inverse``, also ``inverse [N]`` such that ``voxels[inverse[i]]`` is the
    voxel of input point ``i`` (for averaging point features per voxel).

    The reference's function has the same purpose but cannot run as shipped (it
    passes a dtype as ``device=`` and skips the sort that its unique step needs,
    minuet/nn/functional/voxelize.py:10-35); this one follows the documented
    intent: floor, sort, unique.
    """
    if coordinates.ndim != 2:
        raise ValueError(f"coordinates must be [N, D] but found {coordinates.ndim}-D")
    size = torch.as_tensor(voxel_size, dtype=coordinates.dtype, device=coordinates.device)
    voxels = torch.floor(coordinates / size).to(torch.int32)
    index = build_sorted_index(voxels, batch_dims=batch_dims)
    sorted_voxels = voxels[index]
    unique, indices = unique_coordinates(sorted_voxels, batch_dims=batch_dims)
    new_batch_dims = None
    if batch_dims is not None:
        new_batch_dims = indices[batch_dims.to(torch.int64)].to(batch_dims.dtype)
    if not return_inverse:
        return unique, new_batch_dims
    # indices[i] = runs closed before sorted row i = the unique voxel of that row; undo the sort
    inverse = torch.empty(voxels.shape[0], dtype=torch.int64, device=voxels.device)
    inverse[index] = indices[:-1].to(torch.int64)
    return unique, new_batch_dims, inverse
