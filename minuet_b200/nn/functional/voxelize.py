"""Voxelisation: float points -> sorted unique integer voxels
(the step before the hot path; API of minuet/nn/functional/voxelize.py)."""
__all__ = ['voxelize']

from typing import Optional

import torch

from minuet_b200 import _lib, engine
from minuet_b200.nn.functional.hash import unique_coordinates
from minuet_b200.nn.functional.indexing import build_sorted_index


def voxelize(coordinates: torch.Tensor, voxel_size, batch_dims: Optional[torch.Tensor] = None,
             return_inverse: bool = False, features: Optional[torch.Tensor] = None):
    """Floor ``coordinates / voxel_size`` to int32 voxels, sort them (cloud-major,
    then lexicographically) and drop duplicates.

    Returns ``(voxels [U, D], batch_dims [B + 1] or None)`` and, with
    ``return_inverse``, also ``inverse [N]`` such that ``voxels[inverse[i]]`` is the
    voxel of input point ``i``.  With ``features [N, C]`` (fp32 / fp16 / bf16) the
    result also carries ``voxel_features [U, C]``, the mean of the features of the
    points of every voxel (one kernel over the sorted runs, fp32 sums in a fixed
    order), appended last: ``(voxels, batch_dims[, inverse], voxel_features)``.

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
    result = [unique, new_batch_dims]
    run_ids = indices[:-1].to(torch.int64).contiguous()
    if return_inverse:
        # indices[i] = runs closed before sorted row i = the unique voxel of that row; undo the sort
        inverse = torch.empty(voxels.shape[0], dtype=torch.int64, device=voxels.device)
        inverse[index] = run_ids
        result.append(inverse)
    if features is not None:
        if features.ndim != 2 or features.shape[0] != coordinates.shape[0]:
            raise ValueError("features must be [N, C] with one row per point")
        engine.require_cuda(features)
        feats = features.contiguous()
        means = torch.empty((unique.shape[0], feats.shape[1]), dtype=feats.dtype,
                            device=feats.device)
        _lib.check(engine.lib().mn_voxel_mean(
            engine.ptr(feats), feats.shape[0], feats.shape[1], engine.dtype_code(feats.dtype),
            engine.ptr(index.to(torch.int64).contiguous()), engine.ptr(run_ids), engine.ptr(means),
            engine.stream_ptr(feats.device)), "voxel_mean")
        result.append(means)
    return tuple(result)
