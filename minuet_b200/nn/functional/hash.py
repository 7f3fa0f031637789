"""Unique over sorted coordinates (mirror of minuet/nn/functional/hash.py)."""
__all__ = ['unique_coordinates']

from typing import Optional

import torch

from minuet_b200 import _lib, engine


def unique_coordinates(coordinates: torch.Tensor, batch_dims: Optional[torch.Tensor] = None):
    """Remove duplicates from **sorted** coordinates
    (minuet/nn/functional/hash.py:28-50).

    Returns ``(unique [U, D], indices [N + 1])`` where ``indices[i + 1]`` counts
    the unique rows among the first ``i + 1`` input rows; ``indices`` is int64
    for one cloud and ``batch_dims.dtype`` for a batch
    (csrc/minuet/torch/cuda_unique_coordinates.cu:17,53).  Equal rows on both
    sides of a cloud boundary stay separate.
    """
    engine.require_cuda(coordinates, batch_dims)
    if coordinates.ndim != 2:
        raise RuntimeError(f"coordinates must be a 2-D tensor but found {coordinates.ndim}-D")
    coords = engine.as_i32_coords(coordinates)
    n, ndim = coords.shape
    bd = engine.as_i64(batch_dims)
    nb = 1 if bd is None else bd.numel() - 1
    device = coords.device
    unique = torch.empty((n, ndim), dtype=torch.int32, device=device)
    indices = torch.empty(n + 1, dtype=torch.int64, device=device)
    lib = engine.lib()
    ws = engine.workspace(lib.mn_map_workspace_bytes(n, n, 1), device)
    _lib.check(lib.mn_unique_coordinates(engine.ptr(coords), n, ndim, engine.ptr(bd), nb,
                                         engine.ptr(unique), engine.ptr(indices), engine.ptr(ws),
                                         ws.numel(), engine.stream_ptr(device)),
               "unique_coordinates")
    count = int(indices[n].item())
    unique = unique[:count]
    if coordinates.dtype != torch.int32:
        unique = unique.to(coordinates.dtype)
    if batch_dims is not None and batch_dims.dtype != torch.int64:
        indices = indices.to(batch_dims.dtype)
    return unique, indices
