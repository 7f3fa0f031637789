"""Coordinate arg-sort and kernel-map query (mirror of minuet/nn/functional/indexing.py)."""
__all__ = ['arg_sort_coordinates', 'build_sorted_index', 'query_sorted_index_with_offsets']

import ctypes
from typing import Optional

import numpy as np
import torch

from minuet_b200 import _lib, engine


def arg_sort_coordinates(coordinates: torch.Tensor,
                         batch_dims: Optional[torch.Tensor] = None,
                         dtype: Optional[torch.dtype] = None,
                         enable_flattening: bool = True):
    """Stable arg-sort of ``coordinates`` ([N, D] int32/int64), cloud-major then
    lexicographic with dimension 0 most significant.

    Same contract as ``minuet.nn.functional.arg_sort_coordinates``
    (minuet/nn/functional/indexing.py:14-56): the result is int32 for a single
    cloud, ``batch_dims.dtype`` for a batch, or ``dtype`` when given.
    With ``enable_flattening`` (the default) the coordinates are packed into one
    64-bit key and sorted once; without it, or when the bounding box needs more than
    63 key bits, one stable radix sort runs per dimension and one on the cloud, as in
    the reference's fallback (arg_sort_coodrinates.cu:333-359).  Same permutation
    either way.
    """
    engine.require_cuda(coordinates, batch_dims)
    if coordinates.ndim != 2:
        raise RuntimeError(f"coordinates must be a 2-D tensor but found {coordinates.ndim}-D")
    coords = engine.as_i32_coords(coordinates)
    n, ndim = coords.shape
    bd = engine.as_i64(batch_dims)
    nb = 1 if bd is None else bd.numel() - 1
    out_dtype = dtype or (torch.int32 if batch_dims is None else batch_dims.dtype)
    index = torch.empty(n, dtype=torch.int64, device=coords.device)
    spec = None
    if n > 0 and enable_flattening:
        try:
            spec = engine.make_keyspec([coords], ndim, nb, 0)
        except NotImplementedError:
            spec = None        # the box is wider than one key: sort dimension by dimension
    if n > 0 and spec is None:
        lib = engine.lib()
        ws = engine.workspace(lib.mn_map_workspace_bytes(n, n, 1), coords.device)
        _lib.check(lib.mn_arg_sort_coordinates_by_dimension(
            engine.ptr(coords), n, ndim, engine.ptr(bd), nb, engine.ptr(index),
            engine.ptr(engine.control_block(coords.device)), engine.ptr(ws), ws.numel(),
            engine.stream_ptr(coords.device)), "arg_sort_coordinates_by_dimension")
    elif n > 0:
        lib = engine.lib()
        ws = engine.workspace(lib.mn_map_workspace_bytes(n, n, 1), coords.device)
        _lib.check(lib.mn_arg_sort_coordinates(
            engine.ptr(coords), n, ndim, engine.ptr(bd), nb, ctypes.byref(spec), engine.ptr(index),
            engine.ptr(engine.status_word(coords.device)), engine.ptr(ws), ws.numel(),
            engine.stream_ptr(coords.device)), "arg_sort_coordinates")
    return index if out_dtype == torch.int64 else index.to(out_dtype)


def build_sorted_index(coordinates: torch.Tensor,
                       batch_dims: Optional[torch.Tensor] = None,
                       enable_flattening: bool = True):
    """int64 permutation that sorts the coordinates
    (minuet/nn/functional/indexing.py:59-79)."""
    return arg_sort_coordinates(coordinates, batch_dims=batch_dims, dtype=torch.int64,
                                enable_flattening=enable_flattening)


def query_sorted_index_with_offsets(sources: torch.Tensor,
                                    targets: torch.Tensor,
                                    offsets: torch.Tensor,
                                    source_batch_dims: Optional[torch.Tensor] = None,
                                    target_batch_dims: Optional[torch.Tensor] = None):
    """Kernel map ``[N_weight, N_out]``: entry ``[k, j]`` is the index ``i`` with
    ``sources[i] == targets[j] + offsets[k]`` inside the same cloud, else -1
    (minuet/nn/functional/indexing.py:82-127).  Both coordinate tensors must be
    sorted.  The result has the reference's dtype: the coordinate dtype for one
    cloud, the batch_dims dtype for a batch.
    """
    if (source_batch_dims is None) != (target_batch_dims is None):
        raise ValueError("source_batch_dims and target_batch_dims must be both "
                         "provided or neither provided")
    engine.require_cuda(sources, targets, offsets, source_batch_dims, target_batch_dims)
    for name, t in (("sources", sources), ("targets", targets), ("offsets", offsets)):
        if t.ndim != 2:
            raise RuntimeError(f"Tensor {name} must be 2-D but found {t.ndim}-D")
    ndim = offsets.shape[1]
    if sources.shape[1] != ndim or targets.shape[1] != ndim:
        raise RuntimeError("sources, targets and offsets must agree on the number of dimensions")
    if not (sources.dtype == targets.dtype == offsets.dtype):
        raise RuntimeError("sources, targets and offsets must share one dtype")
    if source_batch_dims is not None:
        if source_batch_dims.numel() <= 1:
            raise RuntimeError("Tensor source_batch_dims should be at least length 2")
        if target_batch_dims.numel() != source_batch_dims.numel():
            raise RuntimeError("Tensor target_batch_dims must have the same length as "
                               "source_batch_dims")
    out_dtype = sources.dtype if source_batch_dims is None else source_batch_dims.dtype
    src, tgt = engine.as_i32_coords(sources), engine.as_i32_coords(targets)
    off = np.ascontiguousarray(offsets.detach().cpu().numpy().astype(np.int32))
    sbd, tbd = engine.as_i64(source_batch_dims), engine.as_i64(target_batch_dims)
    nb = 1 if sbd is None else sbd.numel() - 1
    S, T, O = src.shape[0], tgt.shape[0], off.shape[0]
    kernel_map = torch.empty((O, T), dtype=torch.int32, device=src.device)
    if T > 0 and O > 0:
        margin = int(np.abs(off).max()) if off.size else 0
        spec = engine.make_keyspec([src, tgt], ndim, nb, margin)
        skeys = engine.pack_keys(src, sbd, spec)
        tkeys = skeys if (tgt.data_ptr() == src.data_ptr() and S == T) else \
            engine.pack_keys(tgt, tbd, spec)
        _lib.check(engine.lib().mn_query_sorted_index_with_offsets(
            engine.ptr(skeys), S, engine.ptr(tkeys), T, engine.np_ptr(off), O,
            ctypes.byref(spec), engine.ptr(kernel_map), engine.stream_ptr(src.device)),
            "query_sorted_index_with_offsets")
    return kernel_map if out_dtype == torch.int32 else kernel_map.to(out_dtype)
