"""Kernel-map sizes and masks (mirror of minuet/nn/functional/scan.py)."""
__all__ = ['compute_kernel_map_masks', 'compute_kernel_map_sizes']

import torch

from minuet_b200 import _lib, engine


def _as_i32_map(kernel_map: torch.Tensor) -> torch.Tensor:
    if kernel_map.ndim != 2:
        raise RuntimeError(f"kernel_map must be a 2-D tensor but found {kernel_map.ndim}-D")
    return kernel_map.to(torch.int32).contiguous()


def compute_kernel_map_sizes(kernel_map: torch.Tensor):
    """``sizes[k]`` = number of entries of kernel-map row ``k`` that are not -1
    (minuet/nn/functional/scan.py:8-24); same dtype as the kernel map."""
    engine.require_cuda(kernel_map)
    km = _as_i32_map(kernel_map)
    O, T = km.shape
    sizes = torch.empty(O, dtype=torch.int32, device=km.device)
    _lib.check(engine.lib().mn_compute_kernel_map_sizes(engine.ptr(km), O, T, engine.ptr(sizes),
                                                        engine.stream_ptr(km.device)),
               "compute_kernel_map_sizes")
    return sizes if kernel_map.dtype == torch.int32 else sizes.to(kernel_map.dtype)


def compute_kernel_map_masks(num_sources: int, kernel_map: torch.Tensor,
                             kernel_map_sizes: torch.Tensor):
    """Source and target masks of a kernel map whose rows are already in the
    order the convolution will use (minuet/nn/functional/scan.py:27-48): the
    valid entries of row ``k`` are ranked by target index and the rank is stored
    at ``source_masks[k, source]`` and ``target_masks[k, target]``; every other
    entry is -1.  ``kernel_map_sizes`` is accepted for signature parity (the
    ranks are recomputed from the map)."""
    del kernel_map_sizes
    engine.require_cuda(kernel_map)
    km = _as_i32_map(kernel_map)
    O, T = km.shape
    device = km.device
    source_masks = torch.empty((O, int(num_sources)), dtype=torch.int32, device=device)
    target_masks = torch.empty((O, T), dtype=torch.int32, device=device)
    lib = engine.lib()
    ws = engine.workspace(lib.mn_map_workspace_bytes(int(num_sources), T, max(O, 1)), device)
    _lib.check(lib.mn_compute_kernel_map_masks(engine.ptr(km), O, int(num_sources), T,
                                               engine.ptr(source_masks), engine.ptr(target_masks),
                                               engine.ptr(ws), ws.numel(),
                                               engine.stream_ptr(device)),
               "compute_kernel_map_masks")
    if kernel_map.dtype != torch.int32:
        return source_masks.to(kernel_map.dtype), target_masks.to(kernel_map.dtype)
    return source_masks, target_masks
