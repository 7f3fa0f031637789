"""Gather - grouped GEMM - Scatter forward pass and its stage timers
(mirror of minuet/nn/functional/convolution.py)."""
__all__ = ['cuda_time_gather', 'cuda_time_scatter', 'sparse_convolution_forward',
           'cuda_time_gemm', 'set_gemm_parallel_level']

from typing import Optional

import numpy as np
import torch

from minuet_b200 import _lib, engine

GEMM_PARALLEL_LEVEL = 4


def set_gemm_parallel_level(level: int):
    """Kept for API compatibility (minuet/nn/functional/convolution.py:15-25).
    The reference spreads one cuBLAS call per padding bucket over ``level``
    streams; here every offset is a problem of one grouped launch, so the value
    is stored and otherwise unused."""
    global GEMM_PARALLEL_LEVEL
    GEMM_PARALLEL_LEVEL = level


def _i32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if t is None:
        return None
    return t.contiguous() if t.dtype == torch.int32 else t.to(torch.int32).contiguous()


def _prepare(weights, source_masks, target_masks, kernel_map_sizes, sources=None):
    if source_masks.ndim != 2 or target_masks.ndim != 2:
        raise RuntimeError("source_masks and target_masks must be 2-D tensors")
    if weights.ndim != 3:
        raise RuntimeError(f"weights must be a 3-D tensor but found {weights.ndim}-D")
    O, T = target_masks.shape
    S = source_masks.shape[1]
    if source_masks.shape[0] != O or weights.shape[0] != O or kernel_map_sizes.shape[0] != O:
        raise RuntimeError("source_masks, weights and kernel_map_sizes must have one row per "
                           f"offset ({O})")
    c_in, c_out = weights.shape[1], weights.shape[2]
    if sources is not None:
        if sources.ndim != 2 or sources.shape[1] != c_in:
            raise RuntimeError(f"sources must be [N, {c_in}] but found {tuple(sources.shape)}")
        if sources.dtype != weights.dtype:
            raise RuntimeError(f"sources ({sources.dtype}) and weights ({weights.dtype}) must "
                               "share one dtype")
    sizes_host = engine.host_copy(kernel_map_sizes, np.int32)
    return S, T, O, c_in, c_out, sizes_host


def _workspace(sizes_host, S, T, O, c_in, c_out, code, allow_shortcut, threshold, device):
    nbytes = engine.lib().mn_conv_workspace_bytes(
        engine.np_ptr(sizes_host), O, S, T, c_in, c_out, code, int(bool(allow_shortcut)),
        0 if threshold is None else 1, 0.0 if threshold is None else float(threshold))
    return engine.workspace(nbytes, device)


def sparse_convolution_forward(sources: torch.Tensor,
                               weights: torch.Tensor,
                               source_masks: torch.Tensor,
                               target_masks: torch.Tensor,
                               kernel_map_order: Optional[torch.Tensor],
                               kernel_map_sizes: torch.Tensor,
                               gather_tile_size: int,
                               scatter_tile_size: int,
                               allow_shortcut_matmul: bool = False,
                               parallel: Optional[int] = None,
                               threshold: Optional[float] = 0) -> torch.Tensor:
    """``out[t] = sum_k sum_{(s, t) in map[k]} sources[s] @ weights[order[k]]``
    (minuet/nn/functional/convolution.py:110-155).

    Arguments and result follow the reference; fp32, fp16 and bf16 features are
    supported (accumulation is always fp32).  ``parallel`` and ``threshold`` are
    accepted and do not change the result: the grouped GEMM needs neither side
    streams nor equal-size buckets.  ``*_tile_size`` is the number of channels
    one thread moves per row; 1 (the untuned default) picks 16-byte accesses.
    """
    del parallel
    engine.require_cuda(sources)
    sources = sources.contiguous()
    weights = weights.contiguous()
    sm, tm, order = _i32(source_masks), _i32(target_masks), _i32(kernel_map_order)
    S, T, O, c_in, c_out, sizes_host = _prepare(weights, sm, tm, kernel_map_sizes, sources)
    if sources.shape[0] != S:
        raise RuntimeError(f"sources has {sources.shape[0]} rows but the masks describe {S}")
    code = engine.dtype_code(weights.dtype)
    device = sources.device
    out = torch.empty((T, c_out), dtype=weights.dtype, device=device)
    ws = _workspace(sizes_host, S, T, O, c_in, c_out, code, allow_shortcut_matmul, threshold, device)
    _lib.check(engine.lib().mn_sparse_convolution_forward(
        S, T, O, c_in, c_out, code, engine.ptr(sources), engine.ptr(weights), engine.ptr(sm),
        engine.ptr(tm), engine.ptr(order), engine.np_ptr(sizes_host), int(gather_tile_size),
        int(scatter_tile_size), int(bool(allow_shortcut_matmul)), 0 if threshold is None else 1,
        0.0 if threshold is None else float(threshold), engine.ptr(out),
        engine.ptr(engine.status_word(device)), engine.ptr(ws), ws.numel(),
        engine.stream_ptr(device)), "sparse_convolution_forward")
    return out


def _time_stage(stage, weights, source_masks, target_masks, kernel_map_sizes, tile_size,
                allow_shortcut_matmul, threshold) -> float:
    engine.require_cuda(weights, source_masks, target_masks)
    weights = weights.detach().contiguous()
    sm, tm = _i32(source_masks), _i32(target_masks)
    S, T, O, c_in, c_out, sizes_host = _prepare(weights, sm, tm, kernel_map_sizes)
    code = engine.dtype_code(weights.dtype)
    device = weights.device
    # like the reference's timers (sparse_convolution.cu:294-502) the stage runs
    # on buffers whose contents do not matter
    sources = torch.empty((S, c_in), dtype=weights.dtype, device=device)
    out = torch.empty((T, c_out), dtype=weights.dtype, device=device)
    ws = _workspace(sizes_host, S, T, O, c_in, c_out, code, allow_shortcut_matmul, threshold, device)
    stream = torch.cuda.current_stream(device)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record(stream)
    _lib.check(engine.lib().mn_conv_stage(
        stage, S, T, O, c_in, c_out, code, engine.ptr(sources), engine.ptr(weights),
        engine.ptr(sm), engine.ptr(tm), None, engine.np_ptr(sizes_host), int(tile_size),
        int(bool(allow_shortcut_matmul)), 0 if threshold is None else 1,
        0.0 if threshold is None else float(threshold), engine.ptr(out),
        engine.ptr(engine.status_word(device)), engine.ptr(ws), ws.numel(),
        engine.stream_ptr(device)), "conv_stage")
    end.record(stream)
    end.synchronize()
    return begin.elapsed_time(end)


def cuda_time_gather(weights, source_masks, target_masks, kernel_map_sizes, tile_size: int,
                     allow_shortcut_matmul: bool = False, threshold: float = 0) -> float:
    """Milliseconds of one gather (minuet/nn/functional/convolution.py:28-52)."""
    return _time_stage(0, weights, source_masks, target_masks, kernel_map_sizes, tile_size,
                       allow_shortcut_matmul, threshold)


def cuda_time_scatter(weights, source_masks, target_masks, kernel_map_sizes, tile_size: int,
                      allow_shortcut_matmul: bool = False, threshold: float = 0) -> float:
    """Milliseconds of one scatter (minuet/nn/functional/convolution.py:55-79)."""
    return _time_stage(2, weights, source_masks, target_masks, kernel_map_sizes, tile_size,
                       allow_shortcut_matmul, threshold)


def cuda_time_gemm(weights, source_masks, target_masks, kernel_map_sizes,
                   allow_shortcut_matmul: bool = False, parallel: Optional[int] = None,
                   threshold: float = 0) -> float:
    """Milliseconds of the grouped GEMM (minuet/nn/functional/convolution.py:82-107)."""
    del parallel
    return _time_stage(1, weights, source_masks, target_masks, kernel_map_sizes, 1,
                       allow_shortcut_matmul, threshold)
