"""Gather - grouped GEMM - Scatter forward pass and its stage timers
(mirror of minuet/nn/functional/convolution.py)."""
__all__ = ['cuda_time_gather', 'cuda_time_scatter', 'sparse_convolution_forward',
           'sparse_convolution_forward_fused', 'apply_epilogue', 'cuda_time_gemm',
           'set_gemm_parallel_level', 'dense_forward', 'time_forward', 'estimate_ms',
           'transpose_weights']

import math
from typing import Optional

import numpy as np
import torch

from minuet_b200 import _lib, engine

GEMM_PARALLEL_LEVEL = 4
# Which forward algorithm fp16/bf16 layers use when the call does not say:
# "explicit" = pair lists (or gather - grouped GEMM - scatter where pair lists do not
# apply), "implicit" = the fused output-stationary kernel, "auto" = a cost estimate
# from the map's pair and tile counts (no timing ever runs inside a forward pass; the
# layer autotuner times both and passes its choice with every call)
ALGORITHM = "auto"
# 128-row sub-tiles per CTA tile of the fused kernel when the call does not say
# (0 = chosen by the library)
IMPLICIT_SUB_TILES = 0
# The fused kernel walks the targets sorted by hit word (rows with the same set of
# offsets share tiles, and tiles skip the offsets they do not have); False keeps the
# targets' own order
REORDER_ROWS = True


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
                               threshold: Optional[float] = 0,
                               algorithm: Optional[str] = None,
                               sub_tiles: Optional[int] = None,
                               weights_t: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = sum_k sum_{(s, t) in map[k]} sources[s] @ weights[order[k]]``
    (minuet/nn/functional/convolution.py:110-155).

    Arguments and result follow the reference; fp32, fp16 and bf16 features are
    supported (accumulation is always fp32).  ``parallel`` and ``threshold`` are
    accepted and do not change the result: the grouped GEMM needs neither side
    streams nor equal-size buckets.  ``*_tile_size`` is the number of channels
    one thread moves per row; 1 (the untuned default) picks 16-byte accesses.
    fp16/bf16 layers run either the pair-list forward or the fused implicit-GEMM
    kernel: ``algorithm`` ("explicit" / "implicit"; default: the module-level
    ``ALGORITHM``) and ``sub_tiles`` (row sub-tiles per tile of the fused kernel,
    0 = automatic) are this library's additions to the reference signature and are
    what the layer autotuner tunes; ``weights_t`` is :func:`transpose_weights` of
    ``weights`` for callers whose weights do not change between calls (without it the
    16-bit paths transpose the weights on every call).
    """
    del parallel
    engine.require_cuda(sources)
    if torch.is_grad_enabled() and (sources.requires_grad or weights.requires_grad):
        return _SparseConvolution.apply(sources, weights, source_masks, target_masks,
                                        kernel_map_order, kernel_map_sizes, gather_tile_size,
                                        scatter_tile_size, allow_shortcut_matmul, threshold,
                                        algorithm, sub_tiles)
    sources = sources.contiguous()
    weights = weights.contiguous()
    sm, tm, order = _i32(source_masks), _i32(target_masks), _i32(kernel_map_order)
    S, T, O, c_in, c_out, sizes_host = _prepare(weights, sm, tm, kernel_map_sizes, sources)
    if sources.shape[0] != S:
        raise RuntimeError(f"sources has {sources.shape[0]} rows but the masks describe {S}")
    return _forward(sources, weights, sm, tm, order, sizes_host, gather_tile_size,
                    scatter_tile_size, allow_shortcut_matmul, threshold, algorithm=algorithm,
                    sub_tiles=sub_tiles, weights_t=weights_t)


class _SparseConvolution(torch.autograd.Function):
    """Differentiable sparse convolution (the reference has no backward pass).

    With pairs ``(s, t)`` under offset ``k``: ``out[t] += x[s] W[k]``, hence
    ``dx[s] += dout[t] W[k]^T`` -- the same convolution with the two masks swapped and
    every weight matrix transposed, run by the same kernels -- and
    ``dW[k] = sum over the pairs of x[s]^T dout[t]``, computed per offset from the pair
    rows in rank order (index selection and one fp32 product per offset; written for
    correctness, not tuned)."""

    @staticmethod
    def forward(ctx, sources, weights, source_masks, target_masks, order, sizes, gather_tile,
                scatter_tile, shortcut, threshold, algorithm, sub_tiles):
        x = sources.detach().contiguous()
        w = weights.detach().contiguous()
        sm, tm, od = _i32(source_masks), _i32(target_masks), _i32(order)
        S, T, O, c_in, c_out, sizes_host = _prepare(w, sm, tm, sizes, x)
        if x.shape[0] != S:
            raise RuntimeError(f"sources has {x.shape[0]} rows but the masks describe {S}")
        ctx.save_for_backward(x, w, sm, tm, od if od is not None else torch.empty(0), sizes)
        ctx.has_order = od is not None
        ctx.args = (gather_tile, scatter_tile, shortcut, threshold, algorithm, sub_tiles)
        return _forward(x, w, sm, tm, od, sizes_host, gather_tile, scatter_tile, shortcut,
                        threshold, algorithm=algorithm, sub_tiles=sub_tiles)

    @staticmethod
    def backward(ctx, grad_out):
        x, w, sm, tm, od, sizes = ctx.saved_tensors
        od = od if ctx.has_order else None
        gather_tile, scatter_tile, shortcut, threshold, algorithm, sub_tiles = ctx.args
        grad_out = grad_out.contiguous()
        O = sm.shape[0]
        sizes_host = engine.host_copy(sizes, np.int32)
        grad_x = grad_w = None
        if ctx.needs_input_grad[0]:
            grad_x = _forward(grad_out, w.transpose(1, 2).contiguous(), tm, sm, od, sizes_host,
                              scatter_tile, gather_tile, shortcut, threshold, algorithm=algorithm,
                              sub_tiles=sub_tiles)
        if ctx.needs_input_grad[1]:
            grad_w = torch.zeros_like(w, dtype=torch.float32)
            for p in range(O):
                n = int(sizes_host[p])
                if n == 0:
                    continue
                k = p if od is None else int(od[p])
                s_rows = torch.nonzero(sm[p] >= 0).squeeze(1)
                t_rows = torch.nonzero(tm[p] >= 0).squeeze(1)
                # pair r of this mask row is (source with rank r, target with rank r)
                s_by_rank = torch.empty(n, dtype=torch.int64, device=x.device)
                t_by_rank = torch.empty(n, dtype=torch.int64, device=x.device)
                s_by_rank[sm[p, s_rows].long()] = s_rows
                t_by_rank[tm[p, t_rows].long()] = t_rows
                grad_w[k] = x[s_by_rank].float().t() @ grad_out[t_by_rank].float()
            grad_w = grad_w.to(w.dtype)
        return (grad_x, grad_w) + (None,) * 10


def sparse_convolution_forward_fused(sources: torch.Tensor, weights: torch.Tensor,
                                     source_masks: torch.Tensor, target_masks: torch.Tensor,
                                     kernel_map_order: Optional[torch.Tensor],
                                     kernel_map_sizes: torch.Tensor,
                                     gather_tile_size: int = 1,
                                     scatter_tile_size: int = 1,
                                     allow_shortcut_matmul: bool = False,
                                     threshold: Optional[float] = 0,
                                     scale: Optional[torch.Tensor] = None,
                                     shift: Optional[torch.Tensor] = None,
                                     residual: Optional[torch.Tensor] = None,
                                     relu: bool = False,
                                     algorithm: Optional[str] = None,
                                     sub_tiles: Optional[int] = None,
                                     weights_t: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sparse convolution with a fused epilogue (no counterpart in the reference,
    whose models apply BatchNorm, the residual add and ReLU as separate passes
    over the feature matrix):

        out = relu?( conv(sources) * scale[c] + shift[c] + residual )

    ``scale`` / ``shift`` are ``[C_out]`` (an eval-mode BatchNorm or a bias folded
    into two vectors; applied in fp32), ``residual`` is ``[N_out, C_out]`` in the
    feature dtype.  Layers that take the fused implicit-GEMM kernel apply the
    epilogue inside it; the others run gather - GEMM - scatter and one in-place
    pass over the output."""
    engine.require_cuda(sources)
    sources = sources.contiguous()
    weights = weights.contiguous()
    sm, tm, order = _i32(source_masks), _i32(target_masks), _i32(kernel_map_order)
    S, T, O, c_in, c_out, sizes_host = _prepare(weights, sm, tm, kernel_map_sizes, sources)
    if sources.shape[0] != S:
        raise RuntimeError(f"sources has {sources.shape[0]} rows but the masks describe {S}")
    res = None if residual is None else residual.contiguous()
    if res is not None and (tuple(res.shape) != (T, c_out) or res.dtype != weights.dtype):
        raise RuntimeError("residual must be [N_out, C_out] in the feature dtype")
    return _forward(sources, weights, sm, tm, order, sizes_host, gather_tile_size,
                    scatter_tile_size, allow_shortcut_matmul, threshold, _f32(scale), _f32(shift),
                    res, relu, algorithm=algorithm, sub_tiles=sub_tiles, weights_t=weights_t)


def apply_epilogue(features: torch.Tensor, scale=None, shift=None, residual=None,
                   relu: bool = False) -> torch.Tensor:
    """In place ``features = relu?(features * scale[c] + shift[c] + residual)``."""
    engine.require_cuda(features)
    rows, channels = features.shape
    _lib.check(engine.lib().mn_apply_epilogue(
        engine.ptr(features), rows, channels, engine.dtype_code(features.dtype),
        engine.ptr(_f32(scale)), engine.ptr(_f32(shift)),
        engine.ptr(None if residual is None else residual.contiguous()), int(bool(relu)),
        engine.stream_ptr(features.device)), "apply_epilogue")
    return features


def _f32(v):
    return None if v is None else v.detach().to(torch.float32).contiguous()


def _explicit_forward(sources, weights, sm, tm, order, sizes_host, out, gather_tile_size,
                      scatter_tile_size, allow_shortcut_matmul, threshold):
    O, S = sm.shape
    T = tm.shape[1]
    c_in, c_out = weights.shape[1], weights.shape[2]
    code = engine.dtype_code(weights.dtype)
    device = sources.device
    ws = _workspace(sizes_host, S, T, O, c_in, c_out, code, allow_shortcut_matmul, threshold, device)
    _lib.check(engine.lib().mn_sparse_convolution_forward(
        S, T, O, c_in, c_out, code, engine.ptr(sources), engine.ptr(weights), engine.ptr(sm),
        engine.ptr(tm), engine.ptr(order), engine.np_ptr(sizes_host), int(gather_tile_size),
        int(scatter_tile_size), int(bool(allow_shortcut_matmul)), 0 if threshold is None else 1,
        0.0 if threshold is None else float(threshold), engine.ptr(out),
        engine.ptr(engine.status_word(device)), engine.ptr(ws), ws.numel(),
        engine.stream_ptr(device)), "sparse_convolution_forward")
    return out


def _pairs_forward(sources, weights, sm, tm, order, sizes_host, out, allow_shortcut_matmul,
                   scale=None, shift=None, residual=None, relu=False, weights_t=None) -> bool:
    """Pair-list forward (16-bit, kernel maps that carry hit words).  Returns False,
    without touching ``out``, when this layer cannot take it."""
    O, S = sm.shape
    T = tm.shape[1]
    c_in, c_out = weights.shape[1], weights.shape[2]
    lib = engine.lib()
    code = engine.dtype_code(weights.dtype)
    if not lib.mn_pairs_supported(O, c_in, c_out, code):
        return False
    pair_src = engine.pair_list(sm, tm, sizes_host, allow_shortcut_matmul)
    if pair_src is None:
        return False
    device = sources.device
    shortcut = int(bool(allow_shortcut_matmul))
    ws = engine.workspace(lib.mn_pairs_workspace_bytes(engine.np_ptr(sizes_host), O, S, T, c_in,
                                                       c_out, shortcut), device)
    _lib.check(lib.mn_sparse_convolution_forward_pairs(
        S, T, O, c_in, c_out, code, engine.ptr(sources), engine.ptr(weights),
        engine.ptr(weights_t), engine.ptr(tm),
        engine.ptr(engine.hit_bits(tm)), engine.ptr(pair_src), engine.ptr(order),
        engine.np_ptr(sizes_host), shortcut, engine.ptr(scale), engine.ptr(shift),
        engine.ptr(residual), int(bool(relu)), engine.ptr(out),
        engine.ptr(engine.status_word(device)), engine.ptr(ws), ws.numel(),
        engine.stream_ptr(device)), "sparse_convolution_forward_pairs")
    return True


def transpose_weights(weights: torch.Tensor) -> Optional[torch.Tensor]:
    """``weights [O, c_in, c_out]`` (or ``[c_in, c_out]``) as ``[O, c_out, c_in]``, the
    layout the tensor-core kernels read; None for dtypes those kernels do not take."""
    if weights.dtype not in (torch.float16, torch.bfloat16) or not weights.is_cuda:
        return None
    w = weights.detach().contiguous()
    if w.ndim == 2:
        w = w.unsqueeze(0)
    O, c_in, c_out = w.shape
    out = torch.empty((O, c_out, c_in), dtype=w.dtype, device=w.device)
    _lib.check(engine.lib().mn_transpose_weights(
        engine.ptr(w), O, c_in, c_out, engine.dtype_code(w.dtype), engine.ptr(out),
        engine.stream_ptr(w.device)), "transpose_weights")
    return out


def dense_forward(features, weight, scale=None, shift=None, residual=None, relu=False,
                  weights_t=None):
    """``relu?((features @ weight) * scale + shift + residual)`` for a 1x1x1
    convolution: the tensor-core GEMM of this library for fp16/bf16 (c_in a multiple
    of 8, c_out even, at most 256), its FFMA GEMM plus the epilogue pass otherwise
    (fp32 must not go through TF32: its 10-bit mantissa would break the 1e-5 bound)."""
    engine.require_cuda(features)
    features = features.contiguous()
    weight = weight.contiguous()
    rows, c_in = features.shape
    c_out = weight.shape[1]
    lib = engine.lib()
    if features.dtype in (torch.float16, torch.bfloat16) and features.dtype == weight.dtype and \
            lib.mn_dense_supported(c_in, c_out, engine.dtype_code(features.dtype)):
        device = features.device
        entry = None
        if engine.LAYER_LOG is not None:
            entry = {"S": rows, "T": rows, "O": 1, "E": rows, "c_in": c_in, "c_out": c_out,
                     "algorithm": "dense", "events": engine.event_pair_begin(device)}
            engine.LAYER_LOG.append(entry)
        out = torch.empty((rows, c_out), dtype=features.dtype, device=device)
        ws = engine.workspace(lib.mn_dense_workspace_bytes(c_in, c_out), device)
        res = None if residual is None else residual.contiguous()
        _lib.check(lib.mn_dense_forward(
            rows, c_in, c_out, engine.dtype_code(features.dtype), engine.ptr(features),
            engine.ptr(weight), engine.ptr(weights_t), engine.ptr(_f32(scale)),
            engine.ptr(_f32(shift)), engine.ptr(res),
            int(bool(relu)), engine.ptr(out), engine.ptr(engine.status_word(device)),
            engine.ptr(ws), ws.numel(), engine.stream_ptr(device)), "dense_forward")
        if entry is not None:
            engine.event_pair_end(entry["events"], device)
        return out
    if features.dtype != weight.dtype or features.dtype not in (torch.float32, torch.float16,
                                                                  torch.bfloat16):
        raise RuntimeError(f"features ({features.dtype}) and weight ({weight.dtype}) must share "
                           "one of float32, float16, bfloat16")
    # fp32 and the shapes the tensor-core kernel does not take: the FFMA grouped-GEMM kernel
    device = features.device
    entry = None
    if engine.LAYER_LOG is not None:
        entry = {"S": rows, "T": rows, "O": 1, "E": rows, "c_in": c_in, "c_out": c_out,
                 "algorithm": "dense-ffma", "events": engine.event_pair_begin(device)}
        engine.LAYER_LOG.append(entry)
    out = torch.empty((rows, c_out), dtype=features.dtype, device=device)
    res = None if residual is None else residual.contiguous()
    _lib.check(lib.mn_dense_forward_simt(
        rows, c_in, c_out, engine.dtype_code(features.dtype), engine.ptr(features),
        engine.ptr(weight), engine.ptr(_f32(scale)), engine.ptr(_f32(shift)), engine.ptr(res),
        int(bool(relu)), engine.ptr(out), engine.stream_ptr(device)), "dense_forward_simt")
    if entry is not None:
        engine.event_pair_end(entry["events"], device)
    return out


def _implicit_forward(sources, weights, source_masks, target_masks, order, sizes_host, out,
                      scale=None, shift=None, residual=None, relu=False, sub_tiles=None,
                      weights_t=None):
    O, S = source_masks.shape
    T = target_masks.shape[1]
    c_in, c_out = weights.shape[1], weights.shape[2]
    device = sources.device
    nbr, tile_bits, perm = engine.neighbor_table(source_masks, target_masks, sizes_host,
                                                 reorder=REORDER_ROWS)
    if engine.LAYER_LOG:      # benchmarks read the per-tile offset bits of the logged layer
        engine.LAYER_LOG[-1]["tile_bits"] = tile_bits
    lib = engine.lib()
    ws = engine.workspace(lib.mn_implicit_workspace_bytes(O, c_in, c_out), device)
    _lib.check(lib.mn_sparse_convolution_forward_implicit(
        S, T, O, c_in, c_out, engine.dtype_code(weights.dtype), engine.ptr(sources),
        engine.ptr(weights), engine.ptr(weights_t), engine.ptr(nbr), engine.ptr(tile_bits),
        engine.ptr(perm), engine.ptr(order),
        engine.ptr(scale), engine.ptr(shift), engine.ptr(residual), int(bool(relu)),
        float(sizes_host.sum()) / max(T, 1),
        int(IMPLICIT_SUB_TILES if sub_tiles is None else sub_tiles),
        engine.ptr(out), engine.ptr(engine.status_word(device)), engine.ptr(ws), ws.numel(),
        engine.stream_ptr(device)), "sparse_convolution_forward_implicit")
    return out


def estimate_ms(algorithm: str, S, T, O, c_in, c_out, pairs, shortcut: bool) -> float:
    """Rough cost of one 16-bit forward pass, from fits to measured layers of the
    benchmark network on a B200.  Pair lists move every non-centre pair row three
    times (16-bit read, fp32 product written and read back) at about 2.7 TB/s.  The
    fused kernel pays about 3.3 ns per (128-row tile, offset present in the tile,
    64-channel block) plus 10 ns per tile; with the rows sorted by hit word a tile of a
    map with E/T pairs per row holds about 1 + 2.2 (E/T - 1) of the O offsets.  Only
    the ORDER of the two estimates matters."""
    if algorithm == "implicit":
        tiles = math.ceil(T / 128)
        present = min(float(O), 1.0 + 2.2 * max(pairs / max(T, 1) - 1.0, 0.0)) if REORDER_ROWS else O
        return 0.03 + 1.0e-5 * tiles + 3.3e-6 * tiles * present * math.ceil(c_in / 64) * \
            (0.7 + 0.3 * c_out / 128)
    rest = pairs - (min(S, T) if shortcut else 0)
    return 0.05 + (rest * (8.0 * c_out + 2.0 * c_in) + 2.0 * (S * c_in + T * c_out)) / 2.7e9


def _pick_algorithm(weights, sm, tm, sizes_host, allow_shortcut_matmul, algorithm) -> str:
    """'explicit' or 'implicit' for this call: the caller's choice when it is
    supported, else the module-level ``ALGORITHM``, else the cheaper estimate."""
    O, T = tm.shape
    S = sm.shape[1]
    c_in, c_out = weights.shape[1], weights.shape[2]
    if algorithm in (None, "auto"):
        algorithm = ALGORITHM
    if algorithm not in ("auto", "explicit", "implicit"):
        raise ValueError(f"unknown sparse convolution algorithm {algorithm!r}")
    code = engine.dtype_code(weights.dtype)
    if algorithm == "explicit" or T == 0 or not engine.lib().mn_implicit_supported(
            O, c_in, c_out, code):
        return "explicit"
    if algorithm == "implicit":
        return "implicit"
    if not engine.lib().mn_pairs_supported(O, c_in, c_out, code) or engine.hit_bits(tm) is None:
        return "implicit"      # the explicit path would gather and scatter through HBM
    pairs = float(sizes_host.sum())
    shortcut = bool(allow_shortcut_matmul) and O > 0 and int(sizes_host[-1]) == S == T
    if estimate_ms("implicit", S, T, O, c_in, c_out, pairs, shortcut) < \
            estimate_ms("explicit", S, T, O, c_in, c_out, pairs, shortcut):
        return "implicit"
    return "explicit"


def _forward(sources, weights, sm, tm, order, sizes_host, gather_tile_size, scatter_tile_size,
             allow_shortcut_matmul, threshold, scale=None, shift=None, residual=None, relu=False,
             algorithm=None, sub_tiles=None, weights_t=None):
    T = tm.shape[1]
    c_out = weights.shape[2]
    if weights.dtype != torch.float32 and weights.shape[1] % 8 != 0 and c_out % 8 == 0:
        # few input channels (a network's first layer): zero channels up to a multiple of 8
        # put the layer on the tensor-core paths instead of gather - FFMA GEMM - scatter
        pad = -weights.shape[1] % 8
        sources = torch.nn.functional.pad(sources, (0, pad))
        weights = torch.nn.functional.pad(weights, (0, 0, 0, pad))
        weights_t = None
    out = torch.empty((T, c_out), dtype=weights.dtype, device=sources.device)
    has_epilogue = scale is not None or shift is not None or residual is not None or relu

    def run_explicit():
        # sparse maps with hit words: pair lists, fp32 products, one rounding
        if weights.dtype != torch.float32 and _pairs_forward(
                sources, weights, sm, tm, order, sizes_host, out, allow_shortcut_matmul, scale,
                shift, residual, relu, weights_t):
            return out
        _explicit_forward(sources, weights, sm, tm, order, sizes_host, out, gather_tile_size,
                          scatter_tile_size, allow_shortcut_matmul, threshold)
        if has_epilogue:
            _lib.check(engine.lib().mn_apply_epilogue(
                engine.ptr(out), T, c_out, engine.dtype_code(weights.dtype), engine.ptr(scale),
                engine.ptr(shift), engine.ptr(residual), int(bool(relu)),
                engine.stream_ptr(out.device)), "apply_epilogue")
        return out

    def run_implicit():
        return _implicit_forward(sources, weights, sm, tm, order, sizes_host, out, scale, shift,
                                 residual, relu, sub_tiles, weights_t)

    choice = _pick_algorithm(weights, sm, tm, sizes_host, allow_shortcut_matmul, algorithm)
    log = engine.LAYER_LOG
    if log is not None:
        entry = {"S": sm.shape[1], "T": T, "O": sm.shape[0], "E": int(sizes_host.sum()),
                 "c_in": weights.shape[1], "c_out": c_out, "algorithm": choice,
                 "events": engine.event_pair_begin(sources.device)}
        log.append(entry)
    result = run_implicit() if choice == "implicit" else run_explicit()
    if log is not None:
        engine.event_pair_end(entry["events"], sources.device)
    return result


def time_forward(weights, source_masks, target_masks, kernel_map_order, kernel_map_sizes,
                 allow_shortcut_matmul: bool = False, algorithm: str = "explicit",
                 sub_tiles: int = 0, gather_tile_size: int = 1, scatter_tile_size: int = 1,
                 threshold: Optional[float] = -1, epilogue=(False, False, False, False)) -> float:
    """Milliseconds of one whole forward pass with the given algorithm on buffers whose
    contents do not matter (what the layer autotuner compares).  ``epilogue`` =
    (scale, shift, residual, relu) flags of the fused epilogue the layer runs with."""
    engine.require_cuda(weights, source_masks, target_masks)
    weights = weights.detach().contiguous()
    sm, tm, order = _i32(source_masks), _i32(target_masks), _i32(kernel_map_order)
    S, T, O, c_in, c_out, sizes_host = _prepare(weights, sm, tm, kernel_map_sizes)
    device = weights.device
    sources = torch.zeros((S, c_in), dtype=weights.dtype, device=device)
    scale = torch.ones(c_out, dtype=torch.float32, device=device) if epilogue[0] else None
    shift = torch.zeros(c_out, dtype=torch.float32, device=device) if epilogue[1] else None
    residual = torch.zeros((T, c_out), dtype=weights.dtype, device=device) if epilogue[2] else None
    stream = torch.cuda.current_stream(device)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record(stream)
    _forward(sources, weights, sm, tm, order, sizes_host, gather_tile_size, scatter_tile_size,
             allow_shortcut_matmul, threshold, scale, shift, residual, bool(epilogue[3]),
             algorithm=algorithm, sub_tiles=sub_tiles)
    end.record(stream)
    end.synchronize()
    return begin.elapsed_time(end)


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
