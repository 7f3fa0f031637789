"""``KernelMapCache`` and ``SparseConv`` / ``SparseConv3d``
(API of minuet/nn/convolutions.py)."""
__all__ = ['SparseConv', 'SparseConv3d', 'KernelMapCache', 'fold_batchnorm']

import contextlib
import ctypes
import math
from typing import Any, Dict, Optional, Union

import numpy as np
import torch
from torch.nn import Module

from minuet_b200 import _lib, engine
from minuet_b200.nn import functional as F
from minuet_b200.tensors import SparseTensor
from minuet_b200.utils.helpers import as_tuple, generate_kernel_offsets


class KernelMapCache(object):
    """Builds each kernel map of a forward pass once and shares it between layers.

    Same constructor, methods and return values as the reference class
    (minuet/nn/convolutions.py:18-173).  Coordinates are cached per tensor
    stride, maps per ``(source stride, target stride, kernel size, dilation)``;
    a transposed convolution reuses the map of its forward twin with the two
    masks swapped.  ``reset()`` must be called between unrelated inputs.

    Differences that a caller can observe: mask, order and size tensors are
    int32 whatever the coordinate dtype; ties in the size order are broken by
    offset index (the reference's ``torch.sort`` leaves them unspecified).

    Internally every coordinate set is packed once into 64-bit keys whose layout
    is derived from the bounding box of the first tensor seen after ``reset()``.
    """

    def __init__(self, ndim: int, dtype: torch.dtype, device: Union[str, torch.device],
                 layout: str = "minuet", disable_reordering: bool = False):
        self._ndim = ndim
        self._dtype = dtype
        self._device = torch.device(device)
        self._layout = layout
        self._disable_reordering = disable_reordering
        self._kernel_maps_cache = dict()
        self._coordinates_cache = dict()
        self._offsets_cache = dict()
        self._keys = dict()          # stride -> (coordinates tensor, keys tensor)
        self._spec = None
        self._spec_dev = None        # device copy of the key layout (kept alive with the spec)
        self._root_keys = None       # (coordinates tensor, keys) of the first tensor seen
        self._root = None            # (coords int32, batch_dims int64, num_clouds)

    # -- bookkeeping ------------------------------------------------------------
    def reset(self):
        self._coordinates_cache.clear()
        self._kernel_maps_cache.clear()
        self._keys.clear()
        self._spec = None
        self._spec_dev = None
        self._root_keys = None
        self._root = None

    def _get_kernel_offsets(self, source_stride, kernel_size, kernel_dilation) -> np.ndarray:
        key = (source_stride, kernel_size, kernel_dilation)
        if key not in self._offsets_cache:
            table = generate_kernel_offsets(ndim=self._ndim, kernel_size=kernel_size,
                                            source_stride=source_stride,
                                            dilation=kernel_dilation, layout=self._layout)
            self._offsets_cache[key] = np.ascontiguousarray(table, dtype=np.int32)
        return self._offsets_cache[key]

    def _ensure_spec(self, coordinates, batch_dims, margin: int):
        """Key layout for this forward pass; rebuilt (and every cached key array
        dropped) when a later layer needs a larger margin."""
        if self._root is None:
            bd = engine.as_i64(batch_dims)
            self._root = (engine.as_i32_coords(coordinates), bd,
                          1 if bd is None else bd.numel() - 1)
        if self._spec is None or self._spec.margin < margin:
            coords, bd, num_clouds = self._root
            # bounding box, key layout and the keys of the first tensor in one launch;
            # all of it stays on the device: no read-back here
            self._spec, self._spec_dev, keys = engine.make_keyspec_device(
                coords, bd, self._ndim, num_clouds, max(int(margin), engine.DEFAULT_MARGIN))
            self._keys.clear()
            self._root_keys = (coordinates, keys)
        return self._spec

    def _keys_of(self, coordinates, batch_dims, stride):
        hit = self._keys.get(stride)
        if hit is not None and hit[0] is coordinates:
            return hit[1]
        if self._root_keys is not None and self._root_keys[0] is coordinates:
            self._keys[stride] = self._root_keys
            return self._root_keys[1]
        keys = engine.pack_keys(engine.as_i32_coords(coordinates), engine.as_i64(batch_dims),
                                self._spec)
        self._keys[stride] = (coordinates, keys)
        return keys

    # -- coordinates ------------------------------------------------------------
    def get_target_coordinates(self, source_coordinates: torch.Tensor,
                               source_batch_dims: Optional[torch.Tensor], source_stride,
                               kernel_stride, transposed: bool = False):
        """Coordinates, stride and batch_dims of a layer's output
        (minuet/nn/convolutions.py:58-100): the input itself for stride 1,
        ``unique(floor(c / ts) * ts)`` for a strided layer, and the cached
        coordinates at ``source_stride // kernel_stride`` for a transposed one."""
        ndim = source_coordinates.shape[1]
        source_stride = as_tuple(source_stride, size=ndim, name="source_stride")
        kernel_stride = as_tuple(kernel_stride, size=ndim, name="kernel_stride")
        if source_stride not in self._coordinates_cache:
            self._coordinates_cache[source_stride] = (source_coordinates, source_stride,
                                                      source_batch_dims)
        if transposed:
            target_stride = tuple(a // b for a, b in zip(source_stride, kernel_stride))
        else:
            target_stride = tuple(a * b for a, b in zip(source_stride, kernel_stride))
        if target_stride in self._coordinates_cache:
            return self._coordinates_cache[target_stride]
        if transposed:
            raise RuntimeError("Layer must transpose=True must have its corresponding "
                               "non-transposed layer before its execution")

        engine.require_cuda(source_coordinates, source_batch_dims)
        coords = engine.as_i32_coords(source_coordinates)
        bd = engine.as_i64(source_batch_dims)
        nb = 1 if bd is None else bd.numel() - 1
        n = coords.shape[0]
        device = coords.device
        spec = self._ensure_spec(source_coordinates, source_batch_dims, max(target_stride) - 1)
        ts = np.asarray(target_stride, dtype=np.int32)
        unique = torch.empty((n, ndim), dtype=torch.int32, device=device)
        keys = torch.empty(n, dtype=torch.int64, device=device)
        meta = torch.empty(nb + 3, dtype=torch.int64, device=device)  # count, batch_dims, status
        lib = engine.lib()
        ws = engine.workspace(lib.mn_map_workspace_bytes(n, n, 1), device)
        _lib.check(lib.mn_downsample_coordinates(
            engine.ptr(coords), n, ndim, engine.ptr(bd), nb, engine.np_ptr(ts), ctypes.byref(spec),
            engine.ptr(unique), engine.ptr(keys), engine.ptr(meta),
            engine.ptr(engine.control_block(device)), engine.ptr(ws), ws.numel(),
            engine.stream_ptr(device)), "downsample_coordinates")
        # the one blocking read of a strided level: the number of output rows sets
        # the shapes of everything that follows
        host = engine.read_small(meta)
        engine.raise_on_status(int(host[-1]), device)
        count = int(host[0])
        target_coordinates = unique[:count]
        if source_coordinates.dtype != torch.int32:
            target_coordinates = target_coordinates.to(source_coordinates.dtype)
        target_batch_dims = None
        if source_batch_dims is not None:
            target_batch_dims = meta[1:nb + 2].to(source_batch_dims.dtype)
            engine.remember_host(target_batch_dims, host[1:nb + 2].copy())
        self._keys[target_stride] = (target_coordinates, keys[:count])
        self._coordinates_cache[target_stride] = (target_coordinates, target_stride,
                                                  target_batch_dims)
        return self._coordinates_cache[target_stride]

    # -- kernel maps ------------------------------------------------------------
    def get_kernel_map(self, source_coordinates: torch.Tensor, source_stride,
                       source_batch_dims: Optional[torch.Tensor],
                       target_coordinates: torch.Tensor, target_stride,
                       target_batch_dims: Optional[torch.Tensor], kernel_size, kernel_dilation,
                       disable_reordering: bool = False, transposed: bool = False):
        """``(source_masks, target_masks, kernel_map_order, kernel_map_sizes)`` of
        one convolution geometry (minuet/nn/convolutions.py:102-173)."""
        num_sources, ndim = source_coordinates.shape
        source_stride = as_tuple(source_stride, size=ndim, name="source_stride")
        target_stride = as_tuple(target_stride, size=ndim, name="target_stride")
        kernel_size = as_tuple(kernel_size, size=ndim, name="kernel_size")
        kernel_dilation = as_tuple(kernel_dilation, size=ndim, name="kernel_dilation")
        strides = (target_stride, source_stride) if transposed else (source_stride, target_stride)
        key = (*strides, kernel_size, kernel_dilation)
        if key in self._kernel_maps_cache:
            source_masks, target_masks, order, sizes = self._kernel_maps_cache[key]
            if transposed:
                source_masks, target_masks = target_masks, source_masks
            return source_masks, target_masks, order, sizes
        if transposed:
            raise RuntimeError("Layer must transpose=True must have its corresponding "
                               "non-transposed layer before its execution")

        engine.require_cuda(source_coordinates, target_coordinates)
        offsets = self._get_kernel_offsets(source_stride, kernel_size, kernel_dilation)
        reorder = not (self._disable_reordering or disable_reordering)
        margin = int(np.abs(offsets).max()) + max(max(source_stride), max(target_stride)) - 1
        spec = self._ensure_spec(source_coordinates, source_batch_dims, margin)
        skeys = self._keys_of(source_coordinates, source_batch_dims, source_stride)
        if target_coordinates is source_coordinates:
            tkeys = skeys
        else:
            tkeys = self._keys_of(target_coordinates, target_batch_dims, target_stride)
        result = build_kernel_map(skeys, tkeys, offsets, spec, reorder)
        self._kernel_maps_cache[key] = result
        return result


def build_kernel_map(source_keys: torch.Tensor, target_keys: torch.Tensor, offsets: np.ndarray,
                     spec, reorder: bool):
    """Masks, order and sizes from packed keys.  Up to 32 offsets take the fused
    build; larger kernels go through a materialised kernel map."""
    device = source_keys.device
    S, T, O = source_keys.numel(), target_keys.numel(), offsets.shape[0]
    lib = engine.lib()
    source_masks = torch.empty((O, S), dtype=torch.int32, device=device)
    target_masks = torch.empty((O, T), dtype=torch.int32, device=device)
    # one allocation for the small outputs: order [O], sizes + status word [O + 1] and the
    # per-row hit words [S], [T] (each part starts on a 256-byte boundary)
    pad = lambda n: -(-n // 64) * 64
    small = torch.empty(2 * pad(O + 1) + pad(S) + pad(T), dtype=torch.int32, device=device)
    order = small[:O]
    sizes_status = small[pad(O + 1):pad(O + 1) + O + 1]                  # sizes, status word
    sizes = sizes_status[:O]
    ws = engine.workspace(lib.mn_map_workspace_bytes(S, T, O), device)
    stream = engine.stream_ptr(device)
    if O <= 32:
        # per-row hit words in mask-row order, kept with the masks for the forward kernels
        base = 2 * pad(O + 1)
        source_bits = small[base:base + S]
        target_bits = small[base + pad(S):base + pad(S) + T]
        same = source_keys.data_ptr() == target_keys.data_ptr() and S == T
        _lib.check(lib.mn_build_kernel_map(
            engine.ptr(source_keys), S, engine.ptr(source_keys if same else target_keys), T,
            engine.np_ptr(offsets), O, ctypes.byref(spec), int(reorder), engine.ptr(source_masks),
            engine.ptr(target_masks), engine.ptr(order), engine.ptr(sizes_status),
            engine.ptr(source_bits), engine.ptr(target_bits),
            engine.ptr(engine.control_block(device)), engine.ptr(ws), ws.numel(), stream),
            "build_kernel_map")
        engine.remember_bits(source_masks, target_masks, source_bits, target_bits)
    else:
        kernel_map = torch.empty((O, T), dtype=torch.int32, device=device)
        _lib.check(lib.mn_query_sorted_index_with_offsets(
            engine.ptr(source_keys), S, engine.ptr(target_keys), T, engine.np_ptr(offsets), O,
            ctypes.byref(spec), engine.ptr(kernel_map), stream), "query_sorted_index_with_offsets")
        _lib.check(lib.mn_compute_kernel_map_sizes(engine.ptr(kernel_map), O, T, engine.ptr(sizes),
                                                   stream), "compute_kernel_map_sizes")
        if reorder:
            sorted_sizes, order64 = torch.sort(sizes, stable=True)
            sizes.copy_(sorted_sizes)
            order = order64.to(torch.int32)
            kernel_map = kernel_map[order64]
        else:
            order = torch.arange(O, dtype=torch.int32, device=device)
        sizes_status[O:].copy_(engine.status_word(device))
        _lib.check(lib.mn_compute_kernel_map_masks(
            engine.ptr(kernel_map), O, S, T, engine.ptr(source_masks), engine.ptr(target_masks),
            engine.ptr(ws), ws.numel(), stream), "compute_kernel_map_masks")
    # the GEMM plan needs the sizes on the host: start the copy (sizes + status
    # word) now, wait for it only when a convolution asks
    engine.remember_host(sizes, engine.PendingHostCopy(sizes_status))
    return source_masks, target_masks, (order if reorder else None), sizes


class SparseConv(Module):
    r"""Sparse convolution over a :class:`SparseTensor`
    (minuet/nn/convolutions.py:176-499).

    With input points :math:`P`, tensor stride :math:`s` and kernel stride
    :math:`k` the output points are
    :math:`Q = \{\lfloor p / (sk) \rfloor \cdot sk : p \in P\}` and
    :math:`F^Q_i = \sum_j \sum_k [p_j = q_i + \delta_k] \, F^P_j W_k` over the
    offsets :math:`\delta_k` of :func:`generate_kernel_offsets`.

    Parameters are ``kernel`` of shape ``[K^D, C_in, C_out]`` and an optional
    ``bias`` ``[C_out]`` (same names and shapes as the reference, so its
    state_dicts load).  A 1x1x1 convolution with stride and dilation 1 is a plain
    matrix product and needs no kernel map cache.
    """

    # Bucket thresholds only decide how the reference pads its cuBLAS batches; here the
    # grouped GEMM takes every offset at its own size, so the key stays in the config
    # (files written by the reference load) and only these few values are ever timed.
    __AVAILABLE_THRESHOLD__ = [-1, 0.0, 0.5, None]
    __AVAILABLE_SUB_TILES__ = [1, 2, 3, 4]
    __NUM_TUNING_ROUNDS__ = 10

    def __init__(self, ndim: int, in_channels: int, out_channels: int, kernel_size,
                 stride=1, dilation=1, bias: bool = False, transposed: bool = False,
                 dtype: Optional[torch.dtype] = None, device: Optional[torch.device] = None):
        super().__init__()
        self.ndim = ndim
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.kernel_size = as_tuple(kernel_size, size=ndim, name="kernel_size")
        self.stride = as_tuple(stride, size=ndim, name="stride")
        self.dilation = as_tuple(dilation, size=ndim, name="dilation")
        self.transposed = transposed
        volume = int(np.prod(self.kernel_size))
        self.kernel = torch.nn.Parameter(
            torch.empty(volume, in_channels, out_channels, dtype=dtype, device=device))
        if bias:
            self.bias = torch.nn.Parameter(torch.empty(out_channels, dtype=dtype, device=device))
        else:
            self.register_parameter('bias', None)
        self.reset_parameters()
        self._kernel_map_cache: Optional[KernelMapCache] = None
        # threshold / tile sizes: the reference's keys (minuet/nn/convolutions.py:277-281);
        # algorithm ("auto", "explicit", "implicit") and sub_tiles (row sub-tiles per tile
        # of the fused kernel, 0 = automatic) are the knobs that matter on this library
        self._tunable_config = {'threshold': -1,
                                'gather_tile_size': min(in_channels, 1),
                                'scatter_tile_size': min(out_channels, 1),
                                'algorithm': 'auto',
                                'sub_tiles': 0}
        self._tuning_data = None
        self._tuning_maps = None
        self._tuning_epilogue = (False, False, False, False)
        self._frozen_kernel_t = None

    def reset_parameters(self):
        """Uniform init in ``+-1/sqrt(fan * K^D)`` with ``fan`` the input channels
        (output channels when transposed), minuet/nn/convolutions.py:311-319."""
        fan = self.out_channels if self.transposed else self.in_channels
        bound = 1.0 / math.sqrt(fan * self.kernel.shape[0])
        self._frozen_kernel_t = None
        with torch.no_grad():
            self.kernel.uniform_(-bound, bound)
            if self.bias is not None:
                self.bias.uniform_(-bound, bound)

    def freeze_weights(self, frozen: bool = True):
        """Inference preparation: keep the kernel in the layout the tensor-core kernels
        read, so that forward passes stop transposing it on every call.  The copy is
        taken NOW; call again (or ``freeze_weights(False)``) after changing the kernel.
        Moving or casting the module, ``train()`` and ``reset_parameters`` drop it."""
        self._frozen_kernel_t = F.transpose_weights(self.kernel) if frozen else None
        return self

    def train(self, mode: bool = True):
        if mode:
            self._frozen_kernel_t = None
        return super().train(mode)

    def _apply(self, fn, *args, **kwargs):
        self._frozen_kernel_t = None
        return super()._apply(fn, *args, **kwargs)

    def set_kernel_map_cache(self, cache: KernelMapCache):
        self._kernel_map_cache = cache

    @property
    def tunable_config(self) -> Dict[str, Any]:
        return self._tunable_config

    @property
    def is_trivial(self) -> bool:
        return all(v == 1 for v in self.stride + self.dilation + self.kernel_size)

    @property
    def _allow_shortcut_matmul(self) -> bool:
        return (all(v == 1 for v in self.dilation + self.stride)
                and not self._kernel_map_cache._disable_reordering)

    def extra_repr(self) -> str:
        parts = [f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}"]
        if any(v != 1 for v in self.stride):
            parts.append(f"stride={self.stride}")
        if any(v != 1 for v in self.dilation):
            parts.append(f"dilation={self.dilation}")
        if self.bias is None:
            parts.append("bias=False")
        if self.transposed:
            parts.append("transposed=True")
        return ", ".join(parts)

    # -- autotuning ---------------------------------------------------------------
    def _sweep(self, timer, candidates, arg_name, config_key, stop_on_error=False, **fixed):
        """Time every candidate on the recorded maps and keep the fastest."""
        best = None
        for value in candidates:
            try:
                times = [timer(weights=self.kernel, source_masks=sm, target_masks=tm,
                               kernel_map_sizes=sz,
                               allow_shortcut_matmul=self._allow_shortcut_matmul,
                               **{arg_name: value}, **fixed)
                         for _ in range(self.__NUM_TUNING_ROUNDS__)
                         for sm, tm, sz in self._tuning_data]
            except RuntimeError:
                if not stop_on_error:
                    raise
                F.cuda_reset_error()
                print(f"Threshold {value} overflows memory exiting tuning")
                print(f"optimal={self._tunable_config[config_key]}")
                break
            mean = float(np.mean(times))
            if best is None or mean < best:
                best = mean
                self._tunable_config[config_key] = value

    def _time_algorithm(self, algorithm: str, sub_tiles: int) -> float:
        """Mean milliseconds of a whole forward pass over the recorded maps (after one
        untimed pass, which builds whatever the algorithm derives from the map once:
        pair lists, neighbour tables)."""
        kw = dict(allow_shortcut_matmul=self._allow_shortcut_matmul, algorithm=algorithm,
                  sub_tiles=sub_tiles, epilogue=self._tuning_epilogue)
        for sm, tm, order, sz in self._tuning_maps:
            F.time_forward(self.kernel, sm, tm, order, sz, **kw)
        times = [F.time_forward(self.kernel, sm, tm, order, sz,
                                allow_shortcut_matmul=self._allow_shortcut_matmul,
                                algorithm=algorithm, sub_tiles=sub_tiles,
                                gather_tile_size=self._tunable_config['gather_tile_size'],
                                scatter_tile_size=self._tunable_config['scatter_tile_size'],
                                threshold=self._tunable_config['threshold'],
                                epilogue=self._tuning_epilogue)
                 for _ in range(self.__NUM_TUNING_ROUNDS__)
                 for sm, tm, order, sz in self._tuning_maps]
        return float(np.mean(times))

    @contextlib.contextmanager
    def autotune(self, free_buffers: bool = True):
        """Record the kernel maps this layer sees inside the ``with`` block, then
        time the candidates for ``__NUM_TUNING_ROUNDS__`` rounds each and keep the
        fastest (minuet/nn/convolutions.py:337-444): for fp32 layers (gather - grouped
        GEMM - scatter) ``threshold``, ``gather_tile_size`` and ``scatter_tile_size`` as
        the reference does; for fp16/bf16 layers ``algorithm`` (pair lists against the
        fused kernel) and the fused kernel's ``sub_tiles``."""
        try:
            self._tuning_data = list()
            self._tuning_maps = list()
            if free_buffers:
                F.cuda_free_buffers()
            yield
            if free_buffers:
                F.cuda_free_buffers()
            if self.is_trivial or not self._tuning_data:
                return
            lib = engine.lib()
            code = engine.dtype_code(self.kernel.dtype)
            volume = self.kernel.shape[0]
            # 16-bit layers with few input channels run zero-padded to a multiple of 8
            c_in = self.in_channels
            if self.kernel.dtype != torch.float32 and self.out_channels % 8 == 0:
                c_in = -(-c_in // 8) * 8
            pairs_ok = self.kernel.dtype != torch.float32 and bool(lib.mn_pairs_supported(
                volume, c_in, self.out_channels, code))
            if not pairs_ok:
                self._sweep(F.cuda_time_gemm, self.__AVAILABLE_THRESHOLD__, 'threshold',
                            'threshold', stop_on_error=True)
                threshold = self._tunable_config['threshold']
                divisors = lambda c: [t for t in range(1, c + 1) if c % t == 0]
                self._sweep(F.cuda_time_gather, divisors(self.in_channels), 'tile_size',
                            'gather_tile_size', threshold=threshold)
                self._sweep(F.cuda_time_scatter, divisors(self.out_channels), 'tile_size',
                            'scatter_tile_size', threshold=threshold)
            if lib.mn_implicit_supported(volume, c_in, self.out_channels, code):
                n_pad = -(-self.out_channels // 16) * 16
                best, choice = self._time_algorithm('explicit', 0), ('explicit', 0)
                for sub in self.__AVAILABLE_SUB_TILES__:
                    if sub * n_pad > 512:
                        break
                    ms = self._time_algorithm('implicit', sub)
                    if ms < best:
                        best, choice = ms, ('implicit', sub)
                self._tunable_config['algorithm'], self._tunable_config['sub_tiles'] = choice
            else:
                self._tunable_config['algorithm'] = 'explicit'
            if free_buffers:
                F.cuda_free_buffers()
        finally:
            self._tuning_data = None
            self._tuning_maps = None

    # -- forward ------------------------------------------------------------------
    def prepare(self, coordinates: torch.Tensor, stride, batch_dims: Optional[torch.Tensor]):
        """Build (or find in the cache) the output coordinates and the kernel map this
        layer needs for inputs at ``coordinates`` / ``stride``, without running it, and
        return ``(coordinates, stride, batch_dims)`` of its output.  A model that calls
        this for all its layers before the first convolution has every blocking read
        and every kernel-map build behind it when the feature kernels start, and its
        forward pass then runs without a host wait (see ``SparseUNet.plan``)."""
        if self.is_trivial:
            return coordinates, stride, batch_dims
        cache = self._kernel_map_cache
        if cache is None:
            raise ValueError("Kernel map cache must be specified")
        out_c, out_s, out_bd = cache.get_target_coordinates(
            source_coordinates=coordinates, source_batch_dims=batch_dims, source_stride=stride,
            kernel_stride=self.stride, transposed=self.transposed)
        cache.get_kernel_map(
            source_coordinates=coordinates, source_stride=stride, source_batch_dims=batch_dims,
            target_coordinates=out_c, target_stride=out_s, target_batch_dims=out_bd,
            kernel_size=self.kernel_size, kernel_dilation=self.dilation,
            transposed=self.transposed)
        return out_c, out_s, out_bd

    def _lookup(self, inputs: SparseTensor):
        """Output coordinates and the kernel map of this layer for ``inputs``."""
        cache = self._kernel_map_cache
        if cache is None:
            raise ValueError("Kernel map cache must be specified")
        coordinates, stride, batch_dims = cache.get_target_coordinates(
            source_coordinates=inputs.C, source_batch_dims=inputs.batch_dims,
            source_stride=inputs.stride, kernel_stride=self.stride, transposed=self.transposed)
        source_masks, target_masks, order, sizes = cache.get_kernel_map(
            source_coordinates=inputs.C, source_stride=inputs.stride,
            source_batch_dims=inputs.batch_dims, target_coordinates=coordinates,
            target_stride=stride, target_batch_dims=batch_dims, kernel_size=self.kernel_size,
            kernel_dilation=self.dilation, transposed=self.transposed)
        if self._tuning_data is not None:
            self._tuning_data.append((source_masks, target_masks, sizes))
            self._tuning_maps.append((source_masks, target_masks, order, sizes))
        return coordinates, stride, batch_dims, source_masks, target_masks, order, sizes

    def forward(self, inputs: SparseTensor) -> SparseTensor:
        features = inputs.F
        if self.is_trivial and torch.is_grad_enabled() and (
                features.requires_grad or self.kernel.requires_grad):
            # training: the plain product, differentiated by autograd
            out = features @ self.kernel.view(self.in_channels, self.out_channels)
            if self.bias is not None:
                out = out + self.bias
            return SparseTensor(out, inputs.C, stride=inputs.stride, batch_dims=inputs.batch_dims)
        if self.is_trivial:
            bias = None if self.bias is None else self.bias.detach().float()
            out = F.dense_forward(features, self.kernel.view(self.in_channels, self.out_channels),
                                  shift=bias, weights_t=self._frozen_kernel_t)
            return SparseTensor(out, inputs.C, stride=inputs.stride, batch_dims=inputs.batch_dims)
        else:
            coordinates, stride, batch_dims, source_masks, target_masks, order, sizes = \
                self._lookup(inputs)
            out = F.sparse_convolution_forward(
                sources=features, weights=self.kernel, source_masks=source_masks,
                target_masks=target_masks, kernel_map_order=order, kernel_map_sizes=sizes,
                gather_tile_size=self._tunable_config["gather_tile_size"],
                scatter_tile_size=self._tunable_config["scatter_tile_size"],
                allow_shortcut_matmul=self._allow_shortcut_matmul,
                threshold=self._tunable_config["threshold"],
                algorithm=self._tunable_config.get("algorithm"),
                sub_tiles=self._tunable_config.get("sub_tiles"),
                weights_t=self._frozen_kernel_t)
        if self.bias is not None:
            out += self.bias
        return SparseTensor(out, coordinates, stride=stride, batch_dims=batch_dims)

    def forward_fused(self, inputs: SparseTensor, scale: Optional[torch.Tensor] = None,
                      shift: Optional[torch.Tensor] = None,
                      residual: Optional[torch.Tensor] = None, relu: bool = False) -> SparseTensor:
        """``relu?((conv(inputs) + bias) * scale + shift + residual)`` with the
        epilogue applied inside the convolution (or in one in-place pass after it).
        Inference only; ``scale`` / ``shift`` are ``[out_channels]`` vectors, e.g.
        an eval-mode BatchNorm folded by :func:`fold_batchnorm`."""
        if self.bias is not None:
            bias = self.bias.detach().float()
            shift = bias * (1.0 if scale is None else scale.float()) + \
                (0.0 if shift is None else shift.float())
        features = inputs.F
        if self.is_trivial:
            out = F.dense_forward(features, self.kernel.view(self.in_channels, self.out_channels),
                                  scale, shift, residual, relu, weights_t=self._frozen_kernel_t)
            return SparseTensor(out, inputs.C, stride=inputs.stride, batch_dims=inputs.batch_dims)
        coordinates, stride, batch_dims, source_masks, target_masks, order, sizes = \
            self._lookup(inputs)
        if self._tuning_data is not None:     # the tuner times the layer with the epilogue it runs
            self._tuning_epilogue = (scale is not None, shift is not None, residual is not None,
                                     bool(relu))
        out = F.sparse_convolution_forward_fused(
            sources=features, weights=self.kernel, source_masks=source_masks,
            target_masks=target_masks, kernel_map_order=order, kernel_map_sizes=sizes,
            gather_tile_size=self._tunable_config["gather_tile_size"],
            scatter_tile_size=self._tunable_config["scatter_tile_size"],
            allow_shortcut_matmul=self._allow_shortcut_matmul,
            threshold=self._tunable_config["threshold"], scale=scale, shift=shift,
            residual=residual, relu=relu, algorithm=self._tunable_config.get("algorithm"),
            sub_tiles=self._tunable_config.get("sub_tiles"), weights_t=self._frozen_kernel_t)
        return SparseTensor(out, coordinates, stride=stride, batch_dims=batch_dims)


def fold_batchnorm(bn: torch.nn.modules.batchnorm._BatchNorm):
    """``(scale, shift)`` fp32 vectors equivalent to an eval-mode BatchNorm:
    ``bn(x) == x * scale + shift``."""
    var = bn.running_var.detach().float()
    mean = bn.running_mean.detach().float()
    weight = torch.ones_like(var) if bn.weight is None else bn.weight.detach().float()
    bias = torch.zeros_like(var) if bn.bias is None else bn.bias.detach().float()
    scale = weight / torch.sqrt(var + bn.eps)
    return scale.contiguous(), (bias - mean * scale).contiguous()


class SparseConv3d(SparseConv):
    """3-D, non-transposed :class:`SparseConv` (minuet/nn/convolutions.py:502-527)."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, dilation=1,
                 bias: bool = False, dtype: Optional[torch.dtype] = None,
                 device: Optional[torch.device] = None):
        super().__init__(ndim=3, in_channels=in_channels, out_channels=out_channels,
                         kernel_size=kernel_size, stride=stride, dilation=dilation, bias=bias,
                         transposed=False, dtype=dtype, device=device)
