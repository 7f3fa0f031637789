"""Host helpers: kernel offset tables, cache attachment, model-level autotune and
the tunable-config JSON (API of minuet/utils/helpers.py)."""
__all__ = ['as_tuple', 'generate_kernel_offsets', 'set_kernel_map_cache',
           'dump_tunable_config', 'load_tunable_config', 'autotune']

import contextlib
import itertools
import json
import os
from collections.abc import Iterable
from typing import Optional

import numpy as np
from torch.nn import Module


def as_tuple(value, *, size: int = 3, name: Optional[str] = None):
    """``value`` repeated ``size`` times when it is a scalar, else checked to have
    ``size`` elements (minuet/utils/helpers.py:138-162)."""
    if not isinstance(value, Iterable):
        return (value,) * size
    value = tuple(value)
    if len(value) != size:
        raise ValueError(f"{name or 'Value'} must be a scalar or a iterable of size {size} "
                         f"but found {len(value)} elements")
    return value


def generate_kernel_offsets(ndim: int, kernel_size, source_stride, dilation,
                            layout: str = "minuet") -> np.ndarray:
    """Offset table ``[prod(kernel_size), ndim]`` of a sparse convolution.

    Per dimension the taps are ``-k//2 .. k//2`` for odd ``k`` and
    ``-k//2 + 1 .. k//2`` for even ``k`` (so ``k = 2`` gives ``{0, 1}``), scaled by
    ``source_stride * dilation``.  Row ``i`` of the table belongs to weight
    ``kernel[i]``.  Layouts (minuet/utils/helpers.py:165-212): ``"minuet"`` lists
    the taps with dimension 0 slowest; ``"minkowski"`` with dimension 0 fastest;
    ``"torchsparse"`` like ``"minkowski"`` for odd kernel volumes and like
    ``"minuet"`` for even ones.
    """
    kernel_size = as_tuple(kernel_size, size=ndim, name="kernel_size")
    source_stride = as_tuple(source_stride, size=ndim, name="source_stride")
    dilation = as_tuple(dilation, size=ndim, name="dilation")
    if layout not in ("minuet", "minkowski", "torchsparse"):
        raise NotImplementedError(f"unknown kernel offset layout {layout!r}")
    taps = [range(-(k // 2) + (1 - k % 2), k // 2 + 1) for k in kernel_size]
    volume = int(np.prod(kernel_size))
    fastest_first = layout == "minkowski" or (layout == "torchsparse" and volume % 2 == 1)
    if fastest_first:
        rows = [tuple(reversed(t)) for t in itertools.product(*reversed(taps))]
    else:
        rows = list(itertools.product(*taps))
    table = np.asarray(rows, dtype=np.int64).reshape(volume, ndim)
    return table * np.asarray(source_stride) * np.asarray(dilation)


def set_kernel_map_cache(module: Module, cache):
    """Attach ``cache`` to ``module`` and every descendant that has a
    ``set_kernel_map_cache`` method (minuet/utils/helpers.py:29-46)."""
    for sub in module.modules():
        if hasattr(sub, "set_kernel_map_cache"):
            sub.set_kernel_map_cache(cache)
    return module


def dump_tunable_config(module: Module) -> dict:
    """Nested dict of every ``tunable_config`` in the module tree, keyed by child
    names (the JSON format of minuet/utils/helpers.py:118-135)."""
    if hasattr(module, "tunable_config"):
        return module.tunable_config
    return {name: dump_tunable_config(child) for name, child in module.named_children()}


def load_tunable_config(module: Module, config: dict):
    if hasattr(module, "tunable_config"):
        module.tunable_config.update(config)
    for name, child in module.named_children():
        load_tunable_config(child, config=config[name])
    return module


def autotune(model: Module, model_cache, data, cache_path: Optional[str] = None):
    """Tune every layer that has an ``autotune()`` context on the given samples
    (minuet/utils/helpers.py:49-94).  With an existing ``cache_path`` the stored
    JSON is loaded instead; otherwise the result is written there."""
    from minuet_b200.tensors import SparseTensor
    if isinstance(data, SparseTensor):
        data = [data]
    if cache_path is not None and os.path.exists(cache_path):
        with open(cache_path) as reader:
            return load_tunable_config(model, config=json.load(reader))
    with contextlib.ExitStack() as stack:
        for sub in model.modules():
            if hasattr(sub, "autotune"):
                stack.enter_context(sub.autotune())
        for tensor in data:
            model_cache.reset()
            model(tensor)
    if cache_path is not None:
        folder = os.path.dirname(cache_path)
        if folder:
            os.makedirs(folder, exist_ok=True)
        with open(cache_path, "w") as writer:
            json.dump(dump_tunable_config(model), writer, indent=2)
    return model
