__all__ = ['global_avg_pool', 'global_sum_pool', 'global_max_pool']

import torch

from minuet_b200.tensors import SparseTensor


def _per_cloud(x: SparseTensor, fn) -> torch.Tensor:
    if x.batch_dims is None:
        return fn(x.F)
    bounds = x.batch_dims.tolist()
    return torch.stack([fn(x.F[a:b]) for a, b in zip(bounds[:-1], bounds[1:])], dim=0)


def global_avg_pool(x: SparseTensor) -> torch.Tensor:
    """Mean feature per cloud, ``[B, C]`` (minuet/nn/functional/pooling.py)."""
    return _per_cloud(x, lambda f: f.mean(dim=0))


def global_sum_pool(x: SparseTensor) -> torch.Tensor:
    return _per_cloud(x, lambda f: f.sum(dim=0))


def global_max_pool(x: SparseTensor) -> torch.Tensor:
    return _per_cloud(x, lambda f: f.max(dim=0).values)
