"""Global pooling modules (minuet/nn/pooling.py)."""
__all__ = ['GlobalAvgPool', 'GlobalMaxPool', 'GlobalSumPool']

import torch
from torch.nn import Module

from minuet_b200.nn import functional as F
from minuet_b200.tensors import SparseTensor


class GlobalAvgPool(Module):
    def forward(self, x: SparseTensor) -> torch.Tensor:
        return F.global_avg_pool(x)


class GlobalMaxPool(Module):
    def forward(self, x: SparseTensor) -> torch.Tensor:
        return F.global_max_pool(x)


class GlobalSumPool(Module):
    def forward(self, x: SparseTensor) -> torch.Tensor:
        return F.global_sum_pool(x)
