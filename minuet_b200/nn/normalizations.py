"""Batch normalisation on the feature matrix (minuet/nn/normalizations.py)."""
__all__ = ['BatchNorm']

import torch

from minuet_b200.tensors import SparseTensor


class BatchNorm(torch.nn.BatchNorm1d):
    def forward(self, x: SparseTensor):
        return SparseTensor(super().forward(x.F), x.C, stride=x.stride, batch_dims=x.batch_dims)
