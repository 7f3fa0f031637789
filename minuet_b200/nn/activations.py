"""Pointwise activations on the feature matrix (minuet/nn/activations.py)."""
__all__ = ['ReLU', 'ReLU6', 'LeakyReLU']

import torch

from minuet_b200.tensors import SparseTensor


def _on_features(x: SparseTensor, features: torch.Tensor) -> SparseTensor:
    return SparseTensor(features, x.C, stride=x.stride, batch_dims=x.batch_dims)


class ReLU(torch.nn.ReLU):
    def forward(self, x: SparseTensor):
        return _on_features(x, super().forward(x.F))


class ReLU6(torch.nn.ReLU6):
    def forward(self, x: SparseTensor):
        return _on_features(x, super().forward(x.F))


class LeakyReLU(torch.nn.LeakyReLU):
    def forward(self, x: SparseTensor):
        return _on_features(x, super().forward(x.F))
