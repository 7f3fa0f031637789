__all__ = ['cat']

from typing import Sequence

import torch

from minuet_b200.tensors import SparseTensor


def cat(tensors: Sequence[SparseTensor]) -> SparseTensor:
    """Channel-wise concatenation of sparse tensors that share coordinates
    (minuet/nn/functional/concat.py)."""
    if len(tensors) == 0:
        raise ValueError("cat needs at least one tensor")
    first = tensors[0]
    for t in tensors[1:]:
        if t.n != first.n or t.stride != first.stride:
            raise ValueError("cat: tensors must share coordinates and stride")
    return SparseTensor(features=torch.cat([t.F for t in tensors], dim=1),
                        coordinates=first.C, stride=first.stride, batch_dims=first.batch_dims)
