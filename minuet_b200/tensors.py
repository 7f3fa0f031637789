"""``SparseTensor``: features + sorted unique integer coordinates of one or more
point clouds (API of minuet/tensors.py:38-283)."""
__all__ = ['SparseTensor']

from typing import Optional

import torch

from minuet_b200.utils.helpers import as_tuple


def _validate(features: torch.Tensor, coordinates: torch.Tensor):
    if coordinates.ndim != 2:
        raise ValueError(f"The coordinates tensor must be a 2-D tensor but found "
                         f"{coordinates.ndim}-D")
    if coordinates.dtype not in (torch.int32, torch.int64):
        raise ValueError(f"The coordinates tensor must be int32 or int64 "
                         f"but found {coordinates.dtype}")
    if features.shape[0] != coordinates.shape[0]:
        raise ValueError(f"The features tensor indicate {features.shape[0]} coordinates but "
                         f"expected {coordinates.shape[0]} coordinates")
    if features.device != coordinates.device:
        raise ValueError(f"The features tensor is expected to be on the same device as the "
                         f"coordinates tensor {coordinates.device} but found {features.device}")
    if coordinates.requires_grad:
        raise ValueError("The coordinates tensor should never requires gradients")


class SparseTensor(object):
    """Features ``[N, C]`` with coordinates ``[N, D]`` (int32 or int64).

    The coordinates must be unique and sorted (cloud-major, then lexicographic).
    Several clouds share one tensor through ``batch_dims`` (``[B + 1]`` prefix
    offsets: cloud ``i`` owns rows ``batch_dims[i]:batch_dims[i + 1]``); as in the
    reference a ``batch_dims`` of length <= 2 (one cloud) is dropped
    (minuet/tensors.py:77-79).  ``stride`` is the tensor stride of the voxel grid.
    """

    def __init__(self, features: torch.Tensor, coordinates: torch.Tensor, *,
                 stride=1, batch_dims: Optional[torch.Tensor] = None):
        _validate(features, coordinates)
        self._features = features
        self._coordinates = coordinates
        self._stride = as_tuple(stride, size=coordinates.shape[1], name="strides")
        self._batch_dims = batch_dims if (batch_dims is not None and len(batch_dims) > 2) else None

    # -- views ----------------------------------------------------------------
    @property
    def F(self) -> torch.Tensor:
        return self._features

    @F.setter
    def F(self, features: torch.Tensor):
        if features.device != self._features.device:
            raise ValueError(f"The new features is on the device {features.device} which is "
                             f"different from expected {self._features.device}")
        if features.shape != self._features.shape:
            raise ValueError(f"The new features has shape {features.shape} which is different "
                             f"from expected {self._features.shape}")
        self._features = features

    @property
    def C(self) -> torch.Tensor:
        return self._coordinates

    @property
    def stride(self):
        return self._stride

    @property
    def batch_dims(self):
        return self._batch_dims

    @property
    def batch_size(self) -> int:
        return 1 if self._batch_dims is None else len(self._batch_dims) - 1

    @property
    def device(self):
        return self._coordinates.device

    @property
    def dtype(self):
        return self._features.dtype

    @property
    def shape(self):
        return self._features.shape

    @property
    def num_features(self) -> int:
        return self._features.shape[1]

    @property
    def ndim(self) -> int:
        return self._coordinates.shape[1]

    @property
    def n(self) -> int:
        return self._coordinates.shape[0]

    @property
    def requires_grad(self):
        return self._features.requires_grad

    @requires_grad.setter
    def requires_grad(self, value: bool):
        self._features.requires_grad = value

    # -- conversions ------------------------------------------------------------
    def _like(self, features, coordinates=None, batch_dims="same"):
        return SparseTensor(features,
                            self._coordinates if coordinates is None else coordinates,
                            stride=self._stride,
                            batch_dims=self._batch_dims if batch_dims == "same" else batch_dims)

    def clone(self):
        bd = None if self._batch_dims is None else self._batch_dims.clone()
        return self._like(self._features.clone(), self._coordinates.clone(), bd)

    def to(self, device=None, dtype=None, non_blocking: bool = False, copy: bool = False):
        """Move coordinates and features; ``dtype`` applies to the features only.
        With ``copy=False`` the tensor is updated in place and returned, as in
        the reference (minuet/tensors.py:180-204)."""
        kw = dict(device=device, non_blocking=non_blocking, copy=copy)
        coordinates = self._coordinates.to(**kw)
        features = self._features.to(dtype=dtype, **kw)
        if copy:
            bd = None if self._batch_dims is None else self._batch_dims.to(**kw)
            return self._like(features, coordinates, bd)
        self._coordinates, self._features = coordinates, features
        return self

    def cuda(self, device=None, non_blocking: bool = False):
        kw = dict(device=device, non_blocking=non_blocking)
        self._coordinates = self._coordinates.cuda(**kw)
        self._features = self._features.cuda(**kw)
        if self._batch_dims is not None:
            self._batch_dims = self._batch_dims.cuda(**kw)
        return self

    def cpu(self):
        self._coordinates = self._coordinates.cpu()
        self._features = self._features.cpu()
        if self._batch_dims is not None:
            self._batch_dims = self._batch_dims.cpu()
        return self

    def contiguous(self):
        self._coordinates = self._coordinates.contiguous()
        self._features = self._features.contiguous()
        if self._batch_dims is not None:
            self._batch_dims = self._batch_dims.contiguous()
        return self

    def half(self):
        return self._like(self._features.half())

    def detach(self):
        return self._like(self._features.detach())

    def detach_(self):
        self._features = self._features.detach_()
        return self

    def backward(self, **kwargs):
        return self._features.backward(**kwargs)

    def __repr__(self):
        return (f"SparseTensor(n={self.n}, channels={self.num_features}, stride={self._stride}, "
                f"batch_size={self.batch_size}, dtype={self.dtype}, device={self.device})")
