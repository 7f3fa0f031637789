"""Sparse UNet built from the path's own modules (SparseConv3d / SparseConv,
BatchNorm, ReLU, cat).  The reference ships no model zoo; this is the network of
the end-to-end benchmark configurations:

  stem 3^3 conv -> 32 channels;
  4 encoder stages (2^3 stride-2 conv + 2 residual blocks of 3^3 convs) with
  32 / 64 / 128 / 256 channels;
  4 decoder stages (2^3 stride-2 transposed conv, skip concatenation, 2 residual
  blocks); 1x1x1 head to the class logits.
"""
from typing import Sequence

import torch
from torch import nn

from minuet_b200 import engine
from minuet_b200.nn import BatchNorm, ReLU, SparseConv, SparseConv3d, fold_batchnorm
from minuet_b200.nn import functional as F
from minuet_b200.tensors import SparseTensor


class ConvBlock(nn.Sequential):
    """conv - BatchNorm - ReLU.  After :meth:`SparseUNet.fuse` (eval mode only) the
    BatchNorm and ReLU run as the convolution's epilogue instead of as separate
    passes over the feature matrix."""

    def __init__(self, c_in: int, c_out: int, kernel_size: int, stride: int = 1,
                 transposed: bool = False):
        if transposed:
            conv = SparseConv(3, c_in, c_out, kernel_size, stride=stride, transposed=True)
        else:
            conv = SparseConv3d(c_in, c_out, kernel_size, stride=stride)
        super().__init__(conv, BatchNorm(c_out), ReLU(inplace=True))
        self.folded = None

    def forward(self, x: SparseTensor) -> SparseTensor:
        if self.folded is None or self.training:
            return super().forward(x)
        scale, shift = self.folded
        return self[0].forward_fused(x, scale=scale, shift=shift, relu=True)


class ResidualBlock(nn.Module):
    """conv3-BN-ReLU-conv3-BN plus the (projected) input, then ReLU."""

    def __init__(self, c_in: int, c_out: int):
        super().__init__()
        self.body = nn.Sequential(SparseConv3d(c_in, c_out, 3), BatchNorm(c_out),
                                  ReLU(inplace=True), SparseConv3d(c_out, c_out, 3),
                                  BatchNorm(c_out))
        self.project = None
        if c_in != c_out:
            self.project = nn.Sequential(SparseConv3d(c_in, c_out, 1), BatchNorm(c_out))
        self.relu = ReLU(inplace=True)
        self.folded = None

    def forward(self, x: SparseTensor) -> SparseTensor:
        if self.folded is not None and not self.training:
            (s1, b1), (s2, b2), proj = self.folded
            y = self.body[0].forward_fused(x, scale=s1, shift=b1, relu=True)
            if self.project is None:
                skip = x.F
            else:
                skip = self.project[0].forward_fused(x, scale=proj[0], shift=proj[1]).F
            return self.body[3].forward_fused(y, scale=s2, shift=b2, residual=skip, relu=True)
        y = self.body(x)
        skip = x if self.project is None else self.project(x)
        out = SparseTensor(y.F + skip.F, y.C, stride=y.stride, batch_dims=y.batch_dims)
        return self.relu(out)


class SparseUNet(nn.Module):
    def __init__(self, in_channels: int, num_classes: int = 20,
                 channels: Sequence[int] = (32, 64, 128, 256), stem_channels: int = 32):
        super().__init__()
        self.stem = ConvBlock(in_channels, stem_channels, 3)
        self.down = nn.ModuleList()
        self.enc = nn.ModuleList()
        prev = stem_channels
        for c in channels:
            self.down.append(ConvBlock(prev, c, 2, stride=2))
            self.enc.append(nn.Sequential(ResidualBlock(c, c), ResidualBlock(c, c)))
            prev = c
        skips = [stem_channels, *channels[:-1]]
        self.up = nn.ModuleList()
        self.dec = nn.ModuleList()
        for skip_c in reversed(skips):
            self.up.append(ConvBlock(prev, skip_c, 2, stride=2, transposed=True))
            self.dec.append(nn.Sequential(ResidualBlock(2 * skip_c, skip_c),
                                          ResidualBlock(skip_c, skip_c)))
            prev = skip_c
        self.head = SparseConv3d(prev, num_classes, 1)

    def fuse(self):
        """Fold every eval-mode BatchNorm into a per-channel scale/shift and run it,
        the residual add and the ReLU as convolution epilogues.  Call after
        ``eval()`` and after the final dtype/device of the model is set; ``train()``
        switches back to the unfused modules.  The convolution kernels are also frozen
        in the layout the tensor-core kernels read (SparseConv.freeze_weights)."""
        for m in self.modules():
            if isinstance(m, ConvBlock):
                m.folded = fold_batchnorm(m[1])
            elif isinstance(m, ResidualBlock):
                proj = None if m.project is None else fold_batchnorm(m.project[1])
                m.folded = (fold_batchnorm(m.body[1]), fold_batchnorm(m.body[4]), proj)
            elif isinstance(m, SparseConv) and m.kernel.is_cuda:
                m.freeze_weights()      # the weights of a fused model no longer change
        return self

    def plan(self, x: SparseTensor):
        """Coordinates of every stride level and all nine kernel maps of the network,
        built up front: the four blocking reads (one unique count per level) and the
        copies of the per-offset pair counts are then over before the first feature
        kernel is queued, and the forward pass below runs without a host wait."""
        c, s, bd = x.C, x.stride, x.batch_dims
        self.stem[0].prepare(c, s, bd)
        for down, enc in zip(self.down, self.enc):
            c, s, bd = down[0].prepare(c, s, bd)
            enc[0].body[0].prepare(c, s, bd)

    def forward(self, x: SparseTensor) -> SparseTensor:
        if x.F.is_cuda and self.stem[0]._kernel_map_cache is not None:
            self.plan(x)
        x = self.stem(x)
        skips = []
        for down, enc in zip(self.down, self.enc):
            skips.append(x)
            x = enc(down(x))
        for up, dec in zip(self.up, self.dec):
            x = up(x)
            x = dec(F.cat([x, skips.pop()]))
        out = self.head(x)
        if out.F.is_cuda:
            engine.poll_status(out.F.device)   # device-side errors of this pass (no sync)
        return out
