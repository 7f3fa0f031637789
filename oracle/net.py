"""Layer-by-layer CPU forward of a sparse UNet built from minuet_b200 modules
(test infrastructure: only the tests and the benchmark's CPU-baseline leg use it).

Mirrors ``SparseUNet.forward`` with numpy tensors ``(features, coords, stride,
batch_dims)``: convolutions go through the C++ oracle (kernel map + forward pass
with fp64 accumulation), BatchNorm / ReLU / concatenation / residual adds are
numpy.  ``round_to`` rounds every layer output to that torch dtype, as the GPU
pipeline does when it stores 16-bit features.
"""
import numpy as np
import torch

import minuet_b200 as minuet
from minuet_b200.unet import ConvBlock, ResidualBlock, SparseUNet
from minuet_b200.utils.helpers import generate_kernel_offsets


class OracleNet:
    """See the module docstring.  ``pairs`` counts the (source, target) pairs of every
    non-trivial convolution that ran (work done, for throughput reports)."""

    def __init__(self, oracle, round_to=None):
        self.oracle = oracle
        self.levels = {}      # stride -> (coords, batch_dims)
        self.maps = {}
        self.round_to = round_to
        self.pairs = 0

    def _rt(self, x):
        if self.round_to is None:
            return x.astype(np.float32)
        return torch.from_numpy(x.astype(np.float32)).to(self.round_to).float().numpy()

    def conv(self, m, x):
        f, coords, stride, bd = x
        w = self._rt(m.kernel.detach().float().cpu().numpy())
        k = m.kernel_size[0]
        if m.is_trivial:
            return self._rt(f @ w[0]), coords, stride, bd
        self.levels.setdefault(stride, (coords, bd))
        s = m.stride[0]
        if m.transposed:
            tstride = stride // s
            tcoords, tbd = self.levels[tstride]
            key = (tstride, stride, k)
            mp = self.maps[key]
            sm, tm = mp["target_masks"], mp["source_masks"]
        else:
            tstride = stride * s
            if tstride not in self.levels:
                self.levels[tstride] = self.oracle.downsample(coords, tstride, bd)
            tcoords, tbd = self.levels[tstride]
            key = (stride, tstride, k)
            if key not in self.maps:
                off = generate_kernel_offsets(3, k, stride, 1).astype(np.int32)
                self.maps[key] = self.oracle.build_kernel_map(coords, tcoords, off, bd, tbd)
            mp = self.maps[key]
            sm, tm = mp["source_masks"], mp["target_masks"]
        self.pairs += int(mp["sizes"].sum())
        out = self.oracle.conv_forward(f, w, sm, tm, mp["order"], acc64=True)
        return self._rt(out), tcoords, tstride, tbd

    def bn(self, m, x):
        f, c, s, bd = x
        scale = (m.weight / torch.sqrt(m.running_var + m.eps)).detach().float().cpu().numpy()
        shift = (m.bias - m.running_mean * m.weight / torch.sqrt(m.running_var + m.eps))
        return self._rt(self._rt(f) * scale + shift.detach().float().cpu().numpy()), c, s, bd

    def relu(self, x):
        return (np.maximum(x[0], 0), *x[1:])

    def seq(self, mods, x):
        for m in mods:
            x = self.apply(m, x)
        return x

    def apply(self, m, x):
        if isinstance(m, ResidualBlock):
            y = self.seq(m.body, x)
            skip = x if m.project is None else self.seq(m.project, x)
            return self.relu((self._rt(y[0] + skip[0]), *y[1:]))
        if isinstance(m, (torch.nn.Sequential, ConvBlock)):
            return self.seq(m, x)
        if isinstance(m, minuet.nn.SparseConv):
            return self.conv(m, x)
        if isinstance(m, minuet.nn.BatchNorm):
            return self.bn(m, x)
        if isinstance(m, minuet.nn.ReLU):
            return self.relu(x)
        raise TypeError(type(m))

    def forward(self, net: SparseUNet, x):
        x = self.apply(net.stem, x)
        skips = []
        for down, enc in zip(net.down, net.enc):
            skips.append(x)
            x = self.apply(enc, self.apply(down, x))
        for up, dec in zip(net.up, net.dec):
            x = self.apply(up, x)
            s = skips.pop()
            x = (np.concatenate([x[0], s[0]], axis=1), *x[1:])
            x = self.apply(dec, x)
        return self.apply(net.head, x)
