"""Sparse UNet end to end on the GPU against a layer-by-layer oracle forward
(CPU oracle convolutions + numpy BatchNorm/ReLU/concat).  fp32 within 1e-4 of
the output scale (about forty chained layers), fp16 within 2e-2."""
import numpy as np
import pytest
import torch

import minuet_b200 as minuet
from minuet_b200 import synth
from minuet_b200.unet import ConvBlock, ResidualBlock, SparseUNet
from minuet_b200.utils.helpers import generate_kernel_offsets
from oracle.net import OracleNet

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.float16, 2e-2)])
def test_small_unet_matches_oracle(oracle_lib, dtype, tol):
    torch.manual_seed(0)
    rng = np.random.default_rng(0)
    coords, bd = synth.random_small_batch(rng, 2, 3000, 40)
    feats = rng.random((len(coords), 3)).astype(np.float32)
    net = SparseUNet(3, num_classes=5, channels=(8, 16, 32), stem_channels=8).to(DEV).eval()
    for m in net.modules():      # non-trivial BatchNorm statistics
        if isinstance(m, minuet.nn.BatchNorm):
            m.running_mean.uniform_(-0.2, 0.2)
            m.running_var.uniform_(0.5, 1.5)
            m.weight.data.uniform_(0.5, 1.5)
            m.bias.data.uniform_(-0.2, 0.2)
    net = net.to(dtype)
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=DEV)
    minuet.set_kernel_map_cache(net, cache)
    x = minuet.SparseTensor(torch.as_tensor(feats, device=DEV).to(dtype),
                            torch.as_tensor(coords, device=DEV),
                            batch_dims=torch.as_tensor(bd, device=DEV))
    with torch.no_grad():
        out = net(x)
    assert out.F.shape == (len(coords), 5) and out.C is x.C and out.stride == (1, 1, 1)
    rt = None if dtype == torch.float32 else dtype
    o = OracleNet(oracle_lib, round_to=rt)
    f0 = feats if rt is None else torch.from_numpy(feats).to(rt).float().numpy()
    want = o.forward(net, (f0, coords, 1, bd))[0]
    got = out.F.float().cpu().numpy()
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= tol * scale, np.abs(got - want).max() / scale
    # second pass on a reset cache gives identical bits (deterministic summation order)
    cache.reset()
    with torch.no_grad():
        again = net(x)
    assert torch.equal(again.F, out.F)
    # BatchNorm / ReLU / residual folded into the convolution epilogues: same function
    net.fuse()
    cache.reset()
    with torch.no_grad():
        fused = net(x)
    got = fused.F.float().cpu().numpy()
    assert np.abs(got - want).max() <= tol * scale, np.abs(got - want).max() / scale


@pytest.mark.parametrize("algorithm", ["explicit", "implicit"])
def test_fused_epilogue_both_algorithms(oracle_lib, algorithm):
    from minuet_b200.nn import functional as F
    from minuet_b200.nn.functional import convolution as conv_mod
    rng = np.random.default_rng(3)
    coords, bd = synth.random_small_batch(rng, 2, 4000, 22)
    c_in, c_out = 32, 48
    x = rng.standard_normal((len(coords), c_in)).astype(np.float32)
    res = rng.standard_normal((len(coords), c_out)).astype(np.float32)
    scale = rng.uniform(0.5, 1.5, c_out).astype(np.float32)
    shift = rng.uniform(-0.3, 0.3, c_out).astype(np.float32)
    conv = minuet.nn.SparseConv3d(c_in, c_out, 3, bias=True, dtype=torch.float16, device=DEV)
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=DEV)
    minuet.set_kernel_map_cache(conv, cache)
    xt = torch.as_tensor(x, device=DEV).half()
    rt = torch.as_tensor(res, device=DEV).half()
    inp = minuet.SparseTensor(xt, torch.as_tensor(coords, device=DEV),
                              batch_dims=torch.as_tensor(bd, device=DEV))
    old = conv_mod.ALGORITHM
    conv_mod.ALGORITHM = algorithm
    try:
        out = conv.forward_fused(inp, scale=torch.as_tensor(scale, device=DEV),
                                 shift=torch.as_tensor(shift, device=DEV), residual=rt, relu=True)
    finally:
        conv_mod.ALGORITHM = old
    off = generate_kernel_offsets(3, 3, 1, 1).astype(np.int32)
    m = oracle_lib.build_kernel_map(coords, coords, off, bd, bd)
    ref = oracle_lib.conv_forward(xt.float().cpu().numpy(), conv.kernel.detach().float().cpu().numpy(),
                                  m["source_masks"], m["target_masks"], m["order"], acc64=True)
    ref = (ref + conv.bias.detach().float().cpu().numpy()) * scale + shift + rt.float().cpu().numpy()
    ref = np.maximum(ref, 0)
    got = out.F.float().cpu().numpy()
    np.testing.assert_allclose(got, ref, rtol=1e-2, atol=1e-3)


def _randomise_batchnorm(net):
    for m in net.modules():
        if isinstance(m, minuet.nn.BatchNorm):
            m.running_mean.uniform_(-0.2, 0.2)
            m.running_var.uniform_(0.5, 1.5)
            m.weight.data.uniform_(0.5, 1.5)
            m.bias.data.uniform_(-0.2, 0.2)


@pytest.mark.parametrize("scene", ["outdoor120k", "indoor200k"])
def test_full_width_unet_matches_oracle(oracle_lib, scene):
    """The benchmark network itself (stem 32, encoder 32/64/128/256, decoder with
    the 256->128 / 128->64 / 64->32 concatenation layers, 20 classes), fp16, on one
    cloud of each benchmark geometry, unfused and fused, with every layer forced
    through the fused implicit-GEMM kernel and through gather - GEMM - scatter."""
    from minuet_b200.nn.functional import convolution as conv_mod
    torch.manual_seed(1)
    rng = np.random.default_rng(1)
    if scene == "outdoor120k":
        coords = synth.outdoor_cloud(3000, 120_000)
        feats = np.concatenate([coords.astype(np.float32) * 0.05,
                                rng.random((len(coords), 1), dtype=np.float32)], axis=1)
    else:
        coords = synth.indoor_cloud(2000, 200_000)
        feats = rng.random((len(coords), 3), dtype=np.float32)
    net = SparseUNet(feats.shape[1], num_classes=20).to(DEV).eval()
    _randomise_batchnorm(net)
    net = net.half()
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=DEV)
    minuet.set_kernel_map_cache(net, cache)
    x = minuet.SparseTensor(torch.as_tensor(feats, device=DEV).half(),
                            torch.as_tensor(coords, device=DEV))
    o = OracleNet(oracle_lib, round_to=torch.float16)
    f0 = torch.from_numpy(feats).half().float().numpy()
    want = o.forward(net, (f0, coords, 1, None))[0]
    scale = np.abs(want).max()
    old = conv_mod.ALGORITHM
    try:
        for algorithm in ("implicit", "explicit"):
            conv_mod.ALGORITHM = algorithm
            for fused in (False, True):
                if fused:
                    net.fuse()
                cache.reset()
                with torch.no_grad():
                    out = net(x)
                got = out.F.float().cpu().numpy()
                assert got.shape == (len(coords), 20)
                err = np.abs(got - want).max() / scale
                assert err <= 2e-2, (algorithm, fused, err)
            for m in net.modules():      # back to the unfused modules for the next algorithm
                if isinstance(m, (ConvBlock, ResidualBlock)):
                    m.folded = None
    finally:
        conv_mod.ALGORITHM = old


def test_status_word_is_reported_on_the_forward_path():
    """A timed-out tensor-core kernel sets bit 2 of the device status word.  The
    bit is written here from the host (no kernel is made to time out); the next
    forward passes must raise the matching error, not the key-box one."""
    from minuet_b200 import engine
    torch.manual_seed(0)
    rng = np.random.default_rng(0)
    coords, bd = synth.random_small_batch(rng, 1, 2000, 24)
    net = SparseUNet(3, num_classes=4, channels=(8, 16), stem_channels=8).to(DEV).half().eval()
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=DEV)
    minuet.set_kernel_map_cache(net, cache)
    x = minuet.SparseTensor(torch.rand(len(coords), 3, device=DEV).half(),
                            torch.as_tensor(coords, device=DEV))
    with torch.no_grad():
        net(x)
    torch.cuda.synchronize()
    engine.check_status(DEV)                      # clean
    engine.status_word(DEV).fill_(engine.STATUS_TC_TIMEOUT)
    with pytest.raises(RuntimeError, match="tensor-core"):
        for _ in range(3):                        # asynchronous: at the latest one pass later
            cache.reset()
            with torch.no_grad():
                net(x)
            torch.cuda.synchronize()
    assert int(engine.status_word(DEV).item()) == 0
    engine.status_word(DEV).fill_(engine.STATUS_KEY_BOX)
    with pytest.raises(RuntimeError, match="bounding box"):
        engine.check_status(DEV)


@pytest.mark.needs_grad
def test_small_unet_trains_one_step():
    """The whole network is differentiable: a training step on a small batch changes the
    loss and leaves finite gradients on every parameter."""
    torch.manual_seed(1)
    rng = np.random.default_rng(7)
    coords, bd = synth.random_small_batch(rng, 2, 2000, 30)
    feats = torch.as_tensor(rng.random((len(coords), 3)).astype(np.float32), device=DEV)
    labels = torch.as_tensor(rng.integers(0, 5, len(coords)), device=DEV)
    net = SparseUNet(3, num_classes=5, channels=(8, 16), stem_channels=8).to(DEV).train()
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=DEV)
    minuet.set_kernel_map_cache(net, cache)
    opt = torch.optim.SGD(net.parameters(), lr=0.05)
    x = minuet.SparseTensor(feats, torch.as_tensor(coords, device=DEV),
                            batch_dims=torch.as_tensor(bd, device=DEV))
    losses = []
    for _ in range(3):
        cache.reset()
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(net(x).F, labels)
        loss.backward()
        for name, p in net.named_parameters():
            assert p.grad is not None and torch.isfinite(p.grad).all(), name
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0]
