"""Gather - GEMM - Scatter on the GPU against the CPU oracle.

Tolerances: fp32 within 1e-5 relative (of the output scale); fp16 element-wise
|got - want| <= 1e-2 * |want| + 1e-3 against an fp64-accumulated computation on
the same rounded inputs (bf16 keeps 8 mantissa bits against fp16's 11, so its
bounds are eight times wider; the reference has no bf16 path to compare with).
"""
import numpy as np
import pytest
import torch

import minuet_b200 as minuet
from minuet_b200 import synth
from minuet_b200.nn import functional as F
from minuet_b200.utils.helpers import generate_kernel_offsets

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a, dtype=None):
    return torch.as_tensor(np.ascontiguousarray(a), dtype=dtype, device=DEV)


def assert_close(got, want, dtype):
    got = got.detach().float().cpu().numpy()
    scale = max(float(np.abs(want).max()), 1e-6)
    if dtype == torch.float32:
        assert np.abs(got - want).max() <= 1e-5 * scale, np.abs(got - want).max() / scale
    else:
        # fp16: 1e-2 relative / 1e-3 absolute, element-wise; bf16 keeps 8 mantissa
        # bits against 11, so its bounds are 8x wider
        k = 1.0 if dtype == torch.float16 else 8.0
        np.testing.assert_allclose(got, want, rtol=k * 1e-2, atol=k * 1e-3)


def run_layer(oracle_lib, src, sbd, c_in, c_out, kernel, stride, dtype, seed=0, tiles=(1, 1),
              threshold=-1, transposed_check=False):
    rng = np.random.default_rng(seed)
    ksize = int(np.prod(np.broadcast_to(kernel, 3)))
    x = rng.standard_normal((len(src), c_in)).astype(np.float32)
    w = synth.kaiming_normal((ksize, c_in, c_out), seed + 1)
    xt, wt = dev(x).to(dtype), dev(w).to(dtype)
    x_r, w_r = xt.float().cpu().numpy(), wt.float().cpu().numpy()   # rounded inputs
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=DEV)
    conv = minuet.nn.SparseConv3d(c_in, c_out, kernel, stride=stride, dtype=dtype, device=DEV)
    conv.kernel.data.copy_(wt)
    conv.tunable_config.update(gather_tile_size=tiles[0], scatter_tile_size=tiles[1],
                               threshold=threshold)
    minuet.set_kernel_map_cache(conv, cache)
    inp = minuet.SparseTensor(xt, dev(src), batch_dims=None if sbd is None else dev(sbd))
    out = conv(inp)
    off = generate_kernel_offsets(3, kernel, 1, 1).astype(np.int32)
    if stride == 1:
        tgt, tbd = src, sbd
    else:
        tgt, tbd = oracle_lib.downsample(src, stride, sbd)
    m = oracle_lib.build_kernel_map(src, tgt, off, sbd, tbd)
    want = oracle_lib.conv_forward(x_r, w_r, m["source_masks"], m["target_masks"], m["order"],
                                   acc64=True)
    assert out.F.dtype == dtype and out.F.shape == (len(tgt), c_out)
    assert np.array_equal(out.C.cpu().numpy(), tgt)
    assert_close(out.F, want, dtype)
    return conv, cache, inp, out, want


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("c_in,c_out", [(32, 32), (3, 16), (4, 20), (16, 64), (96, 48)])
def test_submanifold_layer(oracle_lib, dtype, c_in, c_out):
    rng = np.random.default_rng(1)
    src, sbd = synth.random_small_batch(rng, 2, 4000, 24)
    run_layer(oracle_lib, src, sbd, c_in, c_out, 3, 1, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("kernel,stride", [(2, 2), (3, 2), (2, 1)])
def test_strided_layer(oracle_lib, dtype, kernel, stride):
    rng = np.random.default_rng(2)
    src, sbd = synth.random_small_batch(rng, 3, 3000, 30, low=-9)
    run_layer(oracle_lib, src, sbd, 16, 32, kernel, stride, dtype)


@pytest.mark.parametrize("tiles", [(2, 2), (4, 8), (16, 16), (32, 32)])
def test_tile_sizes_and_threshold_do_not_change_results(oracle_lib, tiles):
    rng = np.random.default_rng(3)
    src, _ = synth.random_small_batch(rng, 1, 5000, 20)
    for threshold in (-1, 0.3, None):
        run_layer(oracle_lib, src, None, 32, 32, 3, 1, torch.float16, tiles=tiles,
                  threshold=threshold)


def test_transposed_layer_and_bias(oracle_lib):
    rng = np.random.default_rng(4)
    src, sbd = synth.random_small_batch(rng, 2, 3000, 26)
    conv, cache, inp, down, _ = run_layer(oracle_lib, src, sbd, 8, 16, 2, 2, torch.float32)
    up = minuet.nn.SparseConv(3, 16, 8, 2, stride=2, transposed=True, bias=True, device=DEV)
    minuet.set_kernel_map_cache(up, cache)
    out = up(down)
    assert out.C is inp.C and out.stride == (1, 1, 1)
    # oracle: same map with masks swapped, weights by the same offset index
    off = generate_kernel_offsets(3, 2, 1, 1).astype(np.int32)
    tgt, tbd = oracle_lib.downsample(src, 2, sbd)
    m = oracle_lib.build_kernel_map(src, tgt, off, sbd, tbd)
    want = oracle_lib.conv_forward(down.F.float().cpu().numpy(), up.kernel.detach().cpu().numpy(),
                                   m["target_masks"], m["source_masks"], m["order"], acc64=True)
    want = want + up.bias.detach().cpu().numpy()
    assert_close(out.F, want, torch.float32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n,c_in,c_out", [(10, 8, 5), (5000, 64, 20), (3001, 96, 32), (777, 4, 20)])
def test_trivial_conv_needs_no_cache(oracle_lib, dtype, n, c_in, c_out):
    """A 1x1x1 convolution is out = F @ W[0] (minuet/nn/convolutions.py:448-454);
    the oracle computes it as a forward pass over the identity kernel map."""
    rng = np.random.default_rng(n)
    conv = minuet.nn.SparseConv3d(c_in, c_out, 1, bias=True, dtype=dtype, device=DEV)
    xt = dev(rng.standard_normal((n, c_in)).astype(np.float32)).to(dtype)
    coords = torch.arange(3 * n, dtype=torch.int32, device=DEV).view(n, 3)
    out = conv(minuet.SparseTensor(xt, coords))          # no cache set: must not be needed
    ident = np.arange(n, dtype=np.int32)[None]
    want = oracle_lib.conv_forward(xt.float().cpu().numpy(),
                                   conv.kernel.detach().float().cpu().numpy(), ident, ident,
                                   None, acc64=True)
    want = want + conv.bias.detach().float().cpu().numpy()
    assert out.F.dtype == dtype and out.F.shape == (n, c_out) and out.C is coords
    assert_close(out.F, want, dtype)
    # fused epilogue on the same layer
    scale = dev(rng.uniform(0.5, 1.5, c_out).astype(np.float32))
    shift = dev(rng.uniform(-0.3, 0.3, c_out).astype(np.float32))
    fused = conv.forward_fused(minuet.SparseTensor(xt, coords), scale=scale, shift=shift, relu=True)
    want2 = np.maximum(want * scale.cpu().numpy() + shift.cpu().numpy(), 0)
    assert_close(fused.F, want2, dtype)


def test_empty_rows_and_no_shortcut(oracle_lib):
    """A cache with reordering disabled takes the no-shortcut path; targets with
    no neighbour at all must come out as zeros."""
    src = synth.sort_unique(np.array([[0, 0, 0], [10, 10, 10], [10, 10, 11], [50, 0, 0]]))
    x = np.arange(4 * 4, dtype=np.float32).reshape(4, 4)
    w = synth.kaiming_normal((27, 4, 4), 0)
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=DEV, disable_reordering=True)
    conv = minuet.nn.SparseConv3d(4, 4, 3, device=DEV)
    conv.kernel.data.copy_(dev(w))
    minuet.set_kernel_map_cache(conv, cache)
    out = conv(minuet.SparseTensor(dev(x), dev(src)))
    off = generate_kernel_offsets(3, 3, 1, 1).astype(np.int32)
    km = oracle_lib.query(src, src, off)
    assert_close(out.F, oracle_lib.conv_bruteforce(x, w, km).astype(np.float32), torch.float32)


def test_functional_forward_with_foreign_size_tensor(oracle_lib):
    """sparse_convolution_forward on masks that did not come from the cache
    (sizes are then read back from the device)."""
    rng = np.random.default_rng(6)
    src, _ = synth.random_small_batch(rng, 1, 2000, 16)
    off = generate_kernel_offsets(3, 3, 1, 1).astype(np.int32)
    m = oracle_lib.build_kernel_map(src, src, off)
    x = rng.standard_normal((len(src), 8)).astype(np.float32)
    w = synth.kaiming_normal((27, 8, 8), 3)
    out = F.sparse_convolution_forward(
        sources=dev(x), weights=dev(w), source_masks=dev(m["source_masks"]),
        target_masks=dev(m["target_masks"]), kernel_map_order=dev(m["order"]),
        kernel_map_sizes=dev(m["sorted_sizes"]), gather_tile_size=1, scatter_tile_size=1,
        allow_shortcut_matmul=True)
    want = oracle_lib.conv_forward(x, w, m["source_masks"], m["target_masks"], m["order"], True)
    assert_close(out, want, torch.float32)
    with pytest.raises(RuntimeError):
        F.sparse_convolution_forward(
            sources=dev(x).half(), weights=dev(w), source_masks=dev(m["source_masks"]),
            target_masks=dev(m["target_masks"]), kernel_map_order=dev(m["order"]),
            kernel_map_sizes=dev(m["sorted_sizes"]), gather_tile_size=1, scatter_tile_size=1)


def test_config0_single_layer_fp32(oracle_lib):
    """50 000 uniform voxels, SparseConv3d(32, 32, 3), fp32."""
    src = synth.uniform_cloud()
    run_layer(oracle_lib, src, None, 32, 32, 3, 1, torch.float32)


@pytest.mark.parametrize("c", [16, 64, 256])
def test_outdoor_fp16_sweep_point(oracle_lib, c):
    src, sbd = synth.outdoor_batch(2, n_voxels=60_000)
    run_layer(oracle_lib, src, sbd, c, c, 3, 1, torch.float16)


def test_stage_timers_and_autotune(oracle_lib):
    rng = np.random.default_rng(8)
    src, _ = synth.random_small_batch(rng, 1, 3000, 20)
    conv, cache, inp, out, want = run_layer(oracle_lib, src, None, 16, 16, 3, 1, torch.float16)
    sm, tm, order, sizes = cache.get_kernel_map(inp.C, 1, None, inp.C, 1, None, 3, 1)
    for fn in (F.cuda_time_gather, F.cuda_time_scatter):
        assert fn(conv.kernel, sm, tm, sizes, tile_size=8, allow_shortcut_matmul=True) > 0
    assert F.cuda_time_gemm(conv.kernel, sm, tm, sizes, allow_shortcut_matmul=True) > 0
    conv.__class__.__NUM_TUNING_ROUNDS__ = 1
    try:
        minuet.autotune(conv, cache, inp)
    finally:
        conv.__class__.__NUM_TUNING_ROUNDS__ = 10
    cfg = conv.tunable_config
    assert 16 % cfg["gather_tile_size"] == 0 and 16 % cfg["scatter_tile_size"] == 0
    # a 16-bit layer: the tuner decided between pair lists and the fused kernel
    assert cfg["algorithm"] in ("explicit", "implicit") and 0 <= cfg["sub_tiles"] <= 4
    cache.reset()
    assert_close(conv(inp).F, want, torch.float16)
    # every tunable value gives the same function
    for algorithm, sub in (("explicit", 0), ("implicit", 1), ("implicit", 3), ("auto", 0)):
        conv.tunable_config.update(algorithm=algorithm, sub_tiles=sub)
        assert_close(conv(inp).F, want, torch.float16)
    # an fp32 layer tunes the reference's three keys on the gather - GEMM - scatter path
    conv32, cache32, inp32, _, want32 = run_layer(oracle_lib, src, None, 8, 8, 3, 1, torch.float32)
    conv32.__class__.__NUM_TUNING_ROUNDS__ = 1
    try:
        minuet.autotune(conv32, cache32, inp32)
    finally:
        conv32.__class__.__NUM_TUNING_ROUNDS__ = 10
    cfg = conv32.tunable_config
    assert 8 % cfg["gather_tile_size"] == 0 and 8 % cfg["scatter_tile_size"] == 0
    assert cfg["threshold"] in conv32.__AVAILABLE_THRESHOLD__ and cfg["algorithm"] == "explicit"
    cache32.reset()
    assert_close(conv32(inp32).F, want32, torch.float32)


@pytest.mark.parametrize("algorithm", ["explicit", "implicit"])
def test_frozen_weights_give_the_same_bits(oracle_lib, algorithm):
    """freeze_weights() only removes the per-call transpose: identical output bits, and a
    kernel changed afterwards is picked up by freezing again (or by un-freezing)."""
    rng = np.random.default_rng(21)
    src, sbd = synth.random_small_batch(rng, 2, 3000, 20)
    conv, cache, inp, out, want = run_layer(oracle_lib, src, sbd, 32, 64, 3, 1, torch.float16)
    conv.tunable_config.update(algorithm=algorithm)
    base = conv(inp).F.clone()
    conv.freeze_weights()
    assert conv._frozen_kernel_t.shape == (27, 64, 32)
    assert torch.equal(conv(inp).F, base)
    with torch.no_grad():
        conv.kernel.mul_(2.0)
    assert torch.equal(conv(inp).F, base)                    # still the frozen copy
    conv.freeze_weights()
    doubled = conv(inp).F
    conv.freeze_weights(False)
    assert torch.equal(conv(inp).F, doubled)
    assert_close(doubled, 2.0 * want, torch.float16)
    conv.freeze_weights()
    conv.half()                                               # moving / casting drops the copy
    assert conv._frozen_kernel_t is None
    # 1x1x1 convolution
    head = minuet.nn.SparseConv3d(32, 20, 1, dtype=torch.float16, device=DEV)
    y = head(inp).F.clone()
    head.freeze_weights()
    assert torch.equal(head(inp).F, y)


@pytest.mark.needs_grad
@pytest.mark.parametrize("stride,kernel", [(1, 3), (2, 2)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_backward_matches_autograd_of_the_pairwise_sum(oracle_lib, stride, kernel, dtype):
    """Gradients of a layer (and of the transposed layer that shares its map) against
    autograd on the same function written with torch index operations over the oracle's
    kernel map, in float64."""
    rng = np.random.default_rng(41)
    src, sbd = synth.random_small_batch(rng, 2, 1500, 16)
    c_in, c_out = 8, 16
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=DEV)
    conv = minuet.nn.SparseConv3d(c_in, c_out, kernel, stride=stride, bias=True, dtype=dtype, device=DEV)
    back = minuet.nn.SparseConv(3, c_out, c_in, kernel, stride=stride, transposed=True, dtype=dtype,
                                device=DEV)
    minuet.set_kernel_map_cache(conv, cache)
    minuet.set_kernel_map_cache(back, cache)
    x = torch.as_tensor(rng.standard_normal((len(src), c_in)), device=DEV).to(dtype).requires_grad_()
    inp = minuet.SparseTensor(x, dev(src), batch_dims=dev(sbd))
    mid = conv(inp)
    out = back(mid) if stride > 1 else mid
    g = torch.as_tensor(rng.standard_normal(tuple(out.F.shape)), device=DEV).to(dtype)
    (out.F * g).sum().backward()

    # the same function with torch ops, float64
    off = generate_kernel_offsets(3, kernel, 1, 1).astype(np.int32)
    tgt, tbd = (src, sbd) if stride == 1 else oracle_lib.downsample(src, stride, sbd)
    km = oracle_lib.build_kernel_map(src, tgt, off, sbd, tbd)["kernel_map"]    # [O, T] -> source row
    x64 = x.detach().double().requires_grad_()
    w64 = conv.kernel.detach().double().requires_grad_()
    b64 = conv.bias.detach().double().requires_grad_()
    wb64 = back.kernel.detach().double().requires_grad_()
    y = torch.zeros((len(tgt), c_out), dtype=torch.float64, device=DEV)
    z = torch.zeros((len(src), c_in), dtype=torch.float64, device=DEV)
    pairs = []
    for o in range(len(off)):
        t_rows = torch.as_tensor(np.nonzero(km[o] >= 0)[0], device=DEV)
        s_rows = torch.as_tensor(km[o][km[o] >= 0].astype(np.int64), device=DEV)
        pairs.append((s_rows, t_rows))
        y = y.index_add(0, t_rows, x64[s_rows] @ w64[o])
    y = y + b64
    if stride > 1:
        for o, (s_rows, t_rows) in enumerate(pairs):       # transposed: coarse -> fine
            z = z.index_add(0, s_rows, y[t_rows] @ wb64[o])
        ref = z
    else:
        ref = y
    (ref * g.double()).sum().backward()
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    def close(got, want):
        scale = float(want.abs().max()) + 1e-12
        assert float((got.double() - want).abs().max()) <= tol * scale
    close(out.F.detach(), ref.detach())
    close(x.grad, x64.grad)
    close(conv.kernel.grad, w64.grad)
    close(conv.bias.grad, b64.grad)
    if stride > 1:
        close(back.kernel.grad, wb64.grad)


def test_neighbor_table_sorted_by_hit_word(oracle_lib):
    """Kernel maps from the fused build carry hit words: the table's rows are then the
    targets in stable order of their hit word, nbr / tile_bits are in that order, and the
    fused forward gives the same function with and without the reordering."""
    from minuet_b200 import engine
    from minuet_b200.nn.functional import convolution as conv_mod
    rng = np.random.default_rng(31)
    src, sbd = synth.random_small_batch(rng, 2, 6000, 30)
    conv, cache, inp, out, want = run_layer(oracle_lib, src, sbd, 32, 32, 3, 1, torch.float16)
    sm, tm, order, sizes = cache.get_kernel_map(inp.C, 1, inp.batch_dims, inp.C, 1, inp.batch_dims, 3, 1)
    hs = engine.host_copy(sizes)
    nbr, tile_bits, perm = engine.neighbor_table(sm, tm, hs)
    nat, nat_bits, none = engine.neighbor_table(sm, tm, hs, reorder=False)
    assert none is None and perm is not None
    words = engine.hit_bits(tm).cpu().numpy().astype(np.uint32)
    p = perm.cpu().numpy()
    assert np.array_equal(np.sort(p), np.arange(len(src)))
    rev = np.array([int(format(int(w), "027b")[::-1], 2) for w in words], dtype=np.int64)
    for shift in (1, 2, 4, 8, 16):      # rank of the reversed word in the reflected Gray sequence
        rev ^= rev >> shift
    assert np.array_equal(p, np.argsort(rev, kind="stable"))     # rare offsets = high key bits
    # only the (tile, offset) blocks whose tile bit is set are written; the others have no pair
    got, ref, tb = nbr.cpu().numpy(), nat.cpu().numpy()[:, p], tile_bits.cpu().numpy()
    for tile in range(len(tb)):
        rows = slice(tile * 128, (tile + 1) * 128)
        for o in range(27):
            if (int(tb[tile]) >> o) & 1:
                assert np.array_equal(got[o, rows], ref[o, rows])
            else:
                assert (ref[o, rows] == -1).all()
    # fewer (tile, offset) stages than in the targets' own order
    count = lambda b: int(sum(bin(int(v) & 0xffffffff).count("1") for v in b.cpu().numpy()))
    assert count(tile_bits) < count(nat_bits)
    conv.tunable_config.update(algorithm="implicit")
    scale = torch.rand(32, device=DEV) + 0.5
    res = torch.randn(len(src), 32, device=DEV).half()
    outs = []
    for flag in (True, False):
        conv_mod.REORDER_ROWS = flag
        try:
            outs.append(conv.forward_fused(inp, scale=scale, residual=res, relu=True).F)
        finally:
            conv_mod.REORDER_ROWS = True
    assert torch.equal(outs[0], outs[1])      # same sums in the same order, other rows per tile
    assert_close(conv(inp).F, want, torch.float16)


def test_neighbor_table_matches_kernel_map(oracle_lib):
    """mn_build_neighbor_table turns masks back into the (mask-row ordered) kernel
    map and marks, per 128-target tile, the offsets that have any pair."""
    from minuet_b200 import engine
    rng = np.random.default_rng(12)
    src, sbd = synth.random_small_batch(rng, 2, 3000, 20)
    tgt, tbd = oracle_lib.downsample(src, 2, sbd)
    for kernel, s_, t_, sb, tb in ((3, src, src, sbd, sbd), (2, src, tgt, sbd, tbd)):
        off = generate_kernel_offsets(3, kernel, 1, 1).astype(np.int32)
        m = oracle_lib.build_kernel_map(s_, t_, off, sb, tb)
        sm, tm = dev(m["source_masks"]), dev(m["target_masks"])
        nbr, bits, perm = engine.neighbor_table(sm, tm, m["sorted_sizes"])
        assert perm is None          # masks that did not come with hit words keep their order
        want = m["kernel_map"][m["order"]]
        assert np.array_equal(nbr.cpu().numpy(), want)
        T = len(t_)
        got_bits = bits.cpu().numpy().astype(np.uint32)
        for tile in range((T + 127) // 128):
            rows = want[:, tile * 128:(tile + 1) * 128]
            expect = sum(1 << p for p in range(len(off)) if (rows[p] >= 0).any())
            assert int(got_bits[tile]) == expect


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_apply_epilogue(dtype):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((1000, 24)).astype(np.float32)
    res = rng.standard_normal((1000, 24)).astype(np.float32)
    scale = rng.uniform(0.5, 2, 24).astype(np.float32)
    shift = rng.uniform(-1, 1, 24).astype(np.float32)
    xt, rt = dev(x).to(dtype), dev(res).to(dtype)
    want = np.maximum(xt.float().cpu().numpy() * scale + shift + rt.float().cpu().numpy(), 0)
    F.apply_epilogue(xt, dev(scale), dev(shift), rt, relu=True)
    tol = 1e-6 if dtype == torch.float32 else (1e-2 if dtype == torch.float16 else 4e-2)
    np.testing.assert_allclose(xt.float().cpu().numpy(), want, rtol=tol, atol=tol)


@pytest.mark.parametrize("algorithm", ["explicit", "implicit"])
@pytest.mark.parametrize("kernel,stride,c_in,c_out", [(3, 1, 64, 64), (2, 2, 32, 64), (3, 2, 16, 8),
                                                      (3, 1, 8, 256), (3, 1, 136, 24)])
def test_both_algorithms(oracle_lib, algorithm, kernel, stride, c_in, c_out):
    from minuet_b200.nn.functional import convolution as conv_mod
    rng = np.random.default_rng(5)
    src, sbd = synth.random_small_batch(rng, 2, 3500, 18)
    old = conv_mod.ALGORITHM
    conv_mod.ALGORITHM = algorithm
    try:
        run_layer(oracle_lib, src, sbd, c_in, c_out, kernel, stride, torch.float16)
    finally:
        conv_mod.ALGORITHM = old


def _dense_batch(seed, clouds=2, draws=50_000, extent=72):
    rng = np.random.default_rng(seed)
    return synth.random_small_batch(rng, clouds, draws, extent)


@pytest.mark.parametrize("algorithm", ["implicit", "explicit"])
@pytest.mark.parametrize("c_in,c_out", [(64, 64), (128, 256), (32, 128)])
def test_benchmark_size_tiles_with_full_epilogue(oracle_lib, algorithm, c_in, c_out):
    """More than 75 776 targets, so that the fused kernel runs with two 128-row
    sub-tiles per CTA tile, once with two accumulator sets in TMEM (C_out = 64,
    128) and once with one (C_out = 256); scale + shift + residual + ReLU applied;
    the same inputs through gather - GEMM - scatter."""
    from minuet_b200.nn.functional import convolution as conv_mod
    coords, bd = _dense_batch(21)
    assert len(coords) >= 76_000
    rng = np.random.default_rng(22)
    x = rng.standard_normal((len(coords), c_in)).astype(np.float32)
    res = rng.standard_normal((len(coords), c_out)).astype(np.float32)
    scale = rng.uniform(0.5, 1.5, c_out).astype(np.float32)
    shift = rng.uniform(-0.3, 0.3, c_out).astype(np.float32)
    w = synth.kaiming_normal((27, c_in, c_out), 23)
    conv = minuet.nn.SparseConv3d(c_in, c_out, 3, dtype=torch.float16, device=DEV)
    conv.kernel.data.copy_(dev(w).half())
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=DEV)
    minuet.set_kernel_map_cache(conv, cache)
    xt, rt = dev(x).half(), dev(res).half()
    inp = minuet.SparseTensor(xt, dev(coords), batch_dims=dev(bd))
    old = conv_mod.ALGORITHM
    conv_mod.ALGORITHM = algorithm
    try:
        out = conv.forward_fused(inp, scale=dev(scale), shift=dev(shift), residual=rt, relu=True)
        plain = conv(inp)
    finally:
        conv_mod.ALGORITHM = old
    off = generate_kernel_offsets(3, 3, 1, 1).astype(np.int32)
    m = oracle_lib.build_kernel_map(coords, coords, off, bd, bd)
    ref = oracle_lib.conv_forward(xt.float().cpu().numpy(), conv.kernel.detach().float().cpu().numpy(),
                                  m["source_masks"], m["target_masks"], m["order"], acc64=True)
    assert_close(plain.F, ref, torch.float16)
    ref = np.maximum(ref * scale + shift + rt.float().cpu().numpy(), 0)
    assert_close(out.F, ref, torch.float16)
