"""Map step on the GPU against the CPU oracle: bit-exact integers."""
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


def host(t):
    return t.detach().cpu().numpy()


# ---------------------------------------------------------------------------
# arg sort
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("ndim,n", [(3, 1), (3, 5), (3, 4097), (3, 100_003), (1, 1000), (2, 5000),
                                    (4, 3000)])
def test_arg_sort_single(oracle_lib, ndim, n):
    rng = np.random.default_rng(n + ndim)
    coords = rng.integers(-50, 50, size=(n, ndim)).astype(np.int32)   # many duplicates: stability
    got = host(F.arg_sort_coordinates(dev(coords)))
    assert got.dtype == np.int32
    assert np.array_equal(got, oracle_lib.arg_sort(coords))
    got64 = F.build_sorted_index(dev(coords))
    assert got64.dtype == torch.int64 and np.array_equal(host(got64), oracle_lib.arg_sort(coords))


def test_arg_sort_batched_with_empty_cloud(oracle_lib):
    rng = np.random.default_rng(11)
    coords = rng.integers(-300, 300, size=(20_000, 3)).astype(np.int32)
    bd = np.array([0, 7000, 7000, 12_345, 20_000], np.int64)
    got = F.arg_sort_coordinates(dev(coords), batch_dims=dev(bd))
    assert got.dtype == torch.int64
    assert np.array_equal(host(got), oracle_lib.arg_sort(coords, bd))
    got32 = F.arg_sort_coordinates(dev(coords), batch_dims=dev(bd, torch.int32))
    assert got32.dtype == torch.int32
    assert np.array_equal(host(got32), oracle_lib.arg_sort(coords, bd))


def test_arg_sort_empty_and_int64_coords(oracle_lib):
    assert F.arg_sort_coordinates(torch.empty((0, 3), dtype=torch.int32, device=DEV)).numel() == 0
    rng = np.random.default_rng(2)
    coords = rng.integers(-10**6, 10**6, size=(3000, 3)).astype(np.int64)
    got = host(F.arg_sort_coordinates(dev(coords)))
    assert np.array_equal(got, oracle_lib.arg_sort(coords.astype(np.int32)))


def test_arg_sort_of_a_box_wider_than_one_key(oracle_lib):
    """A bounding box of 3 x 31 bits does not fit a 63-bit key: the sort then runs
    dimension by dimension (the reference's fallback) and gives the same permutation."""
    rng = np.random.default_rng(5)
    coords = rng.integers(-2**30, 2**30, size=(50_000, 3)).astype(np.int32)
    coords[:2] = [[-2**30, -2**30, -2**30], [2**30 - 1, 2**30 - 1, 2**30 - 1]]
    coords[100:2000] = coords[2100:4000]                # duplicates: stability shows
    got = host(F.arg_sort_coordinates(dev(coords)))
    assert np.array_equal(got, oracle_lib.arg_sort(coords))
    bd = np.array([0, 20_000, 20_000, 50_000], np.int64)
    got = host(F.arg_sort_coordinates(dev(coords), batch_dims=dev(bd)))
    assert np.array_equal(got, oracle_lib.arg_sort(coords, bd))


@pytest.mark.parametrize("ndim", [1, 3, 4])
def test_arg_sort_without_flattening_is_the_same_permutation(oracle_lib, ndim):
    rng = np.random.default_rng(6 + ndim)
    coords = rng.integers(-40, 40, size=(30_011, ndim)).astype(np.int32)
    bd = np.array([0, 9000, 30_011], np.int64)
    for b in (None, bd):
        flat = F.arg_sort_coordinates(dev(coords), batch_dims=None if b is None else dev(b))
        by_dim = F.arg_sort_coordinates(dev(coords), batch_dims=None if b is None else dev(b),
                                        enable_flattening=False)
        assert torch.equal(flat, by_dim)
        assert np.array_equal(host(by_dim), oracle_lib.arg_sort(coords, b))


# ---------------------------------------------------------------------------
# unique
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("n", [1, 2, 2047, 2048, 2049, 50_000])
def test_unique_single(oracle_lib, n):
    rng = np.random.default_rng(n)
    coords = rng.integers(0, 12, size=(n, 3)).astype(np.int32)
    coords = coords[oracle_lib.arg_sort(coords)]
    uniq, indices = F.unique_coordinates(dev(coords))
    want_u, want_i = oracle_lib.unique(coords)
    assert indices.dtype == torch.int64
    assert np.array_equal(host(uniq), want_u) and np.array_equal(host(indices), want_i)


def test_unique_batched_and_empty(oracle_lib):
    rng = np.random.default_rng(5)
    coords = rng.integers(0, 6, size=(9000, 3)).astype(np.int32)
    bd = np.array([0, 3000, 3000, 3001, 9000], np.int64)
    coords = coords[oracle_lib.arg_sort(coords, bd)]
    uniq, indices = F.unique_coordinates(dev(coords), batch_dims=dev(bd, torch.int32))
    want_u, want_i = oracle_lib.unique(coords, bd)
    assert indices.dtype == torch.int32
    assert np.array_equal(host(uniq), want_u) and np.array_equal(host(indices), want_i)
    uniq, indices = F.unique_coordinates(torch.empty((0, 3), dtype=torch.int32, device=DEV))
    assert uniq.shape == (0, 3) and host(indices).tolist() == [0]


# ---------------------------------------------------------------------------
# kernel map query, sizes, masks (reference-style API)
# ---------------------------------------------------------------------------
def _targets(oracle_lib, src, sbd, stride):
    if stride == 1:
        return src, sbd
    return oracle_lib.downsample(src, stride, sbd)


@pytest.mark.parametrize("kernel,stride,dilation", [(3, 1, 1), (2, 1, 1), (3, 2, 1), (2, 2, 1),
                                                    (3, 1, 2), (5, 1, 1), ((3, 1, 2), 1, 1)])
@pytest.mark.parametrize("batched", [False, True])
def test_query_sizes_masks(oracle_lib, kernel, stride, dilation, batched):
    rng = np.random.default_rng(17)
    src, sbd = synth.random_small_batch(rng, 3 if batched else 1, 6000, 40, low=-13)
    if not batched:
        sbd = None
    tgt, tbd = _targets(oracle_lib, src, sbd, stride)
    off = generate_kernel_offsets(3, kernel, 1, dilation).astype(np.int32)
    want = oracle_lib.query(src, tgt, off, sbd, tbd)
    got = F.query_sorted_index_with_offsets(dev(src), dev(tgt), dev(off),
                                            None if sbd is None else dev(sbd),
                                            None if tbd is None else dev(tbd))
    assert got.dtype == (torch.int64 if batched else torch.int32)
    assert np.array_equal(host(got), want)
    sizes = F.compute_kernel_map_sizes(got)
    want_sizes = oracle_lib.sizes(want)
    assert np.array_equal(host(sizes), want_sizes)
    order, _ = oracle_lib.order(want_sizes)
    sm, tm = F.compute_kernel_map_masks(len(src), got[dev(order, torch.int64)], sizes)
    want_sm, want_tm = oracle_lib.masks(want[order], len(src))
    assert np.array_equal(host(sm), want_sm) and np.array_equal(host(tm), want_tm)


def test_query_edge_cases(oracle_lib):
    off = generate_kernel_offsets(3, 3, 1, 1).astype(np.int32)
    one = np.array([[5, -7, 3]], np.int32)
    got = host(F.query_sorted_index_with_offsets(dev(one), dev(one), dev(off)))
    assert np.array_equal(got, oracle_lib.query(one, one, off))
    empty = torch.empty((0, 3), dtype=torch.int32, device=DEV)
    assert F.query_sorted_index_with_offsets(dev(one), empty, dev(off)).shape == (27, 0)
    got = host(F.query_sorted_index_with_offsets(empty, dev(one), dev(off)))
    assert (got == -1).all()
    # a dense block: every interior voxel has all 27 neighbours
    g = np.stack(np.meshgrid(*[np.arange(12)] * 3, indexing="ij"), -1).reshape(-1, 3).astype(np.int32)
    got = host(F.query_sorted_index_with_offsets(dev(g), dev(g), dev(off)))
    assert np.array_equal(got, oracle_lib.query(g, g, off))


@pytest.mark.parametrize("ndim", [1, 2, 4])
def test_query_other_ndim(oracle_lib, ndim):
    rng = np.random.default_rng(ndim)
    src, _ = synth.random_small_batch(rng, 1, 3000, 30 if ndim > 1 else 5000, ndim=ndim)
    off = generate_kernel_offsets(ndim, 3, 1, 1).astype(np.int32)
    got = host(F.query_sorted_index_with_offsets(dev(src), dev(src), dev(off)))
    assert np.array_equal(got, oracle_lib.query(src, src, off))


# ---------------------------------------------------------------------------
# KernelMapCache: fused target coordinates + fused map build
# ---------------------------------------------------------------------------
def _check_map(oracle_lib, result, src, tgt, off, sbd, tbd, reorder=True):
    sm, tm, order, sizes = result
    want = oracle_lib.build_kernel_map(src, tgt, off, sbd, tbd, reorder=reorder)
    assert np.array_equal(host(sizes), want["sorted_sizes"])
    if reorder:
        assert np.array_equal(host(order), want["order"])
    else:
        assert order is None
    assert np.array_equal(host(tm), want["target_masks"])
    assert np.array_equal(host(sm), want["source_masks"])


@pytest.mark.parametrize("batched", [False, True])
@pytest.mark.parametrize("n", [3, 1500, 30_000])
def test_cache_submanifold_and_strided(oracle_lib, batched, n):
    rng = np.random.default_rng(n)
    src, sbd = synth.random_small_batch(rng, 4 if batched else 1, n, 64, low=-20)
    if not batched:
        sbd = None
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=DEV)
    d_src = dev(src)
    d_sbd = None if sbd is None else dev(sbd)
    # 3^3 stride 1
    off3 = generate_kernel_offsets(3, 3, 1, 1).astype(np.int32)
    c1 = cache.get_target_coordinates(d_src, d_sbd, 1, 1)
    assert c1[0] is d_src
    r = cache.get_kernel_map(d_src, 1, d_sbd, c1[0], c1[1], c1[2], 3, 1)
    _check_map(oracle_lib, r, src, src, off3, sbd, sbd)
    assert cache.get_kernel_map(d_src, 1, d_sbd, c1[0], c1[1], c1[2], 3, 1)[0] is r[0]
    # 2^3 stride 2 down, then 3^3 at stride 2, then transposed back up
    tgt_c, tgt_s, tgt_bd = cache.get_target_coordinates(d_src, d_sbd, 1, 2)
    want_c, want_bd = oracle_lib.downsample(src, 2, sbd)
    assert tgt_s == (2, 2, 2) and np.array_equal(host(tgt_c), want_c)
    if batched:
        assert np.array_equal(host(tgt_bd), want_bd)
    off2 = generate_kernel_offsets(3, 2, 1, 1).astype(np.int32)
    down = cache.get_kernel_map(d_src, 1, d_sbd, tgt_c, tgt_s, tgt_bd, 2, 1)
    _check_map(oracle_lib, down, src, want_c, off2, sbd, want_bd)
    assert int(host(down[3]).sum()) == len(src)
    off3s2 = generate_kernel_offsets(3, 3, 2, 1).astype(np.int32)
    r2 = cache.get_kernel_map(tgt_c, 2, tgt_bd, tgt_c, tgt_s, tgt_bd, 3, 1)
    _check_map(oracle_lib, r2, want_c, want_c, off3s2, want_bd, want_bd)
    up_c = cache.get_target_coordinates(tgt_c, tgt_bd, 2, 2, transposed=True)
    assert up_c[0] is d_src and up_c[1] == (1, 1, 1)
    up = cache.get_kernel_map(tgt_c, 2, tgt_bd, d_src, 1, d_sbd, 2, 1, transposed=True)
    assert up[0] is down[1] and up[1] is down[0]
    # 3^3 stride 2 strided map and a no-reorder cache
    cache.reset()
    t2 = cache.get_target_coordinates(d_src, d_sbd, 1, 2)
    r3 = cache.get_kernel_map(d_src, 1, d_sbd, t2[0], t2[1], t2[2], 3, 1)
    _check_map(oracle_lib, r3, src, want_c, off3, sbd, want_bd)
    plain = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=DEV, disable_reordering=True)
    r4 = plain.get_kernel_map(d_src, 1, d_sbd, d_src, 1, d_sbd, 3, 1)
    _check_map(oracle_lib, r4, src, src, off3, sbd, sbd, reorder=False)


def test_cache_large_kernel_takes_unfused_path(oracle_lib):
    rng = np.random.default_rng(9)
    src, _ = synth.random_small_batch(rng, 1, 4000, 24)
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=DEV)
    d_src = dev(src)
    r = cache.get_kernel_map(d_src, 1, None, d_src, 1, None, 5, 1)
    _check_map(oracle_lib, r, src, src, generate_kernel_offsets(3, 5, 1, 1).astype(np.int32),
               None, None)


def test_cache_rejects_foreign_coordinates():
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=DEV)
    a = dev(synth.sort_unique(np.random.default_rng(0).integers(0, 50, size=(500, 3))))
    cache.get_kernel_map(a, 1, None, a, 1, None, 3, 1)
    far = dev(np.array([[10_000, 0, 0]], np.int32))
    # the out-of-box flag travels with the (lazy) host copy of the sizes, which
    # is what a convolution waits for before it plans its GEMMs
    from minuet_b200 import engine
    sizes = cache.get_kernel_map(far, 2, None, far, 2, None, 3, 1)[3]
    with pytest.raises(RuntimeError):
        engine.host_copy(sizes)
    cache.reset()
    sizes = cache.get_kernel_map(far, 2, None, far, 2, None, 3, 1)[3]
    assert engine.host_copy(sizes).sum() == 1


@pytest.mark.parametrize("kind", ["uniform50k", "outdoor4"])
def test_config_scale_maps(oracle_lib, kind):
    """Benchmark-size inputs: the 50 000-voxel uniform cloud and the 4 x 120 000
    outdoor batch, all four kernel/stride combinations."""
    if kind == "uniform50k":
        src, sbd = synth.uniform_cloud(), None
    else:
        src, sbd = synth.outdoor_batch(4)
    d_src, d_sbd = dev(src), None if sbd is None else dev(sbd)
    want_c, want_bd = oracle_lib.downsample(src, 2, sbd)
    for kernel, stride in [(3, 1), (2, 1), (3, 2), (2, 2)]:
        cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=DEV)
        tc, ts, tbd = cache.get_target_coordinates(d_src, d_sbd, 1, stride)
        r = cache.get_kernel_map(d_src, 1, d_sbd, tc, ts, tbd, kernel, 1)
        off = generate_kernel_offsets(3, kernel, 1, 1).astype(np.int32)
        if stride == 1:
            _check_map(oracle_lib, r, src, src, off, sbd, sbd)
        else:
            assert np.array_equal(host(tc), want_c)
            _check_map(oracle_lib, r, src, want_c, off, sbd, want_bd)
        # size-independent properties
        sm, tm, order, sizes = (host(t) for t in r)
        assert np.array_equal((sm >= 0).sum(1), sizes) and np.array_equal((tm >= 0).sum(1), sizes)
        if kernel == 3 and stride == 1:
            assert sizes[-1] == len(src) and order[-1] == 13
        if kernel == 2 and stride == 2:
            assert sizes.sum() == len(src)


def test_dense_block_takes_the_general_search_path(oracle_lib):
    """A solid 40^3 block: the table window of a 512-row tile spans three full
    x-slabs (4800 keys), more than the shared-memory window, so the search falls
    back to per-group windows and global binary search."""
    g = np.stack(np.meshgrid(*[np.arange(40)] * 3, indexing="ij"), -1).reshape(-1, 3).astype(np.int32)
    off = generate_kernel_offsets(3, 3, 1, 1).astype(np.int32)
    got = host(F.query_sorted_index_with_offsets(dev(g), dev(g), dev(off)))
    assert np.array_equal(got, oracle_lib.query(g, g, off))
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=DEV)
    d_g = dev(g)
    _check_map(oracle_lib, cache.get_kernel_map(d_g, 1, None, d_g, 1, None, 3, 1), g, g, off,
               None, None)
    tc, ts, tbd = cache.get_target_coordinates(d_g, None, 1, 2)
    want_c, _ = oracle_lib.downsample(g, 2, None)
    assert np.array_equal(host(tc), want_c)
    _check_map(oracle_lib, cache.get_kernel_map(d_g, 1, None, tc, ts, tbd, 2, 1), g, want_c,
               generate_kernel_offsets(3, 2, 1, 1).astype(np.int32), None, None)


def test_indoor_batch_maps(oracle_lib):
    """Indoor-scene-like batch (4 x 200 000 voxels at 2 cm): dense surfaces, many
    pairs per voxel; 3^3 stride 1 and the 2^3 stride 2 down-sampling map."""
    src, sbd = synth.indoor_batch(4)
    d_src, d_sbd = dev(src), dev(sbd)
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=DEV)
    off3 = generate_kernel_offsets(3, 3, 1, 1).astype(np.int32)
    r = cache.get_kernel_map(d_src, 1, d_sbd, d_src, 1, d_sbd, 3, 1)
    _check_map(oracle_lib, r, src, src, off3, sbd, sbd)
    tc, ts, tbd = cache.get_target_coordinates(d_src, d_sbd, 1, 2)
    want_c, want_bd = oracle_lib.downsample(src, 2, sbd)
    assert np.array_equal(host(tc), want_c) and np.array_equal(host(tbd), want_bd)
    off2 = generate_kernel_offsets(3, 2, 1, 1).astype(np.int32)
    r2 = cache.get_kernel_map(d_src, 1, d_sbd, tc, ts, tbd, 2, 1)
    _check_map(oracle_lib, r2, src, want_c, off2, sbd, want_bd)
    assert int(host(r2[3]).sum()) == len(src)


def test_short_workspace_and_bad_shapes_are_errors_not_faults():
    """Host-side fault injection: a workspace that is too small, a kernel with more
    offsets than the library supports and a mask/weight mismatch come back as
    status codes with a message; nothing is launched with bad pointers."""
    import ctypes
    from minuet_b200 import _lib, engine
    lib = _lib.load()
    km = torch.full((27, 5000), -1, dtype=torch.int32, device=DEV)
    sm = torch.empty((27, 5000), dtype=torch.int32, device=DEV)
    tm = torch.empty((27, 5000), dtype=torch.int32, device=DEV)
    ws = torch.empty(64, dtype=torch.uint8, device=DEV)
    st = lib.mn_compute_kernel_map_masks(engine.ptr(km), 27, 5000, 5000, engine.ptr(sm),
                                         engine.ptr(tm), engine.ptr(ws), ws.numel(),
                                         engine.stream_ptr(torch.device(DEV)))
    assert st == _lib.MN_ERR_WORKSPACE and "workspace" in _lib.last_error()
    big = torch.zeros((200, 3), dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError):
        F.query_sorted_index_with_offsets(dev(np.zeros((4, 3), np.int32)),
                                          dev(np.zeros((4, 3), np.int32)), big)
    with pytest.raises(RuntimeError):
        F.sparse_convolution_forward(torch.zeros(10, 8, device=DEV), torch.zeros(27, 8, 8, device=DEV),
                                     torch.zeros((26, 10), dtype=torch.int32, device=DEV),
                                     torch.zeros((27, 10), dtype=torch.int32, device=DEV), None,
                                     torch.zeros(27, dtype=torch.int32, device=DEV), 1, 1)
    torch.cuda.synchronize()


def test_voxelize_with_inverse():
    rng = np.random.default_rng(21)
    pts = rng.uniform(-3.0, 3.0, size=(20_000, 3)).astype(np.float32)
    bd = np.array([0, 8_000, 20_000], np.int64)
    vox, vbd, inv = F.voxelize(dev(pts), 0.25, batch_dims=dev(bd), return_inverse=True)
    want = []
    for a, b in zip(bd[:-1], bd[1:]):
        want.append(synth.sort_unique(np.floor(pts[a:b] / np.float32(0.25)).astype(np.int64)))
    assert np.array_equal(host(vox), np.concatenate(want))
    assert host(vbd).tolist() == [0, len(want[0]), len(want[0]) + len(want[1])]
    back = host(vox)[host(inv)]
    assert np.array_equal(back, np.floor(pts / np.float32(0.25)).astype(np.int32))
    # every point of cloud g lands in a voxel of cloud g
    assert (host(inv)[:8000] < len(want[0])).all() and (host(inv)[8000:] >= len(want[0])).all()


@pytest.mark.parametrize("dtype,channels", [(torch.float32, 5), (torch.float16, 64), (torch.bfloat16, 3),
                                            (torch.float32, 300)])
def test_voxelize_averages_point_features(dtype, channels):
    """voxel_features[u] = mean of the features of the points that fall into voxel u
    (numpy: float64 sums over the inverse indices)."""
    rng = np.random.default_rng(23)
    pts = rng.uniform(-2.0, 2.0, size=(30_000, 3)).astype(np.float32)
    bd = np.array([0, 11_000, 30_000], np.int64)
    feats = torch.as_tensor(rng.standard_normal((len(pts), channels)).astype(np.float32)).to(dtype)
    vox, vbd, inv, vf = F.voxelize(dev(pts), 0.2, batch_dims=dev(bd), return_inverse=True,
                                   features=feats.to(DEV))
    assert vf.dtype == dtype and vf.shape == (vox.shape[0], channels)
    inv_h = host(inv)
    f64 = feats.double().numpy()
    sums = np.zeros((vox.shape[0], channels))
    np.add.at(sums, inv_h, f64)
    want = sums / np.bincount(inv_h, minlength=vox.shape[0])[:, None]
    tol = {torch.float32: 1e-6, torch.float16: 1e-3, torch.bfloat16: 8e-3}[dtype]
    np.testing.assert_allclose(vf.double().cpu().numpy(), want, rtol=tol, atol=tol)
    # without inverse indices the features still come last; same values
    vox2, vbd2, vf2 = F.voxelize(dev(pts), 0.2, batch_dims=dev(bd), features=feats.to(DEV))
    assert torch.equal(vox2, vox) and torch.equal(vf2, vf)
    # single points per voxel are copied through unchanged
    lone = np.arange(200, dtype=np.float32)[:, None].repeat(3, 1) * 2.0
    v3, _, f3 = F.voxelize(dev(lone), 1.0, features=feats[:200].to(DEV))
    assert torch.equal(f3, feats[:200].to(DEV))


def test_int64_coordinates_through_a_layer(oracle_lib):
    rng = np.random.default_rng(22)
    src, sbd = synth.random_small_batch(rng, 2, 2500, 20, low=-7)
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int64, device=DEV)
    conv = minuet.nn.SparseConv3d(8, 8, 2, stride=2, device=DEV)
    minuet.set_kernel_map_cache(conv, cache)
    x = minuet.SparseTensor(torch.randn(len(src), 8, device=DEV), dev(src, torch.int64),
                            batch_dims=dev(sbd, torch.int32))
    out = conv(x)
    want_c, want_bd = oracle_lib.downsample(src, 2, sbd)
    assert out.C.dtype == torch.int64 and np.array_equal(host(out.C), want_c)
    assert out.batch_dims.dtype == torch.int32 and np.array_equal(host(out.batch_dims), want_bd)
    off = generate_kernel_offsets(3, 2, 1, 1).astype(np.int32)
    m = oracle_lib.build_kernel_map(src, want_c, off, sbd, want_bd)
    ref = oracle_lib.conv_forward(x.F.cpu().numpy(), conv.kernel.detach().cpu().numpy(),
                                  m["source_masks"], m["target_masks"], m["order"], acc64=True)
    assert np.abs(host(out.F) - ref).max() <= 1e-5 * np.abs(ref).max()
