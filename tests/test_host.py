"""Host-side logic and the C ABI surface (no GPU needed)."""
import ctypes
import json
import os
import re

import numpy as np
import pytest
import torch

import minuet_b200 as minuet
from minuet_b200 import _lib
from minuet_b200.utils.helpers import as_tuple, generate_kernel_offsets

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


def test_library_exports_every_declared_symbol(mn_lib):
    header = open(os.path.join(ROOT, "include", "minuet_b200.h")).read()
    declared = set(re.findall(r"\b(mn_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_lib.PROTOTYPES), declared ^ set(_lib.PROTOTYPES)
    for name in declared:
        assert hasattr(mn_lib, name), name
    assert mn_lib.mn_version() >= 1


def test_offsets_match_reference_golden():
    golden = json.load(open(os.path.join(GOLDEN, "kernel_offsets.json")))
    assert golden["cases"]
    for case in golden["cases"]:
        got = generate_kernel_offsets(case["ndim"], case["kernel_size"], case["source_stride"],
                                      case["dilation"], case["layout"])
        assert got.tolist() == case["offsets"], case


def test_offsets_even_kernel_and_binding():
    off = generate_kernel_offsets(3, 2, 1, 1)
    assert off.tolist() == [[0, 0, 0], [0, 0, 1], [0, 1, 0], [0, 1, 1],
                            [1, 0, 0], [1, 0, 1], [1, 1, 0], [1, 1, 1]]
    off = generate_kernel_offsets(3, 3, 2, 1)
    assert off[0].tolist() == [-2, -2, -2] and off[13].tolist() == [0, 0, 0]
    with pytest.raises(NotImplementedError):
        generate_kernel_offsets(3, 3, 1, 1, layout="other")


def test_as_tuple():
    assert as_tuple(2) == (2, 2, 2)
    assert as_tuple([1, 2, 3]) == (1, 2, 3)
    with pytest.raises(ValueError):
        as_tuple((1, 2), size=3, name="stride")


def test_plan_buckets_matches_oracle(mn_lib, oracle_lib):
    rng = np.random.default_rng(0)
    for trial in range(200):
        o = int(rng.integers(1, 40))
        sizes = np.sort(rng.integers(0, 10 ** int(rng.integers(1, 6)), size=o)).astype(np.int32)
        if trial % 7 == 0:
            sizes[:] = np.sort(rng.integers(1, 4, size=o))
        for threshold in (-1.0, 0.0, 0.05, 0.5, 2.0, None):
            if threshold is not None and threshold >= 0 and sizes[0] == 0:
                continue  # 0/0 redundancy: undefined in the reference too
            buckets = np.zeros(o + 1, np.int64)
            cumsum = np.zeros(o + 1, np.int64)
            nb = ctypes.c_int64(0)
            st = mn_lib.mn_plan_buckets(sizes.ctypes.data_as(ctypes.c_void_p), o,
                                        0 if threshold is None else 1,
                                        0.0 if threshold is None else threshold,
                                        buckets.ctypes.data_as(ctypes.c_void_p),
                                        cumsum.ctypes.data_as(ctypes.c_void_p), ctypes.byref(nb))
            assert st == 0
            want_b, want_c = oracle_lib.plan_buckets(sizes, threshold)
            assert buckets[:nb.value + 1].tolist() == want_b.tolist()
            assert cumsum.tolist() == want_c.tolist()


def test_keyspec_layout(mn_lib):
    mm = np.array([-5, 0, 10, 0, 100, 7, 10, 0], np.int32)
    spec = _lib.KeySpec()
    assert mn_lib.mn_keyspec_make(mm.ctypes.data_as(ctypes.c_void_p), 3, 4, 2, ctypes.byref(spec)) == 0
    assert list(spec.base)[:3] == [-7, -2, 8]
    assert list(spec.extent)[:3] == [109, 11, 4]
    assert list(spec.bits)[:3] == [7, 4, 3]
    assert list(spec.shift)[:3] == [7, 3, 0]
    assert spec.cloud_shift == 14 and spec.cloud_bits == 2 and spec.total_bits == 16
    huge = np.array([-2**30, -2**30, -2**30, 0, 2**30, 2**30, 2**30, 0], np.int32)
    assert mn_lib.mn_keyspec_make(huge.ctypes.data_as(ctypes.c_void_p), 3, 1, 0,
                                  ctypes.byref(spec)) == _lib.MN_ERR_UNSUPPORTED
    assert b"63" in mn_lib.mn_last_error()


def test_bad_arguments_are_reported_without_a_gpu(mn_lib):
    spec = _lib.KeySpec()
    st = mn_lib.mn_keyspec_make(None, 3, 1, 0, ctypes.byref(spec))
    assert st == _lib.MN_ERR_BAD_ARG and mn_lib.mn_last_error()
    sizes = np.array([5, 9], np.int32)
    st = mn_lib.mn_sparse_convolution_forward(4, 4, 2, 8, 8, 0, None, None, None, None, None,
                                              sizes.ctypes.data_as(ctypes.c_void_p), 1, 1, 1, 1,
                                              0.0, None, None, None, 0, None)
    assert st == _lib.MN_ERR_BAD_ARG          # sizes exceed min(S, T)
    with pytest.raises(RuntimeError):
        _lib.check(st, "conv")


def test_sparse_tensor_contract():
    f = torch.zeros(4, 2)
    c = torch.zeros(4, 3, dtype=torch.int32)
    x = minuet.SparseTensor(f, c, stride=2, batch_dims=torch.tensor([0, 4]))
    assert x.stride == (2, 2, 2) and x.batch_dims is None and x.batch_size == 1
    assert x.n == 4 and x.ndim == 3 and x.num_features == 2
    y = minuet.SparseTensor(f, c, batch_dims=torch.tensor([0, 1, 4]))
    assert y.batch_size == 2
    with pytest.raises(ValueError):
        minuet.SparseTensor(f, c.float())
    with pytest.raises(ValueError):
        minuet.SparseTensor(f[:3], c)
    with pytest.raises(ValueError):
        minuet.SparseTensor(f, c[0])
    with pytest.raises(ValueError):
        x.F = torch.zeros(3, 2)
    assert x.half().dtype == torch.float16


def test_no_cpu_path():
    c = torch.zeros(4, 3, dtype=torch.int32)
    with pytest.raises(NotImplementedError):
        minuet.nn.functional.arg_sort_coordinates(c)
    with pytest.raises(NotImplementedError):
        minuet.nn.functional.unique_coordinates(c)
    with pytest.raises(ValueError):
        minuet.nn.functional.query_sorted_index_with_offsets(c, c, c, source_batch_dims=c)


def test_module_surface_and_tunable_config(tmp_path):
    net = torch.nn.Sequential(minuet.nn.SparseConv3d(4, 8, 3), minuet.nn.BatchNorm(8),
                              minuet.nn.ReLU(), minuet.nn.SparseConv(3, 8, 4, 2, stride=2,
                                                                    transposed=True))
    conv = net[0]
    assert conv.kernel.shape == (27, 4, 8) and conv.bias is None
    assert conv.tunable_config == {'threshold': -1, 'gather_tile_size': 1, 'scatter_tile_size': 1,
                                   'algorithm': 'auto', 'sub_tiles': 0}
    # a configuration file written by the reference (three keys) still loads
    minuet.load_tunable_config(conv, {'threshold': 0.5, 'gather_tile_size': 2,
                                      'scatter_tile_size': 4})
    assert conv.tunable_config['algorithm'] == 'auto' and conv.tunable_config['threshold'] == 0.5
    conv.tunable_config.update(threshold=-1, gather_tile_size=1, scatter_tile_size=1)
    assert set(conv.state_dict()) == {"kernel"}
    bound = 1 / np.sqrt(4 * 27)
    assert float(conv.kernel.abs().max()) <= bound
    assert float(net[3].kernel.abs().max()) <= 1 / np.sqrt(4 * 8)  # transposed: fan = out_channels
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device="cpu")
    minuet.set_kernel_map_cache(net, cache)
    assert conv._kernel_map_cache is cache and net[3]._kernel_map_cache is cache
    cfg = minuet.dump_tunable_config(net)
    assert set(cfg) == {"0", "1", "2", "3"} and cfg["0"]["threshold"] == -1
    cfg["0"]["gather_tile_size"] = 4
    minuet.load_tunable_config(net, json.loads(json.dumps(cfg)))
    assert conv.tunable_config["gather_tile_size"] == 4
    with pytest.raises(ValueError):
        minuet.nn.SparseConv3d(4, 8, 3)(minuet.SparseTensor(torch.zeros(2, 4),
                                                            torch.zeros(2, 3, dtype=torch.int32)))
    with pytest.raises(RuntimeError):
        cache.get_target_coordinates(torch.zeros(2, 3, dtype=torch.int32), None, 2, 2,
                                     transposed=True)


def _pack_numpy(coords, clouds, spec):
    """numpy twin of the device key packing (mn_keyspec layout)."""
    keys = clouds.astype(np.uint64) << np.uint64(spec.cloud_shift)
    for k in range(spec.ndim):
        field = (coords[:, k].astype(np.int64) - spec.base[k]).astype(np.uint64)
        keys |= field << np.uint64(spec.shift[k])
    return keys


def test_key_layout_preserves_order_and_offset_addition(mn_lib):
    """Properties the Map-step kernels rely on: unsigned key order equals
    (cloud, lexicographic) order, and key(c + offset) == key(c) + delta(offset)
    as plain 64-bit arithmetic for every offset within the margin."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=60, deadline=None)
    @given(st.integers(1, 3), st.integers(0, 9), st.integers(1, 40), st.integers(0, 2 ** 20),
           st.integers(0, 10 ** 6))
    def check(ndim_minus_1, margin, n, span, seed):
        ndim = ndim_minus_1 + 1
        rng = np.random.default_rng(seed)
        lo = rng.integers(-2 ** 20, 2 ** 20, size=ndim)
        coords = (lo + rng.integers(0, span + 1, size=(n, ndim))).astype(np.int32)
        clouds = np.sort(rng.integers(0, 5, size=n))
        mm = np.zeros(8, np.int32)
        mm[:ndim] = coords.min(0)
        mm[4:4 + ndim] = coords.max(0)
        spec = _lib.KeySpec()
        status = mn_lib.mn_keyspec_make(mm.ctypes.data_as(ctypes.c_void_p), ndim, 5, margin,
                                        ctypes.byref(spec))
        # bits the box needs: per dimension the width of (extent + 2 * margin), plus 3 cloud bits
        need = 3 + sum(max(1, int(int(mm[4 + k]) - int(mm[k]) + 2 * margin).bit_length())
                       for k in range(ndim))
        if need > 63:
            # documented limit: one 64-bit key per voxel
            assert status == _lib.MN_ERR_UNSUPPORTED and b"63" in mn_lib.mn_last_error()
            return
        assert status == 0
        keys = _pack_numpy(coords, clouds, spec)
        # order
        want = np.lexsort(tuple(coords[:, k] for k in range(ndim - 1, -1, -1)) + (clouds,))
        got = np.argsort(keys, kind="stable")
        assert np.array_equal(keys[got], keys[want])
        # offsets within the margin never borrow across fields
        off = rng.integers(-margin, margin + 1, size=ndim)
        delta = sum(int(off[k]) << int(spec.shift[k]) for k in range(ndim))
        moved = _pack_numpy(coords + off.astype(np.int32), clouds, spec)
        assert np.array_equal(moved.astype(np.int64), keys.astype(np.int64) + delta)
        assert spec.total_bits <= 63

    check()


def test_status_word_decoding():
    """Each bit of the device status word maps to its own exception and message."""
    from minuet_b200 import engine
    assert engine.decode_status(0) is None
    box = engine.decode_status(engine.STATUS_KEY_BOX)
    assert isinstance(box, RuntimeError) and "bounding box" in str(box)
    tc = engine.decode_status(engine.STATUS_TC_TIMEOUT)
    assert isinstance(tc, RuntimeError) and "tensor-core" in str(tc) and "invalid" in str(tc)
    assert "bounding box" not in str(tc)
    both = engine.decode_status(engine.STATUS_KEY_BOX | engine.STATUS_TC_TIMEOUT)
    assert "tensor-core" in str(both) and "bounding box" in str(both)
    wide = engine.decode_status(engine.STATUS_KEY_BITS)
    assert isinstance(wide, NotImplementedError) and "63" in str(wide)
