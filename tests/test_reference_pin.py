"""Pins the CPU oracle against the reference's OWN CUDA implementation.

oracle/build_ref.py compiles the reference's unmodified .cu files (read in place
from a reference checkout) plus a thin C shim into oracle/_ref/libminuet_ref.so.
On a GPU box these tests run the reference kernels and require the oracle to
agree: bit-exact for the integer stages, 1e-5 of the output scale for the fp32
forward pass (cuBLAS summation order is unspecified).  They are skipped where
the library was not built.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

from minuet_b200 import synth
from minuet_b200.utils.helpers import generate_kernel_offsets

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libminuet_ref.so")
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libminuet_ref.so not built (needs a reference checkout)")
    lib = ctypes.CDLL(REF_LIB)
    lib.ref_last_error.restype = ctypes.c_char_p
    return lib


def dev(a, dtype=None):
    return torch.as_tensor(np.ascontiguousarray(a), dtype=dtype, device=DEV)


def p(t):
    return ctypes.c_void_p(t.data_ptr())


def ok(lib, rc):
    assert rc == 0, lib.ref_last_error().decode()


I64 = ctypes.c_int64


def ref_query(lib, src, tgt, off, sbd=None, tbd=None):
    d_src, d_tgt, d_off = dev(src), dev(tgt), dev(off)
    out = torch.empty((len(off), len(tgt)), dtype=torch.int32, device=DEV)
    if sbd is None:
        ok(lib, lib.ref_query(I64(len(src)), I64(len(tgt)), I64(len(off)), p(d_src), p(d_tgt),
                              p(d_off), p(out), None))
    else:
        d_sbd, d_tbd = dev(sbd, torch.int32), dev(tbd, torch.int32)
        ok(lib, lib.ref_multi_query(I64(len(sbd) - 1), I64(len(off)), p(d_sbd), p(d_tbd), p(d_src),
                                    p(d_tgt), p(d_off), p(out), None))
    return out


@pytest.mark.parametrize("n", [1, 777, 50_000])
def test_arg_sort(ref, oracle_lib, n):
    rng = np.random.default_rng(n)
    coords = rng.integers(-40, 40, size=(n, 3)).astype(np.int32)
    d_coords = dev(coords)     # every device tensor stays referenced until its call returns
    for flatten in (1, 0):
        out = torch.empty(n, dtype=torch.int32, device=DEV)
        ok(ref, ref.ref_arg_sort(I64(n), p(d_coords), p(out), flatten, None))
        assert np.array_equal(out.cpu().numpy(), oracle_lib.arg_sort(coords))
    # no empty cloud here: the reference's per-cloud bounding boxes come from a
    # reduce-by-key over cloud ids (arg_sort_coodrinates.cu:155-215), which
    # compacts away empty clouds and then pairs boxes with the wrong clouds
    bd = np.array([0, n // 3, n] if n >= 3 else [0, n], np.int64)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    d_bd = dev(bd, torch.int32)
    ok(ref, ref.ref_multi_arg_sort(I64(n), I64(len(bd) - 1), p(d_coords), p(d_bd), p(out), 1,
                                   None))
    assert np.array_equal(out.cpu().numpy(), oracle_lib.arg_sort(coords, bd))


def test_unique(ref, oracle_lib):
    rng = np.random.default_rng(1)
    coords = rng.integers(0, 9, size=(20_000, 3)).astype(np.int32)
    bd = np.array([0, 5000, 5000, 20_000], np.int64)
    single = coords[oracle_lib.arg_sort(coords)]
    n = len(single)
    idx = torch.empty(n + 1, dtype=torch.int64, device=DEV)
    out = torch.empty((n, 3), dtype=torch.int32, device=DEV)
    count = I64(0)
    d_single = dev(single)
    ok(ref, ref.ref_unique(I64(n), p(d_single), p(idx), p(out), ctypes.byref(count), None))
    want_u, want_i = oracle_lib.unique(single)
    assert count.value == len(want_u)
    assert np.array_equal(idx.cpu().numpy(), want_i)
    assert np.array_equal(out[:count.value].cpu().numpy(), want_u)
    multi = coords[oracle_lib.arg_sort(coords, bd)]
    idx32 = torch.empty(n + 1, dtype=torch.int32, device=DEV)
    d_multi, d_bd = dev(multi), dev(bd, torch.int32)
    ok(ref, ref.ref_multi_unique(I64(n), I64(len(bd)), p(d_multi), p(d_bd), p(idx32), p(out),
                                 ctypes.byref(count), None))
    want_u, want_i = oracle_lib.unique(multi, bd)
    assert count.value == len(want_u)
    assert np.array_equal(idx32.cpu().numpy(), want_i)
    assert np.array_equal(out[:count.value].cpu().numpy(), want_u)


@pytest.mark.parametrize("kernel,stride", [(3, 1), (2, 1), (3, 2), (2, 2)])
@pytest.mark.parametrize("kind", ["small", "small_batched", "uniform50k", "outdoor4"])
def test_query_sizes_masks(ref, oracle_lib, kernel, stride, kind):
    rng = np.random.default_rng(3)
    if kind == "small":
        src, sbd = synth.random_small_batch(rng, 1, 5000, 30, low=-11)[0], None
    elif kind == "small_batched":
        src, sbd = synth.random_small_batch(rng, 3, 3000, 24, low=-5)
    elif kind == "uniform50k":
        src, sbd = synth.uniform_cloud(), None
    else:
        src, sbd = synth.outdoor_batch(4)
    tgt, tbd = (src, sbd) if stride == 1 else oracle_lib.downsample(src, stride, sbd)
    off = generate_kernel_offsets(3, kernel, 1, 1).astype(np.int32)
    km = ref_query(ref, src, tgt, off, sbd, tbd)
    want = oracle_lib.query(src, tgt, off, sbd, tbd)
    assert np.array_equal(km.cpu().numpy(), want)
    O, T, S = len(off), len(tgt), len(src)
    sizes = torch.empty(O, dtype=torch.int32, device=DEV)
    ok(ref, ref.ref_sizes(I64(O), I64(T), p(km), p(sizes), None))
    want_sizes = oracle_lib.sizes(want)
    assert np.array_equal(sizes.cpu().numpy(), want_sizes)
    order, sorted_sizes = oracle_lib.order(want_sizes)
    km_sorted = km[dev(order, torch.int64)].contiguous()
    sm = torch.empty((O, S), dtype=torch.int32, device=DEV)
    tm = torch.empty((O, T), dtype=torch.int32, device=DEV)
    d_sorted_sizes = dev(sorted_sizes)
    ok(ref, ref.ref_masks(I64(O), I64(S), I64(T), p(km_sorted), p(d_sorted_sizes), p(sm), p(tm),
                          None))
    want_sm, want_tm = oracle_lib.masks(want[order], S)
    assert np.array_equal(sm.cpu().numpy(), want_sm)
    assert np.array_equal(tm.cpu().numpy(), want_tm)


@pytest.mark.parametrize("threshold", [-1.0, 0.5, None])
@pytest.mark.parametrize("kernel,stride,shortcut", [(3, 1, 1), (3, 1, 0), (2, 2, 0)])
def test_forward_fp32(ref, oracle_lib, threshold, kernel, stride, shortcut):
    rng = np.random.default_rng(5)
    src, sbd = synth.random_small_batch(rng, 2, 4000, 22)
    tgt, tbd = (src, sbd) if stride == 1 else oracle_lib.downsample(src, stride, sbd)
    off = generate_kernel_offsets(3, kernel, 1, 1).astype(np.int32)
    m = oracle_lib.build_kernel_map(src, tgt, off, sbd, tbd)
    c_in, c_out = 32, 32
    x = rng.standard_normal((len(src), c_in)).astype(np.float32)
    w = synth.kaiming_normal((len(off), c_in, c_out), 7)
    out = torch.empty((len(tgt), c_out), dtype=torch.float32, device=DEV)
    d_sm, d_tm = dev(m["source_masks"]), dev(m["target_masks"])
    d_order, d_sizes, d_x, d_w = dev(m["order"]), dev(m["sorted_sizes"]), dev(x), dev(w)
    torch.cuda.synchronize()
    # tile size 1 is what an untuned reference layer uses (convolutions.py:277-281)
    ok(ref, ref.ref_conv_forward(
        I64(len(src)), I64(len(tgt)), I64(len(off)), 1 if threshold is None else 0,
        ctypes.c_double(0.0 if threshold is None else threshold), I64(4), shortcut, I64(c_in),
        I64(c_out), p(d_sm), p(d_tm), p(d_order), p(d_sizes), p(d_x), p(d_w), p(out), I64(1),
        I64(1), None))
    want = oracle_lib.conv_forward(x, w, m["source_masks"], m["target_masks"], m["order"], acc64=True)
    got = out.cpu().numpy()
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
