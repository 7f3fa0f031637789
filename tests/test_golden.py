"""The CPU oracle against golden vectors produced by the reference's own CUDA
implementation (tests/golden/reference_golden.npz, written on a GPU box by
tests/golden/make_reference_golden.py).  Runs without a GPU."""
import importlib.util
import os

import numpy as np
import pytest

from minuet_b200.utils.helpers import generate_kernel_offsets

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden", "reference_golden.npz")


@pytest.fixture(scope="module")
def golden():
    if not os.path.exists(GOLDEN):
        pytest.skip("reference golden vectors not generated yet")
    spec = importlib.util.spec_from_file_location(
        "make_reference_golden", os.path.join(HERE, "golden", "make_reference_golden.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    data = np.load(GOLDEN)
    src, bd, raw, x, w = gen.inputs()
    assert int(data["n_src"]) == len(src) and int(data["src_checksum"]) == src.astype(np.int64).sum()
    return data, gen, (src, bd, raw, x, w)


def test_arg_sort_and_unique(golden, oracle_lib):
    data, gen, (src, bd, raw, x, w) = golden
    assert np.array_equal(oracle_lib.arg_sort(raw), data["arg_sort"])
    raw_bd = np.array([0, 300, 700], np.int64)
    order = oracle_lib.arg_sort(raw, raw_bd)
    assert np.array_equal(order, data["multi_arg_sort"])
    rows, indices = oracle_lib.unique(raw[order], raw_bd)
    assert np.array_equal(indices, data["multi_unique_indices"])
    assert np.array_equal(rows, data["multi_unique_rows"])


@pytest.mark.parametrize("kernel,stride", [(3, 1), (2, 1), (3, 2), (2, 2)])
def test_map_and_forward(golden, oracle_lib, kernel, stride):
    data, gen, (src, bd, raw, x, w) = golden
    tag = f"k{kernel}s{stride}"
    tgt, tbd = (src, bd) if stride == 1 else oracle_lib.downsample(src, stride, bd)
    assert np.array_equal(tgt, data[tag + "_targets"])
    off = generate_kernel_offsets(3, kernel, 1, 1).astype(np.int32)
    m = oracle_lib.build_kernel_map(src, tgt, off, bd, tbd)
    assert np.array_equal(m["kernel_map"], data[tag + "_kernel_map"])
    assert np.array_equal(m["sizes"], data[tag + "_sizes"])
    assert np.array_equal(m["source_masks"], data[tag + "_source_masks"])
    assert np.array_equal(m["target_masks"], data[tag + "_target_masks"])
    want = data[tag + "_forward"]
    for acc64 in (False, True):
        got = oracle_lib.conv_forward(x, w[kernel], m["source_masks"], m["target_masks"],
                                      m["order"], acc64=acc64)
        assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
