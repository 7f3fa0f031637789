"""The CPU oracle against brute force and against the identities the reference's
formulas imply (it has no tests of its own to pin to)."""
import numpy as np
import pytest

from minuet_b200 import synth
from minuet_b200.utils.helpers import generate_kernel_offsets


def _lexsorted(coords):
    order = np.lexsort(coords.T[::-1])
    return order


@pytest.mark.parametrize("ndim", [1, 2, 3, 4])
def test_arg_sort_matches_lexsort(oracle_lib, ndim):
    rng = np.random.default_rng(ndim)
    coords = rng.integers(-20, 20, size=(500, ndim)).astype(np.int32)
    index = oracle_lib.arg_sort(coords)
    # stable: equals numpy's stable lexsort
    assert np.array_equal(index, np.lexsort(coords.T[::-1]))


def test_arg_sort_batched_is_cloud_major(oracle_lib):
    rng = np.random.default_rng(0)
    coords = rng.integers(0, 9, size=(300, 3)).astype(np.int32)
    bd = np.array([0, 100, 100, 220, 300])
    index = oracle_lib.arg_sort(coords, bd)
    for g in range(4):
        seg = index[bd[g]:bd[g + 1]]
        assert ((seg >= bd[g]) & (seg < bd[g + 1])).all()
        want = np.lexsort(coords[bd[g]:bd[g + 1]].T[::-1]) + bd[g]
        assert np.array_equal(seg, want)


def test_unique_and_indices(oracle_lib):
    coords = np.array([[0, 0, 1], [0, 0, 1], [0, 2, 0], [1, 0, 0], [1, 0, 0], [1, 0, 0]], np.int32)
    uniq, indices = oracle_lib.unique(coords)
    assert uniq.tolist() == [[0, 0, 1], [0, 2, 0], [1, 0, 0]]
    assert indices.tolist() == [0, 0, 1, 2, 2, 2, 3]
    # equal rows on both sides of a cloud boundary stay separate
    uniq, indices = oracle_lib.unique(coords, np.array([0, 1, 6]))
    assert uniq.tolist() == [[0, 0, 1], [0, 0, 1], [0, 2, 0], [1, 0, 0]]
    assert indices.tolist() == [0, 1, 2, 3, 3, 3, 4]


def test_downsample_floor_division(oracle_lib):
    coords = synth.sort_unique(np.array([[-3, 0, 1], [-1, 5, 2], [0, 0, 0], [1, 1, 1], [2, 3, 4]]))
    out, _ = oracle_lib.downsample(coords, 2)
    want = synth.sort_unique((coords // 2) * 2)
    assert np.array_equal(out, want)


@pytest.mark.parametrize("kernel,stride", [(3, 1), (2, 1), (3, 2), (2, 2)])
def test_query_matches_bruteforce(oracle_lib, kernel, stride):
    rng = np.random.default_rng(7)
    src, sbd = synth.random_small_batch(rng, 3, 250, 10, low=-4)
    if stride == 1:
        tgt, tbd = src, sbd
    else:
        tgt, tbd = oracle_lib.downsample(src, stride, sbd)
    off = generate_kernel_offsets(3, kernel, 1, 1).astype(np.int32)
    got = oracle_lib.query(src, tgt, off, sbd, tbd)
    want = oracle_lib.query_bruteforce(src, tgt, off, sbd, tbd)
    assert np.array_equal(got, want)
    if kernel == 2 and stride == 2:
        # every source lies in exactly one 2^3 cell of its floored target
        assert (got != -1).sum() == len(src)


def test_masks_are_rank_bijections(oracle_lib):
    rng = np.random.default_rng(3)
    src, _ = synth.random_small_batch(rng, 1, 400, 9)
    off = generate_kernel_offsets(3, 3, 1, 1).astype(np.int32)
    r = oracle_lib.build_kernel_map(src, src, off)
    km, sizes, order = r["kernel_map"], r["sizes"], r["order"]
    assert sizes[13] == len(src)                      # centre offset hits every voxel
    assert np.array_equal(sizes, sizes[::-1])         # delta and -delta pair up
    assert np.array_equal(r["sorted_sizes"], np.sort(sizes))
    assert order[-1] == 13
    for p, o in enumerate(order):
        sm, tm = r["source_masks"][p], r["target_masks"][p]
        n = sizes[o]
        assert sorted(sm[sm >= 0].tolist()) == list(range(n))
        assert sorted(tm[tm >= 0].tolist()) == list(range(n))
        t_idx = np.nonzero(tm >= 0)[0]
        # equal ranks pair the target with the source the kernel map names
        s_of_rank = np.empty(n, np.int64)
        s_of_rank[sm[sm >= 0]] = np.nonzero(sm >= 0)[0]
        assert np.array_equal(s_of_rank[tm[t_idx]], km[o][t_idx])


def test_plan_buckets_cases(oracle_lib):
    sizes = np.array([1, 1, 2, 10, 10, 11, 100], np.int32)
    b, c = oracle_lib.plan_buckets(sizes, -1)
    assert b.tolist() == list(range(8)) and c.tolist() == [0, 1, 2, 4, 14, 24, 35, 135]
    b, c = oracle_lib.plan_buckets(sizes, None)
    assert b.tolist() == [0, 7] and c[-1] == 700
    b, c = oracle_lib.plan_buckets(sizes, 0.0)
    assert b.tolist() == [0, 2, 3, 5, 6, 7]
    b, c = oracle_lib.plan_buckets(sizes, 0.5)
    assert b[0] == 0 and b[-1] == 7 and np.all(np.diff(b) > 0)


def test_conv_matches_bruteforce(oracle_lib):
    rng = np.random.default_rng(5)
    src, _ = synth.random_small_batch(rng, 1, 300, 8)
    off = generate_kernel_offsets(3, 3, 1, 1).astype(np.int32)
    r = oracle_lib.build_kernel_map(src, src, off)
    x = rng.standard_normal((len(src), 6)).astype(np.float32)
    w = rng.standard_normal((27, 6, 5)).astype(np.float32)
    want = oracle_lib.conv_bruteforce(x, w, r["kernel_map"])
    for acc64 in (False, True):
        got = oracle_lib.conv_forward(x, w, r["source_masks"], r["target_masks"], r["order"], acc64)
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
