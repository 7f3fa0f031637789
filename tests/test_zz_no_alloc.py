"""mn_unique_coordinates_static: the variant of the unique op for callers that
must not allocate device memory (code inside a CUDA stream capture, allocator-
free hot loops, plugins with a fixed memory budget).  Its scratch is a fixed
array inside the library, so it takes no workspace.  Called through the C ABI
and compared, bit for bit, with mn_unique_coordinates on two calls in a row
(the second on different, smaller data, so stale scratch contents would show).

This file sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from minuet_b200 import _lib

DEV = "cuda:0"
MAX_ROWS = 16 * 1024 * 1024


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _sorted_rows(rng, n, extent, clouds):
    rows = rng.integers(0, extent, size=(n, 3)).astype(np.int32)
    bounds = np.linspace(0, n, clouds + 1).astype(np.int64)
    for a, b in zip(bounds[:-1], bounds[1:]):
        seg = rows[a:b]
        rows[a:b] = seg[np.lexsort(seg.T[::-1])]
    return rows, bounds


def _run_both(lib, rows, bounds):
    n = len(rows)
    coords = torch.as_tensor(rows, device=DEV)
    bd = None if bounds is None else torch.as_tensor(bounds, device=DEV)
    nb = 1 if bounds is None else len(bounds) - 1
    stream = ctypes.c_void_p(torch.cuda.current_stream(DEV).cuda_stream)
    ws = torch.empty(int(lib.mn_map_workspace_bytes(n, n, 1)), dtype=torch.uint8, device=DEV)
    want_u = torch.full((n, 3), -7, dtype=torch.int32, device=DEV)
    want_i = torch.full((n + 1,), -7, dtype=torch.int64, device=DEV)
    got_u, got_i = want_u.clone(), want_i.clone()
    _lib.check(lib.mn_unique_coordinates(_ptr(coords), n, 3, _ptr(bd), nb, _ptr(want_u),
                                         _ptr(want_i), _ptr(ws), ws.numel(), stream))
    _lib.check(lib.mn_unique_coordinates_static(_ptr(coords), n, 3, _ptr(bd), nb, _ptr(got_u),
                                                _ptr(got_i), stream))
    torch.cuda.synchronize()
    count = int(want_i[n])
    assert count > 0 and int(got_i[n]) == count
    assert torch.equal(got_i, want_i)
    assert torch.equal(got_u[:count], want_u[:count])
    return count


@pytest.mark.gpu
def test_static_unique_matches_workspace_variant_twice_in_a_row():
    lib = _lib.load()
    with torch.cuda.device(DEV):
        rng = np.random.default_rng(0)
        rows, bounds = _sorted_rows(rng, 300_000, 40, 3)
        first = _run_both(lib, rows, bounds)
        rows, _ = _sorted_rows(rng, 5_000, 9, 1)
        second = _run_both(lib, rows, None)
        assert second < first


@pytest.mark.gpu
def test_static_unique_rejects_more_rows_than_its_scratch_holds():
    lib = _lib.load()
    with torch.cuda.device(DEV):
        idx = torch.zeros(1, dtype=torch.int64, device=DEV)
        st = lib.mn_unique_coordinates_static(None, MAX_ROWS + 1, 3, None, 1, None, _ptr(idx), None)
    assert st == _lib.MN_ERR_BAD_ARG
    assert str(MAX_ROWS) in _lib.last_error()


@pytest.mark.gpu
def test_static_unique_allocates_nothing_and_takes_the_largest_size():
    """The call leaves torch's allocator untouched, and the
    largest accepted size (exactly the scratch capacity) runs and counts correctly."""
    lib = _lib.load()
    with torch.cuda.device(DEV):
        n = MAX_ROWS
        # sorted rows with every value repeated four times: n / 4 distinct coordinates
        base = torch.arange(n, dtype=torch.int32, device=DEV) // 4
        coords = torch.stack([base >> 16, (base >> 8) & 255, base & 255], dim=1).contiguous()
        uniq = torch.empty((n, 3), dtype=torch.int32, device=DEV)
        idx = torch.empty(n + 1, dtype=torch.int64, device=DEV)
        stream = ctypes.c_void_p(torch.cuda.current_stream(DEV).cuda_stream)
        # one warm call first: it looks up the scratch array's address for this device
        _lib.check(lib.mn_unique_coordinates_static(_ptr(coords), 1000, 3, None, 1, _ptr(uniq),
                                                    _ptr(idx), stream))
        torch.cuda.synchronize()
        held, reserved = torch.cuda.memory_allocated(DEV), torch.cuda.memory_reserved(DEV)
        _lib.check(lib.mn_unique_coordinates_static(_ptr(coords), n, 3, None, 1, _ptr(uniq),
                                                    _ptr(idx), stream))
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(DEV) == held
        assert torch.cuda.memory_reserved(DEV) == reserved
        assert int(idx[n]) == n // 4
        assert torch.equal(uniq[:n // 4], coords[::4])
