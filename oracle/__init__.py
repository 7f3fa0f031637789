"""CPU oracle for the sparse-convolution hot path (test infrastructure only).

Only the tests, the smoke check and the benchmark's CPU-baseline leg may import
this package; the product (``minuet_b200``) never does.  ``build()`` compiles
``minuet_oracle.cpp`` into ``oracle/_build/libminuet_oracle.so`` with g++ and
OpenMP; every other function is a thin numpy/ctypes wrapper over one ``orc_*``
entry point, plus brute-force numpy twins used to cross-check the C++ code on
small inputs.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "minuet_oracle.cpp")
_OUT_DIR = os.path.join(_HERE, "_build")
_OUT = os.path.join(_OUT_DIR, "libminuet_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle if the shared object is missing or older than the source."""
    if (not force and os.path.exists(_OUT)
            and os.path.getmtime(_OUT) >= os.path.getmtime(_SRC)):
        return _OUT
    os.makedirs(_OUT_DIR, exist_ok=True)
    cmd = ["g++", "-O3", "-march=native", "-std=c++17", "-fopenmp", "-fPIC",
           "-shared", _SRC, "-o", _OUT]
    try:
        subprocess.check_call(cmd)
    except subprocess.CalledProcessError:
        cmd.remove("-march=native")
        subprocess.check_call(cmd)
    return _OUT


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_OUT):
            build()
        _lib = ctypes.CDLL(_OUT)
        _lib.orc_unique.restype = ctypes.c_int64
        _lib.orc_downsample.restype = ctypes.c_int64
        _lib.orc_plan_buckets.restype = ctypes.c_int64
        _lib.orc_num_threads.restype = ctypes.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _bd(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int64)


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    """Override OMP_NUM_THREADS for the oracle (launchers such as torchrun export 1)."""
    lib().orc_set_num_threads(ctypes.c_int(int(n)))


def arg_sort(coords, batch_dims=None):
    coords = _i32(coords)
    n, d = coords.shape
    bd = _bd(batch_dims)
    index = np.empty(n, dtype=np.int64)
    lib().orc_arg_sort(ctypes.c_int64(n), ctypes.c_int(d), _p(coords),
                       ctypes.c_int64(0 if bd is None else len(bd) - 1), _p(bd), _p(index))
    return index


def unique(coords, batch_dims=None):
    coords = _i32(coords)
    n, d = coords.shape
    bd = _bd(batch_dims)
    out = np.empty((n, d), dtype=np.int32)
    indices = np.empty(n + 1, dtype=np.int64)
    u = lib().orc_unique(ctypes.c_int64(n), ctypes.c_int(d), _p(coords),
                         ctypes.c_int64(0 if bd is None else len(bd) - 1), _p(bd),
                         _p(out), _p(indices))
    return out[:u].copy(), indices


def downsample(coords, tstride, batch_dims=None):
    coords = _i32(coords)
    n, d = coords.shape
    ts = _i32(np.broadcast_to(np.asarray(tstride), (d,)))
    bd = _bd(batch_dims)
    nb = 0 if bd is None else len(bd) - 1
    out = np.empty((n, d), dtype=np.int32)
    obd = None if bd is None else np.empty(nb + 1, dtype=np.int64)
    u = lib().orc_downsample(ctypes.c_int64(n), ctypes.c_int(d), _p(coords), _p(ts),
                             ctypes.c_int64(nb), _p(bd), _p(out), _p(obd))
    return out[:u].copy(), obd


def query(sources, targets, offsets, source_batch_dims=None, target_batch_dims=None):
    sources, targets, offsets = _i32(sources), _i32(targets), _i32(offsets)
    s, d = sources.shape
    t, o = targets.shape[0], offsets.shape[0]
    sbd, tbd = _bd(source_batch_dims), _bd(target_batch_dims)
    out = np.empty((o, t), dtype=np.int32)
    lib().orc_query(ctypes.c_int64(s), ctypes.c_int64(t), ctypes.c_int64(o), ctypes.c_int(d),
                    _p(sources), _p(targets), _p(offsets),
                    ctypes.c_int64(0 if sbd is None else len(sbd) - 1), _p(sbd), _p(tbd), _p(out))
    return out


def sizes(kernel_map):
    kernel_map = _i32(kernel_map)
    o, t = kernel_map.shape
    out = np.empty(o, dtype=np.int32)
    lib().orc_sizes(ctypes.c_int64(o), ctypes.c_int64(t), _p(kernel_map), _p(out))
    return out


def order(sz):
    sz = _i32(sz)
    o = len(sz)
    ordr = np.empty(o, dtype=np.int32)
    ssz = np.empty(o, dtype=np.int32)
    lib().orc_order(ctypes.c_int64(o), _p(sz), _p(ordr), _p(ssz))
    return ordr, ssz


def masks(kernel_map, num_sources):
    kernel_map = _i32(kernel_map)
    o, t = kernel_map.shape
    sm = np.empty((o, num_sources), dtype=np.int32)
    tm = np.empty((o, t), dtype=np.int32)
    lib().orc_masks(ctypes.c_int64(o), ctypes.c_int64(num_sources), ctypes.c_int64(t),
                    _p(kernel_map), _p(sm), _p(tm))
    return sm, tm


def plan_buckets(sorted_sizes, threshold):
    """threshold: float, or None to fuse every offset into one bucket."""
    sz = _i32(sorted_sizes)
    o = len(sz)
    buckets = np.zeros(o + 1, dtype=np.int64)
    cumsum = np.zeros(o + 1, dtype=np.int64)
    nb = lib().orc_plan_buckets(ctypes.c_int64(o), _p(sz),
                                ctypes.c_int(1 if threshold is None else 0),
                                ctypes.c_double(0.0 if threshold is None else float(threshold)),
                                _p(buckets), _p(cumsum))
    return buckets[:nb + 1].copy(), cumsum


def conv_forward(features, weights, source_masks, target_masks, order_=None, acc64=False):
    x = np.ascontiguousarray(features, dtype=np.float32)
    w = np.ascontiguousarray(weights, dtype=np.float32)
    sm, tm = _i32(source_masks), _i32(target_masks)
    o, s = sm.shape
    t = tm.shape[1]
    cin, cout = w.shape[1], w.shape[2]
    ordr = None if order_ is None else _i32(order_)
    out = np.empty((t, cout), dtype=np.float32)
    lib().orc_conv_forward(ctypes.c_int64(s), ctypes.c_int64(t), ctypes.c_int64(o),
                           ctypes.c_int64(cin), ctypes.c_int64(cout), _p(sm), _p(tm), _p(ordr),
                           _p(x), _p(w), _p(out), ctypes.c_int(1 if acc64 else 0))
    return out


def build_kernel_map(sources, targets, offsets, sbd=None, tbd=None, reorder=True):
    """query -> sizes -> stable size order -> masks, as KernelMapCache.get_kernel_map
    does (minuet/nn/convolutions.py:149-170).  Returns a dict of numpy arrays."""
    km = query(sources, targets, offsets, sbd, tbd)
    sz = sizes(km)
    if reorder:
        ordr, ssz = order(sz)
        km_sorted = km[ordr]
    else:
        ordr, ssz, km_sorted = None, sz, km
    sm, tm = masks(km_sorted, len(sources))
    return {"kernel_map": km, "sizes": sz, "order": ordr, "sorted_sizes": ssz,
            "source_masks": sm, "target_masks": tm}


# ---------------------------------------------------------------------------
# brute-force numpy twins (small inputs only)
# ---------------------------------------------------------------------------

def query_bruteforce(sources, targets, offsets, sbd=None, tbd=None):
    """Dictionary lookup of target + offset among the sources of the same cloud."""
    sources, targets, offsets = map(np.asarray, (sources, targets, offsets))
    s, t, o = len(sources), len(targets), len(offsets)
    sbd = np.array([0, s]) if sbd is None else np.asarray(sbd)
    tbd = np.array([0, t]) if tbd is None else np.asarray(tbd)
    out = np.full((o, t), -1, dtype=np.int32)
    for g in range(len(sbd) - 1):
        table = {tuple(int(v) for v in sources[i]): i for i in range(sbd[g], sbd[g + 1])}
        for j in range(tbd[g], tbd[g + 1]):
            for k in range(o):
                key = tuple(int(v) for v in (targets[j] + offsets[k]))
                out[k, j] = table.get(key, -1)
    return out


def conv_bruteforce(features, weights, kernel_map):
    """Sum over offsets (natural offset order) in float64; kernel_map is [O,T] unordered."""
    x = np.asarray(features, dtype=np.float64)
    w = np.asarray(weights, dtype=np.float64)
    o, t = kernel_map.shape
    out = np.zeros((t, w.shape[2]), dtype=np.float64)
    for k in range(o):
        valid = kernel_map[k] != -1
        out[valid] += x[kernel_map[k][valid]] @ w[k]
    return out
