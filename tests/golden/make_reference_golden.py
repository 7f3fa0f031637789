"""Writes reference_golden.npz: outputs of the reference's OWN CUDA implementation
(oracle/_ref/libminuet_ref.so, built from the reference checkout by
oracle/build_ref.py) on small seeded inputs.  Needs a GPU:

    python tests/golden/make_reference_golden.py reference_golden.npz

The committed copy lives beside this script; tests/test_golden.py checks the CPU
oracle against it without a GPU.  Inputs are regenerated from the seeds below,
only outputs (and the inputs' checksums) are stored.
"""
import ctypes
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from minuet_b200 import synth  # noqa: E402
from minuet_b200.utils.helpers import generate_kernel_offsets  # noqa: E402

DEV = "cuda:0"
I64 = ctypes.c_int64
CASES = [(3, 1), (2, 1), (3, 2), (2, 2)]


def inputs():
    rng = np.random.default_rng(20240)
    src, bd = synth.random_small_batch(rng, 2, 450, 14, low=-5)
    raw = rng.integers(-6, 6, size=(700, 3)).astype(np.int32)
    x = rng.standard_normal((len(src), 8)).astype(np.float32)
    w = {k: synth.kaiming_normal((k ** 3, 8, 8), 11 + k) for k in (2, 3)}
    return src, bd, raw, x, w


def downsample_numpy(src, bd, stride):
    out, obd = [], [0]
    for a, b in zip(bd[:-1], bd[1:]):
        u = synth.sort_unique((src[a:b] // stride) * stride)
        out.append(u)
        obd.append(obd[-1] + len(u))
    return np.concatenate(out).astype(np.int32), np.asarray(obd, np.int64)


def main(out_path):
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libminuet_ref.so"))
    lib.ref_last_error.restype = ctypes.c_char_p

    def ok(rc):
        assert rc == 0, lib.ref_last_error().decode()

    def dev(a, dtype=None):
        return torch.as_tensor(np.ascontiguousarray(a), dtype=dtype, device=DEV)

    def p(t):
        return ctypes.c_void_p(t.data_ptr())

    src, bd, raw, x, w = inputs()
    out = {"src_checksum": np.int64(src.astype(np.int64).sum()), "n_src": np.int64(len(src))}

    d_raw = dev(raw)
    idx = torch.empty(len(raw), dtype=torch.int32, device=DEV)
    ok(lib.ref_arg_sort(I64(len(raw)), p(d_raw), p(idx), 1, None))
    out["arg_sort"] = idx.cpu().numpy()
    raw_bd = np.array([0, 300, 700], np.int64)
    d_rbd = dev(raw_bd, torch.int32)
    ok(lib.ref_multi_arg_sort(I64(len(raw)), I64(2), p(d_raw), p(d_rbd), p(idx), 1, None))
    out["multi_arg_sort"] = idx.cpu().numpy()

    sorted_raw = raw[out["multi_arg_sort"]]
    d_sr = dev(sorted_raw)
    uidx = torch.empty(len(raw) + 1, dtype=torch.int32, device=DEV)
    uout = torch.empty((len(raw), 3), dtype=torch.int32, device=DEV)
    count = I64(0)
    ok(lib.ref_multi_unique(I64(len(raw)), I64(3), p(d_sr), p(d_rbd), p(uidx), p(uout),
                            ctypes.byref(count), None))
    out["multi_unique_indices"] = uidx.cpu().numpy()
    out["multi_unique_rows"] = uout[:count.value].cpu().numpy()

    d_src, d_sbd = dev(src), dev(bd, torch.int32)
    for kernel, stride in CASES:
        tag = f"k{kernel}s{stride}"
        tgt, tbd = (src, bd) if stride == 1 else downsample_numpy(src, bd, stride)
        off = generate_kernel_offsets(3, kernel, 1, 1).astype(np.int32)
        d_tgt, d_tbd, d_off = dev(tgt), dev(tbd, torch.int32), dev(off)
        O, T, S = len(off), len(tgt), len(src)
        km = torch.empty((O, T), dtype=torch.int32, device=DEV)
        ok(lib.ref_multi_query(I64(len(bd) - 1), I64(O), p(d_sbd), p(d_tbd), p(d_src), p(d_tgt),
                               p(d_off), p(km), None))
        sizes = torch.empty(O, dtype=torch.int32, device=DEV)
        ok(lib.ref_sizes(I64(O), I64(T), p(km), p(sizes), None))
        h_sizes = sizes.cpu().numpy()
        order = np.argsort(h_sizes, kind="stable").astype(np.int32)
        d_sorted_sizes = dev(h_sizes[order])
        km_sorted = km[dev(order, torch.int64)].contiguous()
        sm = torch.empty((O, S), dtype=torch.int32, device=DEV)
        tm = torch.empty((O, T), dtype=torch.int32, device=DEV)
        ok(lib.ref_masks(I64(O), I64(S), I64(T), p(km_sorted), p(d_sorted_sizes), p(sm), p(tm),
                         None))
        d_order, d_x, d_w = dev(order), dev(x), dev(w[kernel])
        y = torch.empty((T, 8), dtype=torch.float32, device=DEV)
        torch.cuda.synchronize()
        ok(lib.ref_conv_forward(I64(S), I64(T), I64(O), 0, ctypes.c_double(-1.0), I64(4),
                                1 if stride == 1 else 0, I64(8), I64(8), p(sm), p(tm), p(d_order),
                                p(d_sorted_sizes), p(d_x), p(d_w), p(y), I64(1), I64(1), None))
        out[tag + "_targets"] = tgt
        out[tag + "_kernel_map"] = km.cpu().numpy()
        out[tag + "_sizes"] = h_sizes
        out[tag + "_source_masks"] = sm.cpu().numpy()
        out[tag + "_target_masks"] = tm.cpu().numpy()
        out[tag + "_forward"] = y.cpu().numpy()
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1])
