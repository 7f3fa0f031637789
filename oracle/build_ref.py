"""Compile the reference's own CUDA sources for the hot path, where they lie in
the reference checkout, together with oracle/ref_shim.cu into
oracle/_ref/libminuet_ref.so (sm_100a).  Only nvcc is used: the reference's
cmake build is not run and none of its sources are copied.

    python oracle/build_ref.py [/path/to/reference]

The library is test infrastructure: tests/test_reference_pin.py and
tests/golden/make_reference_golden.py load it on a GPU box to pin the CPU oracle
against the reference implementation.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libminuet_ref.so")
REF_SOURCES = [
    "minuet/cuda/buffer_pool.cu", "minuet/cuda/context.cu", "minuet/cuda/event.cu",
    "minuet/cuda/memory.cu", "minuet/cuda/helpers.cu",
    "minuet/cuda/functions/arg_sort_coodrinates.cu", "minuet/cuda/functions/query_sorted_index.cu",
    "minuet/cuda/functions/scan.cu", "minuet/cuda/functions/unique_coordinates.cu",
    "minuet/cuda/functions/sparse_convolution.cu",
    "minuet/cpu/context.cpp", "minuet/cpu/memory.cpp",
]


DEFAULT_REFERENCE = os.environ.get("MINUET_REFERENCE_ROOT", os.path.join(os.sep, "root", "reference"))


def build(reference_root=DEFAULT_REFERENCE, force=False):
    csrc = os.path.join(reference_root, "csrc")
    if not os.path.isdir(csrc):
        print(f"reference checkout not found at {reference_root}; keeping any prebuilt {OUT}")
        return None
    shim = os.path.join(HERE, "ref_shim.cu")
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(shim):
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    flags = ["-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a",
             "--expt-extended-lambda", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
             "-w", "-I", csrc, "-DMINUET_ENABLE_CUDA"]
    jobs = []
    objs = []
    for src in REF_SOURCES + [shim]:
        path = src if os.path.isabs(src) else os.path.join(csrc, src)
        stem = os.path.relpath(path, csrc if path.startswith(csrc) else HERE)
        obj = os.path.join(OUT_DIR, stem.replace(os.sep, "_").rsplit(".", 1)[0] + ".o")
        objs.append(obj)
        cmd = [nvcc, *flags, "-x", "cu", "-c", path, "-o", obj]
        jobs.append((path, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    ok = True
    for path, p in jobs:
        out, _ = p.communicate()
        if p.returncode != 0:
            ok = False
            sys.stderr.write(f"--- {path}\n{out.decode()[-4000:]}\n")
    if not ok:
        print("reference build failed; the reference pin tests will be skipped")
        return None
    subprocess.check_call([nvcc, "-shared", "-o", OUT, *objs, "-lcublas", "-lcudart"])
    for obj in objs:
        os.remove(obj)
    return OUT


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("-") else DEFAULT_REFERENCE
    print(build(root, force="--force" in sys.argv))
