"""Build libminuet_b200.so in-tree with nvcc for sm_100a.

Run as ``python -m minuet_b200.build`` (or through ``__graft_entry__.build()``).
The shared object lands next to this file so that it travels with the source
tree; nothing is written outside the package directory.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libminuet_b200.so")
SOURCES = ["mn_api.cu", "mn_map_keys.cu", "mn_map_sort.cu", "mn_map_query.cu", "mn_gms.cu",
           "mn_gemm_tc.cu", "mn_conv_implicit.cu", "mn_conv_pairs.cu", "mn_voxel.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall"]


def _stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(HERE, "..", "include", "minuet_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return OUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    obj_dir = os.path.join(HERE, "_obj")
    os.makedirs(obj_dir, exist_ok=True)
    procs = []
    objs = []
    for src in SOURCES:
        obj = os.path.join(obj_dir, src.replace(".cu", ".o"))
        objs.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        text = out.decode()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src}\n{text}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see the log above")
    subprocess.check_call([nvcc, "-shared", "-o", OUT, *objs, "-lcudart", "-lcuda"])
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
