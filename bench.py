"""Benchmark of the Map step (kernel-map build) on synthetic outdoor clouds.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload: a batch of 4 outdoor-scan-like clouds of 120 000 voxels per GPU; one
BUILD makes, on a cold KernelMapCache, the four kernel maps
(kernel 3^3 / 2^3) x (stride 1 / 2), including the strided target coordinates
(floor, sort, unique); one STEP is --repeats such builds back to back (so that the
timed region is long enough for the clock sampler).  The metric is source voxels
processed per second, summed over the four maps (Mvoxels/s).  With N > 1 every
rank owns its own batch (weak scaling, no collective on the data path); the time
is the max over ranks.

The same line carries the gather / GEMM / scatter sweep over channel widths
("gms_sweep") and the sparse-UNet forward on 64 clouds ("unet") with its own
roofline and CPU baseline.

Prints ONE JSON line on rank 0.
"""
import argparse
import ctypes
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

MAPS = [(3, 1), (2, 1), (3, 2), (2, 2)]       # (kernel size, kernel stride)
CLOUDS_PER_GPU = 4
VOXELS_PER_CLOUD = 120_000
METRIC = "kernel-map Mvoxels/s"
UNIT = "Mvoxels/s"
TRAFFIC_TABLE = os.path.join(ROOT, "profiles", "dram_traffic_map_step_C1.txt")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


# ---------------------------------------------------------------------------
# CPU arm: the oracle restatement on the host cores
# ---------------------------------------------------------------------------
def oracle_step(oracle, coords, bd, offsets, repeats=1):
    for _ in range(repeats - 1):
        oracle_step(oracle, coords, bd, offsets)
    tgt2, tbd2 = oracle.downsample(coords, 2, bd)
    out = []
    for kernel, stride in MAPS:
        tgt, tbd = (coords, bd) if stride == 1 else (tgt2, tbd2)
        out.append(oracle.build_kernel_map(coords, tgt, offsets[kernel], bd, tbd))
    return out


def run_cpu(steps, warmup, coords, bd, min_seconds=0.0, repeats=1):
    # torchrun exports OMP_NUM_THREADS=1; the CPU arm uses every core this process may run on
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    os.environ["OMP_NUM_THREADS"] = str(cores)
    import oracle
    from minuet_b200.utils.helpers import generate_kernel_offsets
    oracle.build()
    oracle.set_num_threads(cores)
    offsets = {k: generate_kernel_offsets(3, k, 1, 1).astype(np.int32) for k in (2, 3)}
    for _ in range(warmup):
        oracle_step(oracle, coords, bd, offsets, repeats)
    t0 = time.perf_counter()
    done = 0
    while done < steps or time.perf_counter() - t0 < min_seconds:
        oracle_step(oracle, coords, bd, offsets, repeats)
        done += 1
    dt = time.perf_counter() - t0
    voxels = len(MAPS) * len(coords) * done * repeats
    return voxels / dt / 1e6, dt / done * 1e3, done, oracle.num_threads()


def reference_arm(args):
    """The reference has no CPU implementation of this path (every functional
    wrapper raises NotImplementedError off-GPU), so its CPU arm is the oracle
    restatement, all host threads, on the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from minuet_b200 import synth
    coords, bd = synth.outdoor_batch(CLOUDS_PER_GPU, seed0=1000, n_voxels=VOXELS_PER_CLOUD)
    # a bounded sample: at most 4 builds per step, so that the driver's K steps end in minutes
    repeats = max(1, min(args.repeats, 4))
    value, ms, done, cores = run_cpu(args.steps, args.warmup, coords, bd, repeats=repeats)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT,
        "n_gpus": args.gpus, "steps": done, "warmup": args.warmup, "ms_per_step": round(ms, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int32",
        "data": "synthetic",
        "config": workload_config(len(coords), repeats),
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{done} steps of {repeats} builds (4 cold kernel maps each) of "
                                   "one 4-cloud batch"},
        "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def reference_cuda_arm(args):
    """Optional extra (not the contract's reference arm): the reference's OWN CUDA
    kernels, recompiled for sm_100 into oracle/_ref/libminuet_ref.so, timed on the
    same workload with CUDA events -- batched query + sizes + (stable order on the
    host side of the shim) + masks per map, plus arg-sort + unique for the strided
    target coordinates.  Prints one JSON line with impl = "reference-cuda"."""
    import torch
    from minuet_b200 import synth
    from minuet_b200.utils.helpers import generate_kernel_offsets
    path = os.path.join(ROOT, "oracle", "_ref", "libminuet_ref.so")
    if not os.path.exists(path) or not torch.cuda.is_available():
        print(json.dumps({"impl": "reference-cuda", "unavailable": "oracle/_ref library or GPU missing"}))
        return
    lib = ctypes.CDLL(path)
    lib.ref_last_error.restype = ctypes.c_char_p
    I64 = ctypes.c_int64
    dev = torch.device("cuda", 0)
    coords, bd = synth.outdoor_batch(CLOUDS_PER_GPU, seed0=1000, n_voxels=VOXELS_PER_CLOUD)
    S = len(coords)
    d_src = torch.as_tensor(coords, device=dev)
    d_sbd = torch.as_tensor(bd, device=dev, dtype=torch.int32)
    offs = {k: torch.as_tensor(generate_kernel_offsets(3, k, 1, 1).astype(np.int32), device=dev)
            for k in (2, 3)}

    def p(t):
        return ctypes.c_void_p(t.data_ptr())

    def ok(rc):
        if rc != 0:
            raise RuntimeError(lib.ref_last_error().decode())

    def step():
        # strided targets as KernelMapCache.get_target_coordinates does it
        floored = (d_src // 2) * 2
        index = torch.empty(S, dtype=torch.int32, device=dev)
        ok(lib.ref_multi_arg_sort(I64(S), I64(CLOUDS_PER_GPU), p(floored), p(d_sbd), p(index), 1, None))
        sorted_c = floored[index.long()].contiguous()
        uidx = torch.empty(S + 1, dtype=torch.int32, device=dev)
        uout = torch.empty((S, 3), dtype=torch.int32, device=dev)
        count = I64(0)
        ok(lib.ref_multi_unique(I64(S), I64(CLOUDS_PER_GPU + 1), p(sorted_c), p(d_sbd), p(uidx),
                                p(uout), ctypes.byref(count), None))
        tgt2 = uout[:count.value].contiguous()
        tbd2 = uidx[d_sbd.long()].contiguous()
        for kernel, stride in MAPS:
            tgt, tbd = (d_src, d_sbd) if stride == 1 else (tgt2, tbd2)
            O, T = kernel ** 3, tgt.shape[0]
            km = torch.empty((O, T), dtype=torch.int32, device=dev)
            ok(lib.ref_multi_query(I64(CLOUDS_PER_GPU), I64(O), p(d_sbd), p(tbd), p(d_src), p(tgt),
                                   p(offs[kernel]), p(km), None))
            sizes = torch.empty(O, dtype=torch.int32, device=dev)
            ok(lib.ref_sizes(I64(O), I64(T), p(km), p(sizes), None))
            sizes, order = torch.sort(sizes)
            km = km[order].contiguous()
            sm = torch.empty((O, S), dtype=torch.int32, device=dev)
            tm = torch.empty((O, T), dtype=torch.int32, device=dev)
            ok(lib.ref_masks(I64(O), I64(S), I64(T), p(km), p(sizes.int().contiguous()), p(sm), p(tm), None))

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(args.steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step()
        b.record()
        b.synchronize()
        total += a.elapsed_time(b)
    value = len(MAPS) * S * args.steps / (total * 1e-3) / 1e6
    print(json.dumps({"impl": "reference-cuda", "metric": METRIC, "value": round(value, 2),
                      "unit": UNIT, "n_gpus": 1, "steps": args.steps,
                      "ms_per_step": round(total / args.steps, 4),
                      "note": "reference's own CUDA kernels (CUB/cuBLAS based, no sm_100-specific "
                              "code) recompiled for sm_100a; same inputs, device-resident",
                      "config": workload_config(S)}), flush=True)


def workload_config(n_voxels_per_gpu, repeats=1):
    return {"workload": "C1 kernel-map build: 4 outdoor clouds x ~120k voxels per GPU, maps "
                        "(3^3,s1) (2^3,s1) (3^3,s2) (2^3,s2), cold cache, int32 coords",
            "voxels_per_gpu": int(n_voxels_per_gpu), "maps_per_build": len(MAPS),
            "builds_per_step": int(repeats),
            "l2": "flushed between timed steps (512 MiB write); every build writes ~0.22 GB of "
                  "masks, more than L2 holds, before the next one reads its inputs"}


def dram_traffic(kernel):
    """Measured DRAM bytes per build of one kernel name, from the committed table
    (columns: kernel, launches per build, read bytes, written bytes), or None."""
    if not os.path.exists(TRAFFIC_TABLE):
        return None
    with open(TRAFFIC_TABLE) as f:
        for row in f:
            cols = row.split()
            if len(cols) >= 4 and cols[0] == kernel:
                try:
                    return float(cols[2]) + float(cols[3])
                except ValueError:
                    return None
    return None


def profile_kernels(lib, fn, reps):
    """Per-kernel launch counts and device milliseconds (the library's own event pairs
    around every launch, on the launching stream) over ``reps`` calls of ``fn``."""
    import torch
    lib.mn_profile_enable(1)
    for _ in range(reps):
        fn()
    torch.cuda.synchronize()
    lib.mn_profile_enable(0)
    buf = ctypes.create_string_buffer(1 << 16)
    lib.mn_profile_report(buf, len(buf))
    out = {}
    for row in buf.value.decode().splitlines():
        name, count, ms = row.rsplit(" ", 2)
        out[name] = {"launches": int(count) / reps, "ms": float(ms) / reps}
    return out


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.proc = None
        self.path = None
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return
        fd, self.path = tempfile.mkstemp(suffix=".csv")
        os.close(fd)
        self.out = open(self.path, "w")
        self.proc = subprocess.Popen([exe, f"--query-gpu={self.FIELDS}", "--format=csv,noheader",
                                      "-i", str(gpu_index), "-lms", "50"],
                                     stdout=self.out, stderr=subprocess.DEVNULL)

    def stop(self, windows=()):
        """Median SM clock and throttle reasons over the samples that fall inside
        the given (start, end) wall-clock windows; all samples when none does."""
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.out.close()
        import datetime
        rows = []
        with open(self.path) as f:
            for row in f:
                cols = [c.strip() for c in row.split(",")]
                if len(cols) < 9:
                    continue
                try:
                    ts = datetime.datetime.strptime(cols[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    rows.append((ts, float(cols[1].split()[0]), float(cols[2].split()[0]),
                                 [c.lower().startswith("active") for c in cols[5:9]]))
                except ValueError:
                    continue
        os.unlink(self.path)
        if not rows:
            return None
        inside = [r for r in rows if any(a <= r[0] <= b for a, b in windows)]
        window = "timed region"
        if len(inside) < 3:
            inside, window = rows, "whole run (timed region shorter than the sampling period)"
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = sorted({n for r in inside for n, on in zip(names, r[3]) if on})
        return {"sm_mhz": float(np.median([r[1] for r in inside])),
                "sm_max_mhz": float(max(r[2] for r in inside)), "reasons": reasons,
                "samples": len(inside), "window": window}


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def kernel_bytes(name, S, T2, num_clouds):
    """Algorithmic bytes per BUILD of one kernel name, summed over its launches.
    S source voxels; T2 stride-2 target voxels; O = k^3 offsets per map."""
    T_of = {1: S, 2: T2}
    total = 0
    for kernel, stride in MAPS:
        O, T = kernel ** 3, T_of[stride]
        mirrored = stride == 1 and kernel % 2 == 1
        if name == "emit_masks_kernel":
            # hit words read, both masks and the row-ordered hit words written
            total += 4 * (S + T) + 4 * O * (S + T) + 4 * (S + T)
        elif name == "search_kernel<bits>" and mirrored:
            total += 8 * S + 4 * T                    # keys read once (S == T), words written
        elif name == "search_kernel<bits,rev>" and not mirrored:
            total += 8 * (S + T) + 4 * (S + T)        # both key arrays read, both word arrays written
    if name == "root_keys_kernel":
        total = 12 * S + 8 * S                        # coordinates read, packed keys written
    elif name == "radix_sort_kernel":
        total = 12 * S + 8 * S                        # coordinates read (floored + packed on the fly), sorted keys written
    elif name == "unique_keys_kernel":
        total = 8 * S + (12 + 8) * T2 + 8 * (num_clouds + 3)   # keys read, coordinates + keys written
    return total


def gpu_arm(args):
    import torch
    import minuet_b200 as minuet
    from minuet_b200 import _lib, engine, synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import datetime
        import torch.distributed as dist
        # a short collective timeout: a rank that fails must not hold the others for long
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))

    lib = _lib.load()
    R = max(1, args.repeats)
    coords, bd = synth.outdoor_batch(CLOUDS_PER_GPU, seed0=1000 + 100 * rank,
                                     n_voxels=VOXELS_PER_CLOUD)
    S = len(coords)
    h_coords = torch.from_numpy(coords).pin_memory()
    h_bd = torch.from_numpy(bd).pin_memory()
    d_coords, d_bd = h_coords.to(dev), h_bd.to(dev)
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=dev)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)

    def build(c, b):
        cache.reset()
        out = []
        for kernel, stride in MAPS:
            tc, ts, tbd = cache.get_target_coordinates(c, b, 1, stride)
            out.append(cache.get_kernel_map(c, 1, b, tc, ts, tbd, kernel, 1))
        return out

    def step():
        for _ in range(R):
            build(d_coords, d_bd)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """Per-step CUDA events on the current stream; L2 flushed between steps."""
        total = 0.0
        for _ in range(steps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            total += a.elapsed_time(b)
        return total

    sampler = ClockSampler(local) if rank == 0 else None
    for _ in range(max(args.warmup, 3)):
        step()
    T2 = int(cache.get_target_coordinates(d_coords, d_bd, 1, 2)[0].shape[0])
    engine.check_status(dev)

    # ---- device-resident inputs ------------------------------------------------
    barrier()
    launches0 = lib.mn_launch_count()
    w0 = time.time()
    ms_total = timed(step, args.steps)
    barrier()
    w1 = time.time()
    t_wall = w1 - w0
    launches = lib.mn_launch_count() - launches0

    # ---- host buffers in, sizes out (end to end) ---------------------------------
    # Double-buffered input pipeline: the copy of build i + 1's coordinates from pinned host
    # memory runs on a copy stream while build i computes, and the host reads build i's
    # results (per-offset sizes + status word of the four maps) after it has queued build
    # i + 1.  Every build's copy in and read back happen inside the timed region.
    copy_stream = torch.cuda.Stream(device=dev)
    slots = [(torch.empty_like(d_coords), torch.empty_like(d_bd)) for _ in range(2)]
    copied = [torch.cuda.Event() for _ in range(2)]
    released = [torch.cuda.Event() for _ in range(2)]

    def stage_inputs(i):
        c, b = slots[i % 2]
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(released[i % 2])     # the build that last read this slot is done
            c.copy_(h_coords, non_blocking=True)
            b.copy_(h_bd, non_blocking=True)
            copied[i % 2].record(copy_stream)

    def e2e_step():
        main = torch.cuda.current_stream(dev)
        for k in range(2):
            released[k].record(main)
        stage_inputs(0)
        got = pending = None
        for i in range(R):
            if i + 1 < R:
                stage_inputs(i + 1)
            main.wait_event(copied[i % 2])
            c, b = slots[i % 2]
            out = build(c, b)
            released[i % 2].record(main)
            # the masks stay on the GPU for the convolutions; what the host consumes per map
            # is the per-offset sizes (they size the GEMM problems) and the status word, which
            # every build already copies to pinned memory without a kernel of its own
            if pending is not None:
                got = [engine.host_copy(o[3]) for o in pending]
            pending = out
        got = [engine.host_copy(o[3]) for o in pending]
        return got

    for _ in range(2):
        e2e_step()
    barrier()
    w2 = time.time()
    ms_e2e = timed(e2e_step, args.steps)
    barrier()
    w3 = time.time()
    clocks = sampler.stop([(w0, w1), (w2, w3)]) if sampler is not None else None
    engine.check_status(dev)

    times = torch.tensor([ms_total, ms_e2e], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e = (float(v) for v in times.cpu())
    voxels_all = len(MAPS) * S * world
    if dist is not None:
        counts = torch.tensor([len(MAPS) * S], dtype=torch.int64, device=dev)
        dist.all_reduce(counts)
        voxels_all = int(counts.item())
    builds = args.steps * R
    value = voxels_all * builds / (ms_total * 1e-3) / 1e6
    e2e_value = voxels_all * builds / (ms_e2e * 1e-3) / 1e6

    unet = None
    if not args.no_unet:
        del flush
        torch.cuda.empty_cache()
        unet = unet_section(args, torch, dist, dev, rank, world, lib)
        flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- per-kernel times (separate, untimed pass) ---------------------------------
    # The library times every launch with an event pair on the launching stream.  A pair
    # also counts the time the stream sat idle before the launch reached the GPU, and the
    # host needs longer to prepare a launch than these kernels run, so each group of
    # launches is queued behind a few L2-flushing fills: the GPU is still busy with them
    # while the host enqueues the group, and the pairs then bracket execution only.
    def pad():
        for _ in range(4):
            flush.zero_()

    def cold_build():
        cache.reset()
        for kernel, stride in MAPS:
            pad()
            tc, ts, tbd = cache.get_target_coordinates(d_coords, d_bd, 1, stride)
            pad()
            cache.get_kernel_map(d_coords, 1, d_bd, tc, ts, tbd, kernel, 1)

    kernels = profile_kernels(lib, cold_build, 10)
    top = max(kernels, key=lambda k: kernels[k]["ms"])
    peaks, peak_kind = measured_peaks()
    hbm = peaks["hbm_gbs"]

    def line_of(name):
        nbytes = kernel_bytes(name, S, T2, CLOUDS_PER_GPU)
        ms = kernels[name]["ms"]
        gbs = nbytes / (ms * 1e-3) / 1e9 if nbytes and ms > 0 else None
        return {"kernel": name, "achieved": None if gbs is None else round(gbs, 1),
                "frac": None if gbs is None else round(gbs / hbm, 4),
                "algorithmic_bytes_per_build": nbytes, "kernel_ms_per_build": round(ms, 4),
                "launches_per_build": kernels[name]["launches"],
                "traffic": dram_traffic(name)}

    T_of = {1: S, 2: T2}
    stage_bytes = sum(12 * (S + T_of[s]) + 4 * k ** 3 * (S + T_of[s]) for k, s in MAPS)
    stage_bytes_with_map = stage_bytes + sum(4 * k ** 3 * T_of[s] for k, s in MAPS)
    gpu_ms = sum(v["ms"] for v in kernels.values())
    ms_build = ms_total / builds
    top_line = line_of(top)
    roofline = {
        "bound": "hbm", "kernel": top, "achieved": top_line["achieved"], "peak": hbm,
        "unit": "GB/s", "frac": top_line["frac"],
        "peak_source": ("measured (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured"
                        else "fallback 6650 GB/s"),
        # dram__bytes_read + dram__bytes_write of this kernel's launches of one build, from the
        # committed ncu table; null when the table has no row for the kernel
        "traffic": top_line["traffic"],
        "algorithmic_bytes_per_build": top_line["algorithmic_bytes_per_build"],
        "kernel_ms_per_build": top_line["kernel_ms_per_build"],
        "launches_per_build": top_line["launches_per_build"],
        "whole_step": {
            "algorithmic_bytes_fused": stage_bytes,
            "algorithmic_bytes_with_kernel_map": stage_bytes_with_map,
            "gpu_busy_ms": round(gpu_ms, 4),
            "gbs_over_gpu_busy_time": round(stage_bytes / (gpu_ms * 1e-3) / 1e9, 1),
            "gbs_over_step_time": round(stage_bytes / (ms_build * 1e-3) / 1e9, 1),
            "frac_over_step_time": round(stage_bytes / (ms_build * 1e-3) / 1e9 / hbm, 4),
        },
        # the kernel that moves most of the build's bytes, next to the one that takes most time
        "byte_dominant_kernel": line_of("emit_masks_kernel") if "emit_masks_kernel" in kernels else None,
        "kernels": [line_of(k) for k in sorted(kernels, key=lambda k: -kernels[k]["ms"])],
    }

    # ---- CPU baseline on this box's host cores (bounded) ---------------------------
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        v, ms, done, cores = run_cpu(3, 1, coords, bd, min_seconds=10.0)
        cpu = {"value": round(v, 3), "unit": UNIT, "cores": cores, "kind": "port",
               "sample": f"{done} builds of the same 4-cloud batch ({ms:.1f} ms per build)"}

    sweep = None
    if world == 1 and not args.no_gms_sweep:
        chans = tuple(int(c) for c in args.gms_channels.split(","))
        sweep = gms_sweep(torch, minuet, lib, cache, d_coords, d_bd, channels=chans)
        # the same sweep on the single 50 000-voxel uniform cloud of the fp32 configuration
        u_coords = torch.from_numpy(synth.uniform_cloud()).to(dev)
        u_cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=dev)
        sweep["uniform50k"] = gms_sweep(torch, minuet, lib, u_cache, u_coords, None, channels=chans)
        sweep["uniform50k"]["map"] = "3^3 stride 1 on 50 000 uniform voxels in [0,256)^3"

    h2d = h_coords.numel() * 4 + h_bd.numel() * 8
    # per build: sizes + status word of every map, and the stride-2 level's counts
    d2h = sum((k ** 3 + 1) * 4 for k, _ in MAPS) + (CLOUDS_PER_GPU + 3) * 8
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_total / args.steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int32", "data": "synthetic",
        "config": workload_config(S, R),
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": int(h2d * R),
                "d2h_bytes_per_step": int(d2h * R), "ms_per_step": round(ms_e2e / args.steps, 4),
                "returns": "per-offset pair counts of the four maps and the status word"},
        "gpu_launches": int(launches),
        "ms_per_build": round(ms_build, 4),
        "roofline": roofline,
        "cpu_baseline": cpu,
        "gms_sweep": sweep,
        "unet": unet,
        "wall_s": round(t_wall, 3),
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def gms_sweep(torch, minuet, lib, cache, d_coords, d_bd, channels=(16, 32, 64, 128, 256), rounds=5):
    """Gather / grouped GEMM / scatter on the 3^3 stride-1 map of the given batch, fp16
    features and weights (fp32 accumulate), per channel width:

    * the three stage kernels behind the reference's timers (cuda_time_gather / _gemm /
      _scatter), gather and scatter at the fastest tile size among the divisors of C (what
      the layer autotuner picks), charged with the bytes the kernel must move on THIS map
      (rows that have a pair) and, beside it, with the fusion-agnostic stage formula;
    * the whole layer through the two forward paths that 16-bit layers actually take (pair
      lists, fused implicit GEMM at its best sub-tile count), against the layer's bound.
    """
    from minuet_b200 import engine
    from minuet_b200.nn import functional as F
    peaks, _ = measured_peaks()
    hbm, tensor = peaks["hbm_gbs"], peaks["bf16_tflops"]
    tc = cache.get_target_coordinates(d_coords, d_bd, 1, 1)
    sm, tm, order, sizes = cache.get_kernel_map(d_coords, 1, d_bd, tc[0], tc[1], tc[2], 3, 1)
    h_sizes = engine.host_copy(sizes)
    S = T = d_coords.shape[0]
    O = len(h_sizes)
    E = int(h_sizes.sum())
    E1, O1 = E - int(h_sizes[-1]), O - 1            # the centre offset takes the shortcut
    centre = 1 << (O - 1)                            # its bit in the row-ordered hit words
    s_hit = int((engine.hit_bits(sm) & ~centre).ne(0).sum())
    t_hit = int((engine.hit_bits(tm) & ~centre).ne(0).sum())

    def per_launch(names, fn):
        got = profile_kernels(lib, fn, rounds)
        ms = [got[n]["ms"] for n in names if n in got]
        return sum(ms) if ms else float("nan")

    def frac(value, peak):
        f = value / peak
        return {"frac": round(f, 3)} if f <= 1.2 else {
            "frac": round(f, 3), "suspect": "above 1.2 of the measured peak: the charged bytes "
                                            "overstate what the kernel moved"}

    out = {}
    for c in channels:
        w = torch.randn(O, c, c, device=d_coords.device).half()
        kw = dict(weights=w, source_masks=sm, target_masks=tm, kernel_map_sizes=sizes,
                  allow_shortcut_matmul=True)
        divisors = [t for t in range(1, c + 1) if c % t == 0]
        best = {}
        for stage, fn, kernel in (("gather", F.cuda_time_gather, "gather_kernel"),
                                  ("scatter", F.cuda_time_scatter, "scatter_kernel")):
            fn(tile_size=1, **kw)
            for t in divisors:
                ms = per_launch([kernel], lambda: fn(tile_size=t, **kw))
                if stage not in best or ms < best[stage][1]:
                    best[stage] = (t, ms)
        F.cuda_time_gemm(**kw)
        gemm_ms = per_launch(["gemm_tc_kernel", "gemm_simt_kernel"], lambda: F.cuda_time_gemm(**kw))
        # bytes the stage must move on this map / the stage formula over all S (or T) rows
        g_honest = s_hit * c * 2 + E1 * c * 2 + 4 * E1
        g_survey = S * c * 2 + 4 * O1 * S + E1 * c * 2
        s_honest = E1 * c * 2 + T * c * 2 + 4 * E1
        s_survey = E1 * c * 2 + 4 * O1 * T + T * c * 2
        flops = 2.0 * E * c * c
        gemm_bytes = E * 2 * c * 2 + O * c * c * 2
        tg, ts = best["gather"][1], best["scatter"][1]
        row = {
            "gather": {"tile_size": best["gather"][0], "ms": round(tg, 4),
                       "bytes_on_this_map": g_honest, "gbs": round(g_honest / tg / 1e6, 1),
                       **frac(g_honest / tg / 1e6, hbm),
                       "bytes_stage_formula": g_survey,
                       "gbs_stage_formula": round(g_survey / tg / 1e6, 1)},
            "scatter": {"tile_size": best["scatter"][0], "ms": round(ts, 4),
                        "bytes_on_this_map": s_honest, "gbs": round(s_honest / ts / 1e6, 1),
                        **frac(s_honest / ts / 1e6, hbm),
                        "bytes_stage_formula": s_survey,
                        "gbs_stage_formula": round(s_survey / ts / 1e6, 1)},
            "gemm": {"ms": round(gemm_ms, 4), "tflops": round(flops / gemm_ms / 1e9, 2),
                     "frac_tensor": round(flops / gemm_ms / 1e9 / tensor, 4),
                     "gbs": round(gemm_bytes / gemm_ms / 1e6, 1),
                     "frac_hbm": round(gemm_bytes / gemm_ms / 1e6 / hbm, 3),
                     "bound": "hbm" if c <= 32 else "tensor"},
        }
        # whole layer, the paths 16-bit layers take
        layer = {}
        fw = dict(weights=w, source_masks=sm, target_masks=tm, kernel_map_order=order,
                  kernel_map_sizes=sizes, allow_shortcut_matmul=True)
        code = engine.dtype_code(w.dtype)
        if lib.mn_pairs_supported(O, c, c, code):
            F.time_forward(algorithm="explicit", **fw)
            layer["pairs_ms"] = round(float(np.mean(
                [F.time_forward(algorithm="explicit", **fw) for _ in range(rounds)])), 4)
            got = profile_kernels(lib, lambda: F.time_forward(algorithm="explicit", **fw), rounds)
            layer["pairs_kernels_ms"] = {k: round(v["ms"], 4) for k, v in got.items()}
        if lib.mn_implicit_supported(O, c, c, code):
            n_pad = -(-c // 16) * 16
            for sub in (1, 2, 3, 4):
                if sub * n_pad > 512:
                    break
                F.time_forward(algorithm="implicit", sub_tiles=sub, **fw)
                ms = float(np.mean([F.time_forward(algorithm="implicit", sub_tiles=sub, **fw)
                                    for _ in range(rounds)]))
                if "implicit_ms" not in layer or ms < layer["implicit_ms"]:
                    layer["implicit_ms"], layer["implicit_sub_tiles"] = round(ms, 4), sub
        if layer:
            best_ms = min(v for k, v in layer.items() if k in ("pairs_ms", "implicit_ms"))
            bound_bytes = S * c * 2 + T * c * 2 + O * c * c * 2 + 4 * O * (S + T)
            bound_ms = max(bound_bytes / hbm / 1e6, flops / tensor / 1e9)
            layer.update(best_ms=best_ms, tflops=round(flops / best_ms / 1e9, 2),
                         frac_tensor=round(flops / best_ms / 1e9 / tensor, 4),
                         bound_ms=round(bound_ms, 4), frac_of_bound=round(bound_ms / best_ms, 3))
        row["layer"] = layer
        out[str(c)] = row
    return {"map": "3^3 stride 1 on the benchmark batch", "S": int(S), "pairs": E,
            "pairs_without_centre": E1, "source_rows_with_a_pair": s_hit,
            "target_rows_with_a_pair": t_hit, "dtype": "f16", "channels": out}


UNET_CLOUDS = 64          # C4: 64 outdoor clouds in total, sharded over the ranks
UNET_SEED0 = 3000


def _make_cloud(seed):
    from minuet_b200 import synth
    return synth.outdoor_cloud(seed, VOXELS_PER_CLOUD)


def _make_indoor_cloud(seed):
    from minuet_b200 import synth
    return synth.indoor_cloud(seed, 200_000)


def layer_bound(entry, hbm_gbs, tensor_tflops, elem=2):
    """Fusion-agnostic lower bound of one convolution layer: every operand crosses HBM
    once (features in, features out, weights, one 32-bit word per mask entry) against
    2 E c_in c_out flops on the tensor pipe.  Returns (bytes, flops, milliseconds)."""
    S, T, O, E = entry["S"], entry["T"], entry["O"], entry["E"]
    ci, co = entry["c_in"], entry["c_out"]
    nbytes = S * ci * elem + T * co * elem + O * ci * co * elem + (4 * O * (S + T) if O > 1 else 0)
    flops = 2.0 * E * ci * co
    return nbytes, flops, max(nbytes / hbm_gbs / 1e6, flops / tensor_tflops / 1e9)


def unet_section(args, torch, dist, dev, rank, world, lib):
    """Sparse UNet (fp16, random weights, eval-mode BatchNorm) on 64 outdoor clouds
    sharded by cloud over the ranks; the per-voxel outputs are gathered on rank 0 with
    point-to-point NCCL messages.  Strong scaling: the 64 clouds are the whole job at
    every N."""
    import concurrent.futures
    import minuet_b200 as minuet
    from minuet_b200 import engine, sharding
    from minuet_b200.unet import SparseUNet

    indoor = args.unet_config == "c3"       # C3: 8 indoor scenes x 200k voxels, RGB features
    n_clouds = 8 if indoor and args.unet_clouds == UNET_CLOUDS else args.unet_clouds
    per_cloud = 200_000 if indoor else VOXELS_PER_CLOUD
    shards = sharding.assign_clouds([per_cloud] * n_clouds, world)
    mine = shards[rank]
    with concurrent.futures.ProcessPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as pool:
        if indoor:
            clouds = list(pool.map(_make_indoor_cloud, [2000 + i for i in mine]))
        else:
            clouds = list(pool.map(_make_cloud, [UNET_SEED0 + i for i in mine]))
    coords = np.ascontiguousarray(np.concatenate(clouds).astype(np.int32))
    bd = np.zeros(len(clouds) + 1, dtype=np.int64)
    bd[1:] = np.cumsum([len(c) for c in clouds])
    rng = np.random.default_rng(UNET_SEED0 + 7919 * rank)
    if indoor:
        feats = rng.random((len(coords), 3), dtype=np.float32)
    else:
        feats = np.concatenate([coords.astype(np.float32) * 0.05,
                                rng.random((len(coords), 1), dtype=np.float32)], axis=1)
    h_coords = torch.from_numpy(coords).pin_memory()
    h_bd = torch.from_numpy(bd).pin_memory()
    h_feats = torch.from_numpy(feats).half().pin_memory()
    d_coords, d_bd, d_feats = h_coords.to(dev), h_bd.to(dev), h_feats.to(dev)
    # the generators make clouds of exactly per_cloud voxels, so every rank knows every
    # rank's row count from the shard plan and the gather needs no count exchange
    assert len(coords) == per_cloud * len(mine)
    rows_per_rank = [per_cloud * len(s) for s in shards]

    torch.manual_seed(0)
    net = SparseUNet(feats.shape[1], num_classes=20).to(dev).half().eval().fuse()
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=dev)
    minuet.set_kernel_map_cache(net, cache)

    def local_forward(c, b, f):
        cache.reset()
        with torch.no_grad():
            return net(minuet.SparseTensor(f, c, batch_dims=b))

    def forward(c, b, f, labels=False):
        out = local_forward(c, b, f).F
        if labels:          # class labels: one byte per voxel instead of 20 fp16 logits
            out = out.argmax(dim=1, keepdim=True).to(torch.uint8)
        if dist is not None:
            return sharding.gather_rows(out, dst=0, counts=rows_per_rank)   # every rank calls it
        return [out]

    def timed(fn, steps):
        total = 0.0
        for _ in range(steps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            if dist is not None:
                dist.barrier()
            a.record()
            fn()
            b.record()
            b.synchronize()
            total += a.elapsed_time(b)
        return total

    # per-layer tuning on this rank's shard (pair lists against the fused kernel, sub-tiles)
    tuned = None
    if not args.no_autotune:
        rounds = minuet.nn.SparseConv.__NUM_TUNING_ROUNDS__
        minuet.nn.SparseConv.__NUM_TUNING_ROUNDS__ = 3
        try:
            minuet.autotune(net, cache, [minuet.SparseTensor(d_feats, d_coords, batch_dims=d_bd)])
        finally:
            minuet.nn.SparseConv.__NUM_TUNING_ROUNDS__ = rounds
        tuned = {}
        for m in net.modules():
            if isinstance(m, minuet.nn.SparseConv) and not m.is_trivial:
                key = f"{m.tunable_config['algorithm']}/{m.tunable_config['sub_tiles']}"
                tuned[key] = tuned.get(key, 0) + 1

    steps, warm = args.unet_steps, 3
    for _ in range(warm):
        forward(d_coords, d_bd, d_feats)
    engine.check_status(dev)
    launches0 = lib.mn_launch_count()
    ms = timed(lambda: forward(d_coords, d_bd, d_feats), steps)
    launches = lib.mn_launch_count() - launches0

    def e2e():
        c = h_coords.to(dev, non_blocking=True)
        b = h_bd.to(dev, non_blocking=True)
        f = h_feats.to(dev, non_blocking=True)
        parts = forward(c, b, f, labels=True)
        if parts is not None:      # rank 0: per-voxel class labels go back to the host
            return [p.cpu() for p in parts]
        return None

    e2e()
    ms_e2e = timed(e2e, steps)
    engine.check_status(dev)
    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = (float(v) for v in t.cpu())

    kernels = roofline = None
    if rank == 0:
        got = profile_kernels(lib, lambda: local_forward(d_coords, d_bd, d_feats), 1)   # rank-local
        kernels = {k: {"launches": int(v["launches"]), "ms": round(v["ms"], 4)}
                   for k, v in sorted(got.items(), key=lambda kv: -kv[1]["ms"])}
        # per-layer shapes and device times of one more rank-local forward
        peaks, peak_kind = measured_peaks()
        hbm, tensor = peaks["hbm_gbs"], peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
        engine.LAYER_LOG = []
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        local_forward(d_coords, d_bd, d_feats)
        b.record()
        torch.cuda.synchronize()
        log, engine.LAYER_LOG = engine.LAYER_LOG, None
        local_ms = a.elapsed_time(b)
        layers, sum_bytes, sum_flops, sum_bound, sum_meas = [], 0, 0.0, 0.0, 0.0
        for e in log:
            nbytes, flops, bound = layer_bound(e, hbm, tensor)
            meas = e["events"][0].elapsed_time(e["events"][1])
            sum_bytes += nbytes
            sum_flops += flops
            sum_bound += bound
            sum_meas += meas
            # fused layers: pairs / (128 rows x (tile, offset) stages issued) = the share of the
            # MMA rows that carry a pair (the rest are zero rows of tiles that hold the offset)
            useful = None
            if e.get("tile_bits") is not None:
                tb = e["tile_bits"].to(torch.int64) & 0xffffffff
                stages_issued = int(((tb[:, None] >> torch.arange(32, device=tb.device)) & 1).sum())
                useful = round(e["E"] / max(128 * stages_issued, 1), 3)
            layers.append([e["S"], e["T"], e["O"], e["E"], e["c_in"], e["c_out"], e["algorithm"],
                           round(bound, 4), round(meas, 4), useful])
        # the nine kernel maps of the forward (one per stride level and kernel size)
        map_bytes = 0
        seen = set()
        for e in log:
            key = (min(e["S"], e["T"]), max(e["S"], e["T"]), e["O"])
            if e["O"] > 1 and key not in seen:
                seen.add(key)
                map_bytes += 12 * (e["S"] + e["T"]) + 4 * e["O"] * (e["S"] + e["T"])
        map_bound = map_bytes / hbm / 1e6
        roofline = {
            "bound": "per layer max(bytes / HBM, flops / tensor), summed; kernel maps at HBM",
            "peak_hbm_gbs": hbm, "peak_tensor_tflops": tensor,
            "peak_source": peak_kind + (" (sustained bf16 figure: the layers run inside a long step)"
                                        if "bf16_tflops_sustained" in peaks else ""),
            "layer_columns": ["S", "T", "O", "E", "c_in", "c_out", "algorithm", "bound_ms",
                              "measured_ms", "useful_mma_row_fraction"],
            "layers": layers,
            "sum_layer_bytes": int(sum_bytes), "sum_layer_flops": sum_flops,
            "sum_layer_bound_ms": round(sum_bound, 3), "sum_layer_measured_ms": round(sum_meas, 3),
            "kernel_maps": len(seen), "kernel_map_bytes": int(map_bytes),
            "kernel_map_bound_ms": round(map_bound, 3),
            "forward_ms_rank0_shard": round(local_ms, 3),
            "frac": round((sum_bound + map_bound) / local_ms, 4),
            "achieved_tflops": round(sum_flops / local_ms / 1e9, 2),
        }

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = unet_cpu_baseline(torch, feats.shape[1], clouds[0], feats[:len(clouds[0])])
    if dist is not None:
        dist.barrier()
    if rank != 0:
        return None
    out_bytes = sum(rows_per_rank)
    return {
        "metric": "sparse-UNet fp16 clouds/sec", "value": round(n_clouds * steps / (ms * 1e-3), 2),
        "unit": "clouds/s", "scaling": "strong", "ms_per_step": round(ms / steps, 3),
        "steps": steps, "warmup": warm,
        "config": {"workload": ("C3: UNet on 8 indoor scenes x 200k voxels, RGB fp16 features"
                                if indoor else
                                "C4: UNet (stem 32, encoder 32/64/128/256, decoder mirror, 20 "
                                "classes) on 64 outdoor clouds x 120k voxels, 4-channel fp16 "
                                "features") + ", clouds sharded over the GPUs; rank 0 receives "
                               "every rank's fp16 logits (device-resident leg) or uint8 class "
                               "labels (end-to-end leg) as point-to-point NCCL messages",
                   "clouds_total": n_clouds, "clouds_on_rank0": len(mine),
                   "voxels_on_rank0": int(len(coords)), "autotuned_layers": tuned},
        "e2e": {"value": round(n_clouds * steps / (ms_e2e * 1e-3), 2), "unit": "clouds/s",
                "ms_per_step": round(ms_e2e / steps, 3),
                "h2d_bytes_per_step": int(h_coords.numel() * 4 + h_bd.numel() * 8 + h_feats.numel() * 2),
                "d2h_bytes_per_step": int(out_bytes),
                "returns": "one uint8 class label per voxel of all clouds, on rank 0's host"},
        "gpu_launches": int(launches),
        "library_launches_per_forward": int(launches / max(steps, 1)),
        "blocking_host_reads_per_forward": 4,   # one unique count per stride level, all in SparseUNet.plan
        "roofline": roofline,
        "cpu_baseline": cpu,
        "library_kernel_ms_rank0_one_step": kernels,
    }


def unet_cpu_baseline(torch, in_channels, cloud, feats):
    """The same network, layer by layer, through the CPU restatement (kernel maps and
    convolutions in C++/OpenMP with fp64 accumulation, BatchNorm/ReLU/concat in numpy)
    on ONE cloud of the batch."""
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    os.environ["OMP_NUM_THREADS"] = str(cores)
    import oracle
    from oracle.net import OracleNet
    from minuet_b200.unet import SparseUNet
    oracle.build()
    oracle.set_num_threads(cores)
    torch.manual_seed(0)
    net = SparseUNet(in_channels, num_classes=20).half().eval()
    f0 = torch.from_numpy(feats).half().float().numpy()
    c0 = np.ascontiguousarray(cloud.astype(np.int32))
    t0 = time.perf_counter()
    done = 0
    while done < 1 or time.perf_counter() - t0 < 10.0:
        OracleNet(oracle, round_to=torch.float16).forward(net, (f0, c0, 1, None))
        done += 1
    dt = time.perf_counter() - t0
    return {"value": round(done / dt, 4), "unit": "clouds/s", "cores": oracle.num_threads(),
            "kind": "port",
            "sample": f"{done} forward passes of one {len(c0)}-voxel cloud of the batch "
                      f"({dt / done:.2f} s each), cold kernel maps every pass"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "reference-cuda"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-unet", action="store_true",
                    help="skip the secondary end-to-end UNet measurement")
    ap.add_argument("--unet-steps", type=int, default=5)
    ap.add_argument("--no-autotune", action="store_true",
                    help="UNet layers keep the cost-model choice instead of being timed")
    ap.add_argument("--unet-clouds", type=int, default=UNET_CLOUDS,
                    help="clouds in the UNet job (64 = the benchmark configuration)")
    ap.add_argument("--gms-channels", default="16,32,64,128,256")
    ap.add_argument("--unet-config", default="c4", choices=["c3", "c4"],
                    help="c4: 64 outdoor clouds (default); c3: 8 indoor scenes with RGB features")
    ap.add_argument("--no-gms-sweep", action="store_true",
                    help="skip the gather / grouped GEMM / scatter sweep over C in 16..256 (fp16)")
    ap.add_argument("--repeats", type=int, default=32,
                    help="cold builds of the four maps per timed step")
    args = ap.parse_args()
    if args.impl == "reference-cuda":
        reference_cuda_arm(args)
    elif args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
