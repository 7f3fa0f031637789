"""Benchmark of the Map step (kernel-map build) on synthetic outdoor clouds.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload: a batch of 4 outdoor-scan-like clouds of 120 000 voxels per GPU; one
step builds, on a cold KernelMapCache, the four kernel maps
(kernel 3^3 / 2^3) x (stride 1 / 2), including the strided target coordinates
(floor, sort, unique).  The metric is source voxels processed per second, summed
over the four maps (Mvoxels/s).  With N > 1 every rank owns its own batch (weak
scaling, no collective on the data path); the time is the max over ranks.

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


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


# ---------------------------------------------------------------------------
# CPU arm: the oracle restatement on the host cores
# ---------------------------------------------------------------------------
def oracle_step(oracle, coords, bd, offsets):
    tgt2, tbd2 = oracle.downsample(coords, 2, bd)
    out = []
    for kernel, stride in MAPS:
        tgt, tbd = (coords, bd) if stride == 1 else (tgt2, tbd2)
        out.append(oracle.build_kernel_map(coords, tgt, offsets[kernel], bd, tbd))
    return out


def run_cpu(steps, warmup, coords, bd, min_seconds=0.0):
    # torchrun exports OMP_NUM_THREADS=1; the CPU arm uses every core this process may run on
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    os.environ["OMP_NUM_THREADS"] = str(cores)
    import oracle
    from minuet_b200.utils.helpers import generate_kernel_offsets
    oracle.build()
    oracle.set_num_threads(cores)
    offsets = {k: generate_kernel_offsets(3, k, 1, 1).astype(np.int32) for k in (2, 3)}
    for _ in range(warmup):
        oracle_step(oracle, coords, bd, offsets)
    t0 = time.perf_counter()
    done = 0
    while done < steps or time.perf_counter() - t0 < min_seconds:
        oracle_step(oracle, coords, bd, offsets)
        done += 1
    dt = time.perf_counter() - t0
    voxels = len(MAPS) * len(coords) * done
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
    value, ms, done, cores = run_cpu(args.steps, args.warmup, coords, bd)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT,
        "n_gpus": args.gpus, "steps": done, "warmup": args.warmup, "ms_per_step": round(ms, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int32",
        "data": "synthetic",
        "config": workload_config(len(coords)),
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{done} full steps (4 cold map builds of one 4-cloud batch)"},
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


def workload_config(n_voxels_per_gpu):
    return {"workload": "C1 kernel-map build: 4 outdoor clouds x ~120k voxels per GPU, maps "
                        "(3^3,s1) (2^3,s1) (3^3,s2) (2^3,s2), cold cache, int32 coords",
            "voxels_per_gpu": int(n_voxels_per_gpu), "maps_per_step": len(MAPS),
            "l2": "flushed between timed steps (512 MiB write); per-step outputs ~0.5 GB > L2"}


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
                                      "-i", str(gpu_index), "-lms", "100"],
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
def kernel_bytes(name, S, T_by_stride, num_clouds):
    """Algorithmic bytes per step of one kernel name, summed over its launches.
    S source voxels; T target voxels per kernel stride; O = k^3."""
    total = 0
    for kernel, stride in MAPS:
        O, T = kernel ** 3, T_by_stride[stride]
        mirrored = stride == 1 and kernel % 2 == 1
        if name == "emit_masks_kernel":
            total += 4 * O * (S + T) + 4 * (S + T)          # masks written, hit words read
        elif name == "search_kernel<bits>":
            total += 8 * (S + T) + 4 * T + 4 * O * ((T + 1023) // 1024)   # keys read, words + counts written
            if not mirrored:
                total += 8 * (S + T) + 4 * S + 4 * O * ((S + 1023) // 1024)
    if name == "pack_kernel":
        total = (12 + 8) * S * 2                              # source keys + floored keys
    return total


def gpu_arm(args):
    import torch
    import minuet_b200 as minuet
    from minuet_b200 import _lib, synth

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
    coords, bd = synth.outdoor_batch(CLOUDS_PER_GPU, seed0=1000 + 100 * rank,
                                     n_voxels=VOXELS_PER_CLOUD)
    S = len(coords)
    h_coords = torch.from_numpy(coords).pin_memory()
    h_bd = torch.from_numpy(bd).pin_memory()
    d_coords, d_bd = h_coords.to(dev), h_bd.to(dev)
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=dev)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)

    def step(c, b):
        cache.reset()
        out = []
        for kernel, stride in MAPS:
            tc, ts, tbd = cache.get_target_coordinates(c, b, 1, stride)
            out.append(cache.get_kernel_map(c, 1, b, tc, ts, tbd, kernel, 1))
        return out

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
        step(d_coords, d_bd)
    T_by_stride = {1: S, 2: int(cache.get_target_coordinates(d_coords, d_bd, 1, 2)[0].shape[0])}

    # ---- device-resident inputs ------------------------------------------------
    barrier()
    launches0 = lib.mn_launch_count()
    w0 = time.time()
    ms_total = timed(lambda: step(d_coords, d_bd), args.steps)
    barrier()
    w1 = time.time()
    t_wall = w1 - w0
    launches = lib.mn_launch_count() - launches0

    # ---- host buffers in, sizes/order out (end to end) ---------------------------
    def e2e_step():
        c = h_coords.to(dev, non_blocking=True)
        b = h_bd.to(dev, non_blocking=True)
        out = step(c, b)
        # the masks stay on the GPU for the convolutions; what the host consumes
        # per map is the size-sorted order
        return torch.cat([o[2] for o in out]).cpu()      # one read for the four maps

    for _ in range(2):
        e2e_step()
    barrier()
    w2 = time.time()
    ms_e2e = timed(e2e_step, args.steps)
    barrier()
    w3 = time.time()
    clocks = sampler.stop([(w0, w1), (w2, w3)]) if sampler is not None else None

    times = torch.tensor([ms_total, ms_e2e], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e = (float(v) for v in times.cpu())
    voxels_all = len(MAPS) * S * world      # every rank holds S voxels (same generator sizes)
    if dist is not None:
        counts = torch.tensor([len(MAPS) * S], dtype=torch.int64, device=dev)
        dist.all_reduce(counts)
        voxels_all = int(counts.item())
    value = voxels_all * args.steps / (ms_total * 1e-3) / 1e6
    e2e_value = voxels_all * args.steps / (ms_e2e * 1e-3) / 1e6

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
    lib.mn_profile_enable(1)
    prof_steps = 5
    for _ in range(prof_steps):
        flush.zero_()
        step(d_coords, d_bd)
    torch.cuda.synchronize()
    lib.mn_profile_enable(0)
    buf = ctypes.create_string_buffer(1 << 16)
    lib.mn_profile_report(buf, len(buf))
    kernels = {}
    for row in buf.value.decode().splitlines():
        name, count, ms = row.rsplit(" ", 2)
        kernels[name] = {"launches_per_step": int(count) / prof_steps,
                         "ms_per_step": float(ms) / prof_steps}
    top = max(kernels, key=lambda k: kernels[k]["ms_per_step"])
    peaks, peak_kind = measured_peaks()
    top_bytes = kernel_bytes(top, S, T_by_stride, CLOUDS_PER_GPU)
    top_ms = kernels[top]["ms_per_step"]
    achieved = top_bytes / (top_ms * 1e-3) / 1e9 if top_bytes else None
    stage_bytes = sum(12 * (S + T_by_stride[s]) + 4 * k ** 3 * (S + T_by_stride[s]) for k, s in MAPS)
    stage_bytes_with_map = stage_bytes + sum(4 * k ** 3 * T_by_stride[s] for k, s in MAPS)
    gpu_ms = sum(v["ms_per_step"] for v in kernels.values())
    # the kernel that moves most of the step's bytes (the mask emission) next to the
    # kernel that takes most of its time (the search, which is instruction bound)
    byte_dominant = None
    if "emit_masks_kernel" in kernels:
        eb = kernel_bytes("emit_masks_kernel", S, T_by_stride, CLOUDS_PER_GPU)
        ems = kernels["emit_masks_kernel"]["ms_per_step"]
        byte_dominant = {"kernel": "emit_masks_kernel", "algorithmic_bytes_per_step": eb,
                         "kernel_ms_per_step": round(ems, 4),
                         "achieved": round(eb / (ems * 1e-3) / 1e9, 1), "unit": "GB/s",
                         "frac": round(eb / (ems * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)}
    roofline = {
        "bound": "hbm", "kernel": top,
        "achieved": None if achieved is None else round(achieved, 1),
        "peak": peaks["hbm_gbs"], "unit": "GB/s",
        "frac": None if achieved is None else round(achieved / peaks["hbm_gbs"], 4),
        "peak_source": peak_kind + " (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured"
        else "fallback 6650 GB/s",
        # dram__bytes_read + dram__bytes_write of the search launches of one step under ncu
        # (3.9 MB read per search direction, 7 directions; the hit words and tile counts they
        # write were still in L2 when the kernels ended), profiles/search_and_emit_kernels_C1.md
        "traffic": 27.3e6 if top.startswith("search_kernel") else None,
        "algorithmic_bytes_per_step": top_bytes,
        "kernel_ms_per_step": round(top_ms, 4),
        "launches_per_step": kernels[top]["launches_per_step"],
        "whole_step": {
            "algorithmic_bytes_fused": stage_bytes,
            "algorithmic_bytes_with_kernel_map": stage_bytes_with_map,
            "gpu_busy_ms": round(gpu_ms, 4),
            "gbs_over_gpu_busy_time": round(stage_bytes / (gpu_ms * 1e-3) / 1e9, 1),
            "gbs_over_step_time": round(stage_bytes / (ms_total / args.steps * 1e-3) / 1e9, 1),
        },
        "byte_dominant_kernel": byte_dominant,
        "kernels": {k: {"ms_per_step": round(v["ms_per_step"], 4),
                        "launches_per_step": v["launches_per_step"]}
                    for k, v in sorted(kernels.items(), key=lambda kv: -kv[1]["ms_per_step"])},
    }

    # ---- CPU baseline on this box's host cores (bounded) ---------------------------
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        v, ms, done, cores = run_cpu(3, 1, coords, bd, min_seconds=10.0)
        cpu = {"value": round(v, 3), "unit": UNIT, "cores": cores, "kind": "port",
               "sample": f"{done} full steps of the same 4-cloud batch ({ms:.1f} ms/step)"}

    sweep = None
    if world == 1 and args.gms_sweep:
        chans = tuple(int(c) for c in args.gms_channels.split(","))
        sweep = gms_sweep(torch, minuet, cache, d_coords, d_bd, channels=chans)
        # the same sweep on the single 50 000-voxel uniform cloud of the fp32 configuration
        u_coords = torch.from_numpy(synth.uniform_cloud()).to(dev)
        u_cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=dev)
        sweep["uniform50k"] = gms_sweep(torch, minuet, u_cache, u_coords, None, channels=chans)
        sweep["uniform50k"]["map"] = "3^3 stride 1 on 50 000 uniform voxels in [0,256)^3"

    h2d = h_coords.numel() * 4 + h_bd.numel() * 8
    d2h = sum((k ** 3 + 1) * 4 + k ** 3 * 4 for k, _ in MAPS) + (CLOUDS_PER_GPU + 3) * 8 + 32
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_total / args.steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int32", "data": "synthetic",
        "config": workload_config(S),
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h), "ms_per_step": round(ms_e2e / args.steps, 4)},
        "gpu_launches": int(launches),
        "roofline": roofline,
        "cpu_baseline": cpu,
        "gms_sweep": sweep,
        "unet": unet,
        "wall_s": round(t_wall, 3),
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def gms_sweep(torch, minuet, cache, d_coords, d_bd, channels=(16, 32, 64, 128, 256), rounds=5):
    """Gather / grouped GEMM / scatter stage times on the 3^3 stride-1 map of the
    benchmark batch, fp16 features and weights (fp32 accumulate)."""
    from minuet_b200 import engine
    from minuet_b200.nn import functional as F
    peaks, _ = measured_peaks()
    tc = cache.get_target_coordinates(d_coords, d_bd, 1, 1)
    sm, tm, order, sizes = cache.get_kernel_map(d_coords, 1, d_bd, tc[0], tc[1], tc[2], 3, 1)
    h_sizes = engine.host_copy(sizes)
    S = T = d_coords.shape[0]
    O = len(h_sizes)
    E = int(h_sizes.sum())
    E1, O1 = E - int(h_sizes[-1]), O - 1            # centre offset takes the shortcut
    out = {}
    for c in channels:
        w = torch.randn(O, c, c, device=d_coords.device).half()
        kw = dict(weights=w, source_masks=sm, target_masks=tm, kernel_map_sizes=sizes,
                  allow_shortcut_matmul=True)
        for fn in (F.cuda_time_gather, F.cuda_time_scatter):
            fn(tile_size=1, **kw)
        F.cuda_time_gemm(**kw)
        # kernel times from the library's own event pairs around each launch (the
        # stage timers above also count the host's launch latency)
        lib = engine.lib()
        lib.mn_profile_enable(1)
        for _ in range(rounds):
            F.cuda_time_gather(tile_size=1, **kw)
            F.cuda_time_gemm(**kw)
            F.cuda_time_scatter(tile_size=1, **kw)
        torch.cuda.synchronize()
        lib.mn_profile_enable(0)
        buf = ctypes.create_string_buffer(1 << 14)
        lib.mn_profile_report(buf, len(buf))
        per = {}
        for row in buf.value.decode().splitlines():
            name, count, kms = row.rsplit(" ", 2)
            per[name] = float(kms) / int(count)
        tg = per.get("gather_kernel", float("nan"))
        ts = per.get("scatter_kernel", float("nan"))
        tm_ = per.get("gemm_tc_kernel", per.get("gemm_simt_kernel", float("nan")))
        gather_bytes = S * c * 2 + 4 * O1 * S + E1 * c * 2
        scatter_bytes = E1 * c * 2 + 4 * O1 * T + 2 * T * c * 2
        flops = 2.0 * E * c * c
        gemm_bytes = E * 2 * c * 2 + O * c * c * 2
        out[str(c)] = {
            "gather_ms": round(tg, 4), "gather_gbs": round(gather_bytes / tg / 1e6, 1),
            "gather_frac_hbm": round(gather_bytes / tg / 1e6 / peaks["hbm_gbs"], 3),
            "gemm_ms": round(tm_, 4), "gemm_tflops": round(flops / tm_ / 1e9, 2),
            "gemm_frac_tensor": round(flops / tm_ / 1e9 / peaks["bf16_tflops"], 4),
            "gemm_gbs": round(gemm_bytes / tm_ / 1e6, 1),
            "scatter_ms": round(ts, 4), "scatter_gbs": round(scatter_bytes / ts / 1e6, 1),
            "scatter_frac_hbm": round(scatter_bytes / ts / 1e6 / peaks["hbm_gbs"], 3),
        }
    return {"map": "3^3 stride 1 on the benchmark batch", "S": int(S), "pairs": E,
            "pairs_without_centre": E1, "dtype": "f16", "channels": out}


UNET_CLOUDS = 64          # C4: 64 outdoor clouds in total, sharded over the ranks
UNET_SEED0 = 3000


def _make_cloud(seed):
    from minuet_b200 import synth
    return synth.outdoor_cloud(seed, VOXELS_PER_CLOUD)


def _make_indoor_cloud(seed):
    from minuet_b200 import synth
    return synth.indoor_cloud(seed, 200_000)


def unet_section(args, torch, dist, dev, rank, world, lib):
    """Sparse UNet (fp16, random weights, eval-mode BatchNorm) on 64 outdoor clouds
    sharded by cloud over the ranks; the logits are gathered with NCCL.  Strong
    scaling: the 64 clouds are the whole job at every N."""
    import concurrent.futures
    import minuet_b200 as minuet
    from minuet_b200 import sharding
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

    torch.manual_seed(0)
    net = SparseUNet(feats.shape[1], num_classes=20).to(dev).half().eval().fuse()
    cache = minuet.nn.KernelMapCache(ndim=3, dtype=torch.int32, device=dev)
    minuet.set_kernel_map_cache(net, cache)

    def local_forward(c, b, f):
        cache.reset()
        with torch.no_grad():
            return net(minuet.SparseTensor(f, c, batch_dims=b))

    def forward(c, b, f):
        out = local_forward(c, b, f)
        if dist is not None:
            return sharding.gather_rows(out.F, dst=0)   # collective: every rank calls it
        return [out.F]

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

    steps, warm = args.unet_steps, 3
    for _ in range(warm):
        forward(d_coords, d_bd, d_feats)
    launches0 = lib.mn_launch_count()
    ms = timed(lambda: forward(d_coords, d_bd, d_feats), steps)
    launches = lib.mn_launch_count() - launches0

    def e2e():
        c = h_coords.to(dev, non_blocking=True)
        b = h_bd.to(dev, non_blocking=True)
        f = h_feats.to(dev, non_blocking=True)
        parts = forward(c, b, f)
        if parts is not None:      # rank 0: per-voxel class labels go back to the host
            return [p.argmax(dim=1).to(torch.uint8).cpu() for p in parts]
        return None

    e2e()
    ms_e2e = timed(e2e, steps)
    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = (float(v) for v in t.cpu())

    kernels = None
    if rank == 0:
        lib.mn_profile_enable(1)
        local_forward(d_coords, d_bd, d_feats)      # rank-local: no collective in here
        torch.cuda.synchronize()
        lib.mn_profile_enable(0)
        buf = ctypes.create_string_buffer(1 << 16)
        lib.mn_profile_report(buf, len(buf))
        kernels = {}
        for row in buf.value.decode().splitlines():
            name, count, kms = row.rsplit(" ", 2)
            kernels[name] = {"launches": int(count), "ms": round(float(kms), 4)}
        kernels = dict(sorted(kernels.items(), key=lambda kv: -kv[1]["ms"]))
    if dist is not None:
        dist.barrier()
    if rank != 0:
        return None
    return {
        "metric": "sparse-UNet fp16 clouds/sec", "value": round(n_clouds * steps / (ms * 1e-3), 2),
        "unit": "clouds/s", "scaling": "strong", "ms_per_step": round(ms / steps, 3),
        "steps": steps, "warmup": warm,
        "config": {"workload": ("C3: UNet on 8 indoor scenes x 200k voxels, RGB fp16 features"
                                if indoor else
                                "C4: UNet (stem 32, encoder 32/64/128/256, decoder mirror, 20 "
                                "classes) on 64 outdoor clouds x 120k voxels, 4-channel fp16 "
                                "features") + ", clouds sharded over the GPUs, NCCL gather of "
                               "the logits",
                   "clouds_total": n_clouds, "clouds_on_rank0": len(mine),
                   "voxels_on_rank0": int(len(coords))},
        "e2e": {"value": round(n_clouds * steps / (ms_e2e * 1e-3), 2), "unit": "clouds/s",
                "ms_per_step": round(ms_e2e / steps, 3),
                "h2d_bytes_per_step": int(h_coords.numel() * 4 + h_bd.numel() * 8 + h_feats.numel() * 2),
                "d2h_bytes_per_step": int(n_clouds * per_cloud)},
        "gpu_launches": int(launches),
        "library_kernel_ms_rank0_one_step": kernels,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "reference-cuda"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-unet", action="store_true",
                    help="skip the secondary end-to-end UNet measurement")
    ap.add_argument("--unet-steps", type=int, default=5)
    ap.add_argument("--unet-clouds", type=int, default=UNET_CLOUDS,
                    help="clouds in the UNet job (64 = the benchmark configuration)")
    ap.add_argument("--gms-channels", default="16,32,64,128,256")
    ap.add_argument("--unet-config", default="c4", choices=["c3", "c4"],
                    help="c4: 64 outdoor clouds (default); c3: 8 indoor scenes with RGB features")
    ap.add_argument("--gms-sweep", action="store_true",
                    help="also time gather / grouped GEMM / scatter for C in 16..256 (fp16)")
    args = ap.parse_args()
    if args.impl == "reference-cuda":
        reference_cuda_arm(args)
    elif args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
