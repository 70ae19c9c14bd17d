#!/usr/bin/env python
"""Benchmark of the data-movement hot path: device-to-device copy GB/s (read + write bytes counted).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one DtoD copy of a 1 GiB buffer (inputs larger than L2, so no flush is needed between steps).
`value` times the copy kernel through the C-ABI (lcb_copy_d2d) with the source already in HBM; `e2e` times
the same copy through the public libreCu* API from pinned HOST buffers (HtoD -> DtoD -> DtoH inside the
timed region).  With N > 1 (one process per GPU under torchrun) every rank copies its own 1 GiB shard --
weak scaling, no data-path collective -- and the NVLink paths (peer push, all-to-all, broadcast) are
measured as well and reported under "nvlink".  Rank 0 prints one JSON line.

`--impl reference` times the reference's CPU statement of the path -- multithreaded memcpy on the host
cores (oracle/lcb_oracle.c) -- on the same workload and metric.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

GiB = 1 << 30
MiB = 1 << 20
WORKLOAD_BYTES = GiB
METRIC = "dtod_copy_GBps"
UNIT = "GB/s"
NVLINK_NOMINAL = 900.0   # GB/s per direction per GPU
SRC_STABLE = 0x100       # LCB_COPY_SRC_STABLE: nothing in flight on the stream writes the copy's source
# dram__bytes_read.sum + dram__bytes_write.sum of the very launch the bench times (1 GiB, AUTO | SRC_STABLE ->
# copy_tma_kernel<3,2,0>, 12 KiB per CTA) from an ncu capture of `bench.py --case copy_auto_stable --bytes
# 1073741824`: reads 1.0738 GB (the source), writes 1.0244 GB (the destination less ~50 MB still dirty in L2 at
# kernel exit)
NCU_TRAFFIC_1GIB = 2_098_200_000


def measured_hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


# ---------------------------------------------------------------------------------------------------
# checks against the host oracle (outside every timed region)
# ---------------------------------------------------------------------------------------------------
WINDOW = 16 * MiB


def host_windows_ok(api, stream, dev_ptr: int, nbytes: int, expect, salt: int) -> bool:
    """Device-to-host copies of the first, the last and three seeded-random 16 MiB windows of a device range,
    each compared byte for byte with `expect(offset, n)`, the bytes the HOST oracle says belong there.  The
    device-side comparator judges the whole range; this is the independent check of it (and of the device-side
    generator) by the reference's own criterion, equality after DtoH
    (tests/dma_chronological_consistency/main.cpp:73-85)."""
    import numpy as np

    win = min(WINDOW, nbytes)
    offs = {0, nbytes - win}
    rng = np.random.default_rng(salt)
    while len(offs) < 5 and nbytes - win >= 8 * 5:
        offs.add(int(rng.integers(0, (nbytes - win) // 8 + 1)) * 8)
    host = np.empty(win, np.uint8)
    for off in sorted(offs):
        stream.memcpy(host, dev_ptr + off, win)
        stream.run()
        if not np.array_equal(host, expect(off, win)):
            return False
    return True


def stream_expect(seed: int, base_offset: int = 0):
    """expect() of a range that holds the seeded stream `seed` from byte `base_offset` (a multiple of 8) on."""
    import oracle  # the checker

    return lambda off, n: oracle.random_window(base_offset + off, n, seed)


def device_equal(api, stream, a_ptr: int, b_ptr: int, nbytes: int, res) -> bool:
    import numpy as np

    api.lcb_check(api.lib.lcb_compare_bytes(a_ptr, b_ptr, nbytes, res.ptr, stream.native), "compare")
    r = np.zeros(2, np.uint64)
    stream.memcpy(r, res, 16)
    stream.run()
    return int(r[0]) == 0


def describe_copy(api, dst_ptr: int, src_ptr: int, nbytes: int, path: int) -> str:
    buf = C.create_string_buffer(200)
    if api.lib.lcb_copy_d2d_describe(dst_ptr, src_ptr, nbytes, path, 0, buf, 200) != 0:
        return "?"
    return buf.value.decode()


# ---------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return
        fd, self.path = tempfile.mkstemp(suffix=".csv")
        os.close(fd)
        self.proc = subprocess.Popen(
            [exe, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.gpu)],
            stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        time.sleep(0.3)

    def stop(self):
        if self.proc is None:
            return None
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in Path(self.path).read_text().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, v in zip(names, parts[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if not sm:
            return None
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------
# reference arm: the CPU statement of the path on the host cores
# ---------------------------------------------------------------------------------------------------
def cpu_memcpy_gbps(nbytes: int, threads: int, reps: int):
    import numpy as np

    import oracle  # CPU baseline leg: the one place the benchmark executes the oracle

    src = oracle.random_bytes(nbytes, seed=1)
    dst = np.zeros(nbytes, np.uint8)
    best = oracle.mt_seconds(dst, src, op=0, value=0, threads=threads, reps=reps)
    return 2.0 * nbytes / best / 1e9, best


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import numpy as np

    import oracle

    threads = host_threads()
    n = WORKLOAD_BYTES
    src = oracle.random_bytes(n, seed=1)
    dst = np.zeros(n, np.uint8)
    for _ in range(max(args.warmup, 1)):
        oracle.mt_seconds(dst, src, 0, 0, threads, 1)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.mt_seconds(dst, src, 0, 0, threads, 1)
    dt = time.perf_counter() - t0
    ms = dt / args.steps * 1e3
    value = 2.0 * n / (dt / args.steps) / 1e9
    assert np.array_equal(dst[:4096], src[:4096])
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": "dtod_copy_1GiB_aligned", "bytes_per_gpu": n, "bytes": n, "seed": 1,
                   "algorithmic_bytes_per_step_per_gpu": 2 * n,
                   "note": "reference's CPU statement of the path: multithreaded memcpy of the same seeded bytes"},
        "cpu_baseline": {"value": round(value, 2), "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{args.steps} x memcpy of 1 GiB split over {threads} threads"},
        "e2e": {"value": round(value, 2), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------
def timed_loop(api, stream, fn, steps):
    """fn() enqueues one step on stream.native; returns average ms per step (CUDA events on that stream)."""
    t = api.Timer()
    t.start(stream.native)
    for _ in range(steps):
        fn()
    t.stop(stream.native)
    ms = t.elapsed_ms() / steps
    t.destroy()
    return ms


def run_ours(args):
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    multi = world > 1
    dist = None
    torch = None
    # Libraries underneath (NCCL prints its version line) write to file descriptor 1; the contract is ONE line on
    # stdout, so everything but the final JSON line is sent to stderr.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    if multi:
        import torch
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from librecuda_b200 import api

    lib = api.lib
    ctx = api.Context(local_rank, api.CU_CTX_SCHED_YIELD)
    stream = api.Stream()
    native = stream.native
    n = WORKLOAD_BYTES
    steps, warmup = args.steps, max(args.warmup, 3)

    def barrier():
        if multi:
            dist.barrier()
            torch.cuda.synchronize()
        api.lcb_check(lib.lcb_stream_synchronize(native), "sync")

    def max_over_ranks(ms: float) -> float:
        if not multi:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    import numpy as np

    src, dst = api.DeviceBuffer(n + 256), api.DeviceBuffer(n + 256)
    res = api.DeviceBuffer(16)
    api.lcb_check(lib.lcb_fill_splitmix64(src.ptr, n + 256, 1 + rank, native), "fill")
    stream.memset_d8(dst, 0, n + 256)
    stream.run()

    # The source is never written inside the loop, so the copy may load ahead of the stream wait
    # (LCB_COPY_SRC_STABLE); libreCuMemCpy sets the same flag by itself from its command list.
    copy_path = SRC_STABLE

    def copy_step():
        api.lcb_check(lib.lcb_copy_d2d_ex(dst.ptr, src.ptr, n, copy_path, 0, native), "lcb_copy_d2d_ex")

    for _ in range(warmup):
        copy_step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    ms_local = timed_loop(api, stream, copy_step, steps)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = max_over_ranks(ms_local)
    value = world * 2.0 * n / (ms * 1e-3) / 1e9
    launches = steps

    # bit-exactness of what was just timed, outside the timed region: the whole range on the device, and
    # windows of it on the host against the oracle's regeneration of the seeded stream
    verified = device_equal(api, stream, dst.ptr, src.ptr, n, res) and api.device_error_word() == 0
    verified = verified and host_windows_ok(api, stream, dst.ptr, n, stream_expect(1 + rank), salt=11)

    peak, peak_kind = measured_hbm_peak()
    achieved = 2.0 * n / (ms_local * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "lcb_copy_d2d_ex(AUTO | SRC_STABLE) -> " + describe_copy(api, dst.ptr, src.ptr, n, copy_path),
                "achieved": round(achieved, 1),
                "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": round(achieved / peak, 4),
                "frac_of_nominal_8000": round(achieved / 8000.0, 4), "traffic": NCU_TRAFFIC_1GIB,
                "traffic_note": "dram read+write bytes of this 1 GiB launch under ncu (reads = source size, writes = "
                                "destination size minus ~50 MB left dirty in L2 at kernel exit)"}

    def frac_entry(nbytes_moved, t_ms, extra=None):
        gbps = nbytes_moved / (t_ms * 1e-3) / 1e9
        e = {"GBps": round(gbps, 1), "ms": round(t_ms, 4), "frac_of_measured_hbm": round(gbps / peak, 4),
             "frac_of_nominal_8000": round(gbps / 8000.0, 4)}
        if extra:
            e.update(extra)
        return e

    def measure(fn, reps=None):
        for _ in range(3):
            fn()
        barrier()
        return timed_loop(api, stream, fn, reps or steps)

    # ---- the metric's other single-GPU members (cfg2, cfg3): sizes from the 256 MiB boundary up, misaligned
    #      offsets, memset / index fill / y = 2x + 1.  Copies count read + write bytes, fills written bytes.
    also = {}
    words = n // 4
    copy_cases = (("dtod_copy_128MiB_aligned", 128 * MiB, 0, 0), ("dtod_copy_256MiB_aligned", 256 * MiB, 0, 0),
                  ("dtod_copy_512MiB_aligned", 512 * MiB, 0, 0), ("dtod_copy_1GiB_src+1_dst+0", n, 1, 0),
                  ("dtod_copy_1GiB_src+64_dst+1", n, 64, 1))
    for name, nb, so, do in copy_cases:
        stream.memset_d8(dst, 0, nb + 256)
        stream.run()
        t_ms = measure(lambda: api.lcb_check(lib.lcb_copy_d2d_ex(dst.ptr + do, src.ptr + so, nb, copy_path, 0, native), name))
        ok = device_equal(api, stream, dst.ptr + do, src.ptr + so, nb, res)
        # host windows: the destination holds the source stream from byte `so` on; the oracle generates 8-byte
        # aligned windows, so compare against a slice of a slightly larger one
        import oracle

        def expect(off, m, so=so):
            lo = (so + off) // 8 * 8
            w = oracle.random_window(lo, m + 16, 1 + rank)
            return w[(so + off) - lo:(so + off) - lo + m]

        ok = ok and host_windows_ok(api, stream, dst.ptr + do, nb, expect, salt=nb % 1009 + so)
        also[name] = frac_entry(2 * nb, t_ms, {"verified": ok, "kernel": describe_copy(api, dst.ptr + do, src.ptr + so, nb, copy_path)})
    # the same 1 GiB copy without the flag (loads wait for the previous kernel like the stores)
    also["dtod_copy_1GiB_aligned_loads_wait_too"] = frac_entry(
        2 * n, measure(lambda: api.lcb_check(lib.lcb_copy_d2d(dst.ptr, src.ptr, n, native), "copy")),
        {"kernel": describe_copy(api, dst.ptr, src.ptr, n, 0)})

    fills = (("memset_d32_1GiB", n, lambda: api.lcb_check(lib.lcb_memset_d32(dst.ptr, 0x40490FDB, words, native), "memset")),
             ("memset_d8_1GiB", n, lambda: api.lcb_check(lib.lcb_memset_d8(dst.ptr, 0xA5, n, native), "memset")),
             ("memset_d8_256MiB", 256 * MiB, lambda: api.lcb_check(lib.lcb_memset_d8(dst.ptr, 0x5A, 256 * MiB, native), "memset")),
             ("index_fill_f32_1GiB", n, lambda: api.lcb_check(lib.lcb_index_fill_f32(dst.ptr, words, native), "index_fill")))
    for name, nb, fn in fills:
        also[name] = frac_entry(nb, measure(fn))
    # memset and index fill against host loops (windows); the last fill run is the index fill over all of dst
    def index_expect(off, m):
        first = off // 4
        return np.arange(first, first + m // 4, dtype=np.uint64).astype(np.float32).view(np.uint8)

    also["index_fill_f32_1GiB"]["verified"] = host_windows_ok(api, stream, dst.ptr, n, index_expect, salt=5)
    api.lcb_check(lib.lcb_memset_d32(dst.ptr, 0x40490FDB, words, native), "memset")
    also["memset_d32_1GiB"]["verified"] = host_windows_ok(
        api, stream, dst.ptr, n, lambda off, m: np.full(m // 4, 0x40490FDB, np.uint32).view(np.uint8), salt=6)

    # y = 2x + 1 over 1 GiB of floats read and 1 GiB written (cfg4's kernel stage): 8 bytes per element
    t_ms = measure(lambda: api.lcb_check(lib.lcb_axpb_f32(dst.ptr, src.ptr, 2.0, 1.0, words, native), "axpb"))
    also["axpb_f32_y=2x+1_1GiB"] = frac_entry(2 * n, t_ms)

    for name, fn, nbytes in (("vendor_cudaMemcpyAsync_d2d_1GiB", lambda: api.lcb_check(lib.lcb_vendor_memcpy_d2d(dst.ptr, src.ptr, n, native), "vendor copy"), 2 * n),
                             ("vendor_cudaMemsetAsync_1GiB", lambda: api.lcb_check(lib.lcb_vendor_memset_d8(dst.ptr, 0xA5, n, native), "vendor memset"), n)):
        also[name] = frac_entry(nbytes, measure(fn), {"note": "CUDA runtime's own path, for comparison"})

    ref_gpu = reference_kernel_on_gpu(api, stream, src, dst, steps)
    if ref_gpu is not None:
        also["reference_HighBW_kernel_sm100a_128MiB"] = ref_gpu

    small_ops = run_small_ops(api, stream, src, dst)
    for b in (src, dst):
        b.free()

    # 8 GiB aligned (the largest member of the DtoD sweep): its own buffers, freed again before the rest
    big = 8 * GiB
    bsrc, bdst = api.DeviceBuffer(big), api.DeviceBuffer(big)
    api.lcb_check(lib.lcb_fill_splitmix64(bsrc.ptr, big, 1 + rank, native), "fill")
    stream.memset_d8(bdst, 0, big)
    stream.run()
    t_ms = measure(lambda: api.lcb_check(lib.lcb_copy_d2d_ex(bdst.ptr, bsrc.ptr, big, copy_path, 0, native), "copy 8 GiB"), reps=max(3, steps // 4))
    ok = device_equal(api, stream, bdst.ptr, bsrc.ptr, big, res) and host_windows_ok(api, stream, bdst.ptr, big, stream_expect(1 + rank), salt=8)
    also["dtod_copy_8GiB_aligned"] = frac_entry(2 * big, t_ms, {"verified": ok, "kernel": describe_copy(api, bdst.ptr, bsrc.ptr, big, copy_path)})
    bsrc.free()
    bdst.free()
    shortfalls = [k for k, v in also.items() if (k.startswith("dtod_copy") or k.startswith("memset") or k.startswith("index"))
                  and "128MiB" not in k and v["frac_of_nominal_8000"] < 0.85]
    also["below_0.85_of_8000_from_256MiB_up"] = shortfalls

    # end to end through the public API with HOST buffers: HtoD -> DtoD -> DtoH inside the timed region
    e2e = run_e2e(api, ctx, n, max(2, min(steps, 10)), max_over_ranks, barrier, world)

    nvlink = run_nvlink(api, stream, rank, world, dist, torch, steps, barrier, max_over_ranks) if multi else None

    cpu = None
    if rank == 0 and not multi:
        threads = host_threads()
        v, best = cpu_memcpy_gbps(n, threads, reps=8)
        cpu = {"value": round(v, 2), "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"best of 8 x memcpy of the same 1 GiB seeded buffer split over {threads} threads"}

    res.free()
    stream.destroy()
    if multi:
        dist.barrier()
        dist.destroy_process_group()
    if multi and rank == 0:
        # the single-process entry points (one context per GPU in THIS process) over all N GPUs; the other ranks
        # have released their buffers and are exiting
        try:
            nvlink["one_process"] = run_one_process(api, ctx, world, max(3, min(steps, 10)))
        except Exception as exc:  # reported, never hidden: the line below says what failed
            nvlink["one_process"] = {"error": f"{type(exc).__name__}: {exc}"}

    if rank == 0:
        all_ok = verified and all(v.get("verified", True) for v in also.values() if isinstance(v, dict))
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u8", "data": "synthetic",
            "config": {"workload": "dtod_copy_1GiB_aligned", "bytes_per_gpu": n, "bytes": n, "seed": 1,
                       "algorithmic_bytes_per_step_per_gpu": 2 * n,
                       "l2": "inputs larger than L2 (1 GiB source + 1 GiB destination per step), no flush",
                       "launch": "lcb_copy_d2d_ex with LCB_COPY_SRC_STABLE (the source is not written in the loop)",
                       "parallelism": f"{world} independent shards, no data-path collective"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
            "verified_bit_exact": all_ok, "also": also, "small_ops": small_ops,
        }
        if nvlink is not None:
            line["nvlink"] = nvlink
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        print(json.dumps(line), flush=True)
    return 0 if verified else 1


def run_small_ops(api, stream, src, dst):
    """Cost of tiny operations, the reference's own measurements: back-to-back small copies on one stream (CUDA
    events around 2 000 launches enqueued from Python: the larger of the device's and the host's cost per launch), and
    1 025 launches of an empty kernel from 1 025 modules loaded from one image
    (tests/many_kernels_launch/main.cpp:49-90: host time from the first libreCuLaunchKernel to the return of
    libreCuStreamCommence, divided by the launches; the device time between two events is reported beside it)."""
    lib = api.lib
    native = stream.native
    out = {}
    reps = 2000
    for label, nb in (("copy_4KiB", 4096), ("copy_1MiB", MiB)):
        fn = lambda: api.lcb_check(lib.lcb_copy_d2d(dst.ptr, src.ptr, nb, native), "small copy")
        for _ in range(50):
            fn()
        out[f"lcb_{label}_us_per_op_back_to_back"] = round(timed_loop(api, stream, fn, reps) * 1e3, 3)
    # the same 4 KiB copies through the public API: record, commence, await (host clock: includes recording)
    stream.run()
    t0 = time.perf_counter()
    for _ in range(reps):
        stream.memcpy(dst, src, 4096)
    stream.commence()
    t1 = time.perf_counter()
    stream.await_()
    t2 = time.perf_counter()
    out["libreCuMemCpy_4KiB_us_per_op_host_record_and_commence"] = round((t1 - t0) / reps * 1e6, 3)
    out["libreCuMemCpy_4KiB_us_per_op_until_await_returns"] = round((t2 - t0) / reps * 1e6, 3)
    cubin = ROOT / "tests" / "fixtures" / "_bin" / "fixture_kernels.cubin"
    if cubin.exists():
        image = cubin.read_bytes()
        count = 1025
        mods = [api.Module(image) for _ in range(count)]
        fns = [m.function("empty_kernel") for m in mods]
        start, end = api.Event(), api.Event()
        for f in fns[:8]:
            stream.launch(f, (1, 1, 1), (1, 1, 1), 0, [])
        stream.run()
        start.record(stream)
        t0 = time.perf_counter()
        for f in fns:
            stream.launch(f, (1, 1, 1), (1, 1, 1), 0, [])
        end.record(stream)
        stream.commence()
        t1 = time.perf_counter()
        stream.await_()
        out["empty_kernel_1025_launches_1025_modules"] = {
            "us_per_launch_host_record_and_commence": round((t1 - t0) / count * 1e6, 3),
            "us_per_launch_device": round(api.elapsed_ms(start, end) / count * 1e3, 3)}
        for e in (start, end):
            e.destroy()
        for m in mods:
            m.unload()
    return out


def reference_kernel_on_gpu(api, stream, src, dst, steps):
    """The reference's own HighBW copy kernel (driverapi/kernels/memcpy/memcpy.cu, compiled for sm_100a from the
    reference checkout into oracle/_ref/ at build time) at the largest size its dispatcher launches correctly,
    128 MiB with grid (size/4096, 1) x 256 threads (driverapi/src/memcopy.cpp:93-107), beside this library's
    copy of the same 128 MiB.  Returns None when the image is not there."""
    cubin = ROOT / "oracle" / "_ref" / "ref_memcpy_sm100a.cubin"
    if not cubin.exists():
        return None
    n = 128 * MiB
    mod = api.Module(cubin.read_bytes())
    fn = mod.function("memcpyKernelHighBW")
    start, end = api.Event(), api.Event()

    def timed(record_one):
        for _ in range(3):
            record_one()
        stream.run()
        start.record(stream)
        for _ in range(steps):
            record_one()
        end.record(stream)
        stream.run()
        return api.elapsed_ms(start, end) / steps

    ms_ref = timed(lambda: stream.launch(fn, (n // 4096, 1, 1), (256, 1, 1), 0, [C.c_void_p(dst.ptr), C.c_void_p(src.ptr)]))
    ms_own = timed(lambda: stream.memcpy(dst, src, n))
    for e in (start, end):
        e.destroy()
    mod.unload()
    gb = lambda ms: round(2.0 * n / (ms * 1e-3) / 1e9, 1)
    return {"reference_kernel_GBps": gb(ms_ref), "this_library_GBps": gb(ms_own), "bytes": n,
            "note": "both through libreCuLaunchKernel / libreCuMemCpy on one stream, timed with libreCuEvent*"}


def run_e2e(api, ctx, n, steps, max_over_ranks, barrier, world, piece=64 * MiB, layout="roundrobin", measure_pcie=True):
    """End to end through the public API on pinned HOST buffers, timed with the API's own events.

    serial:    the call sequence of the reference's tests/memcopy/main.cpp:47-57 on one stream
               (HtoD 1 GiB -> DtoD -> DtoH 1 GiB).
    pipelined: the same bytes cut into pieces.  layout "lanes": one stream carries every HtoD in order, a second
               the DtoD kernels, a third every DtoH; piece k of one lane waits for piece k of the lane before it
               through libreCuStreamWaitEvent, so each PCIe direction has one queue that never waits behind the
               other direction.  layout "roundrobin": pieces dealt to four streams, each running HtoD -> DtoD ->
               DtoH of its piece.  The pipelined figure is the reported e2e value.
    pcie:      one-way HtoD and DtoH of the same pinned buffers, timed alone in this run; the full-duplex bound
               of a step is the slower direction's time."""
    import numpy as np

    S = 4
    streams = [api.Stream() for _ in range(S)]
    hin, hout = api.PinnedBuffer(n), api.PinnedBuffer(n)
    hin.array[:] = np.resize(np.arange(251, dtype=np.uint8), n)
    a, b = api.DeviceBuffer(n), api.DeviceBuffer(n)
    start, end = api.Event(), api.Event()
    joins = [api.Event() for _ in range(S)]
    pieces = [(off, min(piece, n - off)) for off in range(0, n, piece)]
    ev_h = [api.Event() for _ in pieces]
    ev_k = [api.Event() for _ in pieces]
    ev_d = [api.Event() for _ in pieces]

    def serial_step():
        st = streams[0]
        st.memcpy(a, hin.array, n)
        st.memcpy(b, a, n)
        st.memcpy(hout.array, b, n)

    def h2d_step():
        streams[0].memcpy(a, hin.array, n)

    def d2h_step():
        streams[0].memcpy(hout.array, b, n)

    def duplex_step():  # both directions at once on independent buffers: what the link gives with nothing else in the way
        streams[0].memcpy(a, hin.array, n)
        streams[1].memcpy(hout.array, b, n)

    def roundrobin_step():
        for i, (off, m) in enumerate(pieces):
            st = streams[i % S]
            st.memcpy(a.view(off, m), hin.array[off:off + m], m)
            st.memcpy(b.view(off, m), a.view(off, m), m)
            st.memcpy(hout.array[off:off + m], b.view(off, m), m)

    primed = [False]

    def lanes_step():
        # piece i of a step may only overwrite a[i] / b[i] once the previous step's reader of that piece is done
        up, mid, down = streams[0], streams[1], streams[2]
        for i, (off, m) in enumerate(pieces):
            if primed[0]:
                up.wait_event(ev_k[i])
            up.memcpy(a.view(off, m), hin.array[off:off + m], m)
            ev_h[i].record(up)
        up.commence()  # an event has to be submitted before a stream that waits for it is
        for i, (off, m) in enumerate(pieces):
            mid.wait_event(ev_h[i])
            if primed[0]:
                mid.wait_event(ev_d[i])
            mid.memcpy(b.view(off, m), a.view(off, m), m)
            ev_k[i].record(mid)
        mid.commence()
        for i, (off, m) in enumerate(pieces):
            down.wait_event(ev_k[i])
            down.memcpy(hout.array[off:off + m], b.view(off, m), m)
            ev_d[i].record(down)
        down.commence()
        primed[0] = True

    def timed(step_fn, multi_stream, reps):
        for _ in range(2):
            step_fn()
        for st in streams:
            st.run()
        barrier()
        start.record(streams[0])
        streams[0].commence()
        if multi_stream:  # the other streams start after the start event
            for st in streams[1:]:
                st.wait_event(start)
        for _ in range(reps):
            step_fn()
        if multi_stream:
            for i in range(1, S):
                joins[i].record(streams[i])
                streams[i].commence()
                streams[0].wait_event(joins[i])
        end.record(streams[0])
        streams[0].commence()
        for st in streams:
            st.await_()
        return max_over_ranks(api.elapsed_ms(start, end) / reps)

    def check():
        return bool(np.array_equal(hout.array[::4099], hin.array[::4099]) and np.array_equal(hout.array[-4096:], hin.array[-4096:]))

    hout.array[:] = 0
    ms_serial = timed(serial_step, False, max(2, steps // 2))
    ok = check()
    hout.array[:] = 0
    ms_pipe = timed(lanes_step if layout == "lanes" else roundrobin_step, True, steps)
    ok = ok and check()
    pcie = None
    if measure_pcie:
        ms_h = timed(h2d_step, False, max(2, steps // 2))
        ms_d = timed(d2h_step, False, max(2, steps // 2))
        ms_dup = timed(duplex_step, True, max(2, steps // 2))
        bound_ms = max(ms_h, ms_d)
        pcie = {"h2d_GBps": round(n / (ms_h * 1e-3) / 1e9, 2), "d2h_GBps": round(n / (ms_d * 1e-3) / 1e9, 2),
                "full_duplex_bound_ms": round(bound_ms, 3), "frac": round(bound_ms / ms_pipe, 4),
                "duplex_measured_ms": round(ms_dup, 3), "duplex_measured_GBps": round(2.0 * n / (ms_dup * 1e-3) / 1e9, 2),
                "frac_of_duplex_measured": round(ms_dup / ms_pipe, 4),
                "note": "one-way copies of the same pinned 1 GiB buffers timed alone in this run; bound = the slower "
                        "direction's time (both directions fully overlapped); frac = bound / pipelined step time. "
                        "duplex_measured = 1 GiB HtoD and 1 GiB DtoH of independent buffers issued together on two "
                        "streams, nothing else running: what the link delivers when both directions are busy"}
    for e in [start, end] + joins + ev_h + ev_k + ev_d:
        e.destroy()
    for x in (a, b):
        x.free()
    hin.free()
    hout.free()
    for st in streams:
        st.destroy()
    gbps = lambda ms: round(world * 2.0 * n / (ms * 1e-3) / 1e9, 2)
    path = (f"libreCuMemCpy HtoD -> DtoD -> DtoH on pinned host buffers in {piece // MiB} MiB pieces; one stream per "
            "stage (all HtoD / all DtoD / all DtoH), piece k chained across them with libreCuStreamWaitEvent"
            if layout == "lanes" else
            f"libreCuMemCpy HtoD -> DtoD -> DtoH on pinned host buffers in {piece // MiB} MiB pieces over 4 streams")
    return {"value": gbps(ms_pipe), "unit": UNIT, "h2d_bytes_per_step": n, "d2h_bytes_per_step": n,
            "ms_per_step": round(ms_pipe, 3), "steps": steps, "verified": ok,
            "path": path + ", timed with libreCuEvent* (PCIe-bound)", "pcie": pcie,
            "serial_one_stream": {"value": gbps(ms_serial), "ms_per_step": round(ms_serial, 3)}}


def alltoall_expect(G, chunk, me):
    """expect() of rank `me`'s receive buffer after an all-to-all: slot r holds chunk `me` of rank r's send buffer,
    which is the seeded stream 100 + r."""
    import numpy as np

    import oracle

    def expect(off, m):
        parts = []
        while m > 0:
            r, inner = divmod(off, chunk)
            take = min(m, chunk - inner)
            parts.append(oracle.random_window(me * chunk + inner, take, 100 + r))
            off += take
            m -= take
        return parts[0] if len(parts) == 1 else np.concatenate(parts)

    return expect


def run_nvlink(api, stream, rank, world, dist, torch, steps, barrier, max_over_ranks):
    """NVLink paths at world size G, one process per GPU: peer copies (rank r <-> r+1), all-to-all (own fused
    kernels and NCCL), partitioned copy, broadcast from rank 0 (NCCL).  GB/s per GPU per direction; fractions of
    900 (nominal) and of the copy-engine peer copy measured in this run.  Every figure is verified afterwards:
    the whole destination on the device, windows of it on the host against the oracle."""
    import numpy as np

    lib = api.lib
    native = stream.native
    G = world
    chunk = GiB  # all-to-all chunk per GPU pair; (G-1) * chunk leaves and enters every GPU
    shard = GiB
    send = api.DeviceBuffer(G * chunk)
    recv = api.DeviceBuffer(G * chunk)
    api.lcb_check(lib.lcb_fill_splitmix64(send.ptr, G * chunk, 100 + rank, native), "fill")
    stream.memset_d8(recv, 0, G * chunk)
    stream.run()
    from librecuda_b200 import multirank as mr

    peers = mr.open_peers(dist, recv)          # every rank's receive buffer (targets of remote stores)
    send_peers = mr.open_peers(dist, send)     # every rank's send buffer (sources of remote loads)
    peer_arr = (C.c_void_p * G)(*peers)
    send_arr = (C.c_void_p * G)(*send_peers)
    out = {"world": G, "nominal_GBps": NVLINK_NOMINAL}
    resb = api.DeviceBuffer(16)
    scratch = api.DeviceBuffer(chunk)          # expected bytes, regenerated on the device at the right stream position

    def report(name, bytes_per_gpu, ms):
        gbps = bytes_per_gpu / (ms * 1e-3) / 1e9
        out[name] = {"GBps_per_gpu_per_direction": round(gbps, 1), "ms": round(ms, 4),
                     "frac_of_nominal_900": round(gbps / NVLINK_NOMINAL, 4)}

    def measure(name, fn, bytes_per_gpu, reps=None):
        for _ in range(3):
            fn()
        barrier()
        ms = max_over_ranks(timed_loop(api, stream, fn, reps or steps))
        barrier()
        report(name, bytes_per_gpu, ms)

    def holds_stream(ptr, nbytes, seed, base, salt):
        """[ptr, ptr + nbytes) == bytes [base, base + nbytes) of seeded stream `seed`: device compare + host windows."""
        ok = True
        for off in range(0, nbytes, chunk):
            m = min(chunk, nbytes - off)
            api.lcb_check(lib.lcb_fill_splitmix64_at(scratch.ptr, m, seed, (base + off) // 8, native), "fill")
            ok = ok and device_equal(api, stream, ptr + off, scratch.ptr, m, resb)
        return ok and host_windows_ok(api, stream, ptr, nbytes, stream_expect(seed, base), salt)

    # 1. partitioned peer copy, every port busy: rank r moves a 1 GiB shard from / to its neighbour.
    #    pull = the destination GPU loads from the source GPU (faster direction), push = the source GPU stores.
    prev = (rank - 1) % G
    prev_send = send_peers[prev]
    nxt_recv = peers[(rank + 1) % G]
    shifts = (
        ("p2p_shift_copy_engine_1GiB", lambda: api.lcb_check(lib.lcb_vendor_memcpy_d2d(nxt_recv, send.ptr, shard, native), "peer engine")),
        ("p2p_shift_pull_1GiB", lambda: api.lcb_check(lib.lcb_copy_d2d(recv.ptr, prev_send, shard, native), "peer pull")),
        ("p2p_shift_push_1GiB", lambda: api.lcb_check(lib.lcb_copy_d2d(nxt_recv, send.ptr, shard, native), "peer push")),
    )
    for name, fn in shifts:
        barrier()
        stream.memset_d8(recv, 0, shard)
        stream.run()
        barrier()
        measure(name, fn, shard)
        out[name]["verified"] = holds_stream(recv.ptr, shard, 100 + prev, 0, salt=21)
    # the denominator "measured peer copy": the copy engines' ring shift of this very run
    out["measured_peer_copy_GBps"] = out["p2p_shift_copy_engine_1GiB"]["GBps_per_gpu_per_direction"]

    # 2. all-to-all: one fused kernel per rank (push = remote stores, pull = remote loads).
    #    Each form starts from a zeroed receive buffer and is verified afterwards.
    def clear_recv():
        barrier()
        stream.memset_d8(recv, 0, G * chunk)
        stream.run()
        barrier()

    def verify_recv(ptr):
        # slot r of my receive buffer must be chunk `rank` of rank r's send buffer
        barrier()
        ok = True
        for r in range(G):
            api.lcb_check(lib.lcb_fill_splitmix64_at(scratch.ptr, chunk, 100 + r, rank * chunk // 8, native), "fill")
            ok = ok and device_equal(api, stream, ptr + r * chunk, scratch.ptr, chunk, resb)
        return ok and host_windows_ok(api, stream, ptr, G * chunk, alltoall_expect(G, chunk, rank), salt=31 + rank)

    # the copy-engine form: G-1 peer copies per rank kept in lock-step through flags in each other's memory (every
    # GPU has one sender at a time), the local chunk as a kernel on a second stream beside them
    flags = api.DeviceBuffer(4096)
    stream.memset_d8(flags, 0, 4096)
    stream.run()
    flag_peers = mr.open_peers(dist, flags)
    flag_arr = (C.c_void_p * G)(*flag_peers)
    side = api.Stream()
    epoch = [0]

    def a2a_engines():
        epoch[0] += 1
        api.lcb_check(lib.lcb_stream_wait_stream(side.native, native), "fork")
        api.lcb_check(lib.lcb_alltoall_engines(peer_arr, send.ptr, chunk, G, rank, flags.ptr, flag_arr, epoch[0], 250,
                                               native, side.native), "a2a engines")
        api.lcb_check(lib.lcb_stream_wait_stream(native, side.native), "join")

    forms = (
        ("alltoall_own_push", lambda: api.lcb_check(lib.lcb_alltoall_push(peer_arr, send.ptr, chunk, G, rank, native), "a2a push")),
        ("alltoall_copy_engines_lockstep", a2a_engines),
        ("alltoall_own_pull", lambda: api.lcb_check(lib.lcb_alltoall_pull(send_arr, recv.ptr, chunk, G, rank, native), "a2a pull")),
    )
    for name, fn in forms:
        clear_recv()
        measure(name, fn, (G - 1) * chunk)
        out[name]["verified"] = verify_recv(recv.ptr) and api.device_error_word() == 0
    side.destroy()
    barrier()
    mr.close_peers(dist, flag_peers)
    barrier()
    flags.free()

    # 3. partitioned copy of an 8 GiB buffer that lives on rank 0: shard g (2 MiB-aligned boundaries from
    #    libreCuPartitionPlan) is pulled by rank g into its own memory; rank 0 keeps shard 0 with a local copy.
    total = 8 * GiB
    big = api.DeviceBuffer(total if rank == 0 else 4096)
    if rank == 0:
        api.lcb_check(lib.lcb_fill_splitmix64(big.ptr, total, 3, native), "fill")
        stream.run()
    big_peers = mr.open_peers(dist, big)
    off, ln = mr.shard_of(total, G, rank)
    mine = api.DeviceBuffer(max(ln, 16))
    measure("partitioned_8GiB_from_rank0", lambda: api.lcb_check(lib.lcb_copy_d2d(mine.ptr, big_peers[0] + off, ln, native), "shard pull"),
            total * (G - 1) // G)
    out["partitioned_8GiB_from_rank0"]["note"] = "GB/s leaving rank 0 (its NVLink egress): (G-1)/G of 8 GiB / max-over-ranks time"
    out["partitioned_8GiB_from_rank0"]["verified"] = holds_stream(mine.ptr, ln, 3, off, salt=41) if ln else True
    mine.free()
    barrier()
    mr.close_peers(dist, big_peers)
    barrier()
    big.free()

    # 4. all-to-all and broadcast through NCCL (torch.distributed): the named library path.  Buffers are filled
    #    and checked with this library's device-side generator / comparator and the host oracle.
    ts = torch.empty(G * chunk, dtype=torch.uint8, device="cuda")
    tr = torch.zeros(G * chunk, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    api.lcb_check(lib.lcb_fill_splitmix64(ts.data_ptr(), G * chunk, 100 + rank, native), "fill")
    stream.run()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        dist.all_to_all_single(tr, ts)
    barrier()
    ev0.record()
    for _ in range(steps):
        dist.all_to_all_single(tr, ts)
    ev1.record()
    torch.cuda.synchronize()
    ms = max_over_ranks(ev0.elapsed_time(ev1) / steps)
    report("alltoall_nccl", (G - 1) * chunk, ms)
    out["alltoall_nccl"]["verified"] = verify_recv(tr.data_ptr())
    del ts, tr
    bsz = 4 * GiB
    tb = torch.zeros(bsz, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()  # torch's fill runs on torch's stream; the generator below on this library's
    if rank == 0:
        api.lcb_check(lib.lcb_fill_splitmix64(tb.data_ptr(), bsz, 3, native), "fill")
        stream.run()
    for _ in range(2):
        dist.broadcast(tb, 0)
    barrier()
    nb = max(2, steps // 2)
    ev0.record()
    for _ in range(nb):
        dist.broadcast(tb, 0)
    ev1.record()
    torch.cuda.synchronize()
    ms = max_over_ranks(ev0.elapsed_time(ev1) / nb)
    report("broadcast_nccl_4GiB", bsz, ms)
    out["broadcast_nccl_4GiB"]["verified"] = holds_stream(tb.data_ptr(), bsz, 3, 0, salt=51)
    del tb
    torch.cuda.empty_cache()
    barrier()
    mr.close_peers(dist, peers)
    mr.close_peers(dist, send_peers)
    barrier()
    for b in (send, recv, resb, scratch):
        b.free()
    peer_rate = out["measured_peer_copy_GBps"]
    for name, entry in out.items():
        if isinstance(entry, dict) and "GBps_per_gpu_per_direction" in entry:
            entry["frac_of_measured_peer_copy"] = round(entry["GBps_per_gpu_per_direction"] / peer_rate, 4)
        if isinstance(entry, dict) and "verified" in entry:  # a check counts only if it held on every rank
            entry["verified"] = max_over_ranks(0.0 if entry["verified"] else 1.0) == 0.0
    return out


def run_one_process(api, ctx0, G, reps):
    """The single-process entry points -- one context per GPU in THIS process, peer access between all of them --
    over all G GPUs: libreCuMemcpyPartitioned (8 GiB from GPU 0), libreCuAllToAll in its three forms (1 GiB per GPU
    pair) and libreCuBroadcast in its forms (4 GiB from GPU 0).  Timed on the devices: an event on every stream
    before and after `reps` back-to-back calls (every collective starts after everything earlier on all its
    streams), the slowest stream counts.  Each form starts from cleared destinations and is verified on every
    GPU: whole buffers on the device, windows on the host against the oracle."""
    lib = api.lib
    chunk, bsz, total = GiB, 4 * GiB, 8 * GiB
    ctxs = [ctx0] + [api.Context(g, api.CU_CTX_SCHED_YIELD) for g in range(1, G)]
    streams = []
    for c in ctxs:
        c.set_current()
        for peer in ctxs:
            if peer is not c:
                c.enable_peer_access(peer)
        streams.append(api.Stream())
    natives = [s.native for s in streams]
    arr = lambda xs: (C.c_void_p * G)(*xs)
    stp = arr([s.handle for s in streams])
    starts, ends = [api.Event() for _ in range(G)], [api.Event() for _ in range(G)]
    res, scratch = [], []
    for g in range(G):
        ctxs[g].set_current()
        res.append(api.DeviceBuffer(16))
        scratch.append(api.DeviceBuffer(chunk))

    def on(g):
        ctxs[g].set_current()
        return g

    def await_all():
        for s in streams:
            s.await_()

    def timed(fn):
        for _ in range(2):
            fn()
        await_all()
        for g in range(G):
            starts[g].record(streams[g])
            streams[g].commence()
        for _ in range(reps):
            fn()
        for g in range(G):
            ends[g].record(streams[g])
            streams[g].commence()
        await_all()
        return max(api.elapsed_ms(starts[g], ends[g]) for g in range(G)) / reps

    def holds_stream(g, ptr, nbytes, seed, base, salt):
        on(g)
        ok = True
        for off in range(0, nbytes, chunk):
            m = min(chunk, nbytes - off)
            api.lcb_check(lib.lcb_fill_splitmix64_at(scratch[g].ptr, m, seed, (base + off) // 8, natives[g]), "fill")
            ok = ok and device_equal(api, streams[g], ptr + off, scratch[g].ptr, m, res[g])
        return ok and host_windows_ok(api, streams[g], ptr, nbytes, stream_expect(seed, base), salt)

    out = {"gpus": G, "timing": f"CUDA events on every stream around {reps} back-to-back calls, slowest stream"}

    def entry(gbps, ms, verified, **extra):
        e = {"GBps_per_gpu_per_direction": round(gbps, 1), "ms": round(ms, 4), "frac_of_nominal_900": round(gbps / NVLINK_NOMINAL, 4),
             "verified": bool(verified)}
        e.update(extra)
        return e

    # ---- all-to-all ----------------------------------------------------------------------------------------------
    send, recv = [], []
    for g in range(G):
        on(g)
        send.append(api.DeviceBuffer(G * chunk))
        recv.append(api.DeviceBuffer(G * chunk))
        api.lcb_check(lib.lcb_fill_splitmix64(send[g].ptr, G * chunk, 100 + g, natives[g]), "fill")
    on(0)
    sp, rp = arr([b.ptr for b in send]), arr([b.ptr for b in recv])
    for form, name in ((0, "libreCuAllToAll_0_fused_push_kernels"), (2, "libreCuAllToAll_2_copy_engines"), (1, "libreCuAllToAll_1_nccl")):
        for g in range(G):
            on(g)
            streams[g].memset_d8(recv[g], 0, G * chunk)
            streams[g].run()
        on(0)
        try:
            ms = timed(lambda: api.check(lib.libreCuAllToAll(rp, sp, chunk, G, stp, form), name))
        except api.LibreCudaError as exc:
            out[name] = {"error": str(exc)}
            continue
        ok = True
        for g in range(G):
            on(g)
            for r in range(G):
                api.lcb_check(lib.lcb_fill_splitmix64_at(scratch[g].ptr, chunk, 100 + r, g * chunk // 8, natives[g]), "fill")
                ok = ok and device_equal(api, streams[g], recv[g].ptr + r * chunk, scratch[g].ptr, chunk, res[g])
            ok = ok and host_windows_ok(api, streams[g], recv[g].ptr, G * chunk, alltoall_expect(G, chunk, g), salt=61 + g)
        out[name] = entry((G - 1) * chunk / (ms * 1e-3) / 1e9, ms, ok)
    for g in range(G):
        on(g)
        send[g].free()
        recv[g].free()

    # ---- broadcast ---------------------------------------------------------------------------------------------------
    bufs = []
    for g in range(G):
        on(g)
        bufs.append(api.DeviceBuffer(bsz))
    on(0)
    api.lcb_check(lib.lcb_fill_splitmix64(bufs[0].ptr, bsz, 3, natives[0]), "fill")
    streams[0].run()
    bp = arr([b.ptr for b in bufs])
    forms = [(5, "libreCuBroadcast_5_two_trees_of_kernels"), (4, "libreCuBroadcast_4_ring_of_kernels"), (3, "libreCuBroadcast_3_multicast_stores"), (0, "libreCuBroadcast_0_pull_and_forward_kernels"),
             (2, "libreCuBroadcast_2_copy_engine_chain"), (1, "libreCuBroadcast_1_nccl")]
    for form, name in forms:
        for g in range(1, G):
            on(g)
            streams[g].memset_d8(bufs[g], 0, bsz)
            streams[g].run()
        on(0)
        try:
            ms = timed(lambda: api.check(lib.libreCuBroadcast(bp, 0, bsz, G, stp, form), name))
        except api.LibreCudaError as exc:
            out[name] = {"error": str(exc)}
            continue
        ok = all(holds_stream(g, bufs[g].ptr, bsz, 3, 0, salt=71 + g) for g in range(G))
        ran = C.c_int(-1)
        api.check(lib.libreCuBroadcastLastForm(C.byref(ran)), "libreCuBroadcastLastForm")
        out[name] = entry(bsz / (ms * 1e-3) / 1e9, ms, ok, form_that_ran=ran.value)
    for g in range(G):
        on(g)
        bufs[g].free()

    # ---- partitioned copy: 8 GiB on GPU 0, shard g to GPU g (pulled by GPU g on its stream) ---------------------------
    on(0)
    src = api.DeviceBuffer(total)
    api.lcb_check(lib.lcb_fill_splitmix64(src.ptr, total, 3, natives[0]), "fill")
    streams[0].run()
    offs = api.partition_plan(total, G, 0)
    dsts = []
    for g in range(G):
        on(g)
        dsts.append(api.DeviceBuffer(max(offs[g + 1] - offs[g], 16)))
        streams[g].memset_d8(dsts[g], 0, dsts[g].nbytes)
        streams[g].run()
    on(0)
    dp = arr([d.ptr for d in dsts])

    def partitioned():
        api.check(lib.libreCuMemcpyPartitioned(dp, src.ptr, total, G, 0, stp), "libreCuMemcpyPartitioned")
        for s in streams:
            s.commence()

    ms = timed(partitioned)
    ok = all(holds_stream(g, dsts[g].ptr, offs[g + 1] - offs[g], 3, offs[g], salt=81 + g) for g in range(G) if offs[g + 1] > offs[g])
    out["libreCuMemcpyPartitioned_8GiB_from_gpu0"] = entry(total * (G - 1) // G / (ms * 1e-3) / 1e9, ms, ok,
                                                           note="GB/s leaving GPU 0: (G-1)/G of 8 GiB / time")
    for g in range(G):
        on(g)
        dsts[g].free()
    on(0)
    src.free()
    for g in range(G):
        on(g)
        res[g].free()
        scratch[g].free()
        streams[g].destroy()
    for e in starts + ends:
        e.destroy()
    for c in ctxs[1:]:
        c.destroy()
    on(0)
    return out


def run_case(args):
    """`--case NAME [--bytes N] [--reps R]`: launches ONE kernel of the library a few times on a small, fixed case
    and prints the CUDA-event time of each launch -- the command line that goes under a profiler (one kernel, a
    few launches, a few hundred MiB on the device).  Not a benchmark line.
      copy_auto | copy_auto_stable | copy_vec | copy_vec_stable | copy_tma | copy_tma_stable | copy_misaligned
      memset | index_fill | axpb | alltoall_2gpu (two contexts in this process, one fused push kernel per GPU)"""
    from librecuda_b200 import api

    lib = api.lib
    n = args.bytes
    ctx = api.Context(0)
    st = api.Stream()
    nat = st.native
    a, b = api.DeviceBuffer(n + 4096), api.DeviceBuffer(n + 4096)
    api.lcb_check(lib.lcb_fill_splitmix64(a.ptr, n + 4096, 1, nat), "fill")
    st.memset_d8(b, 0, n + 4096)
    st.run()
    case = args.case
    if case == "alltoall_2gpu":
        ctx1 = api.Context(1)
        ctx1.enable_peer_access(ctx)
        st1 = api.Stream()
        a1, b1 = api.DeviceBuffer(n), api.DeviceBuffer(n)
        api.lcb_check(lib.lcb_fill_splitmix64(a1.ptr, n, 2, st1.native), "fill")
        st1.run()
        t1 = api.Timer()      # events belong to the device that is current when they are created
        ctx.set_current()
        ctx.enable_peer_access(ctx1)
        t0 = api.Timer()
        recv = (C.c_void_p * 2)(b.ptr, b1.ptr)
        chunk = n // 2 // 16 * 16
        for _ in range(args.reps):
            ctx.set_current()
            t0.start(nat)
            api.lcb_check(lib.lcb_alltoall_push(recv, a.ptr, chunk, 2, 0, nat), "push 0")
            t0.stop(nat)
            ctx1.set_current()
            t1.start(st1.native)
            api.lcb_check(lib.lcb_alltoall_push(recv, a1.ptr, chunk, 2, 1, st1.native), "push 1")
            t1.stop(st1.native)
            ms1 = t1.elapsed_ms()
            ctx.set_current()
            print(f"alltoall_2gpu chunk {chunk} bytes: gpu0 {t0.elapsed_ms():.4f} ms, gpu1 {ms1:.4f} ms "
                  f"({chunk} bytes cross NVLink per GPU and direction, {chunk} stay local)")
        return 0
    paths = {"copy_auto": 0, "copy_auto_stable": SRC_STABLE, "copy_vec": 1, "copy_vec_stable": 1 | SRC_STABLE, "copy_tma": 2,
             "copy_tma_stable": 2 | SRC_STABLE, "copy_misaligned": SRC_STABLE}

    def launch():
        if case in paths:
            so = 1 if case == "copy_misaligned" else 0
            return lib.lcb_copy_d2d_ex(b.ptr, a.ptr + so, n, paths[case], 0, nat)
        if case == "memset":
            return lib.lcb_memset_d32(b.ptr, 0x40490FDB, n // 4, nat)
        if case == "index_fill":
            return lib.lcb_index_fill_f32(b.ptr, n // 4, nat)
        if case == "axpb":
            return lib.lcb_axpb_f32(b.ptr, a.ptr, 2.0, 1.0, n // 4, nat)
        raise SystemExit(f"unknown case {case}")

    if case in paths:
        print(describe_copy(api, b.ptr, a.ptr + (1 if case == "copy_misaligned" else 0), n, paths[case]))
    t = api.Timer()
    for _ in range(args.reps):
        t.start(nat)
        api.lcb_check(launch(), case)
        t.stop(nat)
        print(f"{case} {n} bytes: {t.elapsed_ms():.4f} ms")
    assert api.device_error_word() == 0
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--case", default=None, help="launch one kernel a few times on a small case (for a profiler) and exit")
    ap.add_argument("--bytes", type=int, default=256 * MiB)
    ap.add_argument("--reps", type=int, default=3)
    args = ap.parse_args()
    if args.case:
        return run_case(args)
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
