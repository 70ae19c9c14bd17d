"""Runs ONE kernel of the library a few times on a small, fixed case -- the command to put under a profiler.

    python -m librecuda_b200.profile_case copy   [--bytes N] [--reps R] [--path auto|vec|tma|vec32] [--src-off A] [--dst-off B]
    python -m librecuda_b200.profile_case memset [--bytes N] [--reps R] [--path auto|vec|bulk]
    python -m librecuda_b200.profile_case index_fill | axpb | checksum | alltoall_self
    python -m librecuda_b200.profile_case sweep  [--max-log2 33]     (timing table, not for a profiler)
    python -m librecuda_b200.profile_case multigpu [--gpus G] [--bytes N]   (one process driving G GPUs)

The default 256 MiB per buffer is larger than the 126 MB L2 (DRAM counters stay meaningful) and small
enough for a multi-pass capture to finish in about a minute.  Prints the CUDA-event time per launch.
"""
from __future__ import annotations

import argparse
import ctypes as C

from . import api

PATHS = {"auto": 0, "vec": 1, "tma": 2, "small": 3, "vec32": 4}
MEMSET_PATHS = {"auto": 0, "vec": 1, "bulk": 2}


def sweep(max_log2: int):
    """DtoD copy and memset GB/s for sizes 4 KiB .. 2^max_log2 and a few src/dst byte offsets, timed with CUDA
    events over back-to-back launches (best of 3 batches).  Copies count read + write bytes."""
    lib = api.lib
    api.Context(0)
    st = api.Stream()
    nat = st.native
    top = 1 << max_log2
    a, b = api.DeviceBuffer(top + 256), api.DeviceBuffer(top + 256)
    api.lcb_check(lib.lcb_fill_splitmix64(a.ptr, top, 1, nat), "fill")
    st.memset_d8(b, 0, top)
    st.run()
    t = api.Timer()

    def timed(fn, reps):
        for _ in range(3):
            api.lcb_check(fn(), "launch")
        best = 1e30
        for _ in range(3):
            t.start(nat)
            for _ in range(reps):
                api.lcb_check(fn(), "launch")
            t.stop(nat)
            best = min(best, t.elapsed_ms() / reps)
        return best

    offsets = [(0, 0), (1, 0), (0, 3), (7, 7), (64, 1)]
    print("| bytes | " + " | ".join(f"copy src+{so} dst+{do}" for so, do in offsets) + " | memset D8 | us per aligned copy |")
    print("|---|" + "---|" * (len(offsets) + 2))
    for k in range(12, max_log2 + 1):
        n = 1 << k
        reps = 200 if n <= (16 << 20) else (20 if n <= (1 << 30) else 5)
        cells = []
        us = 0.0
        for so, do in offsets:
            ms = timed(lambda: lib.lcb_copy_d2d(b.ptr + do, a.ptr + so, n, nat), reps)
            if (so, do) == (0, 0):
                us = ms * 1e3
            cells.append(f"{2 * n / (ms * 1e-3) / 1e9:.1f}")
        ms = timed(lambda: lib.lcb_memset_d8(b.ptr, 0x5A, n, nat), reps)
        cells.append(f"{n / (ms * 1e-3) / 1e9:.1f}")
        print(f"| {n} | " + " | ".join(cells) + f" | {us:.1f} |", flush=True)
    assert api.device_error_word() == 0
    t.destroy()


def multigpu(n_gpus: int, nbytes: int, reps: int):
    """libreCuBroadcast and libreCuAllToAll, own kernels against NCCL, in ONE process with a context per GPU.
    Host wall clock around Commence..Await of all streams (the operations take milliseconds); GB/s per GPU:
    broadcast = bytes / time, all-to-all = (G-1) * chunk / time."""
    import time

    lib = api.lib
    api.init()
    G = min(n_gpus, api.device_count())
    ctxs = [api.Context(i) for i in range(G)]
    streams, bufs, send, recv = [], [], [], []
    chunk = nbytes // G // 16 * 16
    for c in ctxs:
        c.set_current()
        for peer in ctxs:
            if peer is not c:
                c.enable_peer_access(peer)
        streams.append(api.Stream())
        bufs.append(api.DeviceBuffer(nbytes))
        send.append(api.DeviceBuffer(G * chunk))
        recv.append(api.DeviceBuffer(G * chunk))
        api.lcb_check(lib.lcb_fill_splitmix64(send[-1].ptr, G * chunk, 40 + len(send), streams[-1].native), "fill")
        streams[-1].run()
    ctxs[0].set_current()
    arr = lambda xs: (C.c_void_p * G)(*xs)
    bp, sp, rp = arr([b.ptr for b in bufs]), arr([b.ptr for b in send]), arr([b.ptr for b in recv])
    stp = arr([s.handle for s in streams])

    def timed(fn):
        best = 1e30
        for i in range(reps + 2):
            t0 = time.perf_counter()
            api.check(fn(), "collective")
            for s in streams:
                s.await_()
            if i >= 2:
                best = min(best, time.perf_counter() - t0)
        return best

    print(f"{G} GPUs, one process; broadcast {nbytes} bytes from device 0, all-to-all {chunk} bytes per pair")
    for name, use_nccl in (("own kernels", 0), ("NCCL", 1)):
        t = timed(lambda: lib.libreCuBroadcast(bp, 0, nbytes, G, stp, use_nccl))
        print(f"broadcast  {name:12s} {t * 1e3:8.3f} ms  {nbytes / t / 1e9:7.1f} GB/s")
        t = timed(lambda: lib.libreCuAllToAll(rp, sp, chunk, G, stp, use_nccl))
        print(f"all-to-all {name:12s} {t * 1e3:8.3f} ms  {(G - 1) * chunk / t / 1e9:7.1f} GB/s per GPU")
    for piece in (0, 32, 64, 128):
        api.tune(bcast_engine_piece_mib=piece)
        t = timed(lambda: lib.libreCuBroadcast(bp, 0, nbytes, G, stp, 2))
        print(f"broadcast  engine chain, {piece or 'auto'} MiB pieces {t * 1e3:8.3f} ms  {nbytes / t / 1e9:7.1f} GB/s")
    api.tune_reset()
    t = timed(lambda: lib.libreCuAllToAll(rp, sp, chunk, G, stp, 2))
    print(f"all-to-all {'copy engines':12s} {t * 1e3:8.3f} ms  {(G - 1) * chunk / t / 1e9:7.1f} GB/s per GPU")
    # one peer copy through libreCuMemCpy, device 0 -> device 1: copy engine (default) against the copy kernel
    for engine in (1, 0):
        api.tune(peer_copy_engine=engine)
        t = timed(lambda: lib.libreCuMemCpy(bufs[1].ptr, bufs[0].ptr, nbytes, streams[0].handle, False)
                  or lib.libreCuStreamCommence(streams[0].handle))
        print(f"peer copy  {'engine' if engine else 'kernel':12s} {t * 1e3:8.3f} ms  {nbytes / t / 1e9:7.1f} GB/s")
    api.tune_reset()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["copy", "memset", "index_fill", "axpb", "checksum", "compare", "alltoall_self", "sweep", "multigpu"])
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--max-log2", type=int, default=33)
    ap.add_argument("--bytes", type=int, default=256 << 20)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--path", default="auto")
    ap.add_argument("--src-off", type=int, default=0)
    ap.add_argument("--dst-off", type=int, default=0)
    args = ap.parse_args()
    if args.kernel == "sweep":
        return sweep(args.max_log2)
    if args.kernel == "multigpu":
        return multigpu(args.gpus, args.bytes if args.bytes != (256 << 20) else (4 << 30), max(args.reps, 5))
    lib = api.lib
    api.Context(0)
    st = api.Stream()
    nat = st.native
    n = args.bytes
    a, b = api.DeviceBuffer(n + 4096), api.DeviceBuffer(n + 4096)
    api.lcb_check(lib.lcb_fill_splitmix64(a.ptr, n + 4096, 1, nat), "fill")
    st.memset_d8(b, 0, n + 4096)
    st.run()
    scratch, out = api.DeviceBuffer(lib.lcb_checksum_scratch_bytes()), api.DeviceBuffer(8)
    res = api.DeviceBuffer(16)
    peers = (C.c_void_p * 2)(b.ptr, b.ptr + (n // 32) * 16)

    def launch():
        if args.kernel == "copy":
            return lib.lcb_copy_d2d_ex(b.ptr + args.dst_off, a.ptr + args.src_off, n, PATHS[args.path], 0, nat)
        if args.kernel == "memset":
            return lib.lcb_memset_ex(b.ptr, 0x40490FDB, 4, n // 4, MEMSET_PATHS[args.path], 0, nat)
        if args.kernel == "index_fill":
            return lib.lcb_index_fill_f32(b.ptr, n // 4, nat)
        if args.kernel == "axpb":
            return lib.lcb_axpb_f32(b.ptr, a.ptr, 2.0, 1.0, n // 4, nat)
        if args.kernel == "checksum":
            return lib.lcb_checksum64(a.ptr, n, scratch.ptr, out.ptr, nat)
        if args.kernel == "compare":
            return lib.lcb_compare_bytes(a.ptr + args.src_off, b.ptr + args.dst_off, n, res.ptr, nat)
        # two "ranks" folded onto one GPU: both halves of the send buffer land in this GPU's memory
        return lib.lcb_alltoall_push(peers, a.ptr, (n // 64) * 16, 2, 0, nat)

    t = api.Timer()
    for _ in range(args.reps):
        t.start(nat)
        api.lcb_check(launch(), args.kernel)
        t.stop(nat)
        print(f"{args.kernel} {args.path} {n} bytes: {t.elapsed_ms():.4f} ms")
    assert api.device_error_word() == 0
    t.destroy()


if __name__ == "__main__":
    main()
