"""Behaviour of the libreCu* API on the GPU: the reference's golden call sequences, the recorded-then-
commenced execution contract, ordering (async flag, events, cross-stream waits), modules and launches."""
import ctypes as C
import time

import numpy as np
import pytest

import oracle
from librecuda_b200 import api
from conftest import FIXTURE_CUBIN
from gpu_util import to_device, to_host

pytestmark = pytest.mark.gpu
MiB = 1 << 20
lib = api.lib


@pytest.fixture(scope="module")
def module(ctx):
    ctx.set_current()
    m = api.Module(FIXTURE_CUBIN.read_bytes())
    yield m
    m.unload()


def test_device_queries(ctx):
    assert api.device_count() >= 1
    assert api.device_attribute(api.ATTR_COMPUTE_CAPABILITY_MAJOR, ctx.device) == 10
    assert api.device_attribute(api.ATTR_MAX_SHARED_MEMORY_PER_BLOCK, ctx.device) == 49152
    assert api.device_attribute(api.ATTR_MAX_SHARED_MEMORY_PER_BLOCK_OPTIN, ctx.device) >= 200 * 1024
    assert "B200" in api.device_name(ctx.device)
    v = C.c_int()
    assert lib.libreCuDeviceGetAttribute(C.byref(v), 1, ctx.device) == api.ERROR_INVALID_VALUE
    d = C.c_void_p()
    assert lib.libreCuDeviceGet(C.byref(d), 1000) == api.ERROR_INVALID_DEVICE
    cur = C.c_void_p()
    assert lib.libreCuCtxGetCurrent(C.byref(cur)) == 0 and cur.value == ctx.handle
    assert lib.libreCuInit(0) == 0  # idempotent


def test_alloc_alignment_free_rules(ctx):
    ptrs = []
    for n in (1, 100, 4096, 5000, 17 * MiB):
        b = api.DeviceBuffer(n)
        assert b.ptr % 4096 == 0
        ptrs.append(b)
    p = C.c_void_p()
    assert lib.libreCuMemAlloc(C.byref(p), 0, False) == api.ERROR_INVALID_VALUE
    assert lib.libreCuMemFree(ptrs[-1].ptr + 4096) == api.ERROR_INVALID_VALUE  # not an allocation base
    for b in ptrs:
        b.free()
    assert lib.libreCuMemFree(ptrs[0].ptr or 8) == api.ERROR_INVALID_VALUE


def test_golden_g1_dma_chronological_consistency(stream):
    # reference tests/dma_chronological_consistency/main.cpp: HtoD, five chained DtoD, DtoH on ONE stream,
    # a single Commence + Await; copy-engine and kernel work alternate and must stay in order
    n = MiB + 128 + 3
    host = (np.arange(n) % 256).astype(np.uint8)
    back = np.zeros(n, np.uint8)
    bufs = [api.DeviceBuffer(n) for _ in range(6)]
    stream.memcpy(bufs[0], host, n)
    for i in range(5):
        stream.memcpy(bufs[i + 1], bufs[i], n)
    stream.memcpy(back, bufs[5], n)
    assert not back.any()  # nothing runs before Commence
    stream.run()
    assert np.array_equal(back, host)
    for b in bufs:
        b.free()


def test_golden_g2_memcopy_floats(stream):
    src = np.arange(1, 11, dtype=np.float32)
    dst = np.zeros(10, np.float32)
    a, b = api.DeviceBuffer(40), api.DeviceBuffer(40)
    stream.memcpy(a, src, 40)
    stream.memcpy(b, a, 40)
    stream.memcpy(dst, b, 40)
    stream.run()
    assert dst.tolist() == [float(i) for i in range(1, 11)]
    a.free()
    b.free()


def test_host_buffer_is_read_at_execution_time_not_at_record_time(stream):
    n = 4096
    host = np.full(n, 1, np.uint8)
    d = api.DeviceBuffer(n)
    stream.memcpy(d, host, n)
    host[:] = 2            # after recording, before Commence
    stream.run()
    assert (to_host(stream, d, n) == 2).all()
    d.free()


def test_directional_copies_check_pointer_classes(stream):
    h = np.zeros(64, np.uint8)
    d = api.DeviceBuffer(64)
    s = stream.handle
    assert lib.libreCuMemcpyHtoD(d.ptr, h.ctypes.data, 64, s) == 0
    assert lib.libreCuMemcpyDtoH(h.ctypes.data, d.ptr, 64, s) == 0
    assert lib.libreCuMemcpyDtoD(d.ptr, d.ptr + 32, 32, s) == 0
    assert lib.libreCuMemcpyHtoD(h.ctypes.data, d.ptr, 64, s) == api.ERROR_INVALID_VALUE
    assert lib.libreCuMemcpyDtoH(d.ptr, h.ctypes.data, 64, s) == api.ERROR_INVALID_VALUE
    assert lib.libreCuMemcpyDtoD(d.ptr, h.ctypes.data, 64, s) == api.ERROR_INVALID_VALUE
    assert lib.libreCuMemsetD8(h.ctypes.data, 0, 64, s) == api.ERROR_INVALID_VALUE
    assert lib.libreCuMemsetD32(d.ptr + 2, 0, 4, s) == api.ERROR_INVALID_VALUE
    stream.run()
    d.free()


def test_config1_roundtrip_1mib_and_scalar_store(stream, module):
    # 1 MiB of seeded bytes HtoD -> DtoD -> DtoH equals host memcpy; a kernel stores 3.14159f to a 1-element buffer
    n = MiB
    src = oracle.random_bytes(n, seed=0)
    back = np.zeros(n, np.uint8)
    a, b, f = api.DeviceBuffer(n), api.DeviceBuffer(n), api.DeviceBuffer(4)
    stream.memcpy(a, src, n)
    stream.memcpy(b, a, n)
    stream.memcpy(back, b, n)
    stream.launch(module.function("store_value"), (1, 1, 1), (1, 1, 1), 0, [C.c_void_p(f.ptr), C.c_float(3.14159)])
    one = np.zeros(1, np.float32)
    stream.memcpy(one, f, 4)
    stream.run()
    want = np.empty(n, np.uint8)
    oracle.lib.orc_memcpy(want.ctypes.data, src.ctypes.data, n)
    assert np.array_equal(back, want)
    assert one.view(np.uint32)[0] == 0x40490FD0
    for x in (a, b, f):
        x.free()


def test_config2_index_kernel_over_2d_grid(stream, module):
    # 256 Mi elements: libreCuMemsetD32 to pi's bit pattern, then a user kernel out[i] = float(i) on a 2-D grid
    n = 1 << 28
    dev = api.DeviceBuffer(4 * n)
    stream.memset_d32(dev, 0x40490FDB, n)
    head = np.zeros(1024, np.uint32)
    stream.memcpy(head, dev.view(4 * (n - 1024)), 4096)
    blocks = n // 256
    gx = 32768
    stream.launch(module.function("index_fill_2d"), (gx, blocks // gx, 1), (256, 1, 1), 0, [C.c_void_p(dev.ptr), C.c_size_t(n)])
    stream.run()
    assert (head == 0x40490FDB).all()
    got = to_host(stream, dev, 4 * n).view(np.uint32)
    assert np.array_equal(got, oracle.index_fill_f32(n).view(np.uint32))
    dev.free()


def test_module_enumeration_and_errors(ctx, module):
    names = module.function_names()
    for want in ("index_fill_2d", "axpb", "store_value", "store_sum", "read_struct", "smem_sum", "spin_then_increment", "empty_kernel"):
        assert want in names
    f = C.c_void_p()
    assert lib.libreCuModuleGetFunction(C.byref(f), module.handle, b"nope") == api.ERROR_NOT_FOUND
    arr = (C.c_void_p * 1)()
    assert lib.libreCuModuleEnumerateFunctions(arr, 1, module.handle) == api.ERROR_INVALID_VALUE  # too few slots
    m = C.c_void_p()
    assert lib.libreCuModuleLoadData(C.byref(m), b"this is not a cubin image....", 29) == api.ERROR_INVALID_IMAGE


def test_launch_parameter_kinds(stream, module):
    out = api.DeviceBuffer(16, map_to_cpu=True)
    host_view = (C.c_float * 4).from_address(out.ptr)
    # short + float + module-scope global: 314 + 0.31415 + 0x69 (reference tests/write_float/main.cpp:82-113)
    stream.launch(module.function("store_sum"), (1, 1, 1), (1, 1, 1), 0, [C.c_void_p(out.ptr), C.c_short(314), C.c_float(0.31415)])
    stream.run()
    assert host_view[0] == np.float32(np.float32(314) + np.float32(0.31415) + np.float32(105))

    class S(C.Structure):
        _fields_ = [("x", C.c_int), ("y", C.c_int), ("z", C.c_int), ("w", C.c_int), ("h", C.c_int), ("d", C.c_int),
                    ("text", C.c_char * 33), ("last", C.c_char)]
    s = S(1, 2, 3, 64, 5, 6, b"hello", b"Z")
    iout = api.DeviceBuffer(8, map_to_cpu=True)
    stream.launch(module.function("read_struct"), (1, 1, 1), (1, 1, 1), 0, [s, C.c_void_p(iout.ptr)])
    stream.run()
    ints = (C.c_int * 2).from_address(iout.ptr)
    assert ints[0] == 64 and ints[1] == ord("Z")   # reference tests/kernel_struct_param prints 64

    fn = module.function("smem_sum")
    api.check(lib.libreCuFuncSetAttribute(fn, api.FUNC_ATTR_MAX_DYNAMIC_SHARED_SIZE_BYTES, 8192))
    stream.launch(fn, (1, 1, 1), (1, 1, 1), 8192, [C.c_void_p(out.ptr), C.c_short(314), C.c_float(0.31415)])
    stream.run()
    assert host_view[0] == np.float32(np.float32(314) + np.float32(0.31415))
    assert lib.libreCuFuncSetAttribute(fn, api.FUNC_ATTR_MAX_DYNAMIC_SHARED_SIZE_BYTES, 1 << 30) == api.ERROR_INVALID_VALUE

    # argument values are captured at the call, not at Commence
    v = C.c_float(1.5)
    stream.launch(module.function("store_value"), (1, 1, 1), (1, 1, 1), 0, [C.c_void_p(out.ptr), v])
    v.value = 99.0
    stream.run()
    assert host_view[0] == 1.5
    out.free()
    iout.free()


def test_launch_validation(stream, module):
    fn = module.function("store_value")
    p = [C.c_void_p(0), C.c_float(0)]
    arr = (C.c_void_p * 2)(C.cast(C.pointer(p[0]), C.c_void_p), C.cast(C.pointer(p[1]), C.c_void_p))
    s = stream.handle
    assert lib.libreCuLaunchKernel(fn, 1, 1, 1, 1, 1, 1, 0, s, arr, 1, None, False) == api.ERROR_INVALID_VALUE  # numParams
    assert lib.libreCuLaunchKernel(fn, 1, 1, 1, 2048, 1, 1, 0, s, arr, 2, None, False) == api.ERROR_LAUNCH_OUT_OF_RESOURCES
    assert lib.libreCuLaunchKernel(fn, 1, 70000, 1, 1, 1, 1, 0, s, arr, 2, None, False) == api.ERROR_LAUNCH_OUT_OF_RESOURCES
    assert lib.libreCuLaunchKernel(fn, 1, 1, 1, 1, 1, 1, 0, None, arr, 2, None, False) == api.ERROR_INVALID_VALUE
    assert lib.libreCuLaunchKernel(None, 1, 1, 1, 1, 1, 1, 0, s, arr, 2, None, False) == api.ERROR_INVALID_VALUE
    # zero-parameter kernel with an empty params array (reference tests/many_kernels_launch/main.cpp:65-76)
    stream.launch(module.function("empty_kernel"), (1, 1, 1), (1, 1, 1), 0, [])
    stream.run()


def test_many_modules_from_one_image(ctx):
    image = FIXTURE_CUBIN.read_bytes()
    mods = [api.Module(image) for _ in range(130)]
    st = api.Stream()
    for m in mods:
        st.launch(m.function("empty_kernel"), (1, 1, 1), (1, 1, 1), 0, [])
    st.run()
    for m in mods:
        m.unload()
    st.destroy()


def _cycles(ms):
    return C.c_longlong(int(ms * 1.5e6))  # ~1.5 GHz: exact duration is irrelevant, only that it is long


def test_compute_dma_compute_ordering(stream, module):
    # reference tests/compute_chronological_consistency: kernel -> 4-byte DtoD -> kernel on one stream;
    # expected "compute" value 2 and "dma" value 1
    comp, dma = api.DeviceBuffer(4, map_to_cpu=True), api.DeviceBuffer(4, map_to_cpu=True)
    cv, dv = C.c_float.from_address(comp.ptr), C.c_float.from_address(dma.ptr)
    cv.value = 0.0
    dv.value = 0.0
    fn = module.function("spin_then_increment")
    stream.launch(fn, (1, 1, 1), (1, 1, 1), 0, [C.c_void_p(comp.ptr), _cycles(20)])
    stream.memcpy(dma, comp, 4)
    stream.launch(fn, (1, 1, 1), (1, 1, 1), 0, [C.c_void_p(comp.ptr), _cycles(20)])
    stream.run()
    assert cv.value == 2.0 and dv.value == 1.0
    comp.free()
    dma.free()


def test_async_flag_overlaps_and_next_ordered_op_joins(stream, module):
    fn = module.function("spin_then_increment")
    outs = [api.DeviceBuffer(4, map_to_cpu=True) for _ in range(5)]
    for o in outs:
        C.c_float.from_address(o.ptr).value = 0.0

    def timed(async_):
        t0 = time.perf_counter()
        for o in outs:
            stream.launch(fn, (1, 1, 1), (1, 1, 1), 0, [C.c_void_p(o.ptr), _cycles(60)], async_=async_)
        stream.run()
        return time.perf_counter() - t0

    timed(False)  # warm-up
    timed(True)   # creates the side lanes (they are made on first use) outside the timed runs
    serial = timed(False)
    overlapped = min(timed(True), timed(True))
    assert overlapped < 0.6 * serial, (serial, overlapped)   # five ~40 ms kernels side by side vs back to back
    # an ordered copy after async launches sees all of them
    total = api.DeviceBuffer(4, map_to_cpu=True)
    for o in outs:
        stream.launch(fn, (1, 1, 1), (1, 1, 1), 0, [C.c_void_p(o.ptr), _cycles(5)], async_=True)
    stream.memcpy(total, outs[-1], 4)
    stream.run()
    assert C.c_float.from_address(total.ptr).value == 6.0   # six runs above, one increment each
    assert all(C.c_float.from_address(o.ptr).value == 6.0 for o in outs)
    for o in outs + [total]:
        o.free()


def test_events_timing_and_states(stream, module):
    fn = module.function("spin_then_increment")
    out = api.DeviceBuffer(4, map_to_cpu=True)
    start, end, never = api.Event(), api.Event(), api.Event()
    assert lib.libreCuEventSynchronize(never.handle) == api.ERROR_INVALID_VALUE  # never recorded
    start.record(stream)
    stream.launch(fn, (1, 1, 1), (1, 1, 1), 0, [C.c_void_p(out.ptr), _cycles(30)])
    end.record(stream)
    assert lib.libreCuEventSynchronize(end.handle) == api.ERROR_NOT_READY       # recorded, not commenced
    ms = C.c_float()
    assert lib.libreCuEventElapsedTime(C.byref(ms), start.handle, end.handle) == api.ERROR_NOT_READY
    stream.commence()
    end.synchronize()            # reference tests/stream_events: synchronize, elapsed, then Await
    assert 5.0 < api.elapsed_ms(start, end) < 500.0
    stream.await_()
    assert end.timestamp_ns() > start.timestamp_ns() > 0
    assert end.query()
    other = api.Stream()
    foreign = api.Event()
    foreign.record(other)
    other.run()
    assert lib.libreCuEventElapsedTime(C.byref(ms), start.handle, foreign.handle) == api.ERROR_INVALID_VALUE  # two streams
    # events can be recorded again
    start.record(stream)
    end.record(stream)
    stream.run()
    assert api.elapsed_ms(start, end) < 5.0
    for e in (start, end, never, foreign):
        e.destroy()
    other.destroy()
    out.free()


def test_await_reports_a_kernel_that_gave_up_a_bounded_wait(stream):
    # a copy whose bulk ring gives up a wait is incomplete although the stream finishes without a CUDA error; a
    # program written for the reference only looks at the status of Await, so Await has to say so.  The give-up
    # path is driven by the self-test kernel (a wait nothing completes, small try limit): no fault, no hang.
    stream.run()
    assert api.device_error_word() == 0
    api.lcb_check(lib.lcb_selftest_wait_timeout(2000, stream.native), "selftest")
    assert lib.libreCuStreamAwait(stream.handle) == api.ERROR_UNKNOWN      # reported once ...
    assert lib.libreCuStreamAwait(stream.handle) == api.SUCCESS            # ... and cleared
    assert api.device_error_word() == 0
    # the same through an event
    ev = api.Event()
    api.lcb_check(lib.lcb_selftest_wait_timeout(2000, stream.native), "selftest")
    ev.record(stream)
    stream.commence()
    assert lib.libreCuEventSynchronize(ev.handle) == api.ERROR_UNKNOWN
    assert lib.libreCuEventSynchronize(ev.handle) == api.SUCCESS
    stream.run()
    ev.destroy()
    # and the stream still copies
    src = np.arange(100000, dtype=np.uint8)
    d, out = api.DeviceBuffer(100000), np.zeros(100000, np.uint8)
    stream.memcpy(d, src, 100000)
    stream.memcpy(out, d, 100000)
    stream.run()
    assert np.array_equal(out, src)
    d.free()


def test_host_wait_deadline_from_the_environment():
    # LIBRECUDA_WAIT_TIMEOUT_MS is read once per process, so the case runs in a child: a kernel that spins for
    # a quarter of a second (bounded by its cycle count, nothing hangs), a 50 ms limit -> Await and EventSynchronize give up with
    # NOT_READY while it runs, and succeed when repeated after it has finished
    import os
    import subprocess
    import sys
    from pathlib import Path

    code = """
import ctypes as C, sys, time
from librecuda_b200 import api
from pathlib import Path
lib = api.lib
ctx = api.Context(0)
m = api.Module(Path(sys.argv[1]).read_bytes())
fn = m.function("spin_then_increment")
st = api.Stream()
out = api.DeviceBuffer(4, map_to_cpu=True)
C.c_float.from_address(out.ptr).value = 0.0
ev = api.Event()
st.launch(fn, (1, 1, 1), (1, 1, 1), 0, [C.c_void_p(out.ptr), C.c_longlong(int(0.25 * 1.9e9))])
ev.record(st)
st.commence()
t0 = time.perf_counter()
a = lib.libreCuStreamAwait(st.handle)
t1 = time.perf_counter()
b = lib.libreCuEventSynchronize(ev.handle)
t2 = time.perf_counter()
time.sleep(0.6)
c = lib.libreCuStreamAwait(st.handle)
d = lib.libreCuEventSynchronize(ev.handle)
print(a, b, c, d, round(t1 - t0, 3), round(t2 - t1, 3), C.c_float.from_address(out.ptr).value)
"""
    root = Path(__file__).resolve().parent.parent
    run = subprocess.run([sys.executable, "-c", code, str(FIXTURE_CUBIN)], capture_output=True, text=True, timeout=120, cwd=str(root),
                         env={**os.environ, "LIBRECUDA_WAIT_TIMEOUT_MS": "50"})
    assert run.returncode == 0, run.stderr[-2000:]
    a, b, c, d, dt_await, dt_event, value = run.stdout.split()
    assert (int(a), int(b)) == (api.ERROR_NOT_READY, api.ERROR_NOT_READY)
    assert (int(c), int(d)) == (api.SUCCESS, api.SUCCESS)
    assert 0.04 < float(dt_await) < 0.3 and 0.04 < float(dt_event) < 0.3
    assert float(value) == 1.0


def test_event_timestamps_keep_their_resolution_across_epochs(stream):
    # timestamps are measured against a chain of epochs (a new one every couple of seconds of activity), not as
    # one float distance from context creation: two events microseconds apart must not collapse, and the
    # distance between events seconds apart must agree with the host clock
    import time
    a, b, c, d = (api.Event() for _ in range(4))
    a.record(stream)
    stream.run()
    t0 = time.perf_counter()
    time.sleep(2.3)                       # long enough for the next record to start a new epoch
    b.record(stream)
    buf = api.DeviceBuffer(64 << 20)
    stream.memset_d8(buf, 1, 64 << 20)    # ~10 us of work between b and c
    c.record(stream)
    stream.run()
    host_ns = (time.perf_counter() - t0) * 1e9
    time.sleep(2.3)
    d.record(stream)
    stream.run()
    ta, tb, tc, td = (e.timestamp_ns() for e in (a, b, c, d))
    assert ta < tb < tc < td
    assert 2.0e9 < tb - ta < host_ns + 0.2e9
    assert 2_000 < tc - tb < 2_000_000    # microseconds, not zero and not the float step of an old origin
    assert abs((tc - tb) - api.elapsed_ms(b, c) * 1e6) < 2_000
    assert td - tc > 2.0e9
    for e in (a, b, c, d):
        e.destroy()
    buf.free()


def test_copy_chain_with_loads_ahead_of_the_wait_stays_ordered(stream):
    # the stream layer lets a copy load before the previous kernel has drained only when nothing in flight writes
    # its source; a chain a -> b -> c -> d (every source written by the kernel before it), interleaved with
    # independent copies and memsets, must still give exactly the sequential result
    n = 24 << 20
    rng = np.random.default_rng(5)
    host = rng.integers(0, 256, n, dtype=np.uint8)
    bufs = [api.DeviceBuffer(n + 64) for _ in range(5)]
    stream.memcpy(bufs[0], host, n)
    stream.run()
    for rep in range(3):
        stream.memset_d8(bufs[4], rep, n)                      # independent of the chain
        stream.memcpy(bufs[1].view(1, n), bufs[0], n)          # a -> b (misaligned destination)
        stream.memcpy(bufs[2], bufs[1].view(1, n), n)          # b -> c: source written by the copy before
        stream.memset_d8(bufs[3], 0xEE, n)
        stream.memcpy(bufs[3].view(16, n // 2), bufs[2], n // 2)   # c -> d (first half)
        stream.memcpy(bufs[0], bufs[2], n)                     # c -> a: same bytes back
        stream.memcpy(bufs[4], bufs[3], n)                     # d -> e: half 0xEE, half data shifted by 16
    out = np.zeros(n, np.uint8)
    stream.memcpy(out, bufs[4], n)
    stream.run()
    want = np.full(n, 0xEE, np.uint8)
    want[16:16 + n // 2] = host[:n // 2]
    assert np.array_equal(out, want)
    stream.memcpy(out, bufs[0], n)
    stream.run()
    assert np.array_equal(out, host)
    for b in bufs:
        b.free()


def test_stream_wait_event_orders_across_streams(ctx, module):
    fn = module.function("spin_then_increment")
    a, b = api.Stream(), api.Stream()
    val = api.DeviceBuffer(4, map_to_cpu=True)
    seen = api.DeviceBuffer(4, map_to_cpu=True)
    C.c_float.from_address(val.ptr).value = 0.0
    ev = api.Event()
    assert lib.libreCuStreamWaitEvent(b.handle, ev.handle) == api.ERROR_INVALID_VALUE  # never recorded
    a.launch(fn, (1, 1, 1), (1, 1, 1), 0, [C.c_void_p(val.ptr), _cycles(60)])
    ev.record(a)
    b.wait_event(ev)
    b.memcpy(seen, val, 4)
    assert lib.libreCuStreamCommence(b.handle) == api.ERROR_NOT_READY  # the event's stream was not commenced
    a.commence()
    b.commence()
    b.await_()
    assert C.c_float.from_address(seen.ptr).value == 1.0
    a.await_()
    for x in (a, b):
        x.destroy()
    ev.destroy()
    val.free()
    seen.free()


def _four_stream_pipeline(ctx, n_elems, iterations, pinned):
    """Config 4: four streams, each HtoD -> y = 2x + 1 -> DtoH per iteration; stream s iteration k waits for the
    event stream (s+1)%4 recorded at the end of iteration k-1."""
    S = 4
    nbytes = 4 * n_elems
    streams = [api.Stream() for _ in range(S)]
    xs = [oracle.random_f32(n_elems, seed=2 + s) for s in range(S)]
    if pinned:
        pin_in = [api.PinnedBuffer(nbytes) for _ in range(S)]
        pin_out = [api.PinnedBuffer(nbytes) for _ in range(S)]
        for s in range(S):
            pin_in[s].array[:] = xs[s].view(np.uint8)
        h_in = [p.array for p in pin_in]
        h_out = [p.array for p in pin_out]
    else:
        h_in = [x.view(np.uint8) for x in xs]
        h_out = [np.zeros(nbytes, np.uint8) for _ in range(S)]
    dx = [api.DeviceBuffer(nbytes) for _ in range(S)]
    dy = [api.DeviceBuffer(nbytes) for _ in range(S)]
    events = [[api.Event() for _ in range(iterations)] for _ in range(S)]
    for k in range(iterations):
        for s in range(S):
            st = streams[s]
            if k > 0:
                st.wait_event(events[(s + 1) % S][k - 1])
            st.memcpy(dx[s], h_in[s], nbytes)
            api.check(lib.libreCuMemcpyDtoD(dy[s].ptr, dx[s].ptr, 0, st.handle))  # zero-byte copies are legal no-ops
            st.launch(_four_stream_pipeline.fn, ((n_elems + 255) // 256, 1, 1), (256, 1, 1), 0,
                      [C.c_void_p(dy[s].ptr), C.c_void_p(dx[s].ptr), C.c_float(2.0), C.c_float(1.0), C.c_size_t(n_elems)])
            st.memcpy(h_out[s], dy[s], nbytes)
            events[s][k].record(st)
        for st in streams:
            st.commence()
    for st in streams:
        st.await_()
    for s in range(S):
        want = oracle.axpb_f32(xs[s], 2.0, 1.0)
        assert np.array_equal(np.asarray(h_out[s]).view(np.uint32), want.view(np.uint32))
        stamps = [events[s][k].timestamp_ns() for k in range(iterations)]
        assert all(a <= b for a, b in zip(stamps, stamps[1:])), "event timestamps must be monotone per stream"
        for k in range(1, iterations):  # the cross-stream dependency really held
            assert events[s][k].timestamp_ns() >= events[(s + 1) % S][k - 1].timestamp_ns()
    for s in range(S):
        for e in events[s]:
            e.destroy()
        dx[s].free()
        dy[s].free()
        streams[s].destroy()
    if pinned:
        for p in pin_in + pin_out:
            p.free()


def test_config4_four_stream_ordering_1000_iterations(ctx, module):
    _four_stream_pipeline.fn = module.function("axpb")
    _four_stream_pipeline(ctx, n_elems=64 * 1024, iterations=1000, pinned=False)


def test_config4_four_stream_ordering_full_size(ctx, module):
    # the full configuration: 64 MiB float32 per copy, 4 streams, 1000 iterations chained by cross-stream events
    _four_stream_pipeline.fn = module.function("axpb")
    _four_stream_pipeline(ctx, n_elems=16 * MiB, iterations=1000, pinned=True)


@pytest.mark.parametrize("n", [MiB - 1, MiB, MiB + 1, 8 * MiB, 8 * MiB + 1, 32 * MiB + 5, 71 * MiB + 13])
def test_pageable_host_copies_through_the_staging_ring(stream, n):
    # ordinary (pageable) host memory on both sides, sizes around the slot (8 MiB) and ring (4 slots) boundaries
    src = oracle.random_bytes(n + 3, seed=8)[3:]          # deliberately not page- or 16-byte aligned
    back = np.zeros(n + 1, np.uint8)[1:]
    d = api.DeviceBuffer(n + 64)
    stream.memcpy(d.view(5), src, n)
    stream.memcpy(back, d.view(5), n)
    stream.run()
    assert np.array_equal(back, src)
    # interleaved directions and an async copy on a side lane share the same ring
    back2 = np.zeros(n, np.uint8)
    e = api.DeviceBuffer(n + 64)
    stream.memcpy(e, src, n, async_=True)
    stream.memcpy(back, d.view(5), n)
    stream.memcpy(d, e, n)
    stream.memcpy(back2, d, n)
    stream.run()
    assert np.array_equal(back, src) and np.array_equal(back2, src)
    d.free()
    e.free()


def test_host_copies_beyond_4_gib(stream):
    # the reference rejects HtoD/DtoH transfers of UINT32_MAX bytes or more (driverapi/src/cmdqueue.cpp:735)
    from gpu_util import device_checksum

    n = (1 << 32) + 4096 + 3
    words = (n + 7) // 8
    host = np.arange(words, dtype=np.uint64).view(np.uint8)[:n]       # cheap to make, position-dependent
    dev = api.DeviceBuffer(n + 8)
    scratch, out = api.DeviceBuffer(api.lib.lcb_checksum_scratch_bytes()), api.DeviceBuffer(8)
    stream.memcpy(dev, host, n)
    stream.run()
    assert device_checksum(stream, dev.ptr, n, scratch, out) == oracle.checksum64(host)
    back = np.zeros(n, np.uint8)
    stream.memcpy(back, dev, n)
    stream.run()
    assert np.array_equal(back[:4096], host[:4096]) and np.array_equal(back[-8192:], host[-8192:])
    assert np.array_equal(back[(1 << 32) - 64:(1 << 32) + 64], host[(1 << 32) - 64:(1 << 32) + 64])
    assert oracle.checksum64(back) == oracle.checksum64(host)
    for b in (dev, scratch, out):
        b.free()


def test_failed_submission_drops_only_the_failed_operation(stream, module):
    # a launch the driver rejects on the host (dynamic shared memory above 48 KiB without the opt-in attribute):
    # Commence reports the error, the operations recorded after it are kept for the next Commence
    a_h, b_h = np.full(4096, 7, np.uint8), np.full(4096, 9, np.uint8)
    a, b = api.DeviceBuffer(4096), api.DeviceBuffer(4096)
    out = api.DeviceBuffer(4)
    stream.memcpy(a, a_h, 4096)
    stream.launch(module.function("store_value"), (1, 1, 1), (1, 1, 1), 100 * 1024, [C.c_void_p(out.ptr), C.c_float(1.0)])
    stream.memcpy(b, b_h, 4096)
    st = lib.libreCuStreamCommence(stream.handle)
    assert st != api.SUCCESS
    stream.run()          # submits what was left
    assert (to_host(stream, a, 4096) == 7).all() and (to_host(stream, b, 4096) == 9).all()
    for x in (a, b, out):
        x.free()
