"""Python mirror of the libreCu* API (include/librecuda.h) over ctypes.

Same names, argument meaning and error behaviour as the C API: every wrapper forwards to the exported
function of the same name and raises `LibreCudaError` carrying the status code when the call does not
return LIBRECUDA_SUCCESS.  The small classes only hold handles; there is no Python-side data path.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _native as N

lib = N.lib

SUCCESS = 0
ERROR_INVALID_VALUE = 1
ERROR_OUT_OF_MEMORY = 2
ERROR_NOT_INITIALIZED = 3
ERROR_INVALID_DEVICE = 101
ERROR_INVALID_IMAGE = 200
ERROR_INVALID_CONTEXT = 201
ERROR_NOT_FOUND = 500
ERROR_NOT_READY = 600
ERROR_LAUNCH_OUT_OF_RESOURCES = 701
ERROR_COMPAT_NOT_SUPPORTED_ON_DEVICE = 804
ERROR_UNKNOWN = 999

CU_CTX_SCHED_SPIN = 0x01
CU_CTX_SCHED_YIELD = 0x02
CU_CTX_SCHED_BLOCKING_SYNC = 0x04

ATTR_MAX_SHARED_MEMORY_PER_BLOCK = 8
ATTR_COMPUTE_CAPABILITY_MAJOR = 75
ATTR_COMPUTE_CAPABILITY_MINOR = 76
ATTR_MAX_SHARED_MEMORY_PER_BLOCK_OPTIN = 97
FUNC_ATTR_MAX_DYNAMIC_SHARED_SIZE_BYTES = 8


class LibreCudaError(RuntimeError):
    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(f"{what} -> {error_string(status)} ({status})")


def error_string(status: int):
    out = C.c_char_p()
    lib.libreCuGetErrorString(status, C.byref(out))
    return out.value.decode() if out.value else None


def check(status: int, what: str = "libreCu call"):
    if status != SUCCESS:
        raise LibreCudaError(status, what)


def _ptr(x) -> int:
    """Address of a DeviceBuffer / numpy array / int."""
    if isinstance(x, DeviceBuffer):
        return x.ptr
    if isinstance(x, np.ndarray):
        return x.ctypes.data
    return int(x)


def init(flags: int = 0):
    check(lib.libreCuInit(flags), "libreCuInit")


def device_count() -> int:
    n = C.c_int()
    check(lib.libreCuDeviceGetCount(C.byref(n)), "libreCuDeviceGetCount")
    return n.value


def device_get(ordinal: int) -> int:
    d = C.c_void_p()
    check(lib.libreCuDeviceGet(C.byref(d), ordinal), "libreCuDeviceGet")
    return d.value


def device_attribute(attr: int, device: int) -> int:
    v = C.c_int()
    check(lib.libreCuDeviceGetAttribute(C.byref(v), attr, device), "libreCuDeviceGetAttribute")
    return v.value


def device_name(device: int) -> str:
    buf = C.create_string_buffer(256)
    check(lib.libreCuDeviceGetName(buf, 256, device), "libreCuDeviceGetName")
    return buf.value.decode()


class Context:
    def __init__(self, ordinal: int = 0, flags: int = CU_CTX_SCHED_YIELD):
        init()
        self.device = device_get(ordinal)
        self.ordinal = ordinal
        h = C.c_void_p()
        check(lib.libreCuCtxCreate_v2(C.byref(h), flags, self.device), "libreCuCtxCreate_v2")
        self.handle = h.value

    def set_current(self):
        check(lib.libreCuCtxSetCurrent(self.handle), "libreCuCtxSetCurrent")

    def enable_peer_access(self, peer: "Context"):
        """Let the CURRENT context access memory of `peer`."""
        check(lib.libreCuCtxEnablePeerAccess(peer.handle, 0), "libreCuCtxEnablePeerAccess")

    def destroy(self):
        if self.handle:
            check(lib.libreCuCtxDestroy(self.handle), "libreCuCtxDestroy")
            self.handle = None


class DeviceBuffer:
    """A libreCuMemAlloc allocation (or a view `base + offset` into one)."""

    def __init__(self, nbytes: int, map_to_cpu: bool = False, _ptr: int | None = None, _owner=None):
        self.nbytes = nbytes
        self.owner = _owner
        if _ptr is not None:
            self.ptr = _ptr
            return
        p = C.c_void_p()
        check(lib.libreCuMemAlloc(C.byref(p), nbytes, map_to_cpu), "libreCuMemAlloc")
        self.ptr = p.value

    def view(self, offset: int, nbytes: int | None = None) -> "DeviceBuffer":
        n = self.nbytes - offset if nbytes is None else nbytes
        assert 0 <= offset and offset + n <= self.nbytes
        return DeviceBuffer(n, _ptr=self.ptr + offset, _owner=self)

    def free(self):
        if self.owner is None and self.ptr:
            check(lib.libreCuMemFree(self.ptr), "libreCuMemFree")
            self.ptr = 0


class PinnedBuffer:
    """Page-locked host memory from libreCuMemAllocHost, exposed as a numpy uint8 array."""

    def __init__(self, nbytes: int):
        p = C.c_void_p()
        check(lib.libreCuMemAllocHost(C.byref(p), nbytes), "libreCuMemAllocHost")
        self.ptr = p.value
        self.nbytes = nbytes
        self.array = np.ctypeslib.as_array((C.c_ubyte * nbytes).from_address(self.ptr))

    def free(self):
        if self.ptr:
            self.array = None
            check(lib.libreCuMemFreeHost(self.ptr), "libreCuMemFreeHost")
            self.ptr = 0


class Event:
    def __init__(self):
        h = C.c_void_p()
        check(lib.libreCuEventCreate(C.byref(h), 0), "libreCuEventCreate")
        self.handle = h.value

    def record(self, stream: "Stream"):
        check(lib.libreCuEventRecord(self.handle, stream.handle), "libreCuEventRecord")

    def synchronize(self):
        check(lib.libreCuEventSynchronize(self.handle), "libreCuEventSynchronize")

    def query(self) -> bool:
        st = lib.libreCuEventQuery(self.handle)
        if st == ERROR_NOT_READY:
            return False
        check(st, "libreCuEventQuery")
        return True

    def timestamp_ns(self) -> int:
        t = C.c_uint64()
        check(lib.libreCuEventGetTimestamp(C.byref(t), self.handle), "libreCuEventGetTimestamp")
        return t.value

    def destroy(self):
        if self.handle:
            check(lib.libreCuEventDestroy(self.handle), "libreCuEventDestroy")
            self.handle = None


def elapsed_ms(start: Event, end: Event) -> float:
    ms = C.c_float()
    check(lib.libreCuEventElapsedTime(C.byref(ms), start.handle, end.handle), "libreCuEventElapsedTime")
    return ms.value


class Stream:
    def __init__(self):
        h = C.c_void_p()
        check(lib.libreCuStreamCreate(C.byref(h), 0), "libreCuStreamCreate")
        self.handle = h.value

    @property
    def native(self) -> int:
        p = C.c_void_p()
        check(lib.libreCuStreamGetNativeHandle(C.byref(p), self.handle), "libreCuStreamGetNativeHandle")
        return p.value or 0

    def memcpy(self, dst, src, nbytes: int, async_: bool = False):
        check(lib.libreCuMemCpy(_ptr(dst), _ptr(src), nbytes, self.handle, async_), "libreCuMemCpy")

    def memset_d8(self, dst, value: int, count: int):
        check(lib.libreCuMemsetD8(_ptr(dst), value, count, self.handle), "libreCuMemsetD8")

    def memset_d16(self, dst, value: int, count: int):
        check(lib.libreCuMemsetD16(_ptr(dst), value, count, self.handle), "libreCuMemsetD16")

    def memset_d32(self, dst, value: int, count: int):
        check(lib.libreCuMemsetD32(_ptr(dst), value, count, self.handle), "libreCuMemsetD32")

    def wait_event(self, event: Event):
        check(lib.libreCuStreamWaitEvent(self.handle, event.handle), "libreCuStreamWaitEvent")

    def launch(self, function: int, grid, block, smem: int, params, async_: bool = False):
        """`params`: list of ctypes values (c_void_p, c_float, c_size_t, structs ...)."""
        n = len(params)
        arr = (C.c_void_p * max(n, 1))()
        for i, p in enumerate(params):
            arr[i] = C.cast(C.pointer(p), C.c_void_p)
        check(
            lib.libreCuLaunchKernel(function, grid[0], grid[1], grid[2], block[0], block[1], block[2], smem,
                                    self.handle, arr, n, None, async_),
            "libreCuLaunchKernel",
        )

    def commence(self):
        check(lib.libreCuStreamCommence(self.handle), "libreCuStreamCommence")

    def await_(self):
        check(lib.libreCuStreamAwait(self.handle), "libreCuStreamAwait")

    def run(self):
        """Commence followed by Await, the pattern every reference program uses."""
        self.commence()
        self.await_()

    def destroy(self):
        if self.handle:
            check(lib.libreCuStreamDestroy(self.handle), "libreCuStreamDestroy")
            self.handle = None


class Module:
    def __init__(self, image: bytes):
        self._image = image
        h = C.c_void_p()
        check(lib.libreCuModuleLoadData(C.byref(h), image, len(image)), "libreCuModuleLoadData")
        self.handle = h.value

    def function_names(self):
        n = C.c_uint32()
        check(lib.libreCuModuleGetFunctionCount(C.byref(n), self.handle), "libreCuModuleGetFunctionCount")
        arr = (C.c_void_p * max(n.value, 1))()
        check(lib.libreCuModuleEnumerateFunctions(arr, n.value, self.handle), "libreCuModuleEnumerateFunctions")
        names = []
        for i in range(n.value):
            s = C.c_char_p()
            check(lib.libreCuFuncGetName(C.byref(s), arr[i]), "libreCuFuncGetName")
            names.append(s.value.decode())
        return names

    def function(self, name: str) -> int:
        f = C.c_void_p()
        check(lib.libreCuModuleGetFunction(C.byref(f), self.handle, name.encode()), "libreCuModuleGetFunction")
        return f.value

    def unload(self):
        if self.handle:
            check(lib.libreCuModuleUnload(self.handle), "libreCuModuleUnload")
            self.handle = None


def partition_plan(total: int, parts: int, align: int = 0):
    out = (C.c_size_t * (parts + 1))()
    check(lib.libreCuPartitionPlan(total, parts, align, out), "libreCuPartitionPlan")
    return list(out)


# ---- kernel layer (lcb_*) conveniences ---------------------------------------------------------------------

def lcb_check(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what} failed: cudaError {rc}")


def tune(**knobs):
    for k, v in knobs.items():
        lcb_check(lib.lcb_tune(k.encode(), int(v)), f"lcb_tune({k})")


def tune_reset():
    lcb_check(lib.lcb_tune(b"reset", 0), "lcb_tune(reset)")


class Timer:
    """CUDA-event stopwatch on a raw stream (lcb_timer_*)."""

    def __init__(self):
        h = C.c_void_p()
        lcb_check(lib.lcb_timer_create(C.byref(h)), "lcb_timer_create")
        self.handle = h.value

    def start(self, native_stream: int):
        lcb_check(lib.lcb_timer_start(self.handle, native_stream), "lcb_timer_start")

    def stop(self, native_stream: int):
        lcb_check(lib.lcb_timer_stop(self.handle, native_stream), "lcb_timer_stop")

    def elapsed_ms(self) -> float:
        ms = C.c_float()
        lcb_check(lib.lcb_timer_elapsed_ms(self.handle, C.byref(ms)), "lcb_timer_elapsed_ms")
        return ms.value

    def destroy(self):
        if self.handle:
            lib.lcb_timer_destroy(self.handle)
            self.handle = None


def device_error_word() -> int:
    w = C.c_uint()
    lcb_check(lib.lcb_device_error_word(C.byref(w)), "lcb_device_error_word")
    return w.value
