"""ctypes loader for the CPU oracle (oracle/lcb_oracle.c) and, when built, the reference's own DtoD
dispatcher compiled for the host (oracle/_ref/libref_memcopy.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke test and by the CPU-baseline leg of the
benchmark -- never by the librecuda_b200 package.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ORACLE_SO = HERE / "_build" / "liblcb_oracle.so"
REF_SO = HERE / "_ref" / "libref_memcopy.so"


def _build_oracle():
    src = HERE / "lcb_oracle.c"
    if ORACLE_SO.exists() and ORACLE_SO.stat().st_mtime >= src.stat().st_mtime:
        return
    ORACLE_SO.parent.mkdir(exist_ok=True)
    subprocess.run(
        ["gcc", "-O2", "-fPIC", "-shared", "-pthread", "-ffp-contract=off", "-o", str(ORACLE_SO), str(src)],
        check=True,
    )


_build_oracle()
lib = C.CDLL(str(ORACLE_SO))


class Launch(C.Structure):
    _fields_ = [("kernel", C.c_int), ("grid_x", C.c_uint64), ("grid_y", C.c_uint64),
                ("offset", C.c_uint64), ("n", C.c_uint64)]


vp, sz, u64 = C.c_void_p, C.c_size_t, C.c_uint64
lib.orc_fill_bytes.argtypes = [vp, sz, u64]
lib.orc_fill_window.argtypes = [vp, sz, u64, u64]
lib.orc_fill_f32.argtypes = [vp, sz, u64]
lib.orc_ref_d2d_plan.argtypes = [u64, C.POINTER(Launch)]
lib.orc_ref_d2d_run.argtypes = [vp, vp, u64]
lib.orc_ref_d2d_run.restype = u64
lib.orc_memcpy.argtypes = [vp, vp, sz]
lib.orc_memset_d8.argtypes = [vp, C.c_uint8, sz]
lib.orc_memset_d16.argtypes = [vp, C.c_uint16, sz]
lib.orc_memset_d32.argtypes = [vp, C.c_uint32, sz]
lib.orc_index_fill_f32.argtypes = [vp, sz]
lib.orc_axpb_f32.argtypes = [vp, vp, C.c_float, C.c_float, sz]
lib.orc_checksum64.argtypes = [vp, sz]
lib.orc_checksum64.restype = u64
lib.orc_partition.argtypes = [u64, C.c_int, u64, C.POINTER(u64)]
lib.orc_alltoall.argtypes = [C.POINTER(vp), C.POINTER(vp), sz, C.c_int]
lib.orc_mt_run.argtypes = [vp, vp, sz, C.c_int, C.c_int, C.c_int, C.c_int]
lib.orc_mt_run.restype = C.c_double


def random_bytes(n: int, seed: int) -> np.ndarray:
    a = np.empty(n, np.uint8)
    lib.orc_fill_bytes(a.ctypes.data, n, seed)
    return a


def random_window(byte_offset: int, n: int, seed: int) -> np.ndarray:
    """Bytes [byte_offset, byte_offset + n) of the seeded stream that random_bytes(., seed) starts; the offset
    must be a multiple of 8 (the generator is keyed by 64-bit word position)."""
    if byte_offset % 8:
        raise ValueError("window offset must be a multiple of 8")
    a = np.empty(n, np.uint8)
    lib.orc_fill_window(a.ctypes.data, n, seed, byte_offset // 8)
    return a


def random_f32(n: int, seed: int) -> np.ndarray:
    a = np.empty(n, np.float32)
    lib.orc_fill_f32(a.ctypes.data, n, seed)
    return a


def ref_d2d_plan(size: int):
    plan = (Launch * 3)()
    n = lib.orc_ref_d2d_plan(size, plan)
    return [(p.kernel, p.grid_x, p.grid_y, p.offset, p.n) for p in plan[:n]]


def ref_d2d_run(dst: np.ndarray, src: np.ndarray, size: int) -> int:
    return lib.orc_ref_d2d_run(dst.ctypes.data, src.ctypes.data, size)


def memset(dst: np.ndarray, value: int, elem: int):
    view = dst.view({1: np.uint8, 2: np.uint16, 4: np.uint32}[elem])
    {1: lib.orc_memset_d8, 2: lib.orc_memset_d16, 4: lib.orc_memset_d32}[elem](view.ctypes.data, value, view.size)


def index_fill_f32(n: int) -> np.ndarray:
    a = np.empty(n, np.float32)
    lib.orc_index_fill_f32(a.ctypes.data, n)
    return a


def axpb_f32(x: np.ndarray, a: float, b: float) -> np.ndarray:
    y = np.empty_like(x)
    lib.orc_axpb_f32(y.ctypes.data, x.ctypes.data, a, b, x.size)
    return y


def checksum64(a: np.ndarray) -> int:
    a = np.ascontiguousarray(a).view(np.uint8)
    return lib.orc_checksum64(a.ctypes.data, a.size)


def partition(total: int, parts: int, align: int):
    out = (u64 * (parts + 1))()
    rc = lib.orc_partition(total, parts, align, out)
    if rc:
        raise ValueError("bad partition arguments")
    return list(out)


def alltoall(send):
    """send: list of n uint8 arrays of n*chunk bytes -> list of n received arrays."""
    n = len(send)
    chunk = send[0].size // n
    recv = [np.zeros(n * chunk, np.uint8) for _ in range(n)]
    rp = (vp * n)(*[r.ctypes.data for r in recv])
    sp = (vp * n)(*[s.ctypes.data for s in send])
    lib.orc_alltoall(rp, sp, chunk, n)
    return recv


def mt_seconds(dst: np.ndarray, src, op: int, value: int, threads: int, reps: int) -> float:
    """Best-of-`reps` seconds of a `threads`-way memcpy (op 0) or memset (op 1) over dst.nbytes."""
    return lib.orc_mt_run(dst.ctypes.data, src.ctypes.data if src is not None else None, dst.nbytes, op, value,
                          threads, reps)


# ---- the reference's own dispatcher + kernels on the host (only where oracle/_ref was built) ---------------
ref = None
if REF_SO.exists():
    ref = C.CDLL(str(REF_SO))
    ref.ref_memcpy_d2d.argtypes = [vp, vp, u64, C.c_int, C.c_int, C.POINTER(u64)]
    ref.ref_status_name.argtypes = [C.c_int]
    ref.ref_status_name.restype = C.c_char_p


def reference_d2d(dst: np.ndarray, src: np.ndarray, size: int, execute: bool = True, async_: bool = False):
    """Runs the reference's memcpyD2D on host buffers; returns its launch log
    [(kernel, grid_x, grid_y, offset, n, async), ...]."""
    if ref is None:
        raise RuntimeError("oracle/_ref is not built (oracle/build_ref.sh needs a reference checkout)")
    log = (u64 * 48)()
    n = ref.ref_memcpy_d2d(dst.ctypes.data, src.ctypes.data, size, int(execute), int(async_), log)
    if n < 0:
        raise RuntimeError(f"reference memcpyD2D failed with status {-n}")
    return [tuple(log[6 * i: 6 * i + 6]) for i in range(n)]
