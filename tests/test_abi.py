"""The C-ABI boundary, without a GPU: the shared library loads, exports every symbol the public headers
declare (functions and the status data symbols), and the host-only logic behaves like the reference's."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

import oracle
from librecuda_b200 import _native as N
from librecuda_b200 import api

INCLUDE = Path(__file__).resolve().parent.parent / "include"


def _declared(header: str, prefix: str):
    text = (INCLUDE / header).read_text()
    text = re.sub(r"//.*", "", text)
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(" + prefix + r"\w+)\s*\(", text)))


def test_every_lcb_symbol_is_exported_and_bound():
    names = _declared("lcb200_kernels.h", "lcb_")
    assert len(names) >= 20
    for name in names:
        assert hasattr(N.lib, name), f"{name} declared in lcb200_kernels.h but not exported"
        assert name in N.LCB_FUNCTIONS, f"{name} has no ctypes prototype"


def test_every_librecu_symbol_is_exported_and_bound():
    names = _declared("librecuda.h", "libreCu")
    assert len(names) >= 30 + 25
    for name in names:
        assert hasattr(N.lib, name), f"{name} declared in librecuda.h but not exported"
        assert name in N.LIBRECU_FUNCTIONS, f"{name} has no ctypes prototype"


def test_reference_surface_is_complete():
    # the 30 entry points of the reference header (driverapi/include/librecuda.h:37-114)
    ref30 = """libreCuInit libreCuDeviceGetCount libreCuDeviceGet libreCuGetErrorString libreCuCtxCreate_v2
    libreCuCtxDestroy libreCuCtxSetCurrent libreCuCtxGetCurrent libreCuMemAlloc libreCuMemCpy libreCuMemFree
    libreCuStreamCreate libreCuStreamDestroy libreCuDeviceGetName libreCuDeviceGetAttribute libreCuFuncSetAttribute
    libreCuModuleLoadData libreCuModuleGetFunctionCount libreCuModuleEnumerateFunctions libreCuFuncGetName
    libreCuModuleGetFunction libreCuLaunchKernel libreCuEventCreate libreCuEventRecord libreCuEventSynchronize
    libreCuEventElapsedTime libreCuEventDestroy libreCuStreamCommence libreCuStreamAwait libreCuModuleUnload""".split()
    assert len(ref30) == 30
    for name in ref30:
        assert hasattr(N.lib, name)


def test_status_values_are_data_symbols():
    for name, value in N.STATUS_VARIABLES.items():
        assert C.c_int.in_dll(N.lib, name).value == value
        assert api.error_string(value) == name
    assert api.error_string(12345) is None  # unknown code: null name, success status


@pytest.mark.skipif(oracle.ref is None, reason="oracle/_ref not built (no reference checkout)")
def test_status_names_match_reference_table():
    for value in list(N.STATUS_VARIABLES.values()) + [7, 12345]:
        want = oracle.ref.ref_status_name(value)
        got = api.error_string(value)
        assert (want.decode() if want else None) == got


def test_version_string():
    assert N.lib.lcb_version().startswith(b"lcb200")


def test_calls_before_init_or_without_context_fail_like_the_reference(gpu_count):
    n = C.c_int()
    if gpu_count == 0:
        # no driver here: init must fail loudly, never fall back
        assert N.lib.libreCuInit(0) == api.ERROR_COMPAT_NOT_SUPPORTED_ON_DEVICE
        assert N.lib.libreCuDeviceGetCount(C.byref(n)) == api.ERROR_NOT_INITIALIZED
        p = C.c_void_p()
        assert N.lib.libreCuMemAlloc(C.byref(p), 4096, False) == api.ERROR_INVALID_CONTEXT
        s = C.c_void_p()
        assert N.lib.libreCuStreamCreate(C.byref(s), 0) == api.ERROR_INVALID_CONTEXT
    assert N.lib.libreCuDeviceGetCount(None) == api.ERROR_INVALID_VALUE
    assert N.lib.libreCuMemCpy(None, None, 4, None, False) == api.ERROR_INVALID_VALUE
    assert N.lib.libreCuMemFree(None) == api.ERROR_INVALID_VALUE
    assert N.lib.libreCuCtxSetCurrent(None) == api.ERROR_INVALID_CONTEXT
    assert N.lib.libreCuCtxDestroy(None) == api.ERROR_INVALID_CONTEXT
    assert N.lib.libreCuEventSynchronize(None) == api.ERROR_INVALID_VALUE


def test_kernel_layer_rejects_bad_arguments_without_touching_a_gpu():
    assert N.lib.lcb_copy_d2d(None, None, 0, None) == 0          # empty copy is a no-op
    assert N.lib.lcb_copy_d2d(None, 16, 16, None) == 1
    assert N.lib.lcb_copy_d2d_ex(16, 32, 16, 99, 0, None) == 1   # unknown path
    assert N.lib.lcb_copy_d2d_ex(16, 33, 64, 2, 0, None) == 1    # bulk path needs congruent pointers
    assert N.lib.lcb_memset_ex(16, 0, 3, 4, 0, 0, None) == 1     # element size 3
    assert N.lib.lcb_memset_d32(18, 0, 4, None) == 1             # misaligned for 4-byte elements
    assert N.lib.lcb_memset_d8(None, 0, 0, None) == 0
    assert N.lib.lcb_index_fill_f32(6, 4, None) == 1
    assert N.lib.lcb_tune(b"no_such_knob", 1) == 1
    assert N.lib.lcb_checksum_scratch_bytes() >= 8 * 1185
    peers = (C.c_void_p * 2)(4096, 8192)
    assert N.lib.lcb_alltoall_push(peers, 4096, 24, 2, 0, None) == 1   # chunk not a multiple of 16
    assert N.lib.lcb_alltoall_push(peers, 4096, 32, 2, 5, None) == 1   # rank out of range
    assert N.lib.lcb_alltoall_pull(peers, 4096, 24, 2, 0, None) == 1
    assert N.lib.lcb_alltoall_pull(peers, 4097, 32, 2, 0, None) == 1   # misaligned receive buffer


@pytest.mark.parametrize("total,parts,align", [(8 << 30, 8, 0), (8 << 30, 4, 2 << 20), (10 * (1 << 20) + 5, 4, 2 << 20),
                                               (1 << 20, 8, 0), (0, 3, 4096), (4097, 2, 4096), (100, 7, 16), (5, 1, 16)])
def test_partition_plan_matches_oracle(total, parts, align):
    assert api.partition_plan(total, parts, align) == oracle.partition(total, parts, align or (2 << 20))


def test_partition_plan_rejects_bad_arguments():
    out = (C.c_size_t * 4)()
    assert N.lib.libreCuPartitionPlan(100, 0, 16, out) == api.ERROR_INVALID_VALUE
    assert N.lib.libreCuPartitionPlan(100, 2, 24, out) == api.ERROR_INVALID_VALUE
    assert N.lib.libreCuPartitionPlan(100, 2, 16, None) == api.ERROR_INVALID_VALUE


def test_tunables_roundtrip_and_environment_override():
    import subprocess
    import sys

    assert N.lib.lcb_tune(b"bcast_piece_mib", 48) == 0 and N.lib.lcb_tune_get(b"bcast_piece_mib") == 48
    assert N.lib.lcb_tune(b"reset", 0) == 0 and N.lib.lcb_tune_get(b"bcast_piece_mib") == 64
    assert N.lib.lcb_tune_get(b"no_such_knob") == -1
    code = ("from librecuda_b200 import _native as N; "
            "print(N.lib.lcb_tune_get(b'a2a_ctas_sm'), N.lib.lcb_tune_get(b'pdl'), N.lib.lcb_tune_get(b'auto_tma_min_mib'))")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=str(INCLUDE.parent),
                         env={**__import__("os").environ, "LCB_TUNE": "a2a_ctas_sm=7,pdl=0,bogus=3"})
    assert out.returncode == 0, out.stderr
    assert out.stdout.split() == ["7", "0", "96"]


def test_tunables_refuse_values_that_would_break_a_kernel():
    # a refused value leaves the previous one in place; "reset" returns to the start-up configuration
    lib = N.lib
    assert lib.lcb_tune(b"memset_threads", 128) == 0
    for knob, bad in ((b"memset_threads", 32), (b"memset_threads", 0), (b"memset_threads", 1024), (b"memset_threads", 100),
                      (b"copy_vec_threads", 32), (b"copy_vec_threads", -64), (b"copy_vec_threads", 544),
                      (b"copy_vec_unroll", 3), (b"memset_unroll", 0), (b"copy_cache_mode", 9), (b"tma_chunk", 1000),
                      (b"tma_chunk", 131072), (b"tma_stages", 1), (b"tma_lookahead", 0), (b"pdl", 2), (b"a2a_ctas_sm", -1)):
        before = lib.lcb_tune_get(knob)
        assert lib.lcb_tune(knob, bad) == 1, (knob, bad)
        assert lib.lcb_tune_get(knob) == before, (knob, bad)
    assert lib.lcb_tune_get(b"memset_threads") == 128
    assert lib.lcb_tune(b"copy_vec_threads", 0) == 0 and lib.lcb_tune(b"copy_vec_threads", 256) == 0
    assert lib.lcb_tune(b"reset", 0) == 0
    assert lib.lcb_tune_get(b"memset_threads") == 256 and lib.lcb_tune_get(b"copy_vec_threads") == 0


def test_copy_plan_query_follows_the_dispatcher():
    # no GPU needed: the query runs the dispatcher's own decision code without launching
    lib = N.lib
    buf = C.create_string_buffer(200)

    def plan(dst, src, n, path=0):
        assert lib.lcb_copy_d2d_describe(dst, src, n, path, 0, buf, 200) == 0
        return buf.value.decode()

    MiB = 1 << 20
    assert plan(4096, 1 << 40, 4096).startswith("copy_vec_kernel<-1,1,")              # small path
    assert plan(4096, 1 << 40, 32 * MiB).startswith("copy_vec_kernel<-1,")           # vector kernel below 96 MiB
    assert plan(4096, 1 << 40, 256 * MiB).startswith("copy_tma_kernel<3,2,0>, 21846 CTAs")   # 12 KiB chunks
    assert plan(4096, 1 << 40, 1 << 30).startswith("copy_tma_kernel<3,2,0>, 87382 CTAs")     # the same shape at every size
    assert plan(4096, (1 << 40) + 1, 1 << 30).startswith("copy_vec_kernel<0,4,2>, 32768 CTAs x 512")  # realign by 1 byte
    assert plan(4096, (1 << 40) + 13, 1 << 30).startswith("copy_vec_kernel<3,4,2>")
    assert "loads before the stream wait" in plan(4096, 1 << 40, 1 << 30, 0x100)
    assert "loads before the stream wait" not in plan(4096, 1 << 40, 1 << 30, 0)
    assert lib.lcb_copy_d2d_describe(4096, (1 << 40) + 1, 1 << 20, 2, 0, buf, 200) == 1      # bulk path refused
    assert lib.lcb_copy_d2d_describe(4096, 1 << 40, 1 << 20, 0x400, 0, buf, 200) == 1        # unknown flag
    lib.lcb_tune(b"auto_tma_min_mib", -1)
    try:
        assert plan(4096, 1 << 40, 1 << 30).startswith("copy_vec_kernel<-1,4,2>, 32768 CTAs x 512")
    finally:
        lib.lcb_tune(b"reset", 0)
