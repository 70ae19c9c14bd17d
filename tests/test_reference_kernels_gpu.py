"""The reference's own copy kernels (driverapi/kernels/memcpy/memcpy.cu, compiled for sm_100a from the
reference checkout by oracle/build_ref.sh) run on the B200 with the launch plan of the reference's dispatcher
(driverapi/src/memcopy.cpp:77-158, restated and pinned in the oracle), through this library's module loader
and libreCuLaunchKernel.  Their output must be byte-identical to this library's copy of the same buffers.
Skipped when the image was not built (no reference checkout at build time)."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

import oracle
from librecuda_b200 import api
from gpu_util import to_device, to_host

pytestmark = pytest.mark.gpu
MiB = 1 << 20
CUBIN = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "ref_memcpy_sm100a.cubin"
NAMES = {1: "memcpyKernelHighBW", 2: "memcpyKernelLowLatency", 3: "memcpyKernelTrailing"}


@pytest.fixture(scope="module")
def ref_module(ctx):
    if not CUBIN.exists():
        pytest.skip("oracle/_ref/ref_memcpy_sm100a.cubin not built")
    ctx.set_current()
    m = api.Module(CUBIN.read_bytes())
    assert sorted(m.function_names()) == sorted(NAMES.values())
    yield m
    m.unload()


def _reference_copy(stream, module, dst, src, size):
    """What the reference's memcpyD2D enqueues: first kernel ordered, the others may overlap it."""
    for i, (kernel, gx, gy, off, n) in enumerate(oracle.ref_d2d_plan(size)):
        if gx == 0:
            continue  # the reference issues a zero-block launch here (a defect); nothing would run
        params = [C.c_void_p(dst + off), C.c_void_p(src + off)]
        if kernel != 1:
            params.append(C.c_size_t(n))
        stream.launch(module.function(NAMES[kernel]), (gx, gy, 1), (256, 1, 1), 0, params, async_=(i > 0))


@pytest.mark.parametrize("size", [4, 40, 4096, 65536, MiB, MiB + 4, MiB + 131, 2 * MiB + 5, 16 * MiB + 4100, 128 * MiB])
def test_reference_kernels_and_this_library_agree_on_the_gpu(stream, ref_module, size):
    src_h = oracle.random_bytes(size, seed=1)
    src = api.DeviceBuffer(size + 64)
    d_ref, d_own = api.DeviceBuffer(size + 64), api.DeviceBuffer(size + 64)
    res = api.DeviceBuffer(16)
    to_device(stream, src, src_h)
    stream.memset_d8(d_ref, 0xEE, size + 64)
    stream.memset_d8(d_own, 0xEE, size + 64)
    _reference_copy(stream, ref_module, d_ref.ptr, src.ptr, size)
    stream.memcpy(d_own, src, size)
    stream.run()
    api.lcb_check(api.lib.lcb_compare_bytes(d_ref.ptr, d_own.ptr, size + 64, res.ptr, stream.native), "cmp")
    api.lcb_check(api.lib.lcb_stream_synchronize(stream.native), "sync")
    r = to_host(stream, res, 16).view("<u8")
    assert int(r[0]) == 0, f"{int(r[0])} bytes differ, first at {int(r[1])}"
    got = to_host(stream, d_ref, min(size, 4 * MiB))
    assert np.array_equal(got, src_h[:got.size])
    for b in (src, d_ref, d_own, res):
        b.free()
