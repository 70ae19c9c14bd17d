"""lcb_checksum64_noalloc -- the checksum entry point for callers that cannot allocate device memory (their
pool already owns the free HBM, or their host forbids allocating calls).  It must give exactly what
lcb_checksum64 gives with caller-provided scratch, call after call, because its built-in scratch array is
shared by every call and keeps the previous call's contents.  Runs last so that a failure here cannot hide
any other test's result."""
import ctypes as C

import numpy as np
import pytest

from librecuda_b200 import api

pytestmark = pytest.mark.gpu
MiB = 1 << 20


def _read_u64(stream, buf) -> int:
    host = np.zeros(1, np.uint64)
    stream.memcpy(host, buf, 8)
    stream.run()
    return int(host[0])


def test_noalloc_checksum_matches_scratch_version_twice_in_a_row(ctx):
    ctx.set_current()
    lib = api.lib
    stream = api.Stream()
    native = stream.native
    n = 96 * MiB + 13                       # many CTAs' worth of partial sums plus a ragged tail
    data = api.DeviceBuffer(n + 8)
    scratch = api.DeviceBuffer(lib.lcb_checksum_scratch_bytes())
    want_buf, got_buf = api.DeviceBuffer(8), api.DeviceBuffer(8)
    seen = []
    for call, (seed, nbytes) in enumerate([(21, n), (22, n - 5 * MiB - 3)]):   # two calls, back to back
        api.lcb_check(lib.lcb_fill_splitmix64(data.ptr, n, seed, native), "lcb_fill_splitmix64")
        api.lcb_check(lib.lcb_checksum64(data.ptr, nbytes, scratch.ptr, want_buf.ptr, native), "lcb_checksum64")
        api.lcb_check(lib.lcb_checksum64_noalloc(data.ptr, nbytes, got_buf.ptr, native), "lcb_checksum64_noalloc")
        want, got = _read_u64(stream, want_buf), _read_u64(stream, got_buf)
        assert got == want, f"call {call}: built-in scratch gave {got:#x}, caller scratch gave {want:#x}"
        seen.append(got)
    assert seen[0] != seen[1]               # the second answer is not a leftover of the first
    # tiny and empty inputs go through the same array
    for nbytes in (0, 3, 8, 4096):
        api.lcb_check(lib.lcb_checksum64(data.ptr, nbytes, scratch.ptr, want_buf.ptr, native), "lcb_checksum64")
        api.lcb_check(lib.lcb_checksum64_noalloc(data.ptr, nbytes, got_buf.ptr, native), "lcb_checksum64_noalloc")
        assert _read_u64(stream, got_buf) == _read_u64(stream, want_buf)
    # beyond the stated maximum: refused before anything is launched
    limit = lib.lcb_checksum64_noalloc_max_bytes()
    assert limit == 64 << 30
    assert lib.lcb_checksum64_noalloc(data.ptr, limit + 8, got_buf.ptr, native) == 1
    assert lib.lcb_checksum64_noalloc(data.ptr + 4, 64, got_buf.ptr, native) == 1   # misaligned source
    assert lib.lcb_checksum64_noalloc(None, 64, got_buf.ptr, native) == 1
    for b in (data, scratch, want_buf, got_buf):
        b.free()
    stream.destroy()
