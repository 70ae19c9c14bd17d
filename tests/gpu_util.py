"""Helpers for the GPU parity tests: device arenas with guard bands and host round trips through the
libreCu* API."""
import ctypes as C

import numpy as np

from librecuda_b200 import api

GUARD = 256
GUARD_BYTE = 0xC5


def to_device(stream, dev, host: np.ndarray):
    stream.memcpy(dev, host, host.nbytes)
    stream.run()


def to_host(stream, dev, nbytes: int) -> np.ndarray:
    out = np.empty(nbytes, np.uint8)
    stream.memcpy(out, dev, nbytes)
    stream.run()
    return out


def device_compare(stream, a_ptr: int, b_ptr: int, nbytes: int, result_buf):
    """(mismatch count, first mismatch index) of two device ranges, computed on the device."""
    api.lcb_check(api.lib.lcb_compare_bytes(a_ptr, b_ptr, nbytes, result_buf.ptr, stream.native), "lcb_compare_bytes")
    api.lcb_check(api.lib.lcb_stream_synchronize(stream.native), "sync")
    r = to_host(stream, result_buf, 16).view("<u8")
    return int(r[0]), int(r[1])


def device_checksum(stream, ptr: int, nbytes: int, scratch, out) -> int:
    api.lcb_check(api.lib.lcb_checksum64(ptr, nbytes, scratch.ptr, out.ptr, stream.native), "lcb_checksum64")
    api.lcb_check(api.lib.lcb_stream_synchronize(stream.native), "sync")
    return int(to_host(stream, out, 8).view("<u8")[0])


WINDOW = 16 << 20


def host_window_mismatches(stream, dev_ptr: int, nbytes: int, expect, salt: int = 0, extra_offsets=()):
    """Copies the first, the last and three seeded-random 16 MiB windows of a device range (plus windows starting at
    `extra_offsets`) to the host and compares each with `expect(offset, n)`, the bytes the HOST oracle puts
    there.  Returns the offsets of the windows that differ.  This is the check that does not rest on any of the
    library's own kernels: equality after a device-to-host copy, as in the reference's
    tests/dma_chronological_consistency/main.cpp:73-85."""
    win = min(WINDOW, nbytes)
    offs = {0, nbytes - win}
    rng = np.random.default_rng(1234 + salt)
    while len(offs) < 5 and nbytes - win >= 40:
        offs.add(int(rng.integers(0, (nbytes - win) // 8 + 1)) * 8)
    offs.update(o for o in extra_offsets if 0 <= o <= nbytes - win)
    bad = []
    host = np.empty(win, np.uint8)
    for off in sorted(offs):
        stream.memcpy(host, dev_ptr + off, win)
        stream.run()
        if not np.array_equal(host, expect(off, win)):
            bad.append(off)
    return bad


def seeded_stream_expect(seed: int, first_byte: int = 0):
    """expect() for a device range that holds the oracle's seeded stream from byte `first_byte` on (any value: the
    oracle generates 8-byte aligned windows, a slice of a slightly larger one is returned)."""
    import oracle

    def expect(off, n):
        lo = (first_byte + off) // 8 * 8
        skip = first_byte + off - lo
        return oracle.random_window(lo, n + 16, seed)[skip:skip + n]

    return expect
