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
