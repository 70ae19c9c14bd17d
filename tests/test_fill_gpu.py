"""Parity of memset (D8/D16/D32), index fill and the y = a*x + b kernel with the oracle's host loops."""
import numpy as np
import pytest

import oracle
from librecuda_b200 import api
from gpu_util import GUARD, GUARD_BYTE, device_checksum, to_device, to_host

pytestmark = pytest.mark.gpu
MiB = 1 << 20


def _memset_cases(stream, cases, path):
    """cases: (elem_bytes, value, count, byte_offset)"""
    slot = lambda nb: (nb + 2 * GUARD + 64 + 255) // 256 * 256
    total = sum(slot(e * c) for e, _, c, _ in cases)
    base = np.full(total, GUARD_BYTE, np.uint8)
    dev = api.DeviceBuffer(total)
    to_device(stream, dev, base)
    want = base.copy()
    pos = 0
    for e, v, c, off in cases:
        at = pos + GUARD + off
        api.lcb_check(api.lib.lcb_memset_ex(dev.ptr + at, v, e, c, path, 0, stream.native), "lcb_memset_ex")
        oracle.memset(want[at:at + e * c], v & ((1 << (8 * e)) - 1), e)
        pos += slot(e * c)
    got = to_host(stream, dev, total)
    dev.free()
    bad = np.flatnonzero(got != want)
    assert bad.size == 0, f"first mismatch at arena byte {int(bad[0])}, {bad.size} differ"


COUNTS = sorted(set(range(0, 70)) | {127, 128, 129, 1023, 1024, 1025, 4095, 4096, 4097, 65537})


@pytest.mark.parametrize("path", [0, 1, 2])
def test_memset_small_all_alignments(stream, path):
    cases = [(1, 0xA7, c, o) for c in COUNTS for o in range(0, 17)]
    cases += [(2, 0xBEEF, c, o) for c in COUNTS for o in range(0, 18, 2)]
    cases += [(4, 0x40490FDB, c, o) for c in COUNTS for o in range(0, 20, 4)]
    _memset_cases(stream, cases, path)


@pytest.mark.parametrize("path", [0, 1, 2])
def test_memset_mid_and_large(stream, path):
    cases = [(1, 0x5A, MiB + 131, 1), (1, 0, 9 * MiB + 3, 15), (2, 0x1234, 3 * MiB + 1, 6), (4, 0xDEADBEEF, 5 * MiB + 3, 4),
             (4, 0x40490FDB, 16 * MiB, 0), (1, 0xFF, 40 * MiB + 17, 3)]
    _memset_cases(stream, cases, path)


@pytest.mark.parametrize("knobs", [dict(memset_chunk=65536, memset_issuers=2, memset_bulk_ctas_sm=3),
                                   dict(memset_chunk=8192, memset_issuers=8, memset_bulk_ctas_sm=1, memset_cache_hint=1),
                                   dict(memset_chunk=16384, memset_issuers=1, memset_bulk_ctas_sm=4),
                                   dict(memset_threads=512, memset_unroll=2, memset_ctas_sm=1)])
def test_memset_configurations(stream, knobs):
    try:
        api.tune(**knobs)
        for path in (1, 2):
            _memset_cases(stream, [(1, 0x3C, 7 * MiB + 5, 3), (4, 0xCAFEF00D, 2 * MiB + 1, 8), (2, 0xA55A, 70001, 2)], path)
    finally:
        api.tune_reset()


def test_memset_rejects_misaligned_elements(stream):
    d = api.DeviceBuffer(4096)
    assert api.lib.lcb_memset_d32(d.ptr + 2, 1, 4, stream.native) == 1
    assert api.lib.lcb_memset_d16(d.ptr + 1, 1, 4, stream.native) == 1
    d.free()


def test_config_fill_1gib_d32_then_index_fill(stream):
    # 256 Mi float32: memset D32 to the bit pattern of pi, then out[i] = float(i); both against host loops
    n = 1 << 28
    dev = api.DeviceBuffer(4 * n)
    scratch, out = api.DeviceBuffer(api.lib.lcb_checksum_scratch_bytes()), api.DeviceBuffer(8)
    stream.memset_d32(dev, 0x40490FDB, n)
    stream.run()
    want = np.empty(n, np.uint32)
    oracle.memset(want, 0x40490FDB, 4)
    assert device_checksum(stream, dev.ptr, 4 * n, scratch, out) == oracle.checksum64(want)
    got = to_host(stream, dev, 4 * n).view(np.uint32)
    assert np.array_equal(got, want)
    del got
    api.lcb_check(api.lib.lcb_index_fill_f32(dev.ptr, n, stream.native), "lcb_index_fill_f32")
    wantf = oracle.index_fill_f32(n)
    assert device_checksum(stream, dev.ptr, 4 * n, scratch, out) == oracle.checksum64(wantf)
    gotf = to_host(stream, dev, 4 * n).view(np.uint32)
    assert np.array_equal(gotf, wantf.view(np.uint32))
    for b in (dev, scratch, out):
        b.free()


@pytest.mark.parametrize("n,off", [(0, 0), (1, 0), (3, 1), (4, 2), (5, 3), (1000, 1), (MiB + 3, 0), (MiB + 2, 3), ((1 << 24) + 77, 1)])
def test_index_fill_edges(stream, n, off):
    dev = api.DeviceBuffer(4 * (n + 8) + 64)
    to_device(stream, dev, np.full(4 * (n + 8) + 64, GUARD_BYTE, np.uint8))
    api.lcb_check(api.lib.lcb_index_fill_f32(dev.ptr + 4 * off, n, stream.native), "lcb_index_fill_f32")
    got = to_host(stream, dev, 4 * (n + 8) + 64)
    want = np.full(4 * (n + 8) + 64, GUARD_BYTE, np.uint8)
    want[4 * off:4 * (off + n)] = oracle.index_fill_f32(n).view(np.uint8)
    assert np.array_equal(got, want)
    dev.free()


@pytest.mark.parametrize("n,xo,yo", [(1, 0, 0), (7, 0, 0), (4099, 0, 0), (4099, 1, 0), (4099, 0, 3), (MiB * 4 + 5, 0, 0), (MiB + 1, 2, 1)])
def test_axpb_matches_host_two_rounding_loop(stream, n, xo, yo):
    x_h = oracle.random_f32(n, seed=2)
    x, y = api.DeviceBuffer(4 * (n + 4)), api.DeviceBuffer(4 * (n + 4))
    to_device(stream, x.view(4 * xo), x_h.view(np.uint8))
    api.lcb_check(api.lib.lcb_axpb_f32(y.ptr + 4 * yo, x.ptr + 4 * xo, 2.0, 1.0, n, stream.native), "lcb_axpb_f32")
    got = to_host(stream, y.view(4 * yo), 4 * n).view(np.uint32)
    assert np.array_equal(got, oracle.axpb_f32(x_h, 2.0, 1.0).view(np.uint32))
    x.free()
    y.free()
