"""Parity of the device-to-device copy kernels (called through the C-ABI) with the oracle: bit-exact
against host memcpy on the same seeded bytes, guard bands intact, for every path, alignment class and size
class, plus the golden vectors generated from the reference."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

import oracle
from librecuda_b200 import api
from gpu_util import (GUARD, GUARD_BYTE, device_checksum, device_compare, host_window_mismatches, seeded_stream_expect,
                      to_device, to_host)

pytestmark = pytest.mark.gpu
MiB = 1 << 20
AUTO, VEC, TMA, SMALL, VEC32, TMA2, PHASED = 0, 1, 2, 3, 4, 5, 6
SRC_STABLE, NO_PDL = 0x100, 0x200   # flags OR'ed into the path argument
GOLDEN = json.loads((Path(__file__).parent / "golden" / "ref_d2d_golden.json").read_text())


def _copy(stream, dst, src, n, path=AUTO, ctas=0):
    api.lcb_check(api.lib.lcb_copy_d2d_ex(dst, src, n, path, ctas, stream.native), "lcb_copy_d2d_ex")


def _run_cases(stream, cases, path):
    """cases: list of (size, src_off, dst_off).  All copies go into one arena, one read-back, host check."""
    slot = lambda n: (n + 2 * GUARD + 64 + 255) // 256 * 256
    total = sum(slot(n) for n, _, _ in cases)
    src_h = oracle.random_bytes(total, seed=1)
    dst_h = np.full(total, GUARD_BYTE, np.uint8)
    src_d, dst_d = api.DeviceBuffer(total), api.DeviceBuffer(total)
    to_device(stream, src_d, src_h)
    to_device(stream, dst_d, dst_h)
    pos = 0
    placed = []
    for n, so, do in cases:
        s, d = pos + GUARD + so, pos + GUARD + do
        _copy(stream, dst_d.ptr + d, src_d.ptr + s, n, path)
        placed.append((n, s, d))
        pos += slot(n)
    got = to_host(stream, dst_d, total)
    want = dst_h.copy()
    for n, s, d in placed:
        oracle.lib.orc_memcpy(want[d:].ctypes.data, src_h[s:].ctypes.data, n)
    bad = np.flatnonzero(got != want)
    src_d.free()
    dst_d.free()
    if bad.size:
        i = int(bad[0])
        which = [(n, s, d) for n, s, d in placed if d - GUARD <= i < d + n + GUARD]
        raise AssertionError(f"first mismatch at arena byte {i} (case size/src/dst {which}), {bad.size} bytes differ")
    assert api.device_error_word() == 0


SMALL_SIZES = sorted(set(range(0, 100)) | {127, 128, 129, 255, 256, 257, 511, 512, 513, 1023, 1024, 1025, 4095, 4096,
                                           4097, 8191, 16384 + 5, 65535, 65536, 65537})
OFFSETS = [0, 1, 2, 3, 4, 5, 7, 8, 9, 12, 13, 15, 16, 17, 31, 64]


@pytest.mark.parametrize("path", [AUTO, VEC, SMALL])
def test_small_sizes_all_alignment_classes(stream, path):
    # every (src mod 16, dst mod 16) relation incl. all 15 realign shifts, every head/tail length
    cases = [(n, so, do) for n in SMALL_SIZES for so in OFFSETS for do in (0, 1, 3, 7, 8, 15)]
    _run_cases(stream, cases, path)


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_sizes_and_offsets(stream, seed):
    rng = np.random.default_rng(seed)
    cases = []
    for _ in range(400):
        n = int(2 ** rng.uniform(0, 23))           # 1 byte .. 8 MiB, log-uniform
        cases.append((n + int(rng.integers(0, 17)), int(rng.integers(0, 64)), int(rng.integers(0, 64))))
    _run_cases(stream, cases, AUTO)


def test_all_sixteen_by_sixteen_phase_pairs(stream):
    cases = [(1000 + 3 * so + do, so, do) for so in range(16) for do in range(16)]
    _run_cases(stream, cases, VEC)
    _run_cases(stream, [(70000 + so, so, do) for so in range(16) for do in range(16)], AUTO)


@pytest.mark.parametrize("path", [AUTO, VEC, TMA, TMA2, PHASED])
def test_mid_and_large_sizes(stream, path):
    sizes = [MiB - 1, MiB, MiB + 131, 2 * MiB + 5, 3 * MiB + 4099, 16 * MiB + 4100, 64 * MiB + 17]
    offs = [(0, 0), (64, 64), (16, 48)] if path in (TMA, TMA2, PHASED) else [(0, 0), (1, 0), (0, 3), (7, 7), (64, 1), (3, 64), (5, 9)]
    _run_cases(stream, [(n, so, do) for n in sizes for so, do in offs], path)


@pytest.mark.parametrize("path", [AUTO | SRC_STABLE, VEC | SRC_STABLE, SMALL | SRC_STABLE, AUTO | NO_PDL, AUTO | SRC_STABLE | NO_PDL])
def test_launch_flags_do_not_change_the_result(stream, path):
    # SRC_STABLE lets the loads run ahead of the wait for the previous kernel on the stream; the copies of one
    # arena are launched back to back, so every launch overlaps the tail of the one before it
    sizes = [1, 15, 16, 17, 4097, 65535, 65536, MiB + 131, 3 * MiB + 4099, 16 * MiB + 4100]
    offs = [(0, 0), (1, 0), (0, 3), (7, 7), (64, 1), (5, 9)]
    _run_cases(stream, [(n, so, do) for n in sizes for so, do in offs], path)


def test_loads_ahead_of_the_wait_on_the_bulk_path(stream):
    cases = [(n, o, o + 16 * k) for n in (1, 17, 16385, 3 * 16384 + 7, 200001, 7 * MiB + 33, 130 * MiB + 5)
             for o in (0, 5) for k in (0, 2)]
    _run_cases(stream, cases, TMA | SRC_STABLE)
    api.tune(tma_ctas_sm=1, tma_chunk=8192, tma_stages=8, tma_lookahead=6)   # persistent ring
    try:
        _run_cases(stream, cases, TMA | SRC_STABLE)
    finally:
        api.tune_reset()


def test_copy_plan_query_names_what_is_launched(stream):
    import ctypes as C
    buf = C.create_string_buffer(200)
    a, b = api.DeviceBuffer(300 * MiB), api.DeviceBuffer(300 * MiB)
    for n, off, want in ((4096, 0, "copy_vec_kernel<-1,1,2>"), (200 * MiB, 0, "copy_tma_kernel<3,2,0>"),
                         (200 * MiB, 3, "copy_vec_kernel<0,4,2>"), (64 * MiB, 0, "copy_vec_kernel<-1,4,2>")):
        assert api.lib.lcb_copy_d2d_describe(b.ptr, a.ptr + off, n, AUTO, 0, buf, 200) == 0
        assert buf.value.decode().startswith(want), buf.value
    a.free()
    b.free()


@pytest.mark.parametrize("knobs", [dict(phase_chunk=32768, phase_stages=6, phase_ns=4000), dict(phase_chunk=8192, phase_stages=24, phase_ns=0),
                                   dict(phase_chunk=65536, phase_stages=3, phase_ns=1000), dict(phase_chunk=4096, phase_stages=2, phase_ns=2000)])
def test_phase_grouped_copy_configurations(stream, knobs):
    api.tune(**knobs)
    try:
        cases = [(n, o, o + 16 * k) for n in (0, 1, 17, 16385, 200001, 5 * MiB + 33, 40 * MiB + 5) for o in (0, 5) for k in (0, 2)]
        _run_cases(stream, cases, PHASED)
    finally:
        api.tune_reset()


@pytest.mark.parametrize("path", [TMA, TMA2, PHASED])
def test_bulk_path_edges_and_small_bodies(stream, path):
    # congruent but not 16-byte aligned pointers: head and tail bytes ride along with the bulk ring
    cases = [(n, o, o + 16 * k) for n in (0, 1, 15, 16, 17, 31, 33, 1000, 16384, 16385, 3 * 16384 + 7, 200001)
             for o in (0, 1, 5, 15) for k in (0, 2)]
    _run_cases(stream, cases, path)


@pytest.mark.parametrize("knobs", [dict(tma2_stages=4, tma2_depth=1, tma2_chunk=4096), dict(tma2_stages=8, tma2_depth=4, tma2_chunk=16384),
                                   dict(tma2_stages=16, tma2_depth=8, tma2_chunk=8192, tma_cache_hint=1),
                                   dict(tma2_stages=24, tma2_depth=4, tma2_chunk=8192)])
def test_two_issuer_ring_configurations(stream, knobs):
    try:
        api.tune(**knobs)
        _run_cases(stream, [(n, o, o) for n in (5 * MiB + 48, 333333, 65536 * 7, 40 * MiB + 16) for o in (0, 16)], TMA2)
    finally:
        api.tune_reset()


def test_bulk_path_rejects_mutually_misaligned(stream):
    a = api.DeviceBuffer(4096)
    assert api.lib.lcb_copy_d2d_ex(a.ptr + 1, a.ptr + 2048, 64, TMA, 0, stream.native) == 1
    assert api.lib.lcb_copy_d2d_ex(a.ptr + 16, a.ptr + 2048, 64, VEC32, 0, stream.native) == 1
    a.free()


def test_32_byte_vector_path(stream):
    cases = [(n, o, o + 32 * k) for n in (0, 1, 31, 32, 33, 63, 65, 1000, 4096, 65536 + 9, 5 * MiB + 77, 33 * MiB)
             for o in (0, 1, 16, 31) for k in (0, 3)]
    _run_cases(stream, cases, VEC32)


@pytest.mark.parametrize("knobs", [dict(tma_stages=8, tma_lookahead=6, tma_chunk=8192, tma_ctas_sm=1), dict(tma_stages=4, tma_lookahead=2, tma_chunk=8192),
                                   dict(tma_stages=8, tma_lookahead=6, tma_chunk=16384, tma_cache_hint=1),
                                   dict(tma_stages=16, tma_lookahead=12, tma_chunk=8192, tma_ctas_sm=1),
                                   dict(tma_stages=3, tma_lookahead=2, tma_chunk=65536),
                                   dict(tma_stages=6, tma_lookahead=3, tma_chunk=32768, tma_ctas_sm=1),
                                   dict(tma_stages=12, tma_lookahead=8, tma_chunk=4096)])
def test_bulk_ring_configurations(stream, knobs):
    try:
        api.tune(**knobs)
        _run_cases(stream, [(n, o, o) for n in (5 * MiB + 48, 333333, 65536 * 7) for o in (0, 16)], TMA)
    finally:
        api.tune_reset()


@pytest.mark.parametrize("knobs", [dict(copy_vec_threads=512, copy_vec_unroll=1), dict(copy_vec_threads=256, copy_vec_unroll=2),
                                   dict(copy_vec_threads=512, copy_vec_unroll=8), dict(copy_vec_threads=256, copy_vec_unroll=4, copy_cache_mode=1),
                                   dict(copy_cache_mode=0), dict(copy_vec_threads=512, copy_vec_unroll=4, copy_vec_ctas_sm=1),
                                   dict(copy_vec_threads=128, copy_vec_unroll=8, copy_vec_ctas_sm=2)])
def test_vector_kernel_configurations(stream, knobs):
    try:
        api.tune(**knobs)
        _run_cases(stream, [(n, so, do) for n in (9 * MiB + 77, 123457) for so, do in [(0, 0), (3, 0), (0, 9), (64, 6)]], VEC)
    finally:
        api.tune_reset()


def test_tiny_grids_cover_everything(stream):
    # one CTA (and an odd CTA count) must still walk the whole buffer
    n = 5 * MiB + 999
    src_h = oracle.random_bytes(n, seed=7)
    s, d = api.DeviceBuffer(n + 64), api.DeviceBuffer(n + 64)
    to_device(stream, s, src_h)
    for path, ctas, so, do in [(VEC, 1, 0, 0), (VEC, 3, 1, 0), (TMA, 1, 16, 32), (TMA, 5, 0, 0), (TMA2, 1, 0, 16), (TMA2, 7, 0, 0)]:
        to_device(stream, d, np.zeros(n + 64, np.uint8))
        _copy(stream, d.ptr + do, s.ptr + so, n - 64, path, ctas)
        got = to_host(stream, d, n + 64)
        assert np.array_equal(got[do:do + n - 64], src_h[so:so + n - 64])
        assert not got[:do].any() and not got[do + n - 64:].any()
    s.free()
    d.free()


@pytest.mark.parametrize("case", [c for c in GOLDEN["cases"] if "dst_sha256" in c], ids=lambda c: str(c["size"]))
def test_reference_golden_vectors(stream, case):
    # same seeded source the reference copied on the host when the golden file was made
    n = case["size"]
    src_h = oracle.random_bytes(n, seed=GOLDEN["seed"])
    s, d = api.DeviceBuffer(n + 16), api.DeviceBuffer(n + 16)
    to_device(stream, s, src_h)
    to_device(stream, d, np.zeros(n + 16, np.uint8))
    _copy(stream, d.ptr, s.ptr, n)
    got = to_host(stream, d, n + 16)
    assert hashlib.sha256(got[:n].tobytes()).hexdigest() == case["dst_sha256"]
    assert not got[n:].any()
    s.free()
    d.free()


def test_bounded_wait_gives_up_with_an_error_status_and_the_device_stays_usable(stream):
    # failure detection without a fault: a wait that can never be satisfied runs out of tries, the kernel
    # reports it through the sticky error word and returns
    assert api.device_error_word() == 0
    assert api.lib.lcb_selftest_wait_timeout(0, stream.native) == 1          # limits are enforced on the host
    assert api.lib.lcb_selftest_wait_timeout(10**7, stream.native) == 1
    api.lcb_check(api.lib.lcb_selftest_wait_timeout(2000, stream.native), "selftest")
    assert api.device_error_word() == 1      # reported ...
    assert api.device_error_word() == 0      # ... and cleared by the read
    _run_cases(stream, [(3 * MiB + 5, 0, 0), (MiB, 1, 2)], AUTO)   # copies still work afterwards
    _run_cases(stream, [(5 * MiB + 48, 16, 16)], TMA)


def test_flag_wait_is_bounded_and_flag_post_releases_it(stream):
    # the wait that keeps copy-engine schedules of different GPUs in step: satisfied by a post, and -- when nobody
    # posts -- over after its time limit with bit 1 of the error word, the device fully usable afterwards
    import time
    flag = api.DeviceBuffer(4096)
    stream.memset_d8(flag, 0, 4096)
    stream.run()
    lib = api.lib
    assert lib.lcb_flag_wait(flag.ptr, 1, 0, stream.native) == 1            # a limit is mandatory ...
    assert lib.lcb_flag_wait(flag.ptr, 1, 60000, stream.native) == 1        # ... and at most ten seconds
    assert lib.lcb_flag_wait(flag.ptr + 2, 1, 100, stream.native) == 1      # misaligned word
    api.lcb_check(lib.lcb_flag_post(flag.ptr + 8, 7, stream.native), "post")
    api.lcb_check(lib.lcb_flag_wait(flag.ptr + 8, 7, 1000, stream.native), "wait")   # already there
    api.lcb_check(lib.lcb_flag_wait(flag.ptr + 8, 5, 1000, stream.native), "wait")   # counters only grow
    api.lcb_check(lib.lcb_stream_synchronize(stream.native), "sync")
    assert api.device_error_word() == 0
    t0 = time.perf_counter()
    api.lcb_check(lib.lcb_flag_wait(flag.ptr + 8, 8, 150, stream.native), "wait")    # nobody posts 8
    api.lcb_check(lib.lcb_stream_synchronize(stream.native), "sync")
    assert 0.1 < time.perf_counter() - t0 < 1.0
    assert api.device_error_word() == 2      # reported ...
    assert api.device_error_word() == 0      # ... and cleared
    _run_cases(stream, [(3 * MiB + 5, 0, 0)], AUTO)   # copies still work afterwards
    flag.free()


def test_device_helpers_agree_with_oracle(stream):
    n = 3 * MiB + 5
    buf, res = api.DeviceBuffer(n + 8), api.DeviceBuffer(16)
    scratch, out = api.DeviceBuffer(api.lib.lcb_checksum_scratch_bytes()), api.DeviceBuffer(8)
    api.lcb_check(api.lib.lcb_fill_splitmix64(buf.ptr, n, 11, stream.native), "fill")
    got = to_host(stream, buf, n)
    want = oracle.random_bytes(n, seed=11)
    assert np.array_equal(got, want)
    for m in (n, n - 5, 8, 3, 4096):
        assert device_checksum(stream, buf.ptr, m, scratch, out) == oracle.checksum64(want[:m])
        assert device_checksum(stream, buf.ptr, m, scratch, out) == oracle.checksum64(want[:m])  # scratch is reusable
    # the kernel reads 16-byte pairs: a source 8 but not 16 bytes aligned, odd and even word counts, no pair at all
    for off in (8, 24):
        for m in (0, 1, 8, 15, 16, 17, 24, 4096 + 8, 3 * MiB - 24, 3 * MiB - 19):
            assert device_checksum(stream, buf.ptr + off, m, scratch, out) == oracle.checksum64(want[off:off + m]), (off, m)
    other = api.DeviceBuffer(n + 8)
    to_device(stream, other, want)
    assert device_compare(stream, buf.ptr, other.ptr, n, res) == (0, 2**64 - 1)
    planted = want.copy()
    planted[[100, 4097, n - 1]] ^= 0x40
    to_device(stream, other, planted)
    assert device_compare(stream, buf.ptr, other.ptr, n, res) == (3, 100)
    assert device_compare(stream, buf.ptr + 3, other.ptr + 3, n - 3, res) == (3, 97)   # misaligned operands
    for b in (buf, res, scratch, out, other):
        b.free()


SWEEP_OFFSETS = [0, 1, 3, 7, 64]


def _sweep(stream, sizes, pairs, host_pairs=()):
    """DtoD sweep with everything verified on the device: seeded source (seed 1), compare against the
    source range, guard bands either side of the destination, and checksum(src) == checksum(dst).  For the
    offset pairs in `host_pairs` the destination is ALSO checked on the host: windows of it (first, last, three
    random ones and, past 4 GiB, one that straddles the 4 GiB offset) are copied back and compared with the
    oracle's own regeneration of the seeded stream, so no kernel of this library judges that part."""
    top = max(sizes)
    src = api.DeviceBuffer(top + 128)
    dst = api.DeviceBuffer(top + 128 + 2 * GUARD)
    res, out = api.DeviceBuffer(16), api.DeviceBuffer(8)
    scratch = api.DeviceBuffer(api.lib.lcb_checksum_scratch_bytes())
    guard = api.DeviceBuffer(GUARD)
    stream.memset_d8(guard, GUARD_BYTE, GUARD)
    stream.run()
    api.lcb_check(api.lib.lcb_fill_splitmix64(src.ptr, top + 128, 1, stream.native), "fill")
    # the generator itself, against the host oracle, over the whole source (windows incl. the 4 GiB boundary)
    assert host_window_mismatches(stream, src.ptr, top + 128, seeded_stream_expect(1), salt=1, extra_offsets=STRADDLE) == []
    for n in sizes:
        for so, do in pairs:
            d = dst.ptr + GUARD + do
            stream.memset_d8(dst.view(do, n + 2 * GUARD), GUARD_BYTE, n + 2 * GUARD)
            stream.run()
            api.lcb_check(api.lib.lcb_copy_d2d(d, src.ptr + so, n, stream.native), "lcb_copy_d2d")
            assert device_compare(stream, d, src.ptr + so, n, res)[0] == 0, (n, so, do)
            assert device_compare(stream, d - GUARD, guard.ptr, GUARD, res)[0] == 0, ("front guard", n, so, do)
            assert device_compare(stream, d + n, guard.ptr, GUARD, res)[0] == 0, ("back guard", n, so, do)
            if (so, do) in host_pairs and n >= (1 << 20):
                bad = host_window_mismatches(stream, d, n, seeded_stream_expect(1, so), salt=n % 977 + so,
                                             extra_offsets=[o - so for o in STRADDLE])
                assert bad == [], (n, so, do, bad)
        # 8-byte aligned pair for the checksum property
        api.lcb_check(api.lib.lcb_copy_d2d(dst.ptr + GUARD, src.ptr + 64, n, stream.native), "lcb_copy_d2d")
        assert device_checksum(stream, dst.ptr + GUARD, n, scratch, out) == device_checksum(stream, src.ptr + 64, n, scratch, out)
    assert api.device_error_word() == 0
    for b in (src, dst, res, out, scratch, guard):
        b.free()


# windows that start 8 MiB before a 4 GiB multiple of the source stream: 32-bit index slips show up there
STRADDLE = [(4 << 30) - (8 << 20), (8 << 30) - (16 << 20)]


def test_dtod_sweep_powers_of_two_all_offset_pairs(stream):
    # 4 KiB ... 1 GiB, src/dst offsets {0,1,3,7,64}^2
    _sweep(stream, [1 << k for k in range(12, 31)], [(a, b) for a in SWEEP_OFFSETS for b in SWEEP_OFFSETS],
           host_pairs=[(0, 0), (1, 3), (64, 7)])


def test_dtod_sweep_largest_sizes(stream):
    # 2, 4 and 8 GiB: 64-bit offsets everywhere (the reference over-launches from 256 MiB on)
    pairs = [(a, b) for a in SWEEP_OFFSETS for b in SWEEP_OFFSETS]
    _sweep(stream, [1 << 31, 1 << 32, 1 << 33], pairs, host_pairs=pairs)


def test_host_window_check_catches_one_wrong_byte_past_4_gib(stream):
    # the negative of the check above: an 8 GiB copy is right, but the HOST side of the comparison is given one
    # flipped byte at stream position 4 GiB + 12345; the window that straddles 4 GiB must report it, and only it
    n = 1 << 33
    src, dst = api.DeviceBuffer(n), api.DeviceBuffer(n)
    api.lcb_check(api.lib.lcb_fill_splitmix64(src.ptr, n, 1, stream.native), "fill")
    api.lcb_check(api.lib.lcb_copy_d2d(dst.ptr, src.ptr, n, stream.native), "lcb_copy_d2d")
    truth = seeded_stream_expect(1)
    planted_at = (4 << 30) + 12345

    def planted(off, m):
        w = truth(off, m).copy()
        if off <= planted_at < off + m:
            w[planted_at - off] ^= 0x01
        return w

    def only_windows_over_the_plant(bad):
        return STRADDLE[0] in bad and all(w <= planted_at < w + (16 << 20) for w in bad)

    assert host_window_mismatches(stream, dst.ptr, n, truth, salt=3, extra_offsets=STRADDLE) == []
    assert only_windows_over_the_plant(host_window_mismatches(stream, dst.ptr, n, planted, salt=3, extra_offsets=STRADDLE))
    # and a wrong byte on the DEVICE side at the same place is caught the same way
    flip = np.array([0], np.uint8)
    stream.memcpy(flip, dst.ptr + planted_at, 1)
    stream.run()
    flip ^= 0x80
    stream.memcpy(dst.ptr + planted_at, flip, 1)
    stream.run()
    assert only_windows_over_the_plant(host_window_mismatches(stream, dst.ptr, n, truth, salt=3, extra_offsets=STRADDLE))
    src.free()
    dst.free()
