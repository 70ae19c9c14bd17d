"""Pins the CPU oracle: known-answer vectors, the golden file generated from the reference itself
(tests/golden/ref_d2d_golden.json), the reference's own test vectors, and -- where oracle/_ref was built --
the reference's dispatcher + kernels running live on the host."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

import oracle

GOLDEN = json.loads((Path(__file__).parent / "golden" / "ref_d2d_golden.json").read_text())
MiB = 1 << 20


def test_splitmix64_known_answers():
    # published splitmix64 outputs for state 0 (first four draws)
    want = [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F, 0xF88BB8A8724C81EC]
    got = oracle.random_bytes(32, seed=0).view("<u8")
    assert [int(x) for x in got] == want


def test_random_bytes_prefix_property_and_ragged_tail():
    a = oracle.random_bytes(1000, seed=1)
    for n in (0, 1, 7, 8, 9, 63, 999):
        assert np.array_equal(oracle.random_bytes(n, seed=1), a[:n])
    assert not np.array_equal(oracle.random_bytes(64, seed=2), a[:64])


def test_random_f32_range_and_exactness():
    x = oracle.random_f32(1 << 16, seed=2)
    assert x.dtype == np.float32 and (x >= 0).all() and (x < 1).all()
    w = oracle.random_bytes(8 << 16, seed=2).view("<u8")
    assert np.array_equal(x, ((w >> np.uint64(40)).astype(np.float32) / np.float32(1 << 24)))


@pytest.mark.parametrize("case", GOLDEN["cases"], ids=lambda c: str(c["size"]))
def test_plan_matches_reference_golden(case):
    plan = oracle.ref_d2d_plan(case["size"])
    assert [list(p) for p in plan] == [l[:5] for l in case["launches"]]


@pytest.mark.parametrize("case", [c for c in GOLDEN["cases"] if "dst_sha256" in c], ids=lambda c: str(c["size"]))
def test_emulated_kernels_match_reference_golden_bytes(case):
    size = case["size"]
    src = oracle.random_bytes(size, seed=GOLDEN["seed"])
    dst = np.zeros(size + 16, np.uint8)
    oob = oracle.ref_d2d_run(dst, src, size)
    assert oob == 0
    assert hashlib.sha256(dst[:size].tobytes()).hexdigest() == case["dst_sha256"]
    assert (dst[size:] == 0).all() and case["guard_clean"]
    # and that is what a plain memcpy gives: the reference's acceptance criterion
    assert np.array_equal(dst[:size], src)


def test_reference_overlaunch_defect_is_reported_not_replicated():
    # >= 256 MiB the reference's HighBW grid is (size/4096, ceil(size/4096/65535)): gridY x too many blocks
    plan = oracle.ref_d2d_plan(256 * MiB)
    assert plan == [(1, 65536, 2, 0, 0)]
    n = 65536 * 4096
    src = np.zeros(n, np.uint8)
    dst = np.zeros(n, np.uint8)
    assert oracle.ref_d2d_run(dst, src, n) == n  # one extra copy's worth of bytes would land out of bounds


@pytest.mark.skipif(oracle.ref is None, reason="oracle/_ref not built (no reference checkout)")
@pytest.mark.parametrize("size", [1, 3, 4, 4095, 4096, MiB, MiB + 131, 2 * MiB + 5, 3 * MiB + 4099])
def test_oracle_equals_live_reference(size):
    src = oracle.random_bytes(size, seed=5)
    d_ref = np.zeros(size + 32, np.uint8)
    d_orc = np.zeros(size + 32, np.uint8)
    log = oracle.reference_d2d(d_ref, src, size, execute=True)
    oracle.ref_d2d_run(d_orc, src, size)
    assert [l[:5] for l in log] == oracle.ref_d2d_plan(size)
    assert np.array_equal(d_ref, d_orc)
    assert np.array_equal(d_ref[:size], src) and (d_ref[size:] == 0).all()


@pytest.mark.skipif(oracle.ref is None, reason="oracle/_ref not built (no reference checkout)")
def test_reference_sync_flags():
    # logically synchronous copy: only the first kernel carries async=false, the rest may overlap it
    log = oracle.reference_d2d(np.zeros(1, np.uint8), np.zeros(1, np.uint8), MiB + 131, execute=False)
    assert [l[5] for l in log] == [0, 1, 1]
    names = {0: b"LIBRECUDA_SUCCESS", 804: b"LIBRECUDA_ERROR_COMPAT_NOT_SUPPORTED_ON_DEVICE", 999: b"LIBRECUDA_ERROR_UNKNOWN"}
    for code, name in names.items():
        assert oracle.ref.ref_status_name(code) == name
    assert oracle.ref.ref_status_name(12345) is None


def test_golden_g1_dma_chronological_consistency():
    # reference tests/dma_chronological_consistency/main.cpp:33-36,56-85: 1 MiB + 131 bytes of i % 256,
    # HtoD -> five chained DtoD -> DtoH must come back equal
    n = MiB + 128 + 3
    host = (np.arange(n) % 256).astype(np.uint8)
    bufs = [host.copy()] + [np.zeros(n, np.uint8) for _ in range(5)]
    for i in range(5):
        oracle.ref_d2d_run(bufs[i + 1], bufs[i], n)
    assert np.array_equal(bufs[-1], host)
    assert [p[0] for p in oracle.ref_d2d_plan(n)] == [1, 2, 3]  # the size is chosen to need all three kernels


def test_golden_g2_memcopy_floats():
    # reference tests/memcopy/main.cpp:33-35,47-62: ten floats 1..10 round trip
    src = np.arange(1, 11, dtype=np.float32)
    dst = np.zeros(10, np.float32)
    oracle.ref_d2d_run(dst.view(np.uint8), src.view(np.uint8), 40)
    assert dst.tolist() == [float(i) for i in range(1, 11)]


def test_golden_g3_indexing_all_ones_is_a_d32_fill():
    # reference tests/indexing/main.cpp:82-114: every element must be 1.0f == bit pattern 0x3F800000
    a = np.zeros(50256 * 768 // 64, np.float32)
    oracle.memset(a, 0x3F800000, 4)
    assert (a == 1.0).all()


def test_memset_patterns():
    a = np.zeros(64, np.uint8)
    oracle.memset(a, 0xAB, 1)
    assert (a == 0xAB).all()
    oracle.memset(a, 0xBEEF, 2)
    assert (a.view("<u2") == 0xBEEF).all()
    oracle.memset(a, 0x40490FDB, 4)
    assert (a.view("<u4") == 0x40490FDB).all() and abs(float(a.view("<f4")[0]) - 3.14159265) < 1e-6


def test_index_fill_rounding_above_2_pow_24():
    n = (1 << 24) + 10
    a = oracle.index_fill_f32(n)
    assert a[1 << 24] == 16777216.0 and a[(1 << 24) + 1] == 16777216.0 and a[(1 << 24) + 3] == 16777220.0
    assert np.array_equal(a, np.arange(n, dtype=np.uint64).astype(np.float32))


def test_axpb_two_roundings():
    x = oracle.random_f32(4096, seed=2)
    y = oracle.axpb_f32(x, 2.0, 1.0)
    assert np.array_equal(y, (np.float32(2.0) * x) + np.float32(1.0))


def test_checksum_is_order_independent_sum_and_detects_swaps():
    a = oracle.random_bytes(4099, seed=3)
    c = oracle.checksum64(a)
    assert c == oracle.checksum64(a.copy())
    b = a.copy()
    b[8:16], b[16:24] = a[16:24].copy(), a[8:16].copy()  # swapping two words changes position-keyed terms
    assert oracle.checksum64(b) != c
    b = a.copy()
    b[-1] ^= 1
    assert oracle.checksum64(b) != c


@pytest.mark.parametrize("total,parts,align", [(8 << 30, 8, 2 << 20), (8 << 30, 2, 2 << 20), (10 * MiB + 5, 4, 2 << 20),
                                               (MiB, 8, 2 << 20), (0, 3, 4096), (4097, 2, 4096), (100, 7, 16)])
def test_partition_properties(total, parts, align):
    off = oracle.partition(total, parts, align)
    assert off[0] == 0 and off[-1] == total and len(off) == parts + 1
    assert all(a <= b for a, b in zip(off, off[1:]))
    assert all(o % align == 0 for o in off[1:-1] if o != total)
    sizes = [b - a for a, b in zip(off, off[1:])]
    assert max(sizes) - min(s for s in sizes if s or True) <= max(sizes)  # shards are contiguous and cover total
    assert sum(sizes) == total


def test_alltoall_model():
    n, chunk = 4, 48
    send = [oracle.random_bytes(n * chunk, seed=10 + r) for r in range(n)]
    recv = oracle.alltoall(send)
    for j in range(n):
        for r in range(n):
            assert np.array_equal(recv[j][r * chunk:(r + 1) * chunk], send[r][j * chunk:(j + 1) * chunk])


def test_mt_baseline_runs_and_copies():
    src = oracle.random_bytes(8 * MiB + 13, seed=4)
    dst = np.zeros_like(src)
    t = oracle.mt_seconds(dst, src, op=0, value=0, threads=3, reps=2)
    assert t > 0 and np.array_equal(dst, src)
    t = oracle.mt_seconds(dst, None, op=1, value=0x5A, threads=4, reps=1)
    assert t > 0 and (dst == 0x5A).all()


def test_seeded_stream_windows_match_the_stream_and_a_pure_python_restatement():
    # any window of the position-keyed stream equals the same bytes of the stream generated from its start ...
    full = oracle.random_bytes(1 << 20, seed=7)
    for off, n in ((0, 100), (8, 8), (4096 * 8, 1003), ((1 << 20) - 64, 64)):
        assert np.array_equal(oracle.random_window(off, n, 7), full[off:off + n])
    with pytest.raises(ValueError):
        oracle.random_window(3, 8, 7)
    # ... and far past 4 GiB it still follows the definition: word i = mix64(seed + (i + 1) * golden) mod 2^64
    M, G = (1 << 64) - 1, 0x9E3779B97F4A7C15

    def mix64(z):
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        return z ^ (z >> 31)

    for byte_off in ((4 << 30) - 8, 4 << 30, (7 << 30) + 4096):
        w = oracle.random_window(byte_off, 24, 1).view("<u8")
        i0 = byte_off // 8
        assert [int(x) for x in w] == [mix64((1 + (i0 + k + 1) * G) & M) for k in range(3)]
