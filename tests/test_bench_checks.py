"""The host side of the benchmark's verification (no GPU): the functions that say which bytes belong at an offset
of a destination buffer must agree with the oracle's own models, or every `verified` flag would be hollow."""
import sys
from pathlib import Path

import numpy as np

import oracle

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import bench  # noqa: E402


def test_alltoall_expectation_matches_the_oracle_exchange():
    G, chunk = 4, 4096 + 64
    send = [oracle.random_bytes(G * chunk, seed=100 + r) for r in range(G)]   # the bench seeds rank r with 100 + r
    recv = oracle.alltoall(send)
    for me in range(G):
        expect = bench.alltoall_expect(G, chunk, me)
        assert np.array_equal(expect(0, G * chunk), recv[me])
        for off, m in ((8, 100), (chunk - 16, 48), (2 * chunk + 8, chunk + 64), (G * chunk - 24, 24)):   # across slot borders
            assert np.array_equal(expect(off, m), recv[me][off:off + m]), (me, off, m)


def test_stream_expectation_is_a_window_of_the_seeded_stream():
    full = oracle.random_bytes(1 << 16, seed=3)
    expect = bench.stream_expect(3, base_offset=4096)
    assert np.array_equal(expect(0, 100), full[4096:4196])
    assert np.array_equal(expect(8 * 7, 1000), full[4096 + 56:4096 + 56 + 1000])


def test_host_window_check_picks_first_last_and_random_windows():
    # a fake stream whose memcpy "reads back" a host array: the checker must look at both ends and report a
    # difference planted in the last byte
    data = oracle.random_bytes(40 << 20, seed=9)

    class FakeStream:
        def __init__(self):
            self.reads = []

        def memcpy(self, host, dev_ptr, n):
            self.reads.append((dev_ptr, n))
            host[:] = data[dev_ptr:dev_ptr + n]

        def run(self):
            pass

    st = FakeStream()
    assert bench.host_windows_ok(None, st, 0, data.size, lambda off, n: data[off:off + n], salt=1)
    offs = sorted(o for o, _ in st.reads)
    assert offs[0] == 0 and offs[-1] == data.size - bench.WINDOW and len(offs) == 5
    wrong = data.copy()
    wrong[-1] ^= 1
    assert not bench.host_windows_ok(None, FakeStream(), 0, data.size, lambda off, n: wrong[off:off + n], salt=1)
    small = FakeStream()                                  # a range smaller than one window is read whole
    assert bench.host_windows_ok(None, small, 0, 1 << 20, lambda off, n: data[off:off + n], salt=2)
    assert small.reads == [(0, 1 << 20)]
