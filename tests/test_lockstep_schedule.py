"""The lock-step schedule of the copy-engine all-to-all (lcb_alltoall_engines_step, the function the launcher itself
follows), replayed on the CPU as a discrete-event simulation with arbitrary copy durations and start skews: no GPU
may ever have two senders at once, every rank must finish (no circular wait), and every chunk must arrive."""
import ctypes as C
import heapq
import random

import pytest

from librecuda_b200 import _native as N


def step_plan(n, rank, step):
    out = [C.c_int() for _ in range(5)]
    assert N.lib.lcb_alltoall_engines_step(n, rank, step, *[C.byref(o) for o in out]) == 0
    return [o.value for o in out]   # dest, wait_slot, wait_previous_call, post_rank, post_slot


def simulate(n, calls, rng):
    flags = [[0] * n for _ in range(n)]                 # flags[rank][slot]
    prog = {r: (1, 1) for r in range(n)}                # next (epoch, step) of every rank
    ready_at = {r: rng.uniform(0, 5) for r in range(n)}  # when the rank's stream reaches its next operation
    busy = {}                                           # receiver -> (sender, end time)
    intervals = {r: [] for r in range(n)}
    delivered = set()
    events = []                                         # (time, kind, rank, payload)
    waiting = set(range(n))
    now = 0.0
    done = set()
    for _ in range(200000):
        progressed = False
        for r in sorted(waiting):
            epoch, step = prog[r]
            dest, wslot, wprev, prank, pslot = step_plan(n, r, step)
            need = epoch - 1 if wprev else epoch
            if wslot >= 0 and not (wprev and epoch == 1) and flags[r][wslot] < need:
                continue                                # still spinning on its flag
            start = max(now, ready_at[r])
            dur = rng.uniform(0.5, 2.0)
            heapq.heappush(events, (start + dur, r, dest, start, epoch, step, prank, pslot))
            waiting.discard(r)
            progressed = True
        if not events:
            break
        end, r, dest, start, epoch, step, prank, pslot = heapq.heappop(events)
        now = end
        intervals[dest].append((start, end, r))
        delivered.add((epoch, r, dest))
        if prank >= 0:
            flags[prank][pslot] = epoch
        ready_at[r] = end + rng.uniform(0, 0.3)         # engine-to-kernel switch and the like
        step += 1
        if step == n:
            epoch, step = epoch + 1, 1
        if epoch > calls:
            done.add(r)
        else:
            prog[r] = (epoch, step)
            waiting.add(r)
        if len(done) == n:
            break
    return done, intervals, delivered


@pytest.mark.parametrize("n", [3, 4, 5, 8, 16])
def test_one_sender_per_gpu_at_any_time_and_no_deadlock(n):
    rng = random.Random(n)
    for trial in range(5):
        calls = 4
        done, intervals, delivered = simulate(n, calls, rng)
        assert len(done) == n, f"ranks stuck: {set(range(n)) - done}"
        assert delivered == {(e, r, d) for e in range(1, calls + 1) for r in range(n) for d in range(n) if d != r}
        for dest, spans in intervals.items():
            spans.sort()
            for (s0, e0, a), (s1, e1, b) in zip(spans, spans[1:]):
                assert s1 >= e0 - 1e-12, f"GPU {dest}: rank {b} started at {s1} while rank {a} was sending until {e0}"


def test_two_ranks_need_no_flags_and_bad_arguments_are_refused():
    assert step_plan(2, 0, 1) == [1, -1, 0, -1, -1]
    assert step_plan(2, 1, 1) == [0, -1, 0, -1, -1]
    out = [C.c_int() for _ in range(5)]
    refs = [C.byref(o) for o in out]
    assert N.lib.lcb_alltoall_engines_step(4, 0, 0, *refs) == 1      # steps start at 1
    assert N.lib.lcb_alltoall_engines_step(4, 0, 4, *refs) == 1
    assert N.lib.lcb_alltoall_engines_step(4, 4, 1, *refs) == 1
    assert N.lib.lcb_alltoall_engines_step(17, 0, 1, *refs) == 1


def test_the_simulation_sees_collisions_when_the_flags_are_ignored(monkeypatch):
    # the same replay with every wait and post removed (what the unsynchronised engine schedule did): receivers do
    # get two senders at once, so a pass of the test above is not vacuous
    import sys

    me = sys.modules[__name__]
    real = me.step_plan
    monkeypatch.setattr(me, "step_plan", lambda n, r, s: [real(n, r, s)[0], -1, 0, -1, -1])
    done, intervals, _ = simulate(5, 3, random.Random(1))
    assert len(done) == 5
    overlaps = 0
    for spans in intervals.values():
        spans.sort()
        overlaps += sum(1 for a, b in zip(spans, spans[1:]) if b[0] < a[1] - 1e-12)
    assert overlaps > 0
