"""The chunk protocol of the fused broadcasts (ring_bcast_warp_kernel / tree_bcast_kernel) replayed on the CPU as a
discrete-event simulation: every GPU has a few warps per role, a warp takes the next ticket of its role, waits for
that chunk's flag (the root does not wait), forwards the chunk to the role's children for a random time and posts
their flags.  With the topology the library itself uses (lcb_bcast_tree_plan; a plain chain for the ring), any
number of warps and any durations, every GPU must receive every chunk exactly once and every warp must leave --
nobody can wait in a circle, because a warp that waits holds nothing a sender needs."""
import ctypes as C
import heapq
import random

import pytest

from librecuda_b200 import _native as N


def tree_children(n, root):
    out = {}
    for r in range(n):
        parents = (C.c_int * 2)()
        kids = (C.c_int * 4)()
        assert N.lib.lcb_bcast_tree_plan(n, root, r, parents, kids) == 0
        out[r] = ([k for k in kids[0:2] if k >= 0], [k for k in kids[2:4] if k >= 0])
    return out


def chain_children(n, root):
    # the ring: one role that covers every chunk, the next GPU of the chain as the only child
    return {(root + k) % n: ([(root + k + 1) % n] if k + 1 < n else [], []) for k in range(n)}


def simulate(n, root, children, nchunks, split, warps, rng):
    """children[g] = (kids of role 0, kids of role 1); role 0 owns chunks [0, split), role 1 [split, nchunks)."""
    ranges = [(0, split), (split, nchunks)]
    arrived = [[0] * nchunks for _ in range(n)]        # how often chunk c was delivered to GPU g
    ticket = [[0, 0] for _ in range(n)]
    parked = {}                                          # (gpu, chunk) -> warps waiting for that flag
    events = []                                          # (time, seq, gpu, role, chunk) = a forward finishes
    left = [0] * n
    seq = 0

    def next_chunk(g, role, now):
        """A warp of (g, role) takes tickets until it has something to wait for or to send."""
        nonlocal seq
        lo, hi = ranges[role]
        while True:
            c = lo + ticket[g][role]
            ticket[g][role] += 1
            if c >= hi:
                left[g] += 1
                return
            if g != root and not arrived[g][c]:
                parked.setdefault((g, c), []).append(role)
                return
            if children[g][role]:
                seq += 1
                heapq.heappush(events, (now + rng.uniform(0.2, 3.0), seq, g, role, c))
                return
            # a role without children only waits: the chunk is there, take the next ticket

    for g in range(n):
        for role in (0, 1):
            for _ in range(warps[g][role]):
                next_chunk(g, role, rng.uniform(0.0, 5.0) if g != root else 0.0)
    while events:
        now, _, g, role, c = heapq.heappop(events)
        for kid in children[g][role]:
            arrived[kid][c] += 1
            for waiting_role in parked.pop((kid, c), []):
                if children[kid][waiting_role]:
                    seq += 1
                    heapq.heappush(events, (now + rng.uniform(0.2, 3.0), seq, kid, waiting_role, c))
                else:
                    next_chunk(kid, waiting_role, now)
        next_chunk(g, role, now)
    return arrived, left, parked


@pytest.mark.parametrize("n", [2, 3, 4, 5, 8, 9, 16])
@pytest.mark.parametrize("topology", ["trees", "chain"])
def test_every_chunk_arrives_once_and_every_warp_leaves(n, topology):
    rng = random.Random(1000 * n + len(topology))
    for root in {0, n // 2, n - 1}:
        for nchunks in (1, 2, 37, 150):
            split = nchunks // 2 if topology == "trees" else nchunks
            children = tree_children(n, root) if topology == "trees" else chain_children(n, root)
            warps = [[rng.randint(1, 6), rng.randint(1, 6)] for _ in range(n)]
            arrived, left, parked = simulate(n, root, children, nchunks, split, warps, rng)
            assert not parked, f"warps still wait for {sorted(parked)[:4]}"
            for g in range(n):
                assert left[g] == sum(warps[g]), f"GPU {g}: a warp never left"
                if g != root:
                    assert arrived[g] == [1] * nchunks, f"GPU {g} misses chunks or got one twice"


def test_the_replay_notices_a_broken_topology():
    # a chain whose third member forwards to nobody: the GPUs behind it must be seen waiting for ever
    n, root = 5, 0
    children = chain_children(n, root)
    children[2] = ([], [])
    rng = random.Random(5)
    arrived, left, parked = simulate(n, root, children, 20, 20, [[3, 1]] * n, rng)
    assert {g for g, _ in parked} == {3, 4}
    assert arrived[3] == [0] * 20 and arrived[4] == [0] * 20 and left[3] < 4 and left[4] < 4
    assert arrived[1] == [1] * 20 and arrived[2] == [1] * 20 and left[0] == 4
