"""The topology of the two-tree broadcast (lcb_bcast_tree_plan, the function libreCuBroadcast form 5 itself follows),
checked on the CPU for every group size and root: both trees span all ranks from the root, parents and children
agree, nobody forwards in both trees (so nobody sends more than one buffer's worth), and the depth is
1 + floor(log2(n - 1)) instead of the chain's n - 1."""
import ctypes as C

import pytest

from librecuda_b200 import _native as N


def plan(n, root, rank):
    parents = (C.c_int * 2)()
    kids = (C.c_int * 4)()
    assert N.lib.lcb_bcast_tree_plan(n, root, rank, parents, kids) == 0
    return list(parents), list(kids)


@pytest.mark.parametrize("n", list(range(2, 18)) + [33, 64])
def test_both_trees_span_the_group_with_logarithmic_depth(n):
    for root in range(n):
        plans = {r: plan(n, root, r) for r in range(n)}
        assert plans[root][0] == [-1, -1]
        for tree in (0, 1):
            kids_of = {r: [k for k in plans[r][1][2 * tree:2 * tree + 2] if k >= 0] for r in range(n)}
            assert len(kids_of[root]) == 1, "the root sends each half exactly once"
            depth = {root: 0}
            frontier = [root]
            while frontier:
                nxt = []
                for r in frontier:
                    for k in kids_of[r]:
                        assert k not in depth, "a rank receives a half twice"
                        assert plans[k][0][tree] == r, "parent and child disagree"
                        depth[k] = depth[r] + 1
                        nxt.append(k)
                frontier = nxt
            assert set(depth) == set(range(n)), "a rank is not reached"
            assert max(depth.values()) == 1 + (n - 1).bit_length() - 1
        for r in range(n):
            if r == root or n == 2:
                continue
            first, second = plans[r][1][:2], plans[r][1][2:]
            assert not (any(k >= 0 for k in first) and any(k >= 0 for k in second)), \
                f"rank {r} forwards in both trees: it would send two buffers' worth"


def test_plan_refuses_bad_arguments():
    parents = (C.c_int * 2)()
    kids = (C.c_int * 4)()
    assert N.lib.lcb_bcast_tree_plan(1, 0, 0, parents, kids) != 0
    assert N.lib.lcb_bcast_tree_plan(4, 4, 0, parents, kids) != 0
    assert N.lib.lcb_bcast_tree_plan(4, 0, -1, parents, kids) != 0
    assert N.lib.lcb_bcast_tree_plan(4, 0, 1, None, kids) != 0


def test_node_launcher_refuses_bad_arguments_before_touching_the_gpu():
    four = (C.c_void_p * 4)()
    buf = C.c_void_p(0x10000)
    call = N.lib.lcb_bcast_tree_node
    assert call(buf, None, four, four, 0, 8192, 0, 1, 100, 0, None) == 0              # nothing to do
    assert call(None, None, four, four, 1 << 20, 8192, 64, 1, 100, 0, None) != 0       # no buffer
    assert call(buf, None, four, four, 1 << 20, 8192, 64, 0, 100, 0, None) != 0        # epoch 0 is "never posted"
    assert call(buf, None, four, four, 1 << 20, 2048, 64, 1, 100, 0, None) != 0        # chunk too small
    assert call(buf, None, four, four, (1 << 20) + 8, 8192, 64, 1, 100, 0, None) != 0  # not whole vectors
    assert call(C.c_void_p(0x10008), None, four, four, 1 << 20, 8192, 64, 1, 100, 0, None) != 0  # misaligned
    assert call(buf, None, four, four, 1 << 20, 8192, 64, 1, 0, 0, None) != 0          # unbounded wait
    assert call(buf, None, four, four, 1 << 20, 8192, 129, 1, 100, 0, None) != 0       # split beyond the last chunk
    kids = (C.c_void_p * 4)(0x20000, None, None, None)
    assert call(buf, None, kids, four, 1 << 20, 8192, 64, 1, 100, 0, None) != 0        # a child without flags
    assert call(buf, None, four, four, 1 << 20, 8192, 64, 1, 100, 0, None) == 0        # a root without children
