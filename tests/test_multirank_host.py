"""World-size-2 gloo runs (CPU) of the host-side logic behind `bench.py --gpus N` and multi-process users:
payload exchange, max-over-ranks timing, shard plans, and the all-to-all slot arithmetic against the oracle."""
import os
import socket

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from librecuda_b200 import multirank as mr

    got = mr.exchange_bytes(dist, bytes([rank]) * 72)
    ok = got == [bytes([r]) * 72 for r in range(world)]
    ok &= mr.max_over_ranks(dist, 1.5 + rank) == 1.5 + world - 1
    total = 10 * (1 << 20) + 5
    off, ln = mr.shard_of(total, world, rank, 2 << 20)
    plan = oracle.partition(total, world, 2 << 20)
    ok &= (off, ln) == (plan[rank], plan[rank + 1] - plan[rank])
    # all-to-all slot arithmetic: what rank r stores into peer j's buffer lands at offset r * chunk
    chunk = 64
    send = oracle.random_bytes(world * chunk, seed=100 + rank)
    sends = mr.exchange_bytes(dist, send.tobytes())
    recv = np.zeros(world * chunk, np.uint8)
    for r in range(world):
        peer_send = np.frombuffer(sends[r], np.uint8)
        recv[r * chunk:(r + 1) * chunk] = peer_send[rank * chunk:(rank + 1) * chunk]
    want = oracle.alltoall([np.frombuffer(s, np.uint8).copy() for s in sends])[rank]
    ok &= bool(np.array_equal(recv, want))
    dist.barrier()
    dist.destroy_process_group()
    q.put((rank, bool(ok)))


@pytest.mark.timeout(180)
def test_two_rank_host_logic_over_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=150) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert results == {0: True, 1: True}


def test_reference_arm_only_rank0_prints(tmp_path):
    # under torchrun the reference arm runs on rank 0 alone; other ranks exit 0 silently
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    res = subprocess.run([sys.executable, str(root / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "1"],
                         env=env, capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and res.stdout.strip() == ""
