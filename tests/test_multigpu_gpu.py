"""Multi-GPU data movement inside one process (one context per GPU, peer access over NVLink): partitioned
copy, peer copy in both directions, the fused all-to-all, broadcast -- own kernels and the NCCL variants --
all bit-exact against the oracle's host models.  Needs at least two GPUs."""
import ctypes as C

import numpy as np
import pytest

import oracle
from librecuda_b200 import api

pytestmark = pytest.mark.gpu
MiB = 1 << 20
lib = api.lib


@pytest.fixture(scope="module")
def gpus(ctx, gpu_count):
    if gpu_count < 2:
        pytest.skip("needs >= 2 GPUs")
    n = min(gpu_count, 8)
    ctxs = [ctx] + [api.Context(i) for i in range(1, n)]
    for c in ctxs:
        c.set_current()
        for peer in ctxs:
            if peer is not c:
                can = C.c_int()
                api.check(lib.libreCuDeviceCanAccessPeer(C.byref(can), c.device, peer.device))
                assert can.value == 1
                c.enable_peer_access(peer)
                c.enable_peer_access(peer)  # idempotent
    streams = []
    for c in ctxs:
        c.set_current()
        streams.append(api.Stream())
    ctxs[0].set_current()
    yield ctxs, streams
    for s in streams:
        s.destroy()
    ctxs[0].set_current()


def _alloc_on(c, nbytes):
    c.set_current()
    return api.DeviceBuffer(nbytes)


def _upload(ctxs, streams, g, buf, host):
    ctxs[g].set_current()
    streams[g].memcpy(buf, host, host.nbytes)
    streams[g].run()


def _download(ctxs, streams, g, buf, nbytes):
    ctxs[g].set_current()
    out = np.empty(nbytes, np.uint8)
    streams[g].memcpy(out, buf, nbytes)
    streams[g].run()
    return out


@pytest.mark.parametrize("engine", [0, 1])
@pytest.mark.parametrize("so,do", [(0, 0), (1, 0), (16, 3)])
def test_peer_copy_push_and_pull(gpus, so, do, engine):
    # engine = 1: cross-GPU copies of 1 MiB and more go to the copy engines (by default: from 64 MiB); 0: always the copy kernel
    api.tune(peer_copy_engine=engine)
    try:
        _peer_copy_push_and_pull(gpus, so, do)
    finally:
        api.tune_reset()


def _peer_copy_push_and_pull(gpus, so, do):
    ctxs, streams = gpus
    n = 9 * MiB + 77
    src_h = oracle.random_bytes(n + 64, seed=3)
    a = _alloc_on(ctxs[0], n + 64)
    b = _alloc_on(ctxs[1], n + 64)
    _upload(ctxs, streams, 0, a, src_h)
    _upload(ctxs, streams, 1, b, np.zeros(n + 64, np.uint8))
    # push: kernel on GPU 0 stores into GPU 1's memory
    ctxs[0].set_current()
    api.check(lib.libreCuMemcpyPeer(b.ptr + do, a.ptr + so, n, streams[0].handle, False))
    streams[0].run()
    got = _download(ctxs, streams, 1, b, n + 64)
    assert np.array_equal(got[do:do + n], src_h[so:so + n]) and not got[:do].any() and not got[do + n:].any()
    # pull: kernel on GPU 1 loads from GPU 0's memory
    _upload(ctxs, streams, 1, b, np.zeros(n + 64, np.uint8))
    ctxs[1].set_current()
    api.check(lib.libreCuMemcpyPeer(b.ptr + do, a.ptr + so, n, streams[1].handle, False))
    streams[1].run()
    got = _download(ctxs, streams, 1, b, n + 64)
    assert np.array_equal(got[do:do + n], src_h[so:so + n])
    ctxs[0].set_current()
    a.free()
    ctxs[1].set_current()
    b.free()
    ctxs[0].set_current()


def test_partitioned_copy_scatter(gpus):
    ctxs, streams = gpus
    G = len(ctxs)
    total = 41 * MiB + 12345
    off = oracle.partition(total, G, 2 << 20)
    src_h = oracle.random_bytes(total, seed=3)
    src = _alloc_on(ctxs[0], total)
    _upload(ctxs, streams, 0, src, src_h)
    dsts = [_alloc_on(ctxs[g], max(off[g + 1] - off[g], 1) + 64) for g in range(G)]
    for g in range(G):
        _upload(ctxs, streams, g, dsts[g], np.zeros(dsts[g].nbytes, np.uint8))
    ctxs[0].set_current()
    dp = (C.c_void_p * G)(*[d.ptr for d in dsts])
    # all shards pushed by GPU 0 on separate streams of GPU 0 would share one port; here shard g is PULLED by GPU g
    sp = (C.c_void_p * G)(*[s.handle for s in streams])
    api.check(lib.libreCuMemcpyPartitioned(dp, src.ptr, total, G, 0, sp))
    for s in streams:
        s.commence()
    for s in streams:
        s.await_()
    for g in range(G):
        got = _download(ctxs, streams, g, dsts[g], dsts[g].nbytes)
        n = off[g + 1] - off[g]
        assert np.array_equal(got[:n], src_h[off[g]:off[g + 1]]) and not got[n:].any()
    for g in range(G):
        ctxs[g].set_current()
        dsts[g].free()
    ctxs[0].set_current()
    src.free()


@pytest.mark.parametrize("use_nccl", [0, 1, 2])
def test_all_to_all(gpus, use_nccl):
    ctxs, streams = gpus
    G = len(ctxs)
    chunk = 3 * MiB + 48
    send_h = [oracle.random_bytes(G * chunk, seed=30 + r) for r in range(G)]
    want = oracle.alltoall(send_h)
    send = [_alloc_on(ctxs[g], G * chunk) for g in range(G)]
    recv = [_alloc_on(ctxs[g], G * chunk) for g in range(G)]
    for g in range(G):
        _upload(ctxs, streams, g, send[g], send_h[g])
        _upload(ctxs, streams, g, recv[g], np.zeros(G * chunk, np.uint8))
    ctxs[0].set_current()
    rp = (C.c_void_p * G)(*[b.ptr for b in recv])
    sp = (C.c_void_p * G)(*[b.ptr for b in send])
    stp = (C.c_void_p * G)(*[s.handle for s in streams])
    api.check(lib.libreCuAllToAll(rp, sp, chunk, G, stp, use_nccl))
    for s in streams:
        s.await_()
    for g in range(G):
        assert np.array_equal(_download(ctxs, streams, g, recv[g], G * chunk), want[g]), f"rank {g}"
    for g in range(G):
        ctxs[g].set_current()
        send[g].free()
        recv[g].free()
    ctxs[0].set_current()


@pytest.mark.parametrize("use_nccl", [0, 1, 2])
def test_collective_starts_after_async_work_recorded_before_it(gpus, use_nccl):
    # the send buffers are filled by async=true uploads (side lanes of each stream) that are only recorded when
    # the collective is called: it has to submit them and start after them on every GPU
    ctxs, streams = gpus
    G = len(ctxs)
    chunk = 24 * MiB
    send_h = [oracle.random_bytes(G * chunk, seed=70 + r) for r in range(G)]
    want = oracle.alltoall(send_h)
    send = [_alloc_on(ctxs[g], G * chunk) for g in range(G)]
    recv = [_alloc_on(ctxs[g], G * chunk) for g in range(G)]
    for g in range(G):
        ctxs[g].set_current()
        streams[g].memset_d8(send[g], 0, G * chunk)
        streams[g].run()
        for j in range(G):  # one async upload per chunk: several side lanes in flight
            streams[g].memcpy(send[g].ptr + j * chunk, send_h[g][j * chunk:(j + 1) * chunk], chunk, async_=True)
    ctxs[0].set_current()
    rp = (C.c_void_p * G)(*[b.ptr for b in recv])
    sp = (C.c_void_p * G)(*[b.ptr for b in send])
    stp = (C.c_void_p * G)(*[s.handle for s in streams])
    api.check(lib.libreCuAllToAll(rp, sp, chunk, G, stp, use_nccl))
    for s in streams:
        s.await_()
    for g in range(G):
        assert np.array_equal(_download(ctxs, streams, g, recv[g], G * chunk), want[g]), f"rank {g}"
    for g in range(G):
        ctxs[g].set_current()
        send[g].free()
        recv[g].free()
    ctxs[0].set_current()


@pytest.mark.parametrize("pull", [False, True])
def test_all_to_all_recorded_per_rank(gpus, pull):
    # the per-rank half (push: remote stores, pull: remote loads) is an ordinary recorded stream operation
    ctxs, streams = gpus
    G = len(ctxs)
    chunk = MiB + 16
    send_h = [oracle.random_bytes(G * chunk, seed=50 + r) for r in range(G)]
    want = oracle.alltoall(send_h)
    send = [_alloc_on(ctxs[g], G * chunk) for g in range(G)]
    recv = [_alloc_on(ctxs[g], G * chunk) for g in range(G)]
    rp = (C.c_void_p * G)(*[b.ptr for b in recv])
    sp = (C.c_void_p * G)(*[b.ptr for b in send])
    for g in range(G):
        ctxs[g].set_current()
        streams[g].memcpy(send[g], send_h[g], G * chunk)
        if not pull:
            api.check(lib.libreCuAllToAllPush(rp, send[g].ptr, chunk, G, g, streams[g].handle))
    if pull:  # every send buffer must be complete before anyone loads from it
        for s in streams:
            s.run()
        for g in range(G):
            ctxs[g].set_current()
            api.check(lib.libreCuAllToAllPull(sp, recv[g].ptr, chunk, G, g, streams[g].handle))
    for s in streams:
        s.commence()
    for s in streams:
        s.await_()
    for g in range(G):
        assert np.array_equal(_download(ctxs, streams, g, recv[g], G * chunk), want[g])
    assert lib.libreCuAllToAllPush(rp, send[0].ptr, 24, G, 0, streams[0].handle) == api.ERROR_INVALID_VALUE
    assert lib.libreCuAllToAllPull(sp, recv[0].ptr, 24, G, 0, streams[0].handle) == api.ERROR_INVALID_VALUE
    assert lib.libreCuAllToAllPull(sp, recv[0].ptr, 32, G, G, streams[0].handle) == api.ERROR_INVALID_VALUE
    for g in range(G):
        ctxs[g].set_current()
        send[g].free()
        recv[g].free()
    ctxs[0].set_current()


def test_lockstep_engine_all_to_all_per_rank(gpus):
    # lcb_alltoall_engines is the form for one process per GPU; here every "rank" is a stream on its own GPU of this
    # process.  Three calls in a row with growing epochs: the flags posted by one call gate the first step of the
    # next.  (With two GPUs there is nothing to keep in step and no flag is touched.)
    ctxs, streams = gpus
    G = len(ctxs)
    chunk = 5 * MiB + 16
    send, recv, flags = [], [], []
    for g in range(G):
        send.append(_alloc_on(ctxs[g], G * chunk))
        recv.append(_alloc_on(ctxs[g], G * chunk))
        flags.append(_alloc_on(ctxs[g], 4096))
        _upload(ctxs, streams, g, flags[g], np.zeros(4096, np.uint8))
    rp = (C.c_void_p * G)(*[b.ptr for b in recv])
    fp = (C.c_void_p * G)(*[b.ptr for b in flags])
    for epoch in (1, 2, 3):
        send_h = [oracle.random_bytes(G * chunk, seed=90 + 10 * epoch + r) for r in range(G)]
        want = oracle.alltoall(send_h)
        for g in range(G):
            _upload(ctxs, streams, g, send[g], send_h[g])
            _upload(ctxs, streams, g, recv[g], np.zeros(G * chunk, np.uint8))
        for g in range(G):
            ctxs[g].set_current()
            api.lcb_check(lib.lcb_alltoall_engines(rp, send[g].ptr, chunk, G, g, flags[g].ptr, fp, epoch, 500,
                                                   streams[g].native, None), "lcb_alltoall_engines")
        for g in range(G):
            ctxs[g].set_current()
            api.lcb_check(lib.lcb_stream_synchronize(streams[g].native), "sync")
            assert api.device_error_word() == 0, f"rank {g}: a flag wait ran out"
        for g in range(G):
            assert np.array_equal(_download(ctxs, streams, g, recv[g], G * chunk), want[g]), f"epoch {epoch} rank {g}"
    ctxs[0].set_current()
    assert lib.lcb_alltoall_engines(rp, send[0].ptr, chunk, G, G, flags[0].ptr, fp, 1, 2000, streams[0].native, None) == 1
    if G > 2:
        assert lib.lcb_alltoall_engines(rp, send[0].ptr, chunk, G, 0, None, fp, 1, 2000, streams[0].native, None) == 1
        assert lib.lcb_alltoall_engines(rp, send[0].ptr, chunk, G, 0, flags[0].ptr, fp, 0, 2000, streams[0].native, None) == 1
    for g in range(G):
        ctxs[g].set_current()
        for b in (send[g], recv[g], flags[g]):
            b.free()
    ctxs[0].set_current()


def test_lockstep_engine_all_to_all_recorded(gpus):
    # the same exchange as a recorded stream operation (libreCuAllToAllEngines): runs at Commence, its local chunk on
    # a side lane that the next ordered operation joins; a DtoH recorded after it sees the complete result
    ctxs, streams = gpus
    G = len(ctxs)
    chunk = 2 * MiB + 32
    send_h = [oracle.random_bytes(G * chunk, seed=120 + r) for r in range(G)]
    want = oracle.alltoall(send_h)
    send = [_alloc_on(ctxs[g], G * chunk) for g in range(G)]
    recv = [_alloc_on(ctxs[g], G * chunk) for g in range(G)]
    flags = [_alloc_on(ctxs[g], 4096) for g in range(G)]
    rp = (C.c_void_p * G)(*[b.ptr for b in recv])
    fp = (C.c_void_p * G)(*[b.ptr for b in flags])
    for g in range(G):
        _upload(ctxs, streams, g, flags[g], np.zeros(4096, np.uint8))
        _upload(ctxs, streams, g, recv[g], np.zeros(G * chunk, np.uint8))
    for g in range(G):
        ctxs[g].set_current()
        streams[g].memcpy(send[g], send_h[g], G * chunk)
        api.check(lib.libreCuAllToAllEngines(rp, send[g].ptr, chunk, G, g, fp, 1, 500, streams[g].handle))
    # nothing ran yet: recorded only.  All ranks must be commenced before any is awaited (they wait for each other)
    for s in streams:
        s.commence()
    for s in streams:
        s.await_()
    for g in range(G):
        assert np.array_equal(_download(ctxs, streams, g, recv[g], G * chunk), want[g]), f"rank {g}"
    ctxs[0].set_current()
    assert lib.libreCuAllToAllEngines(rp, send[0].ptr, chunk, G, 0, fp, 1, 0, streams[0].handle) == api.ERROR_INVALID_VALUE
    if G > 2:
        assert lib.libreCuAllToAllEngines(rp, send[0].ptr, chunk, G, 0, None, 1, 2000, streams[0].handle) == api.ERROR_INVALID_VALUE
    for g in range(G):
        ctxs[g].set_current()
        for b in (send[g], recv[g], flags[g]):
            b.free()
    ctxs[0].set_current()


@pytest.mark.parametrize("use_nccl", [0, 1, 2, 3, 4, 5])
@pytest.mark.parametrize("root", [0, 1])
def test_broadcast(gpus, use_nccl, root):
    ctxs, streams = gpus
    G = len(ctxs)
    n = 37 * MiB + 1001
    api.tune(bcast_engine_piece_mib=4)     # form 2 with more than two GPUs: ten pieces, the last one ragged
    api.tune(bcast_mc_piece_mib=4, bcast_mc_slots=3)   # form 3: ten pieces through a ring of three slots, ragged end
    api.tune(bcast_ring_chunk_kib=16, bcast_ring_ctas=37)   # forms 4 and 5: 2369 chunks over 37 CTAs, the last chunk ragged
    try:
        _broadcast(ctxs, streams, G, n, use_nccl, root)
    finally:
        api.tune_reset()


@pytest.mark.parametrize("per_warp,chunk_kib,ctas,tickets", [(1, 8, 5, 1), (1, 8, 5, 0), (1, 0, 0, 1), (0, 16, 37, 0), (0, 0, 0, 0)])
def test_ring_broadcast_chunk_per_warp_and_per_cta(gpus, per_warp, chunk_kib, ctas, tickets):
    # Form 4 with either kernel: a chunk (and its flag) per warp -- handed out by ticket or by a fixed stride -- or
    # per CTA, with few workers and small chunks (every worker takes many turns, the last chunk ragged) and with
    # the shapes the library picks; the last GPU of the chain as root, twice in a row (the second call waits on
    # the next epoch of the same flag words and starts from ticket counters the first call must have reset).
    ctxs, streams = gpus
    G = len(ctxs)
    api.tune(bcast_ring_warp=per_warp, bcast_ring_chunk_kib=chunk_kib, bcast_ring_ctas=ctas, bcast_ring_tickets=tickets)
    try:
        _broadcast(ctxs, streams, G, 37 * MiB + 1001, 4, G - 1)
        _broadcast(ctxs, streams, G, 37 * MiB + 1001, 4, G - 1)
    finally:
        api.tune_reset()
    for g in range(G):
        ctxs[g].set_current()
        assert api.device_error_word() == 0
    ctxs[0].set_current()


@pytest.mark.parametrize("chunk_kib,ctas,tickets", [(4, 2, 1), (4, 2, 0), (8, 5, 1), (0, 0, 1)])
def test_two_tree_broadcast(gpus, chunk_kib, ctas, tickets):
    # Form 5: few warps and small chunks (every warp of either role takes many turns; an odd number of chunks, the
    # last one ragged) and the shapes the library picks; every rank as root in turn, so that every rank is inner
    # node, leaf and root of both trees; then a buffer of less than one chunk and one of two chunks.
    ctxs, streams = gpus
    G = len(ctxs)
    api.tune(bcast_ring_chunk_kib=chunk_kib, bcast_ring_ctas=ctas, bcast_ring_tickets=tickets)
    try:
        for root in range(G):
            _broadcast(ctxs, streams, G, 21 * MiB + 1001, 5, root)
        _broadcast(ctxs, streams, G, 1040, 5, 0)
        _broadcast(ctxs, streams, G, 2 * (chunk_kib or 8) * 1024, 5, G - 1)
    finally:
        api.tune_reset()
    for g in range(G):
        ctxs[g].set_current()
        assert api.device_error_word() == 0
    ctxs[0].set_current()


def _broadcast(ctxs, streams, G, n, use_nccl, root):
    data = oracle.random_bytes(n, seed=3)
    bufs = [_alloc_on(ctxs[g], n) for g in range(G)]
    for g in range(G):
        _upload(ctxs, streams, g, bufs[g], data if g == root else np.zeros(n, np.uint8))
    ctxs[0].set_current()
    bp = (C.c_void_p * G)(*[b.ptr for b in bufs])
    stp = (C.c_void_p * G)(*[s.handle for s in streams])
    api.check(lib.libreCuBroadcast(bp, root, n, G, stp, use_nccl))
    ran = C.c_int(-9)
    api.check(lib.libreCuBroadcastLastForm(C.byref(ran)))
    assert ran.value == use_nccl, "the requested form did not run (a B200 group supports every form)"
    for s in streams:
        s.await_()
    for g in range(G):
        assert np.array_equal(_download(ctxs, streams, g, bufs[g], n), data), f"rank {g}"
    for g in range(G):
        ctxs[g].set_current()
        bufs[g].free()
    ctxs[0].set_current()


def test_multicast_broadcast_large_misaligned_destinations_and_repeats(gpus):
    # form 3 (multimem stores through NVSwitch): default piece size, destinations at odd offsets (the local copy
    # out of the staging slab realigns), the last root, twice in a row through the same ring of slots; a root
    # buffer that is not 16-byte aligned takes the documented fall-back and must still deliver
    ctxs, streams = gpus
    G = len(ctxs)
    n = 200 * MiB + 7
    data = oracle.random_bytes(n, seed=33)
    root = G - 1
    bufs = [_alloc_on(ctxs[g], n + 64) for g in range(G)]
    offs = [0 if g == root else (1 + 3 * g) % 16 for g in range(G)]
    for rep, shift in ((0, 0), (1, 0), (2, 8)):
        roff = shift if shift else 0
        for g in range(G):
            _upload(ctxs, streams, g, bufs[g], np.zeros(n + 64, np.uint8))
        ctxs[root].set_current()
        streams[root].memcpy(bufs[root].ptr + roff, data, n)
        streams[root].run()
        ctxs[0].set_current()
        bp = (C.c_void_p * G)(*[b.ptr + (roff if g == root else offs[g]) for g, b in enumerate(bufs)])
        stp = (C.c_void_p * G)(*[s.handle for s in streams])
        api.check(lib.libreCuBroadcast(bp, root, n, G, stp, 3))
        ran = C.c_int(-9)
        api.check(lib.libreCuBroadcastLastForm(C.byref(ran)))
        assert ran.value == (3 if roff % 16 == 0 else (0 if G == 2 else 2))   # misaligned root: the documented fall-back
        for s in streams:
            s.await_()
        for g in range(G):
            got = _download(ctxs, streams, g, bufs[g], n + 64)
            o = roff if g == root else offs[g]
            assert np.array_equal(got[o:o + n], data), f"rep {rep} rank {g}"
            assert not got[:o].any() and not got[o + n:].any(), f"rep {rep} rank {g}: bytes outside the range"
    for g in range(G):
        ctxs[g].set_current()
        bufs[g].free()
    ctxs[0].set_current()


def test_kernel_copy_into_unreachable_peer_memory_is_refused_not_faulted(gpu_count, ctx):
    # a copy kernel on one GPU touching another GPU's memory without peer access would fault the GPU; a context
    # that was never given access through libreCuCtxEnablePeerAccess is refused at the API instead
    if gpu_count < 2:
        pytest.skip("needs >= 2 GPUs")
    ctx.set_current()
    near = api.DeviceBuffer(4096)          # device 0
    fresh = api.Context(1)                 # a new context on device 1: no peer access recorded for it
    far = api.DeviceBuffer(4096)           # device 1
    st = api.Stream()                      # stream of the fresh context
    assert lib.libreCuMemCpy(near.ptr, far.ptr, 4096, st.handle, False) == api.ERROR_INVALID_VALUE
    assert lib.libreCuMemCpy(far.ptr, near.ptr, 4096, st.handle, False) == api.ERROR_INVALID_VALUE
    assert lib.libreCuMemsetD8(near.ptr, 0, 4096, st.handle) == api.ERROR_INVALID_VALUE
    assert lib.libreCuMemsetD8(far.ptr, 0, 4096, st.handle) == api.SUCCESS      # its own memory is fine
    st.run()
    fresh.enable_peer_access(ctx)          # now allowed
    assert lib.libreCuMemCpy(near.ptr, far.ptr, 4096, st.handle, False) == api.SUCCESS
    st.run()
    st.destroy()
    far.free()
    ctx.set_current()
    near.free()
