"""Host-side plumbing for one-process-per-GPU runs (torch.distributed is used for rendezvous only).

The data path never goes through here: ranks exchange the 72-byte IPC handles of their buffers, open their
peers' buffers with libreCuIpcOpenMemHandle, and from then on the library's kernels store straight into peer
memory.  These helpers are backend-agnostic (gloo on CPU for tests, nccl on the GPUs).
"""
from __future__ import annotations

import ctypes as C

from . import api


def exchange_bytes(dist, payload: bytes) -> list:
    """All-gather one bytes object per rank; result[r] is rank r's payload."""
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, payload)
    return out


def max_over_ranks(dist, value: float, device=None) -> float:
    """Maximum of a per-rank scalar (device-timed milliseconds) over all ranks."""
    import torch

    t = torch.tensor([value], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def shard_of(total: int, world: int, rank: int, align: int = 0):
    """(offset, length) of rank's contiguous shard of `total` bytes (libreCuPartitionPlan boundaries)."""
    off = api.partition_plan(total, world, align)
    return off[rank], off[rank + 1] - off[rank]


def export_handle(buf) -> bytes:
    h = C.create_string_buffer(api.N.IPC_HANDLE_SIZE)
    api.check(api.lib.libreCuIpcGetMemHandle(h, buf.ptr), "libreCuIpcGetMemHandle")
    return h.raw


def open_peers(dist, buf) -> list:
    """Device pointers of every rank's `buf` (own pointer for the own rank).  Close the foreign ones with
    close_peers before freeing."""
    rank = dist.get_rank()
    handles = exchange_bytes(dist, export_handle(buf))
    ptrs = []
    for r, h in enumerate(handles):
        if r == rank:
            ptrs.append(buf.ptr)
        else:
            p = C.c_void_p()
            api.check(api.lib.libreCuIpcOpenMemHandle(C.byref(p), h), "libreCuIpcOpenMemHandle")
            ptrs.append(p.value)
    return ptrs


def close_peers(dist, ptrs):
    rank = dist.get_rank()
    for r, p in enumerate(ptrs):
        if r != rank:
            api.check(api.lib.libreCuIpcCloseMemHandle(p), "libreCuIpcCloseMemHandle")
