"""Host side of row sharding: the split of a matrix's rows over ranks and the exchange of arena handles.

One process per GPU.  The data path is inside the library (results of a row shard are pushed into every peer's arena by
the matvec kernels over NVLink); torch.distributed is used only to hand the 64-byte CUDA IPC handles around once.
"""
import ctypes as C

import numpy as np

from . import _lib


def shard_range(rows, rank, world):
    """(row0, nrows) of rank `rank`: the library's own rule (it_shard_range), pure host arithmetic."""
    L = _lib.load()
    r0, n = C.c_size_t(), C.c_size_t()
    _lib.check(L.it_shard_range(rows, rank, world, C.byref(r0), C.byref(n)))
    return r0.value, n.value


def gather_rows(slices):
    """Full output row from the per-rank slices in rank order (what the arena of every rank holds after a sharded op)."""
    return np.concatenate(slices, axis=-1)


def attach_peers(L, ctx, rank, world, group=None):
    """Exchanges the arena handles of all ranks and attaches them to `ctx`; with world == 1 it attaches the context to itself."""
    mine = (C.c_ubyte * 64)()
    _lib.check(L.it_ctx_ipc_handle(ctx, mine))
    handles = [bytes(mine)]
    if world > 1:
        import torch.distributed as dist
        handles = [None] * world
        dist.all_gather_object(handles, bytes(mine), group=group)
    blob = (C.c_ubyte * (64 * world)).from_buffer_copy(b"".join(handles))
    _lib.check(L.it_ctx_attach_peers(ctx, rank, world, blob))
    if world > 1:
        import torch.distributed as dist
        dist.barrier(group=group)      # nobody pushes into an arena that its owner has not finished setting up
