"""Batch sharding across GPUs and the gather of the outputs into rank 0's memory.

The reference has no multi-device code.  Inference forward passes are independent per sample, so
each rank (one process per GPU) holds a full weight replica and evaluates a contiguous slice of the
batch with no communication; the only exchange is a device-to-device copy of each rank's output
rows into one buffer that lives in rank 0's memory (CUDA IPC mapping, so the copy goes over
NVLink / NVSwitch as plain peer stores — no NCCL on the data path, no TMA from peer memory).
torch.distributed is used for the rendezvous only (exchange of the IPC handle, barriers).
"""
import ctypes

import numpy as np


def batch_slice(global_batch, rank, world):
    """Contiguous slice [start, end) of the batch owned by `rank`; remainders go to the low ranks."""
    base, rem = divmod(global_batch, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def row_offsets(global_batch, world, row_bytes):
    """Byte offset of each rank's rows inside the gathered output."""
    return [batch_slice(global_batch, r, world)[0] * row_bytes for r in range(world)]


def share_from_rank0(dist, world, payload):
    """Rank 0's `payload` (any picklable object) on every rank; a no-op for one rank."""
    box = [payload]
    if world > 1:
        dist.broadcast_object_list(box, src=0)
    return box[0]


def max_over_ranks(dist, world, values, device=None):
    """Element-wise maximum of a list of floats over all ranks (the slowest rank sets the time)."""
    if world <= 1:
        return [float(v) for v in values]
    import torch
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.cpu()]


class OutputGather:
    """Rank 0 owns `global_rows * row_bytes` bytes; every rank writes its rows into it."""

    def __init__(self, ctx, dist, rank, world, global_rows, row_bytes):
        from . import lib, _P
        self.ctx, self.dist, self.rank, self.world, self.lib = ctx, dist, rank, world, lib
        self.row_bytes, self.global_rows = row_bytes, global_rows
        self.offsets = row_offsets(global_rows, world, row_bytes)
        self.buf = None
        payload = None
        if rank == 0:
            self.buf = ctx.alloc(global_rows * row_bytes)
            handle = (ctypes.c_uint8 * 64)()
            off = ctypes.c_uint64(0)
            ctx._ck(lib.sage_ipc_export(ctx.h, self.buf, handle, ctypes.byref(off)))
            payload = (bytes(handle), off.value)
            self.base = lib.sage_buf_ptr(self.buf)
            self.base_off = 0
        payload = share_from_rank0(dist, world, payload)
        if rank != 0:
            handle = (ctypes.c_uint8 * 64).from_buffer_copy(payload[0])
            p = _P()
            ctx._ck(lib.sage_ipc_open(ctx.h, handle, ctypes.byref(p)))
            self.base, self.base_off = p.value, payload[1]

    def write(self, session_var):
        """Asynchronously copies this rank's evaluated output into its rows of rank 0's buffer."""
        from . import _P
        ptr, n = _P(), ctypes.c_size_t(0)
        self.ctx._ck(self.lib.sage_var_buffer(self.ctx.s, session_var.h, ctypes.byref(ptr), ctypes.byref(n)))
        self.ctx._ck(self.lib.sage_peer_write_ptr(self.ctx.h, _P(self.base), ctypes.c_size_t(self.base_off + self.offsets[self.rank]),
                                                  ptr, n))
        return n.value

    def read(self, shape, dtype=np.float32):
        """Rank 0: the gathered array (call after every rank has synchronised)."""
        assert self.rank == 0
        return self.ctx.download(self.buf, shape, dtype)

    def close(self):
        if self.rank != 0 and self.base:
            self.lib.sage_ipc_close(self.ctx.h, ctypes.c_void_p(self.base))
            self.base = None
