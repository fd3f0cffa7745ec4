"""Batch-dimension data parallelism: one process per GPU, images sharded over
ranks, parameter gradients summed with one all-reduce.

Every image is independent in forward and dX (the batch index only appears in
x / y / dx offsets, crates/katsu-core/src/conv2d.rs:233-246); only dW (and the
matmul dB, tensor.rs:437-443) reduce over the batch, so those are the only
values that cross GPUs.  The reference itself is single-threaded; this module
has no counterpart there.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import cabi


def shard(total: int, rank: int, world: int) -> tuple[int, int]:
    """(first item, item count) of `rank`'s contiguous share; remainders go to the low ranks."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(total, world)
    count = base + (1 if rank < extra else 0)
    first = rank * base + min(rank, extra)
    return first, count


class GradBucket:
    """One flat device buffer holding every parameter gradient back to back, so
    a backward pass ends in a single all-reduce.  Kernels write dW straight
    into their slice (`ptr(name)`); nothing is packed or copied."""

    ALIGN = 64  # floats; keeps every slice 256-byte aligned for 128-bit accesses

    def __init__(self, ctx: cabi.Context, sizes: dict[str, int]):
        self.ctx, self.offsets, self.sizes = ctx, {}, dict(sizes)
        cursor = 0
        for name, count in sizes.items():
            self.offsets[name] = cursor
            cursor += -(-count // self.ALIGN) * self.ALIGN
        self.count = cursor
        self.base = ctx.alloc(cursor)

    def ptr(self, name: str) -> int:
        return self.base + 4 * self.offsets[name]

    def allreduce(self) -> None:
        self.ctx.call("katsu_cuda_allreduce_sum", self.base, self.count)

    def read(self, name: str) -> np.ndarray:
        return self.ctx.download(self.ptr(name), self.sizes[name])

    def free(self) -> None:
        self.ctx.free(self.base)
        self.base = 0


def init_comm(ctx: cabi.Context, dist, rank: int, world: int) -> None:
    """Creates the context's NCCL communicator; the unique id travels over the
    already-initialised torch.distributed group (any backend)."""
    ident = [None]
    if rank == 0:
        buf = (ctypes.c_uint8 * cabi.COMM_ID_BYTES)()
        cabi.check(ctx.lib.katsu_cuda_comm_unique_id(buf))
        ident[0] = bytes(buf)
    dist.broadcast_object_list(ident, src=0)
    raw = (ctypes.c_uint8 * cabi.COMM_ID_BYTES).from_buffer_copy(ident[0])
    ctx.call("katsu_cuda_comm_init", raw, world, rank)
