"""Tensor-parallel communicator (one process per GPU, NCCL underneath).

The reference has nothing of the kind.  Rank 0 makes a 128-byte id with
``unique_id()``; the caller ships it to the other ranks (torch.distributed, a
pipe, a file) and every rank calls ``Comm(dev, id, rank, world)``.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check
from .api import Device, Tensor


def unique_id() -> bytes:
    from . import _lib
    buf = C.create_string_buffer(128)
    check(_lib.load().tlc_comm_unique_id(buf))
    return buf.raw


class Comm:
    def __init__(self, dev: Device, uid: bytes, rank: int, world: int):
        if len(uid) != 128:
            raise ValueError("a communicator id has 128 bytes")
        self.dev, self.rank, self.world = dev, rank, world
        h = C.c_void_p()
        check(dev.lib.tlc_comm_init(dev.handle, C.create_string_buffer(uid, 128), rank, world, C.byref(h)))
        self.handle = h

    def close(self) -> None:
        if self.handle and self.dev.handle:
            self.dev.lib.tlc_comm_destroy(self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def all_reduce(self, t: Tensor) -> Tensor:
        """In-place f16 sum over the ranks."""
        check(self.dev.lib.tlc_allreduce_f16(self.dev.handle, self.handle, t.ptr, t.size))
        return t

    def all_gather(self, t: Tensor) -> Tensor:
        out = self.dev.empty((self.world,) + tuple(t.shape))
        check(self.dev.lib.tlc_allgather_f16(self.dev.handle, self.handle, t.ptr, out.ptr, t.size))
        return out


def shard_ranges(n: int, world: int) -> list[tuple[int, int]]:
    """[start, stop) of each rank's contiguous share of n units (n must divide evenly)."""
    if n % world:
        raise ValueError(f"{n} units do not divide over {world} ranks")
    step = n // world
    return [(r * step, (r + 1) * step) for r in range(world)]


def combine_row_parallel(partials: list[np.ndarray]) -> np.ndarray:
    """What the all-reduce computes: f16 partial outputs summed (NCCL sums f16 in f32 per element pair-wise;
    the host emulation sums in f32 and rounds once)."""
    acc = np.zeros(partials[0].shape, np.float32)
    for p in partials:
        acc += p.astype(np.float32)
    return acc.astype(np.float16)
