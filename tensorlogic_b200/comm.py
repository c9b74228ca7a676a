"""Tensor-parallel communicator (one process per GPU, NCCL underneath).

The reference has nothing of the kind.  Rank 0 makes a 128-byte id with
``unique_id()``; the caller ships it to the other ranks (torch.distributed, a
pipe, a file) and every rank calls ``Comm(dev, id, rank, world)``.
``enable_p2p`` then maps the ranks' exchange blocks into one another (CUDA IPC)
so that the small all-reduces of a decode step run as one kernel over NVLink.
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

    def enable_p2p(self, max_elems: int, gather) -> None:
        """Sets up the peer-memory exchange for all-reduces of up to ``max_elems`` f16 values.

        ``gather(blob: bytes) -> list[bytes]`` must return every rank's blob in rank order (for
        instance ``torch.distributed.all_gather_object``); it carries the 64-byte CUDA IPC handles."""
        buf = C.create_string_buffer(64)
        check(self.dev.lib.tlc_comm_p2p_export(self.handle, max_elems, buf))
        blobs = gather(buf.raw)
        if len(blobs) != self.world or any(len(b) != 64 for b in blobs):
            raise ValueError("gather() must return one 64-byte handle per rank")
        check(self.dev.lib.tlc_comm_p2p_import(self.handle, C.create_string_buffer(b"".join(blobs), 64 * self.world)))

    @property
    def p2p_ready(self) -> bool:
        return bool(self.dev.lib.tlc_comm_p2p_ready(self.handle))

    def all_reduce_residual(self, partial: Tensor, residual: Tensor | None = None) -> Tensor:
        """residual + sum over the ranks of ``partial`` (which may be overwritten); one peer-memory
        kernel when the exchange is enabled and the vector fits, NCCL + add otherwise."""
        out = self.dev.empty(partial.shape)
        check(self.dev.lib.tlc_allreduce_residual_f16(self.dev.handle, self.handle, partial.ptr,
                                                      residual.ptr if residual is not None else None, out.ptr,
                                                      partial.size))
        return out

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
