"""Communicator of the expert-parallel path: one rank per GPU over NCCL, through the C ABI's
``pto_comm_*`` / ``pto_all_to_all*`` entry points.

It stands where the reference's level-3 runtime creates its communication domains and runs the
``all_to_all`` / ``all_to_all_v`` builtins (python/pypto/runtime/builtins/collectives/all_to_all_v/
templates/kernel.cpp.in:96-160).  torch supplies device buffers and streams only; when the ranks were
started by ``torch.distributed`` the 128-byte id travels through its store, nothing else.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _lib

UNIQUE_ID_BYTES = 128


def unique_id() -> bytes:
    """A fresh communicator id (rank 0 makes it and hands it to every other rank)."""
    buf = C.create_string_buffer(UNIQUE_ID_BYTES)
    _lib.check(_lib.load().pto_comm_unique_id(buf))
    return buf.raw


class Communicator:
    """``Communicator(rank, world, uid, device)`` is collective: every rank constructs it."""

    def __init__(self, rank: int, world: int, uid: bytes, device: int | None = None):
        if len(uid) != UNIQUE_ID_BYTES:
            raise ValueError(f"the communicator id must be {UNIQUE_ID_BYTES} bytes")
        self.rank, self.world = int(rank), int(world)
        self.device = torch.cuda.current_device() if device is None else int(device)
        h = C.c_void_p()
        _lib.check(_lib.load().pto_comm_init(self.rank, self.world, uid, self.device, C.byref(h)))
        self._h = h

    @classmethod
    def from_torch_distributed(cls, group=None, device: int | None = None) -> "Communicator":
        """Bootstrap from an initialised ``torch.distributed`` group: only the id goes through it."""
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        box = [unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        return cls(rank, world, box[0], device)

    def close(self) -> None:
        if self._h is not None:
            h, self._h = self._h, None
            _lib.check(_lib.load().pto_comm_destroy(h))

    def __enter__(self):
        return self

    def __exit__(self, *_exc):
        self.close()

    def _stream(self) -> int:
        return torch.cuda.current_stream(torch.device("cuda", self.device)).cuda_stream

    def all_to_all(self, send: torch.Tensor, recv: torch.Tensor) -> None:
        """Block p of ``send`` (numel / world elements) lands in block ``rank`` of rank p's ``recv``."""
        if send.numel() != recv.numel() or send.numel() % self.world or send.dtype != recv.dtype:
            raise ValueError("all_to_all: equal-sized tensors of one dtype, divisible by the world size")
        nbytes = send.numel() // self.world * send.element_size()
        _lib.check(_lib.load().pto_all_to_all(self._h, send.data_ptr(), recv.data_ptr(), nbytes, self._stream()))

    def all_to_all_v(self, send: torch.Tensor, send_rows, recv: torch.Tensor, recv_rows) -> None:
        """Send ``send_rows[p]`` consecutive rows to rank p, receive ``recv_rows[p]`` rows from rank p
        (source-rank order in ``recv``).  Rows are the leading dimension; exact counts."""
        if len(send_rows) != self.world or len(recv_rows) != self.world:
            raise ValueError("all_to_all_v: one row count per rank")
        row_bytes = (send.numel() // send.shape[0] if send.shape[0] else recv.numel() // max(recv.shape[0], 1)) \
            * send.element_size()
        if sum(send_rows) > send.shape[0] or sum(recv_rows) > recv.shape[0]:
            raise ValueError("all_to_all_v: row counts exceed the buffers")
        if row_bytes == 0:
            return
        sr = (C.c_int64 * self.world)(*[int(v) for v in send_rows])
        rr = (C.c_int64 * self.world)(*[int(v) for v in recv_rows])
        _lib.check(_lib.load().pto_all_to_all_v(self._h, send.data_ptr(), sr, recv.data_ptr(), rr, row_bytes,
                                                self._stream()))
