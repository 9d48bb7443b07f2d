"""Handle to a buffer resident on a worker (python/pypto/runtime/device_tensor.py:43-112)."""

from __future__ import annotations

from typing import Sequence

import torch


class DeviceTensor:
    __slots__ = ("data_ptr", "shape", "dtype", "buffer")

    def __init__(self, data_ptr: int, shape: Sequence[int], dtype: torch.dtype, *, buffer=None):
        if isinstance(data_ptr, bool) or not isinstance(data_ptr, int) or data_ptr <= 0:
            raise ValueError(f"DeviceTensor.data_ptr must be a positive int, got {data_ptr!r}")
        shape = tuple(shape)
        for d in shape:
            if isinstance(d, bool) or not isinstance(d, int):
                raise TypeError(f"DeviceTensor.shape must contain ints, got {shape!r}")
        if not shape:
            raise ValueError("DeviceTensor.shape must be non-empty")
        if any(d <= 0 for d in shape):
            raise ValueError(f"DeviceTensor.shape must be all positive, got {shape}")
        if not isinstance(dtype, torch.dtype):
            raise TypeError(f"DeviceTensor.dtype must be torch.dtype, got {type(dtype).__name__}")
        self.data_ptr, self.shape, self.dtype, self.buffer = data_ptr, shape, dtype, buffer

    @property
    def nbytes(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n * torch.empty(0, dtype=self.dtype).element_size()

    def numel(self) -> int:
        return self.nbytes // torch.empty(0, dtype=self.dtype).element_size()

    def __repr__(self):
        return f"DeviceTensor(data_ptr=0x{self.data_ptr:x}, shape={self.shape}, dtype={self.dtype})"


class StackedDeviceTensor:
    """A rank-sharded resident tensor: shard i (shape ``full_shape[1:]``) lives on worker ``worker_ids[i]`` of
    a ``DistributedWorker`` (python/pypto/runtime/device_tensor.py of the reference; made by
    ``DistributedWorker.alloc_stacked_tensor``).  ``handle`` names the shards inside the rank processes."""

    __slots__ = ("handle", "full_shape", "dtype", "worker_ids", "owner")

    def __init__(self, handle: int, full_shape, dtype: torch.dtype, worker_ids, owner=None):
        self.handle, self.full_shape, self.dtype = handle, tuple(full_shape), dtype
        self.worker_ids, self.owner = tuple(worker_ids), owner

    @property
    def shape(self):
        return self.full_shape

    def __repr__(self):
        return f"StackedDeviceTensor(shape={self.full_shape}, dtype={self.dtype}, workers={self.worker_ids})"
