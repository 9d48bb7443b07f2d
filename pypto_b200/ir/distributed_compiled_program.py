"""``DistributedConfig`` and ``DistributedCompiledProgram``: the level-3 (multi-GPU) call contract of the
reference (python/pypto/ir/distributed_compiled_program.py:60-117, 163-583) over one process per GPU.

``ir.compile(program, distributed_config=DistributedConfig(device_ids=[...]))`` resolves the program's
HOST-level orchestrator to a rank-side fused body (``pypto_b200.runtime.distributed_programs``).  Host tensors
carry a leading rank dimension; rank r works on slice r on GPU ``device_ids[r]``."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import torch

from ..language import Direction


@dataclass
class DistributedConfig:
    """Same fields and constraints as the reference's dataclass (:60-117).  ``num_sub_workers``, ``runtime`` and
    ``aicpu_thread_num`` configure the Ascend host runtime; they are validated and not used here."""

    device_ids: list[int] = field(default_factory=lambda: [0])
    num_sub_workers: int = 0
    runtime: str = "tensormap_and_ringbuffer"
    aicpu_thread_num: int = 0

    def __post_init__(self) -> None:
        if not self.device_ids:
            raise ValueError("DistributedConfig.device_ids must not be empty")
        if any(d < 0 for d in self.device_ids):
            raise ValueError(
                f"DistributedConfig.device_ids must be non-negative device indices, got {self.device_ids}")
        if len(set(self.device_ids)) != len(self.device_ids):
            raise ValueError(f"DistributedConfig.device_ids must be distinct, got {self.device_ids}")
        if self.num_sub_workers < 0:
            raise ValueError(f"DistributedConfig.num_sub_workers must be non-negative, got {self.num_sub_workers}")
        if self.aicpu_thread_num < 0 or self.aicpu_thread_num == 1:
            raise ValueError("DistributedConfig.aicpu_thread_num must be 0 (architecture default) or at least 2, "
                             f"got {self.aicpu_thread_num}")


class DistributedCompiledProgram:
    def __init__(self, entry, fused, platform: str, distributed_config: DistributedConfig, program=None):
        self.entry, self.fused, self._platform, self.distributed_config = entry, fused, platform, distributed_config
        self._program = program
        self.params = entry.params

    program = property(lambda s: s._program)
    platform = property(lambda s: s._platform)
    world_size = property(lambda s: len(s.distributed_config.device_ids))

    def __repr__(self):
        return (f"<DistributedCompiledProgram {self.entry.name} on {self._platform} "
                f"devices={self.distributed_config.device_ids}>")

    def _full_args(self, args):
        """In-place call (one argument per parameter) or return style (inputs only; outputs allocated with
        ``torch.zeros`` from their annotated shapes and returned) -- :403-473 of the reference."""
        params = self.params
        n_in = [p for p in params if p.direction is not Direction.Out]
        if len(args) == len(params):
            return list(args), []
        if len(args) == len(n_in):
            it, full, returned = iter(args), [], []
            for p in params:
                if p.direction is Direction.Out:
                    if not (p.is_tensor and p.type.shape and p.type.dtype):
                        raise TypeError(f"return-style call needs a static shape and dtype for output '{p.name}'")
                    t = torch.zeros(p.type.shape, dtype=p.type.dtype.torch_dtype)
                    returned.append(t)
                    full.append(t)
                else:
                    full.append(next(it))
            return full, returned
        expected = f"{len(params)} (in-place) or {len(n_in)} (return)"
        raise TypeError(f"DistributedCompiledProgram expects {expected} arguments, got {len(args)}. "
                        f"Parameters: {[p.name for p in params]}")

    def __call__(self, *args, config=None):
        """One-shot execution with host ``torch.Tensor`` arguments only (resident tensors belong to a prepared
        ``DistributedWorker``): start the ranks, run once, stop them."""
        from ..runtime.device_tensor import DeviceTensor, StackedDeviceTensor
        if any(isinstance(a, (DeviceTensor, StackedDeviceTensor)) for a in args):
            raise TypeError(
                "One-shot DistributedCompiledProgram calls cannot accept DeviceTensor or StackedDeviceTensor: "
                "use `with compiled.prepare() as worker:`, allocate with `worker.alloc_stacked_tensor()`, then "
                "call `worker.run(...)`.")
        full, returned = self._full_args(args)
        for p, a in zip(self.params, full):
            if not isinstance(a, torch.Tensor):
                raise TypeError("One-shot distributed programs only support host torch.Tensor parameters. "
                                f"Parameter {p.name!r} got {type(a).__name__}")
        with self.prepare(config) as worker:
            worker.run(self, *full, config=config)
        if not returned:
            return None
        return returned[0] if len(returned) == 1 else tuple(returned)

    def prepare(self, config=None, *, extra_compiled: Sequence["DistributedCompiledProgram"] = (),
                startup_timeout_s: float | None = None, **_ascend_only):
        """A reusable ``DistributedWorker`` (set up once, dispatch many): one process per GPU with its
        communicator; resident rank-sharded tensors through ``alloc_stacked_tensor``."""
        from ..runtime.distributed_runner import DistributedWorker
        return DistributedWorker([self, *extra_compiled], config, startup_timeout_s=startup_timeout_s)
