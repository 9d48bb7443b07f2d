"""``compile`` and ``CompiledProgram``: the call contract of the reference's compiled
artefact (python/pypto/ir/compiled_program.py:559-705, 1364-1414) on top of fused CUDA
operators.

compile() does not lower DSL bodies.  It takes the program's orchestration entry (name,
parameter names, directions, annotated shapes/dtypes -- all plain Python objects in the
signature) and looks the entry up in the fused-operator table
(``pypto_b200.runtime.fused_programs``).  A program with no fused kernel raises
``NotImplementedError``; nothing falls back to the CPU.
"""

from __future__ import annotations

import atexit
from typing import Any

import torch

from ..backend import PLATFORM_TO_BACKEND, BackendType
from ..language import Direction, Function, Program, TensorType
from .pass_manager import OptimizationStrategy

_implicit_workers: dict[int, Any] = {}


def _implicit_worker(config):
    """One cached worker per device for calls made outside a ``with ChipWorker`` block (the
    reference builds and tears down a Worker per one-shot call, device_runner.py:821-842;
    keeping it alive avoids re-creating the stream and staging buffers)."""
    from ..runtime.worker import ChipWorker
    w = _implicit_workers.get(config.device_id)
    if w is None or not w.initialized:
        w = _implicit_workers[config.device_id] = ChipWorker(config)
    return w


@atexit.register
def _close_implicit_workers():
    for w in _implicit_workers.values():
        try:
            w.close()
        except Exception:
            pass
    _implicit_workers.clear()


class CompiledProgram:
    def __init__(self, entry: Function, fused, platform: str, backend_type: BackendType, program=None):
        self.entry, self.fused, self.platform, self.backend_type = entry, fused, platform, backend_type
        self.program = program
        self.params = entry.params
        self.op_names = tuple(fused.op_names)

    def __repr__(self):
        return f"<CompiledProgram {self.entry.name} -> {'+'.join(self.op_names)} on {self.platform}>"

    # ---- argument handling (compiled_program.py:589-655) ----
    def _coerce_args(self, args):
        from ..runtime.device_tensor import DeviceTensor
        params = self.params
        n_in = [p for p in params if p.direction is not Direction.Out]
        returned = []
        if len(args) == len(params):
            full = list(args)
        elif len(args) == len(n_in):
            it = iter(args)
            full = []
            for p in params:
                if p.direction is Direction.Out:
                    if not (p.is_tensor and p.type.shape and p.type.dtype):
                        raise TypeError(f"return-style call needs a static shape and dtype for output '{p.name}'")
                    t = torch.zeros(p.type.shape, dtype=p.type.dtype.torch_dtype)
                    returned.append(t)
                    full.append(t)
                else:
                    full.append(next(it))
        else:
            raise TypeError(f"{self.entry.name}() takes {len(params)} arguments ({len(n_in)} without outputs), "
                            f"got {len(args)}")
        for p, a in zip(params, full):
            if not p.is_tensor:
                if isinstance(a, (torch.Tensor, DeviceTensor)):
                    raise TypeError(f"argument '{p.name}' is a scalar parameter, got a tensor")
                continue
            if not isinstance(a, (torch.Tensor, DeviceTensor)):
                raise TypeError(f"argument '{p.name}' must be a torch.Tensor or DeviceTensor, got {type(a).__name__}")
            if isinstance(a, torch.Tensor):
                if a.is_cuda:
                    raise TypeError(f"argument '{p.name}': pass host tensors or DeviceTensor handles, not CUDA tensors")
                if not a.is_contiguous():
                    raise ValueError(f"argument '{p.name}' must be contiguous")
            tt: TensorType = p.type
            if tt.dtype is not None and a.dtype != tt.dtype.torch_dtype:
                raise TypeError(f"argument '{p.name}' has dtype {a.dtype}, expected {tt.dtype.torch_dtype}")
            if tt.shape is not None and all(isinstance(s, int) for s in tt.shape) and tuple(a.shape) != tt.shape:
                raise ValueError(f"argument '{p.name}' has shape {tuple(a.shape)}, expected {tt.shape}")
        return full, returned

    def _invoke(self, worker, args, config=None):
        from ..runtime.device_tensor import DeviceTensor
        full, returned = self._coerce_args(args)
        host = {p.name: a for p, a in zip(self.params, full)}
        plan = self.fused.plan(self, host, worker)   # host-side reads (config tensor), validation
        replace = plan.get("replace", {})
        dev, staged = {}, []
        try:
            for p, a in zip(self.params, full):
                if not p.is_tensor:
                    continue
                a = replace.get(p.name, a)
                if isinstance(a, DeviceTensor):
                    if not worker.owns(a):
                        raise ValueError(f"argument '{p.name}': DeviceTensor is not a live allocation owned by this worker")
                    dev[p.name] = a
                    continue
                nbytes = a.numel() * a.element_size()
                ptr = worker._stage_alloc(max(nbytes, 1))
                staged.append((p, a, ptr, nbytes))
                if p.direction is not Direction.Out and p.name not in plan.get("host_only", ()):
                    worker._copy_to_async(ptr, a, nbytes)
                dev[p.name] = DeviceTensor(ptr, tuple(a.shape) or (1,), a.dtype)
            self.fused.launch(worker, dev, host, plan)
            for p, a, ptr, nbytes in staged:
                if p.direction is not Direction.In or p.name in plan.get("copy_back", ()):
                    worker._copy_from_async(a, ptr, nbytes)
            # one wait for the whole call; it also reads the device error word, so a clamped block id, a refused
            # index or a wait that ran out raises here instead of returning a silently wrong output
            worker.device_status()
        finally:
            for p, a, ptr, nbytes in staged:
                worker._stage_release(ptr, max(nbytes, 1))
        if returned:
            return returned[0] if len(returned) == 1 else tuple(returned)
        return None

    def __call__(self, *args, config=None):
        from ..runtime.run_config import RunConfig
        from ..runtime.worker import ChipWorker
        w = ChipWorker.current()
        if w is not None:
            w._check_binding(self)
            return self._invoke(w, args, config)
        cfg = config or RunConfig(platform=self.platform)
        if cfg.platform != self.platform:
            raise ValueError(f"config targets platform {cfg.platform!r}, program was compiled for {self.platform!r}")
        return self._invoke(_implicit_worker(cfg), args, cfg)


def compile(program, *, output_dir=None, strategy=OptimizationStrategy.Default, backend_type=None,  # noqa: A001
            platform: str | None = None, distributed_config=None, **_ignored) -> CompiledProgram:
    """Resolve ``program`` to its fused CUDA operator(s).  ``program`` is a ``@pl.program``
    class wrapper, a ``pl.Function`` or a JIT function."""
    from ..runtime import fused_programs
    from ..runtime.run_config import default_platform
    platform = platform or default_platform()
    if platform not in PLATFORM_TO_BACKEND:
        raise ValueError(f"Invalid platform {platform!r}")
    bt = PLATFORM_TO_BACKEND[platform]
    if bt is not BackendType.CudaSM100:
        from .. import BackendUnavailable
        raise BackendUnavailable(f"platform {platform!r} targets {bt.name}: its code generator and toolchain are "
                                 "not part of this build; compile for platform 'b200'")
    if distributed_config is not None:
        return _compile_distributed(program, platform, distributed_config)
    if isinstance(program, Program):
        entry = program.entry
    elif isinstance(program, Function):
        entry = program
    else:
        raise TypeError(f"compile() expects a @pl.program class or a pl.function, got {type(program).__name__}")
    if entry is None:
        raise ValueError("program has no functions")
    try:
        fused = fused_programs.lookup(entry)
    except NotImplementedError:
        # the reference's plugin hook: an orchestration that only dispatches external kernels
        from ..runtime import extern_kernel
        fused = extern_kernel.match(entry, program if isinstance(program, Program) else None)
        if fused is None:
            # a program under another name that computes what a fused operator computes
            fused = fused_programs.from_idiom(entry, program if isinstance(program, Program) else None)
        if fused is None:
            raise
    return CompiledProgram(entry, fused, platform, bt, program)


def _compile_distributed(program, platform: str, distributed_config):
    """Level-3 compile (python/pypto/ir/compile.py with ``distributed_config=``): resolve the HOST-level
    orchestrator of ``program`` to the rank-side fused body."""
    from ..runtime import distributed_programs
    from .distributed_compiled_program import DistributedCompiledProgram, DistributedConfig
    if not isinstance(distributed_config, DistributedConfig):
        raise TypeError(f"distributed_config must be a DistributedConfig, got {type(distributed_config).__name__}")
    if not isinstance(program, Program):
        raise TypeError(f"a distributed compile expects a @pl.program class, got {type(program).__name__}")
    entry = program.host_entry or program.entry
    if entry is None:
        raise ValueError("program has no functions")
    fused = distributed_programs.lookup(entry)
    return DistributedCompiledProgram(entry, fused, platform, distributed_config, program)
