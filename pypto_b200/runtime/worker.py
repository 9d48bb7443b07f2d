"""``ChipWorker``: the single-chip runtime object (python/pypto/runtime/worker.py:118-650),
backed by the C ABI's ``pto_worker_*`` entry points instead of ``simpler.Worker``."""

from __future__ import annotations

import contextvars
import ctypes as C
import hashlib
import logging
import os
import weakref

import torch

from .. import _lib
from .device_tensor import DeviceTensor
from .run_config import RunConfig

_ACTIVE: contextvars.ContextVar = contextvars.ContextVar("pypto_b200_active_worker", default=None)

# The runtime logger (the reference's PYPTO_RUNTIME_LOG, docs/en/dev/03-logging.md:9-17): one ``logging`` logger for
# the package; the environment variable sets its level when the application has not configured it.
log = logging.getLogger("pypto_b200")
_level = os.environ.get("PYPTO_RUNTIME_LOG", "").strip().upper()
if _level in ("DEBUG", "INFO", "WARNING", "WARN", "ERROR"):
    log.setLevel(getattr(logging, "WARNING" if _level == "WARN" else _level))
    if not log.handlers and not logging.getLogger().handlers:
        logging.basicConfig(format="%(asctime)s %(name)s %(levelname)s %(message)s")


class ChipWorker:
    """Owns one device: allocations, a stream, registered callables.

    ``init`` / ``close`` are idempotent and ``close`` is retryable; an active worker
    (``with ChipWorker(cfg):``) is found through a ContextVar and reused by
    ``compiled(...)`` calls (worker.py:481-504)."""

    def __init__(self, config: RunConfig | None = None, *, level: int = 2, runtime: str = "b200",
                 enable_sdma: bool = False, auto_init: bool | None = None):
        if level != 2:
            raise ValueError(f"ChipWorker only supports level=2; got level={level}. "
                             "L3+ runtimes go through DistributedWorker.")
        self._config = config or RunConfig()
        self._level, self._runtime = level, runtime
        self._handle = None
        self._initialized = False
        self._owned: dict[int, DeviceTensor] = {}
        self._live_ptrs: dict[int, int] = {}
        self._pool: dict[int, list[int]] = {}   # freed staging blocks by size, reused by one-shot calls
        self._cid_cache: dict[str, int] = {}
        self._kernel_ids: dict[tuple, int] = {}
        self._handles: "weakref.WeakSet[RegistrationHandle]" = weakref.WeakSet()
        self._token = None
        if auto_init is None or auto_init:
            self.init()

    # ---- lifecycle ----
    def init(self) -> None:
        if self._initialized:
            return
        if not self._config.platform.startswith("b200"):
            raise _lib.BackendUnavailable(
                f"platform {self._config.platform!r} needs the Ascend toolchain and runtime; "
                "this build executes on platform 'b200' only")
        lib = _lib.load()
        if not torch.cuda.is_available():
            raise _lib.BackendUnavailable("no CUDA device is visible; there is no CPU fallback")
        h = C.c_void_p()
        _lib.check(lib.pto_worker_create(self._config.device_id, C.byref(h)))
        self._handle, self._initialized = h, True
        # diagnostics flags of the run configuration (runner.py:344-348): a swimlane level asks for timeline ranges
        # (NVTX, trace level 1), the PMU flag for per-callable device times (CUDA events, trace level 2)
        want = 2 if self._config.enable_pmu else (1 if self._config.enable_chip_swimlane else 0)
        if want > lib.pto_get_trace():
            _lib.check(lib.pto_set_trace(want))
        log.info("worker on device %d ready (trace level %d)", self._config.device_id, lib.pto_get_trace())

    def close(self) -> None:
        if not self._initialized:
            return
        for hd in list(self._handles):
            hd._mark_closed()
        lib = _lib.load()
        _lib.check(lib.pto_worker_destroy(self._handle))   # frees everything the worker still owns
        self._handle, self._initialized = None, False
        self._owned.clear(); self._live_ptrs.clear(); self._pool.clear(); self._cid_cache.clear(); self._kernel_ids.clear()

    def __enter__(self):
        self.init()
        self._token = _ACTIVE.set(self)
        return self

    def __exit__(self, *_exc):
        if self._token is not None:
            _ACTIVE.reset(self._token)
            self._token = None
        self.close()

    @staticmethod
    def current():
        return _ACTIVE.get()

    def _require_ready(self, op: str) -> None:
        if not self._initialized:
            raise RuntimeError(f"ChipWorker.{op}: worker is not initialized (or already closed)")

    @staticmethod
    def _require_local_worker_id(worker_id: int, op: str) -> None:
        if worker_id != 0:
            raise ValueError(f"ChipWorker.{op}: worker_id must be 0 for a level-2 worker, got {worker_id}")

    # ---- properties ----
    level = property(lambda s: s._level)
    platform = property(lambda s: s._config.platform)
    device_id = property(lambda s: s._config.device_id)
    runtime = property(lambda s: s._runtime)
    initialized = property(lambda s: s._initialized)

    @property
    def stream(self) -> int:
        self._require_ready("stream")
        return _lib.load().pto_worker_stream(self._handle) or 0

    # ---- memory ----
    def malloc(self, nbytes: int, *, worker_id: int = 0) -> int:
        self._require_ready("malloc"); self._require_local_worker_id(worker_id, "malloc")
        if isinstance(nbytes, bool) or not isinstance(nbytes, int) or nbytes < 0:
            raise ValueError(f"malloc: nbytes must be a non-negative int, got {nbytes!r}")
        p = C.c_uint64()
        _lib.check(_lib.load().pto_malloc(self._handle, nbytes, C.byref(p)))
        self._live_ptrs[p.value] = nbytes
        return p.value

    def free(self, ptr: int, *, worker_id: int = 0) -> None:
        self._require_ready("free"); self._require_local_worker_id(worker_id, "free")
        if ptr not in self._live_ptrs:
            raise ValueError(f"free: 0x{ptr:x} is not a live allocation of this worker (double free?)")
        _lib.check(_lib.load().pto_free(self._handle, ptr))
        del self._live_ptrs[ptr]

    def copy_to(self, dst_dev: int, src_host, nbytes: int, *, worker_id: int = 0) -> None:
        self._require_ready("copy_to"); self._require_local_worker_id(worker_id, "copy_to")
        src = src_host.data_ptr() if isinstance(src_host, torch.Tensor) else int(src_host)
        _lib.check(_lib.load().pto_copy_to(self._handle, dst_dev, src, nbytes))

    def copy_from(self, dst_host, src_dev: int, nbytes: int, *, worker_id: int = 0) -> None:
        self._require_ready("copy_from"); self._require_local_worker_id(worker_id, "copy_from")
        dst = dst_host.data_ptr() if isinstance(dst_host, torch.Tensor) else int(dst_host)
        _lib.check(_lib.load().pto_copy_from(self._handle, dst, src_dev, nbytes))

    def _copy_to_async(self, dst_dev: int, src_host: torch.Tensor, nbytes: int) -> None:
        _lib.check(_lib.load().pto_copy_to_async(self._handle, dst_dev, src_host.data_ptr(), nbytes))

    def _copy_from_async(self, dst_host: torch.Tensor, src_dev: int, nbytes: int) -> None:
        _lib.check(_lib.load().pto_copy_from_async(self._handle, dst_host.data_ptr(), src_dev, nbytes))

    def alloc_tensor(self, shape, dtype, *, init: torch.Tensor | None = None, worker_id: int = 0) -> DeviceTensor:
        """malloc + optional upload; rolled back if the upload fails (runtime_base.py:228-269)."""
        self._require_ready("alloc_tensor")
        shape = tuple(int(s) for s in shape)
        if init is not None:
            if not isinstance(init, torch.Tensor):
                raise TypeError("init must be a torch.Tensor")
            if tuple(init.shape) != shape or init.dtype != dtype:
                raise ValueError(f"init has shape {tuple(init.shape)} / {init.dtype}, expected {shape} / {dtype}")
            if init.is_cuda:
                raise ValueError("init must be a host tensor")
            init = init.contiguous()
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        ptr = self.malloc(nbytes, worker_id=worker_id)
        try:
            t = DeviceTensor(ptr, shape, dtype)
            if init is not None:
                self.copy_to(ptr, init, nbytes, worker_id=worker_id)
        except BaseException:
            self.free(ptr, worker_id=worker_id)
            raise
        self._owned[ptr] = t
        return t

    def free_tensor(self, t: DeviceTensor, *, worker_id: int = 0) -> None:
        self._require_ready("free_tensor")
        if self._owned.get(t.data_ptr) is not t:
            raise ValueError("free_tensor: DeviceTensor is not a live allocation owned by this worker")
        self.free(t.data_ptr, worker_id=worker_id)
        del self._owned[t.data_ptr]

    def owns(self, t: DeviceTensor) -> bool:
        return self._owned.get(t.data_ptr) is t

    def read_tensor(self, t: DeviceTensor) -> torch.Tensor:
        host = torch.empty(t.shape, dtype=t.dtype)
        self.copy_from(host, t.data_ptr, t.nbytes)
        return host

    # staging blocks for one-shot calls with host tensors
    def _stage_alloc(self, nbytes: int) -> int:
        lst = self._pool.get(nbytes)
        return lst.pop() if lst else self.malloc(nbytes)

    def _stage_release(self, ptr: int, nbytes: int) -> None:
        self._pool.setdefault(nbytes, []).append(ptr)

    def synchronize(self) -> None:
        self._require_ready("synchronize")
        _lib.check(_lib.load().pto_synchronize(self._handle))

    def device_status(self) -> tuple[int, int, int, int]:
        self._require_ready("device_status")
        words = (C.c_int32 * 4)()
        _lib.check(_lib.load().pto_device_status(self._handle, words))
        return tuple(words)

    # ---- dispatch ----
    def _cid(self, op_name: str) -> int:
        cid = self._cid_cache.get(op_name)
        if cid is None:
            out = C.c_int32()
            _lib.check(_lib.load().pto_register_callable(self._handle, op_name.encode(), C.byref(out)))
            cid = self._cid_cache[op_name] = out.value
        return cid

    def _task_args(self, tensors: list[DeviceTensor], scalars: list[int]):
        from ..ops import dtype_code
        arr = (_lib.ChipTensor * max(1, len(tensors)))()
        for i, t in enumerate(tensors):
            arr[i].addr, arr[i].start_offset, arr[i].ndims = t.data_ptr, 0, len(t.shape)
            if len(t.shape) > 5:
                raise ValueError("tensors of more than 5 dimensions are not supported")
            for j, s in enumerate(t.shape):
                arr[i].shapes[j] = s
            arr[i].dtype = dtype_code(t.dtype)
        sc = (C.c_uint64 * max(1, len(scalars)))(*[int(s) & 0xFFFFFFFFFFFFFFFF for s in scalars])
        return _lib.TaskArgs(arr, len(tensors), sc, len(scalars)), (arr, sc)

    def launch(self, op_name: str, tensors: list[DeviceTensor], scalars: list[int]) -> None:
        """Run one fused operator: tensors first, then uint64 scalars (the kernel_entry order,
        python/pypto/backend/pto_backend.py:541-629)."""
        self._require_ready("launch")
        args, _keep = self._task_args(tensors, scalars)
        if log.isEnabledFor(logging.DEBUG):
            log.debug("launch %s tensors=%s scalars=%s", op_name, [tuple(t.shape) for t in tensors], list(scalars))
        _lib.check(_lib.load().pto_run(self._handle, self._cid(op_name), C.byref(args)))

    def last_run_ms(self) -> float:
        """Device time of the last callable this worker ran, measured with CUDA events by the runtime; needs trace
        level 2 (``RunConfig(enable_pmu=1)``, ``pto_set_trace(2)`` or ``PTO_TRACE=2``).  Waits for that callable."""
        self._require_ready("last_run_ms")
        ms = C.c_float()
        _lib.check(_lib.load().pto_last_run_ms(self._handle, C.byref(ms)))
        return ms.value

    # ---- external kernels (the reference's external_source / jit.extern hook) ----
    def register_kernel_image(self, image: bytes, entry: str = "kernel_entry") -> int:
        """Load a cubin/PTX image built for sm_100a and return the id of its entry kernel.
        Images are cached per worker by content, so registering the same kernel twice is free."""
        self._require_ready("register_kernel_image")
        key = (hashlib.sha256(image).digest(), entry)
        cid = self._kernel_ids.get(key)
        if cid is None:
            out = C.c_int32()
            buf = C.create_string_buffer(image, len(image))
            _lib.check(_lib.load().pto_register_kernel_image(self._handle, buf, len(image), entry.encode(),
                                                             C.byref(out)))
            cid = self._kernel_ids[key] = out.value
        return cid

    def launch_kernel(self, cid: int, tensors: list[DeviceTensor], scalars: list[int], *, block_num: int = 1,
                      threads_per_block: int = 128) -> None:
        """One launch of an external kernel: `block_num` SPMD blocks (CTAs) of `threads_per_block`
        threads; arguments in the kernel_entry order (tensors, then scalars bit-cast to 64 bits)."""
        self._require_ready("launch_kernel")
        args, _keep = self._task_args(tensors, scalars)
        _lib.check(_lib.load().pto_run_kernel(self._handle, cid, C.byref(args), block_num, threads_per_block))

    def _check_binding(self, compiled) -> None:
        if compiled.platform != self.platform:
            raise ValueError(f"compiled program targets platform {compiled.platform!r} but this worker "
                             f"is bound to {self.platform!r}")

    def run(self, compiled, *args, config: RunConfig | None = None):
        self._require_ready("run")
        self._check_binding(compiled)
        return compiled._invoke(self, args, config)

    def register(self, compiled) -> "RegistrationHandle":
        self._require_ready("register")
        self._check_binding(compiled)
        for op in compiled.op_names:
            self._cid(op)
        h = RegistrationHandle(self, compiled)
        self._handles.add(h)
        return h


class RegistrationHandle:
    """A compiled program bound to a worker; callable until unregistered or the worker closes
    (worker.py:675-775)."""

    def __init__(self, worker: ChipWorker, compiled):
        self._worker, self._compiled, self._closed = worker, compiled, False

    cid = property(lambda s: tuple(s._worker._cid_cache.get(o) for o in s._compiled.op_names))
    compiled = property(lambda s: s._compiled)
    closed = property(lambda s: s._closed)

    def __call__(self, *args, config: RunConfig | None = None):
        if self._closed:
            raise RuntimeError("RegistrationHandle is closed")
        return self._worker.run(self._compiled, *args, config=config)

    def unregister(self) -> None:
        self._closed = True

    def _mark_closed(self) -> None:
        self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *_exc):
        self.unregister()
