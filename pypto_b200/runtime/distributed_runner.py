"""``DistributedWorker``: the prepared multi-GPU runtime object (python/pypto/runtime/distributed_runner.py:
1442-2910 of the reference: set up once, dispatch many, resident rank-sharded tensors).

One child process per GPU (``device_ids[r]`` for rank r), each with its own CUDA context, stream and -- for
more than one rank -- a communicator of ``pypto_b200.comm`` (NCCL over NVLink).  The parent never touches a
GPU: it hands rank-stacked host tensors to the children through shared memory and collects one reply per rank.
A child that fails reports its traceback and exits at once; the parent then stops the other ranks, which may
be blocked in a collective that can no longer complete.
"""

from __future__ import annotations

import os
import queue
import sys
import traceback

import torch

from ..language import Direction
from .device_tensor import StackedDeviceTensor

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _rank_main(rank: int, world: int, device_id: int, uid, programs, cmd_q, res_q) -> None:
    """Body of one rank process.  ``programs``: list of (rank-side fused op, [(param name, direction value)])."""
    try:
        if _ROOT not in sys.path:
            sys.path.insert(0, _ROOT)
        from pypto_b200 import ops
        from pypto_b200.comm import Communicator
        torch.cuda.set_device(device_id)
        dev = torch.device("cuda", device_id)
        comm = Communicator(rank, world, uid, device_id) if world > 1 else None
        resident: dict = {}
        states = [dict() for _ in programs]
        res_q.put((rank, "ready", None))
        while True:
            cmd = cmd_q.get()
            op = cmd[0]
            if op == "close":
                break
            if op == "run":
                _op, prog_idx, specs = cmd
                fused, params = programs[prog_idx]
                t, back = {}, []
                for (name, direction), spec in zip(params, specs):
                    if spec[0] == "host":
                        shard = spec[1][rank]
                        t[name] = shard.to(dev, non_blocking=True)
                        if direction != Direction.In.value:
                            back.append((shard, t[name]))
                    elif spec[0] == "stacked":
                        t[name] = resident[spec[1]]
                    else:
                        t[name] = spec[1]
                fused.run_rank(states[prog_idx], rank, world, comm, t)
                for shard, d in back:
                    shard.copy_(d, non_blocking=True)
                torch.cuda.synchronize()
                res_q.put((rank, "done", tuple(ops.device_status())))
            elif op == "alloc":
                _op, handle, shard = cmd
                resident[handle] = shard.to(dev)
                torch.cuda.synchronize()
                res_q.put((rank, "done", None))
            elif op == "read":
                _op, handle, shard = cmd
                shard.copy_(resident[handle])
                torch.cuda.synchronize()
                res_q.put((rank, "done", None))
            elif op == "free":
                resident.pop(cmd[1], None)
                res_q.put((rank, "done", None))
            else:
                raise ValueError(f"unknown command {op!r}")
        resident.clear()
        if comm is not None:
            comm.close()
        res_q.put((rank, "closed", None))
    except BaseException:
        res_q.put((rank, "error", traceback.format_exc()))
        os._exit(1)     # at once: a peer may wait in a collective for a rank that will not come


class DistributedRunHandle:
    """Outcome of one ``submit``: ``result()`` / ``wait()`` block until every rank has finished the dispatch
    and raise what a rank raised (:97-243 of the reference)."""

    def __init__(self, worker: "DistributedWorker", pending: int):
        self._worker, self._pending, self._done, self._error = worker, pending, pending == 0, None

    def done(self) -> bool:
        return self._done

    def result(self, timeout: float | None = None) -> None:
        if not self._done:
            try:
                replies = self._worker._collect(self._pending, timeout or self._worker.run_timeout_s)
                bad = [(r, st) for r, _k, st in replies if st is not None and st[0] != 0]
                if bad:
                    r, st = bad[0]
                    raise RuntimeError(f"rank {r}: device error word {st} (1 wait timed out, 2 block id outside the "
                                       "pool, 3 index outside its array)")
            except BaseException as e:
                self._error = e
            finally:
                self._done = True
                self._worker._inflight = None
        if self._error is not None:
            raise self._error

    wait = result


class DistributedWorker:
    def __init__(self, compiled_list, config=None, *, startup_timeout_s: float | None = None):
        import torch.multiprocessing as mp

        from .. import _lib
        if not compiled_list:
            raise ValueError("DistributedWorker needs at least one compiled program")
        primary = compiled_list[0]
        for c in compiled_list[1:]:
            self._check_compatible(c, primary)
        if not primary.platform.startswith("b200"):
            raise _lib.BackendUnavailable(f"platform {primary.platform!r} needs the Ascend runtime; this build "
                                          "executes on platform 'b200' only")
        self._compiled = list(compiled_list)
        self._multi_program = len(compiled_list) > 1
        self.device_ids = list(primary.distributed_config.device_ids)
        self.world = len(self.device_ids)
        self.run_timeout_s = 600.0
        self._closed, self._inflight, self._next_handle = True, None, 1
        self._stacked: dict = {}
        if not torch.cuda.is_available() or torch.cuda.device_count() <= max(self.device_ids):
            raise _lib.BackendUnavailable(f"device ids {self.device_ids} need {max(self.device_ids) + 1} visible CUDA "
                                          f"devices, found {torch.cuda.device_count() if torch.cuda.is_available() else 0}; "
                                          "there is no CPU fallback")
        uid = None
        if self.world > 1:
            from .. import comm
            uid = comm.unique_id()
        ctx = mp.get_context("spawn")
        self._res_q = ctx.Queue()
        self._cmd_qs = [ctx.Queue() for _ in range(self.world)]
        programs = [(c.fused, [(p.name, p.direction.value) for p in c.params]) for c in self._compiled]
        self._procs = [ctx.Process(target=_rank_main, daemon=True,
                                   args=(r, self.world, self.device_ids[r], uid, programs, self._cmd_qs[r], self._res_q))
                       for r in range(self.world)]
        self._closed = False
        try:
            for p in self._procs:
                p.start()
            self._collect(self.world, startup_timeout_s or 600.0, expect="ready")
        except BaseException:
            self._kill()
            raise

    @staticmethod
    def _check_compatible(prog, primary) -> None:
        if prog.platform != primary.platform or \
                list(prog.distributed_config.device_ids) != list(primary.distributed_config.device_ids):
            raise ValueError("programs prepared together must agree on platform and device ids")

    # ---- plumbing ----
    def _collect(self, n: int, timeout: float, expect: str = "done"):
        replies = []
        for _ in range(n):
            try:
                msg = self._res_q.get(timeout=timeout)
            except queue.Empty:
                self._kill()
                raise TimeoutError(f"a rank did not answer within {timeout:.0f} s (got {len(replies)} of {n} replies); "
                                   "all ranks were stopped") from None
            if msg[1] == "error":
                self._kill()
                raise RuntimeError(f"rank {msg[0]} failed; all ranks were stopped:\n{msg[2]}")
            if msg[1] != expect:
                self._kill()
                raise RuntimeError(f"rank {msg[0]} answered {msg[1]!r}, expected {expect!r}")
            replies.append(msg)
        return replies

    def _kill(self) -> None:
        for p in getattr(self, "_procs", []):
            if p.is_alive():
                p.terminate()
        for p in getattr(self, "_procs", []):
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join(timeout=10)
        self._closed = True

    def _require_open(self, op: str) -> None:
        if self._closed:
            raise RuntimeError(f"DistributedWorker.{op}: worker is closed")

    def _drain(self) -> None:
        if self._inflight is not None:
            self._inflight.result()

    # ---- resident rank-sharded tensors ----
    def alloc_stacked_tensor(self, host: torch.Tensor, *, worker_ids=None) -> StackedDeviceTensor:
        """Upload shard ``host[i]`` to worker ``worker_ids[i]`` once and keep it there (:2358-2472)."""
        self._require_open("alloc_stacked_tensor")
        if not isinstance(host, torch.Tensor):
            raise TypeError(f"alloc_stacked_tensor(host=...) expects a torch.Tensor, got {type(host).__name__}")
        if host.is_cuda or not host.is_contiguous() or host.dim() < 2:
            raise ValueError("alloc_stacked_tensor: host must be a contiguous CPU tensor [B, *tail]")
        ids = list(range(host.shape[0])) if worker_ids is None else list(worker_ids)
        if len(ids) != host.shape[0] or len(set(ids)) != len(ids) or any(not 0 <= w < self.world for w in ids):
            raise ValueError(f"worker_ids must be {host.shape[0]} distinct ids in [0, {self.world})")
        self._drain()
        handle, self._next_handle = self._next_handle, self._next_handle + 1
        for i, w in enumerate(ids):
            self._cmd_qs[w].put(("alloc", handle, host[i].clone()))
        self._collect(len(ids), self.run_timeout_s)
        st = StackedDeviceTensor(handle, host.shape, host.dtype, ids, owner=self)
        self._stacked[handle] = st
        return st

    def copy_stacked_from(self, stacked: StackedDeviceTensor, host: torch.Tensor) -> None:
        self._require_open("copy_stacked_from")
        if not isinstance(stacked, StackedDeviceTensor) or self._stacked.get(stacked.handle) is not stacked:
            raise TypeError("copy_stacked_from(stacked=...) expects a live StackedDeviceTensor of this worker")
        if tuple(host.shape) != stacked.full_shape or host.dtype != stacked.dtype:
            raise ValueError(f"host must have shape {stacked.full_shape} and dtype {stacked.dtype}")
        self._drain()
        staging = torch.empty_like(host).share_memory_()
        for i, w in enumerate(stacked.worker_ids):
            self._cmd_qs[w].put(("read", stacked.handle, staging[i]))
        self._collect(len(stacked.worker_ids), self.run_timeout_s)
        host.copy_(staging)

    def free_stacked_tensor(self, stacked: StackedDeviceTensor) -> None:
        self._require_open("free_stacked_tensor")
        if self._stacked.pop(stacked.handle, None) is None:
            raise ValueError("free_stacked_tensor: not a live StackedDeviceTensor of this worker")
        self._drain()
        for w in stacked.worker_ids:
            self._cmd_qs[w].put(("free", stacked.handle))
        self._collect(len(stacked.worker_ids), self.run_timeout_s)

    # ---- dispatch ----
    def submit(self, compiled, *args, config=None) -> DistributedRunHandle:
        """Start one dispatch on every rank and return; at most one dispatch is in flight (a second submit first
        waits for the one before it)."""
        self._require_open("submit")
        if compiled not in self._compiled:
            raise ValueError("DistributedWorker.run(compiled) requires a DistributedCompiledProgram registered "
                             "when this worker was constructed.")
        if len(args) != len(compiled.params):
            raise TypeError(f"expected {len(compiled.params)} arguments (in-place), got {len(args)}. "
                            f"Parameters: {[p.name for p in compiled.params]}")
        host, specs = {}, []
        for p, a in zip(compiled.params, args):
            if isinstance(a, StackedDeviceTensor):
                if self._stacked.get(a.handle) is not a:
                    raise ValueError(f"argument '{p.name}': StackedDeviceTensor does not belong to this worker")
                if tuple(a.worker_ids) != tuple(range(self.world)):
                    raise ValueError(f"argument '{p.name}': shard i must live on worker i for this program")
                specs.append(("stacked", a.handle))
            elif isinstance(a, torch.Tensor):
                if a.is_cuda or not a.is_contiguous():
                    raise ValueError(f"argument '{p.name}' must be a contiguous host tensor")
                if a.dim() < 1 or a.shape[0] != self.world:
                    raise ValueError(f"argument '{p.name}' must carry a leading rank dimension of {self.world}, "
                                     f"got shape {tuple(a.shape)}")
                if p.is_tensor and p.type.dtype is not None and a.dtype != p.type.dtype.torch_dtype:
                    raise TypeError(f"argument '{p.name}' has dtype {a.dtype}, expected {p.type.dtype.torch_dtype}")
                if p.is_tensor and p.type.shape is not None and all(isinstance(s, int) for s in p.type.shape) \
                        and tuple(a.shape) != p.type.shape:
                    raise ValueError(f"argument '{p.name}' has shape {tuple(a.shape)}, expected {p.type.shape}")
                host[p.name] = a
                specs.append(("host", a))
            elif p.is_tensor:
                raise TypeError(f"argument '{p.name}' must be a host torch.Tensor or a StackedDeviceTensor, "
                                f"got {type(a).__name__}")
            else:
                specs.append(("scalar", a))
        if len(host) == len([p for p in compiled.params if p.is_tensor]):
            compiled.fused.validate(self.world, host)
        self._drain()
        for s in specs:
            if s[0] == "host":
                s[1].share_memory_()     # the ranks read and write the caller's tensor through shared memory
        idx = self._compiled.index(compiled)
        for q in self._cmd_qs:
            q.put(("run", idx, specs))
        self._inflight = DistributedRunHandle(self, self.world)
        return self._inflight

    def run(self, compiled, *args, config=None) -> None:
        return self.submit(compiled, *args, config=config).result()

    def __call__(self, *args, config=None) -> None:
        if self._multi_program:
            raise TypeError("rt(*args) is ambiguous on a multi-program DistributedWorker; "
                            "dispatch explicitly with rt.run(compiled, *args).")
        return self.run(self._compiled[0], *args, config=config)

    def register(self, compiled):
        from .worker import RegistrationHandle
        self._require_open("register")
        if compiled not in self._compiled:
            raise ValueError("DistributedWorker.register(compiled) requires a DistributedCompiledProgram "
                             "registered when this worker was constructed.")
        return RegistrationHandle(self, compiled)

    # ---- lifecycle ----
    def close(self) -> None:
        if self._closed:
            return
        try:
            self._drain()
            for q in self._cmd_qs:
                q.put(("close",))
            self._collect(self.world, 120.0, expect="closed")
            for p in self._procs:
                p.join(timeout=30)
        finally:
            self._kill()
            self._stacked.clear()

    def __enter__(self):
        return self

    def __exit__(self, *_exc):
        self.close()
