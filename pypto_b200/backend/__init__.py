"""Backend registry with the CUDA target.

Mirrors the reference's registry surface (include/pypto/backend/common/backend.h:53-56,
173-371; python/bindings/modules/backend.cpp:56-59, 204-228): a ``BackendType`` enum, a
singleton ``Backend`` per type with ``get_type_name()`` / ``get_handler()``, and the
module functions ``get_backend_instance``, ``set_backend_type``, ``get_backend_type``,
``reset_for_testing``.  The new member is ``BackendType.CudaSM100`` (platform ``"b200"``,
target arch ``sm_100a``); its op table holds fused-operator kernels of the shared
library instead of per-instruction code generators.  The Ascend members stay in the enum
so that programs naming them still import, but only the CUDA target can execute here.
"""

from __future__ import annotations

import enum


class BackendType(enum.Enum):
    Ascend910B = 0
    Ascend950 = 1
    CudaSM100 = 2


class BackendHandler:
    """Target constants consumers query (cf. include/pypto/backend/common/backend_handler.h:130-475)."""

    def __init__(self, backend_type: BackendType):
        self._type = backend_type

    def get_pto_target_arch(self) -> str:
        return {BackendType.Ascend910B: "a2a3", BackendType.Ascend950: "a5",
                BackendType.CudaSM100: "b200"}[self._type]

    def get_default_platform(self) -> str:
        return "b200" if self._type is BackendType.CudaSM100 else self.get_pto_target_arch() + "sim"

    def get_cuda_arch(self) -> str | None:
        return "sm_100a" if self._type is BackendType.CudaSM100 else None

    def get_sm_count(self) -> int:
        return 148

    def get_shared_memory_per_cta(self) -> int:
        return 227 * 1024

    def get_tensor_memory_columns(self) -> int:
        return 512

    def supports_dtype(self, name: str) -> bool:
        return name.upper() in {"FP32", "BF16", "FP16", "INT32", "INT64", "FP8E4M3FN", "UINT8"}

    def can_execute(self) -> bool:
        return self._type is BackendType.CudaSM100


class Backend:
    def __init__(self, backend_type: BackendType):
        self._type = backend_type
        self._handler = BackendHandler(backend_type)

    def get_type(self) -> BackendType:
        return self._type

    def get_type_name(self) -> str:
        return self._type.name

    def get_handler(self) -> BackendHandler:
        return self._handler

    def get_op_names(self) -> list[str]:
        """Fused operators registered for this target (REGISTER_BACKEND_OP analogue)."""
        if self._type is not BackendType.CudaSM100:
            return []
        from .. import _lib
        return _lib.op_names()


_instances: dict[BackendType, Backend] = {}
_current: BackendType | None = None


def get_backend_instance(backend_type: BackendType) -> Backend:
    if not isinstance(backend_type, BackendType):
        raise TypeError(f"expected BackendType, got {type(backend_type).__name__}")
    if backend_type not in _instances:
        _instances[backend_type] = Backend(backend_type)
    return _instances[backend_type]


def set_backend_type(backend_type: BackendType) -> None:
    """Select the global backend.  As in the reference (backend_config.cpp:24-66) a second
    call with a different type is an error until ``reset_for_testing``."""
    global _current
    if _current is not None and _current is not backend_type:
        raise RuntimeError(f"backend already configured as {_current.name}; cannot switch to {backend_type.name}")
    _current = backend_type


def get_backend_type() -> BackendType:
    if _current is None:
        raise RuntimeError("backend type not configured")
    return _current


def is_configured() -> bool:
    return _current is not None


def reset_for_testing() -> None:
    global _current
    _current = None


PLATFORM_TO_BACKEND = {"a2a3": BackendType.Ascend910B, "a2a3sim": BackendType.Ascend910B,
                       "a5": BackendType.Ascend950, "a5sim": BackendType.Ascend950,
                       "b200": BackendType.CudaSM100}
