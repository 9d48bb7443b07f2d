"""``RunConfig`` with the reference's fields (python/pypto/runtime/runner.py:330-399) and the
added platform ``"b200"`` -> ``BackendType.CudaSM100``.  Ascend-only knobs (ring sizing,
AICPU threads, swimlane levels ...) are accepted, validated the same way and ignored."""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any

from ..backend import PLATFORM_TO_BACKEND, BackendType, get_backend_instance
from ..ir.pass_manager import OptimizationStrategy

_RING_DEPTH = 4
PLATFORMS = ("a2a3sim", "a2a3", "a5sim", "a5", "b200")


def default_platform() -> str:
    return os.environ.get("PYPTO_PLATFORM", "b200")


def _normalize_swimlane_level(v, name):
    if isinstance(v, bool):
        return 4 if v else 0
    if not isinstance(v, int) or not 0 <= v <= 4:
        raise ValueError(f"{name} must be a bool or an int in 0..4, got {v!r}")
    return v


@dataclass
class RunConfig:
    __test__ = False

    platform: str = field(default_factory=default_platform)
    device_id: int = 0
    rtol: float = 1e-5
    atol: float = 1e-5
    strategy: OptimizationStrategy = field(default_factory=lambda: OptimizationStrategy.Default)
    backend_type: BackendType = field(default_factory=lambda: BackendType.CudaSM100)
    dump_passes: Any = False
    save_kernels: bool = False
    save_kernels_dir: str | None = None
    codegen_only: bool = False
    enable_chip_swimlane: int | bool = 0
    enable_dump_args: int = 0
    enable_pmu: int = 0
    enable_dep_gen: bool = False
    enable_scope_stats: bool = False
    compile_profiling: bool = False
    diagnostic_phase: Any = None
    disabled_diagnostics: Any = None
    golden_data_dir: str | None = None
    aicpu_thread_num: int | None = None
    ring_task_window: Any = None
    ring_heap: Any = None
    ring_dep_pool: Any = None
    distributed_config: Any = None
    analyze_auto_scopes_for_deps: bool = False
    memory_planner: Any = None
    dump_ptoas_passes: bool = False

    def __post_init__(self) -> None:
        if self.platform not in PLATFORMS:
            raise ValueError(f"Invalid platform {self.platform!r}. Expected one of {', '.join(map(repr, PLATFORMS))}.")
        # the platform is the source of truth; backend_type follows it (runner.py:371-384)
        self.backend_type = PLATFORM_TO_BACKEND[self.platform]
        arch = get_backend_instance(self.backend_type).get_handler().get_pto_target_arch()
        if not self.platform.startswith(arch):
            self.platform = arch + ("sim" if self.platform.endswith("sim") else "")
        self.enable_chip_swimlane = _normalize_swimlane_level(self.enable_chip_swimlane, "enable_chip_swimlane")
        if self.any_dfx_enabled() and not self.save_kernels:
            self.save_kernels = True
        self._validate_ring_overrides()

    def any_dfx_enabled(self) -> bool:
        return bool(self.enable_chip_swimlane or self.enable_dump_args or self.enable_pmu
                    or self.enable_dep_gen or self.enable_scope_stats)

    def _validate_ring_overrides(self) -> None:
        for name in ("ring_task_window", "ring_heap", "ring_dep_pool"):
            v = getattr(self, name)
            if v is None:
                continue
            if isinstance(v, bool):
                raise ValueError(f"{name} must be an int or a list of {_RING_DEPTH} ints")
            if isinstance(v, int):
                vals = [v]
            elif isinstance(v, (list, tuple)):
                if len(v) != _RING_DEPTH:
                    raise ValueError(f"{name} must have exactly {_RING_DEPTH} entries, got {len(v)}")
                vals = list(v)
                setattr(self, name, vals)
            else:
                raise ValueError(f"{name} must be an int or a list of {_RING_DEPTH} ints")
            for x in vals:
                if isinstance(x, bool) or not isinstance(x, int) or x < 0:
                    raise ValueError(f"{name} entries must be non-negative ints, got {x!r}")
