"""Make ``import pypto`` resolve to this package, so that a program written for the
reference (``import pypto.language as pl``; ``from pypto.runtime import run, RunConfig``;
``from pypto.backend import BackendType``; ``from pypto import ir``) runs unchanged."""

from __future__ import annotations

import importlib
import sys

_SUBMODULES = ("language", "language.distributed", "runtime", "backend", "ir", "ir.pass_manager",
               "ir.compiled_program", "ir.distributed_compiled_program", "runtime.runner", "runtime.distributed_runner", "jit")


def install(name: str = "pypto") -> None:
    import pypto_b200
    if name in sys.modules and sys.modules[name] is not pypto_b200:
        raise RuntimeError(f"a different '{name}' package is already imported")
    sys.modules[name] = pypto_b200
    for sub in _SUBMODULES:
        try:
            mod = importlib.import_module(f"pypto_b200.{sub}")
        except ModuleNotFoundError:
            mod = sys.modules.get(f"pypto_b200.{sub}")
            if mod is None:
                raise
        sys.modules[f"{name}.{sub}"] = mod
