"""pypto_b200: B200 (sm_100a) kernels for the fused operators of pypto's model examples,
behind pypto's program / launch surface.  See ``include/pypto_b200.h`` for the C ABI."""

from ._lib import BackendUnavailable, PtoError  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    import importlib
    if name in ("language", "runtime", "backend", "ir", "jit", "ops", "compat", "moe", "layers"):
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
