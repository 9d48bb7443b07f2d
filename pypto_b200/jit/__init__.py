"""``@pl.jit``: call a DSL function directly with tensors (python/pypto/jit/decorator.py:
2041-2169).  The callable specialises on shapes and dtypes, caches the compiled program under
a key of source hash + shapes + dtypes + scalar values + platform (:2091-2110) and exposes
``_cache``, ``compile`` and ``lower``.  Sub-decorators (``jit.incore``, ``jit.inline``,
``jit.opaque``, ``jit.host``, ``jit.extern``) record helper functions whose bodies are never
executed here."""

from __future__ import annotations

import hashlib

import torch

from ..language import Function, FunctionType


class JITFunction(Function):
    def __init__(self, fn, ftype=FunctionType.Orchestration, attrs=None):
        super().__init__(fn, ftype, attrs)
        self._cache: dict = {}

    def _key(self, args, platform):
        parts = [hashlib.sha256(self.source.encode()).hexdigest(), platform]
        for a in args:
            if hasattr(a, "shape") and hasattr(a, "dtype"):
                parts.append((tuple(a.shape), str(a.dtype)))
            else:
                parts.append(("scalar", repr(a)))
        return tuple(parts)

    def compile(self, *args, config=None):  # noqa: A003
        from .. import ir
        from ..runtime.run_config import RunConfig
        cfg = config or RunConfig()
        key = self._key(args, cfg.platform)
        hit = self._cache.get(key)
        if hit is None:
            hit = self._cache[key] = ir.compile(self, platform=cfg.platform, strategy=cfg.strategy)
        return hit

    def lower(self, *args, config=None):
        return self.compile(*args, config=config)

    def __call__(self, *args, config=None):
        compiled = self.compile(*args, config=config)
        return compiled(*args, config=config)


def _sub(ftype):
    def deco(fn=None, **attrs):
        def wrap(f):
            return Function(f, ftype, attrs)
        return wrap(fn) if fn is not None else wrap
    return deco


class _Jit:
    def __call__(self, fn=None, **attrs):
        def wrap(f):
            return JITFunction(f, FunctionType.Orchestration, attrs)
        return wrap(fn) if fn is not None else wrap

    incore = staticmethod(_sub(FunctionType.InCore))
    inline = staticmethod(_sub(FunctionType.Inline))
    opaque = staticmethod(_sub(FunctionType.Opaque))
    host = staticmethod(_sub(FunctionType.Opaque))

    @staticmethod
    def extern(func=None, *, core_type="aiv", source=None, aic_source=None, aiv_source=None,
               dual_aiv_dispatch=False, include_dirs=None):
        """Signature-only stub backed by a hand-written kernel source
        (python/pypto/jit/decorator.py:2669-2738).  Here the source is CUDA for sm_100a; the
        AIC+AIV ``mixed`` form is recorded but has no single-kernel meaning on a GPU and is
        refused when the program is compiled."""
        if core_type not in ("aic", "aiv", "mixed"):
            raise ValueError(f"@pl.jit.extern core_type must be 'aic', 'aiv', or 'mixed', got {core_type!r}")
        if dual_aiv_dispatch and core_type != "mixed":
            raise ValueError("@pl.jit.extern dual_aiv_dispatch=True requires core_type='mixed'")

        def wrap(f):
            if core_type == "mixed":
                if aic_source is None or aiv_source is None:
                    raise ValueError("@pl.jit.extern(core_type='mixed') requires both aic_source= and aiv_source=")
                single = aiv_source
            else:
                single = source if source is not None else (aic_source or aiv_source)
                if single is None:
                    raise ValueError(f"@pl.jit.extern(core_type={core_type!r}) requires source=")
            return Function(f, FunctionType.AIC if core_type == "aic" else FunctionType.AIV,
                            dict(external_source=single, core_type=core_type, include_dirs=list(include_dirs or ()),
                                 dual_aiv_dispatch=dual_aiv_dispatch))
        return wrap(func) if func is not None else wrap


jit = _Jit()
__all__ = ["jit", "JITFunction"]
del torch
