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
    def extern(source=None, core_type=None, **attrs):
        def wrap(f):
            return Function(f, FunctionType.AIV, dict(attrs, external_source=source, core_type=core_type))
        return wrap


jit = _Jit()
__all__ = ["jit", "JITFunction"]
del torch
