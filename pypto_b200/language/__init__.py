"""The ``pl`` names that the hot-path programs of the reference touch.

This is a compatibility surface, not a compiler front end: ``@pl.program``,
``@pl.function`` and ``@pl.jit`` record each function's name, kind, parameter names,
directions and annotated shapes/dtypes WITHOUT executing its body (the bodies are DSL
text for the reference's AST parser, python/pypto/language/parser/ast_parser.py).  The
launch surface then maps the orchestration entry to a fused CUDA kernel.  Type names
follow python/pypto/language/__init__.py:57-120.
"""

from __future__ import annotations

import enum
import inspect
import sys
import types

import torch


class DataType:
    def __init__(self, name: str, torch_dtype):
        self.name, self.torch_dtype = name, torch_dtype

    def __repr__(self):
        return f"pl.{self.name}"


FP32 = DataType("FP32", torch.float32)
FP16 = DataType("FP16", torch.float16)
BF16 = DataType("BF16", torch.bfloat16)
INT8 = DataType("INT8", torch.int8)
INT16 = DataType("INT16", torch.int16)
INT32 = DataType("INT32", torch.int32)
INT64 = DataType("INT64", torch.int64)
UINT8 = DataType("UINT8", torch.uint8)
UINT32 = DataType("UINT32", torch.int32)
UINT64 = DataType("UINT64", torch.int64)
BOOL = DataType("BOOL", torch.bool)
INDEX = DataType("INDEX", torch.int64)
FP8E4M3FN = DataType("FP8E4M3FN", getattr(torch, "float8_e4m3fn", torch.uint8))
FP8E5M2 = DataType("FP8E5M2", getattr(torch, "float8_e5m2", torch.uint8))
FP8E8M0 = DataType("FP8E8M0", getattr(torch, "float8_e8m0fnu", torch.uint8))      # MX scale codes
FP4 = DataType("FP4", getattr(torch, "float4_e2m1fn_x2", torch.uint8))

_BY_TORCH = {d.torch_dtype: d for d in (FP32, FP16, BF16, INT8, INT16, INT32, INT64, UINT8, BOOL, FP8E4M3FN)}


def dtype_of(torch_dtype) -> DataType:
    return _BY_TORCH[torch_dtype]


class FunctionType(enum.Enum):
    Opaque = 0
    Orchestration = 1
    InCore = 2
    AIC = 3
    AIV = 4
    Inline = 5
    Spmd = 6
    Group = 7


class MemorySpace(enum.Enum):
    DDR = 0
    Vec = 1
    Mat = 2
    Left = 3
    Right = 4
    Acc = 5
    Bias = 6
    LeftScale = 7
    RightScale = 8


Mem = MemorySpace


class Level(enum.Enum):
    CORE = 0
    CORE_GROUP = 1
    CHIP = 2
    HOST = 3


class Role(enum.Enum):
    Worker = 0
    Orchestrator = 1


class SplitMode(enum.Enum):
    NONE = 0
    UP_DOWN = 1
    LEFT_RIGHT = 2


class PadValue(enum.Enum):
    null = 0
    zero = 1
    max = 2
    min = 3


class TensorLayout(enum.Enum):
    """Physical layouts a tensor annotation can name (third item of ``pl.Tensor[[...], dtype, layout]``); the MX
    scale layouts are the ones of tests/st/runtime/ops/test_matmul_mx.py:38-101."""
    ND = 0
    MX_A_ZZ = 1
    MX_B_NN = 2


MX_A_ZZ, MX_B_NN = TensorLayout.MX_A_ZZ, TensorLayout.MX_B_NN


class _Dynamic:
    def __init__(self, name):
        self.name = name

    def __repr__(self):
        return f"dynamic({self.name!r})"


def dynamic(name: str = "?"):
    return _Dynamic(name)


class TensorType:
    """``pl.Tensor[[shape], dtype]`` annotation value."""

    kind = "tensor"

    def __init__(self, shape=None, dtype: DataType | None = None, layout: "TensorLayout | None" = None):
        self.shape = None if shape is None else tuple(shape)
        self.dtype = dtype
        self.layout = layout

    def __repr__(self):
        return f"pl.Tensor[{list(self.shape) if self.shape is not None else '?'}, {self.dtype}]"


class _TensorMeta(type):
    def __getitem__(cls, item):
        if not isinstance(item, tuple):
            item = (item,)
        shape = item[0] if item and isinstance(item[0], (list, tuple)) else None
        dt = next((x for x in item if isinstance(x, DataType)), None)
        t = TensorType(shape, dt, next((x for x in item if isinstance(x, TensorLayout)), None))
        t.kind = cls.kind
        return t


class Tensor(metaclass=_TensorMeta):
    kind = "tensor"


class Tile(metaclass=_TensorMeta):
    kind = "tile"


class ScalarType:
    kind = "scalar"

    def __init__(self, dtype):
        self.dtype = dtype

    def __repr__(self):
        return f"pl.Scalar[{self.dtype}]"


class Scalar:
    def __class_getitem__(cls, dtype):
        return ScalarType(dtype)


class Direction(enum.Enum):
    In = 0
    Out = 1
    InOut = 2


class _Directed:
    def __init__(self, direction, inner):
        self.direction, self.inner = direction, inner

    def __repr__(self):
        return f"pl.{self.direction.name}[{self.inner!r}]"


class Out:
    def __class_getitem__(cls, inner):
        return _Directed(Direction.Out, inner)


class InOut:
    def __class_getitem__(cls, inner):
        return _Directed(Direction.InOut, inner)


class Param:
    def __init__(self, name, annotation):
        self.name = name
        self.direction = Direction.In
        if isinstance(annotation, _Directed):
            self.direction, annotation = annotation.direction, annotation.inner
        if annotation is Tensor or annotation is Tile:
            annotation = TensorType(None, None)
        self.type = annotation
        self.is_tensor = isinstance(annotation, TensorType)

    def __repr__(self):
        return f"Param({self.name}: {self.direction.name} {self.type!r})"


class Function:
    """A decorated DSL function: signature captured, body never executed."""

    def __init__(self, fn, ftype=FunctionType.Opaque, attrs=None):
        self.fn, self.name, self.type = fn, fn.__name__, ftype
        self.attrs = dict(attrs or {})
        self.__name__, self.__doc__ = fn.__name__, fn.__doc__
        try:
            self.source = inspect.getsource(fn)
        except (OSError, TypeError):
            self.source = ""
        sig = inspect.signature(fn)
        ann = dict(getattr(fn, "__annotations__", {}))
        for k, v in ann.items():   # postponed annotations: evaluate in the defining module
            if isinstance(v, str):
                try:
                    ann[k] = eval(v, getattr(fn, "__globals__", {}))  # noqa: S307
                except Exception:
                    ann[k] = None
        self.params = [Param(n, ann.get(n)) for n in sig.parameters if n != "self"]

    @property
    def external_source(self):
        return self.attrs.get("external_source")

    def __call__(self, *a, **k):
        raise RuntimeError(f"DSL function '{self.name}' is not executable Python; compile the program "
                           "that calls it (pypto.runtime.run / ir.compile)")

    def __repr__(self):
        return f"<pl.function {self.name} {self.type.name}>"


def function(fn=None, *, type=FunctionType.Opaque, **attrs):  # noqa: A002 - reference keyword
    def wrap(f):
        return Function(f, type, attrs)
    return wrap(fn) if fn is not None else wrap


class Program:
    """A ``@pl.program`` class: its functions and the orchestration entry."""

    def __init__(self, cls):
        self.cls, self.name = cls, cls.__name__
        self.__name__, self.__doc__ = cls.__name__, cls.__doc__
        self.functions = {k: v for k, v in vars(cls).items() if isinstance(v, Function)}
        orch = [f for f in self.functions.values() if f.type is FunctionType.Orchestration]
        # a level-3 program's entry is its HOST-level orchestrator (@pl.function(level=pl.Level.HOST,
        # role=pl.Role.Orchestrator), tests/st/distributed/test_l3_ep_dispatch_combine.py:455)
        host = [f for f in self.functions.values()
                if f.attrs.get("level") is Level.HOST and f.attrs.get("role") is Role.Orchestrator]
        self.host_entry = host[-1] if host else None
        self.entry = self.host_entry or (orch[-1] if orch else
                                         (list(self.functions.values())[-1] if self.functions else None))

    def __repr__(self):
        return f"<pl.program {self.name} entry={self.entry.name if self.entry else None}>"


def program(cls):
    return Program(cls)


def _unexecuted(name):
    def op(*a, **k):
        raise RuntimeError(f"pl.{name} is a DSL operation; it only has meaning inside a compiled program")
    op.__name__ = name
    return op


class _OpNamespace(types.SimpleNamespace):
    def __getattr__(self, name):
        if name.startswith("_"):     # dunder and protocol probes (_repr_html_, ...): no operation is named so
            raise AttributeError(name)
        return _unexecuted(name)


tensor = _OpNamespace()
tile = _OpNamespace()
array = _OpNamespace()
system = _OpNamespace()


def __getattr__(name):
    """Any other ``pl.<op>`` (load, store, matmul, row_max, range, ...) resolves to a
    placeholder: DSL bodies are never executed here."""
    if name.startswith("_"):         # dunder and protocol probes (_repr_html_, ...): no operation is named so
        raise AttributeError(name)
    if name == "jit":
        from ..jit import jit as _jit
        return _jit
    return _unexecuted(name)


def _install_distributed():
    mod = types.ModuleType(__name__ + ".distributed")
    mod.__doc__ = "Placeholder names of pypto.language.distributed used in signatures."
    mod.DistributedTensor = Tensor

    class NotifyOp(enum.Enum):
        Set = 0
        AtomicAdd = 1

    class WaitCmp(enum.Enum):
        Eq = 0
        Ge = 1

    mod.NotifyOp, mod.WaitCmp = NotifyOp, WaitCmp
    mod.tensor, mod.system = _OpNamespace(), _OpNamespace()
    def _other(name):
        if name.startswith("_"):           # __file__, _repr_html_, ...: tools and notebooks ask for these; no operation is named so
            raise AttributeError(name)
        return _unexecuted(name)

    mod.__getattr__ = _other  # type: ignore[assignment]
    sys.modules[mod.__name__] = mod
    return mod


distributed = _install_distributed()
