"""External kernels: hand-written CUDA attached to a program function.

The reference lets a program name a hand-written device source for one function --
``@pl.function(type=pl.FunctionType.AIV, external_source=path)`` inside a ``@pl.program`` or
``@pl.jit.extern(source=path, core_type="aiv")`` for the JIT style -- with a signature-only stub
(``...`` body); its backend skips code generation for that function and compiles the file where
it lies, so sibling headers stay reachable (python/pypto/jit/decorator.py:2669-2738,
python/pypto/backend/pto_backend.py:1181-1191, 1884-1897,
tests/st/runtime/external_kernel/test_external_kernel.py:50-65).

Here the source is CUDA for sm_100a defining ``extern "C" __global__ void kernel_entry(const
int64_t* args)`` (``include/pypto_b200_device.h`` has the argument accessors).  It is compiled
with nvcc to a cubin at its original path, cached by the content of the file and of the files it
includes, loaded into the worker (``pto_register_kernel_image``) and launched with one CTA per
SPMD block (``pto_run_kernel``).

The orchestration that calls the stubs is not lowered: its body must be a plain sequence of
calls, each optionally under ``with pl.spmd(core_num=N):``, with entry parameters, results of
earlier calls or constants as arguments.  A callee is either an external function or a function
whose name and parameter list are in the fused-operator table (``fused_programs``), so one
orchestration can chain hand-written kernels and fused operators.  Anything else is refused.
"""

from __future__ import annotations

import ast
import hashlib
import inspect
import os
import re
import shutil
import struct
import subprocess
import tempfile
import textwrap
from pathlib import Path

from ..language import Direction, Function, FunctionType, ScalarType
from .fused_programs import FusedOp

ENTRY_SYMBOL = "kernel_entry"
_ROOT_INCLUDE = Path(__file__).resolve().parents[2] / "include"
_INCLUDE_RE = re.compile(r'^\s*#\s*include\s*"([^"]+)"', re.M)


def cache_dir() -> Path:
    d = Path(os.environ.get("PYPTO_B200_CACHE") or Path.home() / ".cache" / "pypto_b200") / "extern"
    d.mkdir(parents=True, exist_ok=True)
    return d


def _dependency_closure(source: Path, include_dirs) -> list[Path]:
    """The entry file and every quoted include that resolves next to the including file or in
    an include directory (system headers and the toolkit are covered by the nvcc version)."""
    seen, todo = [], [source.resolve()]
    while todo:
        f = todo.pop()
        if f in seen or not f.is_file():
            continue
        seen.append(f)
        for name in _INCLUDE_RE.findall(f.read_text(errors="replace")):
            for base in (f.parent, *include_dirs):
                cand = (Path(base) / name).resolve()
                if cand.is_file():
                    todo.append(cand)
                    break
    return seen


def compile_cuda(source, include_dirs=()) -> bytes:
    """nvcc ``source`` (compiled as CUDA whatever its suffix) to a cubin for sm_100a."""
    source = Path(source)
    if not source.is_file():
        raise FileNotFoundError(f"external kernel source not found: {source}")
    include_dirs = [str(Path(d).resolve()) for d in include_dirs]
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: external kernels are compiled when the program is compiled")
    flags = ["-cubin", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
             "-I", str(_ROOT_INCLUDE)]
    for d in include_dirs:
        flags += ["-I", d]
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    h.update(subprocess.run([nvcc, "--version"], capture_output=True, text=True).stdout.encode())
    for f in _dependency_closure(source, [_ROOT_INCLUDE, *include_dirs]):
        h.update(str(f).encode())
        h.update(f.read_bytes())
    out = cache_dir() / f"{source.stem}-{h.hexdigest()[:24]}.cubin"
    if not out.exists():
        with tempfile.NamedTemporaryFile(dir=out.parent, suffix=".cubin", delete=False) as tmp:
            tmp_path = tmp.name
        try:
            r = subprocess.run([nvcc, *flags, "-x", "cu", str(source), "-o", tmp_path], capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed for external kernel {source}:\n{r.stdout}{r.stderr}")
            os.replace(tmp_path, out)
        finally:
            if os.path.exists(tmp_path):
                os.unlink(tmp_path)
    return out.read_bytes()


def resolve_source(fn: Function) -> Path:
    src = fn.attrs.get("external_source") or fn.attrs.get("external_aiv_source")
    p = Path(os.fspath(src))
    if not p.is_absolute():
        here = inspect.getsourcefile(fn.fn)
        p = (Path(here).parent if here else Path.cwd()) / p
    return p


def include_dirs_of(fn: Function) -> list[Path]:
    dirs = fn.attrs.get("include_dirs") or fn.attrs.get("extra_include_dirs") or ()
    here = inspect.getsourcefile(fn.fn)
    base = Path(here).parent if here else Path.cwd()
    return [Path(d) if Path(d).is_absolute() else base / d for d in map(os.fspath, dirs)]


def encode_scalar(value, ptype) -> int:
    """A scalar argument as the 64 bits the kernel reads: integers sign-extended, fp32 as its
    bit pattern (python/pypto/backend/pto_backend.py:541-629 bit-casts scalars to uint64)."""
    name = getattr(getattr(ptype, "dtype", None), "name", "INDEX")
    if name == "FP32":
        return struct.unpack("<I", struct.pack("<f", float(value)))[0]
    if name in ("FP16", "BF16") or name.startswith("FP8"):
        raise TypeError(f"scalar parameters of type {name} are not supported by external kernels")
    if isinstance(value, float) and not float(value).is_integer():
        raise TypeError(f"scalar parameter of type {name} got the non-integral value {value!r}")
    return int(value) & 0xFFFFFFFFFFFFFFFF


class _Step:
    def __init__(self, fn: Function, block_num: int, bindings: list, fused=None):
        self.fn, self.block_num, self.bindings = fn, block_num, bindings   # ("param", name) | ("const", value)
        self.threads = int(fn.attrs.get("threads_per_block", 128))
        self.fused = fused            # a FusedOp when the callee is in the fused-operator table, else None

    def bind(self, values: dict) -> dict:
        """The callee's view of a {entry parameter: value} mapping."""
        return {p.name: (values[v] if kind == "param" else v) for p, (kind, v) in zip(self.fn.params, self.bindings)}


class ExternProgramOp(FusedOp):
    """A program whose orchestration is a sequence of external kernels and fused operators."""

    def __init__(self, entry: Function, steps: list[_Step]):
        self.entry, self.steps = entry, steps
        self._images: dict[int, bytes] = {}
        self.op_names = tuple(dict.fromkeys(n for s in steps if s.fused is not None for n in s.fused.op_names))

    def matches(self, entry) -> bool:
        return entry is self.entry

    def image(self, step: _Step) -> bytes:
        img = self._images.get(id(step.fn))
        if img is None:
            img = self._images[id(step.fn)] = compile_cuda(resolve_source(step.fn), include_dirs_of(step.fn))
        return img

    def plan(self, compiled, host, worker):
        plans, replace, host_only = [], {}, []
        for s in self.steps:
            if s.fused is None:
                plans.append(worker.register_kernel_image(self.image(s), ENTRY_SYMBOL))
                continue
            sub = s.fused.plan(compiled, s.bind(host), worker)
            to_entry = {p.name: v for p, (kind, v) in zip(s.fn.params, s.bindings) if kind == "param"}
            for name, value in sub.get("replace", {}).items():
                replace[to_entry[name]] = value
            host_only += [to_entry[n] for n in sub.get("host_only", ()) if n in to_entry]
            plans.append(sub)
        # a tensor that one step only reads on the host may still be a device operand of another step
        used_on_device = {v for s in self.steps if s.fused is None
                          for p, (kind, v) in zip(s.fn.params, s.bindings) if p.is_tensor}
        return dict(steps=plans, replace=replace, host_only=tuple(n for n in host_only if n not in used_on_device))

    def launch(self, worker, dev, host, plan):
        for step, sp in zip(self.steps, plan["steps"]):
            if step.fused is not None:
                step.fused.launch(worker, step.bind({**host, **dev}), step.bind(host), sp)   # scalars come from the host side
                continue
            tensors, scalars = [], []
            for p, (kind, v) in zip(step.fn.params, step.bindings):
                if p.is_tensor:
                    tensors.append(dev[v])
                else:
                    scalars.append(encode_scalar(host[v] if kind == "param" else v, p.type))
            worker.launch_kernel(sp, tensors, scalars, block_num=step.block_num, threads_per_block=step.threads)


class _Refused(Exception):
    pass


def _namespace(fn) -> dict:
    ns = dict(getattr(fn, "__globals__", {}))
    if getattr(fn, "__closure__", None):
        for name, cell in zip(fn.__code__.co_freevars, fn.__closure__):
            try:
                ns[name] = cell.cell_contents
            except ValueError:
                pass
    return ns


def match(entry: Function, program=None) -> ExternProgramOp | None:
    """An ExternProgramOp if ``entry``'s body is a sequence of external-kernel calls, else None.
    Raises NotImplementedError when it calls external kernels in a way this front end does not follow."""
    if not entry.source:
        return None
    try:
        tree = ast.parse(textwrap.dedent(entry.source))
    except SyntaxError:
        return None
    fdef = next((n for n in ast.walk(tree) if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef))), None)
    if fdef is None:
        return None
    ns = _namespace(entry.fn)
    functions = dict(getattr(program, "functions", {}) or {})
    params = {p.name: p for p in entry.params}
    alias: dict[str, str] = {n: n for n in params}     # local name -> entry tensor parameter
    steps: list[_Step] = []
    saw_extern = False

    def callee(node):
        if isinstance(node, ast.Attribute) and isinstance(node.value, ast.Name) and node.value.id == "self":
            return functions.get(node.attr)
        if isinstance(node, ast.Name):
            f = ns.get(node.id)
            return f if isinstance(f, Function) else None
        return None

    def const(node):
        try:
            v = eval(compile(ast.Expression(node), "<orchestration>", "eval"), ns)  # noqa: S307 - module constants
        except Exception as e:
            raise _Refused(f"argument '{ast.unparse(node)}' is neither an entry parameter nor a constant ({e})")
        if not isinstance(v, (int, float, bool)):
            raise _Refused(f"argument '{ast.unparse(node)}' evaluates to {type(v).__name__}, not a number")
        return v

    def call(node, block_num, target):
        nonlocal saw_extern
        fn = callee(node.func)
        if fn is None:
            raise _Refused(f"call to '{ast.unparse(node.func)}' is neither an external kernel nor a fused operator")
        fused = None
        if fn.attrs.get("external_source") or fn.attrs.get("external_aiv_source"):
            if fn.attrs.get("core_type") not in (None, "aiv", "aic"):
                raise _Refused(f"core_type {fn.attrs.get('core_type')!r}: only single-kernel stubs are supported")
        else:
            from . import fused_programs
            try:
                fused = fused_programs.lookup(fn)
            except NotImplementedError:
                raise _Refused(f"call to '{fn.name}' is neither an external kernel nor a fused operator") from None
        saw_extern = True
        if node.keywords or len(node.args) != len(fn.params):
            raise _Refused(f"'{fn.name}' takes {len(fn.params)} positional arguments")
        bindings, result = [], None
        for p, a in zip(fn.params, node.args):
            if p.is_tensor:
                if not (isinstance(a, ast.Name) and a.id in alias):
                    raise _Refused(f"tensor argument '{ast.unparse(a)}' of '{fn.name}' is not an entry parameter "
                                   "(intermediate tensors are not supported)")
                bindings.append(("param", alias[a.id]))
                if result is None and p.direction is not Direction.In:
                    result = alias[a.id]
            elif isinstance(a, ast.Name) and a.id in params and not params[a.id].is_tensor:
                bindings.append(("param", a.id))
            else:
                bindings.append(("const", const(a)))
        if target is not None:
            if result is None:
                raise _Refused(f"'{fn.name}' has no output tensor to bind '{target}' to")
            alias[target] = result
        steps.append(_Step(fn, block_num, bindings, fused))

    def statement(st, block_num):
        if isinstance(st, ast.Expr) and isinstance(st.value, ast.Constant):
            return                                   # docstring / `...`
        if isinstance(st, (ast.Return, ast.Pass)):
            return
        if isinstance(st, ast.Expr) and isinstance(st.value, ast.Call):
            return call(st.value, block_num, None)
        if isinstance(st, ast.Assign) and len(st.targets) == 1 and isinstance(st.targets[0], ast.Name) \
                and isinstance(st.value, ast.Call):
            return call(st.value, block_num, st.targets[0].id)
        if isinstance(st, ast.With) and len(st.items) == 1 and isinstance(st.items[0].context_expr, ast.Call):
            c = st.items[0].context_expr
            if ast.unparse(c.func).split(".")[-1] == "spmd":
                kw = {k.arg: k.value for k in c.keywords}
                node = kw.get("core_num") or (c.args[0] if c.args else None)
                if node is None:
                    raise _Refused("pl.spmd without core_num")
                n = const(node)
                if not isinstance(n, int) or n < 1:
                    raise _Refused(f"pl.spmd core_num must be a positive int, got {n!r}")
                for inner in st.body:
                    statement(inner, n)
                return
        raise _Refused(f"statement '{ast.unparse(st).splitlines()[0]}' is not a call to an external kernel")

    try:
        for st in fdef.body:
            statement(st, 1)
    except _Refused as e:
        if saw_extern or any(f.attrs.get("external_source") for f in functions.values()):
            raise NotImplementedError(f"program entry '{entry.name}' uses external kernels, but {e}; this front end "
                                      "follows orchestrations that are plain sequences of external-kernel calls "
                                      "and fused-operator calls") from None
        return None
    if not steps:
        return None
    if entry.type not in (FunctionType.Orchestration, FunctionType.Opaque):
        return None
    return ExternProgramOp(entry, steps)


__all__ = ["ExternProgramOp", "compile_cuda", "match", "cache_dir", "encode_scalar", "ENTRY_SYMBOL"]
del ScalarType
