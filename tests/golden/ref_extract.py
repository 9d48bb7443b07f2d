"""Pull plain-torch golden functions out of the reference tree without importing it.

The reference's example and test modules import ``pypto`` at the top, which
cannot be imported without its compiled core.  Their ``golden`` / helper
functions, however, use only ``torch`` and ``struct``.  This helper parses a
reference file, picks named functions (top-level ones and simple constant
assignments by default; with ``nested=True`` functions defined anywhere, e.g.
helpers local to a test method) and executes just those in a namespace holding
torch and struct.  A nested function's free variables become globals of that
namespace: supply them through ``overrides``.
Used by ``make_golden.py`` (fixture generation) and by the CPU test that pins
the oracle whenever the reference tree is present.
"""

from __future__ import annotations

import ast
import os
import struct

import torch

# the reference checkout: $PYPTO_REFERENCE_ROOT, else a directory named "reference" beside this repository
REFERENCE_ROOT = os.environ.get("PYPTO_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))), "reference")


def available() -> bool:
    return os.path.isdir(os.path.join(REFERENCE_ROOT, "examples", "models"))


def _assigned(node: ast.Assign) -> set:
    """Names bound by a simple assignment (``A = ...`` or ``A, B = ...``); empty if it binds anything else."""
    out = set()
    for t in node.targets:
        elts = t.elts if isinstance(t, ast.Tuple) else [t]
        if not all(isinstance(e, ast.Name) for e in elts):
            return set()
        out |= {e.id for e in elts}
    return out


def extract(rel_path: str, names: list[str], overrides: dict | None = None, nested: bool = False) -> dict:
    """Return a namespace with the requested functions / constants of ``rel_path``
    (relative to the reference root).  ``overrides`` replaces module constants (e.g.
    to shrink problem sizes) after the definitions have run, and supplies the free
    variables of functions lifted out of an enclosing scope (``nested=True``)."""
    path = os.path.join(REFERENCE_ROOT, rel_path)
    with open(path, encoding="utf-8") as fh:
        tree = ast.parse(fh.read(), filename=path)
    wanted = []
    seen = set()
    for node in (ast.walk(tree) if nested else tree.body):
        if isinstance(node, ast.FunctionDef) and node.name in names:
            if node.name in seen:
                continue
            seen.add(node.name)
            node.decorator_list = []
            wanted.append(node)
        elif not nested and isinstance(node, ast.Assign) and _assigned(node) and _assigned(node) <= set(names):
            wanted.append(node)
    found = set()
    for n in wanted:
        found |= {n.name} if isinstance(n, ast.FunctionDef) else _assigned(n)
    missing = set(names) - found
    if missing:
        raise KeyError(f"{rel_path}: not found: {sorted(missing)}")
    ns: dict = {"torch": torch, "struct": struct, "__builtins__": __builtins__}
    exec(compile(ast.Module(body=wanted, type_ignores=[]), path, "exec"), ns)
    if overrides:
        ns.update(overrides)
    return ns
