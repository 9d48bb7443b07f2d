"""Pull plain-torch golden functions out of the reference tree without importing it.

The reference's example and test modules import ``pypto`` at the top, which
cannot be imported without its compiled core.  Their ``golden`` / helper
functions, however, use only ``torch`` and ``struct``.  This helper parses a
reference file, picks named top-level functions (and simple constant
assignments) and executes just those in a namespace holding torch and struct.
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


def extract(rel_path: str, names: list[str], overrides: dict | None = None) -> dict:
    """Return a namespace with the requested top-level functions / constants of
    ``rel_path`` (relative to the reference root).  ``overrides`` replaces module
    constants (e.g. to shrink problem sizes) after the definitions have run."""
    path = os.path.join(REFERENCE_ROOT, rel_path)
    with open(path, encoding="utf-8") as fh:
        tree = ast.parse(fh.read(), filename=path)
    wanted = []
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            node.decorator_list = []
            wanted.append(node)
        elif isinstance(node, ast.Assign) and all(
            isinstance(t, ast.Name) and t.id in names for t in node.targets
        ):
            wanted.append(node)
    found = {getattr(n, "name", None) or n.targets[0].id for n in wanted}
    missing = set(names) - found
    if missing:
        raise KeyError(f"{rel_path}: not found: {sorted(missing)}")
    ns: dict = {"torch": torch, "struct": struct, "__builtins__": __builtins__}
    exec(compile(ast.Module(body=wanted, type_ignores=[]), path, "exec"), ns)
    if overrides:
        ns.update(overrides)
    return ns
