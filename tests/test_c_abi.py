"""The shared library loads without a GPU and exports every symbol the header declares."""

import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "pypto_b200.h")).read()
    return sorted(set(re.findall(r"PTO_API\s+[\w\s\*]+?\b(pto_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import __graft_entry__ as entry
    entry.build()
    from pypto_b200 import _lib
    lib = _lib.load()
    names = _declared()
    assert len(names) >= 19
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(names)


def test_op_list_and_version():
    from pypto_b200 import _lib
    assert {"paged_attention", "paged_gather", "rms_norm", "ffn_swiglu", "linear", "rope_kv_append", "scope3",
            "decoder_layer", "matmul_mx", "moe_layer", "llama_mini"} <= set(_lib.op_names())
    assert b"sm_100a" in _lib.load().pto_version()


def test_cpu_tensors_are_refused_not_computed():
    import torch
    from pypto_b200 import BackendUnavailable, ops
    with pytest.raises(BackendUnavailable):
        ops.paged_gather(torch.zeros(4, 4), torch.zeros(1, dtype=torch.int32),
                         torch.zeros(1, dtype=torch.int32), 4)


def test_header_is_plain_c_and_the_library_serves_a_c_host(tmp_path):
    """gcc (C, not C++) compiles a host that includes the public header, dlopens the library and
    makes the first calls of a foreign-language binding.  Without a GPU pto_worker_create must fail
    with a status and a message instead of crashing."""
    import shutil
    import subprocess
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    lib = root / "pypto_b200" / "lib" / "libpypto_b200.so"
    assert lib.exists(), "build the library first (python -m pypto_b200.build)"
    gcc = shutil.which("gcc")
    assert gcc, "gcc is part of this image"
    exe = tmp_path / "c_abi_host"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-I", str(root / "include"), str(root / "tests" / "c_abi_host.c"),
                    "-ldl", "-o", str(exe)], check=True)
    r = subprocess.run([str(exe), str(lib)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "version=" in r.stdout and "op=paged_attention" in r.stdout and "worker_create=" in r.stdout


def test_ctypes_signatures_agree_with_the_header_prototypes():
    """Every prototype of include/pypto_b200.h has a ctypes signature with the same number of parameters and the same
    kind of each (pointer, 32-bit integer, 64-bit integer / size_t, float): a drift between the two is a silent ABI
    error (a float passed where the callee reads an int register, a missing trailing argument)."""
    import ctypes as C
    import re

    from pypto_b200 import _lib
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    hdr = re.sub(r"/\*.*?\*/", "", open(os.path.join(root, "include", "pypto_b200.h")).read(), flags=re.S)
    protos = re.findall(r"PTO_API\s+([\w\s\*]+?)\s*\b(pto_\w+)\s*\(([^;]*?)\)\s*;", hdr, flags=re.S)
    assert len(protos) >= 60

    def kind_c(decl: str) -> str:
        decl = decl.strip()
        if "*" in decl or "[" in decl:
            return "ptr"
        base = re.sub(r"\b\w+$", "", decl).replace("const", "").strip() or decl      # drop the parameter name
        if base in ("float",):
            return "f32"
        if base in ("double",):
            return "f64"
        if base in ("int64_t", "uint64_t", "size_t", "long long", "unsigned long long"):
            return "i64"
        if base in ("int", "int32_t", "uint32_t", "unsigned", "unsigned int"):
            return "i32"
        raise AssertionError(f"parameter type not classified: {decl!r}")

    def kind_py(t) -> str:
        if t in (C.c_float,):
            return "f32"
        if t in (C.c_double,):
            return "f64"
        if t in (C.c_int, C.c_int32, C.c_uint32, C.c_uint):
            return "i32"
        if t in (C.c_int64, C.c_uint64, C.c_size_t, C.c_longlong, C.c_ulonglong):
            return "i64"
        return "ptr"            # c_void_p, c_char_p, POINTER(...), arrays

    for _ret, name, args in protos:
        assert name in _lib.SIGNATURES, f"{name}: no ctypes signature"
        args = args.strip()
        decls = [] if args in ("", "void") else [a for a in args.split(",")]
        sig = _lib.SIGNATURES[name][1]
        assert len(sig) == len(decls), f"{name}: header has {len(decls)} parameters, ctypes {len(sig)}"
        for i, (d, t) in enumerate(zip(decls, sig)):
            assert kind_c(d) == kind_py(t), f"{name}: parameter {i} ({d.strip()!r}) is {kind_c(d)} in the header, {kind_py(t)} in ctypes"
    assert not [k for k in _lib.SIGNATURES if k not in {p[1] for p in protos}], "ctypes signatures without a prototype"
