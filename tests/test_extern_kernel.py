"""External kernels on the host side: the orchestration front end, nvcc compilation and its
cache, argument encoding and the decorator's argument checks.  Mirrors the reference's
tests/st/runtime/external_kernel/test_external_kernel.py:50-65 (program form) and
tests/ut/jit/test_extern_kernel.py:130-160 (JIT form).  No GPU needed: nvcc cross-compiles."""

from pathlib import Path

import pytest

import pypto_b200.language as pl
from pypto_b200 import ir
from pypto_b200.runtime import extern_kernel as ek

KERNELS = Path(__file__).parent / "extern_kernels" / "aiv"
_KERNEL = KERNELS / "spmd_write.cu"
_CORE_NUM, _BASE_CL, _FLOATS_PER_CACHE_LINE = 4, 0, 16
_TOTAL = (_BASE_CL + _CORE_NUM + 1) * _FLOATS_PER_CACHE_LINE


@pl.program
class SpmdWriteExternProgram:
    @pl.function(type=pl.FunctionType.AIV, external_source=_KERNEL)
    def SPMD_WRITE_AIV(self, out: pl.InOut[pl.Tensor[[_TOTAL], pl.FP32]],
                       base_cl: pl.Scalar[pl.INDEX]) -> pl.Tensor[[_TOTAL], pl.FP32]: ...

    @pl.function(type=pl.FunctionType.Orchestration)
    def main(self, out: pl.Out[pl.Tensor[[_TOTAL], pl.FP32]]) -> pl.Tensor[[_TOTAL], pl.FP32]:
        with pl.spmd(core_num=_CORE_NUM):
            out = self.SPMD_WRITE_AIV(out, _BASE_CL)
        return out


def test_program_form_is_matched():
    compiled = ir.compile(SpmdWriteExternProgram, platform="b200")
    op = compiled.fused
    assert isinstance(op, ek.ExternProgramOp) and compiled.op_names == ()
    (step,) = op.steps
    assert step.fn.name == "SPMD_WRITE_AIV" and step.block_num == _CORE_NUM
    assert step.bindings == [("param", "out"), ("const", _BASE_CL)]
    assert ek.resolve_source(step.fn) == _KERNEL


def test_jit_form_is_matched_and_paths_are_relative_to_the_stub():
    @pl.jit.extern(core_type="aiv", source="extern_kernels/aiv/axpy.cu")
    def axpy(x: pl.Tensor, y: pl.InOut[pl.Tensor], alpha: pl.Scalar[pl.FP32]) -> pl.Tensor: ...

    @pl.jit
    def entry(x: pl.Tensor, y: pl.InOut[pl.Tensor], alpha: pl.Scalar[pl.FP32]) -> pl.Tensor:
        with pl.spmd(core_num=8):
            y = axpy(x, y, alpha)
        y = axpy(x, y, 0.5)
        return y

    compiled = ir.compile(entry, platform="b200")
    steps = compiled.fused.steps
    assert [s.block_num for s in steps] == [8, 1]
    assert steps[0].bindings == [("param", "x"), ("param", "y"), ("param", "alpha")]
    assert steps[1].bindings == [("param", "x"), ("param", "y"), ("const", 0.5)]
    assert ek.resolve_source(steps[0].fn) == KERNELS / "axpy.cu"


def test_compiles_to_a_cubin_where_the_source_lies_and_caches(tmp_path, monkeypatch):
    monkeypatch.setenv("PYPTO_B200_CACHE", str(tmp_path))
    img = ek.compile_cuda(_KERNEL)          # includes ../common/cacheline_offset.h relative to the source
    assert img[:4] == b"\x7fELF"
    (cached,) = list((tmp_path / "extern").glob("*.cubin"))
    stamp = cached.stat().st_mtime_ns
    assert ek.compile_cuda(_KERNEL) == img and cached.stat().st_mtime_ns == stamp
    # a change in an included file is a different cache entry
    src = tmp_path / "k" / "aiv"
    src.mkdir(parents=True)
    (tmp_path / "k" / "common").mkdir()
    (src / "spmd_write.cu").write_text(_KERNEL.read_text())
    hdr = tmp_path / "k" / "common" / "cacheline_offset.h"
    hdr.write_text("#pragma once\nconstexpr int FLOATS_PER_CACHE_LINE = 16;\n")
    ek.compile_cuda(src / "spmd_write.cu")
    hdr.write_text("#pragma once\nconstexpr int FLOATS_PER_CACHE_LINE = 32;\n")
    ek.compile_cuda(src / "spmd_write.cu")
    assert len(list((tmp_path / "extern").glob("spmd_write-*.cubin"))) == 3


def test_compile_errors_carry_the_compiler_output(tmp_path, monkeypatch):
    monkeypatch.setenv("PYPTO_B200_CACHE", str(tmp_path))
    bad = tmp_path / "bad.cu"
    bad.write_text('extern "C" __global__ void kernel_entry(const long long* a) { undeclared_name(); }\n')
    with pytest.raises(RuntimeError, match="undeclared_name"):
        ek.compile_cuda(bad)
    with pytest.raises(FileNotFoundError):
        ek.compile_cuda(tmp_path / "missing.cu")


@pl.program
class NormThenAxpy:
    """A fused operator of the table (rms_norm(x, gamma, output)) followed by an external kernel."""

    @pl.function(type=pl.FunctionType.InCore)
    def rms_norm(self, x: pl.Tensor[[32, 64], pl.FP32], gamma: pl.Tensor[[1, 64], pl.FP32],
                 output: pl.Out[pl.Tensor[[32, 64], pl.FP32]]) -> pl.Tensor[[32, 64], pl.FP32]: ...

    @pl.function(type=pl.FunctionType.AIV, external_source=KERNELS / "axpy.cu")
    def axpy(self, x: pl.Tensor[[32, 64], pl.FP32], y: pl.InOut[pl.Tensor[[32, 64], pl.FP32]],
             alpha: pl.Scalar[pl.FP32]) -> pl.Tensor[[32, 64], pl.FP32]: ...

    @pl.function(type=pl.FunctionType.Orchestration)
    def main(self, x: pl.Tensor[[32, 64], pl.FP32], gamma: pl.Tensor[[1, 64], pl.FP32],
             normed: pl.Out[pl.Tensor[[32, 64], pl.FP32]], y: pl.InOut[pl.Tensor[[32, 64], pl.FP32]]):
        normed = self.rms_norm(x, gamma, normed)
        with pl.spmd(core_num=4):
            y = self.axpy(normed, y, 2.0)
        return y


def test_fused_operators_and_external_kernels_chain_in_one_orchestration():
    compiled = ir.compile(NormThenAxpy, platform="b200")
    first, second = compiled.fused.steps
    assert first.fused is not None and first.fused.op_names == ("rms_norm",) and second.fused is None
    assert first.bindings == [("param", "x"), ("param", "gamma"), ("param", "normed")]
    assert second.bindings == [("param", "normed"), ("param", "y"), ("const", 2.0)] and second.block_num == 4
    assert compiled.op_names == ("rms_norm",)


def test_orchestrations_the_front_end_does_not_follow_are_refused():
    @pl.program
    class Mixed:
        @pl.function(type=pl.FunctionType.AIV, external_source=_KERNEL)
        def K(self, out: pl.InOut[pl.Tensor[[_TOTAL], pl.FP32]], base_cl: pl.Scalar[pl.INDEX]): ...

        @pl.function(type=pl.FunctionType.Orchestration)
        def main(self, out: pl.Out[pl.Tensor[[_TOTAL], pl.FP32]]):
            tmp = pl.create_tensor([_TOTAL], dtype=pl.FP32)
            tmp = self.K(tmp, 0)
            return out

    with pytest.raises(NotImplementedError, match="plain sequences of external-kernel calls"):
        ir.compile(Mixed, platform="b200")

    @pl.program
    class NoExtern:
        @pl.function(type=pl.FunctionType.Orchestration)
        def main(self, out: pl.Out[pl.Tensor[[4], pl.FP32]]):
            out = pl.add(out, out)
            return out

    with pytest.raises(NotImplementedError, match="no fused kernel registered"):
        ir.compile(NoExtern, platform="b200")


def test_decorator_argument_checks_match_the_reference():
    with pytest.raises(ValueError, match="requires core_type='mixed'"):
        @pl.jit.extern(core_type="aiv", source="k.cu", dual_aiv_dispatch=True)
        def k(a: pl.Tensor, out: pl.Out[pl.Tensor]): ...
    with pytest.raises(ValueError, match="must be 'aic', 'aiv', or 'mixed'"):
        pl.jit.extern(core_type="gpu", source="k.cu")
    with pytest.raises(ValueError, match="requires source="):
        @pl.jit.extern(core_type="aiv")
        def k2(a: pl.Tensor, out: pl.Out[pl.Tensor]): ...
    with pytest.raises(ValueError, match="requires both aic_source= and aiv_source="):
        @pl.jit.extern(core_type="mixed", aic_source="k.cu")
        def k3(a: pl.Tensor, out: pl.Out[pl.Tensor]): ...


def test_scalar_encoding():
    assert ek.encode_scalar(-1, pl.Scalar[pl.INDEX]) == 0xFFFFFFFFFFFFFFFF
    assert ek.encode_scalar(7, pl.Scalar[pl.INT32]) == 7
    assert ek.encode_scalar(1.0, pl.Scalar[pl.FP32]) == 0x3F800000
    assert ek.encode_scalar(3.0, pl.Scalar[pl.INT64]) == 3
    with pytest.raises(TypeError):
        ek.encode_scalar(0.5, pl.Scalar[pl.INT64])
    with pytest.raises(TypeError):
        ek.encode_scalar(0.5, pl.Scalar[pl.BF16])
