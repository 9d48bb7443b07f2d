"""External kernels end to end on the GPU: a program that dispatches a hand-written CUDA source
across SPMD blocks (the reference's tests/st/runtime/external_kernel/test_external_kernel.py:50-102,
exact golden [0, 1, 2, 3] one cache line apart), the JIT form with two tensors and an fp32
scalar, resident DeviceTensors with a registered handle, and the C-ABI error paths."""

import ctypes as C

import pytest
import torch

import pypto_b200.language as pl
from pypto_b200 import _lib, ir
from pypto_b200.runtime import ChipWorker, RunConfig, run
from pypto_b200.runtime import extern_kernel as ek
from test_extern_kernel import (_BASE_CL, _CORE_NUM, _FLOATS_PER_CACHE_LINE, _KERNEL, _TOTAL, NormThenAxpy,
                                SpmdWriteExternProgram)

pytestmark = pytest.mark.gpu


def _expected():
    out = torch.zeros(_TOTAL, dtype=torch.float32)
    for block_idx in range(_CORE_NUM):
        out[(_BASE_CL + block_idx) * _FLOATS_PER_CACHE_LINE] = float(block_idx)
    return out


def test_program_dispatches_external_kernel_across_spmd_blocks():
    out = torch.zeros(_TOTAL, dtype=torch.float32)
    compiled = run(SpmdWriteExternProgram, out, config=RunConfig(platform="b200"))
    assert torch.equal(out, _expected())
    returned = compiled()                       # return style: the Out tensor is allocated and returned
    assert torch.equal(returned, _expected())


def test_jit_extern_with_two_tensors_and_a_float_scalar():
    @pl.jit.extern(core_type="aiv", source="extern_kernels/aiv/axpy.cu")
    def axpy(x: pl.Tensor, y: pl.InOut[pl.Tensor], alpha: pl.Scalar[pl.FP32]) -> pl.Tensor: ...

    @pl.jit
    def entry(x: pl.Tensor, y: pl.InOut[pl.Tensor], alpha: pl.Scalar[pl.FP32]) -> pl.Tensor:
        with pl.spmd(core_num=8):
            y = axpy(x, y, alpha)
        y = axpy(x, y, 0.5)
        return y

    g = torch.Generator().manual_seed(0)
    x, y = torch.randn(5000, generator=g), torch.randn(5000, generator=g)
    want = 0.5 * x + (2.5 * x + y)
    entry(x, y, 2.5, config=RunConfig(platform="b200"))
    assert torch.equal(y, want)                 # the fixture rounds product and sum separately, as torch does
    assert len(entry._cache) == 1


def test_fused_operator_then_external_kernel_in_one_program():
    from oracle import layer as olayer
    g = torch.Generator().manual_seed(2)
    x, gamma = torch.randn(32, 64, generator=g), torch.rand(1, 64, generator=g) + 0.5
    y0 = torch.randn(32, 64, generator=g)
    normed, y = torch.zeros(32, 64), y0.clone()
    run(NormThenAxpy, x, gamma, normed, y, config=RunConfig(platform="b200"))
    want_norm = olayer.rms_norm_sqrt_div(x, gamma, 1e-5)
    assert torch.allclose(normed, want_norm, rtol=1e-5, atol=1e-5)
    assert torch.equal(y, 2.0 * normed + y0)


def test_resident_tensors_and_registered_handle():
    compiled = ir.compile(SpmdWriteExternProgram, platform="b200")
    with ChipWorker(RunConfig(platform="b200")) as w:
        out = w.alloc_tensor((_TOTAL,), torch.float32, init=torch.full((_TOTAL,), -1.0))
        handle = w.register(compiled)
        for _ in range(40):                     # more launches than argument-ring slots
            handle(out)
        got = w.read_tensor(out)
        w.free_tensor(out)
    want = torch.full((_TOTAL,), -1.0)
    want[_expected() != 0] = _expected()[_expected() != 0]
    want[_BASE_CL * _FLOATS_PER_CACHE_LINE] = 0.0
    assert torch.equal(got, want)


def test_c_abi_error_paths():
    lib = _lib.load()
    img = ek.compile_cuda(_KERNEL)
    with ChipWorker(RunConfig(platform="b200")) as w:
        cid = C.c_int32()
        buf = C.create_string_buffer(img, len(img))
        assert lib.pto_register_kernel_image(w._handle, buf, len(img), b"no_such_entry", C.byref(cid)) == 6
        assert b"no_such_entry" in lib.pto_last_error()
        junk = C.create_string_buffer(b"not an image", 12)
        assert lib.pto_register_kernel_image(w._handle, junk, 12, b"kernel_entry", C.byref(cid)) in (2, 6)
        good = w.register_kernel_image(img)
        assert w.register_kernel_image(img) == good          # cached by content
        args = _lib.TaskArgs(None, 0, None, 0)
        assert lib.pto_run_kernel(w._handle, good, C.byref(args), 0, 128) == 1       # block_num 0
        assert lib.pto_run_kernel(w._handle, good, C.byref(args), 1, 2048) == 1      # too many threads
        assert lib.pto_run_kernel(w._handle, good + 1000, C.byref(args), 1, 128) == 6
        assert lib.pto_unregister_callable(w._handle, good) == 0
        assert lib.pto_run_kernel(w._handle, good, C.byref(args), 1, 128) == 6


def test_bounded_wait_that_runs_out_is_reported_and_the_worker_stays_usable():
    """Failure detection on the device without a fault: an external kernel waits 20 ms for a flag nothing sets, records
    a timeout in the worker's error word and returns; the launch surface raises PTO_DEVICE_TIMEOUT with the site, and
    the same worker then runs the same kernel with the flag set."""
    @pl.jit.extern(core_type="aiv", source="extern_kernels/aiv/wait_for_flag.cu")
    def wait_for_flag(flag: pl.Tensor, out: pl.InOut[pl.Tensor], timeout_us: pl.Scalar[pl.INT64]) -> pl.Tensor: ...

    @pl.jit
    def entry(flag: pl.Tensor, out: pl.InOut[pl.Tensor], timeout_us: pl.Scalar[pl.INT64]) -> pl.Tensor:
        out = wait_for_flag(flag, out, timeout_us)
        return out

    with ChipWorker(RunConfig(platform="b200")) as wk:
        out = torch.zeros(1)
        with pytest.raises(_lib.PtoError) as ei:
            entry(torch.zeros(1, dtype=torch.int32), out, 20000)
        assert ei.value.status == 4 and "site 900" in str(ei.value)          # PTO_DEVICE_TIMEOUT
        assert out.item() == 0.0
        assert wk.device_status() == (0, 0, 0, 0)          # reading the word cleared it
        entry(torch.ones(1, dtype=torch.int32), out, 20000)
        assert out.item() == 1.0
